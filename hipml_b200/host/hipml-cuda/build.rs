// Links libhipml_cuda.so; HIPML_CUDA_LIB names the directory that holds it.
fn main() {
    if let Ok(dir) = std::env::var("HIPML_CUDA_LIB") {
        println!("cargo:rustc-link-search=native={dir}");
    }
    println!("cargo:rustc-link-lib=dylib=hipml_cuda");
    println!("cargo:rerun-if-env-changed=HIPML_CUDA_LIB");
}
