// Section A of the C ABI: the device layer a `hipml-cuda` crate binds in place of
// `hipml-hip`'s amdhip64 block (crates/hipml-hip/src/ffi.rs:29-105), over the CUDA
// runtime. Same conventions: int status, 0 = success, opaque handles, memcpy kinds 1/2/3.
// Also the error-message plumbing shared by the launchers and the built-in kernel table
// behind hipml_module_get_function.
#include <cstring>

#include "common.cuh"

namespace hipml {

namespace {
thread_local char g_message[512] = "";
}

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_message, sizeof(g_message), fmt, ap);
    va_end(ap);
    return code;
}

namespace {

__device__ int g_device_status;

inline int rc(cudaError_t e) { return static_cast<int>(e); }

cudaMemcpyKind kind_of(int kind) {
    switch (kind) {
        case HIPML_MEMCPY_HOST_TO_DEVICE: return cudaMemcpyHostToDevice;
        case HIPML_MEMCPY_DEVICE_TO_HOST: return cudaMemcpyDeviceToHost;
        case HIPML_MEMCPY_DEVICE_TO_DEVICE: return cudaMemcpyDeviceToDevice;
        default: return cudaMemcpyDefault;
    }
}

}  // namespace

int *device_status_word() {
    // One status word per device; the symbol address is resolved per current device.
    int *p = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void **>(&p), g_device_status) != cudaSuccess)
        return nullptr;
    return p;
}

}  // namespace hipml

using namespace hipml;

namespace {
int g_builtin_module;  // its address is the one module handle
}  // namespace

extern "C" {

int hipml_init(unsigned flags) {
    (void)flags;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) return rc(e);
    return HIPML_SUCCESS;
}

int hipml_get_device_count(int *count) { return rc(cudaGetDeviceCount(count)); }

int hipml_get_device(int *device, int ordinal) {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess) return rc(e);
    if (ordinal < 0 || ordinal >= n) return rc(cudaErrorInvalidDevice);
    *device = ordinal;
    return HIPML_SUCCESS;
}

int hipml_set_device(int device) { return rc(cudaSetDevice(device)); }

int hipml_device_get_name(char *name, int len, int device) {
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return rc(e);
    if (len > 0) {
        strncpy(name, prop.name, (size_t)len - 1);
        name[len - 1] = 0;
    }
    return HIPML_SUCCESS;
}

int hipml_device_total_mem(size_t *bytes, int device) {
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) return rc(e);
    *bytes = prop.totalGlobalMem;
    return HIPML_SUCCESS;
}

int hipml_device_compute_capability(int *major, int *minor, int device) {
    cudaError_t e = cudaDeviceGetAttribute(major, cudaDevAttrComputeCapabilityMajor, device);
    if (e != cudaSuccess) return rc(e);
    return rc(cudaDeviceGetAttribute(minor, cudaDevAttrComputeCapabilityMinor, device));
}

const char *hipml_get_error_string(int code) {
    switch (code) {
        case HIPML_ERR_INVALID_ARGUMENT: return "hipml: invalid argument";
        case HIPML_ERR_UNKNOWN_KERNEL: return "hipml: unknown kernel";
        case HIPML_ERR_WORKSPACE: return "hipml: workspace missing or too small";
        case HIPML_ERR_DEVICE_STATUS: return "hipml: a kernel reported a bounded-wait timeout";
        default: return cudaGetErrorString(static_cast<cudaError_t>(code));
    }
}

const char *hipml_last_error_message(void) { return g_message; }

int hipml_malloc(void **ptr, size_t size) { return rc(cudaMalloc(ptr, size)); }
int hipml_free(void *ptr) { return rc(cudaFree(ptr)); }
int hipml_memset(void *dst, int value, size_t size) { return rc(cudaMemset(dst, value, size)); }
int hipml_mem_get_info(size_t *free_bytes, size_t *total_bytes) {
    return rc(cudaMemGetInfo(free_bytes, total_bytes));
}
int hipml_memcpy(void *dst, const void *src, size_t size, int kind) {
    return rc(cudaMemcpy(dst, src, size, kind_of(kind)));
}
int hipml_memcpy_async(void *dst, const void *src, size_t size, int kind, hipml_stream_t stream) {
    return rc(cudaMemcpyAsync(dst, src, size, kind_of(kind), as_stream(stream)));
}
int hipml_device_synchronize(void) { return rc(cudaDeviceSynchronize()); }
int hipml_host_alloc(void **ptr, size_t size) { return rc(cudaMallocHost(ptr, size)); }
int hipml_host_free(void *ptr) { return rc(cudaFreeHost(ptr)); }

int hipml_event_create(hipml_event_t *event) {
    return rc(cudaEventCreate(reinterpret_cast<cudaEvent_t *>(event)));
}
int hipml_event_destroy(hipml_event_t event) {
    return rc(cudaEventDestroy(reinterpret_cast<cudaEvent_t>(event)));
}
int hipml_event_record(hipml_event_t event, hipml_stream_t stream) {
    return rc(cudaEventRecord(reinterpret_cast<cudaEvent_t>(event), as_stream(stream)));
}
int hipml_event_synchronize(hipml_event_t event) {
    return rc(cudaEventSynchronize(reinterpret_cast<cudaEvent_t>(event)));
}
int hipml_event_elapsed_time(float *ms, hipml_event_t start, hipml_event_t stop) {
    return rc(cudaEventElapsedTime(ms, reinterpret_cast<cudaEvent_t>(start),
                                   reinterpret_cast<cudaEvent_t>(stop)));
}

int hipml_stream_create(hipml_stream_t *stream) {
    return rc(cudaStreamCreate(reinterpret_cast<cudaStream_t *>(stream)));
}
int hipml_stream_destroy(hipml_stream_t stream) { return rc(cudaStreamDestroy(as_stream(stream))); }
int hipml_stream_synchronize(hipml_stream_t stream) {
    return rc(cudaStreamSynchronize(as_stream(stream)));
}
int hipml_stream_wait_event(hipml_stream_t stream, hipml_event_t event, unsigned flags) {
    return rc(cudaStreamWaitEvent(as_stream(stream), reinterpret_cast<cudaEvent_t>(event), flags));
}

int hipml_stream_begin_capture(hipml_stream_t stream, int mode) {
    const cudaStreamCaptureMode m = mode == 0   ? cudaStreamCaptureModeGlobal
                                    : mode == 1 ? cudaStreamCaptureModeThreadLocal
                                                : cudaStreamCaptureModeRelaxed;
    return rc(cudaStreamBeginCapture(as_stream(stream), m));
}
int hipml_stream_end_capture(hipml_stream_t stream, hipml_graph_t *graph) {
    return rc(cudaStreamEndCapture(as_stream(stream), reinterpret_cast<cudaGraph_t *>(graph)));
}
int hipml_graph_instantiate(hipml_graph_exec_t *exec, hipml_graph_t graph, void *error_node,
                            char *log_buffer, size_t log_size) {
    (void)error_node;
    if (log_buffer && log_size) log_buffer[0] = 0;
    return rc(cudaGraphInstantiate(reinterpret_cast<cudaGraphExec_t *>(exec),
                                   reinterpret_cast<cudaGraph_t>(graph), 0));
}
int hipml_graph_launch(hipml_graph_exec_t exec, hipml_stream_t stream) {
    return rc(cudaGraphLaunch(reinterpret_cast<cudaGraphExec_t>(exec), as_stream(stream)));
}
int hipml_graph_upload(hipml_graph_exec_t exec, hipml_stream_t stream) {
    return rc(cudaGraphUpload(reinterpret_cast<cudaGraphExec_t>(exec), as_stream(stream)));
}
int hipml_graph_destroy(hipml_graph_t graph) {
    return rc(cudaGraphDestroy(reinterpret_cast<cudaGraph_t>(graph)));
}
int hipml_graph_exec_destroy(hipml_graph_exec_t exec) {
    return rc(cudaGraphExecDestroy(reinterpret_cast<cudaGraphExec_t>(exec)));
}

int hipml_module_load(hipml_module_t *module, const char *file) {
    (void)file;
    *module = &g_builtin_module;
    return HIPML_SUCCESS;
}
int hipml_module_unload(hipml_module_t module) {
    return module == &g_builtin_module
               ? HIPML_SUCCESS
               : fail(HIPML_ERR_INVALID_ARGUMENT, "hipml_module_unload: not a module handle");
}
int hipml_module_get_function(hipml_function_t *function, hipml_module_t module, const char *name) {
    if (module != &g_builtin_module)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "hipml_module_get_function: not a module handle");
    const void *fn = lookup_kv_kernel(name);
    if (!fn) fn = lookup_decode_kernel(name);
    if (!fn) fn = lookup_chunk_kernel(name);
    if (!fn) fn = lookup_cols_kernel(name);
    if (!fn) fn = lookup_front_kernel(name);
    if (fn) {
        *function = const_cast<void *>(fn);
        return HIPML_SUCCESS;
    }
    return fail(HIPML_ERR_UNKNOWN_KERNEL, "kernel %s is not in the module", name);
}
int hipml_module_launch_kernel(hipml_function_t function, unsigned grid_x, unsigned grid_y,
                               unsigned grid_z, unsigned block_x, unsigned block_y,
                               unsigned block_z, unsigned shared_mem_bytes, hipml_stream_t stream,
                               void **kernel_params, void **extra) {
    if (extra != nullptr)
        return fail(HIPML_ERR_INVALID_ARGUMENT, "hipml_module_launch_kernel: extra must be NULL");
    if (function == nullptr)
        return fail(HIPML_ERR_UNKNOWN_KERNEL, "hipml_module_launch_kernel: null function handle");
    return rc(cudaLaunchKernel(function, dim3(grid_x, grid_y, grid_z),
                               dim3(block_x, block_y, block_z), kernel_params, shared_mem_bytes,
                               as_stream(stream)));
}

int hipml_check_device_status(hipml_stream_t stream, int *status) {
    cudaError_t e = cudaStreamSynchronize(as_stream(stream));
    if (e != cudaSuccess) return rc(e);
    int *word = device_status_word();
    if (!word) return rc(cudaGetLastError());
    int value = 0;
    e = cudaMemcpy(&value, word, sizeof(int), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return rc(e);
    if (status) *status = value;
    if (value != 0) {
        const int zero = 0;
        cudaMemcpy(word, &zero, sizeof(int), cudaMemcpyHostToDevice);
        return fail(HIPML_ERR_DEVICE_STATUS, "a kernel's bounded wait ran out (code %d)", value);
    }
    return HIPML_SUCCESS;
}

const char *hipml_version(void) { return "hipml_cuda 0.1 sm_100a"; }

}  // extern "C"
