//! `hipml-cuda`: the CUDA counterpart of `hipml-hip` for the full-attention path.
//!
//! `ffi` declares every symbol of `include/hipml_cuda.h`. `check` is the error convention of
//! `crates/hipml-hip/src/device.rs:111-124`: a non-zero status becomes
//! `Err("{what} failed: {code} ({text})")`, with the text taken from the CUDA runtime for its
//! own codes and from the library's last message for codes >= 10000 (the launchers' argument
//! errors, which carry the sentence the Rust launcher used to build itself).
//!
//! Not compiled where the library is built (no Rust toolchain there); kept in step with the
//! header by `gen_ffi.py` and `tests/test_abi_symbols.py`.
pub mod ffi;

use std::ffi::CStr;

pub const ERR_BASE: i32 = 10000;

pub fn check(what: &str, code: ffi::Status) -> Result<(), String> {
    if code == 0 {
        return Ok(());
    }
    let text = unsafe {
        let p = if code >= ERR_BASE { ffi::hipml_last_error_message() } else { ffi::hipml_get_error_string(code) };
        if p.is_null() { String::from("unknown") } else { CStr::from_ptr(p).to_string_lossy().into_owned() }
    };
    Err(format!("{what} failed: {code} ({text})"))
}

/// Reads and clears the device status word (bounded waits that ran out); `Err` names the code.
pub fn check_device_status(stream: ffi::Stream) -> Result<(), String> {
    let mut status: i32 = 0;
    check("device status", unsafe { ffi::hipml_check_device_status(stream, &mut status) })
}
