//! The quantized entry points of tl_runtime, as they look with this back end behind them.
//!
//! In the reference these live in crates/tl_runtime/src/system.rs:140-382 (`tl_qtensor_matmul` and the QTensor reference
//! counting), crates/tl_runtime/src/gguf.rs:34-196 (`tl_gguf_load`) and crates/tl_runtime/src/tensor_map.rs:110-150,279
//! (`tl_tensor_map_get`, `tl_tensor_map_get_quantized`).  With TL_DEVICE=cuda served by libtlb200 their bodies reduce to
//! the calls below: the loader repacks every quantized tensor once into the tiled device layout, so there is no
//! host-side `Vec<u8>` copy, no lazily filled f32 / transposed caches and no per-call environment lookup.
//! The symbol names and C signatures are the ones src/compiler/codegen/builtins.rs maps (3486-3507, 2620, 2687).
use std::ffi::{c_char, c_void, CString};

use crate::b200_device::st;
use crate::ffi;

/// StringStruct (crates/tl_runtime/src/string_ffi.rs:7-11)
#[repr(C)]
pub struct StringStruct {
    pub ptr: *mut c_char,
    pub len: i64,
}

fn null_on_err<T>(r: Result<*mut T, tl_backend::BackendError>) -> *mut T {
    // tl_runtime records the error for tl_report_runtime_error_loc and hands the JIT a null (error.rs:161-182)
    r.unwrap_or(std::ptr::null_mut())
}

/// tl_gguf_load(path) -> Map*
#[no_mangle]
pub extern "C" fn tl_b200_gguf_load(path: *const StringStruct) -> *mut c_void {
    let mut m: *mut ffi::TlbMap = std::ptr::null_mut();
    let s = path as *const ffi::TlbString;
    null_on_err(st(unsafe { ffi::tlb_gguf_load_str(&mut m, s) }).map(|_| m)) as *mut c_void
}

fn name_of(s: *const StringStruct) -> Option<CString> {
    if s.is_null() {
        return None;
    }
    let s = unsafe { &*s };
    let bytes = unsafe { std::slice::from_raw_parts(s.ptr as *const u8, s.len.max(0) as usize) };
    CString::new(bytes).ok()
}

/// tl_tensor_map_get / tl_tensor_map_get_1d(map, name) -> T*  (dequantised f32, cached in the map)
#[no_mangle]
pub extern "C" fn tl_b200_tensor_map_get(map: *mut c_void, name: *const StringStruct) -> *mut c_void {
    let Some(n) = name_of(name) else { return std::ptr::null_mut() };
    let mut t: *mut ffi::TlbTensor = std::ptr::null_mut();
    null_on_err(st(unsafe { ffi::tlb_map_get(&mut t, map as *mut _, n.as_ptr()) }).map(|_| t)) as *mut c_void
}

/// tl_tensor_map_get_quantized(map, name) -> QTensor*  (a retained handle, as Arc::into_raw of a clone is)
#[no_mangle]
pub extern "C" fn tl_b200_tensor_map_get_quantized(map: *mut c_void, name: *const StringStruct) -> *mut c_void {
    let Some(n) = name_of(name) else { return std::ptr::null_mut() };
    let mut q: *mut ffi::TlbQTensor = std::ptr::null_mut();
    null_on_err(st(unsafe { ffi::tlb_map_get_quantized(&mut q, map as *mut _, n.as_ptr()) }).map(|_| q)) as *mut c_void
}

/// tl_qtensor_matmul(x, w) -> T*: y[M, N] = x[M, K] . W^T.  1-4 rows stream the weight through the fused matvec, more
/// rows run the tensor-core GEMM; F32 / F16 and the other block types take the dense route inside the library.
#[no_mangle]
pub extern "C" fn tl_b200_qtensor_matmul(x: *mut c_void, w: *mut c_void) -> *mut c_void {
    let mut t: *mut ffi::TlbTensor = std::ptr::null_mut();
    null_on_err(st(unsafe { ffi::tlb_qtensor_matmul(&mut t, x as *const _, w as *const _) }).map(|_| t)) as *mut c_void
}

#[no_mangle]
pub extern "C" fn tl_b200_qtensor_retain(w: *mut c_void) {
    unsafe { ffi::tlb_qtensor_retain(w as *mut _) };
}

#[no_mangle]
pub extern "C" fn tl_b200_qtensor_release(w: *mut c_void) {
    unsafe { ffi::tlb_qtensor_release(w as *mut _) };
}

/// KV-cache handle table (crates/tl_runtime/src/llm.rs:105-174): the handle is the pointer as an i64 behind `sret`.
#[no_mangle]
pub extern "C" fn tl_b200_kvcache_new(out: *mut i64, layers: i64) {
    let mut c: *mut ffi::TlbKvCache = std::ptr::null_mut();
    let ok = st(unsafe { ffi::tlb_kvcache_new(&mut c, layers) }).is_ok();
    unsafe { *out = if ok { c as i64 } else { 0 } };
}

#[no_mangle]
pub extern "C" fn tl_b200_kvcache_update(handle: *const i64, layer: i64, k: *mut c_void, v: *mut c_void) {
    let c = unsafe { *handle } as *mut ffi::TlbKvCache;
    unsafe { ffi::tlb_kvcache_update(c, layer, k as *mut _, v as *mut _) };
}

#[no_mangle]
pub extern "C" fn tl_b200_kvcache_get_k(handle: *const i64, layer: i64) -> *mut c_void {
    let c = unsafe { *handle } as *mut ffi::TlbKvCache;
    let mut t: *mut ffi::TlbTensor = std::ptr::null_mut();
    null_on_err(st(unsafe { ffi::tlb_kvcache_get_k(&mut t, c, layer) }).map(|_| t)) as *mut c_void
}

#[no_mangle]
pub extern "C" fn tl_b200_kvcache_get_v(handle: *const i64, layer: i64) -> *mut c_void {
    let c = unsafe { *handle } as *mut ffi::TlbKvCache;
    let mut t: *mut ffi::TlbTensor = std::ptr::null_mut();
    null_on_err(st(unsafe { ffi::tlb_kvcache_get_v(&mut t, c, layer) }).map(|_| t)) as *mut c_void
}

#[no_mangle]
pub extern "C" fn tl_b200_kvcache_free(handle: *const i64) {
    unsafe { ffi::tlb_kvcache_free(*handle as *mut ffi::TlbKvCache) };
}

/// The fused decode session: what a TL program (or tl_runtime's lazy layer) calls to run a whole token in one graph
/// replay instead of ~40 FFI calls per layer.
pub struct DecodeSession(*mut ffi::TlbDecoder);

impl DecodeSession {
    pub fn new(cfg: &ffi::TlbDecoderCfg, weights: *mut c_void) -> Result<Self, tl_backend::BackendError> {
        let mut d: *mut ffi::TlbDecoder = std::ptr::null_mut();
        st(unsafe { ffi::tlb_decoder_create(&mut d, cfg, weights as *mut _) })?;
        Ok(DecodeSession(d))
    }
    /// One token in, the greedy next token out (host to host).
    pub fn step(&mut self, token: i32, pos: i32) -> Result<i32, tl_backend::BackendError> {
        let mut next = -1i32;
        st(unsafe { ffi::tlb_decoder_step(self.0, token, pos, pos, &mut next) })?;
        Ok(next)
    }
    /// A whole prompt through the tensor-core path; returns the greedy token after it.
    pub fn prefill(&mut self, tokens: &[i32], pos0: i32) -> Result<i32, tl_backend::BackendError> {
        let mut next = -1i32;
        st(unsafe { ffi::tlb_decoder_prefill(self.0, tokens.as_ptr(), tokens.len() as i32, pos0, pos0, 1, &mut next) })?;
        Ok(next)
    }
}

impl Drop for DecodeSession {
    fn drop(&mut self) {
        unsafe { ffi::tlb_decoder_destroy(self.0) };
    }
}
