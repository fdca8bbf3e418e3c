//! tl_b200: the B200 back end of TL's quantized-LLM inference path.
//!
//! All arithmetic lives in libtlb200 (hand-written sm_100a CUDA kernels behind a C ABI, include/tlb200.h); this crate
//! is the thin Rust side the reference's crates expect:
//!   * `ffi`          - the C ABI, declaration for declaration;
//!   * `b200_device`  - `impl tl_backend::IDevice for B200Device`, 1:1 delegation for the methods on the path;
//!   * `stream`       - `GpuStream` / `GpuGraph` over tlb_stream_* / tlb_graph_*;
//!   * `quantized`    - what tl_runtime's quantized entry points call instead of their tl_cuda branch: the GGUF loader
//!                      that repacks once, `tl_qtensor_matmul`, and the fused decode session;
//!   * the raw-bytes symbols `tl_cuda_mul_mv_q4_k` / `tl_cuda_mul_mv_q6_k` come from libtlb200 itself under the
//!     reference's names (crates/tl_runtime/src/device_ffi.rs:1805-1833 resolves them at link time).
//! There is no CPU fallback and no dispatch over other back ends in here: without a usable B200 every call returns the
//! library's DeviceError.
pub mod b200_device;
pub mod ffi;
pub mod quantized;
pub mod stream;

pub use b200_device::B200Device;

/// The device object tl_runtime::device_ffi::dispatch hands its closures (one per process, as `CudaDeviceImpl` is).
pub static B200_DEVICE: B200Device = B200Device;

/// Binds the GPU (`device < 0`: LOCAL_RANK, else 0).  Called once from tl_runtime's device selection.
pub fn init(device: i32) -> Result<(), tl_backend::BackendError> {
    b200_device::st(unsafe { ffi::tlb_init(device) })
}
