//! `impl IDevice for B200Device`: the back-end trait of tl_backend (crates/tl_backend/src/device.rs:19-524) over the C ABI
//! of libtlb200.  Every method on the quantized-LLM inference path delegates 1:1 to the entry point that replaces it
//! (the mapping is the comment beside each declaration in include/tlb200.h); every other method of the trait - training,
//! CNN layers, generic elementwise math, file I/O - answers `not on the path` through one macro, since this back end
//! implements that path and nothing else.  tl_runtime::device_ffi::dispatch (crates/tl_runtime/src/device_ffi.rs:84-114)
//! stores the error and returns the FFI error value, as it does for the other back ends.
//!
//! Conventions kept from the reference's GPU back ends: every op returns a new handle with reference count 1; clone /
//! acquire / prepare_return are RC + 1 on the same handle; integers (token ids, shapes) travel as f32 tensors; RoPE is
//! the CUDA back end's rotate-half form (the tl_cpu adjacent-pair form is `ffi::TLB_ROPE_CPU`, which the fused decode
//! session uses to reproduce TL_DEVICE=cpu bit for bit).
use std::ffi::{c_int, c_void, CStr};

use tl_backend::device::{BackendResult, IDevice};
use tl_backend::error::BackendError;

use crate::ffi;

pub struct B200Device;

/// RuntimeErrorCode (crates/tl_runtime/src/error.rs:7-18) -> BackendError, with the library's thread-local message.
pub(crate) fn st(code: ffi::TlbStatus) -> BackendResult<()> {
    if code == ffi::TLB_OK {
        return Ok(());
    }
    let msg = unsafe { CStr::from_ptr(ffi::tlb_last_error()) }.to_string_lossy().into_owned();
    Err(match code {
        1 => BackendError::ShapeMismatch(msg),
        2 => BackendError::DeviceError(msg),
        3 => BackendError::AllocationError(msg),
        4 => BackendError::NullPointerError(msg),
        5 => BackendError::InternalError(msg),
        6 => BackendError::IndexOutOfBounds(msg),
        7 => BackendError::TypeMismatch(msg),
        8 => BackendError::ArgumentError(msg),
        _ => BackendError::Unknown(msg),
    })
}

/// Runs an entry point that writes a new tensor handle through its first argument.
pub(crate) fn out<F: FnOnce(*mut *mut ffi::TlbTensor) -> ffi::TlbStatus>(f: F) -> BackendResult<*mut c_void> {
    let mut t: *mut ffi::TlbTensor = std::ptr::null_mut();
    st(f(&mut t))?;
    Ok(t as *mut c_void)
}

fn shape_i64(rank: usize, shape: *const usize) -> Vec<i64> {
    (0..rank).map(|i| unsafe { *shape.add(i) } as i64).collect()
}

fn not_on_path(name: &str) -> BackendError {
    BackendError::InternalError(format!("{}: not on the quantized-LLM inference path this back end implements", name))
}

/// The trait's methods outside the path: same signatures, one body.
macro_rules! off_path {
    ($( fn $name:ident ( $( $arg:ident : $ty:ty ),* ) -> $ret:ty ; )*) => {
        $( #[allow(unused_variables)] fn $name(&self, $( $arg: $ty ),* ) -> $ret { Err(not_on_path(stringify!($name))) } )*
    };
}

impl IDevice for B200Device {
    fn tensor_new(&self, data: *const f32, rank: usize, shape: *const usize) -> BackendResult<*mut c_void> {
        let dims = shape_i64(rank, shape); out(|o| unsafe { ffi::tlb_tensor_from_host(o, data as *const c_void, ffi::TLB_F32, dims.as_ptr(), rank as c_int) })
    }
    fn tensor_from_i64_array(&self, data: *const i64, len: i64) -> BackendResult<*mut c_void> {
        // TL keeps integers as f32 values (token ids, shapes): widen on the host, as tl_cuda does (crates/tl_cuda/src/ffi_ops.rs:105-116)
        let v: Vec<f32> = (0..len.max(0) as usize).map(|i| unsafe { *data.add(i) } as f32).collect();
        let dims = [len.max(0)];
        out(|o| unsafe { ffi::tlb_tensor_from_host(o, v.as_ptr() as *const c_void, ffi::TLB_F32, dims.as_ptr(), 1) })
    }
    fn tensor_zeros(&self, rank: usize, shape: *const usize, req_grad: bool) -> BackendResult<*mut c_void> {
        let _ = req_grad; let dims = shape_i64(rank, shape); out(|o| unsafe { ffi::tlb_tensor_zeros(o, ffi::TLB_F32, dims.as_ptr(), rank as c_int) })
    }
    fn tensor_new_causal_mask(&self, size: usize) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_new_causal_mask(o, size as i64) })
    }
    fn tensor_to_vec_f32(&self, t: *mut c_void) -> BackendResult<(*mut f32, usize)> {
        let n = unsafe { ffi::tlb_tensor_numel(t as *const _) }.max(0) as usize;
        let mut v = vec![0f32; n].into_boxed_slice();
        st(unsafe { ffi::tlb_tensor_to_host(t as *const _, v.as_mut_ptr() as *mut c_void, n * 4) })?;
        Ok((Box::into_raw(v) as *mut f32, n))   // the caller owns the buffer, as with the other back ends
    }
    fn tensor_scaled_dot_product_attention(&self, q: *mut c_void, k: *mut c_void, v: *mut c_void, mask: *mut c_void) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_sdpa(o, q as *const _, k as *const _, v as *const _, mask as *const _, if mask.is_null() { 0 } else { 1 }) })   // additive mask: the CUDA convention
    }
    fn tensor_top_k_sample(&self, logits: *mut c_void, k: i64) -> BackendResult<*mut c_void> {
        let _ = k; out(|o| unsafe { ffi::tlb_argmax(o, logits as *const _, ffi::TLB_TIE_FIRST) })
    }
    fn tensor_top_p_sample(&self, logits: *mut c_void, p: f64) -> BackendResult<*mut c_void> {
        let _ = p; out(|o| unsafe { ffi::tlb_argmax(o, logits as *const _, ffi::TLB_TIE_FIRST) })   // the reference's CUDA samplers are argmax (autograd.cu:2370-2446)
    }
    fn tensor_temperature_scale(&self, logits: *mut c_void, temperature: f64) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_scale(o, logits as *const _, (1.0 / temperature) as f32) })
    }
    fn tensor_repetition_penalty(&self, logits: *mut c_void, tokens: *mut c_void, penalty: f64) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_repetition_penalty(o, logits as *const _, tokens as *const _, penalty as f32) })
    }
    fn tensor_clone(&self, t: *mut c_void) -> BackendResult<*mut c_void> {
        st(unsafe { ffi::tlb_tensor_retain(t as *mut _) })?; Ok(t)   // clone on the GPU back ends is RC+1 (crates/tl_cuda/src/ffi.rs:16-26)
    }
    fn tensor_shallow_clone(&self, t: *mut c_void) -> BackendResult<*mut c_void> {
        st(unsafe { ffi::tlb_tensor_retain(t as *mut _) })?; Ok(t)
    }
    fn tensor_free(&self, t: *mut c_void) -> BackendResult<()> {
        st(unsafe { ffi::tlb_tensor_release(t as *mut _) })
    }
    fn tensor_release(&self, t: *mut c_void) -> BackendResult<()> {
        st(unsafe { ffi::tlb_tensor_release(t as *mut _) })
    }
    fn tensor_acquire(&self, t: *mut c_void) -> BackendResult<*mut c_void> {
        st(unsafe { ffi::tlb_tensor_retain(t as *mut _) })?; Ok(t)
    }
    fn tensor_release_safe(&self, t: *mut c_void) -> BackendResult<()> {
        st(unsafe { ffi::tlb_tensor_release(t as *mut _) })
    }
    fn tensor_promote(&self, t: *mut c_void) -> BackendResult<()> {
        let _ = t; Ok(())
    }
    fn tensor_register(&self, t: *mut c_void) -> BackendResult<()> {
        let _ = t; Ok(())
    }
    fn tensor_prepare_return(&self, t: *mut c_void) -> BackendResult<*mut c_void> {
        st(unsafe { ffi::tlb_tensor_retain(t as *mut _) })?; Ok(t)
    }
    fn tensor_len(&self, t: *mut c_void) -> BackendResult<usize> {
        Ok(unsafe { ffi::tlb_tensor_numel(t as *const _) }.max(0) as usize)
    }
    fn tensor_dim(&self, t: *mut c_void, dim: usize) -> BackendResult<usize> {
        let mut s = [0i64; 8];
        st(unsafe { ffi::tlb_tensor_shape(t as *const _, s.as_mut_ptr(), 8) })?;
        s.get(dim).map(|d| *d as usize).ok_or_else(|| BackendError::IndexOutOfBounds(format!("dim {} of a rank-{} tensor", dim, unsafe { ffi::tlb_tensor_rank(t as *const _) })))
    }
    fn tensor_numel(&self, t: *mut c_void) -> BackendResult<i64> {
        Ok(unsafe { ffi::tlb_tensor_numel(t as *const _) })
    }
    fn tensor_data(&self, t: *mut c_void) -> BackendResult<*const f32> {
        Ok(unsafe { ffi::tlb_tensor_data(t as *const _) } as *const f32)   // a DEVICE pointer, as with tl_cuda
    }
    fn tensor_device_id(&self, t: *mut c_void) -> BackendResult<i32> {
        let _ = t; Ok(unsafe { ffi::tlb_device_id() })
    }
    fn tensor_get_shape(&self, t: *mut c_void) -> BackendResult<*mut c_void> {
        let rank = unsafe { ffi::tlb_tensor_rank(t as *const _) }.max(0) as usize;
        let mut s = [0i64; 8];
        st(unsafe { ffi::tlb_tensor_shape(t as *const _, s.as_mut_ptr(), 8) })?;
        let v: Vec<f32> = s[..rank].iter().map(|d| *d as f32).collect();
        let dims = [rank as i64];
        out(|o| unsafe { ffi::tlb_tensor_from_host(o, v.as_ptr() as *const c_void, ffi::TLB_F32, dims.as_ptr(), 1) })
    }
    fn tensor_item(&self, t: *mut c_void) -> BackendResult<f32> {
        let n = unsafe { ffi::tlb_tensor_numel(t as *const _) };
        if n < 1 { return Err(BackendError::ShapeMismatch("item on an empty tensor".into())); }
        let flat = out(|o| { let d = [n]; unsafe { ffi::tlb_reshape(o, t as *const _, d.as_ptr(), 1) } })?;
        let first = out(|o| unsafe { ffi::tlb_narrow(o, flat as *const _, 0, 0, 1) });
        unsafe { ffi::tlb_tensor_release(flat as *mut _) };
        let first = first?;
        let mut v = 0f32;
        let r = st(unsafe { ffi::tlb_tensor_to_host(first as *const _, &mut v as *mut f32 as *mut c_void, 4) });
        unsafe { ffi::tlb_tensor_release(first as *mut _) };
        r.map(|_| v)
    }
    fn tensor_item_i64(&self, t: *mut c_void) -> BackendResult<i64> {
        let mut v = 0i64; st(unsafe { ffi::tlb_tensor_item_i64(t as *const _, &mut v) })?; Ok(v)
    }
    fn tensor_add(&self, a: *mut c_void, b: *mut c_void) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_add(o, a as *const _, b as *const _) })
    }
    fn tensor_mul(&self, a: *mut c_void, b: *mut c_void) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_mul(o, a as *const _, b as *const _) })
    }
    fn tensor_matmul(&self, a: *mut c_void, b: *mut c_void) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_matmul(o, a as *const _, b as *const _) })
    }
    fn tensor_scale(&self, t: *mut c_void, s: f32) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_scale(o, t as *const _, s) })
    }
    fn tensor_silu(&self, t: *mut c_void) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_silu(o, t as *const _) })
    }
    fn tensor_softmax(&self, t: *mut c_void, dim: i64) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_softmax(o, t as *const _, dim) })
    }
    fn tensor_argmax(&self, t: *mut c_void, dim: i64, keep_dim: bool) -> BackendResult<*mut c_void> {
        let _ = (dim, keep_dim); out(|o| unsafe { ffi::tlb_argmax(o, t as *const _, ffi::TLB_TIE_FIRST) })   // scans all elements (crates/tl_cpu/src/ffi.rs:1335-1347); first maximum, the CUDA tie rule
    }
    fn tensor_sample(&self, t: *mut c_void, temp: f32, top_p: f32) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_sample(o, t as *const _, temp, top_p, ffi::TLB_TIE_FIRST) })
    }
    fn tensor_reshape_new(&self, t: *mut c_void, new_shape: *mut c_void) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_reshape_new(o, t as *const _, new_shape as *const _) })
    }
    fn tensor_reshape_dims(&self, t: *mut c_void, dims_ptr: *const i64, rank: i64) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_reshape(o, t as *const _, dims_ptr, rank as c_int) })
    }
    fn tensor_transpose(&self, t: *mut c_void, dim0: usize, dim1: usize) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_transpose(o, t as *const _, dim0 as i64, dim1 as i64) })
    }
    fn tensor_narrow(&self, t: *mut c_void, dim: usize, start: usize, len: usize) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_narrow(o, t as *const _, dim as i64, start as i64, len as i64) })
    }
    fn tensor_cat(&self, a: *mut c_void, b: *mut c_void, dim: i64) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_cat(o, a as *const _, b as *const _, dim) })
    }
    fn tensor_cat_i64(&self, a: *mut c_void, b: *mut c_void, dim: i64) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_cat_i64(o, a as *const _, b as *const _, dim) })
    }
    fn tensor_cat2(&self, a: *mut c_void, b: *mut c_void, dim: i64) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_cat(o, a as *const _, b as *const _, dim) })
    }
    fn tensor_cat_4d(&self, a: *mut c_void, b: *mut c_void, dim: i64) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_cat(o, a as *const _, b as *const _, dim) })
    }
    fn tensor_repeat_interleave(&self, t: *mut c_void, repeats: usize, dim: usize) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_repeat_interleave(o, t as *const _, repeats as i64, dim as i64) })
    }
    fn tensor_embedding(&self, weight: *mut c_void, indices: *mut c_void, padding_idx: i64, scale_grad: bool, sparse: bool) -> BackendResult<*mut c_void> {
        let _ = (padding_idx, scale_grad, sparse); out(|o| unsafe { ffi::tlb_embedding(o, weight as *const _, indices as *const _) })
    }
    fn tensor_rms_norm(&self, input: *mut c_void, weight: *mut c_void, eps: f32) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_rms_norm(o, input as *const _, weight as *const _, eps) })
    }
    fn tensor_rope_new_cos(&self, dim: usize, seq_len: usize, base: f32) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_rope_new_cos(o, dim as i64, seq_len as i64, base, ffi::TLB_ROPE_HALF) })   // the CUDA back end's tables: [seq, dim / 2]
    }
    fn tensor_rope_new_sin(&self, dim: usize, seq_len: usize, base: f32) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_rope_new_sin(o, dim as i64, seq_len as i64, base, ffi::TLB_ROPE_HALF) })
    }
    fn tensor_apply_rope(&self, t: *mut c_void, cos: *mut c_void, sin: *mut c_void) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_apply_rope(o, t as *const _, cos as *const _, sin as *const _, ffi::TLB_ROPE_HALF) })
    }
    fn tensor_matmul_4d(&self, a: *mut c_void, b: *mut c_void) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_matmul(o, a as *const _, b as *const _) })
    }
    fn tensor_add_4d(&self, a: *mut c_void, b: *mut c_void) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_add(o, a as *const _, b as *const _) })
    }
    fn tensor_silu_4d(&self, t: *mut c_void) -> BackendResult<*mut c_void> {
        out(|o| unsafe { ffi::tlb_silu(o, t as *const _) })
    }

    off_path! {
        fn tensor_new_i64(data: *const i64, rank: usize, shape: *const usize) -> BackendResult<*mut c_void>;
        fn tensor_ones(rank: usize, shape: *const usize, req_grad: bool) -> BackendResult<*mut c_void>;
        fn tensor_randn_debug(rank: usize, shape: *const usize, seed: u64, req_grad: bool) -> BackendResult<*mut c_void>;
        fn tensor_from_vec_u8(data: *mut c_void, offset: i64, shape_ptr: *const i64, rank: i64) -> BackendResult<*mut c_void>;
        fn tensor_from_vec_u8_f32_shape(data: *mut c_void, offset: i64, shape_ptr: *const f32, rank: i64) -> BackendResult<*mut c_void>;
        fn tensor_from_u8_labels(data: *const u8, len: i64) -> BackendResult<*mut c_void>;
        fn tensor_full(rank: usize, shape: *const usize, value: f32, req_grad: bool) -> BackendResult<*mut c_void>;
        fn tensor_eye(n: usize, req_grad: bool) -> BackendResult<*mut c_void>;
        fn tensor_arange(start: f64, end: f64, step: f64) -> BackendResult<*mut c_void>;
        fn tensor_linspace(start: f64, end: f64, steps: usize) -> BackendResult<*mut c_void>;
        fn tensor_rand(rank: usize, shape: *const usize, req_grad: bool) -> BackendResult<*mut c_void>;
        fn tensor_where_cond(cond: *mut c_void, x: *mut c_void, y: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_var(t: *mut c_void, dim: i32) -> BackendResult<*mut c_void>;
        fn tensor_std(t: *mut c_void, dim: i32) -> BackendResult<*mut c_void>;
        fn tensor_prod(t: *mut c_void, dim: i32) -> BackendResult<*mut c_void>;
        fn tensor_cumsum(t: *mut c_void, dim: i32) -> BackendResult<*mut c_void>;
        fn tensor_norm(t: *mut c_void, p: f32, dim: i32) -> BackendResult<*mut c_void>;
        fn tensor_topk(t: *mut c_void, k: usize, dim: i32) -> BackendResult<*mut c_void>;
        fn tensor_logical_and(a: *mut c_void, b: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_logical_or(a: *mut c_void, b: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_logical_not(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_leaky_relu(t: *mut c_void, negative_slope: f32) -> BackendResult<*mut c_void>;
        fn tensor_elu(t: *mut c_void, alpha: f32) -> BackendResult<*mut c_void>;
        fn tensor_mish(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_mse_loss(pred: *mut c_void, target: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_l1_loss(pred: *mut c_void, target: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_bce_loss(pred: *mut c_void, target: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_nll_loss(pred: *mut c_void, target: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_linear(input: *mut c_void, weight: *mut c_void, bias: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_hardswish(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_hardsigmoid(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_group_norm(input: *mut c_void, num_groups: i64, weight: *mut c_void, bias: *mut c_void, eps: f64) -> BackendResult<*mut c_void>;
        fn tensor_adaptive_avg_pool2d(input: *mut c_void, output_h: i64, output_w: i64) -> BackendResult<*mut c_void>;
        fn tensor_pad(input: *mut c_void, pad_left: i64, pad_right: i64, value: f32) -> BackendResult<*mut c_void>;
        fn tensor_instance_norm(input: *mut c_void, weight: *mut c_void, bias: *mut c_void, eps: f64) -> BackendResult<*mut c_void>;
        fn tensor_dropout2d(input: *mut c_void, p: f64, training: bool) -> BackendResult<*mut c_void>;
        fn tensor_conv1d(input: *mut c_void, weight: *mut c_void, bias: *mut c_void, stride: i64, padding: i64) -> BackendResult<*mut c_void>;
        fn tensor_kl_div_loss(pred: *mut c_void, target: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_conv_transpose2d(input: *mut c_void, weight: *mut c_void, bias: *mut c_void, stride: i64, padding: i64, output_padding: i64) -> BackendResult<*mut c_void>;
        fn tensor_interpolate(input: *mut c_void, output_h: i64, output_w: i64, mode: i64) -> BackendResult<*mut c_void>;
        fn tensor_dot(a: *mut c_void, b: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_fill_(t: *mut c_void, value: f32) -> BackendResult<()>;
        fn tensor_broadcast_to(t: *mut c_void, shape: &[usize]) -> BackendResult<*mut c_void>;
        fn tensor_stack(a: *mut c_void, b: *mut c_void, dim: i64) -> BackendResult<*mut c_void>;
        fn tensor_get(t: *mut c_void, idx: i64) -> BackendResult<f32>;
        fn tensor_get_f32_md(t: *mut c_void, indices: *const i64, rank: i64) -> BackendResult<f32>;
        fn tensor_get_i64_md(t: *mut c_void, indices: *const i64, rank: i64) -> BackendResult<i64>;
        fn tensor_set_f32_md(t: *mut c_void, indices: *const i64, rank: usize, value: f32) -> BackendResult<*mut c_void>;
        fn tensor_sub(a: *mut c_void, b: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_div(a: *mut c_void, b: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_rem(a: *mut c_void, b: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_pow(a: *mut c_void, b: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_cross_entropy(logits: *mut c_void, labels: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_neg(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_abs(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_contiguous(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_eq(a: *mut c_void, b: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_neq(a: *mut c_void, b: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_gt(a: *mut c_void, b: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_lt(a: *mut c_void, b: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_ge(a: *mut c_void, b: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_le(a: *mut c_void, b: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_add_scalar(t: *mut c_void, s: f64) -> BackendResult<*mut c_void>;
        fn tensor_sub_scalar(t: *mut c_void, s: f64) -> BackendResult<*mut c_void>;
        fn tensor_mul_scalar(t: *mut c_void, s: f64) -> BackendResult<*mut c_void>;
        fn tensor_div_scalar(t: *mut c_void, s: f64) -> BackendResult<*mut c_void>;
        fn tensor_pow_scalar(t: *mut c_void, exp: f32) -> BackendResult<*mut c_void>;
        fn tensor_add_assign(a: *mut c_void, b: *mut c_void) -> BackendResult<()>;
        fn tensor_sub_assign(a: *mut c_void, b: *mut c_void) -> BackendResult<()>;
        fn tensor_mul_assign(a: *mut c_void, b: *mut c_void) -> BackendResult<()>;
        fn tensor_div_assign(a: *mut c_void, b: *mut c_void) -> BackendResult<()>;
        fn tensor_mod_assign(a: *mut c_void, b: *mut c_void) -> BackendResult<()>;
        fn tensor_add_assign_scalar_f32(t: *mut c_void, s: f32) -> BackendResult<()>;
        fn tensor_sub_assign_scalar_f32(t: *mut c_void, s: f32) -> BackendResult<()>;
        fn tensor_mul_assign_scalar_f32(t: *mut c_void, s: f32) -> BackendResult<()>;
        fn tensor_div_assign_scalar_f32(t: *mut c_void, s: f32) -> BackendResult<()>;
        fn tensor_mod_assign_scalar_f32(t: *mut c_void, s: f32) -> BackendResult<()>;
        fn tensor_exp(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_log(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_sqrt(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_sin(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_cos(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_tan(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_tanh(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_sigmoid(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_relu(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_gelu(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_sum(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_mean(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_max(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_min(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_max_dim(t: *mut c_void, dim: usize, keep_dim: bool) -> BackendResult<*mut c_void>;
        fn tensor_min_dim(t: *mut c_void, dim: usize, keep_dim: bool) -> BackendResult<*mut c_void>;
        fn tensor_mean_dim(t: *mut c_void, dim: usize, keep_dim: bool) -> BackendResult<*mut c_void>;
        fn tensor_sum_dim(t: *mut c_void, dim: usize, keep_dim: bool) -> BackendResult<*mut c_void>;
        fn tensor_argmin(t: *mut c_void, dim: i64, keep_dim: bool) -> BackendResult<*mut c_void>;
        fn tensor_tril(t: *mut c_void, diagonal: i64) -> BackendResult<*mut c_void>;
        fn tensor_masked_fill_scalar(t: *mut c_void, mask: *mut c_void, value: f64) -> BackendResult<*mut c_void>;
        fn tensor_clamp(t: *mut c_void, min: f64, max: f64) -> BackendResult<*mut c_void>;
        fn tensor_backward(t: *mut c_void) -> BackendResult<()>;
        fn tensor_grad(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_detach(t: *mut c_void, req_grad: bool) -> BackendResult<*mut c_void>;
        fn tensor_enable_grad(t: *mut c_void) -> BackendResult<()>;
        fn tensor_set_requires_grad(t: *mut c_void, req_grad: bool) -> BackendResult<()>;
        fn clear_grads() -> BackendResult<()>;
        fn tensor_clip_grad_value(t: *mut c_void, min: f64, max: f64) -> BackendResult<()>;
        fn tensor_clip_grad_norm(t: *mut c_void, max_norm: f64, norm_type: f64) -> BackendResult<f64>;
        fn tensor_slice(t: *mut c_void, dim: i64, start: i64, len: i64) -> BackendResult<*mut c_void>;
        fn tensor_replace_data(dst: *mut c_void, src: *mut c_void) -> BackendResult<()>;
        fn tensor_to_device(t: *mut c_void, device_id: i32) -> BackendResult<*mut c_void>;
        fn tensor_to_f32(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_to_i64(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_print(t: *mut c_void) -> BackendResult<()>;
        fn tensor_display(t: *mut c_void) -> BackendResult<()>;
        fn tensor_print_1(t: *mut c_void) -> BackendResult<()>;
        fn tensor_print_2(t: *mut c_void) -> BackendResult<()>;
        fn tensor_print_3(t: *mut c_void) -> BackendResult<()>;
        fn tensor_save(t: *mut c_void, path: *const i8) -> BackendResult<()>;
        fn tensor_load(path: *const i8) -> BackendResult<*mut c_void>;
        fn tensor_conv2d(input: *mut c_void, weight: *mut c_void, bias: *mut c_void, stride: usize, padding: usize, dilation: usize, groups: usize) -> BackendResult<*mut c_void>;
        fn tensor_batch_norm(input: *mut c_void, running_mean: *mut c_void, running_var: *mut c_void, weight: *mut c_void, bias: *mut c_void, training: bool, momentum: f64, eps: f64) -> BackendResult<*mut c_void>;
        fn tensor_layer_norm(input: *mut c_void, weight: *mut c_void, bias: *mut c_void, eps: f64) -> BackendResult<*mut c_void>;
        fn tensor_dropout(input: *mut c_void, p: f64, training: bool) -> BackendResult<*mut c_void>;
        fn tensor_max_pool2d(input: *mut c_void, kernel_size: usize, stride: usize, padding: usize) -> BackendResult<*mut c_void>;
        fn tensor_avg_pool2d(input: *mut c_void, kernel_size: usize, stride: usize, padding: usize) -> BackendResult<*mut c_void>;
        fn tensor_transpose_2d(t: *mut c_void) -> BackendResult<*mut c_void>;
        fn tensor_reshape_2d(t: *mut c_void, d0: i64, d1: i64) -> BackendResult<*mut c_void>;
        fn tensor_reshape_3d_to_2d(t: *mut c_void, d0: i64, d1: i64) -> BackendResult<*mut c_void>;
    }
}
