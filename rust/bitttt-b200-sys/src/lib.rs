//! Rust side of the C ABI in `include/bitttt.h`.
//!
//! * [`ffi`]: one `extern "C"` declaration per entry point of the header, same order.
//! * [`BitLinearCuda`] (feature `candle`): the drop-in for `BitLinearCuda::forward` of the
//!   reference engine (`crates/rust_engine/src/kernels/cuda.rs:21-47`): it takes the input tensor
//!   and the `PackedTensor` fields, pulls the device pointers out of the candle storages the way
//!   `kernels/cuda.rs:70-107` does, and calls `bt_linear_forward`.  The packed bytes are uploaded
//!   once per layer (`BitLinearCuda::new`), not on every call.
//!
//! This crate has not been compiled in the environment it was written in (no Rust toolchain
//! there); it is meant to be checked with `cargo check --features candle` on a machine that has one.
#![allow(non_camel_case_types)]

pub mod ffi {
    use core::ffi::{c_char, c_double, c_float, c_int, c_void};

    pub type bt_status = c_int;
    pub const BT_OK: bt_status = 0;
    pub const BT_ERR_SHAPE: bt_status = -1;
    pub const BT_ERR_ALIGN: bt_status = -2;
    pub const BT_ERR_DEVICE: bt_status = -3;
    pub const BT_ERR_CUDA: bt_status = -4;
    pub const BT_ERR_NCCL: bt_status = -5;
    pub const BT_ERR_TIMEOUT: bt_status = -6;
    pub const BT_ERR_NOMEM: bt_status = -7;
    pub const BT_ERR_ARG: bt_status = -8;

    pub type bt_dtype = c_int;
    pub const BT_F32: bt_dtype = 0;
    pub const BT_BF16: bt_dtype = 1;
    pub const BT_I8: bt_dtype = 2;
    pub const BT_I32: bt_dtype = 3;
    pub const BT_F16: bt_dtype = 4;

    #[repr(C)]
    pub struct bt_linear { _private: [u8; 0] }
    #[repr(C)]
    pub struct bt_workspace { _private: [u8; 0] }
    #[repr(C)]
    pub struct bt_kv_cache { _private: [u8; 0] }
    #[repr(C)]
    pub struct bt_model { _private: [u8; 0] }

    #[repr(C)]
    #[derive(Clone, Copy, Debug)]
    pub struct bt_model_config {
        pub arch: c_int,
        pub vocab_size: c_int,
        pub hidden_dim: c_int,
        pub num_layers: c_int,
        pub n_heads: c_int,
        pub n_kv_heads: c_int,
        pub intermediate_dim: c_int,
        pub inner_lr: c_float,
        pub rope_theta: c_double,
        pub max_position_embeddings: c_int,
        pub max_batch: c_int,
        pub tp_rank: c_int,
        pub tp_size: c_int,
    }

    pub type bt_weight_kind = c_int; // BT_W_Q = 0 .. BT_W_TTT_UP = 8
    pub type bt_tensor_kind = c_int; // BT_T_EMBED = 0 .. BT_T_NORM2 = 4

    extern "C" {
        pub fn bt_last_error() -> *const c_char;
        pub fn bt_version() -> c_int;
        pub fn bt_device_count() -> c_int;
        pub fn bt_device_check(device: c_int) -> bt_status;

        pub fn bt_pack_ternary(w_host: *const c_float, n_elem: i64, out_host: *mut u8, scale_out: *mut c_float) -> bt_status;
        pub fn bt_unpack_ternary(packed_host: *const u8, n_elem: i64, scale: c_float, out_host: *mut c_float) -> bt_status;
        pub fn bt_convert_l3_to_l2(l3_host: *const i8, n_out: i64, k_in: i64, n_bases: c_int, l2_out_host: *mut u8) -> bt_status;

        pub fn bt_linear_create(out: *mut *mut bt_linear, packed_host: *const u8, n_out: i64, k_in: i64, n_bases: c_int,
                                scales_host: *const c_float, device: c_int) -> bt_status;
        pub fn bt_linear_destroy(lin: *mut bt_linear) -> bt_status;
        pub fn bt_linear_dims(lin: *const bt_linear, n_out: *mut i64, k_in: *mut i64, n_bases: *mut c_int) -> bt_status;
        pub fn bt_workspace_create(out: *mut *mut bt_workspace, device: c_int, bytes: usize) -> bt_status;
        pub fn bt_workspace_destroy(ws: *mut bt_workspace) -> bt_status;
        pub fn bt_linear_forward(lin: *mut bt_linear, ws: *mut bt_workspace, x_dev: *const c_void, m: i64, x_k: i64,
                                 x_dtype: bt_dtype, y_dev: *mut c_void, y_dtype: bt_dtype, stream: *mut c_void) -> bt_status;
        pub fn bt_linear_forward_q(lin: *mut bt_linear, ws: *mut bt_workspace, q_dev: *const i8, sx_dev: *const c_float, m: i64,
                                   out_dev: *mut c_void, out_dtype: bt_dtype, stream: *mut c_void) -> bt_status;
        pub fn bt_linear_forward_host(lin: *mut bt_linear, x_host: *const c_float, m: i64, x_k: i64, y_host: *mut c_float) -> bt_status;
        pub fn bt_act_quant(x_dev: *const c_void, x_dtype: bt_dtype, m: i64, k: i64, q_dev: *mut i8, s_dev: *mut c_float,
                            qsum_dev: *mut i32, device: c_int, stream: *mut c_void) -> bt_status;
        pub fn bt_linear_forward_noalloc(lin: *mut bt_linear, x_dev: *const c_void, m: i64, x_k: i64, x_dtype: bt_dtype,
                                         y_dev: *mut c_void, y_dtype: bt_dtype, stream: *mut c_void) -> bt_status;
        pub fn bt_linear_create_fused(out: *mut *mut bt_linear, seg_packed_host: *const *const u8, seg_rows: *const i64,
                                      seg_scales: *const c_float, n_seg: c_int, k_in: i64, device: c_int) -> bt_status;

        pub fn bt_ttt_update(w_state_dev: *mut c_float, feat_dev: *const c_float, batch: i64, t_len: i64, d: i64,
                             inner_lr: c_float, chunk: i64, z_dev: *mut c_float, device: c_int, stream: *mut c_void) -> bt_status;

        pub fn bt_kv_create(out: *mut *mut bt_kv_cache, batch: i64, n_kv_heads: i64, head_dim: i64, max_seq_len: i64,
                            device: c_int) -> bt_status;
        pub fn bt_kv_reset(cache: *mut bt_kv_cache) -> bt_status;
        pub fn bt_kv_destroy(cache: *mut bt_kv_cache) -> bt_status;
        pub fn bt_kv_export(cache: *mut bt_kv_cache, b: i64, t_len: i64, k_q_host: *mut u8, k_s_host: *mut c_float,
                            v_q_host: *mut u8, v_s_host: *mut c_float) -> bt_status;
        pub fn bt_kv_import(cache: *mut bt_kv_cache, b: i64, t_len: i64, k_q_host: *const u8, k_s_host: *const c_float,
                            v_q_host: *const u8, v_s_host: *const c_float) -> bt_status;
        pub fn bt_kv_append(cache: *mut bt_kv_cache, k_dev: *const c_float, v_dev: *const c_float, pos_dev: *const i32,
                            batch: i64, stream: *mut c_void) -> bt_status;
        pub fn bt_attn_decode(cache: *mut bt_kv_cache, qkv_dev: *const c_float, pos_dev: *const i32, batch: i64, n_heads: i64,
                              rope_theta: c_double, out_dev: *mut c_float, stream: *mut c_void) -> bt_status;

        pub fn bt_model_create(out: *mut *mut bt_model, cfg: *const bt_model_config, device: c_int) -> bt_status;
        pub fn bt_tp_unique_id(id128_out: *mut u8) -> bt_status;
        pub fn bt_model_tp_init(m: *mut bt_model, id128: *const u8) -> bt_status;
        pub fn bt_model_tp_peer_export(m: *mut bt_model, handle64_out: *mut u8) -> bt_status;
        pub fn bt_model_tp_peer_import(m: *mut bt_model, handles: *const u8) -> bt_status;
        pub fn bt_model_tp_set_timeout(m: *mut bt_model, milliseconds: c_int) -> bt_status;
        pub fn bt_model_tp_destroy(m: *mut bt_model) -> bt_status;
        pub fn bt_model_tp_resync(m: *mut bt_model) -> bt_status;
        pub fn bt_model_set_linear(m: *mut bt_model, layer: c_int, kind: bt_weight_kind, packed_host: *const u8, n_out: i64,
                                   k_in: i64, scale: c_float) -> bt_status;
        pub fn bt_model_set_linear_bases(m: *mut bt_model, layer: c_int, kind: bt_weight_kind, packed_host: *const u8, n_out: i64,
                                         k_in: i64, n_bases: c_int, scales_host: *const c_float) -> bt_status;
        pub fn bt_model_set_tensor(m: *mut bt_model, kind: bt_tensor_kind, layer: c_int, data_host: *const c_float, n_elem: i64) -> bt_status;
        pub fn bt_model_set_tensor_typed(m: *mut bt_model, kind: bt_tensor_kind, layer: c_int, data_host: *const c_float,
                                         n_elem: i64, storage: bt_dtype) -> bt_status;
        pub fn bt_model_finalize(m: *mut bt_model) -> bt_status;
        pub fn bt_model_destroy(m: *mut bt_model) -> bt_status;
        pub fn bt_model_reset(m: *mut bt_model) -> bt_status;
        pub fn bt_model_forward_one(m: *mut bt_model, tokens_host: *const i32, batch: c_int, logits_host: *mut c_float,
                                    next_host: *mut i32) -> bt_status;
        pub fn bt_model_step_dev(m: *mut bt_model, tokens_dev: *const i32, batch: c_int, stream: *mut c_void) -> bt_status;
        pub fn bt_model_prefill(m: *mut bt_model, tokens_host: *const i32, batch: c_int, n_tokens: c_int, ttt_chunk: c_int,
                                logits_host: *mut c_float, next_host: *mut i32) -> bt_status;
        pub fn bt_model_logits(m: *mut bt_model) -> *const c_float;
        pub fn bt_model_next(m: *mut bt_model) -> *const i32;
        pub fn bt_model_pos(m: *const bt_model) -> c_int;
        pub fn bt_model_seek(m: *mut bt_model, pos: c_int) -> bt_status;
        pub fn bt_model_ttt_state(m: *mut bt_model, layer: c_int) -> *mut c_float;
        pub fn bt_model_kv_cache(m: *mut bt_model, layer: c_int) -> *mut bt_kv_cache;
        pub fn bt_model_trace_floats(m: *const bt_model, rows: c_int) -> i64;
        pub fn bt_model_set_trace(m: *mut bt_model, trace_dev: *mut c_float, rows: c_int) -> bt_status;
        pub fn bt_model_ternary_bytes(m: *const bt_model) -> i64;
        pub fn bt_model_enqueue_products(m: *mut bt_model, batch: c_int, as_in_step: c_int, stream: *mut c_void,
                                         n_launches: *mut c_int) -> bt_status;
        pub fn bt_model_launches_per_step(m: *const bt_model, batch: c_int) -> c_int;
    }
}

/// Message of the calling thread's last failed call.
pub fn last_error() -> String {
    unsafe {
        let p = ffi::bt_last_error();
        if p.is_null() { String::new() } else { std::ffi::CStr::from_ptr(p).to_string_lossy().into_owned() }
    }
}

#[derive(Debug)]
pub struct Error { pub status: ffi::bt_status, pub message: String }

impl std::fmt::Display for Error {
    fn fmt(&self, f: &mut std::fmt::Formatter<'_>) -> std::fmt::Result { write!(f, "[bt_status {}] {}", self.status, self.message) }
}
impl std::error::Error for Error {}

fn check(status: ffi::bt_status) -> Result<(), Error> {
    if status == ffi::BT_OK { Ok(()) } else { Err(Error { status, message: last_error() }) }
}

/// Owned handle of one packed BitLinear on the device (`BitLinear::precompute_packed`,
/// `layers/bit_linear.rs:44-50`: the bytes of `PackedTensor.data` and its scale).
pub struct PackedLinear { raw: *mut ffi::bt_linear }

unsafe impl Send for PackedLinear {}
unsafe impl Sync for PackedLinear {} // the handle is immutable after creation (include/bitttt.h)

impl PackedLinear {
    /// `packed`: `[out_features, in_features / 4]` bytes, or `[out, in/4, n_bases]` with `scales.len()` bases.
    pub fn new(packed: &[u8], out_features: usize, in_features: usize, scales: &[f32], device: i32) -> Result<Self, Error> {
        assert_eq!(packed.len(), out_features * (in_features / 4) * scales.len());
        let mut raw = core::ptr::null_mut();
        check(unsafe {
            ffi::bt_linear_create(&mut raw, packed.as_ptr(), out_features as i64, in_features as i64, scales.len() as i32,
                                  scales.as_ptr(), device)
        })?;
        Ok(Self { raw })
    }

    /// `y[m, out] = x[m, in] . W^T` on raw device pointers (f32 in, f32 out), `stream` a `cudaStream_t`.
    ///
    /// # Safety
    /// `x_dev` / `y_dev` must be device pointers on the handle's device, valid for `m * in` / `m * out` floats.
    pub unsafe fn forward_raw(&self, x_dev: *const f32, m: usize, in_features: usize, y_dev: *mut f32,
                              stream: *mut core::ffi::c_void) -> Result<(), Error> {
        check(ffi::bt_linear_forward(self.raw, core::ptr::null_mut(), x_dev as *const _, m as i64, in_features as i64, ffi::BT_F32,
                                     y_dev as *mut _, ffi::BT_F32, stream))
    }
}

impl Drop for PackedLinear {
    fn drop(&mut self) { unsafe { ffi::bt_linear_destroy(self.raw); } }
}

#[cfg(feature = "candle")]
pub use with_candle::BitLinearCuda;

#[cfg(feature = "candle")]
mod with_candle {
    use super::{Error, PackedLinear};
    use candle_core::cuda_backend::cudarc::driver::DevicePtr;
    use candle_core::{DType, Device, Result, Storage, Tensor};

    /// Stands in for `BitLinearCuda` of `crates/rust_engine/src/kernels/cuda.rs:16-47`.  The reference
    /// copies the packed bytes to the host, unpacks them, uploads an f32 matrix and runs a dense GEMM on
    /// every call; here the packed bytes go to the device once and every call streams them as 2-bit tiles.
    pub struct BitLinearCuda { lin: PackedLinear, in_features: usize, out_features: usize }

    impl BitLinearCuda {
        /// From the fields of a `PackedTensor` (`kernels/packing.rs:15-21`): `data` as host bytes, `scale`, shape.
        pub fn new(data: &[u8], scale: f32, out_features: usize, in_features: usize, device_ordinal: usize) -> std::result::Result<Self, Error> {
            Ok(Self { lin: PackedLinear::new(data, out_features, in_features, &[scale], device_ordinal as i32)?, in_features, out_features })
        }

        /// `forward(input [M, K] f32 on a CUDA device) -> [M, N] f32`, the contract of `kernels/cuda.rs:21-24`.
        pub fn forward(&self, input: &Tensor) -> Result<Tensor> {
            let (m, k) = input.dims2()?;
            if k != self.in_features {
                // wording of kernels/cuda.rs:27-35
                candle_core::bail!("Shape mismatch: Input [{}, {}] vs Weight [{}, {}]", m, k, self.out_features, self.in_features);
            }
            let dev = match input.device() {
                Device::Cuda(d) => d.clone(),
                _ => candle_core::bail!("BitLinearCuda called on non-CUDA device"), // kernels/cuda.rs:45
            };
            let input = input.contiguous()?;
            // raw pointers out of the candle storages, read guards dropped at once (kernels/cuda.rs:70-107)
            let inp_ptr = {
                let (storage, _layout) = input.storage_and_layout();
                match &*storage {
                    Storage::Cuda(s) => *s.as_cuda_slice::<f32>()?.device_ptr(),
                    _ => candle_core::bail!("Input must be CUDA F32"),
                }
            };
            let output = Tensor::zeros((m, self.out_features), DType::F32, &Device::Cuda(dev))?;
            let out_ptr = {
                let (storage, _layout) = output.storage_and_layout();
                match &*storage {
                    Storage::Cuda(s) => *s.as_cuda_slice::<f32>()?.device_ptr(),
                    _ => candle_core::bail!("Output alloc failed"),
                }
            };
            // candle 0.8 issues its kernels on the device's default stream; NULL selects the same one
            unsafe {
                self.lin
                    .forward_raw(inp_ptr as usize as *const f32, m, k, out_ptr as usize as *mut f32, core::ptr::null_mut())
                    .map_err(candle_core::Error::wrap)?;
            }
            Ok(output)
        }
    }
}
