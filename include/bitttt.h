/*
 * bitttt.h - C ABI of the B200 (sm_100a) BitLinear inference library.
 *
 * Plain pointers and sizes only; every entry point returns a bt_status (0 = ok,
 * negative = error) and never aborts or traps.  bt_last_error() gives the message of
 * the calling thread's last failure, with the reference's wording for shape errors.
 *
 * Each declaration names the interface of Bit-TTT-Engine that it stands in for
 * (paths relative to the reference project root, RE = crates/rust_engine/src).
 *
 * Pointers named *_dev are CUDA device pointers on the handle's device; *_host are
 * host pointers.  `stream` is a cudaStream_t passed as void* (NULL = default stream).
 * Calls are asynchronous on that stream unless stated otherwise.
 */
#ifndef BITTTT_H
#define BITTTT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int bt_status;
enum {
    BT_OK = 0,
    BT_ERR_SHAPE = -1,   /* dimension mismatch (reference: "Shape mismatch: Input [..] vs Weight [..]") */
    BT_ERR_ALIGN = -2,   /* K % 4 != 0, misaligned pointer */
    BT_ERR_DEVICE = -3,  /* no CUDA device / wrong device */
    BT_ERR_CUDA = -4,    /* a CUDA runtime call failed */
    BT_ERR_NCCL = -5,
    BT_ERR_TIMEOUT = -6, /* a bounded device-side wait ran out */
    BT_ERR_NOMEM = -7,
    BT_ERR_ARG = -8      /* null pointer, unsupported dtype or option */
};

typedef enum { BT_F32 = 0, BT_BF16 = 1, BT_I8 = 2, BT_I32 = 3 } bt_dtype;

/* Message of the calling thread's last failed call ("" if none). */
const char* bt_last_error(void);
/* Library version, major*10000 + minor*100 + patch. */
int bt_version(void);
/* Number of CUDA devices visible (0 if none); never fails. */
int bt_device_count(void);
/* Synchronises `device` and reports a sticky device-side error (bounded wait that ran
 * out) recorded by any kernel of this library since the last call. */
bt_status bt_device_check(int device);

/* ---- packing (host) ----------------------------------------------------------------- */

/* PackedTensor::pack, RE/kernels/packing.rs:50-105: scale = mean|w| + 1e-6,
 * q = clamp(round(w/scale),-1,1), 2-bit codes 00/01/10 = 0/+1/-1, four per byte, LSB
 * first.  out_host holds ceil(n_elem/4) bytes. */
bt_status bt_pack_ternary(const float* w_host, int64_t n_elem, uint8_t* out_host, float* scale_out);
/* PackedTensor::unpack, RE/kernels/packing.rs:108-133. */
bt_status bt_unpack_ternary(const uint8_t* packed_host, int64_t n_elem, float scale, float* out_host);

/* ---- BitLinear ---------------------------------------------------------------------- */

typedef struct bt_linear bt_linear;

/* Stands in for BitLinear::load + precompute_packed (RE/layers/bit_linear.rs:24-50) and
 * for AdaptiveBitLinear::load (RE/layers/adaptive_linear.rs:40-129).
 * packed_host: the packed bytes exactly as the reference stores them:
 *   n_bases == 1: PackedTensor.data, row-major [n_out, k_in/4] (RE/kernels/packing.rs:15-21);
 *   n_bases  > 1: `weight_packed` of a converted checkpoint, [n_out, k_in/4, n_bases]
 *                 (tools/conversion/convert_llama_v2.py:111-151).
 * scales_host: n_bases floats.  k_in must be a multiple of 4 (BT_ERR_ALIGN otherwise;
 * the reference's packer and kernels disagree for such shapes).  The bytes are copied to
 * `device` once, into the library's own streaming layout; the handle is immutable
 * afterwards and may be used from several host threads at once, each with its own
 * workspace and stream.  Synchronous. */
bt_status bt_linear_create(bt_linear** out, const uint8_t* packed_host, int64_t n_out,
                           int64_t k_in, int n_bases, const float* scales_host, int device);
bt_status bt_linear_destroy(bt_linear* lin);
bt_status bt_linear_dims(const bt_linear* lin, int64_t* n_out, int64_t* k_in, int* n_bases);

/* Scratch memory for forward calls (quantised activations).  One workspace serves one
 * stream at a time.  bytes = 0 picks a size good for m <= 64 at k_in <= 16384. */
typedef struct bt_workspace bt_workspace;
bt_status bt_workspace_create(bt_workspace** out, int device, size_t bytes);
bt_status bt_workspace_destroy(bt_workspace* ws);

/* Stands in for BitLinearCuda::forward / BitLinearCpu::forward
 * (RE/kernels/cuda.rs:21-47, RE/kernels/cpu.rs:17-127) as called from BitLinear::forward
 * (RE/layers/bit_linear.rs:65-85): y[m, n_out] = x[m, k_in] . W^T with per-token absmax
 * int8 quantisation of x in front:  y = sum_b ((float)acc_b * scale_b) * s_x[m].
 * x_dtype: BT_F32 or BT_BF16; y_dtype: BT_F32 or BT_BF16.  x_k must equal the handle's
 * k_in, else BT_ERR_SHAPE with the reference's message.  ws may be NULL: a workspace
 * owned by the handle is then used (allocated on first use; calls on one handle with
 * ws == NULL must not overlap). */
bt_status bt_linear_forward(bt_linear* lin, bt_workspace* ws, const void* x_dev, int64_t m,
                            int64_t x_k, bt_dtype x_dtype, void* y_dev, bt_dtype y_dtype,
                            void* stream);

/* Same product on activations that are already int8 (row-major [m, k_in]).  out_dtype
 * BT_I32: raw integer accumulators sum_k q*t of basis 0, [m, n_out] (the bit-exact
 * check against RE/kernels/cpu.rs:73-124 on integer-valued inputs).  BT_F32: scaled like
 * bt_linear_forward using sx_dev[m]. */
bt_status bt_linear_forward_q(bt_linear* lin, bt_workspace* ws, const int8_t* q_dev,
                              const float* sx_dev, int64_t m, void* out_dev,
                              bt_dtype out_dtype, void* stream);

/* Host-buffer convenience with the reference's calling convention for a CUDA device:
 * x and y live in host memory, as the reference's PackedTensor path moves data over
 * PCIe on every call (RE/kernels/cuda.rs:40-42, RE/kernels/packing.rs:108-133).  f32 in,
 * f32 out.  Synchronous. */
bt_status bt_linear_forward_host(bt_linear* lin, const float* x_host, int64_t m, int64_t x_k,
                                 float* y_host);

/* Per-token absmax int8 quantiser (no counterpart kernel in the reference; defined
 * after QuantizedKVCache::quantize_q8, RE/layers/kv_cache.rs:95-119, without the +128
 * zero point): s = max|x|/127, q = clamp(round(x/s), -127, 127), s == 0 -> q = 0.
 * q_dev [m,k] int8, s_dev [m] f32, qsum_dev [m] int32 (sum_k q, may be NULL). */
bt_status bt_act_quant(const void* x_dev, bt_dtype x_dtype, int64_t m, int64_t k, int8_t* q_dev,
                       float* s_dev, int32_t* qsum_dev, int device, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* BITTTT_H */
