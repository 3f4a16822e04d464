// Shared declarations of the library's CUDA translation units: status handling, the
// tiled weight layout, PTX wrappers (mbarrier, bulk copy, mma) and launch entry points.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>

#include "../../include/bitttt.h"

namespace bt {

// ---------------------------------------------------------------------------------------
// Errors
// ---------------------------------------------------------------------------------------
bt_status set_error(bt_status code, const char* fmt, ...);
void clear_error();

#define BT_CUDA_TRY(expr)                                                                   \
    do {                                                                                    \
        cudaError_t _e = (expr);                                                            \
        if (_e != cudaSuccess)                                                              \
            return bt::set_error(BT_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,               \
                                 cudaGetErrorString(_e), __FILE__, __LINE__);               \
    } while (0)

// Sticky device-side error word (one per device, allocated on first use).  Kernels write
// a non-zero code when a bounded wait runs out; bt_device_check reads and clears it.
unsigned int* device_error_word(int device);
int device_sm_count(int device);

// RAII device switch.
struct DeviceGuard {
    int prev = -1;
    bool ok = true;
    explicit DeviceGuard(int dev) {
        if (cudaGetDevice(&prev) != cudaSuccess) { ok = false; return; }
        if (prev != dev && cudaSetDevice(dev) != cudaSuccess) ok = false;
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

// ---------------------------------------------------------------------------------------
// Tiled weight layout ("streaming layout") held in device memory
// ---------------------------------------------------------------------------------------
// One tile = 16 output rows x 256 inputs of ONE basis = 4096 two-bit fields = 1024 bytes.
// Inside a tile, lane L = 4*g + t of a warp (g = L/4, t = L%4) owns two 16-byte chunks:
//   bytes [16*L, 16*L+16)        : row g      , inputs [64*t, 64*t+64) of the tile
//   bytes [512+16*L, 512+16*L+16): row g + 8  , same inputs
// so one warp-wide 16-byte load is 512 contiguous bytes and lands directly in the A
// operand slots of mma.m16n8k32.  Each 2-bit field holds u = t + 1 (t the ternary value:
// 0 -> -1, 1 -> 0, 2 -> +1) instead of the reference's code (00/01/10 = 0/+1/-1,
// kernels/packing.rs:9-13), which lets a single AND isolate a field as an unsigned
// multiple of 4^r; the kernels subtract sum_k q once per token to undo the +1.
// Reference code 11 (decodes to 0, kernels/cpu.rs:59) becomes u = 1.
// Tiles are ordered [basis][row_tile][k_tile]; rows >= n_out and inputs >= k_in are
// padded with u = 1 (weight 0).
constexpr int kTileRows = 16;
constexpr int kTileK = 256;
constexpr int kTileBytes = 1024;

struct TiledWeights {
    const uint8_t* tiles = nullptr;  // device
    int64_t n_out = 0, k_in = 0;
    int64_t row_tiles = 0, k_tiles = 0;
    int n_bases = 1;
    int64_t basis_stride() const { return row_tiles * k_tiles * kTileBytes; }
    int64_t k_pad() const { return k_tiles * kTileK; }
};

// Epilogue selector of the ternary product kernels.
enum Epilogue : int {
    EPI_I32 = 0,        // raw accumulators, int32 [m, n]
    EPI_F32 = 1,        // (acc * s_w) * s_x[m]           -> f32 [m, n]
    EPI_F32_ACCUM = 2,  // out += (acc * s_w) * s_x[m]    (further bases)
    EPI_BF16 = 3,       // bf16((acc * s_w) * s_x[m])
    EPI_SWIGLU = 4,     // rows 0-7 of a tile = gate j, rows 8-15 = up j: out[m, j] = silu(gate)*up
};

// ---------------------------------------------------------------------------------------
// Kernel launchers (defined in the .cu files)
// ---------------------------------------------------------------------------------------

// Re-tiles packed bytes (layout [n_out, k_in/4, n_bases], n_bases = 1 is the in-memory
// PackedTensor layout) that already sit in device memory into the streaming layout.
cudaError_t launch_retile(const uint8_t* src_dev, int64_t n_out, int64_t k_in, int n_bases,
                          uint8_t* tiles_dev, int64_t row_tiles, int64_t k_tiles,
                          cudaStream_t stream);

// Per-token absmax int8 quantiser.  q rows are written with stride q_stride (>= k, bytes
// between k and q_stride are zeroed).  qsum may be null.
cudaError_t launch_act_quant(const void* x, bt_dtype x_dtype, int64_t m, int64_t k, int8_t* q,
                             int64_t q_stride, float* s, int32_t* qsum, cudaStream_t stream);

// Where the int8 activations of a ternary product come from.
enum Prologue : int {
    PRO_Q8 = 0,       // already quantised in global memory (q, qsum, sx)
    PRO_RMSNORM = 1,  // x f32 -> RMSNorm with norm_w -> per-token absmax quantisation, in the kernel
    PRO_ABSMAX = 2,   // x f32 with its per-token max|x| already known (absmax_in) -> quantisation
};

// Ternary product for up to 8 tokens per launch.
struct GemvArgs {
    const uint8_t* tiles;   // one basis
    int64_t row_tiles, k_tiles, n_out;
    int64_t k_in;           // real number of inputs (<= k_tiles*256)
    int prologue;
    const int8_t* q;        // PRO_Q8: [m, q_stride] int8, zero beyond k_in
    int64_t q_stride;
    const int32_t* qsum;    // PRO_Q8: [m]
    const float* sx;        // PRO_Q8: [m] (unused for EPI_I32)
    const float* x;         // PRO_RMSNORM / PRO_ABSMAX: [m, x_stride] f32
    int64_t x_stride;
    const float* norm_w;    // PRO_RMSNORM: [k_in]
    float eps;
    const unsigned int* absmax_in;  // PRO_ABSMAX: [m] bit patterns of max|x| (non-negative floats)
    unsigned int* absmax_out;       // EPI_SWIGLU: [m] running max of |out| via atomicMax on the bits
    const float* sw_tiles;  // [row_tiles][2] weight scale of rows 0-7 / 8-15 of each row tile
    int m;                  // 1..8
    void* out;              // [m, out_stride]
    int64_t out_stride;     // elements between tokens
    int epilogue;
    unsigned int* err;
    bool pdl;               // launch with programmatic stream serialisation
};
cudaError_t launch_gemv(const GemvArgs& a, int sm_count, cudaStream_t stream);
// Largest token count (<= 8) one launch can take for this many 256-input tiles per row; 0 = the layer's rows are
// too long for the kernel's shared memory even with one token.
int gemv_max_tokens(int64_t k_tiles);

// A BitLinear as the kernels see it: tiles of every basis plus one weight scale per
// (basis, row tile) - fused projections (q|k|v, gate|up) carry a different scale per
// segment of rows.
struct LinearDev {
    TiledWeights w;
    const float* scale_tiles = nullptr;  // device, [n_bases][row_tiles][2] (rows 0-7, rows 8-15)
};

// Ternary product of `m` quantised tokens with every basis of `lin` (8 tokens per launch).
// epilogue: EPI_I32 (basis 0 only), EPI_F32, EPI_F32_ACCUM (adds onto out) or EPI_BF16
// (single basis only).
cudaError_t linear_product(const LinearDev& lin, const int8_t* q, int64_t q_stride,
                           const int32_t* qsum, const float* sx, int64_t m, void* out,
                           int64_t out_stride, int epilogue, unsigned int* err, int sm_count,
                           cudaStream_t stream);

// Single-basis product for m <= 8 tokens whose quantisation happens inside the kernel.
struct FusedIn {
    int prologue;                   // PRO_RMSNORM or PRO_ABSMAX
    const float* x;
    int64_t x_stride;
    const float* norm_w;
    float eps;
    const unsigned int* absmax_in;
};
cudaError_t linear_product_fused(const LinearDev& lin, const FusedIn& in, int m, void* out,
                                 int64_t out_stride, int epilogue, unsigned int* absmax_out,
                                 unsigned int* err, int sm_count, cudaStream_t stream);

cudaError_t linear_product_q(const LinearDev& lin, const int8_t* q, int64_t q_stride, const int32_t* qsum,
                             const float* sx, int m, void* out, int64_t out_stride, int epilogue,
                             unsigned int* absmax_out, unsigned int* err, int sm_count, cudaStream_t stream);

// Tensor-core (tcgen05) product for more than 8 tokens: quantises x [m, k_in] (f32 or bf16) into the
// residue-split layout `qtc` (gemm_tc_act_bytes(m, k_tiles) bytes), then runs the product of
// every basis.  sx / qsum: [m] scratch for the per-token scale and sum.
size_t gemm_tc_act_bytes(int64_t m, int64_t k_tiles);
// Byte offset of activation (token tin of its block of nt tokens, input c) inside the block:
// [k_tile][residue c % 4][token group][k' / 16][token % 8][k' % 16], k' = (c % 256) / 4.
__host__ __device__ inline int64_t gemm_tc_act_offset(int c, int tin, int nt) {
    const int kt = c >> 8, r = c & 3, kp = (c & 255) >> 2;
    return (int64_t)kt * (4 * nt * 64) + (int64_t)r * (nt * 64) + (tin >> 3) * 512 + (kp >> 4) * 128 + (tin & 7) * 16 + (kp & 15);
}
// When a product has fewer output tiles than the GPU has SMs, its k range is cut across the CTAs
// of a thread-block cluster, whose int32 partial sums are added through distributed shared memory.
// kernels one launch_gemm_tc call runs for the products themselves
int gemm_tc_kernels(const LinearDev& lin, int64_t m, int sm_count);
cudaError_t launch_gemm_tc(const LinearDev& lin, const void* x, int64_t x_stride, int64_t m, int8_t* qtc, float* sx,
                           int32_t* qsum, void* out, int64_t out_stride, int epilogue, unsigned int* err, int sm_count,
                           cudaStream_t stream,
                           bool prequantised = false,     // qtc / sx / qsum are already filled (x unused)
                           bt_dtype x_dtype = BT_F32);    // element type of x: BT_F32 or BT_BF16

// Kernel attributes (dynamic shared-memory limit, cluster sizes) belong to a device, not to the process: `run(f)`
// calls f() once per device (the current one), under a lock, and remembers success.
struct PerDeviceOnce {
    std::mutex mu;
    bool done[64] = {};
    template <typename F>
    cudaError_t run(F f) {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        std::lock_guard<std::mutex> lock(mu);
        if (dev >= 0 && dev < 64 && done[dev]) return cudaSuccess;
        e = f();
        if (e == cudaSuccess && dev >= 0 && dev < 64) done[dev] = true;
        return e;
    }
};

// Launch with the programmatic-stream-serialisation attribute: the kernel may start while
// its predecessor in the stream is still running and must call griddepcontrol.wait before
// touching anything the predecessor produces.
template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace bt
