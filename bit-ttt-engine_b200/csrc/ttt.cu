// TTT fast-weight update, fused (layers/ttt.rs:48-74 per token, :80-119 per chunk).
// For a chunk X (rows = L2-normalised features): Z = X W^T, D = Z - X, G = D^T X,
// W <- W - lr*G, and every row of the chunk is predicted with the pre-update W.  Row a of
// W only needs X and its own predictions, so one warp owns one row of one state, keeps it
// in registers across all chunks of the launch, and the state is read and written exactly
// once: 2*d*d*4 bytes per state per launch, which is the HBM bound of this kernel.
// The general kernel below accumulates its sums (L2 norm, W row . x, the chunk gradient) in f64 and rounds to f32
// once; the kernel for the small states the models use (d = 32, 64, 128) keeps f64 for the norm only.
// The reference issues ~12 tensor ops and two small batched matmuls per token.
#include "bt_model.cuh"
#include "bt_ptx.cuh"

namespace bt {

namespace {

constexpr int kTttWarps = 8;
constexpr int kMaxChunk = 64;

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// PL = ceil(d / 32) register slots per lane for one row of W.
template <int PL>
__global__ void __launch_bounds__(kTttWarps * 32) ttt_chunk_kernel(float* __restrict__ w,
                                                                  const float* __restrict__ feats,
                                                                  int t_len, int d, float lr, int chunk,
                                                                  float* __restrict__ z_out,
                                                                  unsigned int* __restrict__ absmax_out) {
    extern __shared__ float xh[];  // [chunk][d] normalised features of the current chunk
    __shared__ float inv_norm[kMaxChunk];
    ptx::pdl_wait();
    ptx::pdl_launch_dependents();
    const int b = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a = blockIdx.y * kTttWarps + warp;  // row of W owned by this warp
    const bool active = a < d;
    float* wrow = w + ((int64_t)b * d + (active ? a : 0)) * d;
    float wr[PL];
#pragma unroll
    for (int j = 0; j < PL; ++j) {
        const int c = lane + 32 * j;
        wr[j] = (active && c < d) ? wrow[c] : 0.0f;
    }
    const float* fb = feats + (int64_t)b * t_len * d;
    float* zb = z_out + (int64_t)b * t_len * d;

    for (int start = 0; start < t_len; start += chunk) {
        const int len = min(chunk, t_len - start);
        __syncthreads();  // previous chunk fully consumed
        // L2 norms: n = sqrt(sum f^2) + 1e-6 (layers/ttt.rs:53-54), one warp per row
        for (int t = warp; t < len; t += kTttWarps) {
            double ss = 0.0;
            for (int c = lane; c < d; c += 32) {
                const float f = fb[(int64_t)(start + t) * d + c];
                ss = fma((double)f, (double)f, ss);
            }
            ss = warp_sum(ss);
            if (lane == 0) inv_norm[t] = __fadd_rn(sqrtf((float)ss), 1e-6f);
        }
        __syncthreads();
        for (int i = threadIdx.x; i < len * d; i += blockDim.x)
            xh[i] = __fdiv_rn(fb[(int64_t)start * d + i], inv_norm[i / d]);
        __syncthreads();
        if (active) {
            // predictions with the pre-update row, then the rank-len update
            double g[PL];
#pragma unroll
            for (int j = 0; j < PL; ++j) g[j] = 0.0;
            for (int t = 0; t < len; ++t) {
                const float* xt = xh + t * d;
                double sd = 0.0;
#pragma unroll
                for (int j = 0; j < PL; ++j) {
                    const int c = lane + 32 * j;
                    if (c < d) sd = fma((double)wr[j], (double)xt[c], sd);
                }
                const float s = (float)warp_sum(sd);
                if (lane == 0) {
                    zb[(int64_t)(start + t) * d + a] = s;
                    if (absmax_out) atomicMax(absmax_out + b, __float_as_uint(fabsf(s)));
                }
                const float diff = __fsub_rn(s, xt[a]);
#pragma unroll
                for (int j = 0; j < PL; ++j) {
                    const int c = lane + 32 * j;
                    if (c < d) g[j] = fma((double)diff, (double)xt[c], g[j]);
                }
            }
#pragma unroll
            for (int j = 0; j < PL; ++j) wr[j] = __fsub_rn(wr[j], __fmul_rn((float)g[j], lr));
        }
    }
    if (active) {
#pragma unroll
        for (int j = 0; j < PL; ++j) {
            const int c = lane + 32 * j;
            if (c < d) wrow[c] = wr[j];
        }
    }
}

// Small states (d = 32, 64 or 128): LPR = d / 16 lanes share a row of W, each holding 16 consecutive columns in
// registers, so that the inner loops are plain FMAs on registers.  A row's dot product is finished with log2(LPR)
// shuffles, which also leave z - x in every lane of the row for the gradient.  A warp covers 32 / LPR rows; with
// d <= 64 a CTA of 8 warps covers a whole state, so the chunk is normalised once per state.
// The products W row . x and the chunk gradient are accumulated in f32 like the reference's own matmuls
// (layers/ttt.rs:58-65), in a fixed order (four partial sums per lane, then the lanes of the row), so a result does
// not depend on the batch or on the run; only the L2 norm keeps its f64 sum.  f64 FMAs run at half the f32 rate on
// this part and made the kernel arithmetic-bound at a sixth of the HBM bound.
template <int LPR>
__global__ void __launch_bounds__(kTttWarps * 32, 3) ttt_rows_kernel(float* __restrict__ w,
                                                                    const float* __restrict__ feats,
                                                                    int t_len, int d, float lr, int chunk,
                                                                    float* __restrict__ z_out,
                                                                    unsigned int* __restrict__ absmax_out) {
    constexpr int kCols = 16;                 // columns per lane
    constexpr int kPad = 4;                   // floats between two blocks of 16 columns
    constexpr int kRowsPerWarp = 32 / LPR;
    // [chunk][d + kPad * LPR] normalised features of the current chunk; every block of 16 columns is shifted by 4 more
    // floats, so that the LPR lanes of a row, which read different blocks in the same 16-byte load, hit different banks
    extern __shared__ __align__(16) float xs[];
    const int pitch = d + kPad * LPR;
    ptx::pdl_wait();
    ptx::pdl_launch_dependents();
    const int b = blockIdx.x;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int a = (blockIdx.y * kTttWarps + warp) * kRowsPerWarp + lane / LPR;  // this lane's row of W
    const int blk = lane % LPR;                                                 // and its block of 16 columns
    const bool active = a < d;
    float* wrow = w + ((int64_t)b * d + (active ? a : 0)) * d + blk * kCols;
    float wr[kCols];
#pragma unroll
    for (int i = 0; i < kCols / 4; ++i) {
        const float4 v = active ? reinterpret_cast<const float4*>(wrow)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        wr[4 * i] = v.x; wr[4 * i + 1] = v.y; wr[4 * i + 2] = v.z; wr[4 * i + 3] = v.w;
    }
    const float* fb = feats + (int64_t)b * t_len * d;
    float* zb = z_out + (int64_t)b * t_len * d;
    float run_max = 0.0f;
    constexpr int kPerTok = 16;               // threads that share a token while staging
    constexpr int kElems = LPR;               // d / 16 elements per such thread

    for (int start = 0; start < t_len; start += chunk) {
        const int len = min(chunk, t_len - start);
        __syncthreads();  // previous chunk fully consumed
        // stage the chunk: x / (sqrt(sum x^2) + 1e-6) (layers/ttt.rs:53-55), 16 threads per token,
        // every feature read once
        for (int tb = 0; tb < len; tb += (kTttWarps * 32) / kPerTok) {
            const int t = tb + (int)(threadIdx.x / kPerTok), sub = threadIdx.x % kPerTok;
            float f[kElems];
            double ss = 0.0;
#pragma unroll
            for (int e = 0; e < kElems; ++e) f[e] = t < len ? fb[(int64_t)(start + t) * d + sub + kPerTok * e] : 0.0f;
#pragma unroll
            for (int e = 0; e < kElems; ++e) ss = fma((double)f[e], (double)f[e], ss);
#pragma unroll
            for (int o = kPerTok / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            const float nrm = __fadd_rn(sqrtf((float)ss), 1e-6f);
#pragma unroll
            for (int e = 0; e < kElems; ++e)
                if (t < len) xs[t * pitch + sub + (kPerTok + kPad) * e] = __fdiv_rn(f[e], nrm);
        }
        __syncthreads();
        float g[kCols];
#pragma unroll
        for (int i = 0; i < kCols; ++i) g[i] = 0.0f;
        for (int t = 0; t < len; ++t) {
            const float* xt = xs + t * pitch;
            float x[kCols];
#pragma unroll
            for (int i = 0; i < kCols; i += 4) {
                const float4 v = *reinterpret_cast<const float4*>(xt + blk * (kCols + kPad) + i);
                x[i] = v.x; x[i + 1] = v.y; x[i + 2] = v.z; x[i + 3] = v.w;
            }
            // prediction with the pre-update row: four partial sums, then the lanes of the row
            float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
#pragma unroll
            for (int i = 0; i < kCols; i += 4) {
                s0 = __fmaf_rn(wr[i], x[i], s0);
                s1 = __fmaf_rn(wr[i + 1], x[i + 1], s1);
                s2 = __fmaf_rn(wr[i + 2], x[i + 2], s2);
                s3 = __fmaf_rn(wr[i + 3], x[i + 3], s3);
            }
            float s = __fadd_rn(__fadd_rn(s0, s1), __fadd_rn(s2, s3));
#pragma unroll
            for (int o = LPR / 2; o > 0; o >>= 1) s = __fadd_rn(s, __shfl_xor_sync(0xffffffffu, s, o));
            const float xa = active ? xt[a + kPad * (a / kCols)] : 0.0f;
            if (active && blk == 0) {
                zb[(int64_t)(start + t) * d + a] = s;
                run_max = fmaxf(run_max, fabsf(s));
            }
            // rank-1 piece of the chunk gradient
            const float df = __fsub_rn(s, xa);
#pragma unroll
            for (int i = 0; i < kCols; ++i) g[i] = __fmaf_rn(df, x[i], g[i]);
        }
        // W <- W - lr * G (layers/ttt.rs:68,111)
#pragma unroll
        for (int i = 0; i < kCols; ++i) wr[i] = __fsub_rn(wr[i], __fmul_rn(g[i], lr));
    }
    if (active) {
#pragma unroll
        for (int i = 0; i < kCols / 4; ++i)
            reinterpret_cast<float4*>(wrow)[i] = make_float4(wr[4 * i], wr[4 * i + 1], wr[4 * i + 2], wr[4 * i + 3]);
    }
    if (absmax_out) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) run_max = fmaxf(run_max, __shfl_xor_sync(0xffffffffu, run_max, o));
        if (lane == 0 && run_max > 0.0f) atomicMax(absmax_out + b, __float_as_uint(run_max));
    }
}

template <int LPR>
cudaError_t launch_rows(float* w, const float* feats, int batch, int t_len, int d, float lr, int chunk,
                        float* z_out, cudaStream_t stream, unsigned int* absmax_out, bool pdl) {
    const size_t smem = (size_t)chunk * (d + 4 * LPR) * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(ttt_rows_kernel<LPR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    const int rows_per_cta = kTttWarps * (32 / LPR);
    dim3 grid(batch, (d + rows_per_cta - 1) / rows_per_cta);
    return launch_pdl(ttt_rows_kernel<LPR>, grid, dim3(kTttWarps * 32), smem, stream, pdl, w, feats, t_len, d, lr, chunk, z_out, absmax_out);
}

template <int PL>
cudaError_t launch_pl(float* w, const float* feats, int batch, int t_len, int d, float lr, int chunk,
                      float* z_out, cudaStream_t stream, unsigned int* absmax_out, bool pdl) {
    const size_t smem = (size_t)chunk * d * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(ttt_chunk_kernel<PL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    dim3 grid(batch, (d + kTttWarps - 1) / kTttWarps);
    return launch_pdl(ttt_chunk_kernel<PL>, grid, dim3(kTttWarps * 32), smem, stream, pdl, w, feats, t_len, d, lr, chunk, z_out, absmax_out);
}

}  // namespace

cudaError_t launch_ttt_chunk(float* w, const float* feats, int batch, int t_len, int d, float lr, int chunk,
                             float* z_out, cudaStream_t stream, unsigned int* absmax_out, bool pdl) {
    if (d < 1 || d > 1024 || chunk < 1 || chunk > kMaxChunk || (size_t)chunk * d * 4 > 200 * 1024)
        return cudaErrorInvalidValue;
    if (batch <= 0 || t_len <= 0) return cudaSuccess;
    const int pl = (d + 31) / 32;
    const bool aligned = (reinterpret_cast<uintptr_t>(w) & 15) == 0;  // the row kernels load 16 bytes at a time
    if (aligned && d == 32) return launch_rows<2>(w, feats, batch, t_len, d, lr, chunk, z_out, stream, absmax_out, pdl);
    if (aligned && d == 64) return launch_rows<4>(w, feats, batch, t_len, d, lr, chunk, z_out, stream, absmax_out, pdl);
    if (aligned && d == 128) return launch_rows<8>(w, feats, batch, t_len, d, lr, chunk, z_out, stream, absmax_out, pdl);
    if (pl <= 1) return launch_pl<1>(w, feats, batch, t_len, d, lr, chunk, z_out, stream, absmax_out, pdl);
    if (pl <= 2) return launch_pl<2>(w, feats, batch, t_len, d, lr, chunk, z_out, stream, absmax_out, pdl);
    if (pl <= 4) return launch_pl<4>(w, feats, batch, t_len, d, lr, chunk, z_out, stream, absmax_out, pdl);
    if (pl <= 8) return launch_pl<8>(w, feats, batch, t_len, d, lr, chunk, z_out, stream, absmax_out, pdl);
    if (pl <= 16) return launch_pl<16>(w, feats, batch, t_len, d, lr, chunk, z_out, stream, absmax_out, pdl);
    return launch_pl<32>(w, feats, batch, t_len, d, lr, chunk, z_out, stream, absmax_out, pdl);
}

cudaError_t launch_ttt_step(float* w, const float* feat, int batch, int d, float lr, float* z_out,
                            cudaStream_t stream, unsigned int* absmax_out, bool pdl) {
    return launch_ttt_chunk(w, feat, batch, 1, d, lr, 1, z_out, stream, absmax_out, pdl);
}

}  // namespace bt
