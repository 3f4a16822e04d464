// TTT fast-weight update, fused (layers/ttt.rs:48-74 per token, :80-119 per chunk).
// For a chunk X (rows = L2-normalised features): Z = X W^T, D = Z - X, G = D^T X,
// W <- W - lr*G, and every row of the chunk is predicted with the pre-update W.  Row a of
// W only needs X and its own predictions, so one warp owns one row of one state, keeps it
// in registers across all chunks of the launch, and the state is read and written exactly
// once: 2*d*d*4 bytes per state per launch, which is the HBM bound of this kernel.
// Sums (L2 norm, W row . x, the chunk gradient) are accumulated in f64 and rounded to f32
// once, so that they do not depend on the order in which lanes add them.
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
