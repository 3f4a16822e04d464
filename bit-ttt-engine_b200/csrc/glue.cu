// Small memory-bound kernels around the ternary products of one decode step:
// embedding gather, (RMSNorm | SwiGLU product | identity) + per-token int8 quantisation,
// dense bf16 lm_head, arg-max.  All f32 arithmetic; reference operation order is kept
// wherever a rounding could show (see each kernel).
#include "bt_common.cuh"
#include "bt_model.cuh"
#include "bt_ptx.cuh"

namespace bt {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Block-wide reductions over blockDim.x threads (multiple of 32, <= 1024).
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = warp_sum(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (l == 0) red[w] = v;
    __syncthreads();
    float r = l < nw ? red[l] : 0.0f;
    r = warp_sum(r);
    __syncthreads();
    return r;
}
// REUSE = false: `red` is used by this one reduction only in the kernel, the closing barrier (which protects the
// array against the next use) is left out.
template <bool REUSE = true>
__device__ __forceinline__ float block_max(float v, float* red) {
    v = warp_max(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (l == 0) red[w] = v;
    __syncthreads();
    float r = l < nw ? red[l] : 0.0f;
    r = warp_max(r);
    if (REUSE) __syncthreads();
    return r;
}
template <bool REUSE = true>
__device__ __forceinline__ double block_sum_d(double v, double* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (l == 0) red[w] = v;
    __syncthreads();
    double r = l < nw ? red[l] : 0.0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    if (REUSE) __syncthreads();
    return r;
}
__device__ __forceinline__ int block_sum_i(int v, int* red) {
    v = warp_sum_i(v);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31, nw = blockDim.x >> 5;
    if (l == 0) red[w] = v;
    __syncthreads();
    int r = l < nw ? red[l] : 0;
    r = warp_sum_i(r);
    __syncthreads();
    return r;
}

// ---------------------------------------------------------------------------------------
// embedding gather: h[b, :] = table[token[b], :]   (Embedding::forward, model/llama.rs:208)
// ---------------------------------------------------------------------------------------
__global__ void embed_kernel(const int32_t* __restrict__ tokens, const __nv_bfloat16* __restrict__ table,
                             int hidden, int vocab, float* __restrict__ h, unsigned int* __restrict__ clear,
                             int n_clear, bool f16) {
    ptx::pdl_wait();
    ptx::pdl_launch_dependents();
    const int b = blockIdx.x;
    if (b == 0)
        for (int i = threadIdx.x; i < n_clear; i += blockDim.x) clear[i] = 0u;
    int tok = tokens[b];
    tok = tok < 0 ? 0 : (tok >= vocab ? vocab - 1 : tok);
    const __nv_bfloat16* row = table + (int64_t)tok * hidden;
    if (f16) {  // the table holds IEEE half values (a converted checkpoint's dtype)
        const __half* hrow = reinterpret_cast<const __half*>(row);
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) h[(int64_t)b * hidden + c] = __half2float(hrow[c]);
    } else {
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) h[(int64_t)b * hidden + c] = __bfloat162float(row[c]);
    }
}

// ---------------------------------------------------------------------------------------
// row transform + absmax int8 quantisation, one CTA per token, the row held in shared
// memory so that global memory is read once.
//   PRE_NONE   : v = x
//   PRE_RMSNORM: v = (x / sqrt(mean(x^2) + eps)) * w        (layers/rms_norm.rs:40-55)
//   PRE_SWIGLU : v = silu(gate) * up, x = gate and up interleaved in groups of 8 (the row order of the fused
//                gate|up projection: x[16 j + r] = gate[8 j + r], x[16 j + 8 + r] = up[8 j + r])  (layers/swiglu.rs:31-33)
// then s = max|v|/127, q = clamp(round(v * (127/max|v|))), sum_k q.  `v_out` (optional) receives v.
// ---------------------------------------------------------------------------------------
// Four consecutive floats; `vec` = the address is 16-byte aligned (uniform over the block).
__device__ __forceinline__ float4 load4(const float* p, bool vec) {
    if (vec) return *reinterpret_cast<const float4*>(p);
    return make_float4(p[0], p[1], p[2], p[3]);
}
// The same from bf16 values (`vec` = 16-byte aligned row start; a group of four is then 8-byte aligned).
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p, bool vec) {
    if (vec) {
        const uint2 u = *reinterpret_cast<const uint2*>(p);
        return make_float4(__uint_as_float(u.x << 16), __uint_as_float(u.x & 0xffff0000u), __uint_as_float(u.y << 16),
                           __uint_as_float(u.y & 0xffff0000u));
    }
    return make_float4(__bfloat162float(p[0]), __bfloat162float(p[1]), __bfloat162float(p[2]), __bfloat162float(p[3]));
}

// k must be a multiple of 4 (the packed weight layouts require it anyway).  A thread works on groups of four
// consecutive values; in the tensor-core layout these are the four residues of one k' (see gemm_tc_act_offset),
// which are first laid out in shared memory in the order of that layout's 16-byte pieces and then copied out a
// piece per thread.
template <int PRE, typename T = float>
__global__ void __launch_bounds__(1024) row_quant_kernel(const T* __restrict__ x, int64_t x_stride,
                                                         const float* __restrict__ w, float eps, int k,
                                                         int8_t* __restrict__ q, int64_t q_stride,
                                                         float* __restrict__ s_out,
                                                         int32_t* __restrict__ qsum_out,
                                                         float* __restrict__ v_out, int8_t* __restrict__ qtc,
                                                         int tc_nt, int k_tiles,
                                                         const unsigned int* __restrict__ amax_in,
                                                         unsigned int* __restrict__ amax_out) {
    // amax_in : [rows] bit patterns of max|v| to quantise with (a maximum agreed over several GPUs) instead of
    //           this row's own.  amax_out: values-only mode, the row's v goes to v_out and its max|v| (bits) to
    //           amax_out[row]; nothing is quantised.
    extern __shared__ __align__(16) float row[];  // k floats, then k_tiles * 256 staged bytes (tensor-core layout only)
    __shared__ float red_f[32];
    __shared__ double red_d[32];
    __shared__ int red_i[32];
    ptx::pdl_wait();
    ptx::pdl_launch_dependents();  // a product launched behind this kernel may fetch its weights meanwhile
    const int b = blockIdx.x;
    const T* xr = x + (int64_t)b * x_stride;
    const bool xvec = ((reinterpret_cast<uintptr_t>(xr) & 15) == 0);
    const bool wvec = PRE == PRE_RMSNORM && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    const int groups = k >> 2;
    float amax = 0.0f;
    if (PRE == PRE_RMSNORM) {
        // sum of squares in f64, rounded once: reproducible against the CPU restatement
        double ss = 0.0;
        for (int gi = threadIdx.x; gi < groups; gi += blockDim.x) {
            const float4 v = load4(xr + 4 * gi, xvec);
            *reinterpret_cast<float4*>(row + 4 * gi) = v;
            ss = fma((double)v.x, (double)v.x, ss);
            ss = fma((double)v.y, (double)v.y, ss);
            ss = fma((double)v.z, (double)v.z, ss);
            ss = fma((double)v.w, (double)v.w, ss);
        }
        ss = block_sum_d<false>(ss, red_d);
        const float denom = sqrtf(__fadd_rn((float)(ss / (double)k), eps));
        for (int gi = threadIdx.x; gi < groups; gi += blockDim.x) {
            float4 v = *reinterpret_cast<const float4*>(row + 4 * gi);  // written by this same thread
            const float4 ww = load4(w + 4 * gi, wvec);
            v.x = __fmul_rn(__fdiv_rn(v.x, denom), ww.x);
            v.y = __fmul_rn(__fdiv_rn(v.y, denom), ww.y);
            v.z = __fmul_rn(__fdiv_rn(v.z, denom), ww.z);
            v.w = __fmul_rn(__fdiv_rn(v.w, denom), ww.w);
            *reinterpret_cast<float4*>(row + 4 * gi) = v;
            amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
        }
    } else if (PRE == PRE_SWIGLU) {
        for (int gi = threadIdx.x; gi < groups; gi += blockDim.x) {
            const int c = 4 * gi;  // outputs c .. c + 3: gate at x[16 (c / 8) + c % 8 ..], up 8 further
            const float4 g4 = load4(xr + 16 * (c >> 3) + (c & 7), xvec), u4 = load4(xr + 16 * (c >> 3) + 8 + (c & 7), xvec);
            float4 v;
            v.x = __fmul_rn(__fdiv_rn(g4.x, __fadd_rn(1.0f, expf(-g4.x))), u4.x);
            v.y = __fmul_rn(__fdiv_rn(g4.y, __fadd_rn(1.0f, expf(-g4.y))), u4.y);
            v.z = __fmul_rn(__fdiv_rn(g4.z, __fadd_rn(1.0f, expf(-g4.z))), u4.z);
            v.w = __fmul_rn(__fdiv_rn(g4.w, __fadd_rn(1.0f, expf(-g4.w))), u4.w);
            *reinterpret_cast<float4*>(row + 4 * gi) = v;
            amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
        }
    } else {
        for (int gi = threadIdx.x; gi < groups; gi += blockDim.x) {
            const float4 v = load4(xr + 4 * gi, xvec);
            *reinterpret_cast<float4*>(row + 4 * gi) = v;
            amax = fmaxf(fmaxf(amax, fmaxf(fabsf(v.x), fabsf(v.y))), fmaxf(fabsf(v.z), fabsf(v.w)));
        }
    }
    amax = block_max<false>(amax, red_f);
    if (amax_out) {
        for (int gi = threadIdx.x; gi < groups; gi += blockDim.x)
            *reinterpret_cast<float4*>(v_out + (int64_t)b * k + 4 * gi) = *reinterpret_cast<const float4*>(row + 4 * gi);
        if (threadIdx.x == 0) amax_out[b] = __float_as_uint(amax);
        return;
    }
    if (amax_in) amax = __uint_as_float(amax_in[b]);
    const float s = __fdiv_rn(amax, 127.0f);
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    int local = 0;
    uint8_t* stage = reinterpret_cast<uint8_t*>(row + k);
    int8_t* qr = q ? q + (int64_t)b * q_stride : nullptr;
    const int groups_pad = qtc ? k_tiles * (kTileK / 4) : (int)(q_stride >> 2);
    for (int gi = threadIdx.x; gi < groups_pad; gi += blockDim.x) {
        int v[4] = {0, 0, 0, 0};
        if (gi < groups && amax > 0.0f) {
            const float4 f = *reinterpret_cast<const float4*>(row + 4 * gi);  // this thread's own values again
            v[0] = max(-127, min(127, ptx::round_half_away(__fmul_rn(f.x, inv))));
            v[1] = max(-127, min(127, ptx::round_half_away(__fmul_rn(f.y, inv))));
            v[2] = max(-127, min(127, ptx::round_half_away(__fmul_rn(f.z, inv))));
            v[3] = max(-127, min(127, ptx::round_half_away(__fmul_rn(f.w, inv))));
        }
        local += v[0] + v[1] + v[2] + v[3];
        if (qtc) {
            // residue r of k' = gi % 64 in k-tile gi / 64: staged at [k-tile][residue][k']
            const int kt = gi >> 6, kp = gi & 63;
#pragma unroll
            for (int r = 0; r < 4; ++r) stage[(kt * 4 + r) * 64 + kp] = (uint8_t)v[r];
        }
        if (qr)
            *reinterpret_cast<uint32_t*>(qr + 4 * gi) = (uint32_t)(v[0] & 0xff) | ((uint32_t)(v[1] & 0xff) << 8) |
                                                        ((uint32_t)(v[2] & 0xff) << 16) | ((uint32_t)(v[3] & 0xff) << 24);
    }
    if (v_out)
        for (int gi = threadIdx.x; gi < groups; gi += blockDim.x)
            *reinterpret_cast<float4*>(v_out + (int64_t)b * k + 4 * gi) = *reinterpret_cast<const float4*>(row + 4 * gi);
    const int total = block_sum_i(local, red_i);  // (its barriers also complete the staged bytes)
    if (qtc) {
        // 16-byte pieces [k-tile][residue][k' / 16] -> their places in the token block (gemm_tc_act_offset)
        const int tb = b / tc_nt, tin = b % tc_nt;
        int8_t* blk = qtc + (int64_t)tb * k_tiles * (4 * tc_nt * 64) + (tin >> 3) * 512 + (tin & 7) * 16;
        for (int pid = threadIdx.x; pid < k_tiles * 16; pid += blockDim.x) {
            const int kc = pid & 3, kr = pid >> 2;  // kr = k-tile * 4 + residue
            *reinterpret_cast<uint4*>(blk + (int64_t)kr * (tc_nt * 64) + kc * 128) = *reinterpret_cast<const uint4*>(stage + pid * 16);
        }
    }
    if (threadIdx.x == 0) {
        s_out[b] = s;
        qsum_out[b] = total;
    }
}

// Greedy pick: the LAST index among equal maxima, as Iterator::max_by does in the
// reference's sampler (model/llama.rs:510-515).  One CTA per token.
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, int64_t stride,
                                                      int vocab, int32_t* __restrict__ out) {
    __shared__ float sv[32];
    __shared__ int si[32];
    ptx::pdl_wait();
    const float* row = logits + (int64_t)blockIdx.x * stride;
    float best = -INFINITY;
    int idx = -1;
    if ((reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        // four consecutive values per load, four loads in flight per thread; within a thread the indices rise,
        // so ">=" keeps the last of equal maxima
        const int groups = vocab >> 2;
        for (int g0 = threadIdx.x; g0 < groups; g0 += 4 * blockDim.x) {
            float4 f[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int gi = g0 + u * blockDim.x;
                f[u] = gi < groups ? *reinterpret_cast<const float4*>(row + 4 * gi) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int c = 4 * (g0 + u * blockDim.x);
                if (c < 4 * groups) {
                    if (f[u].x >= best || idx < 0) { best = f[u].x; idx = c; }
                    if (f[u].y >= best) { best = f[u].y; idx = c + 1; }
                    if (f[u].z >= best) { best = f[u].z; idx = c + 2; }
                    if (f[u].w >= best) { best = f[u].w; idx = c + 3; }
                }
            }
        }
        for (int c = 4 * groups + threadIdx.x; c < vocab; c += blockDim.x) {
            const float v = row[c];
            if (v >= best || idx < 0) { best = v; idx = c; }
        }
    } else {
        for (int c = threadIdx.x; c < vocab; c += blockDim.x) {
            const float v = row[c];
            if (v >= best || idx < 0) { best = v; idx = c; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (oi >= 0 && (idx < 0 || ov > best || (ov == best && oi > idx))) { best = ov; idx = oi; }
    }
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) { sv[w] = best; si[w] = idx; }
    __syncthreads();
    if (w == 0) {
        best = l < (blockDim.x >> 5) ? sv[l] : -INFINITY;
        idx = l < (blockDim.x >> 5) ? si[l] : -1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (oi >= 0 && (idx < 0 || ov > best || (ov == best && oi > idx))) { best = ov; idx = oi; }
        }
        if (l == 0) out[blockIdx.x] = idx;
    }
}


// Two packed 16-bit weights -> f32: bf16 by shifting into the high half, IEEE half by conversion.
template <bool F16>
__device__ __forceinline__ void unpack16(uint32_t u, float& lo, float& hi) {
    if (F16) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u));
        lo = f.x; hi = f.y;
    } else {
        lo = __uint_as_float(u << 16);
        hi = __uint_as_float(u & 0xffff0000u);
    }
}

// Dense lm_head (candle_nn::Linear without bias, model/llama.rs:23,266; the converter keeps it in 16 bits,
// tools/conversion/convert_llama_v2.py:265-268) with the final RMSNorm folded in (every CTA normalises the
// hidden vector itself, sum of squares in f64) and a running arg-max per CTA, so that the greedy pick does
// not need a pass over all logits.  Ties keep the larger index (model/llama.rs:510-515).  HBM-bound on W:
// one warp per output row, 16-byte loads, x in shared memory, f32 accumulation.
template <int B, bool F16>
__global__ void __launch_bounds__(256) lm_head_fused_kernel(const __nv_bfloat16* __restrict__ w,
                                                            const float* __restrict__ h,
                                                            const float* __restrict__ norm_w, float eps,
                                                            int hidden, int64_t vocab, float* __restrict__ logits,
                                                            float* __restrict__ cand_val,
                                                            int32_t* __restrict__ cand_idx) {
    extern __shared__ float xs[];  // [B][hidden]
    __shared__ double red_d[32];
    __shared__ float best_v[8][B];
    __shared__ int best_i[8][B];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t warp_global = (int64_t)blockIdx.x * 8 + warp;
    const int64_t warps_total = (int64_t)gridDim.x * 8;
    // warm the first rows of this warp into L2/L1 while the previous kernel drains
    ptx::pdl_wait();
    ptx::pdl_launch_dependents();
    for (int b = 0; b < B; ++b) {
        double ss = 0.0;
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
            const float v = h[(int64_t)b * hidden + c];
            xs[b * hidden + c] = v;
            ss = fma((double)v, (double)v, ss);
        }
        ss = block_sum_d(ss, red_d);
        const float denom = sqrtf(__fadd_rn((float)(ss / (double)hidden), eps));
        for (int c = threadIdx.x; c < hidden; c += blockDim.x)
            xs[b * hidden + c] = __fmul_rn(__fdiv_rn(xs[b * hidden + c], denom), norm_w[c]);
    }
    __syncthreads();
    float bv[B];
    int bi[B];
#pragma unroll
    for (int b = 0; b < B; ++b) { bv[b] = -INFINITY; bi[b] = -1; }
    for (int64_t v = warp_global; v < vocab; v += warps_total) {
        const uint4* wr = reinterpret_cast<const uint4*>(w + v * hidden);
        float acc[B];
#pragma unroll
        for (int b = 0; b < B; ++b) acc[b] = 0.0f;
#pragma unroll 4
        for (int c8 = lane; c8 < hidden / 8; c8 += 32) {
            const uint4 pk = wr[c8];
            const uint32_t u[4] = {pk.x, pk.y, pk.z, pk.w};
            float wf[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) unpack16<F16>(u[j], wf[2 * j], wf[2 * j + 1]);
#pragma unroll
            for (int b = 0; b < B; ++b) {
                const float4 x0 = *reinterpret_cast<const float4*>(xs + b * hidden + c8 * 8);
                const float4 x1 = *reinterpret_cast<const float4*>(xs + b * hidden + c8 * 8 + 4);
                acc[b] = fmaf(wf[0], x0.x, acc[b]);
                acc[b] = fmaf(wf[1], x0.y, acc[b]);
                acc[b] = fmaf(wf[2], x0.z, acc[b]);
                acc[b] = fmaf(wf[3], x0.w, acc[b]);
                acc[b] = fmaf(wf[4], x1.x, acc[b]);
                acc[b] = fmaf(wf[5], x1.y, acc[b]);
                acc[b] = fmaf(wf[6], x1.z, acc[b]);
                acc[b] = fmaf(wf[7], x1.w, acc[b]);
            }
        }
#pragma unroll
        for (int b = 0; b < B; ++b) {
            const float r = warp_sum(acc[b]);
            if (lane == 0) logits[(int64_t)b * vocab + v] = r;
            if (r >= bv[b]) { bv[b] = r; bi[b] = (int)v; }  // v increases: ties keep the later index
        }
    }
    if (lane == 0)
#pragma unroll
        for (int b = 0; b < B; ++b) { best_v[warp][b] = bv[b]; best_i[warp][b] = bi[b]; }
    __syncthreads();
    if (threadIdx.x < B) {
        const int b = threadIdx.x;
        float v = -INFINITY;
        int i = -1;
        for (int wv = 0; wv < 8; ++wv) {
            const float ov = best_v[wv][b];
            const int oi = best_i[wv][b];
            if (oi >= 0 && (i < 0 || ov > v || (ov == v && oi > i))) { v = ov; i = oi; }
        }
        cand_val[(int64_t)b * gridDim.x + blockIdx.x] = v;
        cand_idx[(int64_t)b * gridDim.x + blockIdx.x] = i;
    }
}

__global__ void __launch_bounds__(256) pick_kernel(const float* __restrict__ cand_val,
                                                   const int32_t* __restrict__ cand_idx, int n_cand,
                                                   int32_t* __restrict__ out, int32_t* __restrict__ pos, int n_pos) {
    __shared__ float sv[8];
    __shared__ int si[8];
    ptx::pdl_wait();
    ptx::pdl_launch_dependents();
    const int b = blockIdx.x;
    float v = -INFINITY;
    int i = -1;
    for (int c = threadIdx.x; c < n_cand; c += blockDim.x) {
        const float ov = cand_val[(int64_t)b * n_cand + c];
        const int oi = cand_idx[(int64_t)b * n_cand + c];
        if (oi >= 0 && (i < 0 || ov > v || (ov == v && oi > i))) { v = ov; i = oi; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (oi >= 0 && (i < 0 || ov > v || (ov == v && oi > i))) { v = ov; i = oi; }
    }
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) { sv[w] = v; si[w] = i; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int k = 1; k < 8; ++k) {
            const float ov = sv[k];
            const int oi = si[k];
            if (oi >= 0 && (i < 0 || ov > v || (ov == v && oi > i))) { v = ov; i = oi; }
        }
        out[b] = i;
    }
    if (b == 0 && threadIdx.x < n_pos) pos[threadIdx.x] += 1;  // BitLlama::current_pos += 1, model/llama.rs:269
}

// h += y over n floats (the residual add after a projection whose bases were summed into y first)
__global__ void __launch_bounds__(256) residual_add_kernel(float* __restrict__ h, const float* __restrict__ y, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        h[i] = __fadd_rn(h[i], y[i]);
}

}  // namespace

cudaError_t launch_residual_add(float* h, const float* y, int64_t n, cudaStream_t stream) {
    const int64_t blocks = (n + 255) / 256;
    residual_add_kernel<<<(unsigned)(blocks < 1184 ? blocks : 1184), 256, 0, stream>>>(h, y, n);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------
// launchers
// ---------------------------------------------------------------------------------------
cudaError_t launch_embed(const int32_t* tokens, const __nv_bfloat16* table, int batch, int hidden,
                         int vocab, float* h, cudaStream_t stream, unsigned int* clear, int n_clear, bool pdl, bool f16) {
    return launch_pdl(embed_kernel, dim3(batch), dim3(256), 0, stream, pdl, tokens, table, hidden, vocab, h, clear,
                      n_clear, f16);
}

cudaError_t launch_row_quant(int pre, const float* x, int64_t x_stride, const float* w, float eps,
                             int batch, int k, int8_t* q, int64_t q_stride, float* s, int32_t* qsum,
                             float* v_out, cudaStream_t stream, int8_t* qtc, int k_tiles,
                             const unsigned int* amax_in, unsigned int* amax_out) {
    const int tc_nt = batch <= 64 ? 64 : 128;
    if (amax_out && !v_out) return cudaErrorInvalidValue;
    if (k % 4 != 0 || (q && q_stride % 4 != 0)) return cudaErrorInvalidValue;
    const size_t smem = (size_t)k * sizeof(float) + (qtc ? (size_t)k_tiles * kTileK : 0);
    const int threads = k >= 4096 ? 1024 : (k >= 2048 ? 512 : 256);
    static PerDeviceOnce once;
    cudaError_t ce = once.run([] {
        cudaError_t e = cudaFuncSetAttribute(row_quant_kernel<PRE_NONE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(row_quant_kernel<PRE_RMSNORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(row_quant_kernel<PRE_SWIGLU>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        return e;
    });
    if (ce != cudaSuccess) return ce;
    if (smem > 200 * 1024) return cudaErrorInvalidConfiguration;
    // an ordinary launch (starting early behind a tensor-core product measured slower inside the decode step); the
    // kernel still releases its own dependent at once, so that the product behind it can fetch weights meanwhile
    const dim3 grid((unsigned)batch), block((unsigned)threads);
    if (pre == PRE_RMSNORM)
        return launch_pdl(row_quant_kernel<PRE_RMSNORM>, grid, block, smem, stream, false, x, x_stride, w, eps, k, q, q_stride, s, qsum, v_out, qtc, tc_nt, k_tiles, amax_in, amax_out);
    if (pre == PRE_SWIGLU)
        return launch_pdl(row_quant_kernel<PRE_SWIGLU>, grid, block, smem, stream, false, x, x_stride, w, eps, k, q, q_stride, s, qsum, v_out, qtc, tc_nt, k_tiles, amax_in, amax_out);
    return launch_pdl(row_quant_kernel<PRE_NONE>, grid, block, smem, stream, false, x, x_stride, w, eps, k, q, q_stride, s, qsum, v_out, qtc, tc_nt, k_tiles, amax_in, amax_out);
}

// Identity transform + quantiser on bf16 rows, into the tensor-core product's layout.
cudaError_t launch_row_quant_bf16(const __nv_bfloat16* x, int64_t x_stride, int batch, int k, float* s, int32_t* qsum,
                                  cudaStream_t stream, int8_t* qtc, int k_tiles) {
    const int tc_nt = batch <= 64 ? 64 : 128;
    if (k % 4 != 0 || !qtc) return cudaErrorInvalidValue;
    const size_t smem = (size_t)k * sizeof(float) + (size_t)k_tiles * kTileK;
    const int threads = k >= 4096 ? 1024 : (k >= 2048 ? 512 : 256);
    static PerDeviceOnce once;
    cudaError_t ce = once.run([] { return cudaFuncSetAttribute(row_quant_kernel<PRE_NONE, __nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); });
    if (ce != cudaSuccess) return ce;
    if (smem > 200 * 1024) return cudaErrorInvalidConfiguration;
    return launch_pdl(row_quant_kernel<PRE_NONE, __nv_bfloat16>, dim3((unsigned)batch), dim3((unsigned)threads), smem, stream, false, x, x_stride,
                      (const float*)nullptr, 0.0f, k, (int8_t*)nullptr, (int64_t)0, s, qsum, (float*)nullptr, qtc, tc_nt, k_tiles,
                      (const unsigned int*)nullptr, (unsigned int*)nullptr);
}

cudaError_t launch_argmax(const float* logits, int batch, int vocab, int32_t* out, cudaStream_t stream) {
    argmax_kernel<<<batch, 1024, 0, stream>>>(logits, vocab, vocab, out);
    return cudaGetLastError();
}

int lm_head_max_candidates(int sm_count) { return sm_count * 4; }

template <int B, bool F16>
static cudaError_t launch_lm_head_fused_bt(const __nv_bfloat16* w, const float* h, const float* norm_w, float eps,
                                           int hidden, int64_t vocab, float* logits, float* cand_val,
                                           int32_t* cand_idx, int grid, cudaStream_t stream, bool pdl) {
    const size_t smem = (size_t)B * hidden * sizeof(float);
    static PerDeviceOnce once;
    cudaError_t ce = once.run([] { return cudaFuncSetAttribute(lm_head_fused_kernel<B, F16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024); });
    if (ce != cudaSuccess) return ce;
    if (smem > 200 * 1024) return cudaErrorInvalidConfiguration;
    return launch_pdl(lm_head_fused_kernel<B, F16>, dim3(grid), dim3(256), smem, stream, pdl, w, h, norm_w, eps, hidden,
                      vocab, logits, cand_val, cand_idx);
}
template <int B>
static cudaError_t launch_lm_head_fused_b(const __nv_bfloat16* w, const float* h, const float* norm_w, float eps,
                                          int hidden, int64_t vocab, float* logits, float* cand_val,
                                          int32_t* cand_idx, int grid, cudaStream_t stream, bool pdl, bool f16) {
    return f16 ? launch_lm_head_fused_bt<B, true>(w, h, norm_w, eps, hidden, vocab, logits, cand_val, cand_idx, grid, stream, pdl)
               : launch_lm_head_fused_bt<B, false>(w, h, norm_w, eps, hidden, vocab, logits, cand_val, cand_idx, grid, stream, pdl);
}

cudaError_t launch_lm_head_fused(const __nv_bfloat16* w, const float* h, const float* norm_w, float eps,
                                 int batch, int hidden, int64_t vocab, float* logits, float* cand_val,
                                 int32_t* cand_idx, int* n_cand, int sm_count, cudaStream_t stream, bool pdl, bool f16) {
    if (hidden % 8 != 0 || batch < 1) return cudaErrorInvalidValue;
    // one grid size for every group of tokens, so that the candidate rows share a stride
    const int per_pass = batch > 4 ? 8 : 4;  // tokens per pass over the weights
    const size_t smem_max = (size_t)(batch < per_pass ? batch : per_pass) * hidden * sizeof(float);
    int per_sm = (int)((200 * 1024) / (smem_max + 2048));
    per_sm = per_sm > 4 ? 4 : (per_sm < 1 ? 1 : per_sm);
    const int grid = sm_count * per_sm;
    *n_cand = grid;
    for (int b0 = 0; b0 < batch; b0 += per_pass) {
        const int bc = batch - b0 < per_pass ? batch - b0 : per_pass;
        const float* hb = h + (size_t)b0 * hidden;
        float* lb = logits + (size_t)b0 * vocab;
        float* cv = cand_val + (size_t)b0 * grid;
        int32_t* ci = cand_idx + (size_t)b0 * grid;
        cudaError_t e;
        switch (bc) {
            case 1: e = launch_lm_head_fused_b<1>(w, hb, norm_w, eps, hidden, vocab, lb, cv, ci, grid, stream, pdl, f16); break;
            case 2: e = launch_lm_head_fused_b<2>(w, hb, norm_w, eps, hidden, vocab, lb, cv, ci, grid, stream, pdl, f16); break;
            case 3: e = launch_lm_head_fused_b<3>(w, hb, norm_w, eps, hidden, vocab, lb, cv, ci, grid, stream, pdl, f16); break;
            case 4: e = launch_lm_head_fused_b<4>(w, hb, norm_w, eps, hidden, vocab, lb, cv, ci, grid, stream, pdl, f16); break;
            case 5: e = launch_lm_head_fused_b<5>(w, hb, norm_w, eps, hidden, vocab, lb, cv, ci, grid, stream, pdl, f16); break;
            case 6: e = launch_lm_head_fused_b<6>(w, hb, norm_w, eps, hidden, vocab, lb, cv, ci, grid, stream, pdl, f16); break;
            case 7: e = launch_lm_head_fused_b<7>(w, hb, norm_w, eps, hidden, vocab, lb, cv, ci, grid, stream, pdl, f16); break;
            default: e = launch_lm_head_fused_b<8>(w, hb, norm_w, eps, hidden, vocab, lb, cv, ci, grid, stream, pdl, f16); break;
        }
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

cudaError_t launch_pick(const float* cand_val, const int32_t* cand_idx, int n_cand, int batch, int32_t* out,
                        int32_t* pos, int n_pos, cudaStream_t stream, bool pdl) {
    return launch_pdl(pick_kernel, dim3(batch), dim3(256), 0, stream, pdl, cand_val, cand_idx, n_cand, out, pos, n_pos);
}

}  // namespace bt
