// Fused decode attention over the Q8 KV cache: RoPE (layers/attention.rs:45-84) on the new
// q and k, Q8 append of k and v (layers/kv_cache.rs:95-119), scores = (q.k)/sqrt(hd) over
// positions 0..pos, softmax, .V (layers/attention.rs:198-217), all heads of a KV group in
// one CTA so the cache is read once (the reference materialises repeat_kv copies,
// layers/attention.rs:228-239).  The cache is read in place as u8; nothing is
// re-materialised in f32 (the reference dequantises the whole cache every step,
// layers/kv_cache.rs:84-92).  HBM-bound on the cache bytes: 2*n_kv*T*(hd+4) per sequence.
#include "bt_model.cuh"
#include "bt_ptx.cuh"

namespace bt {

namespace {

constexpr int kAttnWarps = 4;
constexpr int kAttnThreads = kAttnWarps * 32;

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

// Quantise one head vector held in shared memory (hd values) by one warp.
__device__ __forceinline__ void quant_row_warp(const float* v, int hd, uint8_t* q_out, float* s_out, int lane) {
    float amax = 0.0f;
    for (int c = lane; c < hd; c += 32) amax = fmaxf(amax, fabsf(v[c]));
    amax = warp_max(amax);
    const float s = __fdiv_rn(amax, 127.0f);
    for (int c = lane; c < hd; c += 32) {
        float r = s > 0.0f ? roundf(__fdiv_rn(v[c], s)) : 0.0f;
        r = fminf(fmaxf(r + 128.0f, 0.0f), 255.0f);
        q_out[c] = (uint8_t)r;
    }
    if (lane == 0) *s_out = s;
}

// One CTA = one (sequence, KV head, span of positions).  Each warp takes chunks of 32
// positions: (A) lane j dots key row j with the NREP query heads (no cross-lane traffic),
// (B) the chunk's softmax weights are formed with one exp per lane and head, (C) the lanes
// switch to owning head dimensions and accumulate P.V with the weights broadcast by
// shuffle.  Everything between the u8 loads and the final rounding is f64, so the result
// does not depend on how positions are split over lanes, warps and CTAs.
template <int PER_LANE, int NREP>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(AttnArgs a) {
    constexpr int HD = 32 * PER_LANE;
    __shared__ double qs[NREP][HD];
    __shared__ float knew[128], vnew[128];
    __shared__ double red_m[kAttnWarps][NREP], red_l[kAttnWarps][NREP];
    __shared__ double red_acc[kAttnWarps][NREP][HD];
    ptx::pdl_wait();
    ptx::pdl_launch_dependents();

    const int hd = a.head_dim, half = hd >> 1;
    const int b = blockIdx.x / a.n_kv, kvh = blockIdx.x % a.n_kv;
    const int split = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p = a.pos[b];
    const int t_len = p + 1;
    const int t0 = split * a.span;
    const int t1 = min(t_len, t0 + a.span);
    const int64_t qkv_stride = (int64_t)(a.n_heads + 2 * a.n_kv) * hd;
    const float* qkv = a.qkv + b * qkv_stride;
    double* part_base = a.partial + (((int64_t)b * a.n_heads + kvh * NREP) * a.splits + split) * (hd + 2);
    if (t0 >= t_len) {
        // nothing in this span yet: leave an empty partial (max = -inf, sum = 0)
        for (int h = threadIdx.x; h < NREP; h += blockDim.x) {
            double* dst = part_base + (int64_t)h * a.splits * (hd + 2);
            dst[0] = -INFINITY;
            dst[1] = 0.0;
        }
        return;
    }
    const float fp = (float)p;

    // rotate the NREP query heads of this KV group (cos/sin evaluated in f64, rounded once)
    for (int i = threadIdx.x; i < NREP * half; i += blockDim.x) {
        const int h = i / half, c = i % half;
        const float fr = __fmul_rn(fp, a.inv_freq[c]);
        const float cs = (float)cos((double)fr), sn = (float)sin((double)fr);
        const float* qh = qkv + (int64_t)(kvh * NREP + h) * hd;
        const float x1 = qh[c], x2 = qh[half + c];
        qs[h][c] = (double)__fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn));
        qs[h][half + c] = (double)__fadd_rn(__fmul_rn(x1, sn), __fmul_rn(x2, cs));
    }
    const int64_t row_base = ((int64_t)b * a.n_kv + kvh) * a.cache.max_seq;
    // the CTA whose span holds position p appends the new key / value first
    const bool owner = (p >= t0 && p < t1);
    if (owner) {
        const float* kh = qkv + (int64_t)(a.n_heads + kvh) * hd;
        const float* vh = qkv + (int64_t)(a.n_heads + a.n_kv + kvh) * hd;
        for (int c = threadIdx.x; c < half; c += blockDim.x) {
            const float fr = __fmul_rn(fp, a.inv_freq[c]);
            const float cs = (float)cos((double)fr), sn = (float)sin((double)fr);
            const float x1 = kh[c], x2 = kh[half + c];
            knew[c] = __fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn));
            knew[half + c] = __fadd_rn(__fmul_rn(x1, sn), __fmul_rn(x2, cs));
        }
        for (int c = threadIdx.x; c < hd; c += blockDim.x) vnew[c] = vh[c];
    }
    __syncthreads();
    if (owner) {
        if (warp == 0) quant_row_warp(knew, hd, a.cache.k_q + (row_base + p) * hd, a.cache.k_s + row_base + p, lane);
        if (warp == 1) quant_row_warp(vnew, hd, a.cache.v_q + (row_base + p) * hd, a.cache.v_s + row_base + p, lane);
    }
    __syncthreads();  // the block's own global writes are visible to it after the barrier

    double m_run[NREP], l_run[NREP], acc[NREP][PER_LANE];
#pragma unroll
    for (int h = 0; h < NREP; ++h) {
        m_run[h] = -INFINITY;
        l_run[h] = 0.0;
#pragma unroll
        for (int j = 0; j < PER_LANE; ++j) acc[h][j] = 0.0;
    }

    for (int tb = t0 + warp * 32; tb < t1; tb += kAttnWarps * 32) {
        // (A) scores of position tb + lane against the NREP heads
        const int t = tb + lane;
        const bool valid = t < t1;
        double sc[NREP];
#pragma unroll
        for (int h = 0; h < NREP; ++h) sc[h] = 0.0;
        if (valid) {
            const uint4* kr = reinterpret_cast<const uint4*>(a.cache.k_q + (row_base + t) * hd);
            const float ks = a.cache.k_s[row_base + t];
#pragma unroll
            for (int c16 = 0; c16 < HD / 16; ++c16) {
                const uint4 pk = kr[c16];
                const uint32_t wds[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
                for (int wi = 0; wi < 4; ++wi) {
#pragma unroll
                    for (int bi = 0; bi < 4; ++bi) {
                        const int c = c16 * 16 + wi * 4 + bi;
                        // dequantize_q8, kv_cache.rs:122-128: (f32(q) - 128) * s
                        const double kf = (double)__fmul_rn((float)((wds[wi] >> (8 * bi)) & 0xffu) - 128.0f, ks);
#pragma unroll
                        for (int h = 0; h < NREP; ++h) sc[h] = fma(qs[h][c], kf, sc[h]);
                    }
                }
            }
        }
        // (B) softmax weights of the chunk: (q.k) * 1/sqrt(hd) in f32 (attention.rs:202), then f64
        double pw[NREP];
#pragma unroll
        for (int h = 0; h < NREP; ++h) {
            const double s_h = valid ? (double)__fmul_rn((float)sc[h], a.scaling) : -INFINITY;
            double cmax = s_h;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) cmax = fmax(cmax, __shfl_xor_sync(0xffffffffu, cmax, o));
            const double m_new = fmax(m_run[h], cmax);
            const double corr = exp(m_run[h] - m_new);  // exp(-inf) = 0 on the first chunk
            pw[h] = valid ? exp(s_h - m_new) : 0.0;
            double psum = pw[h];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
            l_run[h] = fma(l_run[h], corr, psum);
#pragma unroll
            for (int j = 0; j < PER_LANE; ++j) acc[h][j] *= corr;
            m_run[h] = m_new;
        }
        // (C) acc[h][dims of this lane] += sum_j p_j[h] * v_j[dims]
        const int n_here = min(32, t1 - tb);
        for (int j = 0; j < n_here; ++j) {
            const uint8_t* vr = a.cache.v_q + (row_base + tb + j) * hd + lane * PER_LANE;
            const float vs = a.cache.v_s[row_base + tb + j];
            double vf[PER_LANE];
            if (PER_LANE == 4) {
                const uint32_t w = *reinterpret_cast<const uint32_t*>(vr);
#pragma unroll
                for (int d = 0; d < PER_LANE; ++d) vf[d] = (double)__fmul_rn((float)((w >> (8 * d)) & 0xffu) - 128.0f, vs);
            } else {
#pragma unroll
                for (int d = 0; d < PER_LANE; ++d) vf[d] = (double)__fmul_rn((float)vr[d] - 128.0f, vs);
            }
#pragma unroll
            for (int h = 0; h < NREP; ++h) {
                const double pj = __shfl_sync(0xffffffffu, pw[h], j);
#pragma unroll
                for (int d = 0; d < PER_LANE; ++d) acc[h][d] = fma(pj, vf[d], acc[h][d]);
            }
        }
    }
    // combine the warps of this CTA
#pragma unroll
    for (int h = 0; h < NREP; ++h) {
        if (lane == 0) { red_m[warp][h] = m_run[h]; red_l[warp][h] = l_run[h]; }
#pragma unroll
        for (int j = 0; j < PER_LANE; ++j) red_acc[warp][h][lane * PER_LANE + j] = acc[h][j];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < NREP * hd; i += blockDim.x) {
        const int h = i / hd, c = i % hd;
        double m = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) m = fmax(m, red_m[w][h]);
        double l = 0.0, v = 0.0;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const double scw = red_m[w][h] == -INFINITY ? 0.0 : exp(red_m[w][h] - m);
            l = fma(red_l[w][h], scw, l);
            v = fma(red_acc[w][h][c], scw, v);
        }
        double* dst = part_base + (int64_t)h * a.splits * (hd + 2);
        dst[2 + c] = v;
        if (c == 0) { dst[0] = m; dst[1] = l; }
    }
}

// Merge the per-split partials: out = sum_s e^{m_s - m} acc_s / sum_s e^{m_s - m} l_s.
__global__ void attn_combine_kernel(AttnArgs a) {
    ptx::pdl_wait();
    ptx::pdl_launch_dependents();
    const int hd = a.head_dim;
    const int64_t bh = blockIdx.x;  // b * n_heads + head
    const double* base = a.partial + bh * a.splits * (hd + 2);
    double m = -INFINITY;
    for (int s = 0; s < a.splits; ++s) m = fmax(m, base[s * (hd + 2)]);
    for (int c = threadIdx.x; c < hd; c += blockDim.x) {
        double l = 0.0, v = 0.0;
        for (int s = 0; s < a.splits; ++s) {
            const double ms = base[s * (hd + 2)];
            if (ms == -INFINITY) continue;  // span without positions yet
            const double sc = exp(ms - m);
            l = fma(base[s * (hd + 2) + 1], sc, l);
            v = fma(base[s * (hd + 2) + 2 + c], sc, v);
        }
        const float o = (float)(v / l);
        a.out[bh * hd + c] = o;
        if (a.absmax_out) atomicMax(a.absmax_out + bh / a.n_heads, __float_as_uint(fabsf(o)));
    }
}

}  // namespace

template <int PER_LANE>
static cudaError_t launch_rep(const AttnArgs& a, dim3 grid, cudaStream_t stream) {
    cudaError_t e = cudaSuccess;
    switch (a.n_heads / a.n_kv) {
        case 1: e = launch_pdl(attn_decode_kernel<PER_LANE, 1>, grid, dim3(kAttnThreads), 0, stream, a.pdl, a); break;
        case 2: e = launch_pdl(attn_decode_kernel<PER_LANE, 2>, grid, dim3(kAttnThreads), 0, stream, a.pdl, a); break;
        case 4: e = launch_pdl(attn_decode_kernel<PER_LANE, 4>, grid, dim3(kAttnThreads), 0, stream, a.pdl, a); break;
        default: e = launch_pdl(attn_decode_kernel<PER_LANE, 8>, grid, dim3(kAttnThreads), 0, stream, a.pdl, a); break;
    }
    return e;
}

cudaError_t launch_attn_decode(const AttnArgs& a, cudaStream_t stream) {
    const int rep = a.n_kv > 0 ? a.n_heads / a.n_kv : 0;
    if (a.head_dim % 32 != 0 || a.head_dim > 128 || a.n_heads % a.n_kv != 0 ||
        !(rep == 1 || rep == 2 || rep == 4 || rep == 8))
        return cudaErrorInvalidValue;
    dim3 grid(a.batch * a.n_kv, a.splits);
    cudaError_t e;
    switch (a.head_dim / 32) {
        case 1: e = launch_rep<1>(a, grid, stream); break;
        case 2: e = launch_rep<2>(a, grid, stream); break;
        case 3: e = launch_rep<3>(a, grid, stream); break;
        default: e = launch_rep<4>(a, grid, stream); break;
    }
    if (e != cudaSuccess) return e;
    return launch_pdl(attn_combine_kernel, dim3(a.batch * a.n_heads), dim3(a.head_dim), 0, stream, a.pdl, a);
}

}  // namespace bt
