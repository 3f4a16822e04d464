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

template <int PER_LANE, int NREP>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(AttnArgs a) {
    __shared__ float qs[NREP * 128];
    __shared__ float knew[128], vnew[128];
    __shared__ double red_m[kAttnWarps][NREP], red_l[kAttnWarps][NREP];
    __shared__ double red_acc[kAttnWarps][NREP][32 * PER_LANE];
    ptx::pdl_wait();
    ptx::pdl_launch_dependents();

    const int hd = a.head_dim, half = hd >> 1;
    const int b = blockIdx.x / a.n_kv, kvh = blockIdx.x % a.n_kv;
    const int split = blockIdx.y;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int p = a.pos[b];
    const int t_len = p + 1;
    const int chunk = (t_len + a.splits - 1) / a.splits;
    const int t0 = split * chunk;
    const int t1 = min(t_len, t0 + chunk);
    const int64_t qkv_stride = (int64_t)(a.n_heads + 2 * a.n_kv) * hd;
    const float* qkv = a.qkv + b * qkv_stride;
    const float fp = (float)p;

    // rotate the NREP query heads of this KV group (cos/sin evaluated in f64, rounded once)
    for (int i = threadIdx.x; i < NREP * half; i += blockDim.x) {
        const int h = i / half, c = i % half;
        const float fr = __fmul_rn(fp, a.inv_freq[c]);
        const float cs = (float)cos((double)fr), sn = (float)sin((double)fr);
        const float* qh = qkv + (int64_t)(kvh * NREP + h) * hd;
        const float x1 = qh[c], x2 = qh[half + c];
        qs[h * hd + c] = __fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn));
        qs[h * hd + half + c] = __fadd_rn(__fmul_rn(x1, sn), __fmul_rn(x2, cs));
    }
    const int64_t row_base = ((int64_t)b * a.n_kv + kvh) * a.cache.max_seq;
    // the CTA whose range holds position p appends the new key / value first
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

    // Scores, softmax weights and the weighted sum are carried in f64 and rounded to f32
    // once at the end, so that the result does not depend on how positions are split over
    // warps and CTAs.
    double m_run[NREP], l_run[NREP], acc[NREP][PER_LANE];
    float qreg[NREP][PER_LANE];
#pragma unroll
    for (int h = 0; h < NREP; ++h) {
        m_run[h] = -INFINITY;
        l_run[h] = 0.0;
#pragma unroll
        for (int j = 0; j < PER_LANE; ++j) {
            acc[h][j] = 0.0;
            qreg[h][j] = (lane * PER_LANE + j < hd) ? qs[h * hd + lane * PER_LANE + j] : 0.0f;
        }
    }

    for (int t = t0 + warp; t < t1; t += kAttnWarps) {
        const uint8_t* kr = a.cache.k_q + (row_base + t) * hd + lane * PER_LANE;
        const uint8_t* vr = a.cache.v_q + (row_base + t) * hd + lane * PER_LANE;
        float kf[PER_LANE], vf[PER_LANE];
        const float ks = a.cache.k_s[row_base + t], vs = a.cache.v_s[row_base + t];
#pragma unroll
        for (int j = 0; j < PER_LANE; ++j) {
            kf[j] = __fmul_rn((float)kr[j] - 128.0f, ks);   // dequantize_q8, kv_cache.rs:122-128
            vf[j] = __fmul_rn((float)vr[j] - 128.0f, vs);
        }
#pragma unroll
        for (int h = 0; h < NREP; ++h) {
            double d = 0.0;
#pragma unroll
            for (int j = 0; j < PER_LANE; ++j) d = fma((double)qreg[h][j], (double)kf[j], d);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
            const double sc = (double)__fmul_rn((float)d, a.scaling);  // (q.k) * 1/sqrt(hd), attention.rs:202
            const double m_new = fmax(m_run[h], sc);
            const double corr = exp(m_run[h] - m_new);  // exp(-inf) = 0 on the first key
            const double pe = exp(sc - m_new);
            l_run[h] = fma(l_run[h], corr, pe);
#pragma unroll
            for (int j = 0; j < PER_LANE; ++j) acc[h][j] = fma(acc[h][j], corr, pe * (double)vf[j]);
            m_run[h] = m_new;
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
            const double sc = red_m[w][h] == -INFINITY ? 0.0 : exp(red_m[w][h] - m);
            l = fma(red_l[w][h], sc, l);
            v = fma(red_acc[w][h][c], sc, v);
        }
        const int head = kvh * NREP + h;
        double* dst = a.partial + (((int64_t)b * a.n_heads + head) * a.splits + split) * (hd + 2);
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
            const double sc = ms == -INFINITY ? 0.0 : exp(ms - m);
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
