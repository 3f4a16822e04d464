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

constexpr int kAttnWarps = 16;
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
// q_copy / s_copy: optional second destination (the CTA's prefetched copy of the cache rows).
__device__ __forceinline__ void quant_row_warp(const float* v, int hd, uint8_t* q_out, float* s_out, uint8_t* q_copy,
                                               float* s_copy, int lane) {
    float amax = 0.0f;
    for (int c = lane; c < hd; c += 32) amax = fmaxf(amax, fabsf(v[c]));
    amax = warp_max(amax);
    const float s = __fdiv_rn(amax, 127.0f);
    for (int c = lane; c < hd; c += 32) {
        float r = s > 0.0f ? roundf(__fdiv_rn(v[c], s)) : 0.0f;
        r = fminf(fmaxf(r + 128.0f, 0.0f), 255.0f);
        q_out[c] = (uint8_t)r;
        if (q_copy) q_copy[c] = (uint8_t)r;
    }
    if (lane == 0) {
        *s_out = s;
        if (s_copy) *s_copy = s;
    }
}

// One CTA = one (sequence, KV head, span of positions), 512 threads.  The span is walked
// in tiles of 64 positions; per tile: (1) the K and V rows are dequantised into shared memory,
// (2) thread (head, position, half) forms half of a score with a 64-long f64 dot product, (3) one warp
// per head turns the tile's scores into softmax weights (running max / sum across tiles),
// (4) thread (head, dim) accumulates P.V over the tile.  No cross-thread reduction of the
// accumulators is needed, and everything between the u8 loads and the final rounding is
// f64, so the result does not depend on how positions are cut into tiles and spans.
constexpr int kTilePos = 64;
constexpr int kHalfPad = 68;   // floats per staged half row: 64 + 4, conflict-free 16-byte reads
constexpr int kMaxRep = 8;
constexpr int kRawPos = 128;   // cache rows prefetched per CTA

struct AttnSmem {
    alignas(16) float qs[kMaxRep][128];  // rotated queries (exact f32 values)
    double pw[kMaxRep][kTilePos];
    float sc[kMaxRep][kTilePos];
    double m_run[kMaxRep], l_run[kMaxRep], corr[kMaxRep];
    float knew[128], vnew[128];
    alignas(16) float kf[kTilePos][2][kHalfPad];  // dequantised keys of the tile, two halves of 64 dims
    alignas(16) float vf[kTilePos][128];          // dequantised values of the tile
    // the span's first kRawPos cache rows as stored (u8 + scale), fetched before the kernel
    // waits for its predecessor
    alignas(16) uint8_t kraw[kRawPos * 128];
    alignas(16) uint8_t vraw[kRawPos * 128];
    float ksr[kRawPos], vsr[kRawPos];
};

__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(AttnArgs a) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    AttnSmem& sm = *reinterpret_cast<AttnSmem*>(smem_raw);
#define STAMP(i) do { if (a.dbg && (i) < 8 && threadIdx.x == 0) a.dbg[(blockIdx.y * gridDim.x + blockIdx.x) * 8 + (i)] = ptx::globaltimer(); } while (0)
    STAMP(0);
    const int hd = a.head_dim, half = hd >> 1;
    const int nrep = a.n_heads / a.n_kv;
    const int b = blockIdx.x / a.n_kv, kvh = blockIdx.x % a.n_kv;
    const int split = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int t0 = split * a.span;
    const int64_t row_base = ((int64_t)b * a.n_kv + kvh) * a.cache.max_seq;
    const int row16 = hd / 16;  // 16-byte pieces per row
    // The cache rows of earlier positions were written by earlier steps, so they can be fetched
    // before the dependency wait (whatever sits in rows at or beyond the current position is
    // fetched too and never used; the owner of the new position overwrites its copy below).
    const int raw_rows = max(0, min(min(kRawPos, a.span), a.cache.max_seq - t0));
    {
        const uint4* ksrc = reinterpret_cast<const uint4*>(a.cache.k_q + (row_base + t0) * hd);
        const uint4* vsrc = reinterpret_cast<const uint4*>(a.cache.v_q + (row_base + t0) * hd);
        uint4* kdst = reinterpret_cast<uint4*>(sm.kraw);
        uint4* vdst = reinterpret_cast<uint4*>(sm.vraw);
        const int n16 = raw_rows * row16;
        for (int i0 = tid; i0 < n16; i0 += 2 * kAttnThreads) {
            const int i1 = i0 + kAttnThreads;
            const bool h1 = i1 < n16;
            const uint4 k0 = ksrc[i0], v0 = vsrc[i0];
            uint4 k1 = make_uint4(0u, 0u, 0u, 0u), v1 = k1;
            if (h1) { k1 = ksrc[i1]; v1 = vsrc[i1]; }
            kdst[i0] = k0; vdst[i0] = v0;
            if (h1) { kdst[i1] = k1; vdst[i1] = v1; }
        }
        if (tid < raw_rows) sm.ksr[tid] = a.cache.k_s[row_base + t0 + tid];
        else if (tid >= 256 && tid - 256 < raw_rows) sm.vsr[tid - 256] = a.cache.v_s[row_base + t0 + tid - 256];
    }
    ptx::pdl_wait();
    STAMP(1);

    const int p = a.pos[b];
    const int t_len = p + 1;
    const int t1 = min(t_len, t0 + a.span);
    const int64_t qkv_stride = (int64_t)(a.n_heads + 2 * a.n_kv) * hd;
    const float* qkv = a.qkv + b * qkv_stride;
    double* part_base = a.partial + (((int64_t)b * a.n_heads + kvh * nrep) * a.splits + split) * (hd + 2);
    const bool empty = t0 >= t_len;
    if (empty) {
        // nothing in this span yet: leave an empty partial (max = -inf, sum = 0)
        for (int h = tid; h < nrep; h += blockDim.x) {
            double* dst = part_base + (int64_t)h * a.splits * (hd + 2);
            dst[0] = -INFINITY;
            dst[1] = 0.0;
        }
    }
    if (!empty) {
    const float* cos_p = a.rope_cos + (int64_t)p * half;
    const float* sin_p = a.rope_sin + (int64_t)p * half;

    // rotate the query heads of this KV group: [x1*cos - x2*sin, x1*sin + x2*cos] (attention.rs:79-83)
    for (int i = tid; i < nrep * half; i += blockDim.x) {
        const int h = i / half, c = i % half;
        const float cs = cos_p[c], sn = sin_p[c];
        const float* qh = qkv + (int64_t)(kvh * nrep + h) * hd;
        const float x1 = qh[c], x2 = qh[half + c];
        sm.qs[h][c] = __fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn));
        sm.qs[h][half + c] = __fadd_rn(__fmul_rn(x1, sn), __fmul_rn(x2, cs));
    }
    if (tid < nrep) { sm.m_run[tid] = -INFINITY; sm.l_run[tid] = 0.0; }
    // the CTA whose span holds position p appends the new key / value first
    const bool owner = (p >= t0 && p < t1);
    if (owner) {
        const float* kh = qkv + (int64_t)(a.n_heads + kvh) * hd;
        const float* vh = qkv + (int64_t)(a.n_heads + a.n_kv + kvh) * hd;
        for (int c = tid; c < half; c += blockDim.x) {
            const float cs = cos_p[c], sn = sin_p[c];
            const float x1 = kh[c], x2 = kh[half + c];
            sm.knew[c] = __fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn));
            sm.knew[half + c] = __fadd_rn(__fmul_rn(x1, sn), __fmul_rn(x2, cs));
        }
        for (int c = tid; c < hd; c += blockDim.x) sm.vnew[c] = vh[c];
    }
    __syncthreads();
    if (owner) {
        const bool in_raw = p - t0 < raw_rows;
        if (warp == 0) quant_row_warp(sm.knew, hd, a.cache.k_q + (row_base + p) * hd, a.cache.k_s + row_base + p,
                                      in_raw ? sm.kraw + (p - t0) * hd : nullptr, in_raw ? sm.ksr + (p - t0) : nullptr, lane);
        if (warp == 1) quant_row_warp(sm.vnew, hd, a.cache.v_q + (row_base + p) * hd, a.cache.v_s + row_base + p,
                                      in_raw ? sm.vraw + (p - t0) * hd : nullptr, in_raw ? sm.vsr + (p - t0) : nullptr, lane);
    }
    __syncthreads();  // the block's own global writes are visible to it after the barrier
    STAMP(2);

    // thread-owned output elements (head, dim): items tid, tid + 512
    double acc[2] = {0.0, 0.0};
    const int n_out = nrep * hd;

    for (int tb = t0; tb < t1; tb += kTilePos) {
        const int n_here = min(kTilePos, t1 - tb);
        // (1) stage the tile: every byte is dequantised once, (f32(q) - 128) * s
        //     (dequantize_q8, kv_cache.rs:122-128), into f32 rows
        for (int i = tid; i < n_here * row16; i += blockDim.x) {
            const int r = i / row16, c16 = i % row16;
            const int rr = tb - t0 + r;  // row within the span
            uint4 kv, vv;
            float ks, vs;
            if (rr < raw_rows) {
                kv = reinterpret_cast<const uint4*>(sm.kraw + rr * hd)[c16];
                vv = reinterpret_cast<const uint4*>(sm.vraw + rr * hd)[c16];
                ks = sm.ksr[rr];
                vs = sm.vsr[rr];
            } else {
                kv = reinterpret_cast<const uint4*>(a.cache.k_q + (row_base + tb + r) * hd)[c16];
                vv = reinterpret_cast<const uint4*>(a.cache.v_q + (row_base + tb + r) * hd)[c16];
                ks = a.cache.k_s[row_base + tb + r];
                vs = a.cache.v_s[row_base + tb + r];
            }
            const uint32_t kw[4] = {kv.x, kv.y, kv.z, kv.w}, vw[4] = {vv.x, vv.y, vv.z, vv.w};
            float* kdst = &sm.kf[r][(c16 * 16) >> 6][(c16 * 16) & 63];
            float* vdst = &sm.vf[r][c16 * 16];
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                float4 ko, vo;
                ko.x = __fmul_rn((float)(kw[wi] & 0xffu) - 128.0f, ks);
                ko.y = __fmul_rn((float)((kw[wi] >> 8) & 0xffu) - 128.0f, ks);
                ko.z = __fmul_rn((float)((kw[wi] >> 16) & 0xffu) - 128.0f, ks);
                ko.w = __fmul_rn((float)(kw[wi] >> 24) - 128.0f, ks);
                vo.x = __fmul_rn((float)(vw[wi] & 0xffu) - 128.0f, vs);
                vo.y = __fmul_rn((float)((vw[wi] >> 8) & 0xffu) - 128.0f, vs);
                vo.z = __fmul_rn((float)((vw[wi] >> 16) & 0xffu) - 128.0f, vs);
                vo.w = __fmul_rn((float)(vw[wi] >> 24) - 128.0f, vs);
                *reinterpret_cast<float4*>(kdst + 4 * wi) = ko;
                *reinterpret_cast<float4*>(vdst + 4 * wi) = vo;
            }
        }
        __syncthreads();
        STAMP(3);
        // (2) scores: item = (head, position, half of the head dims); the two halves sit in
        //     neighbouring lanes and are added with one shuffle
        for (int it = tid; it < nrep * kTilePos * 2; it += blockDim.x) {
            const int hf = it & 1, r = (it >> 1) % kTilePos, h = it / (2 * kTilePos);
            const int c0 = hf * 64, cn = min(64, hd - c0);
            double d0 = 0.0, d1 = 0.0;
            if (r < n_here && cn > 0) {
                const float* row = sm.kf[r][hf];
                const float* qh = sm.qs[h] + c0;
#pragma unroll 4
                for (int c = 0; c < cn; c += 4) {
                    const float4 k4 = *reinterpret_cast<const float4*>(row + c);
                    const float4 q4 = *reinterpret_cast<const float4*>(qh + c);
                    d0 = fma((double)q4.x, (double)k4.x, d0);
                    d1 = fma((double)q4.y, (double)k4.y, d1);
                    d0 = fma((double)q4.z, (double)k4.z, d0);
                    d1 = fma((double)q4.w, (double)k4.w, d1);
                }
            }
            double d = d0 + d1;
            d += __shfl_xor_sync(0xffffffffu, d, 1);
            if (hf == 0 && r < n_here) sm.sc[h][r] = __fmul_rn((float)d, a.scaling);  // (q.k) * 1/sqrt(hd), attention.rs:202
        }
        __syncthreads();
        STAMP(4);
        // (3) softmax weights of the tile, one warp per head
        if (warp < nrep) {
            const int h = warp;
            double sv[kTilePos / 32];
            double tmax = -INFINITY;
#pragma unroll
            for (int i = 0; i < kTilePos / 32; ++i) {
                const int r = lane + 32 * i;
                sv[i] = r < n_here ? (double)sm.sc[h][r] : -INFINITY;
                tmax = fmax(tmax, sv[i]);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) tmax = fmax(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
            const double m_old = sm.m_run[h];
            const double m_new = fmax(m_old, tmax);
            double psum = 0.0;
#pragma unroll
            for (int i = 0; i < kTilePos / 32; ++i) {
                const int r = lane + 32 * i;
                const double pe = r < n_here ? exp(sv[i] - m_new) : 0.0;
                sm.pw[h][r] = pe;
                psum += pe;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) psum += __shfl_xor_sync(0xffffffffu, psum, o);
            if (lane == 0) {
                const double corr = exp(m_old - m_new);  // exp(-inf) = 0 on the first tile
                sm.corr[h] = corr;
                sm.l_run[h] = fma(sm.l_run[h], corr, psum);
                sm.m_run[h] = m_new;
            }
        }
        __syncthreads();
        STAMP(5);
        // (4) acc[head, dim] = acc * corr + sum_r p[head, r] * v[r, dim], two chains per thread
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int it = tid + e * kAttnThreads;
            if (it < n_out) {
                const int h = it / hd, dcol = it % hd;
                double v0 = acc[e] * sm.corr[h], v1 = 0.0;
                int r = 0;
                for (; r + 1 < n_here; r += 2) {
                    v0 = fma(sm.pw[h][r], (double)sm.vf[r][dcol], v0);
                    v1 = fma(sm.pw[h][r + 1], (double)sm.vf[r + 1][dcol], v1);
                }
                if (r < n_here) v0 = fma(sm.pw[h][r], (double)sm.vf[r][dcol], v0);
                acc[e] = v0 + v1;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int it = tid + e * kAttnThreads;
        if (it < n_out) {
            const int h = it / hd, dcol = it % hd;
            double* dst = part_base + (int64_t)h * a.splits * (hd + 2);
            dst[2 + dcol] = acc[e];
            if (dcol == 0) { dst[0] = sm.m_run[h]; dst[1] = sm.l_run[h]; }
        }
    }
    }  // !empty
    STAMP(6);
    // only now may the next kernel's CTAs move in: earlier they would take the registers and
    // shared memory that this kernel's later CTAs are waiting for
    ptx::pdl_launch_dependents();

    // The last CTA of this (sequence, KV head) to get here merges the spans:
    // out = sum_s e^{m_s - m} acc_s / sum_s e^{m_s - m} l_s, rounded to f32 once.
    __threadfence();
    __syncthreads();
    __shared__ unsigned int arrived;
    if (tid == 0) arrived = atomicAdd(a.counters + blockIdx.x, 1u);
    __syncthreads();
    STAMP(7);
    if (arrived != (unsigned int)a.splits - 1) return;
    __threadfence();
    if (tid == 0) a.counters[blockIdx.x] = 0;  // ready for the next launch
    const double* group = a.partial + ((int64_t)b * a.n_heads + kvh * nrep) * a.splits * (hd + 2);
    // One batch of independent loads: every span's maximum and sum into shared memory and, at
    // the same time, this thread's output column of the first spans into registers; the weights
    // w_s = e^{m_s - m} are formed while those are in flight.
    constexpr int kMergeBatch = 16;
    double* mw = reinterpret_cast<double*>(sm.vf);          // [nrep][64] maxima, then weights (the tile buffers are free now)
    double* ls = mw + kMaxRep * 64;                          // [nrep][64] sums
    double* lsum = ls + kMaxRep * 64;                        // [nrep] merged denominators
    for (int i = tid; i < nrep * a.splits; i += blockDim.x) {
        const int h = i / a.splits, s2 = i % a.splits;
        const double* src = group + ((int64_t)h * a.splits + s2) * (hd + 2);
        mw[h * 64 + s2] = __ldcg(src);
        ls[h * 64 + s2] = __ldcg(src + 1);
    }
    // (head, column) items: item tid and, for nrep * hd > 512, item tid + 512
    double pre[2][kMergeBatch];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int it = tid + e * kAttnThreads;
        if (it < nrep * hd) {
            const int h = it / hd, c = it % hd;
            const double* base = group + (int64_t)h * a.splits * (hd + 2) + 2 + c;
#pragma unroll
            for (int s2 = 0; s2 < kMergeBatch; ++s2)
                pre[e][s2] = s2 < a.splits ? __ldcg(base + (int64_t)s2 * (hd + 2)) : 0.0;
        }
    }
    __syncthreads();
    if (warp < nrep) {
        const int h = warp;
        double m = -INFINITY;
        for (int s2 = lane; s2 < a.splits; s2 += 32) m = fmax(m, mw[h * 64 + s2]);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmax(m, __shfl_xor_sync(0xffffffffu, m, o));
        double l = 0.0;
        for (int s2 = lane; s2 < a.splits; s2 += 32) {
            const double ms = mw[h * 64 + s2];
            const double w = ms == -INFINITY ? 0.0 : exp(ms - m);  // spans without positions weigh nothing
            l = fma(ls[h * 64 + s2], w, l);
            mw[h * 64 + s2] = w;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
        if (lane == 0) lsum[h] = l;
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int it = tid + e * kAttnThreads;
        if (it < nrep * hd) {
            const int h = it / hd, c = it % hd;
            const double* base = group + (int64_t)h * a.splits * (hd + 2) + 2 + c;
            double v0 = 0.0, v1 = 0.0;
#pragma unroll
            for (int s2 = 0; s2 < kMergeBatch; s2 += 2) {
                // (spans without positions have weight 0 but may hold anything: skip them)
                if (s2 < a.splits && mw[h * 64 + s2] != 0.0) v0 = fma(pre[e][s2], mw[h * 64 + s2], v0);
                if (s2 + 1 < a.splits && mw[h * 64 + s2 + 1] != 0.0) v1 = fma(pre[e][s2 + 1], mw[h * 64 + s2 + 1], v1);
            }
            for (int s2 = kMergeBatch; s2 < a.splits; s2 += 2) {
                if (mw[h * 64 + s2] != 0.0) v0 = fma(__ldcg(base + (int64_t)s2 * (hd + 2)), mw[h * 64 + s2], v0);
                if (s2 + 1 < a.splits && mw[h * 64 + s2 + 1] != 0.0)
                    v1 = fma(__ldcg(base + (int64_t)(s2 + 1) * (hd + 2)), mw[h * 64 + s2 + 1], v1);
            }
            const float o = (float)((v0 + v1) / lsum[h]);
            a.out[((int64_t)b * a.n_heads + kvh * nrep + h) * hd + c] = o;
            if (a.absmax_out) {
                float mx = fabsf(o);
#pragma unroll
                for (int of = 16; of > 0; of >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, of));
                if (lane == 0) atomicMax(a.absmax_out + b, __float_as_uint(mx));
            }
        }
    }
    STAMP(8);
}

__global__ void rope_table_kernel(const float* __restrict__ inv_freq, int max_seq, int half,
                                  float* __restrict__ cos_t, float* __restrict__ sin_t) {
    const int64_t n = (int64_t)max_seq * half;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        const int pos = (int)(i / half), c = (int)(i % half);
        const float fr = __fmul_rn((float)pos, inv_freq[c]);  // f32 product, attention.rs:30
        cos_t[i] = (float)cos((double)fr);
        sin_t[i] = (float)sin((double)fr);
    }
}

}  // namespace

cudaError_t launch_attn_decode(const AttnArgs& a, cudaStream_t stream) {
    const int rep = a.n_kv > 0 ? a.n_heads / a.n_kv : 0;
    if (a.head_dim % 32 != 0 || a.head_dim > 128 || a.n_heads % a.n_kv != 0 || rep < 1 || rep > kMaxRep ||
        a.span % 32 != 0)
        return cudaErrorInvalidValue;
    static bool configured = false;
    if (!configured) {
        cudaError_t e0 = cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              (int)(sizeof(AttnSmem) > 116 * 1024 ? sizeof(AttnSmem) : 116 * 1024));
        if (e0 != cudaSuccess) return e0;
        configured = true;
    }
    dim3 grid(a.batch * a.n_kv, a.splits);
    // When the whole grid fits one CTA per SM, ask for more than half of an SM's shared
    // memory: the block scheduler then cannot pair two CTAs on one SM while others idle
    // (measured: paired CTAs take 22 us instead of 16).
    size_t smem = sizeof(AttnSmem);
    if ((int64_t)grid.x * grid.y <= a.sm_count && smem < 116 * 1024) smem = 116 * 1024;
    return launch_pdl(attn_decode_kernel, grid, dim3(kAttnThreads), smem, stream, a.pdl, a);
}

cudaError_t launch_rope_tables(const float* inv_freq, int max_seq, int half, float* cos_t, float* sin_t,
                               cudaStream_t stream) {
    rope_table_kernel<<<148, 256, 0, stream>>>(inv_freq, max_seq, half, cos_t, sin_t);
    return cudaGetLastError();
}

}  // namespace bt
