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

// One CTA = one (sequence, KV head, span of positions), 512 threads.  The span is walked
// in tiles of 128 positions; per tile: (1) the K and V rows are staged in shared memory,
// (2) thread (position, head) forms one score with a 128-long f64 dot product, (3) one warp
// per head turns the tile's scores into softmax weights (running max / sum across tiles),
// (4) thread (head, dim) accumulates P.V over the tile.  No cross-thread reduction of the
// accumulators is needed, and everything between the u8 loads and the final rounding is
// f64, so the result does not depend on how positions are cut into tiles and spans.
constexpr int kTilePos = 128;
constexpr int kRowPad = 144;  // bytes per staged row: 128 + 16, conflict-free 16-byte reads
constexpr int kMaxRep = 8;

struct AttnSmem {
    double qs[kMaxRep][128];
    double pw[kMaxRep][kTilePos];
    float sc[kMaxRep][kTilePos];
    double m_run[kMaxRep], l_run[kMaxRep], corr[kMaxRep];
    float k_s[kTilePos], v_s[kTilePos];
    float knew[128], vnew[128];
    alignas(16) uint8_t k_rows[kTilePos * kRowPad];
    alignas(16) uint8_t v_rows[kTilePos * kRowPad];
};

__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(AttnArgs a) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    AttnSmem& sm = *reinterpret_cast<AttnSmem*>(smem_raw);
#define STAMP(i) do { if (a.dbg && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) a.dbg[i] = ptx::globaltimer(); } while (0)
    STAMP(0);
    ptx::pdl_wait();
    ptx::pdl_launch_dependents();
    STAMP(1);

    const int hd = a.head_dim, half = hd >> 1;
    const int nrep = a.n_heads / a.n_kv;
    const int b = blockIdx.x / a.n_kv, kvh = blockIdx.x % a.n_kv;
    const int split = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int p = a.pos[b];
    const int t_len = p + 1;
    const int t0 = split * a.span;
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
        sm.qs[h][c] = (double)__fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn));
        sm.qs[h][half + c] = (double)__fadd_rn(__fmul_rn(x1, sn), __fmul_rn(x2, cs));
    }
    if (tid < nrep) { sm.m_run[tid] = -INFINITY; sm.l_run[tid] = 0.0; }
    const int64_t row_base = ((int64_t)b * a.n_kv + kvh) * a.cache.max_seq;
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
        if (warp == 0) quant_row_warp(sm.knew, hd, a.cache.k_q + (row_base + p) * hd, a.cache.k_s + row_base + p, lane);
        if (warp == 1) quant_row_warp(sm.vnew, hd, a.cache.v_q + (row_base + p) * hd, a.cache.v_s + row_base + p, lane);
    }
    __syncthreads();  // the block's own global writes are visible to it after the barrier
    STAMP(2);

    // thread-owned output elements (head, dim): items tid, tid + 512
    double acc[2] = {0.0, 0.0};
    const int n_out = nrep * hd;
    const int row16 = hd / 16;  // 16-byte pieces per row

    for (int tb = t0; tb < t1; tb += kTilePos) {
        const int n_here = min(kTilePos, t1 - tb);
        // (1) stage the tile's K and V rows and scales
        for (int i = tid; i < n_here * row16; i += blockDim.x) {
            const int r = i / row16, c16 = i % row16;
            const uint4 kv = reinterpret_cast<const uint4*>(a.cache.k_q + (row_base + tb + r) * hd)[c16];
            const uint4 vv = reinterpret_cast<const uint4*>(a.cache.v_q + (row_base + tb + r) * hd)[c16];
            *reinterpret_cast<uint4*>(sm.k_rows + r * kRowPad + c16 * 16) = kv;
            *reinterpret_cast<uint4*>(sm.v_rows + r * kRowPad + c16 * 16) = vv;
        }
        for (int r = tid; r < n_here; r += blockDim.x) {
            sm.k_s[r] = a.cache.k_s[row_base + tb + r];
            sm.v_s[r] = a.cache.v_s[row_base + tb + r];
        }
        __syncthreads();
        STAMP(3);
        // (2) scores: item = (head, position); position runs over lanes, so q is a broadcast
        for (int it = tid; it < nrep * kTilePos; it += blockDim.x) {
            const int h = it / kTilePos, r = it % kTilePos;
            if (r < n_here) {
                const uint8_t* row = sm.k_rows + r * kRowPad;
                const float ks = sm.k_s[r];
                double d4[4] = {0.0, 0.0, 0.0, 0.0};  // four independent chains, one per byte lane
                for (int c16 = 0; c16 < row16; ++c16) {
                    const uint4 pk = *reinterpret_cast<const uint4*>(row + c16 * 16);
                    const uint32_t wds[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
                    for (int wi = 0; wi < 4; ++wi)
#pragma unroll
                        for (int bi = 0; bi < 4; ++bi) {
                            // dequantize_q8, kv_cache.rs:122-128: (f32(q) - 128) * s
                            const float kf = __fmul_rn((float)((wds[wi] >> (8 * bi)) & 0xffu) - 128.0f, ks);
                            d4[bi] = fma(sm.qs[h][c16 * 16 + wi * 4 + bi], (double)kf, d4[bi]);
                        }
                }
                const double d = (d4[0] + d4[1]) + (d4[2] + d4[3]);
                sm.sc[h][r] = __fmul_rn((float)d, a.scaling);  // (q.k) * 1/sqrt(hd), attention.rs:202
            }
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
        // (4) acc[head, dim] = acc * corr + sum_r p[head, r] * v[r, dim]
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int it = tid + e * kAttnThreads;
            if (it < n_out) {
                const int h = it / hd, dcol = it % hd;
                double v = acc[e] * sm.corr[h];
                for (int r = 0; r < n_here; ++r) {
                    const float vf = __fmul_rn((float)sm.v_rows[r * kRowPad + dcol] - 128.0f, sm.v_s[r]);
                    v = fma(sm.pw[h][r], (double)vf, v);
                }
                acc[e] = v;
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
    for (int it = tid; it < nrep * hd; it += blockDim.x) {
        const int h = it / hd, c = it % hd;
        const double* base = group + (int64_t)h * a.splits * (hd + 2);
        double m = -INFINITY, l = 0.0, v = 0.0;
        for (int s2 = 0; s2 < a.splits; ++s2) {
            const double ms = __ldcg(base + s2 * (hd + 2));
            const double ls = __ldcg(base + s2 * (hd + 2) + 1);
            const double vs2 = __ldcg(base + s2 * (hd + 2) + 2 + c);
            if (ms == -INFINITY) continue;  // span without positions yet
            const double m_new = fmax(m, ms);
            const double c_old = exp(m - m_new), c_new = exp(ms - m_new);  // exp(-inf) = 0 at first
            l = fma(l, c_old, ls * c_new);
            v = fma(v, c_old, vs2 * c_new);
            m = m_new;
        }
        const float o = (float)(v / l);
        a.out[((int64_t)b * a.n_heads + kvh * nrep + h) * hd + c] = o;
        if (a.absmax_out) {
            float mx = fabsf(o);
#pragma unroll
            for (int of = 16; of > 0; of >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, of));
            if (lane == 0) atomicMax(a.absmax_out + b, __float_as_uint(mx));
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
                                              (int)sizeof(AttnSmem));
        if (e0 != cudaSuccess) return e0;
        configured = true;
    }
    dim3 grid(a.batch * a.n_kv, a.splits);
    return launch_pdl(attn_decode_kernel, grid, dim3(kAttnThreads), sizeof(AttnSmem), stream, a.pdl, a);
}

cudaError_t launch_rope_tables(const float* inv_freq, int max_seq, int half, float* cos_t, float* sin_t,
                               cudaStream_t stream) {
    rope_table_kernel<<<148, 256, 0, stream>>>(inv_freq, max_seq, half, cos_t, sin_t);
    return cudaGetLastError();
}

}  // namespace bt
