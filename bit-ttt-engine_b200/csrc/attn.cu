// Fused decode attention over the Q8 KV cache: RoPE (layers/attention.rs:45-84) on the new
// q and k, Q8 append of k and v (layers/kv_cache.rs:95-119), scores = (q.k)/sqrt(hd) over
// positions 0..pos, softmax, .V (layers/attention.rs:198-217), all heads of a KV group in
// one CTA so the cache is read once (the reference materialises repeat_kv copies,
// layers/attention.rs:228-239).  The cache is read in place as u8; nothing is
// re-materialised in f32 (the reference dequantises the whole cache every step,
// layers/kv_cache.rs:84-92).  HBM-bound on the cache bytes: 2*n_kv*T*(hd+4) per sequence.
//
// Arithmetic.  Both contractions run on the tensor cores (mma.sync.m16n8k16, bf16 operands,
// f32 accumulators) with operands that are exact:
//   * a cache byte b stands for the integer b - 128 in [-128, 127], which bf16 holds exactly;
//     the row scale (one f32 per cached row) is applied to the f32 result;
//   * an f32 factor (a rotated query value, a softmax weight times the value-row scale) is cut
//     into three bf16 pieces hi + mid + lo = x (8 + 8 + 8 significand bits), which ride as
//     extra columns (scores) or rows (P.V) of the same MMA and are added in f32 afterwards.
// Every product is therefore exact and only the f32 accumulation rounds: the result is within
// about 1e-6 relative of the f32 value of layers/attention.rs:202-217.  Softmax runs in f32.
//
// Work split.  One CTA = one (sequence, KV head, span of positions); the spans of one
// (sequence, KV head) form a thread-block cluster, and the partial results (running maximum,
// denominator, unnormalised output) are merged through distributed shared memory: after a
// cluster barrier every CTA of the cluster finishes a slice of the output columns, reading the
// partials of all spans with ld.shared::cluster.  No global scratch, no second launch.
#include <stddef.h>

#include "bt_model.cuh"
#include "bt_ptx.cuh"

namespace bt {

namespace {

constexpr int kAttnWarps = 8;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kTilePos = 128;   // cache rows per tile
constexpr int kMaxRep = 8;      // query heads per KV head
constexpr int kMaxHd = 128;
constexpr int kRowPad = 16;     // bytes added to a cache row in shared memory (row stride = 16 mod 32: 4-byte
                                // fragment loads of 8 consecutive rows fall into different banks)
constexpr int kMaxRowBytes = kMaxHd + kRowPad;
constexpr int kQpStride = kMaxHd + 8;    // bf16 elements per row of the query pieces
constexpr int kSrStride = kTilePos + 4;  // floats per row of the raw scores
constexpr int kPwStride = kTilePos + 8;  // bf16 elements per row of the P.V weights
constexpr int kMaxCluster = 16;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Quantise one head vector held in shared memory (hd values) by one warp:
// s = max|x| / 127, q = u8(round(x / s) + 128)  (quantize_q8, layers/kv_cache.rs:95-119; an all-zero
// row gives s = 0, q = 128).  q_copy / s_copy: optional second destination (a prefetched copy of the row).
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

// G = query vectors that share the K/V rows of a CTA: the NREP heads of a KV group (decode) times the
// QB query positions of a block (prefill).  "Row" below = piece * G + query vector.
template <int G>
struct AttnSmemT {
    static constexpr int kRows = 3 * G;
    static constexpr int kRows16 = (kRows + 15) / 16 * 16;
    // cache rows as stored (u8, rows padded), two tiles: while one is worked on, the next arrives;
    // after the last tile both arrays serve as scratch of the warp reduction
    alignas(16) uint8_t kraw[2][kTilePos * kMaxRowBytes];
    alignas(16) uint8_t vraw[2][kTilePos * kMaxRowBytes];
    alignas(16) float ksr[2][kTilePos];
    alignas(16) float vsr[2][kTilePos];
    alignas(16) __nv_bfloat16 qp[kRows][kQpStride];        // rotated queries
    alignas(16) float sraw[kRows][kSrStride];              // per-piece dot products of the tile
    alignas(16) __nv_bfloat16 pw[kRows16][kPwStride];      // pieces of p * v_scale
    alignas(16) float opart[G * kMaxHd];                   // this span's unnormalised output [query vector][dim] (read by the cluster)
    float ml[2][G];                                        // this span's running maximum / denominator (read by the cluster)
    float corr[G];
    float wmax[G][4];
    float wsum[G][4];
    float knew[kMaxHd], vnew[kMaxHd];
};

// D(16x8, f32) += A(16x16, bf16, row) * B(16x8, bf16, col)
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ptx::smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst_smem, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(ptx::smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// f32(byte `which` of word) - 128 without an integer-to-float conversion: 0x4B0000bb is the float
// 2^23 + b, and subtracting 2^23 + 128 is exact.
__device__ __forceinline__ float byte_minus_128(uint32_t word, int which) {
    return __fsub_rn(__uint_as_float(__byte_perm(word, 0x4B000000u, 0x7540 + which)), 8388736.0f);
}
// two integers in [-128, 127] as a bf16 pair (exact), `lo` in the low half
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    const __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&p);
}
// x = hi + mid + lo with three bf16 terms (the residuals are exact f32 differences)
__device__ __forceinline__ void split3(float x, __nv_bfloat16& hi, __nv_bfloat16& mid, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(x);
    const float r1 = __fsub_rn(x, __bfloat162float(hi));
    mid = __float2bfloat16_rn(r1);
    lo = __float2bfloat16_rn(__fsub_rn(r1, __bfloat162float(mid)));
}

// ---- thread-block cluster primitives -----------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// f32 at the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ float ld_cluster_f32(const float* local, uint32_t rank) {
    uint32_t remote;
    float v;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(ptx::smem_u32(local)), "r"(rank));
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
    return v;
}

// QB = 1: decode, one new token per sequence; blockIdx.y = span of positions, the spans of a (sequence, KV
// head) form a cluster.  QB > 1: prefill, a.q_rows new tokens per sequence whose K/V rows are already in the
// cache; blockIdx.y = block of QB consecutive query positions, which sees the keys up to its own position
// (causal rule of layers/attention.rs:249-262: key j is visible to query i when j <= i + past).
template <int NREP, int QB>
__global__ void __launch_bounds__(kAttnThreads, QB == 1 ? 2 : 1) attn_kernel(AttnArgs a) {
    constexpr int G = NREP * QB;
    using Smem = AttnSmemT<G>;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
    constexpr int kRowsUsed = 3 * G;               // (piece, query vector) rows
    constexpr int NB = (kRowsUsed + 7) / 8;        // 8-column blocks of the score MMAs
    constexpr int MB = (kRowsUsed + 15) / 16;      // 16-row blocks of the P.V MMAs
    const int hd = a.head_dim, half = hd >> 1;
    const int b = blockIdx.x / a.n_kv, kvh = blockIdx.x % a.n_kv;
    const int split = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    // Decode: the spans follow the sequence's current length, not the capacity the launch was planned
    // for: every CTA of a (sequence, KV head) gets an equal share (a multiple of 32 positions) of
    // what the cache holds now.  The position counter is only written by the last kernel of a
    // decode step, and steps do not overlap, so it may be read before the dependency wait.
    // Prefill: p is the position of the sequence's first new token; the block of queries q0 .. q0 + QB - 1
    // walks the keys 0 .. p + q0 + QB - 1.
    const int p = a.pos[b];
    const int q0 = QB == 1 ? 0 : split * QB;
    const int t_len = QB == 1 ? p + 1 : min(p + q0 + QB, p + a.q_rows);
    int span = ((t_len + a.splits - 1) / a.splits + 31) & ~31;
    if (span > a.span) span = a.span;
    const int t0 = QB == 1 ? split * span : 0;
    const int t1 = QB == 1 ? min(t_len, t0 + span) : t_len;
    const int64_t row_base = ((int64_t)b * a.n_kv + kvh) * a.cache.max_seq;
    const int row16 = hd >> 4;            // 16-byte pieces per row
    const int rstride = hd + kRowPad;     // row stride of the tiles in shared memory

    // cache rows [r0, r0 + n) of this (sequence, KV head) -> tile buffer `buf` (asynchronous copies)
    auto fetch_tile = [&](int buf, int r0, int n) {
        const uint8_t* ksrc = a.cache.k_q + (row_base + r0) * hd;
        const uint8_t* vsrc = a.cache.v_q + (row_base + r0) * hd;
        for (int i = tid; i < n * row16; i += kAttnThreads) {
            const int o = (i / row16) * rstride + (i % row16) * 16;
            cp_async16(sm.kraw[buf] + o, ksrc + 16 * i);
            cp_async16(sm.vraw[buf] + o, vsrc + 16 * i);
        }
        for (int i = tid; i < n; i += kAttnThreads) {
            cp_async4(&sm.ksr[buf][i], a.cache.k_s + row_base + r0 + i);
            cp_async4(&sm.vsr[buf][i], a.cache.v_s + row_base + r0 + i);
        }
    };
    // The cache rows of earlier positions were written by earlier steps, so the first tile can be
    // requested before the dependency wait (the row of the current position is fetched too, with
    // whatever it holds; its owner overwrites the copy below).
    const int n_first = max(0, min(kTilePos, t1 - t0));
    if (QB == 1) fetch_tile(0, t0, n_first);  // (prefill: the new rows come from the kernel just before)
    // (piece, query vector) rows of the P.V weights beyond the ones in use stay zero
    for (int i = tid; i < (Smem::kRows16 - kRowsUsed) * kPwStride; i += kAttnThreads)
        sm.pw[kRowsUsed + i / kPwStride][i % kPwStride] = __float2bfloat16_rn(0.0f);
    ptx::pdl_wait();
    if (QB > 1) fetch_tile(0, t0, n_first);

    const int64_t qkv_stride = (int64_t)(a.n_heads + 2 * a.n_kv) * hd;
    const float* qkv = a.qkv + (int64_t)b * a.q_rows * qkv_stride;  // first new token of the sequence
    const bool empty = t0 >= t_len;
    const bool owner = QB == 1 && (p >= t0 && p < t1);
    if (!empty) {
        const float* cos_p = a.rope_cos + (int64_t)p * half;
        const float* sin_p = a.rope_sin + (int64_t)p * half;
        // rotate the query vectors of this CTA, [x1*cos - x2*sin, x1*sin + x2*cos] (attention.rs:79-83),
        // and cut every value into its three bf16 pieces.  Query vector v = (position q0 + v / NREP, head
        // v % NREP); a block that reaches beyond the last new token repeats the last one (never stored).
        for (int i = tid; i < G * half; i += kAttnThreads) {
            const int v = i / half, c = i % half;
            const int h = v % NREP, qi = min(q0 + v / NREP, a.q_rows - 1);
            const float cs = a.rope_cos[(int64_t)(p + qi) * half + c], sn = a.rope_sin[(int64_t)(p + qi) * half + c];
            const float* qh = qkv + (int64_t)qi * qkv_stride + (int64_t)(kvh * NREP + h) * hd;
            const float x1 = qh[c], x2 = qh[half + c];
            const float r1 = __fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn));
            const float r2 = __fadd_rn(__fmul_rn(x1, sn), __fmul_rn(x2, cs));
            split3(r1, sm.qp[v][c], sm.qp[G + v][c], sm.qp[2 * G + v][c]);
            split3(r2, sm.qp[v][half + c], sm.qp[G + v][half + c], sm.qp[2 * G + v][half + c]);
        }
        // the CTA whose span holds position p appends the new key / value first
        if (owner) {
            const float* kh = qkv + (int64_t)(a.n_heads + kvh) * hd;
            const float* vh = qkv + (int64_t)(a.n_heads + a.n_kv + kvh) * hd;
            for (int c = tid; c < half; c += kAttnThreads) {
                const float cs = cos_p[c], sn = sin_p[c];
                const float x1 = kh[c], x2 = kh[half + c];
                sm.knew[c] = __fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn));
                sm.knew[half + c] = __fadd_rn(__fmul_rn(x1, sn), __fmul_rn(x2, cs));
            }
            for (int c = tid; c < hd; c += kAttnThreads) sm.vnew[c] = vh[c];
        }
    }
    if (tid < G) {
        sm.ml[0][tid] = -INFINITY;  // a span without positions keeps these: weight 0 in the merge
        sm.ml[1][tid] = 0.0f;
    }
    cp_async_wait_all();
    __syncthreads();  // first tile landed; rotated q / k / v visible
    if (owner) {
        const bool in_first = p - t0 < n_first;
        if (warp == 0) quant_row_warp(sm.knew, hd, a.cache.k_q + (row_base + p) * hd, a.cache.k_s + row_base + p,
                                      in_first ? sm.kraw[0] + (p - t0) * rstride : nullptr, in_first ? sm.ksr[0] + (p - t0) : nullptr, lane);
        if (warp == 1) quant_row_warp(sm.vnew, hd, a.cache.v_q + (row_base + p) * hd, a.cache.v_s + row_base + p,
                                      in_first ? sm.vraw[0] + (p - t0) * rstride : nullptr, in_first ? sm.vsr[0] + (p - t0) : nullptr, lane);
    }
    __syncthreads();  // the block's own global writes are visible to its later copies after the barrier

    // P.V ownership: warp = (group of 32 dims dg, position group pq); the warp handles the 16-position
    // steps pq, pq + n_pq, ... of every tile for dims 32 dg .. 32 dg + 31.  One 32-bit load of a V row
    // (dims 32 dg + 4 g .. + 3) feeds four MMAs, MMA e holding dim 32 dg + 4 n + e in column n.
    const int n_dg = hd >> 5;
    const int n_pq = kAttnWarps / n_dg;
    const int dg = warp % n_dg, pq = warp / n_dg;
    const bool pv_active = pq < n_pq;
    float acc[MB][4][4];
#pragma unroll
    for (int mb = 0; mb < MB; ++mb)
#pragma unroll
        for (int e = 0; e < 4; ++e)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[mb][e][j] = 0.0f;

    if (!empty) {
        int cur = 0;
        for (int tb = t0; tb < t1; tb += kTilePos) {
            const int n_here = min(kTilePos, t1 - tb);
            if (tb + kTilePos < t1)  // long span: the next tile's rows go into the other buffer meanwhile
                fetch_tile(cur ^ 1, tb + kTilePos, min(kTilePos, t1 - tb - kTilePos));
            const uint8_t* kraw = sm.kraw[cur];
            const uint8_t* vraw = sm.vraw[cur];
            // (1) per-piece dot products S[16 positions x (piece, head)] = K[16 x hd] . q[hd x (piece, head)]:
            //     warp w owns positions 16 w .. 16 w + 15.  Lane (g, t) supplies dims 16 j + 4 t .. + 3 of
            //     rows g and g + 8 in step j (the order of the dims inside a step is free as long as q
            //     follows it).  Rows at or beyond n_here hold anything; they only reach their own row of
            //     S, which the softmax ignores.
            if (16 * warp < n_here) {
                float c[NB][4];
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) c[nb][0] = c[nb][1] = c[nb][2] = c[nb][3] = 0.0f;
                const uint8_t* krow0 = kraw + (16 * warp + g) * rstride + 4 * t;
                const uint8_t* krow1 = krow0 + 8 * rstride;
                for (int j = 0; j < row16; ++j) {
                    const uint32_t w0 = *reinterpret_cast<const uint32_t*>(krow0 + 16 * j);
                    const uint32_t w1 = *reinterpret_cast<const uint32_t*>(krow1 + 16 * j);
                    const uint32_t a0 = pack_bf16(byte_minus_128(w0, 0), byte_minus_128(w0, 1));
                    const uint32_t a2 = pack_bf16(byte_minus_128(w0, 2), byte_minus_128(w0, 3));
                    const uint32_t a1 = pack_bf16(byte_minus_128(w1, 0), byte_minus_128(w1, 1));
                    const uint32_t a3 = pack_bf16(byte_minus_128(w1, 2), byte_minus_128(w1, 3));
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        const int col = nb * 8 + g;  // (piece, head) column this lane feeds
                        uint32_t b0 = 0u, b1 = 0u;
                        if (col < kRowsUsed) {
                            const uint2 q4 = *reinterpret_cast<const uint2*>(&sm.qp[col][16 * j + 4 * t]);
                            b0 = q4.x; b1 = q4.y;
                        }
                        mma_bf16(c[nb], a0, a1, a2, a3, b0, b1);
                    }
                }
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    const int col = nb * 8 + 2 * t;
                    if (col < kRowsUsed) {
                        sm.sraw[col][16 * warp + g] = c[nb][0];
                        sm.sraw[col][16 * warp + g + 8] = c[nb][2];
                    }
                    if (col + 1 < kRowsUsed) {
                        sm.sraw[col + 1][16 * warp + g] = c[nb][1];
                        sm.sraw[col + 1][16 * warp + g + 8] = c[nb][3];
                    }
                }
            }
            __syncthreads();
            // (2) softmax weights of the tile, one (head, position) per thread and round; a warp covers
            //     32 positions of one head.  score = ((q.k_int) * k_scale) * 1/sqrt(hd)  (attention.rs:202)
            constexpr int kSoftItems = (G * kTilePos + kAttnThreads - 1) / kAttnThreads;
            float sv[kSoftItems];
#pragma unroll
            for (int e = 0; e < kSoftItems; ++e) {
                const int it = tid + e * kAttnThreads;
                const int h = it / kTilePos, r = it % kTilePos;
                float s = -INFINITY;
                // prefill: query vector h sits at position p + q0 + h / NREP and sees the keys up to there
                const bool seen = QB == 1 || tb + r <= p + q0 + h / NREP;
                if (h < G && r < n_here && seen) {
                    const float dot = __fadd_rn(__fadd_rn(sm.sraw[h][r], sm.sraw[G + h][r]), sm.sraw[2 * G + h][r]);
                    s = __fmul_rn(__fmul_rn(dot, sm.ksr[cur][r]), a.scaling);
                }
                sv[e] = s;
                const float wm = warp_max(s);
                if (lane == 0 && h < G) sm.wmax[h][(it >> 5) & 3] = wm;
            }
            __syncthreads();
#pragma unroll
            for (int e = 0; e < kSoftItems; ++e) {
                const int it = tid + e * kAttnThreads;
                const int h = it / kTilePos, r = it % kTilePos;
                if (h < G) {  // warp-uniform
                    const float m_old = sm.ml[0][h];
                    const float m_new = fmaxf(fmaxf(m_old, fmaxf(sm.wmax[h][0], sm.wmax[h][1])), fmaxf(sm.wmax[h][2], sm.wmax[h][3]));
                    const bool live = sv[e] != -INFINITY;  // inside the tile and visible to this query
                    const float pe = live ? expf(__fsub_rn(sv[e], m_new)) : 0.0f;
                    // weight of the value row: p * v_scale (the value bytes enter the MMA as integers)
                    const float wv = live ? __fmul_rn(pe, sm.vsr[cur][r]) : 0.0f;
                    split3(wv, sm.pw[h][r], sm.pw[G + h][r], sm.pw[2 * G + h][r]);
                    const float ws = warp_sum(pe);
                    if (lane == 0) sm.wsum[h][(it >> 5) & 3] = ws;
                    if (r == 0) sm.corr[h] = expf(__fsub_rn(m_old, m_new));  // exp(-inf) = 0 on the first tile
                }
            }
            __syncthreads();
            if (tid < G) {  // running sum and maximum (nobody reads them before the next barrier)
                const float m_old = sm.ml[0][tid];
                const float m_new = fmaxf(fmaxf(m_old, fmaxf(sm.wmax[tid][0], sm.wmax[tid][1])), fmaxf(sm.wmax[tid][2], sm.wmax[tid][3]));
                const float psum = __fadd_rn(__fadd_rn(__fadd_rn(sm.wsum[tid][0], sm.wsum[tid][1]), sm.wsum[tid][2]), sm.wsum[tid][3]);
                sm.ml[1][tid] = fmaf(sm.ml[1][tid], sm.corr[tid], psum);
                sm.ml[0][tid] = m_new;
            }
            // (3) O[(piece, head) x 32 dims] = O * corr + W[(piece, head) x positions] . V[positions x dims]
            if (pv_active) {
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) {
                    const int r0 = mb * 16 + g, r1 = r0 + 8;
                    const float c0 = r0 < kRowsUsed ? sm.corr[r0 % G] : 0.0f;
                    const float c1 = r1 < kRowsUsed ? sm.corr[r1 % G] : 0.0f;
#pragma unroll
                    for (int e = 0; e < 4; ++e) { acc[mb][e][0] *= c0; acc[mb][e][1] *= c0; acc[mb][e][2] *= c1; acc[mb][e][3] *= c1; }
                }
                const uint8_t* vcol = vraw + 32 * dg + 4 * g;
                for (int i = pq; 16 * i < n_here; i += n_pq) {
                    const int pos0 = 16 * i + 2 * t;  // this lane's positions of the step: pos0, +1, +8, +9
                    const uint32_t v0 = *reinterpret_cast<const uint32_t*>(vcol + (pos0) * rstride);
                    const uint32_t v1 = *reinterpret_cast<const uint32_t*>(vcol + (pos0 + 1) * rstride);
                    const uint32_t v8 = *reinterpret_cast<const uint32_t*>(vcol + (pos0 + 8) * rstride);
                    const uint32_t v9 = *reinterpret_cast<const uint32_t*>(vcol + (pos0 + 9) * rstride);
                    uint32_t pa[MB][4];
#pragma unroll
                    for (int mb = 0; mb < MB; ++mb) {
                        const int r0 = mb * 16 + g, r1 = r0 + 8;
                        pa[mb][0] = *reinterpret_cast<const uint32_t*>(&sm.pw[r0][pos0]);
                        pa[mb][1] = *reinterpret_cast<const uint32_t*>(&sm.pw[r1][pos0]);
                        pa[mb][2] = *reinterpret_cast<const uint32_t*>(&sm.pw[r0][pos0 + 8]);
                        pa[mb][3] = *reinterpret_cast<const uint32_t*>(&sm.pw[r1][pos0 + 8]);
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const uint32_t b0 = pack_bf16(byte_minus_128(v0, e), byte_minus_128(v1, e));
                        const uint32_t b1 = pack_bf16(byte_minus_128(v8, e), byte_minus_128(v9, e));
#pragma unroll
                        for (int mb = 0; mb < MB; ++mb) mma_bf16(acc[mb][e], pa[mb][0], pa[mb][1], pa[mb][2], pa[mb][3], b0, b1);
                    }
                }
            }
            if (tb + kTilePos < t1) cp_async_wait_all();
            __syncthreads();  // next tile complete and visible; this tile's buffers free again
            cur ^= 1;
        }
        // add the position groups and the three pieces through shared memory (the value tiles are free now)
        float* red = reinterpret_cast<float*>(sm.kraw);  // [n_pq][rows][hd], over the key and value tiles
        static_assert(sizeof(sm.kraw) + sizeof(sm.vraw) >= (size_t)kRowsUsed * 256 * sizeof(float) &&
                      offsetof(Smem, vraw) == offsetof(Smem, kraw) + sizeof(sm.kraw), "reduction scratch");
        if (pv_active) {
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
                const int r0 = mb * 16 + g, r1 = r0 + 8;
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    // MMA e, column n = dim 32 dg + 4 n + e; this lane holds n = 2t and 2t + 1
                    const int d0 = 32 * dg + 4 * (2 * t) + e, d1 = d0 + 4;
                    if (r0 < kRowsUsed) { red[(pq * kRowsUsed + r0) * hd + d0] = acc[mb][e][0]; red[(pq * kRowsUsed + r0) * hd + d1] = acc[mb][e][1]; }
                    if (r1 < kRowsUsed) { red[(pq * kRowsUsed + r1) * hd + d0] = acc[mb][e][2]; red[(pq * kRowsUsed + r1) * hd + d1] = acc[mb][e][3]; }
                }
            }
        }
        __syncthreads();
        for (int it = tid; it < G * hd; it += kAttnThreads) {
            const int h = it / hd, dcol = it % hd;
            float v = 0.0f;
            for (int g2 = 0; g2 < n_pq; ++g2) {
                const float* rr = red + (size_t)g2 * kRowsUsed * hd + dcol;
                v = __fadd_rn(v, __fadd_rn(__fadd_rn(rr[h * hd], rr[(G + h) * hd]), rr[(2 * G + h) * hd]));
            }
            sm.opart[it] = v;
        }
    }
    // only now may the next kernel's CTAs move in: earlier they would take the registers and
    // shared memory that this kernel's later CTAs are waiting for
    ptx::pdl_launch_dependents();

    // Merge of the spans of this (sequence, KV head): out = sum_s e^{m_s - m} o_s / sum_s e^{m_s - m} l_s.
    // Every CTA of the cluster finishes the output columns rank, rank + S, ... from the partials of all spans.
    cluster_sync_all();  // partials of every span written and visible cluster-wide
    {
        // The output columns are dealt evenly to the CTAs of the cluster.  All remote loads of a thread are
        // issued before the first use (fixed trip counts, predicated), so that their latencies overlap.
        const int S = a.splits, rank = (int)cluster_ctarank();
        const int total = G * hd;
        const int per_cta = (total + S - 1) / S;
        float amax = 0.0f;
        for (int i = tid; i < per_cta; i += kAttnThreads) {
            const int it = rank * per_cta + i;
            if (it >= total) break;
            const int h = it / hd;
            float ms[kMaxCluster], ls[kMaxCluster], os[kMaxCluster];
#pragma unroll
            for (int s2 = 0; s2 < kMaxCluster; ++s2) {
                ms[s2] = -INFINITY; ls[s2] = 0.0f; os[s2] = 0.0f;
                if (s2 < S) {
                    ms[s2] = ld_cluster_f32(&sm.ml[0][h], (uint32_t)s2);
                    ls[s2] = ld_cluster_f32(&sm.ml[1][h], (uint32_t)s2);
                    os[s2] = ld_cluster_f32(&sm.opart[it], (uint32_t)s2);
                }
            }
            float m = -INFINITY;
#pragma unroll
            for (int s2 = 0; s2 < kMaxCluster; ++s2) m = fmaxf(m, ms[s2]);
            float num = 0.0f, den = 0.0f;
#pragma unroll
            for (int s2 = 0; s2 < kMaxCluster; ++s2) {
                // a span without positions (maximum -inf) weighs nothing; what its output cells hold is undefined
                const bool live = ms[s2] != -INFINITY;
                const float w = live ? expf(__fsub_rn(ms[s2], m)) : 0.0f;
                den = fmaf(ls[s2], w, den);
                num = fmaf(live ? os[s2] : 0.0f, w, num);
            }
            const float o = __fdiv_rn(num, den);
            const int qi = q0 + h / NREP;  // new token of the sequence this query vector belongs to (decode: 0)
            if (qi < a.q_rows) a.out[(((int64_t)b * a.q_rows + qi) * a.n_heads + kvh * NREP + h % NREP) * hd + (it % hd)] = o;
            amax = fmaxf(amax, fabsf(o));
        }
        if (a.absmax_out) {
            amax = warp_max(amax);
            if (lane == 0 && amax > 0.0f) atomicMax(a.absmax_out + b, __float_as_uint(amax));
        }
    }
    cluster_sync_all();  // nobody leaves while a peer may still read its shared memory
}

// Standalone QuantizedKVCache::append (layers/kv_cache.rs:50-92) for one new token per sequence:
// one warp per (sequence, KV head, k|v) row; k and v arrive already rotated, as the reference's
// caller passes them (layers/attention.rs:180-196).
__global__ void __launch_bounds__(128) kv_append_kernel(KvCacheView cache, const float* __restrict__ k,
                                                        const float* __restrict__ v, const int32_t* __restrict__ pos,
                                                        int batch, int n_kv, int hd) {
    __shared__ float rowbuf[4][kMaxHd];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + warp;  // (b, kvh, which)
    if (row >= batch * n_kv * 2) return;
    const int which = row & 1, kvh = (row >> 1) % n_kv, b = (row >> 1) / n_kv;
    const int p = pos[b];
    if (p < 0 || p >= cache.max_seq) return;
    const float* src = (which ? v : k) + ((int64_t)b * n_kv + kvh) * hd;
    for (int c = lane; c < hd; c += 32) rowbuf[warp][c] = src[c];
    __syncwarp();
    const int64_t r = ((int64_t)b * n_kv + kvh) * cache.max_seq + p;
    quant_row_warp(rowbuf[warp], hd, (which ? cache.v_q : cache.k_q) + r * hd, (which ? cache.v_s : cache.k_s) + r, nullptr,
                   nullptr, lane);
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

// K/V rows of a prefill: for every new token i of every sequence, RoPE on the key at position pos[b] + i
// (layers/attention.rs:180-182) and Q8 append of key and value (layers/kv_cache.rs:50-119) into row
// pos[b] + i of the cache.  One warp per (sequence, token, KV head, k|v); qkv rows are [b][i].
__global__ void __launch_bounds__(128) kv_append_rows_kernel(KvCacheView cache, const float* __restrict__ qkv,
                                                             const int32_t* __restrict__ pos,
                                                             const float* __restrict__ rope_cos,
                                                             const float* __restrict__ rope_sin, int batch, int q_rows,
                                                             int n_heads, int n_kv, int hd) {
    __shared__ float rowbuf[4][kMaxHd];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t item = (int64_t)blockIdx.x * 4 + warp;  // ((b * q_rows + i) * n_kv + kvh) * 2 + which
    if (item >= (int64_t)batch * q_rows * n_kv * 2) return;
    const int which = (int)(item & 1), kvh = (int)((item >> 1) % n_kv);
    const int64_t row = (item >> 1) / n_kv;  // b * q_rows + i
    const int b = (int)(row / q_rows), i = (int)(row % q_rows);
    const int p = pos[b] + i;
    if (p < 0 || p >= cache.max_seq) return;
    const int half = hd >> 1;
    const float* src = qkv + row * (int64_t)(n_heads + 2 * n_kv) * hd + (int64_t)(n_heads + (which ? n_kv : 0) + kvh) * hd;
    if (which) {
        for (int c = lane; c < hd; c += 32) rowbuf[warp][c] = src[c];
    } else {
        for (int c = lane; c < half; c += 32) {
            const float cs = rope_cos[(int64_t)p * half + c], sn = rope_sin[(int64_t)p * half + c];
            const float x1 = src[c], x2 = src[half + c];
            rowbuf[warp][c] = __fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn));
            rowbuf[warp][half + c] = __fadd_rn(__fmul_rn(x1, sn), __fmul_rn(x2, cs));
        }
    }
    __syncwarp();
    const int64_t r = ((int64_t)b * n_kv + kvh) * cache.max_seq + p;
    quant_row_warp(rowbuf[warp], hd, (which ? cache.v_q : cache.k_q) + r * hd, (which ? cache.v_s : cache.k_s) + r, nullptr,
                   nullptr, lane);
}

constexpr size_t kHalfSm = 116 * 1024;
static_assert(sizeof(AttnSmemT<kMaxRep>) <= 110 * 1024, "two CTAs of the decode kernel must fit one SM");
constexpr int kPrefillVectors = 16;  // query vectors per CTA of the prefill kernel: 16 / NREP positions x NREP heads

// How many clusters of each size can be resident at once (a CTA then takes a whole SM): a cluster's CTAs
// must sit in one GPC, so large clusters leave SMs unused, and a GPC with fewer SMs than the cluster
// has CTAs holds none.  Filled once per kernel instance from cudaOccupancyMaxActiveClusters.
struct ClusterTable {
    bool ready = false;
    int active[kMaxCluster + 1] = {0};  // active[s] = resident clusters of s CTAs (0: size unusable)
};

template <int NREP>
cudaError_t configure_rep(const ClusterTable** out) {
    static ClusterTable table;  // per process; every device of a process is the same GPU model
    if (!table.ready) {
        cudaError_t e = cudaFuncSetAttribute(attn_kernel<NREP, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kHalfSm);
        if (e != cudaSuccess) return e;
        e = cudaFuncSetAttribute(attn_kernel<NREP, kPrefillVectors / NREP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)sizeof(AttnSmemT<kPrefillVectors>));
        if (e != cudaSuccess) return e;
        const bool big = cudaFuncSetAttribute(attn_kernel<NREP, 1>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
        for (int s = 1; s <= kMaxCluster; ++s) {
            if (s > 8 && !big) break;
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(1, s, 1);
            cfg.blockDim = dim3(kAttnThreads);
            cfg.dynamicSmemBytes = kHalfSm;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.y = (unsigned)s; attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, attn_kernel<NREP, 1>, &cfg) == cudaSuccess) table.active[s] = n;
        }
        cudaGetLastError();  // a refused attribute or query only rules a cluster size out
        if (table.active[1] < 1) table.active[1] = 1;
        table.ready = true;
    }
    *out = &table;
    return cudaSuccess;
}

template <int NREP>
cudaError_t launch_attn_rep(const AttnArgs& a, cudaStream_t stream) {
    const ClusterTable* table = nullptr;
    cudaError_t e = configure_rep<NREP>(&table);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kAttnThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    if (a.q_rows > 1) {
        // prefill: one CTA per block of query positions, no cluster, ordinary stream order
        constexpr int QB = kPrefillVectors / NREP;
        if (a.splits != 1) return cudaErrorInvalidValue;
        cfg.gridDim = dim3(a.batch * a.n_kv, (a.q_rows + QB - 1) / QB);
        cfg.dynamicSmemBytes = sizeof(AttnSmemT<kPrefillVectors>);
        attr[0].val.clusterDim.y = 1;
        cfg.numAttrs = 1;
        return cudaLaunchKernelEx(&cfg, attn_kernel<NREP, QB>, a);
    }
    if (a.splits < 1 || a.splits > kMaxCluster || table->active[a.splits] < 1) return cudaErrorInvalidValue;
    cfg.gridDim = dim3(a.batch * a.n_kv, a.splits);
    // When the whole grid fits one CTA per SM, ask for more than half of an SM's shared
    // memory: the block scheduler then cannot pair two CTAs on one SM while others idle.
    cfg.dynamicSmemBytes = ((int64_t)a.batch * a.n_kv * a.splits <= a.sm_count) ? kHalfSm : sizeof(AttnSmemT<NREP>);
    attr[0].val.clusterDim.y = (unsigned)a.splits;
    cfg.numAttrs = a.pdl ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, attn_kernel<NREP, 1>, a);
}

const ClusterTable* attn_cluster_table(int rep) {
    const ClusterTable* t = nullptr;
    cudaError_t e = cudaErrorInvalidValue;
    switch (rep) {
        case 1: e = configure_rep<1>(&t); break;
        case 2: e = configure_rep<2>(&t); break;
        case 4: e = configure_rep<4>(&t); break;
        case 8: e = configure_rep<8>(&t); break;
        default: break;
    }
    return e == cudaSuccess ? t : nullptr;
}

}  // namespace

// Cuts the positions of a sequence into spans, one CTA each; the spans of a (sequence, KV head) pair
// form one thread-block cluster.  Fewer pairs than SMs: the largest cluster size, up to SMs / pairs, of
// which as many clusters as there are pairs can be resident at once (one wave, a CTA per SM).  More
// pairs than SMs: two CTAs share an SM and the CTAs run in waves; cutting the positions in 2..4 can fill
// the last wave better (cost model = waves x (tiles of 128 positions per CTA + 1 for the fixed work of a CTA)).
void attn_plan(int64_t batch, int64_t n_kv, int64_t max_seq, int sm_count, int rep, int* splits, int* span) {
    const int64_t pairs = batch * n_kv;
    const ClusterTable* table = attn_cluster_table(rep);
    int64_t want = 1;
    if (pairs >= sm_count) {
        int64_t best_cost = -1;
        for (int64_t s = 1; s <= 4; ++s) {
            if (table && table->active[s] < 1) continue;
            const int64_t sp = ((max_seq + s - 1) / s + 31) / 32 * 32;
            const int64_t waves = (pairs * s + 2 * sm_count - 1) / (2 * sm_count);
            const int64_t cost = waves * ((sp + kTilePos - 1) / kTilePos + 1);
            if (best_cost < 0 || cost < best_cost) { best_cost = cost; want = s; }
        }
    } else {
        const int64_t cap = (int64_t)sm_count / pairs < kMaxCluster ? (int64_t)sm_count / pairs : kMaxCluster;
        for (int64_t s = cap; s >= 1; --s) {
            const int act = table ? table->active[s] : (s <= 8 ? sm_count / (int)s : 0);
            if (act >= pairs) { want = s; break; }
        }
    }
    const int64_t sp = ((max_seq + want - 1) / want + 31) / 32 * 32;
    *span = (int)sp;  // upper bound: the kernel cuts the current length, not max_seq, into `splits` spans
    *splits = (int)want;
}

cudaError_t launch_attn_decode(const AttnArgs& a, cudaStream_t stream) {
    const int rep = a.n_kv > 0 ? a.n_heads / a.n_kv : 0;
    if (a.head_dim % 32 != 0 || a.head_dim > kMaxHd || a.n_heads % a.n_kv != 0 || rep < 1 || rep > kMaxRep ||
        a.span % 32 != 0 || (int64_t)a.span * a.splits < a.cache.max_seq || a.q_rows < 1)
        return cudaErrorInvalidValue;
    switch (rep) {
        case 1: return launch_attn_rep<1>(a, stream);
        case 2: return launch_attn_rep<2>(a, stream);
        case 4: return launch_attn_rep<4>(a, stream);
        case 8: return launch_attn_rep<8>(a, stream);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_kv_append(const KvCacheView& cache, const float* k, const float* v, const int32_t* pos, int batch,
                             int n_kv, int hd, cudaStream_t stream) {
    const int rows = batch * n_kv * 2;
    kv_append_kernel<<<(rows + 3) / 4, 128, 0, stream>>>(cache, k, v, pos, batch, n_kv, hd);
    return cudaGetLastError();
}

cudaError_t launch_kv_append_rows(const KvCacheView& cache, const float* qkv, const int32_t* pos, const float* rope_cos,
                                  const float* rope_sin, int batch, int q_rows, int n_heads, int n_kv, int hd,
                                  cudaStream_t stream) {
    const int64_t items = (int64_t)batch * q_rows * n_kv * 2;
    kv_append_rows_kernel<<<(unsigned)((items + 3) / 4), 128, 0, stream>>>(cache, qkv, pos, rope_cos, rope_sin, batch, q_rows,
                                                                            n_heads, n_kv, hd);
    return cudaGetLastError();
}

cudaError_t launch_rope_tables(const float* inv_freq, int max_seq, int half, float* cos_t, float* sin_t,
                               cudaStream_t stream) {
    rope_table_kernel<<<148, 256, 0, stream>>>(inv_freq, max_seq, half, cos_t, sin_t);
    return cudaGetLastError();
}

}  // namespace bt
