// Fused decode attention over the Q8 KV cache: RoPE (layers/attention.rs:45-84) on the new
// q and k, Q8 append of k and v (layers/kv_cache.rs:95-119), scores = (q.k)/sqrt(hd) over
// positions 0..pos, softmax, .V (layers/attention.rs:198-217), all heads of a KV group in
// one CTA so the cache is read once (the reference materialises repeat_kv copies,
// layers/attention.rs:228-239).  The cache is read in place as u8; nothing is
// re-materialised in f32 (the reference dequantises the whole cache every step,
// layers/kv_cache.rs:84-92).  HBM-bound on the cache bytes: 2*n_kv*T*(hd+4) per sequence.
//
// Arithmetic.  Both contractions are INTEGER products on the tensor cores
// (mma.sync.m16n8k32, 8-bit operands, int32 accumulators), so the cache bytes enter the MMA as
// they lie in memory, without any conversion:
//   * a cache byte b (unsigned) stands for b - 128; the "- 128" is taken out afterwards with the
//     sum of the other operand (for the scores a constant per query, for P.V a column of ones
//     that rides in the same MMAs);
//   * an f32 factor is turned into fixed point relative to a power-of-two bound and cut into
//     four 8-bit digits, which ride as extra columns (scores) or rows (P.V) of the same MMA:
//     a rotated query value q = S * Q / 2^27 with S = the power of two >= max|q| of its vector and
//     |Q| <= 2^27 (four signed 7-bit digits); a weight p * v_scale = B * U / 2^32 with B = the power
//     of two above the largest value-row scale of the chunk and U < 2^32 (four unsigned bytes).
// Every digit product is an exact integer.  The four digit sums of a score are joined in f32 (three
// roundings, no cancellation: each digit weighs 1/128 of the one before), those of an output value in a
// 64-bit integer that is rounded to f32 once.  A query is exact to 2^-28 of its vector's largest
// component, a weight to 2^-33 of the chunk's bound.  Softmax runs in f32.  The result is within about
// 1e-6 relative of the f32 value of layers/attention.rs:202-217.
//
// Order of work.  The positions of a CTA are taken in chunks of up to kChunk positions.  Phase A of a
// chunk streams its KEY tiles (128 positions each) and leaves the f32 scores in shared memory; the
// chunk's maximum then fixes the softmax reference and the weight bound; phase B streams the VALUE
// tiles, turns the scores into weight digits tile by tile and accumulates P.V in int32 over the whole
// chunk.  Only at the end of a chunk do the accumulators become f32 and meet the running output
// (rescaled by exp(m_old - m_new) as usual).  Key and value tiles flow through one ring of three
// buffers, fetched two tiles ahead with cp.async.
//
// Work split.  One CTA = one (sequence, KV head, span of positions); the spans of one
// (sequence, KV head) form a thread-block cluster, and the partial results (running maximum,
// denominator, unnormalised output) are merged through distributed shared memory: after a
// cluster barrier every CTA of the cluster finishes a slice of the output columns, reading the
// partials of all spans with ld.shared::cluster.  No global scratch, no second launch.
#include <stddef.h>

#include <mutex>
#include <type_traits>

#include "bt_model.cuh"
#include "bt_ptx.cuh"

namespace bt {

namespace {

constexpr int kAttnWarps = 8;
constexpr int kAttnThreads = kAttnWarps * 32;
constexpr int kTilePos = 128;   // cache rows per tile
constexpr int kMaxRep = 8;      // query heads per KV head
constexpr int kMaxHd = 128;
constexpr int kRowPad = 32;     // bytes added to a cache row in shared memory: row stride = 32 mod 128, so the 8-byte
                                // fragment loads of 4 consecutive rows and the 4-byte loads of rows r, r+1, r+2, r+3
                                // fall into different banks
constexpr int kMaxRowBytes = kMaxHd + kRowPad;
constexpr int kStages = 3;      // tile buffers of the ring
constexpr int kWStride = kTilePos + 16;  // bytes per row of the weight digits
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
__device__ __forceinline__ long long shfl_xor_ll(long long v, int mask) {
    const int lo = __shfl_xor_sync(0xffffffffu, (int)(v & 0xffffffffll), mask);
    const int hi = __shfl_xor_sync(0xffffffffu, (int)(v >> 32), mask);
    return ((long long)hi << 32) | (unsigned int)lo;
}

// Quantise one head vector held in shared memory (hd values) by one warp:
// s = max|x| / 127, q = u8(round(x / s) + 128)  (quantize_q8, layers/kv_cache.rs:95-119; an all-zero
// row gives s = 0, q = 128).  q_copy: optional second destination (a prefetched copy of the row).
__device__ __forceinline__ void quant_row_warp(const float* v, int hd, uint8_t* q_out, float* s_out, uint8_t* q_copy,
                                               int lane) {
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
    if (lane == 0) *s_out = s;
}

// G = query vectors that share the K/V rows of a CTA: the NREP heads of a KV group (decode) times the
// QB query positions of a block (prefill).  Score column / weight row 4 v + j = digit j of query vector v.
template <int G>
struct AttnSmemT {
    static constexpr int kChunk = G <= 4 ? 1024 : 512;     // positions whose scores are held at once
    static constexpr int kCols = 4 * G;
    static constexpr int kCols8 = (kCols + 7) / 8 * 8;
    static constexpr int kRows16 = (kCols + 15) / 16 * 16;
    alignas(16) uint8_t ring[kStages][kTilePos * kMaxRowBytes];  // key / value tiles as stored (u8), rows padded
    alignas(16) float sbuf[G][kChunk];                      // scores of the chunk (before the chunk: the rotated queries)
    alignas(16) float sc[kStages][kTilePos];                // row scales that came with a key tile
    alignas(16) float vsc[kChunk];                          // value-row scales of the chunk
    alignas(16) int8_t qdig[kCols8][kMaxRowBytes];          // query digits, [column][dim]
    alignas(16) uint8_t wdig[2][kRows16][kWStride];         // weight digits of a tile, [row][position slot], two tiles
    alignas(16) float opart[G * kMaxHd];                    // this span's unnormalised output [query vector][dim] (read by the cluster)
    alignas(16) float part[2 * G * kMaxHd];                 // a chunk's P.V result per position group, [group][vector][dim], before it meets opart
    int dcorr[kCols8];                                      // 128 * sum_d digit[column][d]: the "- 128" of the key bytes
    float qscale[G];                                        // S / 2^27 of a query vector
    float ml[2][G];                                         // this span's running maximum / denominator (read by the cluster)
    float corr[G];
    float wmax[kAttnWarps][G];
    float wsum[kAttnWarps][(G + 7) / 8];
    float wvmax[kAttnWarps];
    float wup, wdown;                                       // weight scale of the chunk: 2^32 / B and B / 2^32
    float knew[kMaxHd], vnew[kMaxHd];
    // Merge of a cluster's spans: every span pushes its partial output columns (and its maximum / denominator) into
    // the CTA that finishes those columns, [span][column of the receiver] and [span][max | denominator][vector].
    // Written by peers only, between the start of the kernel and the cluster barrier; never initialised.
    static constexpr int kRx = G <= 8 ? G * kMaxHd + 16 : 4;  // (more than 8 vectors: prefill, which has no cluster)
    alignas(16) float rx_o[kRx];
    float rx_ml[G <= 8 ? 16 : 1][2][G];
};

// D(16x8, s32) += A(16x32, u8, row) * B(32x8, s8 or u8, col)
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_u8u8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ptx::smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst_smem, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(ptx::smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// all but the newest `N` groups of this thread are complete
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// bytes e of the words v0..v3 as one word (v0.e, v1.e, v2.e, v3.e), e = 0..3: a 4 x 4 byte transpose
__device__ __forceinline__ void transpose4(uint32_t v0, uint32_t v1, uint32_t v2, uint32_t v3, uint32_t (&r)[4]) {
    const uint32_t lo01 = __byte_perm(v0, v1, 0x5140), hi01 = __byte_perm(v0, v1, 0x7362);
    const uint32_t lo23 = __byte_perm(v2, v3, 0x5140), hi23 = __byte_perm(v2, v3, 0x7362);
    r[0] = __byte_perm(lo01, lo23, 0x5410);
    r[1] = __byte_perm(lo01, lo23, 0x7632);
    r[2] = __byte_perm(hi01, hi23, 0x5410);
    r[3] = __byte_perm(hi01, hi23, 0x7632);
}

// f32 to the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ void st_cluster_f32(float* local, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(ptx::smem_u32(local)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
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
// HD: head_dim fixed at compile time (128, 64), or 0 = any multiple of 32 up to 128 read from the arguments.
template <int NREP, int QB, int HD>
__global__ void __launch_bounds__(kAttnThreads, (NREP * QB <= 4) ? 2 : 1) attn_kernel(AttnArgs a) {
    constexpr int G = NREP * QB;
    using Smem = AttnSmemT<G>;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>(smem_raw);
    constexpr int kChunk = Smem::kChunk;
    constexpr int NB = Smem::kCols8 / 8;           // 8-column blocks of the score MMAs (two query vectors each)
    constexpr int MB = Smem::kRows16 / 16;         // 16-row blocks of the P.V MMAs (four query vectors each)
    constexpr int kRounds = (G + kAttnWarps - 1) / kAttnWarps;  // weight rounds per tile: a warp turns one query vector's 128 scores into digits
    constexpr bool kSplitDigits = 2 * G <= kAttnWarps;          // few vectors: two warps share one
    const int hd = HD > 0 ? HD : a.head_dim, half = hd >> 1;
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
    const int row16 = hd >> 4;                            // 16-byte pieces per row
    const int l16 = hd == 128 ? 3 : (hd == 64 ? 2 : (hd == 32 ? 1 : -1));  // their log2 when a power of two
    const int rstride = hd + kRowPad;                    // row stride of the tiles in shared memory

    // The tiles of this CTA in the order they are worked on: per chunk its key tiles, then its value tiles.
    // `Cursor` names one of them; the fetches run two tiles ahead of the work.
    struct Cursor { int chunk0; int phase; int tile; int tiles; };  // first position of the chunk, 0 = keys / 1 = values, tile in chunk, tiles of the chunk
    auto chunk_tiles = [&](int chunk0) { return (min(kChunk, t1 - chunk0) + kTilePos - 1) / kTilePos; };
    auto advance = [&](Cursor& c) {
        if (++c.tile >= c.tiles) {
            c.tile = 0;
            if (++c.phase == 2) { c.phase = 0; c.chunk0 += kChunk; c.tiles = chunk_tiles(c.chunk0); }
        }
    };
    // rows of the tile `c` -> ring buffer `stage` (asynchronous copies); a key tile brings its row scales along
    auto fetch = [&](const Cursor& c, int stage) {
        if (c.chunk0 < t1) {
            const int r0 = c.chunk0 + c.tile * kTilePos;
            const int n = min(kTilePos, t1 - r0);
            const uint8_t* src = (c.phase ? a.cache.v_q : a.cache.k_q) + (row_base + r0) * hd;
            uint8_t* dst = sm.ring[stage];
            if constexpr (HD > 0) {
                // thread -> (row tid / P16 + k RP, 16-byte piece tid % P16): all offsets are compile-time constants
                constexpr int P16 = HD / 16, RP = kAttnThreads / P16, NP = kTilePos / RP;
                const int rr = tid / P16;
                const uint8_t* s0 = src + 16 * tid;
                uint8_t* d0 = dst + rr * (HD + kRowPad) + (tid % P16) * 16;
#pragma unroll
                for (int k = 0; k < NP; ++k)
                    if (rr + k * RP < n) cp_async16(d0 + k * RP * (HD + kRowPad), s0 + k * RP * HD);
            } else if (l16 >= 0) {
                for (int i = tid; i < (n << l16); i += kAttnThreads)
                    cp_async16(dst + (i >> l16) * rstride + ((i & ((1 << l16) - 1)) << 4), src + 16 * i);
            } else {
                for (int i = tid; i < n * row16; i += kAttnThreads)
                    cp_async16(dst + (i / row16) * rstride + (i % row16) * 16, src + 16 * i);
            }
            if (c.phase == 0 && tid < n) cp_async4(&sm.sc[stage][tid], a.cache.k_s + row_base + r0 + tid);
        }
        cp_async_commit();  // one group per tile, also when there is nothing left to fetch
    };

    Cursor fc = {t0, 0, 0, chunk_tiles(t0)};
    const bool empty = t0 >= t_len;
    // The cache rows of earlier positions were written by earlier steps, so the first tile can be requested
    // before the dependency wait; the row of the current position is fetched too, with whatever it holds, and its
    // owner overwrites the copy below.
    if (QB == 1 && !empty) {
        fetch(fc, 0);
        advance(fc);
    }
    // weight rows and query columns beyond the ones in use stay zero
    for (int i = tid; i < (int)(sizeof(sm.wdig) / 4); i += kAttnThreads) reinterpret_cast<uint32_t*>(sm.wdig)[i] = 0u;
    for (int i = tid; i < (int)(sizeof(sm.qdig) / 4); i += kAttnThreads) reinterpret_cast<uint32_t*>(sm.qdig)[i] = 0u;
    if (tid < Smem::kCols8) sm.dcorr[tid] = 0;
    for (int i = tid; i < G * kMaxHd; i += kAttnThreads) sm.opart[i] = 0.0f;
    ptx::pdl_wait();
    if (QB > 1 && !empty) {  // prefill: the new rows come from the kernel just before
        fetch(fc, 0);
        advance(fc);
    }

    const int64_t qkv_stride = (int64_t)(a.n_heads + 2 * a.n_kv) * hd;
    const float* qkv = a.qkv + (int64_t)b * a.q_rows * qkv_stride;  // first new token of the sequence
    const bool owner = QB == 1 && (p >= t0 && p < t1);
    if (!empty) {
        const float* cos_p = a.rope_cos + (int64_t)p * half;
        const float* sin_p = a.rope_sin + (int64_t)p * half;
        // rotate the query vectors of this CTA, [x1*cos - x2*sin, x1*sin + x2*cos] (attention.rs:79-83), into the
        // score buffer (free until the first chunk).  Query vector v = (position q0 + v / NREP, head v % NREP); a
        // block that reaches beyond the last new token repeats the last one (never stored).
        for (int i = tid; i < G * half; i += kAttnThreads) {
            const int v = i / half, c = i % half;
            const int h = v % NREP, qi = min(q0 + v / NREP, a.q_rows - 1);
            const float cs = a.rope_cos[(int64_t)(p + qi) * half + c], sn = a.rope_sin[(int64_t)(p + qi) * half + c];
            const float* qh = qkv + (int64_t)qi * qkv_stride + (int64_t)(kvh * NREP + h) * hd;
            const float x1 = qh[c], x2 = qh[half + c];
            sm.sbuf[v][c] = __fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn));
            sm.sbuf[v][half + c] = __fadd_rn(__fmul_rn(x1, sn), __fmul_rn(x2, cs));
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
    cp_async_wait<0>();
    __syncthreads();  // first tile landed; rotated q / k / v visible
    if (!empty) {
        // Query digits, one warp per vector in turn: S = power of two >= max|q|, Q = round(q / S * 2^27),
        // Q = ((d0 * 128 + d1) * 128 + d2) * 128 + d3 with digits in [-64, 64].
        for (int v = warp; v < G; v += kAttnWarps) {
            float amax = 0.0f;
            for (int c = lane; c < hd; c += 32) amax = fmaxf(amax, fabsf(sm.sbuf[v][c]));
            amax = warp_max(amax);
            int ex = 0;
            if (amax > 0.0f) (void)frexpf(amax, &ex);   // amax = m * 2^ex, m in [0.5, 1)
            const float up = ldexpf(1.0f, 27 - ex);
            int dsum[4] = {0, 0, 0, 0};
            for (int c = lane; c < hd; c += 32) {
                int Q = __float2int_rn(__fmul_rn(sm.sbuf[v][c], up));
                const int d3 = ((Q + 64) & 127) - 64; Q = (Q - d3) >> 7;
                const int d2 = ((Q + 64) & 127) - 64; Q = (Q - d2) >> 7;
                const int d1 = ((Q + 64) & 127) - 64; Q = (Q - d1) >> 7;
                sm.qdig[4 * v + 0][c] = (int8_t)Q;
                sm.qdig[4 * v + 1][c] = (int8_t)d1;
                sm.qdig[4 * v + 2][c] = (int8_t)d2;
                sm.qdig[4 * v + 3][c] = (int8_t)d3;
                dsum[0] += Q; dsum[1] += d1; dsum[2] += d2; dsum[3] += d3;
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) dsum[j] += __shfl_xor_sync(0xffffffffu, dsum[j], o);
                if (lane == 0) sm.dcorr[4 * v + j] = 128 * dsum[j];
            }
            if (lane == 0) sm.qscale[v] = ldexpf(1.0f, ex - 27);
        }
    }
    if (owner) {
        const bool in_first = p - t0 < kTilePos;
        if (warp == 6) quant_row_warp(sm.knew, hd, a.cache.k_q + (row_base + p) * hd, a.cache.k_s + row_base + p,
                                      in_first ? sm.ring[0] + (p - t0) * rstride : nullptr, lane);
        if (warp == 7) quant_row_warp(sm.vnew, hd, a.cache.v_q + (row_base + p) * hd, a.cache.v_s + row_base + p, nullptr, lane);
    }
    __syncthreads();  // the block's own global writes are visible to its later copies after the barrier
    if (owner && p - t0 < kTilePos && tid == 0) sm.sc[0][p - t0] = a.cache.k_s[row_base + p];  // the prefetched copy was stale
    if (!empty) {
        fetch(fc, 1);  // second tile
        advance(fc);
    }

    // P.V ownership: warp = (group of 32 dims dg, position group pq); the warp handles the 32-position steps
    // pq, pq + n_pq, ... of every tile for dims 32 dg .. 32 dg + 31.  Four 32-bit loads of V rows (dims
    // 32 dg + 4 g .. + 3 of four positions) are transposed into the B fragments of four MMAs, MMA e holding
    // dim 32 dg + 4 n + e in column n.
    const int n_dg = hd >> 5;
    const int n_pq = kAttnWarps / n_dg;
    const int dg = warp % n_dg, pq = warp / n_dg;
    int acc[MB][4][4], ones[MB][4];
    float psum[kRounds], mx[NB];
    int dc[NB][2];  // the "- 128" terms of this lane's two columns of every block
    float qs[NB];   // and the scale of the query vector they belong to

    if (!empty) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            dc[nb][0] = sm.dcorr[8 * nb + 2 * t];
            dc[nb][1] = sm.dcorr[8 * nb + 2 * t + 1];
            qs[nb] = 2 * nb + (t >> 1) < G ? sm.qscale[2 * nb + (t >> 1)] : 0.0f;
        }
        int cur = 0;  // ring buffer of the tile being worked on (tiles go through the buffers in turn)
        for (int chunk0 = t0; chunk0 < t1; chunk0 += kChunk) {
            const int clen = min(kChunk, t1 - chunk0);
            const int ctiles = (clen + kTilePos - 1) / kTilePos;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) mx[nb] = -INFINITY;
            // the chunk's value-row scales, needed between the phases: requested now, used then
            // (thread -> positions tid, tid + 256, ...; they go to shared memory in the slot order of the weights)
            float vs_reg[kChunk / kAttnThreads];
#pragma unroll
            for (int i = 0; i < kChunk / kAttnThreads; ++i)
                vs_reg[i] = tid + i * kAttnThreads < clen ? a.cache.v_s[row_base + chunk0 + tid + i * kAttnThreads] : 0.0f;
            // ---- phase A: scores of the chunk.  Warp w owns positions 16 w .. 16 w + 15 of a tile; per 32-dim
            //      step lane (g, t) supplies bytes 32 j + 8 t .. + 7 of rows g and g + 8 (the order of the dims
            //      inside a step is free as long as the query digits follow it). -------------------------------
            for (int ti = 0; ti < ctiles; ++ti, cur = cur + 1 == kStages ? 0 : cur + 1) {
                cp_async_wait<1>();
                __syncthreads();  // the tile landed and is visible; everybody is done with the tile before
                fetch(fc, cur >= 1 ? cur - 1 : kStages - 1);  // two tiles ahead = the buffer of the tile before (three buffers)
                advance(fc);
                const int n_here = min(kTilePos, clen - ti * kTilePos);
                // FULL: a whole tile that every query may see (decode; all but the last tile of a span)
                auto score_tile = [&](auto full_tag) {
                    constexpr bool FULL = decltype(full_tag)::value;
                    if (!FULL && 16 * warp >= n_here) return;
                    const uint8_t* kraw = sm.ring[cur];
                    int c[NB][4];
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) c[nb][0] = c[nb][1] = c[nb][2] = c[nb][3] = 0;
                    const uint8_t* krow0 = kraw + (16 * warp + g) * rstride + 8 * t;
                    const uint8_t* krow1 = krow0 + 8 * rstride;
#pragma unroll
                    for (int j = 0; j < kMaxHd / 32; ++j) {
                        if (32 * j < hd) {
                            const uint2 w0 = *reinterpret_cast<const uint2*>(krow0 + 32 * j);
                            const uint2 w1 = *reinterpret_cast<const uint2*>(krow1 + 32 * j);
#pragma unroll
                            for (int nb = 0; nb < NB; ++nb) {
                                const uint2 q8 = *reinterpret_cast<const uint2*>(&sm.qdig[nb * 8 + g][32 * j + 8 * t]);
                                mma_u8s8(c[nb], w0.x, w1.x, w0.y, w1.y, q8.x, q8.y);
                            }
                        }
                    }
                    // Lane t holds columns 2t, 2t + 1 of block nb: digits (0, 1) (t even) or (2, 3) (t odd) of query
                    // vector 2 nb + t / 2, for rows g and g + 8.  Each lane joins its two digits, the lane pair swaps
                    // halves: the even lane finishes row g, the odd lane row g + 8.  Scores go to shared memory in the
                    // slot order of the weights (position 16 q + 4 i + t' -> slot 16 q + 4 t' + i).
                    const bool odd = t & 1;
                    const int r = 16 * warp + g + (odd ? 8 : 0);
                    const int slot = ti * kTilePos + 16 * warp + 4 * (g & 3) + (g >> 2) + (odd ? 2 : 0);
                    const float ksr = (FULL || r < n_here) ? sm.sc[cur][r] : 0.0f;
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        const int v = 2 * nb + (t >> 1);
                        const float x_lo = fmaf((float)(c[nb][0] - dc[nb][0]), 128.0f, (float)(c[nb][1] - dc[nb][1]));  // row g
                        const float x_hi = fmaf((float)(c[nb][2] - dc[nb][0]), 128.0f, (float)(c[nb][3] - dc[nb][1]));  // row g + 8
                        const float got = __shfl_xor_sync(0xffffffffu, odd ? x_lo : x_hi, 1);
                        if (G % 2 == 0 || v < G) {
                            float s = -INFINITY;
                            // prefill: query vector v sits at position p + q0 + v / NREP and sees the keys up to there
                            const bool seen = FULL || (r < n_here && (QB == 1 || chunk0 + ti * kTilePos + r <= p + q0 + v / NREP));
                            if (seen) {
                                const float dot = __fmul_rn(odd ? fmaf(got, 16384.0f, x_hi) : fmaf(x_lo, 16384.0f, got), qs[nb]);
                                s = __fmul_rn(__fmul_rn(dot, ksr), a.scaling);  // (attention.rs:202)
                            }
                            sm.sbuf[v][slot] = s;
                            mx[nb] = fmaxf(mx[nb], s);
                        }
                    }
                };
                // (prefill: the last new token's position bounds what the block's first query may see)
                if (n_here == kTilePos && (QB == 1 || chunk0 + ti * kTilePos + kTilePos - 1 <= p + q0)) score_tile(std::true_type{});
                else score_tile(std::false_type{});
            }
            // ---- between the phases: the chunk's maximum per query vector, the bound of the weights ----
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                float m = mx[nb];
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 8));
                m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 16));
                if (g == 0 && (t & 1) == 0 && 2 * nb + (t >> 1) < G) sm.wmax[warp][2 * nb + (t >> 1)] = m;
            }
            {
                float vm = 0.0f;
#pragma unroll
                for (int i = 0; i < kChunk / kAttnThreads; ++i) {
                    const int r = tid + i * kAttnThreads;  // position in the chunk -> slot: bits 0-1 and 2-3 swapped
                    sm.vsc[(r & ~15) | ((r & 3) << 2) | ((r >> 2) & 3)] = vs_reg[i];
                    vm = fmaxf(vm, vs_reg[i]);
                }
                vm = warp_max(vm);
                if (lane == 0) sm.wvmax[warp] = vm;
            }
            __syncthreads();
            if (tid < G) {
                const float m_old = sm.ml[0][tid];
                float m_new = m_old;
#pragma unroll
                for (int w = 0; w < kAttnWarps; ++w) m_new = fmaxf(m_new, sm.wmax[w][tid]);
                // nothing visible so far (prefill blocks whose first chunk lies ahead never happen; kept for safety)
                sm.corr[tid] = m_new == -INFINITY ? 1.0f : expf(__fsub_rn(m_old, m_new));  // exp(-inf) = 0 on the first chunk
                sm.ml[0][tid] = m_new;
            }
            if (tid == 32) {
                float vm = 0.0f;
#pragma unroll
                for (int w = 0; w < kAttnWarps; ++w) vm = fmaxf(vm, sm.wvmax[w]);
                int ex = 0;
                if (vm > 0.0f) (void)frexpf(vm, &ex);  // every weight p * v_scale <= vm < 2^ex
                sm.wup = ldexpf(1.0f, 32 - ex);
                sm.wdown = ldexpf(1.0f, ex - 32);
            }
            __syncthreads();
            // ---- phase B: weights and P.V of the chunk ---------------------------------------------------------
#pragma unroll
            for (int mb = 0; mb < MB; ++mb) {
                ones[mb][0] = ones[mb][1] = ones[mb][2] = ones[mb][3] = 0;
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[mb][e][0] = acc[mb][e][1] = acc[mb][e][2] = acc[mb][e][3] = 0;
            }
#pragma unroll
            for (int e = 0; e < kRounds; ++e) psum[e] = 0.0f;
            const float wup = sm.wup;
            for (int ti = 0; ti < ctiles; ++ti, cur = cur + 1 == kStages ? 0 : cur + 1) {
                const int n_here = min(kTilePos, clen - ti * kTilePos);
                uint8_t (*wd)[kWStride] = sm.wdig[ti & 1];
                // weight digits of the tile: a warp takes one query vector per round, lane L the slots 4 L .. 4 L + 3 =
                // positions 16 (L / 4) + 4 i + L % 4, i = 0..3: the four positions that one lane feeds into an MMA
                // lie in one word, and so do the rows it reads from V.
                const bool full_tile = n_here == kTilePos && (QB == 1 || chunk0 + ti * kTilePos + kTilePos - 1 <= p + q0);
                if constexpr (kSplitDigits) {
                    // two warps per query vector (all eight warps busy for four vectors): warp = (vector, half of the
                    // tile's 32 words), lane = (word L % 16, pair of positions L / 16); the lane pair L, L ^ 16 swaps
                    // its weights so that each lane can write two of the word's four digit rows
                    const int v = warp >> 1;
                    if (v < G) {  // warp-uniform
                        const int wi = 16 * (warp & 1) + (lane & 15), sub = lane >> 4;
                        const float2 s2 = *reinterpret_cast<const float2*>(&sm.sbuf[v][ti * kTilePos + 4 * wi + 2 * sub]);
                        const float2 v2 = *reinterpret_cast<const float2*>(&sm.vsc[ti * kTilePos + 4 * wi + 2 * sub]);
                        const float m_new = sm.ml[0][v];
                        const int r0 = 16 * (wi >> 2) + (wi & 3) + 8 * sub;  // positions r0 and r0 + 4
                        const float sv[2] = {s2.x, s2.y}, vv[2] = {v2.x, v2.y};
                        uint32_t u[2];
#pragma unroll
                        for (int i = 0; i < 2; ++i) {
                            const bool live = full_tile || (r0 + 4 * i < n_here && sv[i] != -INFINITY);
                            const float pe = live ? expf(__fsub_rn(sv[i], m_new)) : 0.0f;
                            psum[0] += pe;
                            u[i] = live ? __float2uint_rn(__fmul_rn(__fmul_rn(pe, vv[i]), wup)) : 0u;
                        }
                        const uint32_t o0 = __shfl_xor_sync(0xffffffffu, u[0], 16), o1 = __shfl_xor_sync(0xffffffffu, u[1], 16);
                        uint32_t dig[4];
                        if (sub == 0) transpose4(u[0], u[1], o0, o1, dig); else transpose4(o0, o1, u[0], u[1], dig);
                        // digit j = byte 3 - j: this lane writes digits 2 sub and 2 sub + 1
                        *reinterpret_cast<uint32_t*>(&wd[4 * v + 2 * sub][4 * wi]) = sub == 0 ? dig[3] : dig[1];
                        *reinterpret_cast<uint32_t*>(&wd[4 * v + 2 * sub + 1][4 * wi]) = sub == 0 ? dig[2] : dig[0];
                    }
                } else {
#pragma unroll
                for (int e = 0; e < kRounds; ++e) {
                    const int v = warp + e * kAttnWarps;
                    if (v < G) {  // warp-uniform
                        const float4 s4 = *reinterpret_cast<const float4*>(&sm.sbuf[v][ti * kTilePos + 4 * lane]);
                        const float4 v4 = *reinterpret_cast<const float4*>(&sm.vsc[ti * kTilePos + 4 * lane]);
                        const float m_new = sm.ml[0][v];
                        const int r0 = 16 * (lane >> 2) + (lane & 3);
                        const float sv[4] = {s4.x, s4.y, s4.z, s4.w}, vv[4] = {v4.x, v4.y, v4.z, v4.w};
                        uint32_t u[4], dig[4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            // (beyond the tile the buffer holds anything; a masked score is -inf and gives exp = 0)
                            const bool live = full_tile || (r0 + 4 * i < n_here && sv[i] != -INFINITY);
                            const float pe = live ? expf(__fsub_rn(sv[i], m_new)) : 0.0f;
                            psum[e] += pe;
                            // weight of the value row: p * v_scale (the value bytes enter the MMA as integers)
                            u[i] = live ? __float2uint_rn(__fmul_rn(__fmul_rn(pe, vv[i]), wup)) : 0u;
                        }
                        transpose4(u[0], u[1], u[2], u[3], dig);  // dig[e] = byte e of the four weights; digit j = byte 3 - j
#pragma unroll
                        for (int j = 0; j < 4; ++j) *reinterpret_cast<uint32_t*>(&wd[4 * v + j][4 * lane]) = dig[3 - j];
                    }
                }
                }
                cp_async_wait<1>();
                __syncthreads();  // the tile landed, its weight digits are complete; everybody is done with the tile before
                fetch(fc, cur >= 1 ? cur - 1 : kStages - 1);
                advance(fc);
                const uint8_t* vcol = sm.ring[cur] + 32 * dg + 4 * g;
                auto pv_step = [&](int ks) {
                    uint32_t b0[4], b1[4];
                    {
                        const uint8_t* vp = vcol + (32 * ks + t) * rstride;
                        transpose4(*reinterpret_cast<const uint32_t*>(vp), *reinterpret_cast<const uint32_t*>(vp + 4 * rstride),
                                   *reinterpret_cast<const uint32_t*>(vp + 8 * rstride), *reinterpret_cast<const uint32_t*>(vp + 12 * rstride), b0);
                        vp += 16 * rstride;
                        transpose4(*reinterpret_cast<const uint32_t*>(vp), *reinterpret_cast<const uint32_t*>(vp + 4 * rstride),
                                   *reinterpret_cast<const uint32_t*>(vp + 8 * rstride), *reinterpret_cast<const uint32_t*>(vp + 12 * rstride), b1);
                    }
#pragma unroll
                    for (int mb = 0; mb < MB; ++mb) {
                        const uint8_t* w0 = &wd[16 * mb + g][32 * ks + 4 * t];
                        const uint32_t a0 = *reinterpret_cast<const uint32_t*>(w0);
                        const uint32_t a1 = *reinterpret_cast<const uint32_t*>(w0 + 8 * kWStride);
                        const uint32_t a2 = *reinterpret_cast<const uint32_t*>(w0 + 16);
                        const uint32_t a3 = *reinterpret_cast<const uint32_t*>(w0 + 8 * kWStride + 16);
#pragma unroll
                        for (int e = 0; e < 4; ++e) mma_u8u8(acc[mb][e], a0, a1, a2, a3, b0[e], b1[e]);
                        mma_u8u8(ones[mb], a0, a1, a2, a3, 0x01010101u, 0x01010101u);  // sum of the digits: the "- 128" of the value bytes
                    }
                };
                if (HD == 128 && n_here == kTilePos) {  // two fixed steps per warp
                    pv_step(pq);
                    pv_step(pq + 2);
                } else {
                    for (int ks = pq; 32 * ks < n_here; ks += n_pq) pv_step(ks);
                }
            }
            // ---- end of the chunk: digits together, "- 128" out, to f32, into the running output ----
            // Row 16 mb + g (+ 8) = digit g % 4 of query vector 4 mb + g / 4 (+ 2); the four digits of a vector sit in
            // four lanes that differ in bits 2 and 3 of the lane number.
            {
                const float wdown = sm.wdown;
                const long long weight = 1ll << (8 * (3 - (g & 3)));
#pragma unroll
                for (int mb = 0; mb < MB; ++mb) {
#pragma unroll
                    for (int hrow = 0; hrow < 2; ++hrow) {
                        const int v = 4 * mb + 2 * hrow + (g >> 2);
                        const int one = ones[mb][2 * hrow];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
#pragma unroll
                            for (int cc = 0; cc < 2; ++cc) {
                                long long x = (long long)(acc[mb][e][2 * hrow + cc] - 128 * one) * weight;
                                x += shfl_xor_ll(x, 4);
                                x += shfl_xor_ll(x, 8);
                                // MMA e, column n = dim 32 dg + 4 n + e; this lane holds n = 2t and 2t + 1
                                if ((g & 3) == 0 && v < G)
                                    sm.part[(pq * G + v) * hd + 32 * dg + 4 * (2 * t + cc) + e] = __fmul_rn(__ll2float_rn(x), wdown);
                            }
                        }
                    }
                }
#pragma unroll
                for (int e = 0; e < kRounds; ++e) {
                    const float ws = warp_sum(psum[e]);
                    if (lane == 0) sm.wsum[warp][e] = ws;  // query vector warp + 8 e (two warps per vector: warp / 2)
                }
            }
            __syncthreads();
            for (int it = tid; it < G * hd; it += kAttnThreads) {
                const int v = it / hd;
                float add = sm.part[it];
                for (int g2 = 1; g2 < n_pq; ++g2) add = __fadd_rn(add, sm.part[g2 * G * hd + it]);
                sm.opart[it] = fmaf(sm.opart[it], sm.corr[v], add);
            }
            if (tid < G) {
                const float ps = kSplitDigits ? __fadd_rn(sm.wsum[2 * tid][0], sm.wsum[2 * tid + 1][0]) : sm.wsum[tid % kAttnWarps][tid / kAttnWarps];
                sm.ml[1][tid] = fmaf(sm.ml[1][tid], sm.corr[tid], ps);
            }
            __syncthreads();
        }
    }
    // only now may the next kernel's CTAs move in: earlier they would take the registers and
    // shared memory that this kernel's later CTAs are waiting for
    ptx::pdl_launch_dependents();

    // Merge of the spans of this (sequence, KV head): out = sum_s e^{m_s - m} o_s / sum_s e^{m_s - m} l_s.
    // The output columns are dealt evenly to the CTAs of the cluster.  Every span PUSHES its partial columns into the
    // CTA that finishes them (plain stores into the peer's shared memory), one cluster barrier makes the pushes
    // visible, and the finishing CTA reads local shared memory only: no remote load on the path and no second
    // barrier before the CTAs leave (nobody touches a peer after the barrier).
    {
        const int S = a.splits, rank = S > 1 ? (int)cluster_ctarank() : 0;
        const int total = G * hd;
        float amax = 0.0f;
        auto emit = [&](int it, float o) {
            const int h = it / hd;
            const int qi = q0 + h / NREP;  // new token of the sequence this query vector belongs to (decode: 0)
            if (qi < a.q_rows) a.out[(((int64_t)b * a.q_rows + qi) * a.n_heads + kvh * NREP + h % NREP) * hd + (it % hd)] = o;
            amax = fmaxf(amax, fabsf(o));
        };
        if (S == 1) {
            // one span: its own sums are the result (the weight e^{m - m} is exactly 1)
            for (int it = tid; it < total; it += kAttnThreads) emit(it, __fdiv_rn(sm.opart[it], sm.ml[1][it / hd]));
        } else if constexpr (G <= 8) {
            const int per_cta = (total + S - 1) / S;
            for (int it = tid; it < total; it += kAttnThreads)
                st_cluster_f32(&sm.rx_o[rank * per_cta + it % per_cta], (uint32_t)(it / per_cta), sm.opart[it]);
            for (int i = tid; i < S * 2 * G; i += kAttnThreads) {
                const int dst = i / (2 * G), j = i % (2 * G);
                st_cluster_f32(&sm.rx_ml[rank][j / G][j % G], (uint32_t)dst, sm.ml[j / G][j % G]);
            }
            cluster_sync_all();  // the pushes of every span are complete and visible
            for (int i = tid; i < per_cta; i += kAttnThreads) {
                const int it = rank * per_cta + i;
                if (it >= total) break;
                const int h = it / hd;
                float m = -INFINITY;
                for (int s2 = 0; s2 < S; ++s2) m = fmaxf(m, sm.rx_ml[s2][0][h]);
                float num = 0.0f, den = 0.0f;
                for (int s2 = 0; s2 < S; ++s2) {
                    // a span without positions (maximum -inf) weighs nothing
                    const float ms = sm.rx_ml[s2][0][h];
                    const bool live = ms != -INFINITY;
                    const float w = live ? expf(__fsub_rn(ms, m)) : 0.0f;
                    den = fmaf(sm.rx_ml[s2][1][h], w, den);
                    num = fmaf(live ? sm.rx_o[s2 * per_cta + i] : 0.0f, w, num);
                }
                emit(it, __fdiv_rn(num, den));
            }
        }
        if (a.absmax_out) {
            amax = warp_max(amax);
            if (lane == 0 && amax > 0.0f) atomicMax(a.absmax_out + b, __float_as_uint(amax));
        }
    }
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
    quant_row_warp(rowbuf[warp], hd, (which ? cache.v_q : cache.k_q) + r * hd, (which ? cache.v_s : cache.k_s) + r, nullptr, lane);
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
    quant_row_warp(rowbuf[warp], hd, (which ? cache.v_q : cache.k_q) + r * hd, (which ? cache.v_s : cache.k_s) + r, nullptr, lane);
}

constexpr size_t kHalfSm = 116 * 1024;
static_assert(kStages == 3, "the fetch two tiles ahead reuses the buffer of the tile before");
static_assert(sizeof(AttnSmemT<4>) <= 112 * 1024, "two CTAs of the decode kernel (up to 4 query heads per KV head) must fit one SM");
static_assert(sizeof(AttnSmemT<kMaxRep>) <= kHalfSm, "decode kernel: shared memory");
constexpr int kPrefillVectors = 16;  // query vectors per CTA of the prefill kernel: 16 / NREP positions x NREP heads

// How many clusters of each size can be resident at once (a CTA then takes a whole SM): a cluster's CTAs
// must sit in one GPC, so large clusters leave SMs unused, and a GPC with fewer SMs than the cluster
// has CTAs holds none.  Filled once per kernel instance from cudaOccupancyMaxActiveClusters.
struct ClusterTable {
    bool ready = false;
    int active[kMaxCluster + 1] = {0};  // active[s] = resident clusters of s CTAs (0: size unusable)
};

template <int NREP, int HD>
cudaError_t configure_rep(const ClusterTable** out) {
    static ClusterTable table;        // per process; every device of a process is the same GPU model
    static PerDeviceOnce attributes;  // shared-memory limits and the cluster-size permission: per device
    static bool big = false;
    auto* decode = attn_kernel<NREP, 1, HD>;
    auto* prefill = attn_kernel<NREP, kPrefillVectors / NREP, HD>;
    cudaError_t e = attributes.run([decode, prefill] {
        cudaError_t e2 = cudaFuncSetAttribute(decode, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kHalfSm);
        if (e2 == cudaSuccess)
            e2 = cudaFuncSetAttribute(prefill, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(AttnSmemT<kPrefillVectors>));
        if (e2 != cudaSuccess) return e2;
        big = cudaFuncSetAttribute(decode, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess;
        (void)cudaGetLastError();  // a refused permission only rules the large cluster sizes out
        return cudaSuccess;
    });
    if (e != cudaSuccess) return e;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (!table.ready) {
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
            if (cudaOccupancyMaxActiveClusters(&n, decode, &cfg) == cudaSuccess) table.active[s] = n;
        }
        cudaGetLastError();  // a refused query only rules a cluster size out
        if (table.active[1] < 1) table.active[1] = 1;
        table.ready = true;
    }
    *out = &table;
    return cudaSuccess;
}

template <int NREP, int HD>
cudaError_t launch_attn_rep(const AttnArgs& a, cudaStream_t stream) {
    const ClusterTable* table = nullptr;
    cudaError_t e = configure_rep<NREP, HD>(&table);
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
        return cudaLaunchKernelEx(&cfg, attn_kernel<NREP, QB, HD>, a);
    }
    if (a.splits < 1 || a.splits > kMaxCluster || table->active[a.splits] < 1) return cudaErrorInvalidValue;
    cfg.gridDim = dim3(a.batch * a.n_kv, a.splits);
    // When the whole grid fits one CTA per SM, ask for more than half of an SM's shared
    // memory: the block scheduler then cannot pair two CTAs on one SM while others idle.
    cfg.dynamicSmemBytes = ((int64_t)a.batch * a.n_kv * a.splits <= a.sm_count) ? kHalfSm : sizeof(AttnSmemT<NREP>);
    attr[0].val.clusterDim.y = (unsigned)a.splits;
    cfg.numAttrs = a.pdl ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, attn_kernel<NREP, 1, HD>, a);
}

template <int NREP>
cudaError_t launch_attn_hd(const AttnArgs& a, cudaStream_t stream) {
    if (a.head_dim == 128) return launch_attn_rep<NREP, 128>(a, stream);
    if (a.head_dim == 64) return launch_attn_rep<NREP, 64>(a, stream);
    return launch_attn_rep<NREP, 0>(a, stream);
}

// The cluster limits do not depend on the head size (the query asks for a whole SM per CTA): one table per `rep`.
const ClusterTable* attn_cluster_table(int rep) {
    const ClusterTable* t = nullptr;
    cudaError_t e = cudaErrorInvalidValue;
    switch (rep) {
        case 1: e = configure_rep<1, 128>(&t); break;
        case 2: e = configure_rep<2, 128>(&t); break;
        case 4: e = configure_rep<4, 128>(&t); break;
        case 8: e = configure_rep<8, 128>(&t); break;
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
        case 1: return launch_attn_hd<1>(a, stream);
        case 2: return launch_attn_hd<2>(a, stream);
        case 4: return launch_attn_hd<4>(a, stream);
        case 8: return launch_attn_hd<8>(a, stream);
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
