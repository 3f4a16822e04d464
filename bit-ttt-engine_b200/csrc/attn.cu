// Fused decode attention over the Q8 KV cache: RoPE (layers/attention.rs:45-84) on the new
// q and k, Q8 append of k and v (layers/kv_cache.rs:95-119), scores = (q.k)/sqrt(hd) over
// positions 0..pos, softmax, .V (layers/attention.rs:198-217), all heads of a KV group in
// one CTA so the cache is read once (the reference materialises repeat_kv copies,
// layers/attention.rs:228-239).  The cache is read in place as u8; nothing is
// re-materialised in f32 (the reference dequantises the whole cache every step,
// layers/kv_cache.rs:84-92).  HBM-bound on the cache bytes: 2*n_kv*T*(hd+4) per sequence.
#include <stddef.h>

#include "bt_model.cuh"
#include "bt_ptx.cuh"

namespace bt {

namespace {

constexpr int kAttnWarps = 16;
constexpr int kAttnThreads = kAttnWarps * 32;

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

// One CTA = one (sequence, KV head, span of positions), 512 threads.  The span is walked in
// tiles of 128 positions that sit in shared memory as the cache stores them (u8 rows + one f32
// scale per row; rows padded by 32 bytes so that rows 4i .. 4i+3 fall into different banks); the
// first tile is fetched before the kernel waits for its predecessor.  Both contractions run on
// the f64 tensor-core path (mma.sync.m8n8k4.f64: 256 multiply-adds per warp instruction, the
// same peak as the f64 FMA pipe but one issue slot instead of eight and no cross-lane sums):
//   (1) scores: warp w owns positions 8w .. 8w+7 of the tile (rows of A = dequantised K, widened
//       to f64 by the lane that feeds it), columns of B = the NREP rotated query heads, k = dims;
//   (2) softmax weights: one (head, row) per thread; tile maxima and sums through shared memory;
//   (3) P.V: warp = (32 dims, every n-th group of 4 positions); rows of A = heads (weights),
//       columns of B = dims (one 32-bit load of V feeds four 8-dim blocks), k = positions; the
//       position groups are added once, after the last tile.
// Everything between the u8 loads and the final rounding is f64 on exact f32 values
// ((f32(q) - 128) * s, dequantize_q8, kv_cache.rs:122-128), so the result does not depend
// (beyond f64 rounding) on how positions are cut into tiles, groups and spans.
constexpr int kTilePos = 128;  // = cache rows prefetched per CTA
constexpr int kMaxRep = 8;

constexpr int kRowPad = 32;                 // bytes added to every cache row in shared memory
constexpr int kMaxRowBytes = 128 + kRowPad;
constexpr int kPadD = 132;                  // row length (doubles) of the per-head f64 arrays: rows 8 banks apart

struct AttnSmem {
    alignas(16) double qd[kMaxRep][kPadD];  // rotated queries (exact f32 values, widened)
    double pw[kMaxRep][kPadD];              // softmax weights of the tile (0 beyond the tile's rows)
    float sc[kMaxRep][kTilePos];
    double m_run[kMaxRep], l_run[kMaxRep], corr[kMaxRep], m_next[kMaxRep];
    double wmax[kMaxRep][4], wsum[kMaxRep][4];  // per warp (32 rows) maxima and sums of the tile
    float knew[128], vnew[128];
    // cache rows as stored (padded), two tiles: while one is worked on, the next arrives (cp.async)
    alignas(16) uint8_t kraw[2][kTilePos * kMaxRowBytes];
    alignas(16) uint8_t vraw[2][kTilePos * kMaxRowBytes];
    alignas(16) float ksr[2][kTilePos], vsr[2][kTilePos];
    alignas(16) double red[16 * kMaxRep * 32];  // [position group][head][dim] partial outputs; scratch of the merge
};

// D(8x8, f64) += A(8x4, row) * B(4x8, col): lane (g = lane/4, t = lane%4) holds A[g][t], B[t][g], D[g][2t], D[g][2t+1]
__device__ __forceinline__ void dmma884(double& d0, double& d1, double a, double b) {
    asm("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};" : "+d"(d0), "+d"(d1) : "d"(a), "d"(b));
}

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ptx::smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst_smem, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(ptx::smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// (f32(byte) - 128) * s without an integer-to-float conversion, for byte `which` (0..3) of a
// 32-bit word: 0x4B0000bb is the float 2^23 + b, and subtracting 2^23 + 128 is exact.
__device__ __forceinline__ double dequant_byte(uint32_t word, int which, float s) {
    const uint32_t bits = __byte_perm(word, 0x4B000000u, 0x7540 + which);
    return (double)__fmul_rn(__fsub_rn(__uint_as_float(bits), 8388736.0f), s);
}

template <int NREP>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(AttnArgs a) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    AttnSmem& sm = *reinterpret_cast<AttnSmem*>(smem_raw);
#define STAMP(i) do { if (a.dbg && (i) < 8 && threadIdx.x == 0) a.dbg[(blockIdx.y * gridDim.x + blockIdx.x) * 8 + (i)] = ptx::globaltimer(); } while (0)
    STAMP(0);
    const int hd = a.head_dim, half = hd >> 1;
    constexpr int nrep = NREP;
    const int b = blockIdx.x / a.n_kv, kvh = blockIdx.x % a.n_kv;
    const int split = blockIdx.y;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // The spans follow the sequence's current length, not the capacity the launch was planned
    // for: every CTA of a (sequence, KV head) gets an equal share (a multiple of 32 positions) of
    // what the cache holds now.  The position counter is only written by the last kernel of a
    // decode step, and steps do not overlap, so it may be read before the dependency wait.
    int span = (((a.pos[blockIdx.x / a.n_kv] + 1) + a.splits - 1) / a.splits + 31) & ~31;
    if (span > a.span) span = a.span;
    const int t0 = split * span;
    const int64_t row_base = ((int64_t)b * a.n_kv + kvh) * a.cache.max_seq;
    const int row16 = hd / 16;  // 16-byte pieces per row
    const int rstride = hd + kRowPad;  // row stride of the tiles in shared memory
    // The cache rows of earlier positions were written by earlier steps, so they can be fetched
    // before the dependency wait (whatever sits in rows at or beyond the current position is
    // fetched too and never used; the owner of the new position overwrites its copy below).
    const int raw_rows = max(0, min(min(kTilePos, span), a.cache.max_seq - t0));
    {
        const uint4* ksrc = reinterpret_cast<const uint4*>(a.cache.k_q + (row_base + t0) * hd);
        const uint4* vsrc = reinterpret_cast<const uint4*>(a.cache.v_q + (row_base + t0) * hd);
        const int n16 = raw_rows * row16;
        for (int i0 = tid; i0 < n16; i0 += 2 * kAttnThreads) {
            const int i1 = i0 + kAttnThreads;
            const bool h1 = i1 < n16;
            const uint4 k0 = ksrc[i0], v0 = vsrc[i0];
            uint4 k1 = make_uint4(0u, 0u, 0u, 0u), v1 = k1;
            if (h1) { k1 = ksrc[i1]; v1 = vsrc[i1]; }
            const int o0 = (i0 / row16) * rstride + (i0 % row16) * 16;
            *reinterpret_cast<uint4*>(sm.kraw[0] + o0) = k0;
            *reinterpret_cast<uint4*>(sm.vraw[0] + o0) = v0;
            if (h1) {
                const int o1 = (i1 / row16) * rstride + (i1 % row16) * 16;
                *reinterpret_cast<uint4*>(sm.kraw[0] + o1) = k1;
                *reinterpret_cast<uint4*>(sm.vraw[0] + o1) = v1;
            }
        }
        if (tid < raw_rows) sm.ksr[0][tid] = a.cache.k_s[row_base + t0 + tid];
        else if (tid >= 256 && tid - 256 < raw_rows) sm.vsr[0][tid - 256] = a.cache.v_s[row_base + t0 + tid - 256];
    }
    ptx::pdl_wait();
    STAMP(1);

    const int p = a.pos[b];
    const int t_len = p + 1;
    const int t1 = min(t_len, t0 + span);
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
        sm.qd[h][c] = (double)__fsub_rn(__fmul_rn(x1, cs), __fmul_rn(x2, sn));
        sm.qd[h][half + c] = (double)__fadd_rn(__fmul_rn(x1, sn), __fmul_rn(x2, cs));
    }
    if (tid < nrep) { sm.m_run[tid] = -INFINITY; sm.l_run[tid] = 0.0; }
    // The MMA fragments have 8 head rows / columns.  The arrays of heads that do not exist are
    // zero, so those rows and columns contribute exact zeros without any per-lane condition in the
    // MMA loops.
    for (int i = tid; i < (kMaxRep - nrep) * kPadD; i += blockDim.x) {
        sm.qd[nrep + i / kPadD][i % kPadD] = 0.0;
        sm.pw[nrep + i / kPadD][i % kPadD] = 0.0;
    }
    if (tid >= nrep && tid < kMaxRep) sm.corr[tid] = 0.0;
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
                                      in_raw ? sm.kraw[0] + (p - t0) * rstride : nullptr, in_raw ? sm.ksr[0] + (p - t0) : nullptr, lane);
        if (warp == 1) quant_row_warp(sm.vnew, hd, a.cache.v_q + (row_base + p) * hd, a.cache.v_s + row_base + p,
                                      in_raw ? sm.vraw[0] + (p - t0) * rstride : nullptr, in_raw ? sm.vsr[0] + (p - t0) : nullptr, lane);
    }
    __syncthreads();  // the block's own global writes are visible to it after the barrier
    STAMP(2);

    // fragment coordinates of the f64 MMA: g = row of A / column of B, t = k index
    const int g = lane >> 2, t = lane & 3;
    // P.V ownership: warp = (group of 32 dims dg, position group pg); the warp handles the
    // 4-position groups pg, pg + n_pg, ... of every tile for dims 32 dg .. 32 dg + 31: one
    // 32-bit load of a V row (dims 32 dg + 4 g .. + 3) feeds four MMAs, MMA e holding dim
    // 32 dg + 4 n + e in column n.  Lane (g, t) ends with head g, n = 2t and 2t + 1.
    const int n_dg = hd >> 5;
    const int n_pg = kAttnWarps / n_dg;
    const int dg = warp % n_dg, pg = warp / n_dg;
    const bool pv_active = pg < n_pg;
    double acc[4][2];
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[e][0] = acc[e][1] = 0.0;

    int cur = 0;  // buffer holding the current tile
    for (int tb = t0; tb < t1; tb += kTilePos) {
        const int n_here = min(kTilePos, t1 - tb);
        if (tb + kTilePos < t1) {
            // long span: start fetching the next tile's rows into the other buffer (its previous
            // contents were last read before the barrier that ended the previous tile)
            const int nb = tb + kTilePos, n_next = min(kTilePos, t1 - nb);
            const uint8_t* ksrc = a.cache.k_q + (row_base + nb) * hd;
            const uint8_t* vsrc = a.cache.v_q + (row_base + nb) * hd;
            for (int i = tid; i < n_next * row16; i += blockDim.x) {
                const int o = (i / row16) * rstride + (i % row16) * 16;
                cp_async16(sm.kraw[cur ^ 1] + o, ksrc + 16 * i);
                cp_async16(sm.vraw[cur ^ 1] + o, vsrc + 16 * i);
            }
            for (int i = tid; i < n_next; i += blockDim.x) {
                cp_async4(&sm.ksr[cur ^ 1][i], a.cache.k_s + row_base + nb + i);
                cp_async4(&sm.vsr[cur ^ 1][i], a.cache.v_s + row_base + nb + i);
            }
        }
        const uint8_t* kraw = sm.kraw[cur];
        const uint8_t* vraw = sm.vraw[cur];
        const float* ksr = sm.ksr[cur];
        const float* vsr = sm.vsr[cur];
        STAMP(3);
        // Rows at or beyond n_here hold anything.  P.V walks whole 4-position groups, so the (at most
        // three) rows that complete the last group are cleared: value bytes 128 (= 0), scale 0, and
        // their softmax weights are 0 as well.  (Read after the barriers that follow the scores.)
        {
            const int r_end = (n_here + 3) & ~3;
            for (int i = tid; i < (r_end - n_here) * (hd >> 2); i += blockDim.x) {
                const int r = n_here + i / (hd >> 2);
                *reinterpret_cast<uint32_t*>(sm.vraw[cur] + r * rstride + 4 * (i % (hd >> 2))) = 0x80808080u;
            }
            if (tid >= n_here && tid < r_end) sm.vsr[cur][tid] = 0.0f;
        }
        // (1) scores: S[8 positions x NREP heads] = K[8 x hd] . q[hd x NREP], hd / 4 MMAs per
        //     group of 8 positions.  Lane (g, t) dequantises dims 4i + t of position row0 + g
        //     (byte t of every 32-bit word of its row) and supplies q[head g][4i + t].  Rows at or
        //     beyond n_here hold anything; they only reach their own row of S, which is dropped.
        for (int row0 = 8 * warp; row0 < n_here; row0 += 8 * kAttnWarps) {
            const uint8_t* krow = kraw + (row0 + g) * rstride;
            const float ks = ksr[row0 + g];
            const double* qrow = sm.qd[g];
            double s0 = 0.0, s1 = 0.0, u0 = 0.0, u1 = 0.0;  // two chains: even and odd words
            for (int j = 0; j < row16; ++j) {
                const uint4 kw = *reinterpret_cast<const uint4*>(krow + 16 * j);
                const uint32_t w4[4] = {kw.x, kw.y, kw.z, kw.w};
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const double kv = dequant_byte(w4[e], t, ks);
                    const double qv = qrow[16 * j + 4 * e + t];
                    if (e & 1) dmma884(u0, u1, kv, qv);
                    else dmma884(s0, s1, kv, qv);
                }
            }
            s0 += u0; s1 += u1;
            if (row0 + g < n_here) {
                if (2 * t < NREP) sm.sc[2 * t][row0 + g] = __fmul_rn((float)s0, a.scaling);  // (q.k) * 1/sqrt(hd), attention.rs:202
                if (2 * t + 1 < NREP) sm.sc[2 * t + 1][row0 + g] = __fmul_rn((float)s1, a.scaling);
            }
        }
        __syncthreads();
        STAMP(4);
        // (2) softmax weights of the tile: one (head, row) per thread, so that the f64 exponentials
        //     run on every warp; a warp covers 32 rows of one head, four warps a head.  Tile
        //     maxima and sums go through shared memory in a fixed order.
        constexpr int kSoftItems = (NREP * kTilePos + kAttnThreads - 1) / kAttnThreads;
        double sv[kSoftItems];
#pragma unroll
        for (int e = 0; e < kSoftItems; ++e) {
            const int it = tid + e * kAttnThreads;
            const int h = it / kTilePos, r = it % kTilePos;
            sv[e] = (h < NREP && r < n_here) ? (double)sm.sc[h][r] : -INFINITY;
            double wm = sv[e];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) wm = fmax(wm, __shfl_xor_sync(0xffffffffu, wm, o));
            if (lane == 0 && h < NREP) sm.wmax[h][(it >> 5) & 3] = wm;
        }
        __syncthreads();
#pragma unroll
        for (int e = 0; e < kSoftItems; ++e) {
            const int it = tid + e * kAttnThreads;
            const int h = it / kTilePos, r = it % kTilePos;
            if (h < NREP) {  // warp-uniform
                const double m_old = sm.m_run[h];
                const double m_new = fmax(fmax(m_old, fmax(sm.wmax[h][0], sm.wmax[h][1])), fmax(sm.wmax[h][2], sm.wmax[h][3]));
                const double pe = r < n_here ? exp(sv[e] - m_new) : 0.0;
                sm.pw[h][r] = pe;
                double ws = pe;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ws += __shfl_xor_sync(0xffffffffu, ws, o);
                if (lane == 0) sm.wsum[h][(it >> 5) & 3] = ws;
                if (r == 0) {
                    sm.corr[h] = exp(m_old - m_new);  // exp(-inf) = 0 on the first tile
                    sm.m_next[h] = m_new;
                }
            }
        }
        __syncthreads();
        STAMP(5);
        if (tid < NREP) {  // running sum and maximum (nobody reads them before the next barrier)
            const double psum = ((sm.wsum[tid][0] + sm.wsum[tid][1]) + sm.wsum[tid][2]) + sm.wsum[tid][3];
            sm.l_run[tid] = fma(sm.l_run[tid], sm.corr[tid], psum);
            sm.m_run[tid] = sm.m_next[tid];
        }
        // (3) O[NREP heads x 32 dims] = O * corr + P[heads x positions] . V[positions x dims]
        if (pv_active) {
            const double cr = sm.corr[g];
#pragma unroll
            for (int e = 0; e < 4; ++e) { acc[e][0] *= cr; acc[e][1] *= cr; }
            const double* prow = sm.pw[g];
#pragma unroll 4
            for (int i = pg; 4 * i < n_here; i += n_pg) {
                const int r = 4 * i + t;  // this lane's position of the group
                const uint32_t vw = *reinterpret_cast<const uint32_t*>(vraw + r * rstride + 32 * dg + 4 * g);
                const float vs = vsr[r];
                const double pr = prow[r];
#pragma unroll
                for (int e = 0; e < 4; ++e) dmma884(acc[e][0], acc[e][1], pr, dequant_byte(vw, e, vs));
            }
        }
        if (tb + kTilePos < t1) {
            cp_async_wait_all();
            __syncthreads();  // next tile complete and visible; this tile's buffers free again
            cur ^= 1;
        }
    }
    // add the position groups (fixed order) through shared memory, one (head, dim) per thread
    {
        double* red = sm.red;  // [n_pg][NREP][hd]
        if (pv_active && g < NREP) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                // MMA e, column n = dim 32 dg + 4 n + e; this lane holds n = 2t and 2t + 1
                red[((int64_t)pg * NREP + g) * hd + 32 * dg + 4 * (2 * t) + e] = acc[e][0];
                red[((int64_t)pg * NREP + g) * hd + 32 * dg + 4 * (2 * t + 1) + e] = acc[e][1];
            }
        }
        __syncthreads();
        for (int it = tid; it < NREP * hd; it += blockDim.x) {
            const int h = it / hd, dcol = it % hd;
            double v = 0.0;
            for (int g2 = 0; g2 < n_pg; ++g2) v += red[((int64_t)g2 * NREP + h) * hd + dcol];
            double* dst = part_base + (int64_t)h * a.splits * (hd + 2);
            dst[2 + dcol] = v;
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
    // Release / acquire by one thread around the ticket: the barrier orders every thread's stores
    // of the partial result before thread 0's fence (fences are cumulative), and for the last
    // arrival thread 0's second fence orders the ticket before the loads that follow the barrier
    // (which read through L2).
    __syncthreads();
    __shared__ unsigned int arrived;
    if (tid == 0) {
        __threadfence();
        arrived = atomicAdd(a.counters + blockIdx.x, 1u);
        __threadfence();
    }
    __syncthreads();
    STAMP(7);
    if (arrived != (unsigned int)a.splits - 1) return;
    if (tid == 0) a.counters[blockIdx.x] = 0;  // ready for the next launch
    const double* group = a.partial + ((int64_t)b * a.n_heads + kvh * nrep) * a.splits * (hd + 2);
    // One batch of independent loads: every span's maximum and sum into shared memory and, at
    // the same time, this thread's output column of the first spans into registers; the weights
    // w_s = e^{m_s - m} are formed while those are in flight.
    constexpr int kItems = NREP * 128 > kAttnThreads ? 2 : 1;  // (head, column) outputs per thread
    constexpr int kMergeBatch = kItems == 1 ? 32 : 16;          // spans whose values are fetched up front
    double* mw = sm.red;          // [nrep][64] maxima, then weights (the tile buffers are free now)
    double* ls = mw + kMaxRep * 64;                          // [nrep][64] sums
    double* lsum = ls + kMaxRep * 64;                        // [nrep] reciprocals of the merged denominators
    for (int i = tid; i < nrep * a.splits; i += blockDim.x) {
        const int h = i / a.splits, s2 = i % a.splits;
        const double* src = group + ((int64_t)h * a.splits + s2) * (hd + 2);
        mw[h * 64 + s2] = __ldcg(src);
        ls[h * 64 + s2] = __ldcg(src + 1);
    }
    // (head, column) items: item tid and, for nrep * hd > 512, item tid + 512
    double pre[kItems][kMergeBatch];
#pragma unroll
    for (int e = 0; e < kItems; ++e) {
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
        if (lane == 0) lsum[h] = 1.0 / l;  // one division per head; the outputs multiply
    }
    __syncthreads();
#pragma unroll
    for (int e = 0; e < kItems; ++e) {
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
            const float o = (float)((v0 + v1) * lsum[h]);
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

namespace {
template <int NREP>
cudaError_t launch_attn_rep(const AttnArgs& a, cudaStream_t stream) {
    // the row-group buffer at the end of the shared-memory block scales with the heads per group
    constexpr size_t kRedDoubles = 512 * NREP > 2 * kMaxRep * 64 + kMaxRep ? 512 * NREP : 2 * kMaxRep * 64 + kMaxRep;  // [n_pg][NREP][hd], n_pg * hd = 512
    constexpr size_t kSmem = offsetof(AttnSmem, red) + kRedDoubles * sizeof(double);
    constexpr size_t kHalfSm = 116 * 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e0 = cudaFuncSetAttribute(attn_decode_kernel<NREP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              (int)(kSmem > kHalfSm ? kSmem : kHalfSm));
        if (e0 != cudaSuccess) return e0;
        configured = true;
    }
    dim3 grid(a.batch * a.n_kv, a.splits);
    // When the whole grid fits one CTA per SM, ask for more than half of an SM's shared
    // memory: the block scheduler then cannot pair two CTAs on one SM while others idle.
    size_t smem = kSmem;
    if ((int64_t)grid.x * grid.y <= a.sm_count && smem < kHalfSm) smem = kHalfSm;
    return launch_pdl(attn_decode_kernel<NREP>, grid, dim3(kAttnThreads), smem, stream, a.pdl, a);
}
}  // namespace

cudaError_t launch_attn_decode(const AttnArgs& a, cudaStream_t stream) {
    const int rep = a.n_kv > 0 ? a.n_heads / a.n_kv : 0;
    if (a.head_dim % 32 != 0 || a.head_dim > 128 || a.n_heads % a.n_kv != 0 || rep < 1 || rep > kMaxRep ||
        a.span % 32 != 0)
        return cudaErrorInvalidValue;
    switch (rep) {
        case 1: return launch_attn_rep<1>(a, stream);
        case 2: return launch_attn_rep<2>(a, stream);
        case 4: return launch_attn_rep<4>(a, stream);
        case 8: return launch_attn_rep<8>(a, stream);
        default: return cudaErrorInvalidValue;
    }
}

cudaError_t launch_rope_tables(const float* inv_freq, int max_seq, int half, float* cos_t, float* sin_t,
                               cudaStream_t stream) {
    rope_table_kernel<<<148, 256, 0, stream>>>(inv_freq, max_seq, half, cos_t, sin_t);
    return cudaGetLastError();
}

}  // namespace bt
