// Decode-time ternary product for 1..8 tokens: y[m, n] = sum_k q[m, k] * t[n, k].
//
// Stands in for the inner loops of BitLinearCpu::forward (kernels/cpu.rs:73-124,134-239)
// and the never-launched bit_linear_forward kernel (kernels/bit_op.cu:4-45).
//
// HBM-bound: every weight byte is read exactly once per launch.  Structure:
//   * persistent CTAs (two per SM when shared memory allows); CTA c owns row tiles
//     c, c+G, c+2G, ... (16 rows each);
//   * a producer thread streams the tiles of a row tile (contiguous in the tiled layout)
//     into a shared-memory ring with 1-D bulk async copies that complete on mbarriers -
//     16 KB per stage, so tens of KB per SM are in flight whatever the math warps do;
//   * 16 math warps split each stage along K (one 1 KB tile each).  A lane's two 16-byte
//     chunks are already the A-operand slots of mma.m16n8k32 (u8 x s8 -> s32): one AND
//     per register isolates field r of every byte as an unsigned multiple of 4^r, so the
//     unpack costs one integer instruction per four weights; the four field positions
//     accumulate into four accumulator sets that are shifted back at the end;
//   * the int8 activations sit in shared memory, byte-transposed in groups of 16 so that
//     the B-operand registers match the field order of the A registers;
//   * after the last stage of a row tile every math warp drops its 16x8 partial sums into
//     a shared-memory buffer and signals an mbarrier; a separate epilogue warp adds the 8
//     partials, subtracts sum_k q (undoing the +1 weight offset), scales and stores, so
//     the math warps never stop at a CTA barrier.  Integer accumulation makes the result
//     independent of how K was split;
//   * the quantisation of the activations can run inside the kernel (RMSNorm + absmax
//     quantise, or quantise with a known absmax): every CTA does it redundantly while its
//     first weight stages are already in flight, which removes a kernel boundary per
//     projection from the decode step; with programmatic dependent launch the weight
//     prefetch even starts before the previous kernel has finished.
#include <mutex>

#include "bt_common.cuh"
#include "bt_ptx.cuh"

namespace bt {

namespace {

constexpr int kEpiWarps = 4;
constexpr int kMathWarps = 16;
constexpr int kMathThreads = kMathWarps * 32;
constexpr int kProducerWarp = kMathWarps;
constexpr int kEpilogueWarp0 = kMathWarps + 1;  // first epilogue warp
constexpr int kThreads = (kMathWarps + 1 + kEpiWarps) * 32;
constexpr int kHalfTiles = kMathWarps;               // tiles of one pass over the math warps
constexpr int kHalfBytes = kHalfTiles * kTileBytes;  // 16 KB
constexpr int kAccBufs = 16;                          // accumulate buffers, one per row tile in flight
constexpr int kAccBufInts = 128;                      // [4 accumulator registers][32 lanes]
constexpr int kAccBytes = kAccBufs * kAccBufInts * 4;
constexpr int kMaxStages = 12;
constexpr int kBarBytes = (2 * kMaxStages + kAccBufs + 1) * 8 + kAccBufs * 4 + 8;
constexpr int kEarlyBytes = 64 * 1024;  // weight bytes a CTA requests before its activation loads are issued
constexpr int kTokBytes = 128;  // per-token scale and sum, shared with the epilogue warp
constexpr int kScratchBytes = 512;  // block-reduction scratch of the prologue
constexpr unsigned kErrGemvTimeout = 0x47454d56u;  // 'GEMV'

__device__ __forceinline__ void red_add_s32(int* p, int v) {
    asm volatile("red.shared.add.s32 [%0], %1;" ::"r"(ptx::smem_u32(p)), "r"(v) : "memory");
}

__device__ __forceinline__ uint4 lds128(const void* p) { return *reinterpret_cast<const uint4*>(p); }

// One 1 KB tile: 2 A loads, 4 B loads, 32 ANDs, 8 MMAs.  The four field positions are four
// independent accumulator chains: their first MMAs are issued back to back, then the second.
// FIRST: the tile opens a row tile, its first MMAs start from the zero register (the
// accumulators need no clearing between row tiles).
template <bool FIRST>
__device__ __forceinline__ void tile_mma_r(int (&acc)[4][4], const uint4& w4, const uint4& v4, const uint4 (&b4)[4]) {
#pragma unroll
    for (int f = 0; f < 4; ++f) {
        const uint32_t mask = 0x03030303u << (2 * f);
        if (FIRST) ptx::mma_u8s8_zero(acc[f], w4.x & mask, v4.x & mask, w4.z & mask, v4.z & mask, b4[f].x, b4[f].z);
        else ptx::mma_u8s8(acc[f], w4.x & mask, v4.x & mask, w4.z & mask, v4.z & mask, b4[f].x, b4[f].z);
    }
#pragma unroll
    for (int f = 0; f < 4; ++f) {
        const uint32_t mask = 0x03030303u << (2 * f);
        ptx::mma_u8s8(acc[f], w4.y & mask, v4.y & mask, w4.w & mask, v4.w & mask, b4[f].y, b4[f].w);
    }
}

// ---- reductions over the 256 math threads (named barrier 1) ----------------------------
__device__ __forceinline__ double math_sum_d(double v, double* slot, int warp, int lane) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (lane == 0) slot[warp] = v;
    ptx::named_bar_sync(1, kMathThreads);
    double r = 0.0;
#pragma unroll
    for (int w = 0; w < kMathWarps; ++w) r += slot[w];
    return r;
}
__device__ __forceinline__ float math_max_f(float v, float* slot, int warp, int lane) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (lane == 0) slot[warp] = v;
    ptx::named_bar_sync(1, kMathThreads);
    float r = 0.0f;
#pragma unroll
    for (int w = 0; w < kMathWarps; ++w) r = fmaxf(r, slot[w]);
    return r;
}
// Quantise 16 consecutive values (group j of a token) with multiplier inv = 127/max|x|, store them
// byte-transposed at their place in the activation image, return their sum.
__device__ __forceinline__ int quant_store_group(const float (&v)[16], float inv, uint8_t* dst_token, int j) {
    uint32_t in[4], out[4];
    int sum = 0;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        // |x| <= max|x| makes |x * inv| <= 127 up to two roundings, so the rounded values lie in
        // [-127, 127] and the saturating pack to signed bytes never changes one
        int qv[4];
#pragma unroll
        for (int r = 0; r < 4; ++r) qv[r] = ptx::round_half_away(__fmul_rn(v[4 * b + r], inv));
        const uint32_t word = ptx::pack4_sat_s8(qv[0], qv[1], qv[2], qv[3]);
        sum = ptx::dp4a_s8s8(word, 0x01010101u, sum);
        in[b] = word;
    }
    ptx::transpose4x4(in, out);
    const int kt = j >> 4, tt = (j >> 2) & 3, i = j & 3;
    uint8_t* p = dst_token + kt * kTileK + tt * 16 + i * 4;
#pragma unroll
    for (int r = 0; r < 4; ++r) *reinterpret_cast<uint32_t*>(p + r * 64) = out[r];
    return sum;
}

// The same for half a group: values 8*hf .. 8*hf+7 of group j (two of the four bytes of each word).
__device__ __forceinline__ int quant_store_half(const float (&v)[8], float inv, uint8_t* dst_token, int j, int hf) {
    int qv[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) qv[e] = ptx::round_half_away(__fmul_rn(v[e], inv));
    const uint32_t in0 = ptx::pack4_sat_s8(qv[0], qv[1], qv[2], qv[3]);
    const uint32_t in1 = ptx::pack4_sat_s8(qv[4], qv[5], qv[6], qv[7]);
    const int sum = ptx::dp4a_s8s8(in1, 0x01010101u, ptx::dp4a_s8s8(in0, 0x01010101u, 0));
    const int kt = j >> 4, tt = (j >> 2) & 3, i = j & 3;
    uint8_t* p = dst_token + kt * kTileK + tt * 16 + i * 4 + 2 * hf;
#pragma unroll
    for (int r = 0; r < 4; ++r)
        *reinterpret_cast<uint16_t*>(p + r * 64) = (uint16_t)ptx::prmt(in0, in1, (uint32_t)(r | ((4 + r) << 4)));
    return sum;
}

__device__ __forceinline__ void load16(const float* p, float (&v)[16]) {
#pragma unroll
    for (int b = 0; b < 4; ++b) {
        const float4 f = *reinterpret_cast<const float4*>(p + 4 * b);
        v[4 * b] = f.x; v[4 * b + 1] = f.y; v[4 * b + 2] = f.z; v[4 * b + 3] = f.w;
    }
}

// Builds the int8 activation image of all tokens in shared memory (math warps only) and
// leaves the per-token scale and sum in tok_sx / tok_qsum.
template <int PRO>
__device__ __forceinline__ void stage_activations(const GemvArgs& a, uint8_t* acts, int act_stride, float* tok_sx,
                                                  int* tok_qsum, uint8_t* scratch, int tid, int warp, int lane,
                                                  int k_tiles, const float (&w0)[16], uint64_t* x_issued) {
    // tells the producer that this warp's first activation loads are on their way
    auto loads_issued = [&]() {
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(x_issued);
    };
    const int groups_pad = k_tiles * (kTileK / 16);
    const int groups = (int)(a.k_in >> 4);  // k_in is a multiple of 16 on the fused paths
    double* sl_d = reinterpret_cast<double*>(scratch);            // kMathWarps doubles
    float* sl_f = reinterpret_cast<float*>(scratch + 256);         // kMathWarps floats
    if (PRO == PRO_Q8) {
        for (int n = 0; n < a.m; ++n) {
            const uint4* src = reinterpret_cast<const uint4*>(a.q + (int64_t)n * a.q_stride);
            uint8_t* dst = acts + (size_t)n * act_stride;
            for (int j = tid; j < groups_pad; j += kMathThreads) {
                const uint4 v = src[j];
                const uint32_t in[4] = {v.x, v.y, v.z, v.w};
                uint32_t out[4];
                ptx::transpose4x4(in, out);
                const int kt = j >> 4, tt = (j >> 2) & 3, i = j & 3;
                uint8_t* p = dst + kt * kTileK + tt * 16 + i * 4;
#pragma unroll
                for (int r = 0; r < 4; ++r) *reinterpret_cast<uint32_t*>(p + r * 64) = out[r];
            }
            if (n == 0) loads_issued();
        }
        if (tid < a.m) {
            tok_qsum[tid] = a.qsum[tid];
            tok_sx[tid] = a.sx ? a.sx[tid] : 0.0f;
        }
        return;
    }
    for (int n = 0; n < a.m; ++n) {
        const float* xr = a.x + (int64_t)n * a.x_stride;
        uint8_t* dst = acts + (size_t)n * act_stride;
        int local = 0;
        float s;
        if (PRO == PRO_RMSNORM && 2 * groups <= kMathThreads) {
            // k_in <= 4096: half a group (8 values) per thread, so that all math threads share the work
            const int j = tid >> 1, hf = tid & 1;
            const bool h = j < groups;
            float v[8];
            double ss0 = 0.0, ss1 = 0.0;
            if (h) {
                const float4 f0 = *reinterpret_cast<const float4*>(xr + 16 * j + 8 * hf);
                const float4 f1 = *reinterpret_cast<const float4*>(xr + 16 * j + 8 * hf + 4);
                v[0] = f0.x; v[1] = f0.y; v[2] = f0.z; v[3] = f0.w; v[4] = f1.x; v[5] = f1.y; v[6] = f1.z; v[7] = f1.w;
            }
            if (n == 0) loads_issued();
            if (h) {
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                    ss0 = fma((double)v[e], (double)v[e], ss0);
                    ss1 = fma((double)v[e + 1], (double)v[e + 1], ss1);
                }
            }
            const double ss = math_sum_d(ss0 + ss1, sl_d, warp, lane);
            const float denom = sqrtf(__fadd_rn((float)(ss / (double)a.k_in), a.eps));
            float amax = 0.0f;
            if (h) {
#pragma unroll
                for (int e = 0; e < 8; ++e) { v[e] = __fmul_rn(__fdiv_rn(v[e], denom), w0[e]); amax = fmaxf(amax, fabsf(v[e])); }
            }
            amax = math_max_f(amax, sl_f, warp, lane);
            s = __fdiv_rn(amax, 127.0f);
            const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
            if (h) local += quant_store_half(v, inv, dst, j, hf);
            for (int jp = groups + tid; jp < groups_pad; jp += kMathThreads) {
                const float z[16] = {0};
                quant_store_group(z, 0.0f, dst, jp);
            }
        } else if (PRO == PRO_RMSNORM) {
            // up to two 16-groups per thread held in registers (k_in <= 8192)
            float v0[16], v1[16];
            const int j0 = tid, j1 = tid + kMathThreads;
            const bool h0 = j0 < groups, h1 = j1 < groups;
            double ss = 0.0;
            if (h0) load16(xr + 16 * j0, v0);
            if (h1) load16(xr + 16 * j1, v1);
            if (n == 0) loads_issued();
            if (h0) {
#pragma unroll
                for (int e = 0; e < 16; ++e) ss = fma((double)v0[e], (double)v0[e], ss); }
            if (h1) {
#pragma unroll
                for (int e = 0; e < 16; ++e) ss = fma((double)v1[e], (double)v1[e], ss); }
            ss = math_sum_d(ss, sl_d, warp, lane);
            // x / sqrt(mean(x^2) + eps) * w  (layers/rms_norm.rs:40-55)
            const float denom = sqrtf(__fadd_rn((float)(ss / (double)a.k_in), a.eps));
            float amax = 0.0f;
            if (h0) {
#pragma unroll
                for (int e = 0; e < 16; ++e) { v0[e] = __fmul_rn(__fdiv_rn(v0[e], denom), w0[e]); amax = fmaxf(amax, fabsf(v0[e])); } }
            if (h1) { float w[16]; load16(a.norm_w + 16 * j1, w);
#pragma unroll
                for (int e = 0; e < 16; ++e) { v1[e] = __fmul_rn(__fdiv_rn(v1[e], denom), w[e]); amax = fmaxf(amax, fabsf(v1[e])); } }
            amax = math_max_f(amax, sl_f, warp, lane);
            s = __fdiv_rn(amax, 127.0f);
            const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
            if (h0) local += quant_store_group(v0, inv, dst, j0);
            if (h1) local += quant_store_group(v1, inv, dst, j1);
            for (int j = groups + tid; j < groups_pad; j += kMathThreads) {
                const float z[16] = {0};
                quant_store_group(z, 0.0f, dst, j);
            }
        } else {  // PRO_ABSMAX
            const float amax = __uint_as_float(a.absmax_in[n]);
            s = __fdiv_rn(amax, 127.0f);
            const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
            // four groups per thread per round, all loads of a round issued before any use
            for (int jb0 = 0; jb0 < groups_pad; jb0 += 4 * kMathThreads) {  // same trip count in every thread
                const int jb = jb0 + tid;
                float v[4][16];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int j = jb + u * kMathThreads;
                    if (j < groups) load16(xr + 16 * j, v[u]);
                    else {
#pragma unroll
                        for (int e = 0; e < 16; ++e) v[u][e] = 0.0f;
                    }
                }
                if (n == 0 && jb0 == 0) loads_issued();
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int j = jb + u * kMathThreads;
                    if (j < groups_pad) local += quant_store_group(v[u], inv, dst, j);
                }
            }
        }
        // the sum is only read by the epilogue warps, after the barrier that ends the prologue
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
        if (lane == 0) atomicAdd(&tok_qsum[n], local);
        if (tid == 0) tok_sx[n] = s;
    }
}

// TPW: tiles per math warp and ring stage (a stage is TPW passes of 16 KB).  With K <= 4096 a
// row tile is one pass, so a stage holds TPW row tiles of the CTA (one bulk copy each); with a
// longer K a stage holds up to 16*TPW consecutive tiles of one row tile.  Two tiles per warp
// halve the barrier round trips per byte and put both tiles' shared-memory loads in flight
// before the first MMA.
template <int PRO, int TPW>
__global__ void __launch_bounds__(kThreads, 1) gemv_kernel(GemvArgs a, int nstages, int act_stride) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int kStageBytes = TPW * kHalfBytes;
    constexpr int kStageTiles = TPW * kHalfTiles;
    uint8_t* ring = smem;
    int* accbuf = reinterpret_cast<int*>(ring + (size_t)nstages * kStageBytes);
    uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(accbuf) + kAccBytes);
    uint64_t* empty = full + kMaxStages;
    uint64_t* acc_full = empty + kMaxStages;
    uint64_t* x_issued = acc_full + kAccBufs;  // every math warp has issued its activation loads
    volatile unsigned* acc_gen = reinterpret_cast<volatile unsigned*>(x_issued + 1);
    float* tok_sx = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(full) + kBarBytes);
    int* tok_qsum = reinterpret_cast<int*>(tok_sx + 8);
    uint8_t* scratch = reinterpret_cast<uint8_t*>(tok_sx) + kTokBytes;
    uint8_t* acts = scratch + kScratchBytes;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_tiles = (int)a.k_tiles;
    const bool short_k = k_tiles <= kHalfTiles;  // a row tile is one pass
    const int stages_per_rt = (k_tiles + kStageTiles - 1) / kStageTiles;  // long K only
    const int my_rts = ((int)a.row_tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;  // (32-bit: a 64-bit division is slow)
    const int total_iters = short_k ? (my_rts + TPW - 1) / TPW : my_rts * stages_per_rt;

    // The barriers are set up side by side, one thread each, in the producer's warp, which then only reports at the
    // CTA barrier and goes on to request weights: nothing is copied before the barriers exist, and the set-up of a
    // CTA is on the path of every launch.  The other warps clear the accumulate buffers meanwhile.
    if (warp != kProducerWarp) {
        if (threadIdx.x < 8) tok_qsum[threadIdx.x] = 0;
        const int i0 = threadIdx.x < kProducerWarp * 32 ? threadIdx.x : threadIdx.x - 32;  // the producer's warp left out
        for (int i = i0; i < kAccBufs * kAccBufInts; i += kThreads - 32) accbuf[i] = 0;
        ptx::named_bar_sync(0, kThreads);
    } else {
        if (lane < nstages) {
            ptx::mbar_init(&full[lane], 1);
            ptx::mbar_init(&empty[lane], kMathWarps);
        }
        if (lane >= 16 && lane < 16 + kAccBufs) {
            ptx::mbar_init(&acc_full[lane - 16], kMathWarps);
            acc_gen[lane - 16] = 0;
        }
        if (lane == 15) ptx::mbar_init(x_issued, kMathWarps);
        ptx::mbar_fence_init();
        __syncwarp();
        ptx::named_bar_arrive(0, kThreads);
    }

    if (warp == kProducerWarp) {
        // ---------------- producer: weights do not depend on earlier kernels ----------------
        if (lane == 0) {
            bool ok = true;
            int slot = 0, sk = 0;
            uint32_t wait_parity = 1;  // flips to 0 for the second use of each slot
            bool first_round = true;
            int lt = 0;  // CTA-local row tile: global row tile blockIdx.x + lt * gridDim.x
            // The activation loads of the math warps queue behind whatever this SM has already
            // requested, and the math cannot start before they are back.  So only kEarlyBytes of
            // weights are requested up front (enough to keep HBM busy across the dependency
            // wait); the rest follows once the activation loads have been issued.
            const int early_iters = kEarlyBytes / kStageBytes;
            for (int it = 0; it < total_iters; ++it) {
                if (it == early_iters && ok) ok = ptx::mbar_wait_relaxed(x_issued, 0);
                if (!first_round && ok) ok = ptx::mbar_wait_relaxed(&empty[slot], wait_parity);
                uint8_t* dst = ring + (size_t)slot * kStageBytes;
                if (short_k) {
                    const int n_rt = my_rts - lt < TPW ? my_rts - lt : TPW;
                    const uint32_t bytes = (uint32_t)k_tiles * kTileBytes;
                    ptx::mbar_arrive_expect_tx(&full[slot], bytes * n_rt);
                    for (int u = 0; u < n_rt; ++u) {
                        const int64_t rt = blockIdx.x + (int64_t)(lt + u) * gridDim.x;
                        ptx::bulk_g2s(dst + u * kHalfBytes, a.tiles + rt * k_tiles * kTileBytes, bytes, &full[slot]);
                    }
                    lt += n_rt;
                } else {
                    const int kt0 = sk * kStageTiles;
                    const int nt = k_tiles - kt0 < kStageTiles ? k_tiles - kt0 : kStageTiles;
                    const uint32_t bytes = (uint32_t)nt * kTileBytes;
                    const int64_t rt = blockIdx.x + (int64_t)lt * gridDim.x;
                    ptx::mbar_arrive_expect_tx(&full[slot], bytes);
                    ptx::bulk_g2s(dst, a.tiles + (rt * k_tiles + kt0) * kTileBytes, bytes, &full[slot]);
                    if (++sk == stages_per_rt) { sk = 0; ++lt; }
                }
                if (++slot == nstages) { slot = 0; first_round = false; wait_parity ^= 1; }
                // once the ring is primed, let the next kernel of the stream start its own prefetch
                if (it + 1 == nstages || it + 1 == total_iters) ptx::pdl_launch_dependents();
            }
            if (total_iters == 0) ptx::pdl_launch_dependents();
            if (!ok) atomicExch(a.err, kErrGemvTimeout);
        }
        return;
    }

    if (warp >= kEpilogueWarp0) {
        ptx::pdl_wait();  // the output buffer belongs to earlier kernels until here
        // ---------------- epilogue warps: warp e serves the CTA's row tiles e, e + kEpiWarps, ...
        // Row tile lt is summed by the math warps (shared-memory atomics) into accumulate buffer
        // lt % kAccBufs; the epilogue warp reads the finished sums, clears the buffer and
        // publishes the buffer's generation so that the math warps may use it again. ----------
        const int epi = warp - kEpilogueWarp0;
        // single token, accumulated output: the old value of this warp's first row tile is fetched now, while the
        // math warps still build the activation image (it costs an L2 round trip that would otherwise end the kernel)
        float old_first = 0.f;
        if (a.m == 1 && a.epilogue == EPI_F32_ACCUM && epi < my_rts) {
            const int64_t row0 = (blockIdx.x + (int64_t)epi * gridDim.x) * kTileRows + (lane & 15);
            if (row0 < a.n_out) old_first = reinterpret_cast<const float*>(a.out)[row0];
        }
        ptx::named_bar_sync(2, kMathThreads + 32 * kEpiWarps);  // tok_sx / tok_qsum are ready
        const int t = lane & 3, g = lane >> 2;
        int qs[2] = {0, 0};
        float sx[2] = {0.f, 0.f};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int token = 2 * t + e;
            if (token < a.m) { qs[e] = tok_qsum[token]; sx[e] = tok_sx[token]; }
        }
        bool ok = true;
        float run_max[2] = {0.f, 0.f};  // EPI_SWIGLU: running max|out| of this lane's two tokens
        int64_t rt = blockIdx.x + (int64_t)epi * gridDim.x;
        if (a.m == 1) {
            // Single token: lane r < 16 owns row r of the tile (lanes 16-31 mirror them).
            const int r = lane & 15;
            const int qs0 = tok_qsum[0];
            const float sx0 = tok_sx[0];
            float amax1 = 0.f;
            if (a.epilogue == EPI_SWIGLU) {
                // silu(gate) * up has an exponential and a division, a dependent chain.  Four row tiles
                // (8 columns each) are finished together, one column per lane, so that the chain runs
                // once per four row tiles: chunk c = row tiles 4c .. 4c+3 of the CTA, chunks dealt
                // round-robin to the epilogue warps.
                const int sub = lane >> 3, col8 = lane & 7;
                const int n_chunks = (my_rts + 3) / 4;
                for (int c = epi; c < n_chunks; c += kEpiWarps) {
                    const int lt0 = 4 * c;
                    const int lt = lt0 + sub;
                    const bool valid = lt < my_rts;
                    const int64_t rtile = blockIdx.x + (int64_t)lt * gridDim.x;
                    float swg = 0.f, swu = 0.f;
                    if (valid) { swg = a.sw_tiles[2 * rtile]; swu = a.sw_tiles[2 * rtile + 1]; }
                    for (int s2 = 0; s2 < 4 && lt0 + s2 < my_rts; ++s2)
                        if (ok) ok = ptx::mbar_wait_relaxed(&acc_full[(lt0 + s2) % kAccBufs], (unsigned)((lt0 + s2) / kAccBufs) & 1);
                    int gsum = 0, usum = 0;
                    if (valid) {
                        int* buf = accbuf + (lt % kAccBufs) * kAccBufInts;
                        // rows 0-7 of the tile are gate rows, rows 8-15 the matching up rows
                        gsum = buf[col8]; usum = buf[col8 + 8];
                        buf[col8] = 0; buf[col8 + 8] = 0;
                    }
                    __threadfence_block();
                    __syncwarp();
                    if (lane < 4 && lt0 + lane < my_rts) acc_gen[(lt0 + lane) % kAccBufs] = (unsigned)((lt0 + lane) / kAccBufs) + 1;
                    const int64_t col = rtile * 8 + col8;
                    if (valid && col < a.n_out / 2) {
                        const float y = __fmul_rn(__fmul_rn((float)(gsum - qs0), swg), sx0);
                        const float uv = __fmul_rn(__fmul_rn((float)(usum - qs0), swu), sx0);
                        // silu(g) * u  (layers/swiglu.rs:31-33), f32 throughout like the reference
                        const float act = __fmul_rn(__fdiv_rn(y, __fadd_rn(1.0f, expf(-y))), uv);
                        reinterpret_cast<float*>(a.out)[col] = act;
                        amax1 = fmaxf(amax1, fabsf(act));
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) amax1 = fmaxf(amax1, __shfl_xor_sync(0xffffffffu, amax1, o));
                if (lane == 0) atomicMax(a.absmax_out, __float_as_uint(amax1));
                if (!ok && lane == 0) atomicExch(a.err, kErrGemvTimeout);
                return;
            }
            float sw = 0.f;
            if (a.epilogue != EPI_I32 && epi < my_rts) sw = a.sw_tiles[2 * rt + (r >> 3)];
            float old = old_first;
            for (int lt = epi; lt < my_rts; lt += kEpiWarps) {
                // the next row tile's scale (and old output) come from global memory: fetch them a round early
                float sw_next = 0.f, old_next = 0.f;
                if (a.epilogue != EPI_I32 && lt + kEpiWarps < my_rts) {
                    const int64_t rt_next = rt + (int64_t)kEpiWarps * gridDim.x;
                    sw_next = a.sw_tiles[2 * rt_next + (r >> 3)];
                    if (a.epilogue == EPI_F32_ACCUM && rt_next * kTileRows + r < a.n_out)
                        old_next = reinterpret_cast<const float*>(a.out)[rt_next * kTileRows + r];
                }
                const int b = lt % kAccBufs;
                const unsigned use = (unsigned)(lt / kAccBufs);
                if (ok) ok = ptx::mbar_wait_relaxed(&acc_full[b], use & 1);
                int* buf = accbuf + b * kAccBufInts;
                const int sum = buf[r];
                __syncwarp();
                if (lane < 16) buf[lane] = 0;
                __threadfence_block();
                __syncwarp();
                if (lane == 0) acc_gen[b] = use + 1;
                const int accv = sum - qs0;
                const int64_t row = rt * kTileRows + r;
                if (a.epilogue == EPI_I32) {
                    if (lane < 16 && row < a.n_out) reinterpret_cast<int32_t*>(a.out)[row] = accv;
                } else {
                    const float y = __fmul_rn(__fmul_rn((float)accv, sw), sx0);
                    if (lane < 16 && row < a.n_out) {
                        if (a.epilogue == EPI_F32) reinterpret_cast<float*>(a.out)[row] = y;
                        else if (a.epilogue == EPI_F32_ACCUM)
                            reinterpret_cast<float*>(a.out)[row] = __fadd_rn(old, y);
                        else reinterpret_cast<__nv_bfloat16*>(a.out)[row] = __float2bfloat16_rn(y);
                    }
                }
                sw = sw_next;
                old = old_next;
                rt += (int64_t)kEpiWarps * gridDim.x;
            }
            if (!ok && lane == 0) atomicExch(a.err, kErrGemvTimeout);
            return;
        }
        for (int lt = epi; lt < my_rts; lt += kEpiWarps) {
            float sw[2] = {0.f, 0.f};
            if (a.epilogue != EPI_I32) { sw[0] = a.sw_tiles[2 * rt]; sw[1] = a.sw_tiles[2 * rt + 1]; }
            const int b = lt % kAccBufs;
            const unsigned use = (unsigned)(lt / kAccBufs);
            if (ok) ok = ptx::mbar_wait_relaxed(&acc_full[b], use & 1);
            int* buf = accbuf + b * kAccBufInts;
            int sum[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) { sum[j] = buf[j * 32 + lane]; buf[j * 32 + lane] = 0; }
            __threadfence_block();
            __syncwarp();
            if (lane == 0) acc_gen[b] = use + 1;
            if (a.epilogue == EPI_SWIGLU) {
                // rows 0-7 of the tile are gate rows, rows 8-15 the matching up rows
                const int64_t col = rt * 8 + g;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int token = 2 * t + e;
                    if (token < a.m && col < a.n_out / 2) {
                        const float gv = __fmul_rn(__fmul_rn((float)(sum[e] - qs[e]), sw[0]), sx[e]);
                        const float uv = __fmul_rn(__fmul_rn((float)(sum[2 + e] - qs[e]), sw[1]), sx[e]);
                        // silu(g) * u  (layers/swiglu.rs:31-33), f32 throughout like the reference
                        const float act = __fmul_rn(__fdiv_rn(gv, __fadd_rn(1.0f, expf(-gv))), uv);
                        reinterpret_cast<float*>(a.out)[(int64_t)token * a.out_stride + col] = act;
                        run_max[e] = fmaxf(run_max[e], fabsf(act));
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int64_t row = rt * kTileRows + g + ((j & 2) ? 8 : 0);
                    const int e = j & 1, token = 2 * t + e;
                    if (token < a.m && row < a.n_out) {
                        const int accv = sum[j] - qs[e];
                        const int64_t o = (int64_t)token * a.out_stride + row;
                        if (a.epilogue == EPI_I32) {
                            reinterpret_cast<int32_t*>(a.out)[o] = accv;
                        } else {
                            const float y = __fmul_rn(__fmul_rn((float)accv, sw[j >> 1]), sx[e]);
                            if (a.epilogue == EPI_F32) reinterpret_cast<float*>(a.out)[o] = y;
                            else if (a.epilogue == EPI_F32_ACCUM)
                                reinterpret_cast<float*>(a.out)[o] = __fadd_rn(reinterpret_cast<float*>(a.out)[o], y);
                            else reinterpret_cast<__nv_bfloat16*>(a.out)[o] = __float2bfloat16_rn(y);
                        }
                    }
                }
            }
            rt += (int64_t)kEpiWarps * gridDim.x;
        }
        if (a.epilogue == EPI_SWIGLU) {
            // one atomic per token and warp: fold the lanes that share a token pair (same t)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
#pragma unroll
                for (int o = 4; o < 32; o <<= 1) run_max[e] = fmaxf(run_max[e], __shfl_xor_sync(0xffffffffu, run_max[e], o));
                const int token = 2 * t + e;
                if (g == 0 && token < a.m) atomicMax(a.absmax_out + token, __float_as_uint(run_max[e]));
            }
        }
        if (!ok && lane == 0) atomicExch(a.err, kErrGemvTimeout);
        return;
    }

    // ---------------- math warps ----------------
    const int tid = threadIdx.x;
    const int g = lane >> 2, t = lane & 3;
    // The norm weights do not depend on earlier kernels and usually come from DRAM (nothing
    // else touches them during a step): fetch them before waiting on the dependency.
    float w0[16];
    if (PRO == PRO_RMSNORM) {
        const int groups = (int)(a.k_in >> 4);
        if (2 * groups <= kMathThreads) {  // half a group per thread (see stage_activations)
            if ((tid >> 1) < groups) {
                const float4 f0 = *reinterpret_cast<const float4*>(a.norm_w + 8 * tid);
                const float4 f1 = *reinterpret_cast<const float4*>(a.norm_w + 8 * tid + 4);
                w0[0] = f0.x; w0[1] = f0.y; w0[2] = f0.z; w0[3] = f0.w; w0[4] = f1.x; w0[5] = f1.y; w0[6] = f1.z; w0[7] = f1.w;
            }
        } else if (tid < groups) {
            load16(a.norm_w + 16 * tid, w0);
        }
    }
    ptx::pdl_wait();  // activations belong to earlier kernels until here
    stage_activations<PRO>(a, acts, act_stride, tok_sx, tok_qsum, scratch, tid, warp, lane, k_tiles, w0, x_issued);
    ptx::named_bar_sync(2, kMathThreads + 32 * kEpiWarps);  // activation image complete, epilogue warps may read the scales

    int acc[4][4] = {};  // rewritten by the first tile of every row tile
    // lanes whose MMA column has no token read the last token's row instead: their columns are
    // never stored, and the loads need no predicate
    const uint8_t* my_acts = acts + (size_t)(g < a.m ? g : a.m - 1) * act_stride + t * 16;
    const bool single = a.m == 1;
    bool ok = true;
    int slot = 0;
    uint32_t parity = 0;

    // Row tile lt complete in this warp: fold the four field positions and add the warp's partial
    // sums into the row tile's accumulate buffer (integer atomics: the order of the 16 warps does
    // not matter).  gen_seen is the buffer's generation as read before the tile's math, so the
    // check normally costs nothing; it only spins when the epilogue warps are a whole round of
    // buffers behind.
    auto hand_over = [&](int lt, unsigned gen_seen, bool contributes) {
        const int b = lt % kAccBufs;
        const unsigned use = (unsigned)(lt / kAccBufs);
        if (gen_seen < use && ok) {
            bool got = false;
            for (unsigned i = 0; i < (1u << 22) && !got; ++i) got = acc_gen[b] >= use;
            ok = got;
        }
        int* buf = accbuf + b * kAccBufInts;
        if (contributes) {
            if (single) {
                // one token: only column 0 of the MMA tile is live (lanes with t = 0: rows g and g + 8)
                const int lo = acc[0][0] + (acc[1][0] >> 2) + (acc[2][0] >> 4) + (acc[3][0] >> 6);
                const int hi = acc[0][2] + (acc[1][2] >> 2) + (acc[2][2] >> 4) + (acc[3][2] >> 6);
                if (t == 0) { red_add_s32(buf + g, lo); red_add_s32(buf + g + 8, hi); }
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    red_add_s32(buf + j * 32 + lane, acc[0][j] + (acc[1][j] >> 2) + (acc[2][j] >> 4) + (acc[3][j] >> 6));
            }
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&acc_full[b]);
    };

    if (short_k) {
        // K <= 4096: this warp multiplies the same 256 inputs in every row tile, so its
        // activation registers are loaded once (the activation loads are two thirds of the
        // loop's shared-memory traffic otherwise) and every tile is a whole row tile
        const bool have = warp < k_tiles;
        uint4 b4[4];
#pragma unroll
        for (int f = 0; f < 4; ++f) b4[f] = have ? lds128(my_acts + warp * kTileK + f * 64) : make_uint4(0u, 0u, 0u, 0u);
        int lt = 0;
        for (int it = 0; it < total_iters; ++it) {
            unsigned gen[TPW];
#pragma unroll
            for (int u = 0; u < TPW; ++u) gen[u] = acc_gen[(lt + u) % kAccBufs];
            if (ok) ok = ptx::mbar_wait_bounded(&full[slot], parity);
            const uint8_t* tile = ring + (size_t)slot * kStageBytes + warp * kTileBytes + lane * 16;
            uint4 w4[TPW], v4[TPW];
#pragma unroll
            for (int u = 0; u < TPW; ++u) {
                if (have && lt + u < my_rts) { w4[u] = lds128(tile + u * kHalfBytes); v4[u] = lds128(tile + u * kHalfBytes + 512); }
            }
#pragma unroll
            for (int u = 0; u < TPW; ++u) {
                if (lt + u < my_rts) {
                    if (have) tile_mma_r<true>(acc, w4[u], v4[u], b4);
                    if (u == TPW - 1 || lt + u + 1 == my_rts) {
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive(&empty[slot]);
                    }
                    hand_over(lt + u, gen[u], have);
                }
            }
            lt += TPW;
            if (++slot == nstages) { slot = 0; parity ^= 1; }
        }
    } else {
        int lt = 0, sk = 0;
        unsigned gen = 0;
        for (int it = 0; it < total_iters; ++it) {
            if (sk == 0) gen = acc_gen[lt % kAccBufs];
            if (ok) ok = ptx::mbar_wait_bounded(&full[slot], parity);
            const uint8_t* tile = ring + (size_t)slot * kStageBytes + warp * kTileBytes + lane * 16;
            const int kt0 = sk * kStageTiles + warp;  // this warp's tiles of the stage: kt0, kt0 + 16, ...
            uint4 w4[TPW], v4[TPW];
#pragma unroll
            for (int u = 0; u < TPW; ++u) {
                if (kt0 + u * kHalfTiles < k_tiles) { w4[u] = lds128(tile + u * kHalfBytes); v4[u] = lds128(tile + u * kHalfBytes + 512); }
            }
#pragma unroll
            for (int u = 0; u < TPW; ++u) {
                const int kt = kt0 + u * kHalfTiles;
                if (kt < k_tiles) {
                    uint4 b4[4];
#pragma unroll
                    for (int f = 0; f < 4; ++f) b4[f] = lds128(my_acts + kt * kTileK + f * 64);
                    // tile `warp` of a row tile always exists here (more than 16 tiles): it opens the accumulators
                    if (u == 0 && sk == 0) tile_mma_r<true>(acc, w4[u], v4[u], b4);
                    else tile_mma_r<false>(acc, w4[u], v4[u], b4);
                }
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&empty[slot]);
            if (++slot == nstages) { slot = 0; parity ^= 1; }
            if (++sk == stages_per_rt) {
                sk = 0;
                hand_over(lt, gen, true);
                ++lt;
            }
        }
    }
    if (!ok) {
        if (lane == 0) atomicExch(a.err, kErrGemvTimeout);
        // give copies still in flight a bounded chance to land before the CTA retires
        for (int s = 0; s < nstages && s < total_iters; ++s) {
            const int uses = (total_iters - s + nstages - 1) / nstages;
            ptx::mbar_wait_bounded(&full[s], (uint32_t)((uses - 1) & 1), 1u << 16);
        }
    }
}

int g_configured[64] = {0};
std::mutex g_configured_mu;  // the forward entry points may be called from several host threads

// Fixed shared memory of a launch besides the ring: activation image of m tokens + bookkeeping.
size_t gemv_fixed_smem(int m, int64_t k_tiles) {
    return (size_t)m * (size_t)(k_tiles * kTileK + 64) + kAccBytes + kBarBytes + kTokBytes + kScratchBytes;
}
constexpr size_t kSmemBudget = 220 * 1024;

}  // namespace

// Largest token count (<= 8) whose activation image fits beside a minimal ring; 0 if even one token does not.
int gemv_max_tokens(int64_t k_tiles) {
    for (int m = 8; m >= 1; --m)
        if (gemv_fixed_smem(m, k_tiles) + 2 * kHalfBytes <= kSmemBudget) return m;
    return 0;
}

template <int TPW>
static cudaError_t launch_gemv_t(const GemvArgs& a, int grid, size_t smem, int nstages, int act_stride, cudaStream_t stream) {
    switch (a.prologue) {
        case PRO_RMSNORM: return launch_pdl(gemv_kernel<PRO_RMSNORM, TPW>, dim3(grid), dim3(kThreads), smem, stream, a.pdl, a, nstages, act_stride);
        case PRO_ABSMAX: return launch_pdl(gemv_kernel<PRO_ABSMAX, TPW>, dim3(grid), dim3(kThreads), smem, stream, a.pdl, a, nstages, act_stride);
        default: return launch_pdl(gemv_kernel<PRO_Q8, TPW>, dim3(grid), dim3(kThreads), smem, stream, a.pdl, a, nstages, act_stride);
    }
}

cudaError_t launch_gemv(const GemvArgs& a, int sm_count, cudaStream_t stream) {
    if (a.m < 1 || a.m > 8) return cudaErrorInvalidValue;
    if (a.prologue != PRO_Q8 && (a.k_in % 16 != 0)) return cudaErrorInvalidValue;
    if (a.prologue == PRO_RMSNORM && a.k_in > 16 * 2 * kMathThreads) return cudaErrorInvalidValue;
    if (a.epilogue == EPI_SWIGLU && (!a.absmax_out || a.n_out % 16 != 0)) return cudaErrorInvalidValue;
    const int act_stride = (int)(a.k_tiles * kTileK + 64);
    const size_t fixed = gemv_fixed_smem(a.m, a.k_tiles);
    // One CTA per SM.  The ring takes what shared memory allows, but never more stages than
    // the CTA has iterations.  Stages of two passes (32 KB) are used whenever at least three of
    // them fit beside the activation image; HBM needs well over 100 KB in flight per SM.
    const size_t budget = kSmemBudget;
    if (fixed + 2 * kHalfBytes > budget) return cudaErrorInvalidConfiguration;
    int64_t grid64 = sm_count;
    if (grid64 > a.row_tiles) grid64 = a.row_tiles;
    const int grid = (int)grid64;
    const int64_t rts_per_cta = (a.row_tiles + grid - 1) / grid;
    const bool short_k = a.k_tiles <= kHalfTiles;
    int tpw = (budget - fixed) / (2 * kHalfBytes) >= 3 ? 2 : 1;
    if (short_k && rts_per_cta < 2) tpw = 1;
    const int stage_bytes = tpw * kHalfBytes;
    int nstages = (int)((budget - fixed) / stage_bytes);
    if (nstages > kMaxStages / tpw) nstages = kMaxStages / tpw;
    const int64_t max_iters = short_k ? (rts_per_cta + tpw - 1) / tpw
                                      : rts_per_cta * ((a.k_tiles + tpw * kHalfTiles - 1) / (tpw * kHalfTiles));
    if (nstages > max_iters) nstages = (int)max_iters;
    if (nstages < 1) nstages = 1;
    const size_t smem = (size_t)nstages * stage_bytes + fixed;
    int dev = 0;
    cudaGetDevice(&dev);
    {
        std::lock_guard<std::mutex> lock(g_configured_mu);
        if (dev >= 0 && dev < 64 && !g_configured[dev]) {
            cudaError_t e = cudaFuncSetAttribute(gemv_kernel<PRO_Q8, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_kernel<PRO_RMSNORM, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_kernel<PRO_ABSMAX, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_kernel<PRO_Q8, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_kernel<PRO_RMSNORM, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget);
            if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_kernel<PRO_ABSMAX, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget);
            if (e != cudaSuccess) return e;
            g_configured[dev] = 1;
        }
    }
    return tpw == 2 ? launch_gemv_t<2>(a, grid, smem, nstages, act_stride, stream)
                    : launch_gemv_t<1>(a, grid, smem, nstages, act_stride, stream);
}

cudaError_t linear_product(const LinearDev& lin, const int8_t* q, int64_t q_stride,
                           const int32_t* qsum, const float* sx, int64_t m, void* out,
                           int64_t out_stride, int epilogue, unsigned int* err, int sm_count,
                           cudaStream_t stream) {
    const int bases = epilogue == EPI_I32 ? 1 : lin.w.n_bases;
    if (epilogue == EPI_BF16 && bases > 1) return cudaErrorInvalidValue;
    const size_t elem = epilogue == EPI_BF16 ? 2 : 4;
    // tokens per launch: as many (up to 8) as leave room for the ring beside their activation image
    const int chunk = gemv_max_tokens(lin.w.k_tiles);
    if (chunk < 1) return cudaErrorInvalidConfiguration;
    for (int64_t m0 = 0; m0 < m; m0 += chunk) {
        for (int b = 0; b < bases; ++b) {
            GemvArgs a = {};
            a.tiles = lin.w.tiles + (size_t)b * lin.w.basis_stride();
            a.row_tiles = lin.w.row_tiles;
            a.k_tiles = lin.w.k_tiles;
            a.n_out = lin.w.n_out;
            a.k_in = lin.w.k_in;
            a.prologue = PRO_Q8;
            a.q = q + m0 * q_stride;
            a.q_stride = q_stride;
            a.qsum = qsum + m0;
            a.sx = sx ? sx + m0 : nullptr;
            a.sw_tiles = lin.scale_tiles ? lin.scale_tiles + (size_t)b * lin.w.row_tiles * 2 : nullptr;
            a.m = (int)(m - m0 < chunk ? m - m0 : chunk);
            a.out = reinterpret_cast<uint8_t*>(out) + (size_t)m0 * out_stride * elem;
            a.out_stride = out_stride;
            a.epilogue = (b > 0 && epilogue == EPI_F32) ? EPI_F32_ACCUM : epilogue;
            a.err = err;
            a.pdl = true;  // weight prefetch may overlap the tail of whatever precedes it in the stream
            cudaError_t e = launch_gemv(a, sm_count, stream);
            if (e != cudaSuccess) return e;
        }
    }
    return cudaSuccess;
}

// The product on activations that a quantiser kernel has already written (int8 rows, sums and
// scales in global memory), with the epilogues of the fused decode step.
cudaError_t linear_product_q(const LinearDev& lin, const int8_t* q, int64_t q_stride, const int32_t* qsum,
                             const float* sx, int m, void* out, int64_t out_stride, int epilogue,
                             unsigned int* absmax_out, unsigned int* err, int sm_count, cudaStream_t stream) {
    if (lin.w.n_bases != 1 || m < 1 || m > 8) return cudaErrorInvalidValue;
    GemvArgs a = {};
    a.tiles = lin.w.tiles;
    a.row_tiles = lin.w.row_tiles;
    a.k_tiles = lin.w.k_tiles;
    a.n_out = lin.w.n_out;
    a.k_in = lin.w.k_in;
    a.prologue = PRO_Q8;
    a.q = q;
    a.q_stride = q_stride;
    a.qsum = qsum;
    a.sx = sx;
    a.absmax_out = absmax_out;
    a.sw_tiles = lin.scale_tiles;
    a.m = m;
    a.out = out;
    a.out_stride = out_stride;
    a.epilogue = epilogue;
    a.err = err;
    a.pdl = true;
    return launch_gemv(a, sm_count, stream);
}

cudaError_t linear_product_fused(const LinearDev& lin, const FusedIn& in, int m, void* out,
                                 int64_t out_stride, int epilogue, unsigned int* absmax_out,
                                 unsigned int* err, int sm_count, cudaStream_t stream) {
    if (lin.w.n_bases != 1 || m < 1 || m > 8) return cudaErrorInvalidValue;
    GemvArgs a = {};
    a.tiles = lin.w.tiles;
    a.row_tiles = lin.w.row_tiles;
    a.k_tiles = lin.w.k_tiles;
    a.n_out = lin.w.n_out;
    a.k_in = lin.w.k_in;
    a.prologue = in.prologue;
    a.x = in.x;
    a.x_stride = in.x_stride;
    a.norm_w = in.norm_w;
    a.eps = in.eps;
    a.absmax_in = in.absmax_in;
    a.absmax_out = absmax_out;
    a.sw_tiles = lin.scale_tiles;
    a.m = m;
    a.out = out;
    a.out_stride = out_stride;
    a.epilogue = epilogue;
    a.err = err;
    a.pdl = true;
    return launch_gemv(a, sm_count, stream);
}

}  // namespace bt
