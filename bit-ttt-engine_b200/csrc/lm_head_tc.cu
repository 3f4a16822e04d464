// Dense bf16 lm_head for more than 8 tokens on the tensor cores (tcgen05, kind::f16):
//   logits[m, v] = sum_c W[v, c] * xn[m, c],  xn = RMSNorm(h)   (model/llama.rs:256-266).
// W is bf16; xn is f32 and is split into two bf16 terms hi + lo (error ~2^-17 relative), which
// ride as 2 x 64 columns of one N = 128 product and are added in the epilogue, so the result
// stays within ~1e-5 of the f32 reference instead of the 4e-3 of a plain bf16 cast.
// W is kept in a second, tile-ordered copy (128 rows x 64 inputs per 16 KB tile, 8x16-byte core
// matrices, K-major, no swizzle) so that one 1-D bulk copy fetches an operand tile.
#include "bt_common.cuh"
#include "bt_model.cuh"
#include "bt_ptx.cuh"

namespace bt {

namespace {

constexpr int kRows = 128, kChunk = 64, kTok = 64, kCols = 2 * kTok;  // N = hi | lo
constexpr int kATile = kRows * kChunk * 2;                              // 16 KB
constexpr int kBTile = kCols * kChunk * 2;                              // 16 KB
constexpr int kStages = 4;
constexpr int kThreads = 6 * 32;
constexpr unsigned kErrLmTimeout = 0x4c4d4844u;  // 'LMHD'

// kind::f16: D = f32, A (the weights) and B (the activation pieces) both bf16 or both IEEE half - the two
// operand formats of one instruction must be the same 16-bit type - K-major, M x N tile
__device__ __forceinline__ uint32_t instr_desc_bf16(int m, int n, bool f16) {
    uint32_t d = 0;
    d |= 1u << 4;                    // accumulator format: f32
    d |= (f16 ? 0u : 1u) << 7;       // A format: 0 = f16, 1 = bf16
    d |= (f16 ? 0u : 1u) << 10;      // B format
    d |= (uint32_t)(n >> 3) << 17;
    d |= (uint32_t)(m >> 4) << 24;
    return d;
}

// byte offset of element (row, c) inside a K-major tile with `chunk` 2-byte inputs per row
__device__ __host__ __forceinline__ int64_t tile_off(int row, int c, int chunk) {
    return (int64_t)(row >> 3) * (chunk / 8) * 128 + (c >> 3) * 128 + (row & 7) * 16 + (c & 7) * 2;
}

// row-major bf16 [vocab, hidden] -> tiles [row_set][k_chunk][16 KB]
__global__ void lm_retile_kernel(const __nv_bfloat16* __restrict__ w, int64_t vocab, int hidden,
                                 __nv_bfloat16* __restrict__ tiles) {
    const int64_t row_sets = (vocab + kRows - 1) / kRows;
    const int chunks = hidden / kChunk;
    const int64_t total = row_sets * chunks * (kRows * kChunk);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t tile = i / (kRows * kChunk);
        const int e = (int)(i % (kRows * kChunk));
        const int row = e / kChunk, c = e % kChunk;
        const int64_t rs = tile / chunks;
        const int kc = (int)(tile % chunks);
        const int64_t v = rs * kRows + row;
        const __nv_bfloat16 val = v < vocab ? w[v * hidden + kc * kChunk + c] : __float2bfloat16_rn(0.0f);
        *reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint8_t*>(tiles) + tile * kATile + tile_off(row, c, kChunk)) = val;
    }
}

// RMSNorm of up to 64 tokens, split into bf16 hi | lo, laid out as the B tiles of every k-chunk
// f16: the pieces are IEEE halves (hi + lo = 11 + 11 significand bits; a lo piece below 6e-5 is subnormal and
// keeps an absolute accuracy of 2^-25) to match weights stored as halves; otherwise bf16 (8 + 8 bits).
__global__ void __launch_bounds__(256) lm_prep_kernel(const float* __restrict__ h, const float* __restrict__ norm_w,
                                                      float eps, int hidden, int m, uint8_t* __restrict__ btiles, bool f16) {
    __shared__ double red[32];
    const int token = blockIdx.x;  // 0..63
    const bool real = token < m;
    const float* hr = h + (int64_t)(real ? token : 0) * hidden;
    double ss = 0.0;
    if (real)
        for (int c = threadIdx.x; c < hidden; c += blockDim.x) ss = fma((double)hr[c], (double)hr[c], ss);
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    ss = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) ss += red[w];
    const float denom = sqrtf(__fadd_rn((float)(ss / (double)hidden), eps));
    for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
        const float v = real ? __fmul_rn(__fdiv_rn(hr[c], denom), norm_w[c]) : 0.0f;
        uint8_t* tile = btiles + (int64_t)(c / kChunk) * kBTile;
        if (f16) {
            const __half hi = __float2half_rn(v);
            const __half lo = __float2half_rn(v - __half2float(hi));
            *reinterpret_cast<__half*>(tile + tile_off(token, c % kChunk, kChunk)) = hi;
            *reinterpret_cast<__half*>(tile + tile_off(kTok + token, c % kChunk, kChunk)) = lo;
        } else {
            const __nv_bfloat16 hi = __float2bfloat16_rn(v);
            const __nv_bfloat16 lo = __float2bfloat16_rn(v - __bfloat162float(hi));
            *reinterpret_cast<__nv_bfloat16*>(tile + tile_off(token, c % kChunk, kChunk)) = hi;
            *reinterpret_cast<__nv_bfloat16*>(tile + tile_off(kTok + token, c % kChunk, kChunk)) = lo;
        }
    }
}

__global__ void __launch_bounds__(kThreads, 1) lm_head_tc_kernel(const uint8_t* __restrict__ wtiles,
                                                                 const uint8_t* __restrict__ btiles, int64_t vocab,
                                                                 int hidden, int m, float* __restrict__ logits,
                                                                 unsigned int* err, bool w_f16) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* stage_base = smem;  // kStages x (A tile | B tile)
    uint64_t* full = reinterpret_cast<uint64_t*>(stage_base + (size_t)kStages * (kATile + kBTile));
    uint64_t* empty = full + kStages;
    uint64_t* acc_full = empty + kStages;
    uint64_t* acc_empty = acc_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int chunks = hidden / kChunk;
    const int64_t row_sets = (vocab + kRows - 1) / kRows;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { ptx::mbar_init(&full[s], 1); ptx::mbar_init(&empty[s], 1); }
        ptx::mbar_init(acc_full, 1);
        ptx::mbar_init(acc_empty, 128);
        ptx::mbar_fence_init();
    }
    if (warp == 1) { ptx::tmem_alloc(tmem_slot, kCols); ptx::tmem_relinquish(); }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            int slot = 0; uint32_t par = 1; bool first = true;
            for (int64_t rs = blockIdx.x; rs < row_sets; rs += gridDim.x)
                for (int kc = 0; kc < chunks; ++kc) {
                    if (!first) ok &= ptx::mbar_wait_bounded(&empty[slot], par);
                    uint8_t* st = stage_base + (size_t)slot * (kATile + kBTile);
                    ptx::mbar_arrive_expect_tx(&full[slot], kATile + kBTile);
                    ptx::bulk_g2s(st, wtiles + (rs * chunks + kc) * (int64_t)kATile, kATile, &full[slot]);
                    ptx::bulk_g2s(st + kATile, btiles + (int64_t)kc * kBTile, kBTile, &full[slot]);
                    if (++slot == kStages) { slot = 0; first = false; par ^= 1; }
                }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = instr_desc_bf16(kRows, kCols, w_f16);
            int slot = 0; uint32_t par = 0, acc_par = 0; bool first_tile = true;
            for (int64_t rs = blockIdx.x; rs < row_sets; rs += gridDim.x) {
                if (!first_tile) { ok &= ptx::mbar_wait_bounded(acc_empty, acc_par); acc_par ^= 1; }
                first_tile = false;
                ptx::tc_fence_after();
                for (int kc = 0; kc < chunks; ++kc) {
                    ok &= ptx::mbar_wait_bounded(&full[slot], par);
                    ptx::tc_fence_after();
                    const uint32_t a_addr = ptx::smem_u32(stage_base + (size_t)slot * (kATile + kBTile));
                    const uint32_t b_addr = a_addr + kATile;
#pragma unroll
                    for (int ks = 0; ks < kChunk / 16; ++ks) {  // K = 16 bf16 = 2 core matrices per MMA
                        const uint64_t ad = ptx::smem_desc(a_addr + ks * 256, 128, (kChunk / 8) * 128);
                        const uint64_t bd = ptx::smem_desc(b_addr + ks * 256, 128, (kChunk / 8) * 128);
                        ptx::umma_f16(tmem_base, ad, bd, idesc, (kc > 0 || ks > 0) ? 1u : 0u);
                    }
                    ptx::umma_commit(&empty[slot]);
                    if (++slot == kStages) { slot = 0; par ^= 1; }
                }
                ptx::umma_commit(acc_full);
            }
        }
    } else {
        const int sub = warp & 3;
        uint32_t acc_par = 0;
        for (int64_t rs = blockIdx.x; rs < row_sets; rs += gridDim.x) {
            ok &= ptx::mbar_wait_bounded(acc_full, acc_par);
            acc_par ^= 1;
            ptx::tc_fence_after();
            const int64_t v = rs * kRows + sub * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < kTok; c0 += 32) {
                uint32_t hi[32], lo[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(sub * 32) << 16) + c0;
                ptx::tmem_ld32(taddr, hi);
                ptx::tmem_ld32(taddr + kTok, lo);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int token = c0 + j;
                    if (token < m && v < vocab)
                        logits[(int64_t)token * vocab + v] = __fadd_rn(__uint_as_float(hi[j]), __uint_as_float(lo[j]));
                }
            }
            ptx::tc_fence_before();
            ptx::mbar_arrive(acc_empty);
        }
    }
    if (!ok) atomicExch(err, kErrLmTimeout);
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) ptx::tmem_dealloc(tmem_base, kCols);
}

}  // namespace

size_t lm_head_tc_weight_bytes(int64_t vocab, int hidden) {
    return (size_t)((vocab + kRows - 1) / kRows) * (hidden / kChunk) * kATile;
}
size_t lm_head_tc_act_bytes(int hidden) { return (size_t)(hidden / kChunk) * kBTile; }

cudaError_t launch_lm_retile(const __nv_bfloat16* w, int64_t vocab, int hidden, void* tiles, cudaStream_t stream) {
    if (hidden % kChunk != 0) return cudaErrorInvalidValue;
    lm_retile_kernel<<<1184, 256, 0, stream>>>(w, vocab, hidden, reinterpret_cast<__nv_bfloat16*>(tiles));
    return cudaGetLastError();
}

// logits for up to 64 tokens per pass; h: [batch, hidden] residual stream (RMSNorm applied here)
cudaError_t launch_lm_head_tc(const void* wtiles, const float* h, const float* norm_w, float eps, int batch, int hidden,
                              int64_t vocab, void* btiles, float* logits, unsigned int* err, int sm_count,
                              cudaStream_t stream, bool w_f16) {
    if (hidden % kChunk != 0) return cudaErrorInvalidValue;
    const size_t smem = (size_t)kStages * (kATile + kBTile) + 256;
    static PerDeviceOnce once;
    cudaError_t ce = once.run([smem] { return cudaFuncSetAttribute(lm_head_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); });
    if (ce != cudaSuccess) return ce;
    const int64_t row_sets = (vocab + kRows - 1) / kRows;
    const int grid = (int)(row_sets < sm_count ? row_sets : sm_count);
    for (int b0 = 0; b0 < batch; b0 += kTok) {
        const int bc = batch - b0 < kTok ? batch - b0 : kTok;
        lm_prep_kernel<<<kTok, 256, 0, stream>>>(h + (size_t)b0 * hidden, norm_w, eps, hidden, bc,
                                                 reinterpret_cast<uint8_t*>(btiles), w_f16);
        lm_head_tc_kernel<<<grid, kThreads, smem, stream>>>(reinterpret_cast<const uint8_t*>(wtiles),
                                                           reinterpret_cast<const uint8_t*>(btiles), vocab, hidden, bc,
                                                           logits + (size_t)b0 * vocab, err, w_f16);
    }
    return cudaGetLastError();
}

}  // namespace bt
