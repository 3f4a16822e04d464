// Batched / prefill ternary product on the 5th-generation tensor cores (tcgen05, TMEM):
//   acc[n, m] = sum_k t[n, k] * q[m, k]   for M > 8 tokens.
// Stands in for BitLinearCpu::forward / BitLinearCuda::forward (kernels/cpu.rs:17-127,
// kernels/cuda.rs:21-47) at batch and prefill sizes, where the reference runs a dense f32 GEMM
// on a host-unpacked weight.
//
// Roles inside one CTA (1 per SM, persistent over output tiles of 128 weight rows x NT tokens):
//   warp 0     producer: 1-D bulk copies of the packed weight tiles (8 x 1 KB per 256-input
//              chunk) and of the chunk's int8 activation block into a shared-memory ring;
//   warp 1     MMA issuer (one thread): tcgen05.mma.kind::i8, A = weights (u8), B = activations
//              (s8), both K-major without swizzle, accumulators in TMEM;
//   warps 2-5  unpack: one AND per 16-byte register isolates field r of every byte as an
//              unsigned multiple of 4^r and one 16-byte store puts it into the A tile of
//              residue r, so the four field positions become four independent products
//              with four TMEM accumulators (shifted back in the epilogue); the same warps
//              read TMEM (tcgen05.ld) and store the outputs at the end of a tile.
// A 2-bit field at position r of a byte multiplies the activations k = r (mod 4), hence the
// activations are stored residue-split: B_r[m, k'] = q[m, 4k' + r].
#include "bt_common.cuh"
#include "bt_ptx.cuh"

namespace bt {

namespace {

constexpr int kRows = 128;               // weight rows per tile = UMMA M
constexpr int kChunkK = 256;             // inputs per k-chunk (one weight tile column)
constexpr int kRawBytes = 8 * kTileBytes;  // packed weights of a chunk: 8 row tiles x 1 KB
constexpr int kATileBytes = kRows * 64;  // unpacked A of one residue: 128 rows x 64 k'
constexpr int kStages = 3;
constexpr int kUnpBufs = 2;
constexpr int kTcThreads = 6 * 32;
constexpr unsigned kErrTcTimeout = 0x54434d4du;  // 'TCMM'

// Instruction descriptor for kind::i8: D = s32, A = u8, B = s8, both K-major, M x N tile.
__device__ __forceinline__ uint32_t instr_desc_i8(int m, int n) {
    uint32_t d = 0;
    d |= 2u << 4;                    // accumulator format: s32
    d |= 0u << 7;                    // A format: unsigned 8-bit
    d |= 1u << 10;                   // B format: signed 8-bit
    d |= (uint32_t)(n >> 3) << 17;   // N / 8
    d |= (uint32_t)(m >> 4) << 24;   // M / 16
    return d;
}

struct TcArgs {
    const uint8_t* tiles;      // one basis, tiled layout [row_tile][k_tile][1024]
    int64_t row_tiles, k_tiles, n_out;
    const int8_t* qtc;         // activations: [token_block][k_tile][4 residues][NT/8][4][8][16]
    const int32_t* qsum;       // [m]
    const float* sx;           // [m]
    const float* sw_tiles;     // [row_tiles][2]
    int m;                     // tokens
    void* out;                 // [m, out_stride]
    int64_t out_stride;
    int epilogue;              // EPI_I32 / EPI_F32 / EPI_F32_ACCUM / EPI_BF16
    unsigned int* err;
    // With few output tiles (small N and M) the k range of a tile is cut into k_splits pieces
    // that different CTAs work on; each piece leaves its raw int32 sums in part[split][token][row]
    // and tc_finish_kernel adds them (integers: the result does not depend on the cut).
    int k_splits;
    int32_t* part;
};

template <int NT>
__global__ void __launch_bounds__(kTcThreads, 1) gemm_tc_kernel(TcArgs a) {
    constexpr int kBBytes = 4 * NT * 64;                 // activation block of a chunk (4 residues)
    constexpr int kStageBytes = kRawBytes + kBBytes;
    constexpr uint32_t kTmemCols = 4 * NT;               // four accumulators of NT columns
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* stage_base = smem;                                           // kStages x (raw | B)
    uint8_t* unp_base = stage_base + (size_t)kStages * kStageBytes;       // kUnpBufs x 4 x A tile
    uint64_t* full = reinterpret_cast<uint64_t*>(unp_base + (size_t)kUnpBufs * 4 * kATileBytes);
    uint64_t* empty = full + kStages;
    uint64_t* unp_full = empty + kStages;
    uint64_t* unp_empty = unp_full + kUnpBufs;
    uint64_t* acc_full = unp_empty + kUnpBufs;
    uint64_t* acc_empty = acc_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_tiles = (int)a.k_tiles;
    const int row_sets = (int)((a.row_tiles + 7) / 8);
    const int tok_blocks = (a.m + NT - 1) / NT;
    const int k_splits = a.k_splits;
    const int cps = (k_tiles + k_splits - 1) / k_splits;  // chunks per split (the host makes every split non-empty)
    const int n_tiles = row_sets * tok_blocks * k_splits;  // work units: (row set, token block, k split)

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { ptx::mbar_init(&full[s], 1); ptx::mbar_init(&empty[s], 1); }
        for (int u = 0; u < kUnpBufs; ++u) { ptx::mbar_init(&unp_full[u], 128); ptx::mbar_init(&unp_empty[u], 1); }
        ptx::mbar_init(acc_full, 1);
        ptx::mbar_init(acc_empty, 128);
        ptx::mbar_fence_init();
    }
    if (warp == 1) {  // one warp allocates (and later frees) the tensor memory
        ptx::tmem_alloc(tmem_slot, kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    bool ok = true;
    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            int slot = 0;
            uint32_t par = 1;
            bool first = true;
            for (int unit = blockIdx.x; unit < n_tiles; unit += gridDim.x) {
                const int split = unit % k_splits, tile = unit / k_splits;
                const int rs = tile % row_sets, tb = tile / row_sets;
                const int kt0 = split * cps, kt1 = min(k_tiles, kt0 + cps);
                for (int kt = kt0; kt < kt1; ++kt) {
                    if (!first) ok &= ptx::mbar_wait_bounded(&empty[slot], par);
                    uint8_t* st = stage_base + (size_t)slot * kStageBytes;
                    const int rts = min(8, (int)(a.row_tiles - (int64_t)rs * 8));
                    ptx::mbar_arrive_expect_tx(&full[slot], (uint32_t)(rts * kTileBytes + kBBytes));
                    for (int r8 = 0; r8 < rts; ++r8)
                        ptx::bulk_g2s(st + r8 * kTileBytes,
                                      a.tiles + (((int64_t)rs * 8 + r8) * k_tiles + kt) * kTileBytes, kTileBytes,
                                      &full[slot]);
                    ptx::bulk_g2s(st + kRawBytes, a.qtc + ((int64_t)tb * k_tiles + kt) * kBBytes, kBBytes, &full[slot]);
                    if (++slot == kStages) { slot = 0; first = false; par ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = instr_desc_i8(kRows, NT);
            int slot = 0, u = 0;
            uint32_t par = 0, upar = 0, acc_par = 0;
            bool first_tile = true;
            for (int unit = blockIdx.x; unit < n_tiles; unit += gridDim.x) {
                const int split = unit % k_splits;
                const int kt0 = split * cps, kt1 = min(k_tiles, kt0 + cps);
                if (!first_tile) { ok &= ptx::mbar_wait_bounded(acc_empty, acc_par); acc_par ^= 1; }
                first_tile = false;
                ptx::tc_fence_after();
                for (int kt = kt0; kt < kt1; ++kt) {
                    ok &= ptx::mbar_wait_bounded(&full[slot], par);        // activation block landed
                    ok &= ptx::mbar_wait_bounded(&unp_full[u], upar);      // weights unpacked
                    ptx::tc_fence_after();
                    const uint32_t b_addr = ptx::smem_u32(stage_base + (size_t)slot * kStageBytes + kRawBytes);
                    const uint32_t a_addr = ptx::smem_u32(unp_base + (size_t)u * 4 * kATileBytes);
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
#pragma unroll
                        for (int ks = 0; ks < 2; ++ks) {  // 64 k' per residue = 2 x K32
                            const uint64_t ad = ptx::smem_desc(a_addr + r * kATileBytes + ks * 256, 128, 512);
                            const uint64_t bd = ptx::smem_desc(b_addr + r * (NT * 64) + ks * 256, 128, 512);
                            ptx::umma_i8(tmem_base + r * NT, ad, bd, idesc, (kt > kt0 || ks > 0) ? 1u : 0u);
                        }
                    }
                    ptx::umma_commit(&unp_empty[u]);  // unpacked buffer reusable once these MMAs are done
                    ptx::umma_commit(&empty[slot]);   // and the stage (its activation block)
                    if (++slot == kStages) { slot = 0; par ^= 1; }
                    if (++u == kUnpBufs) { u = 0; upar ^= 1; }
                }
                ptx::umma_commit(acc_full);
            }
        }
    } else {
        // ---------------- unpack + epilogue warps (4 warps = 128 threads, one weight row each) ----
        const int tid = threadIdx.x - 64;              // 0..127 = row inside the tile
        const int sub = warp & 3;                      // TMEM sub-partition this warp may read
        int slot = 0, u = 0;
        uint32_t par = 0, upar = 1, acc_par = 0;
        bool first_unp = true;
        for (int unit = blockIdx.x; unit < n_tiles; unit += gridDim.x) {
            const int split = unit % k_splits, tile = unit / k_splits;
            const int rs = tile % row_sets, tb = tile / row_sets;
            const int rts = min(8, (int)(a.row_tiles - (int64_t)rs * 8));
            const int kt0 = split * cps, kt1 = min(k_tiles, kt0 + cps);
            for (int kt = kt0; kt < kt1; ++kt) {
                ok &= ptx::mbar_wait_bounded(&full[slot], par);
                if (!first_unp) ok &= ptx::mbar_wait_bounded(&unp_empty[u], upar);
                // this thread's row: row tile r8 = tid/16, half = (tid%16)/8, g = tid%8; its 64 packed
                // bytes are the four 16-byte chunks t = 0..3 at ((half*32 + g*4 + t) * 16)
                const int r8 = tid >> 4, half = (tid >> 3) & 1, g = tid & 7;
                const uint8_t* raw = stage_base + (size_t)slot * kStageBytes + r8 * kTileBytes + half * 512 + g * 64;
                uint8_t* dst = unp_base + (size_t)u * 4 * kATileBytes + (tid >> 3) * 512 + (tid & 7) * 16;
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    uint4 w = make_uint4(0x55555555u, 0x55555555u, 0x55555555u, 0x55555555u);  // weight 0
                    if (r8 < rts) w = *reinterpret_cast<const uint4*>(raw + t * 16);
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
                        const uint32_t mask = 0x03030303u << (2 * r);
                        *reinterpret_cast<uint4*>(dst + r * kATileBytes + t * 128) =
                            make_uint4(w.x & mask, w.y & mask, w.z & mask, w.w & mask);
                    }
                }
                ptx::fence_async_smem();  // generic-proxy stores -> visible to the tensor core's reads
                ptx::mbar_arrive(&unp_full[u]);
                if (++slot == kStages) { slot = 0; par ^= 1; }
                if (++u == kUnpBufs) { u = 0; first_unp = false; upar ^= 1; }
            }
            // ---- epilogue of this tile ----
            ok &= ptx::mbar_wait_bounded(acc_full, acc_par);
            acc_par ^= 1;
            ptx::tc_fence_after();
            const int64_t row = (int64_t)rs * kRows + sub * 32 + lane;
            const int64_t rt = row >> 4;
            float sw = 0.f;
            if (a.epilogue != EPI_I32 && rt < a.row_tiles) sw = a.sw_tiles[2 * rt + ((row >> 3) & 1)];
#pragma unroll 1
            for (int c0 = 0; c0 < NT; c0 += 32) {
                uint32_t d0[32], d1[32], d2[32], d3[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(sub * 32) << 16) + c0;
                ptx::tmem_ld32(taddr + 0 * NT, d0);
                ptx::tmem_ld32(taddr + 1 * NT, d1);
                ptx::tmem_ld32(taddr + 2 * NT, d2);
                ptx::tmem_ld32(taddr + 3 * NT, d3);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int token = tb * NT + c0 + j;
                    if (token < a.m && row < a.n_out) {
                        const int folded = (int)d0[j] + ((int)d1[j] >> 2) + ((int)d2[j] >> 4) + ((int)d3[j] >> 6);
                        if (k_splits > 1) {
                            a.part[((int64_t)split * a.m + token) * a.n_out + row] = folded;
                            continue;
                        }
                        const int accv = folded - a.qsum[token];
                        const int64_t o = (int64_t)token * a.out_stride + row;
                        if (a.epilogue == EPI_I32) {
                            reinterpret_cast<int32_t*>(a.out)[o] = accv;
                        } else {
                            const float y = __fmul_rn(__fmul_rn((float)accv, sw), a.sx[token]);
                            if (a.epilogue == EPI_F32) reinterpret_cast<float*>(a.out)[o] = y;
                            else if (a.epilogue == EPI_F32_ACCUM)
                                reinterpret_cast<float*>(a.out)[o] = __fadd_rn(reinterpret_cast<float*>(a.out)[o], y);
                            else reinterpret_cast<__nv_bfloat16*>(a.out)[o] = __float2bfloat16_rn(y);
                        }
                    }
                }
            }
            ptx::tc_fence_before();
            ptx::mbar_arrive(acc_empty);
        }
    }
    if (!ok) atomicExch(a.err, kErrTcTimeout);
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) ptx::tmem_dealloc(tmem_base, kTmemCols);
}

// Per-token absmax int8 quantiser writing the residue-split, core-matrix-ordered layout that
// gemm_tc_kernel copies in bulk: [token_block][k_tile][residue][token_group][kc][token%8][16].
__device__ __forceinline__ float load_act(const float* p) { return *p; }
__device__ __forceinline__ float load_act(const __nv_bfloat16* p) { return __bfloat162float(*p); }

template <int NT, typename T>
__global__ void __launch_bounds__(256) act_quant_tc_kernel(const T* __restrict__ x, int64_t x_stride, int k,
                                                           int k_tiles, int m, int8_t* __restrict__ qtc,
                                                           float* __restrict__ s_out, int32_t* __restrict__ qsum_out) {
    __shared__ float red_f[32];
    __shared__ int red_i[32];
    const int token = blockIdx.x;  // grid covers the padded token count
    const int tb = token / NT, tin = token % NT;
    int8_t* blk = qtc + (int64_t)tb * k_tiles * (4 * NT * 64);
    const bool real = token < m;
    const T* xr = x + (int64_t)(real ? token : 0) * x_stride;
    float amax = 0.0f;
    if (real)
        for (int c = threadIdx.x; c < k; c += blockDim.x) amax = fmaxf(amax, fabsf(load_act(xr + c)));
    // block max
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if ((threadIdx.x & 31) == 0) red_f[threadIdx.x >> 5] = amax;
    __syncthreads();
    amax = 0.0f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) amax = fmaxf(amax, red_f[w]);
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    int local = 0;
    const int k_pad = k_tiles * kChunkK;
    for (int c = threadIdx.x; c < k_pad; c += blockDim.x) {
        int qv = 0;
        if (real && c < k) qv = max(-127, min(127, ptx::round_half_away(__fmul_rn(load_act(xr + c), inv))));
        local += qv;
        blk[gemm_tc_act_offset(c, tin, NT)] = (int8_t)qv;
    }
    for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
    if ((threadIdx.x & 31) == 0) red_i[threadIdx.x >> 5] = local;
    __syncthreads();
    if (threadIdx.x == 0 && real) {
        int tot = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red_i[w];
        s_out[token] = __fdiv_rn(amax, 127.0f);
        qsum_out[token] = tot;
    }
}

// Fewer tiles than half the SMs: cut k so that one wave of CTAs covers the product.
int tc_k_splits(int n_tiles, int64_t k_tiles, int sm_count) {
    if (n_tiles * 2 > sm_count || k_tiles < 4) return 1;
    int want = sm_count / n_tiles;
    if (want > k_tiles / 2) want = (int)(k_tiles / 2);
    const int cps = (int)((k_tiles + want - 1) / want);
    return (int)((k_tiles + cps - 1) / cps);
}

// Adds the k-split pieces of a product and applies the epilogue: one thread per (token, row).
__global__ void __launch_bounds__(256) tc_finish_kernel(TcArgs a) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (int64_t)a.m * a.n_out) return;
    const int token = (int)(idx / a.n_out);
    const int64_t row = idx % a.n_out;
    int accv = -a.qsum[token];
    for (int s2 = 0; s2 < a.k_splits; ++s2) accv += a.part[((int64_t)s2 * a.m + token) * a.n_out + row];
    const int64_t o = (int64_t)token * a.out_stride + row;
    if (a.epilogue == EPI_I32) {
        reinterpret_cast<int32_t*>(a.out)[o] = accv;
        return;
    }
    const float sw = a.sw_tiles[2 * (row >> 4) + ((row >> 3) & 1)];
    const float y = __fmul_rn(__fmul_rn((float)accv, sw), a.sx[token]);
    if (a.epilogue == EPI_F32) reinterpret_cast<float*>(a.out)[o] = y;
    else if (a.epilogue == EPI_F32_ACCUM) reinterpret_cast<float*>(a.out)[o] = __fadd_rn(reinterpret_cast<float*>(a.out)[o], y);
    else reinterpret_cast<__nv_bfloat16*>(a.out)[o] = __float2bfloat16_rn(y);
}

template <int NT>
cudaError_t launch_nt(TcArgs a, int sm_count, int32_t* part, size_t part_bytes, cudaStream_t stream) {
    constexpr int kBBytes = 4 * NT * 64;
    const size_t smem = (size_t)kStages * (kRawBytes + kBBytes) + (size_t)kUnpBufs * 4 * kATileBytes + 256;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        configured = true;
    }
    const int row_sets = (int)((a.row_tiles + 7) / 8);
    const int n_tiles = row_sets * ((a.m + NT - 1) / NT);
    int splits = part ? tc_k_splits(n_tiles, a.k_tiles, sm_count) : 1;
    if ((size_t)splits * a.m * a.n_out * sizeof(int32_t) > part_bytes) splits = 1;
    a.k_splits = splits;
    a.part = splits > 1 ? part : nullptr;
    const int units = n_tiles * splits;
    const int grid = units < sm_count ? units : sm_count;
    gemm_tc_kernel<NT><<<grid, kTcThreads, smem, stream>>>(a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || splits == 1) return e;
    const int64_t total = (int64_t)a.m * a.n_out;
    tc_finish_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace

size_t gemm_tc_part_bytes(int sm_count) {
    // pieces <= SMs / tiles and tokens x rows <= tiles x 128 x 128, hence pieces x tokens x rows <= SMs x 128 x 128
    return (size_t)sm_count * kRows * 128 * sizeof(int32_t);
}

int gemm_tc_kernels(const LinearDev& lin, int64_t m, int sm_count) {
    const int nt = m <= 64 ? 64 : 128;
    const int n_tiles = (int)((lin.w.row_tiles + 7) / 8) * (int)((m + nt - 1) / nt);
    return lin.w.n_bases * (tc_k_splits(n_tiles, lin.w.k_tiles, sm_count) > 1 ? 2 : 1);
}

size_t gemm_tc_act_bytes(int64_t m, int64_t k_tiles) {
    const int64_t nt = m <= 64 ? 64 : 128;
    return (size_t)((m + nt - 1) / nt * k_tiles * 4 * nt * 64);
}

cudaError_t launch_gemm_tc(const LinearDev& lin, const void* x, int64_t x_stride, int64_t m, int8_t* qtc, float* sx,
                           int32_t* qsum, void* out, int64_t out_stride, int epilogue, unsigned int* err, int sm_count,
                           cudaStream_t stream, int32_t* part, size_t part_bytes, bool prequantised, bt_dtype x_dtype) {
    if (lin.w.n_bases != 1 && epilogue == EPI_BF16) return cudaErrorInvalidValue;
    const int nt = m <= 64 ? 64 : 128;
    const int padded = (int)((m + nt - 1) / nt * nt);
    const int k = (int)lin.w.k_in, kts = (int)lin.w.k_tiles;
    if (prequantised) {
    } else if (x_dtype == BT_BF16) {
        const __nv_bfloat16* xb = reinterpret_cast<const __nv_bfloat16*>(x);
        if (nt == 64) act_quant_tc_kernel<64><<<padded, 256, 0, stream>>>(xb, x_stride, k, kts, (int)m, qtc, sx, qsum);
        else act_quant_tc_kernel<128><<<padded, 256, 0, stream>>>(xb, x_stride, k, kts, (int)m, qtc, sx, qsum);
    } else {
        const float* xf = reinterpret_cast<const float*>(x);
        if (nt == 64) act_quant_tc_kernel<64><<<padded, 256, 0, stream>>>(xf, x_stride, k, kts, (int)m, qtc, sx, qsum);
        else act_quant_tc_kernel<128><<<padded, 256, 0, stream>>>(xf, x_stride, k, kts, (int)m, qtc, sx, qsum);
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    for (int b = 0; b < lin.w.n_bases; ++b) {
        TcArgs a = {};
        a.tiles = lin.w.tiles + (size_t)b * lin.w.basis_stride();
        a.row_tiles = lin.w.row_tiles;
        a.k_tiles = lin.w.k_tiles;
        a.n_out = lin.w.n_out;
        a.qtc = qtc;
        a.qsum = qsum;
        a.sx = sx;
        a.sw_tiles = lin.scale_tiles + (size_t)b * lin.w.row_tiles * 2;
        a.m = (int)m;
        a.out = out;
        a.out_stride = out_stride;
        a.epilogue = (b > 0 && epilogue == EPI_F32) ? EPI_F32_ACCUM : epilogue;
        a.err = err;
        e = nt == 64 ? launch_nt<64>(a, sm_count, part, part_bytes, stream) : launch_nt<128>(a, sm_count, part, part_bytes, stream);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace bt
