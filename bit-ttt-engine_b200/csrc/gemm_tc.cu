// Batched / prefill ternary product on the 5th-generation tensor cores (tcgen05, TMEM):
//   acc[n, m] = sum_k t[n, k] * q[m, k]   for M > 8 tokens.
// Stands in for BitLinearCpu::forward / BitLinearCuda::forward (kernels/cpu.rs:17-127,
// kernels/cuda.rs:21-47) at batch and prefill sizes, where the reference runs a dense f32 GEMM
// on a host-unpacked weight.
//
// Roles inside one CTA (1 per SM, persistent over work units of 128 weight rows x NT tokens x a k range):
//   warp 0     producer: 1-D bulk copies of the packed weight tiles (8 x 1 KB per 256-input
//              chunk) and of the chunk's int8 activation block into a shared-memory ring;
//   warp 1     MMA issuer (one thread): tcgen05.mma.kind::i8 with the A operand (weights, u8) in
//              TENSOR MEMORY and the B operand (activations, s8) in shared memory, K-major without
//              swizzle; accumulators in tensor memory, two sets, so that the MMAs of the next unit
//              run while the previous one is drained;
//   warps 2-5  unpack: a thread owns one weight row (= one TMEM lane).  It loads the row's 64 packed
//              bytes of the chunk, isolates field r of every byte with a shift and an AND
//              (values 0, 1, 2 = ternary + 1) and writes the four residue planes with tcgen05.st
//              straight into tensor memory: the unpacked weights never pass through shared memory,
//              whose bandwidth the B operand and the ring need;
//   warps 6-9  epilogue: tcgen05.ld of a finished accumulator set, - sum_k q (the +1 offset), scales, store.
// A 2-bit field at position r of a byte multiplies the activations k = r (mod 4), hence the
// activations are stored residue-split: B_r[m, k'] = q[m, 4k' + r]; the four residue products of a
// chunk accumulate into the same accumulator.
#include "bt_common.cuh"
#include "bt_ptx.cuh"

namespace bt {

namespace {

constexpr int kRows = 128;               // weight rows per tile = UMMA M = TMEM lanes
constexpr int kChunkK = 256;             // inputs per k-chunk (one weight tile column)
constexpr int kRawBytes = 8 * kTileBytes;  // packed weights of a chunk: 8 row tiles x 1 KB
constexpr int kStages = 5;
constexpr int kABufs = 2;                // unpacked-A buffers in tensor memory
constexpr int kAChunkCols = 64;          // TMEM columns of one unpacked chunk: 4 residues x 64 bytes / 4
constexpr int kTcThreads = 10 * 32;
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
    constexpr uint32_t kAccCols = 2 * NT;                // two accumulator sets of NT columns
    constexpr uint32_t kTmemCols = (kAccCols + kABufs * kAChunkCols) <= 256 ? 256 : 512;
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* stage_base = smem;                                           // kStages x (raw | B)
    uint64_t* full = reinterpret_cast<uint64_t*>(stage_base + (size_t)kStages * kStageBytes);
    uint64_t* empty = full + kStages;     // a stage is free again: the MMAs that read its B block are done (1 arrival)
                                          // and the four unpack warps have read its weights (4 arrivals)
    uint64_t* a_full = empty + kStages;   // unpacked chunk in tensor memory (4 arrivals, one per unpack warp)
    uint64_t* a_empty = a_full + kABufs;  // the MMAs that read it are done
    uint64_t* acc_full = a_empty + kABufs;
    uint64_t* acc_empty = acc_full + 2;   // 4 arrivals, one per epilogue warp
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_tiles = (int)a.k_tiles;
    const int row_sets = (int)((a.row_tiles + 7) / 8);
    const int tok_blocks = (a.m + NT - 1) / NT;
    const int k_splits = a.k_splits;
    const int cps = (k_tiles + k_splits - 1) / k_splits;  // chunks per split (the host makes every split non-empty)
    const int n_units = row_sets * tok_blocks * k_splits;  // work units: (row set, token block, k split)

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { ptx::mbar_init(&full[s], 1); ptx::mbar_init(&empty[s], 5); }
        for (int u = 0; u < kABufs; ++u) { ptx::mbar_init(&a_full[u], 4); ptx::mbar_init(&a_empty[u], 1); }
        for (int s = 0; s < 2; ++s) { ptx::mbar_init(&acc_full[s], 1); ptx::mbar_init(&acc_empty[s], 4); }
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
    const uint32_t a_col0 = kAccCols;  // the unpacked-A buffers follow the accumulators

    bool ok = true;
    if (warp == 0) {
        // ---------------- producer ----------------
        if (lane == 0) {
            int g = 0;  // chunks issued so far
            for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x) {
                const int split = unit % k_splits, tile = unit / k_splits;
                const int rs = tile % row_sets, tb = tile / row_sets;
                const int kt0 = split * cps, kt1 = min(k_tiles, kt0 + cps);
                for (int kt = kt0; kt < kt1; ++kt, ++g) {
                    const int slot = g % kStages, use = g / kStages;
                    if (use > 0) ok &= ptx::mbar_wait_bounded(&empty[slot], (uint32_t)((use - 1) & 1));
                    uint8_t* st = stage_base + (size_t)slot * kStageBytes;
                    const int rts = min(8, (int)(a.row_tiles - (int64_t)rs * 8));
                    ptx::mbar_arrive_expect_tx(&full[slot], (uint32_t)(rts * kTileBytes + kBBytes));
                    for (int r8 = 0; r8 < rts; ++r8)
                        ptx::bulk_g2s(st + r8 * kTileBytes,
                                      a.tiles + (((int64_t)rs * 8 + r8) * k_tiles + kt) * kTileBytes, kTileBytes,
                                      &full[slot]);
                    ptx::bulk_g2s(st + kRawBytes, a.qtc + ((int64_t)tb * k_tiles + kt) * kBBytes, kBBytes, &full[slot]);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            const uint32_t idesc = instr_desc_i8(kRows, NT);
            int g = 0, tl = 0;
            for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x, ++tl) {
                const int split = unit % k_splits;
                const int kt0 = split * cps, kt1 = min(k_tiles, kt0 + cps);
                const int sel = tl & 1, acc_use = tl >> 1;
                if (acc_use > 0) ok &= ptx::mbar_wait_bounded(&acc_empty[sel], (uint32_t)((acc_use - 1) & 1));
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)sel * NT;
                for (int kt = kt0; kt < kt1; ++kt, ++g) {
                    const int slot = g % kStages, u = g % kABufs;
                    ok &= ptx::mbar_wait_bounded(&full[slot], (uint32_t)((g / kStages) & 1));   // activation block landed
                    ok &= ptx::mbar_wait_bounded(&a_full[u], (uint32_t)((g / kABufs) & 1));     // weights unpacked into tensor memory
                    ptx::tc_fence_after();
                    const uint32_t b_addr = ptx::smem_u32(stage_base + (size_t)slot * kStageBytes + kRawBytes);
                    const uint32_t a_tmem = tmem_base + a_col0 + (uint32_t)u * kAChunkCols;
#pragma unroll
                    for (int r = 0; r < 4; ++r) {
#pragma unroll
                        for (int ks = 0; ks < 2; ++ks) {  // 64 k' per residue = 2 x K32 = 2 x 8 TMEM columns
                            const uint64_t bd = ptx::smem_desc(b_addr + r * (NT * 64) + ks * 256, 128, 512);
                            ptx::umma_i8_ts(d_tmem, a_tmem + r * 16 + ks * 8, bd, idesc, (kt > kt0 || r > 0 || ks > 0) ? 1u : 0u);
                        }
                    }
                    ptx::umma_commit(&a_empty[u]);   // unpacked buffer reusable once these MMAs are done
                    ptx::umma_commit(&empty[slot]);  // and the stage's activation block
                }
                ptx::umma_commit(&acc_full[sel]);
            }
        }
    } else if (warp < 6) {
        // ---------------- unpack warps (4 warps = 128 threads, one weight row = one TMEM lane each) ----
        const int sub = warp & 3;                      // the TMEM lanes 32 sub .. 32 sub + 31 belong to this warp
        const int row = sub * 32 + lane;               // row inside the 128-row tile
        // this thread's row: row tile r8 = row/16, half = (row%16)/8, g = row%8; its 64 packed bytes of a chunk
        // are the four 16-byte pieces t = 0..3 at ((half*32 + g*4 + t) * 16) of the row tile
        const int r8 = row >> 4, half = (row >> 3) & 1, g8 = row & 7;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(sub * 32) << 16) + a_col0;
        int g = 0;
        for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x) {
            const int split = unit % k_splits, tile = unit / k_splits;
            const int rs = tile % row_sets;
            const int rts = min(8, (int)(a.row_tiles - (int64_t)rs * 8));
            const int kt0 = split * cps, kt1 = min(k_tiles, kt0 + cps);
            for (int kt = kt0; kt < kt1; ++kt, ++g) {
                const int slot = g % kStages, u = g % kABufs, a_use = g / kABufs;
                ok &= ptx::mbar_wait_bounded(&full[slot], (uint32_t)((g / kStages) & 1));
                const uint8_t* raw = stage_base + (size_t)slot * kStageBytes + r8 * kTileBytes + half * 512 + g8 * 64;
                uint4 w[4];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    w[t] = make_uint4(0x55555555u, 0x55555555u, 0x55555555u, 0x55555555u);  // weight 0 (rows beyond the matrix)
                    if (r8 < rts) w[t] = *reinterpret_cast<const uint4*>(raw + t * 16);
                }
                if (a_use > 0) ok &= ptx::mbar_wait_bounded(&a_empty[u], (uint32_t)((a_use - 1) & 1));
                ptx::tc_fence_after();
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    // residue r of the row: piece t holds the inputs 64 t .. 64 t + 63, i.e. k' = 16 t .. 16 t + 15
                    uint32_t v[16];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        v[4 * t + 0] = (w[t].x >> (2 * r)) & 0x03030303u;
                        v[4 * t + 1] = (w[t].y >> (2 * r)) & 0x03030303u;
                        v[4 * t + 2] = (w[t].z >> (2 * r)) & 0x03030303u;
                        v[4 * t + 3] = (w[t].w >> (2 * r)) & 0x03030303u;
                    }
                    ptx::tmem_st16(lane_addr + (uint32_t)u * kAChunkCols + r * 16, v);
                }
                ptx::tmem_st_wait();
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(&a_full[u]);
                    ptx::mbar_arrive(&empty[slot]);  // this warp has read its weights of the stage
                }
            }
        }
    } else {
        // ---------------- epilogue warps (4 warps, TMEM lanes by warp % 4) ----------------
        const int sub = warp & 3;
        int tl = 0;
        for (int unit = blockIdx.x; unit < n_units; unit += gridDim.x, ++tl) {
            const int split = unit % k_splits, tile = unit / k_splits;
            const int rs = tile % row_sets, tb = tile / row_sets;
            const int sel = tl & 1;
            ok &= ptx::mbar_wait_bounded(&acc_full[sel], (uint32_t)((tl >> 1) & 1));
            ptx::tc_fence_after();
            const int64_t row = (int64_t)rs * kRows + sub * 32 + lane;
            const int64_t rt = row >> 4;
            float sw = 0.f;
            if (a.epilogue != EPI_I32 && rt < a.row_tiles) sw = a.sw_tiles[2 * rt + ((row >> 3) & 1)];
#pragma unroll 1
            for (int c0 = 0; c0 < NT; c0 += 32) {
                uint32_t d[32];
                ptx::tmem_ld32(tmem_base + ((uint32_t)(sub * 32) << 16) + (uint32_t)sel * NT + c0, d);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int token = tb * NT + c0 + j;
                    if (token < a.m && row < a.n_out) {
                        if (k_splits > 1) {
                            a.part[((int64_t)split * a.m + token) * a.n_out + row] = (int)d[j];
                            continue;
                        }
                        const int accv = (int)d[j] - a.qsum[token];
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
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&acc_empty[sel]);
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
    const size_t smem = (size_t)kStages * (kRawBytes + kBBytes) + 256;
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
