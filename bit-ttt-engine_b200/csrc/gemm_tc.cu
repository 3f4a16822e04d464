// Batched / prefill ternary product on the 5th-generation tensor cores (tcgen05, TMEM):
//   acc[n, m] = sum_k t[n, k] * q[m, k]   for M > 8 tokens.
// Stands in for BitLinearCpu::forward / BitLinearCuda::forward (kernels/cpu.rs:17-127,
// kernels/cuda.rs:21-47) at batch and prefill sizes, where the reference runs a dense f32 GEMM
// on a host-unpacked weight.
//
// Roles inside one CTA (1 per SM, persistent over work units of RS x 128 weight rows x NT tokens x a k range;
// the RS = 1 or 2 row sets of a unit share every activation block):
//   warp 0     producer: 1-D bulk copies of the packed weight tiles (8 x 1 KB per 256-input
//              chunk) and of the chunk's int8 activation block into a shared-memory ring;
//   warp 1     MMA issuer (one thread): tcgen05.mma.kind::i8 with the A operand (weights, u8) in
//              TENSOR MEMORY and the B operand (activations, s8) in shared memory, K-major without
//              swizzle; accumulators in tensor memory, two sets, so that the MMAs of the next unit
//              run while the previous one is drained;
//   8 unpack warps: a thread owns one weight row (= one TMEM lane) of one row set (with one row set, two warps per
//              lane quarter take the chunks in turn).  It loads the row's 64
//              packed bytes of the chunk, isolates field r of every byte with a shift and an AND (values 0, 1, 2 =
//              ternary + 1) and writes the four residue planes with tcgen05.st straight into tensor memory:
//              the unpacked weights never pass through shared memory, whose bandwidth the B operand and the ring need;
//   4 RS epilogue warps: tcgen05.ld of a finished accumulator set, - sum_k q (the +1 offset), scales, store.
// With few output tiles the k range of a tile is cut over the CTAs of a thread-block cluster; their int32
// partial sums reach the cluster's first CTA through distributed shared memory, and that CTA alone stores.
// Every launch carries the programmatic-dependent-launch attribute: the producer requests the first weight
// tiles (which no kernel writes) before it waits for the kernel in front.
// A 2-bit field at position r of a byte multiplies the activations k = r (mod 4), hence the
// activations are stored residue-split: B_r[m, k'] = q[m, 4k' + r]; the four residue products of a
// chunk accumulate into the same accumulator.
#include <cstdint>
#include <mutex>
#include <type_traits>

#include "bt_common.cuh"
#include "bt_model.cuh"
#include "bt_ptx.cuh"

namespace bt {

namespace {

constexpr int kRows = 128;               // weight rows per MMA = UMMA M = TMEM lanes
constexpr int kSetBytes = 8 * kTileBytes;  // packed weights of 128 rows of a chunk: 8 row tiles x 1 KB
constexpr int kAChunkCols = 64;          // TMEM columns of one unpacked 128-row chunk: 4 residues x 64 bytes / 4
constexpr unsigned kErrTcTimeout = 0x54434d4du;  // 'TCMM'

// A tile is RS x 128 weight rows x NT tokens: the RS row sets share every activation block, which is what a CTA
// pulls most of through L2 (NT x 256 bytes per chunk against RS x 8 KB of packed weights).
// Warps: producer, MMA issuer, 8 unpack warps, 4 RS epilogue warps.  With two row sets two idle warps follow the MMA
// issuer, so that the roles fall on whole warpgroups (4 warps) and can trade registers (setmaxnreg).
__host__ __device__ constexpr int tc_lead_warps(int rs) { return rs == 2 ? 4 : 2; }
__host__ __device__ constexpr int tc_threads(int rs) { return (tc_lead_warps(rs) + 8 + 4 * rs) * 32; }
// Register split of the 128-token, two-row-set kernel: the epilogue warps hold a whole accumulator row (128 values) so
// that the single accumulator set is free again after four tensor-memory loads instead of after the stores.
constexpr int kRegsLead = 40, kRegsUnpack = 64, kRegsEpilogue = 152;
__host__ __device__ constexpr int tc_abufs(int rs) { return rs == 1 ? 4 : 2; }           // unpacked-A buffers in tensor memory
__host__ __device__ constexpr int tc_acc_sets(int nt, int rs) { return (2 * rs * nt + tc_abufs(rs) * rs * kAChunkCols <= 512) ? 2 : 1; }
__host__ __device__ constexpr int tc_stages(int nt, int rs, int s) {
    // ring depth that fits 227 KB next to the partial-sum buffer of a k split
    const int stage = rs * kSetBytes + 4 * nt * 64, part = s > 1 ? rs * kRows * nt * 4 : 0;
    const int n = (225 * 1024 - part) / stage;
    return n > 5 ? 5 : n;
}

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
};

// NT: tokens per tile (64 / 128).  RS: 128-row sets per tile (1 / 2).  S: CTAs of a cluster that share a tile
// along k (1: no cluster work at all).
template <int NT, int RS, int S>
__global__ void __launch_bounds__(tc_threads(RS), 1) gemm_tc_kernel(TcArgs a) {
    static_assert(S == 1 || (NT == 64 && (S == 2 || S == 4 || S == 8)), "k split: 64 tokens, 2 / 4 / 8 CTAs");
    // Eight unpack warps.  RS = 2: one per (row set, TMEM lane quarter).  RS = 1: two per lane quarter, which take
    // the chunks in turn (two independent chains of load - unpack - store, four A buffers).
    constexpr int kUnpackWarps = 8, kEpiWarps = 4 * RS, kUnpackWarp0 = tc_lead_warps(RS), kEpiWarp0 = kUnpackWarp0 + kUnpackWarps;
    constexpr bool kRegSplit = NT == 128 && RS == 2 && S == 1;
    constexpr int kABufs = tc_abufs(RS);
    constexpr int kReaders = RS == 1 ? 4 : 8;            // unpack warps that read one stage's weights and fill one A buffer
    constexpr int kStages = tc_stages(NT, RS, S);
    constexpr int kAccSets = tc_acc_sets(NT, RS);
    constexpr int kRawBytes = RS * kSetBytes;
    constexpr int kBBytes = 4 * NT * 64;                 // activation block of a chunk (4 residues)
    constexpr int kStageBytes = kRawBytes + kBBytes;
    constexpr int kPartBytes = S > 1 ? RS * kRows * NT * 4 : 0;  // this CTA's partial sums of a tile, read by the whole cluster
    constexpr uint32_t kAccCols = kAccSets * RS * NT;
    constexpr uint32_t kTmemCols = (kAccCols + kABufs * RS * kAChunkCols) <= 256 ? 256 : 512;
    static_assert(kAccCols + kABufs * RS * kAChunkCols <= 512, "tensor memory");
    static_assert(kStages >= 3, "ring");
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* stage_base = smem;                                           // kStages x (raw | B)
    int32_t* pbuf = reinterpret_cast<int32_t*>(stage_base + (size_t)kStages * kStageBytes);  // [RS][NT / 4][128 rows][4]
    uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(pbuf) + kPartBytes);
    uint64_t* empty = full + kStages;     // a stage is free again: the MMAs that read its B block are done (1 arrival)
                                          // and the unpack warps that take the chunk have read its weights
    uint64_t* a_full = empty + kStages;   // unpacked chunk in tensor memory (one arrival per unpack warp)
    uint64_t* a_empty = a_full + kABufs;  // the MMAs that read it are done
    uint64_t* acc_full = a_empty + kABufs;
    uint64_t* acc_empty = acc_full + 2;   // one arrival per epilogue warp
    uint64_t* red_full = acc_empty + 2;   // every CTA of the cluster has parked its partial sums of the tile
    uint64_t* red_free = red_full + 1;    // every CTA of the cluster has read this CTA's partial sums
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(red_free + 1);
    int* tok_qsum = reinterpret_cast<int*>(tmem_slot + 2);          // [2][NT] per-token sum of q and scale of the tile being drained
    float* tok_sx = reinterpret_cast<float*>(tok_qsum + 2 * NT);    // (two copies: the row sets' warps may be one tile apart)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k_tiles = (int)a.k_tiles;
    const int row_sets = (int)((a.row_tiles + 8 * RS - 1) / (8 * RS));   // tiles along the rows
    const int tok_blocks = (a.m + NT - 1) / NT;
    const int rank = S > 1 ? (int)ptx::cluster_ctarank() : 0;
    const int cid = blockIdx.x / S, n_clusters = gridDim.x / S;
    const int cps = (k_tiles + S - 1) / S;                 // chunks per split (the host makes every split non-empty)
    const int kt0 = rank * cps, kt1 = min(k_tiles, kt0 + cps);
    const int n_tiles = row_sets * tok_blocks;             // this CTA works on the tiles cid, cid + n_clusters, ...

    if (warp == 0) {  // the barriers side by side, a lane each (the set-up is on the path of every launch)
        if (lane < kStages) { ptx::mbar_init(&full[lane], 1); ptx::mbar_init(&empty[lane], 1 + kReaders); }
        if (lane >= 8 && lane < 8 + kABufs) { ptx::mbar_init(&a_full[lane - 8], kReaders); ptx::mbar_init(&a_empty[lane - 8], 1); }
        if (lane >= 16 && lane < 18) { ptx::mbar_init(&acc_full[lane - 16], 1); ptx::mbar_init(&acc_empty[lane - 16], kEpiWarps); }
        if (lane == 24) ptx::mbar_init(red_full, kEpiWarps * S);
        if (lane == 25) ptx::mbar_init(red_free, kEpiWarps * S);
        ptx::mbar_fence_init();
    }
    if (warp == 1) {  // one warp allocates (and later frees) the tensor memory
        ptx::tmem_alloc(tmem_slot, kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    // The peers' barriers must exist before anybody arrives on them.  Only the epilogue warps ever touch a peer, so
    // everybody reports here and only they wait (at the top of their role): the cluster's start-up skew stays off
    // the path of the first copies and MMAs.
    if (S > 1) asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t a_col0 = kAccCols;  // the unpacked-A buffers follow the accumulators: [buffer][row set][64]

    // With the register split every warpgroup states its share at the top of its branch (the host has checked that the
    // shares fit the register file the launch gives the CTA).
    bool ok = true;
    if (warp < kUnpackWarp0) {
    if constexpr (kRegSplit) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsLead));
    if (warp == 0) {
        // ---------------- producer (whole warp: lane r8 requests row tile r8 of a chunk, so that the small copies are
        //                  issued side by side; lane 0 also registers the byte count and requests the activation block) ----
        {
            // The weights do not depend on earlier kernels: the first stages' weight tiles are requested before the
            // dependency wait, their activation blocks (written by the quantiser just before) after it.
            auto issue = [&](int tile, int kt, int slot, bool raw_part, bool b_part) {
                const int rs = tile % row_sets, tb = tile / row_sets;
                uint8_t* st = stage_base + (size_t)slot * kStageBytes;
                const int rts = min(8 * RS, (int)(a.row_tiles - (int64_t)rs * 8 * RS));
                if (raw_part) {
                    if (lane == 0) ptx::mbar_arrive_expect_tx(&full[slot], (uint32_t)(rts * kTileBytes + kBBytes));
                    if (lane < rts)
                        ptx::bulk_g2s(st + lane * kTileBytes, a.tiles + (((int64_t)rs * 8 * RS + lane) * k_tiles + kt) * kTileBytes, kTileBytes,
                                      &full[slot]);
                }
                if (b_part && lane == 0) ptx::bulk_g2s(st + kRawBytes, a.qtc + ((int64_t)tb * k_tiles + kt) * kBBytes, kBBytes, &full[slot]);
            };
            int g = 0;
            for (int tile = cid; tile < n_tiles && g < kStages; tile += n_clusters)
                for (int kt = kt0; kt < kt1 && g < kStages; ++kt, ++g) issue(tile, kt, g, true, false);
            ptx::pdl_wait();
            g = 0;
            for (int tile = cid; tile < n_tiles; tile += n_clusters) {
                for (int kt = kt0; kt < kt1; ++kt, ++g) {
                    const int slot = g % kStages, use = g / kStages;
                    if (use == 0) { issue(tile, kt, slot, false, true); continue; }
                    ok &= ptx::mbar_wait_bounded(&empty[slot], (uint32_t)((use - 1) & 1));
                    issue(tile, kt, slot, true, true);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            ptx::pdl_wait();  // nothing to do before the first activation block exists; keeps the bounded waits short
            const uint32_t idesc = instr_desc_i8(kRows, NT);
            int g = 0, tl = 0;
            for (int tile = cid; tile < n_tiles; tile += n_clusters, ++tl) {
                const int sel = tl % kAccSets, acc_use = tl / kAccSets;
                if (acc_use > 0) ok &= ptx::mbar_wait_bounded(&acc_empty[sel], (uint32_t)((acc_use - 1) & 1));
                ptx::tc_fence_after();
                for (int kt = kt0; kt < kt1; ++kt, ++g) {
                    const int slot = g % kStages, u = g % kABufs;
                    // One wait per chunk: the unpack warps arrive on a_full after they have seen full[slot] complete, which
                    // covers the stage's activation block as well as its weights.  Every instruction between two MMAs
                    // of this thread costs tensor-pipe time (the queue behind it is short), hence the relaxed wait.
                    ok &= ptx::mbar_spin_relaxed(&a_full[u], (uint32_t)((g / kABufs) & 1));     // weights unpacked into tensor memory
                    ptx::tc_fence_after();
                    const uint32_t b_addr = ptx::smem_u32(stage_base + (size_t)slot * kStageBytes + kRawBytes);
#pragma unroll
                    for (int h = 0; h < RS; ++h) {
                        const uint32_t d_tmem = tmem_base + (uint32_t)(sel * RS + h) * NT;
                        const uint32_t a_tmem = tmem_base + a_col0 + (uint32_t)(u * RS + h) * kAChunkCols;
#pragma unroll
                        for (int r = 0; r < 4; ++r) {
#pragma unroll
                            for (int ks = 0; ks < 2; ++ks) {  // 64 k' per residue = 2 x K32 = 2 x 8 TMEM columns
                                const uint64_t bd = ptx::smem_desc(b_addr + r * (NT * 64) + ks * 256, 128, 512);
                                ptx::umma_i8_ts(d_tmem, a_tmem + r * 16 + ks * 8, bd, idesc, (kt > kt0 || r > 0 || ks > 0) ? 1u : 0u);
                            }
                        }
                    }
                    ptx::umma_commit(&a_empty[u]);   // unpacked buffer reusable once these MMAs are done
                    ptx::umma_commit(&empty[slot]);  // and the stage's activation block
                }
                ptx::umma_commit(&acc_full[sel]);
            }
            // every MMA of this CTA is issued: the kernel behind may start (it waits for this one's results itself)
            ptx::pdl_launch_dependents();
        }
    }
    } else if (warp < kEpiWarp0) {
        if constexpr (kRegSplit) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsUnpack));
        // ---------------- unpack warps: a thread owns one weight row (= one TMEM lane) of one row set ----
        const int sub = warp & 3;                      // the TMEM lanes 32 sub .. 32 sub + 31 belong to this warp
        const int set = (warp - kUnpackWarp0) >> 2;               // RS = 2: row set of the tile; RS = 1: which chunks (even / odd)
        const int h = RS == 2 ? set : 0;
        const int row = sub * 32 + lane;               // row inside the set
        // the row: row tile r8 = row/16, half = (row%16)/8, g = row%8; its 64 packed bytes of a chunk are the four
        // 16-byte pieces t = 0..3 at ((half*32 + g*4 + t) * 16) of the row tile
        const int r8 = h * 8 + (row >> 4), half = (row >> 3) & 1, g8 = row & 7;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(sub * 32) << 16) + a_col0 + (uint32_t)h * kAChunkCols;
        ptx::pdl_wait();
        int g = 0;
        int pending = -1;  // A buffer whose stores are issued but not yet published
        // The stores of a chunk are published (wait, fence, arrive) only after the next chunk's weights have been
        // loaded from shared memory, if those have landed already: the store latency hides behind the loads.
        auto publish = [&]() {
            if (pending < 0) return;
            ptx::tmem_st_wait();
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&a_full[pending]);
            pending = -1;
        };
        for (int tile = cid; tile < n_tiles; tile += n_clusters) {
            const int rs = tile % row_sets;
            const int rts = min(8 * RS, (int)(a.row_tiles - (int64_t)rs * 8 * RS));
            for (int kt = kt0; kt < kt1; ++kt, ++g) {
                if (RS == 1 && (g & 1) != set) continue;
                const int slot = g % kStages, u = g % kABufs, a_use = g / kABufs;
                const uint32_t full_parity = (uint32_t)((g / kStages) & 1);
                if (!__all_sync(0xffffffffu, ptx::mbar_test_wait(&full[slot], full_parity))) {  // (one answer for the whole warp)
                    publish();  // the next weights are not here yet: do not hold the finished buffer back
                    ok &= ptx::mbar_wait_bounded(&full[slot], full_parity);
                }
                const uint8_t* raw = stage_base + (size_t)slot * kStageBytes + r8 * kTileBytes + half * 512 + g8 * 64;
                uint4 w[4];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    w[t] = make_uint4(0x55555555u, 0x55555555u, 0x55555555u, 0x55555555u);  // weight 0 (rows beyond the matrix)
                    if (r8 < rts) w[t] = *reinterpret_cast<const uint4*>(raw + t * 16);
                }
                publish();
                if (a_use > 0) ok &= ptx::mbar_wait_bounded(&a_empty[u], (uint32_t)((a_use - 1) & 1));
                ptx::tc_fence_after();
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    // residue r: piece t holds the inputs 64 t .. 64 t + 63, i.e. k' = 16 t .. 16 t + 15 = columns 4 t .. 4 t + 3
                    uint32_t v[16];
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        v[4 * t + 0] = (w[t].x >> (2 * r)) & 0x03030303u;
                        v[4 * t + 1] = (w[t].y >> (2 * r)) & 0x03030303u;
                        v[4 * t + 2] = (w[t].z >> (2 * r)) & 0x03030303u;
                        v[4 * t + 3] = (w[t].w >> (2 * r)) & 0x03030303u;
                    }
                    ptx::tmem_st16(lane_addr + (uint32_t)(u * RS) * kAChunkCols + r * 16, v);
                }
                pending = u;
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&empty[slot]);  // this warp holds the stage's weights in registers
            }
        }
        publish();
    } else {
        if constexpr (kRegSplit) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsEpilogue));
        // ---------------- epilogue warps (4 per row set, TMEM lanes by warp % 4) ----------------
        const int sub = warp & 3;
        const int h = (warp - kEpiWarp0) >> 2;  // row set of the tile
        const int lrow = sub * 32 + lane;       // row inside the set
        int32_t* pb = pbuf + (size_t)h * (kRows * NT);
        if (S > 1) asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
        ptx::pdl_wait();  // the output (and what EPI_F32_ACCUM adds to) belongs to earlier kernels until here
        // The old value of an accumulated output is fetched apart from its update, so that a thread's loads are all
        // in flight before the first store (a store followed by a load of the same array would serialise them);
        // the per-token terms come through the read-only path for the same reason.
        // The epilogue kind is a compile-time constant of everything below (one copy of the role per kind, chosen once):
        // the unrolled store sequences are long, and a kind switch inside every element made them four times as long -
        // code that is fetched once per tile and does not stay in the instruction cache.
        auto epilogue_role = [&](auto kind) {
        constexpr int EPI = decltype(kind)::value;
        constexpr bool accum = EPI == EPI_F32_ACCUM;
        auto load_old = [&](int token, int64_t row) -> float {
            return (accum && token < a.m && row < a.n_out) ? reinterpret_cast<const float*>(a.out)[(int64_t)token * a.out_stride + row] : 0.0f;
        };
        // i = token inside the tile; tq / ts = the tile's staged per-token terms
        // tqi / tsi: the token's sum of q and scale (read from shared memory by the caller, ahead of its stores)
        auto store_v = [&](int tqi, float tsi, int tb, int i, int n_tok, int64_t row, float sw, uint32_t acc, float old) {
            if (i < n_tok && row < a.n_out) {
                const int accv = (int)acc - tqi;
                const int64_t o = (int64_t)(tb * NT + i) * a.out_stride + row;
                if constexpr (EPI == EPI_I32) {
                    reinterpret_cast<int32_t*>(a.out)[o] = accv;
                } else {
                    const float y = __fmul_rn(__fmul_rn((float)accv, sw), tsi);
                    if constexpr (EPI == EPI_F32) reinterpret_cast<float*>(a.out)[o] = y;
                    else if constexpr (accum) reinterpret_cast<float*>(a.out)[o] = __fadd_rn(old, y);
                    else reinterpret_cast<__nv_bfloat16*>(a.out)[o] = __float2bfloat16_rn(y);
                }
            }
        };
        auto store = [&](const int* tq, const float* ts, int tb, int i, int n_tok, int64_t row, float sw, uint32_t acc, float old) {
            store_v(tq[i], ts[i], tb, i, n_tok, row, sw, acc, old);
        };
        int tl = 0;
        for (int tile = cid; tile < n_tiles; tile += n_clusters, ++tl) {
            const int rs = tile % row_sets, tb = tile / row_sets;
            const int sel = tl % kAccSets;
            // the tile's per-token terms, once per row set's four warps into shared memory (named barrier 1 + h)
            {
                int* tq = tok_qsum + (tl & 1) * NT;
                float* ts = tok_sx + (tl & 1) * NT;
                if (h == 0 || RS == 1) {
                    for (int i = lrow; i < NT; i += kRows) {
                        const int token = tb * NT + i;
                        tq[i] = token < a.m ? __ldg(a.qsum + token) : 0;
                        ts[i] = (token < a.m && EPI != EPI_I32) ? __ldg(a.sx + token) : 0.0f;
                    }
                }
                ptx::named_bar_sync(1, kEpiWarps * 32);  // all epilogue warps: written before read, read before the tile after next overwrites
            }
            ok &= ptx::mbar_wait_bounded(&acc_full[sel], (uint32_t)((tl / kAccSets) & 1));
            ptx::tc_fence_after();
            const int* tq = tok_qsum + (tl & 1) * NT;
            const float* ts = tok_sx + (tl & 1) * NT;
            const int64_t row = ((int64_t)rs * RS + h) * kRows + lrow;
            const int64_t rt = row >> 4;
            float sw = 0.f;
            if (EPI != EPI_I32 && rt < a.row_tiles) sw = __ldg(a.sw_tiles + 2 * rt + ((row >> 3) & 1));
            const uint32_t acc_addr = tmem_base + ((uint32_t)(sub * 32) << 16) + (uint32_t)(sel * RS + h) * NT;
            const int n_tok = min(NT, a.m - tb * NT);  // tokens of this tile that exist
            bool drained = false;
            if constexpr (kRegSplit) {
                // Whole tiles with an f32 output: this thread's whole accumulator row goes to registers and the set is
                // handed back to the MMA issuer before the first store, so that the next tile's MMAs run under this
                // tile's stores.  The store code is kept short (one epilogue kind per loop, no per-element bounds):
                // it is unrolled 128 times and is fetched once per tile.
                // (one decision per warp: the tensor-memory loads are warp-wide instructions)
                if ((EPI == EPI_F32 || accum) && n_tok == NT && __all_sync(0xffffffffu, row < a.n_out)) {
                    drained = true;
                    uint32_t d[NT];
#pragma unroll
                    for (int c0 = 0; c0 < NT; c0 += 32) ptx::tmem_ld32(acc_addr + c0, reinterpret_cast<uint32_t(&)[32]>(d[c0]));
                    ptx::tmem_ld_wait();
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&acc_empty[sel]);
                    float* po = reinterpret_cast<float*>(a.out) + (int64_t)(tb * NT) * a.out_stride + row;
                    const int64_t stride = a.out_stride;
                    if (accum) {
#pragma unroll
                        for (int c0 = 0; c0 < NT; c0 += 16) {
                            float old[16];
#pragma unroll
                            for (int j = 0; j < 16; ++j) old[j] = po[(c0 + j) * stride];
#pragma unroll
                            for (int j = 0; j < 16; ++j)
                                po[(c0 + j) * stride] =
                                    __fadd_rn(old[j], __fmul_rn(__fmul_rn((float)((int)d[c0 + j] - tq[c0 + j]), sw), ts[c0 + j]));
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < NT; ++i)
                            po[i * stride] = __fmul_rn(__fmul_rn((float)((int)d[i] - tq[i]), sw), ts[i]);
                    }
                }
            }
            if (drained) {
                // nothing left to do for this tile
            } else if constexpr (S == 1) {
                if (accum) {
#pragma unroll 1
                    for (int c0 = 0; c0 < NT; c0 += 16) {
                        uint32_t d[16];
                        float old[16];
                        ptx::tmem_ld16(acc_addr + c0, d);
#pragma unroll
                        for (int j = 0; j < 16; ++j) old[j] = load_old(tb * NT + c0 + j, row);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j) store(tq, ts, tb, c0 + j, n_tok, row, sw, d[j], old[j]);
                    }
                } else {
#pragma unroll 1
                    for (int c0 = 0; c0 < NT; c0 += 32) {
                        uint32_t d[32];
                        ptx::tmem_ld32(acc_addr + c0, d);
                        ptx::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) store(tq, ts, tb, c0 + j, n_tok, row, sw, d[j], 0.0f);
                    }
                }
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&acc_empty[sel]);
            } else {
                // Reduce-scatter over the cluster: every CTA parks its partial sums of the whole tile in its own
                // shared memory ([row set][token / 4][row][token % 4], 16 bytes per thread and step), then adds up and
                // stores the NT / S tokens that are its share, reading all S copies through distributed shared memory.
                if (tl > 0) ok &= ptx::mbar_wait_cluster_bounded(red_free, (uint32_t)((tl - 1) & 1));  // everybody has read the previous tile
#pragma unroll 1
                for (int c0 = 0; c0 < NT; c0 += 32) {
                    uint32_t d[32];
                    ptx::tmem_ld32(acc_addr + c0, d);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        *reinterpret_cast<uint4*>(pb + ((size_t)(c0 / 4 + q) * kRows + lrow) * 4) =
                            make_uint4(d[4 * q], d[4 * q + 1], d[4 * q + 2], d[4 * q + 3]);
                }
                ptx::tc_fence_before();
                ptx::fence_cluster();
                __syncwarp();
                if (lane == 0) {
                    ptx::mbar_arrive(&acc_empty[sel]);  // the accumulator set is free for a later tile
                    // (the fence above has published the parked sums: the arrivals need no release of their own)
#pragma unroll
                    for (int pr = 0; pr < S; ++pr) ptx::mbar_arrive_remote_relaxed(ptx::map_to_rank(red_full, (uint32_t)pr));
                }
                ok &= ptx::mbar_wait_cluster_bounded(red_full, (uint32_t)(tl & 1));  // all S copies are complete
                constexpr int kGroups = NT / 4 / S;  // groups of 4 tokens that this CTA finishes
                constexpr int kBatch = 8 / S;        // groups per round: 8 remote 16-byte loads in flight
#pragma unroll 1
                for (int q0 = 0; q0 < kGroups; q0 += kBatch) {
                    float old[kBatch][4];
                    uint4 part[kBatch][S];
#pragma unroll
                    for (int q = 0; q < kBatch; ++q)
#pragma unroll
                        for (int pr = 0; pr < S; ++pr)
                            part[q][pr] = ptx::ld_dsmem_v4(
                                ptx::map_to_rank(pb + ((size_t)(rank * kGroups + q0 + q) * kRows + lrow) * 4, (uint32_t)pr));
#pragma unroll
                    for (int q = 0; q < kBatch; ++q)
#pragma unroll
                        for (int e = 0; e < 4; ++e) old[q][e] = load_old(tb * NT + (rank * kGroups + q0 + q) * 4 + e, row);
                    // the per-token terms too: a shared-memory load between two global stores would wait for the store
                    int tqv[kBatch][4];
                    float tsv[kBatch][4];
#pragma unroll
                    for (int q = 0; q < kBatch; ++q)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            tqv[q][e] = tq[(rank * kGroups + q0 + q) * 4 + e];
                            tsv[q][e] = ts[(rank * kGroups + q0 + q) * 4 + e];
                        }
#pragma unroll
                    for (int q = 0; q < kBatch; ++q) {
                        uint4 s = part[q][0];
#pragma unroll
                        for (int pr = 1; pr < S; ++pr) {
                            s.x += part[q][pr].x; s.y += part[q][pr].y; s.z += part[q][pr].z; s.w += part[q][pr].w;
                        }
                        const int i = (rank * kGroups + q0 + q) * 4;
                        store_v(tqv[q][0], tsv[q][0], tb, i, n_tok, row, sw, s.x, old[q][0]);
                        store_v(tqv[q][1], tsv[q][1], tb, i + 1, n_tok, row, sw, s.y, old[q][1]);
                        store_v(tqv[q][2], tsv[q][2], tb, i + 2, n_tok, row, sw, s.z, old[q][2]);
                        store_v(tqv[q][3], tsv[q][3], tb, i + 3, n_tok, row, sw, s.w, old[q][3]);
                    }
                }
                __syncwarp();
                if (lane == 0) {
                    // the peers' sums have been read and used: nothing of this thread is left to order
#pragma unroll
                    for (int pr = 0; pr < S; ++pr) ptx::mbar_arrive_remote_relaxed(ptx::map_to_rank(red_free, (uint32_t)pr));
                }
            }
        }
        };
        switch (a.epilogue) {
            case EPI_I32: epilogue_role(std::integral_constant<int, EPI_I32>{}); break;
            case EPI_F32: epilogue_role(std::integral_constant<int, EPI_F32>{}); break;
            case EPI_F32_ACCUM: epilogue_role(std::integral_constant<int, EPI_F32_ACCUM>{}); break;
            default: epilogue_role(std::integral_constant<int, EPI_BF16>{}); break;
        }
    }
    if (!ok) atomicExch(a.err, kErrTcTimeout);
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) ptx::tmem_dealloc(tmem_base, kTmemCols);
    if (S > 1) {
        // Nobody leaves while a peer may still read its shared memory or arrive on its barriers: the last of both is
        // the peers' arrival on red_free for this CTA's last tile (they read the parked sums before it, and arrived on
        // red_full before that).  One warp waits for it; the CTA lives as long as that warp.
        const int my_tiles = cid < n_tiles ? (n_tiles - cid + n_clusters - 1) / n_clusters : 0;
        if (warp == 2 && my_tiles > 0 && !ptx::mbar_wait_cluster_bounded(red_free, (uint32_t)((my_tiles - 1) & 1)))
            atomicExch(a.err, kErrTcTimeout);
    }
}

// One kernel variant (token tile NT, RS row sets per tile, S CTAs per cluster): its shared memory and how many
// clusters fit on the GPU at once (a cluster lives inside one GPC, so this is not SMs / S), asked of the runtime once.
struct TcVariant {
    size_t smem = 0;
    int max_clusters = 0;
    cudaError_t status = cudaErrorNotReady;
};

template <int NT, int RS, int S>
const TcVariant& tc_variant(int sm_count) {
    static TcVariant v;              // cluster limit: once per process (every device of a process is the same GPU model)
    static PerDeviceOnce attributes;  // the kernel's shared-memory limit: once per device
    v.smem = (size_t)tc_stages(NT, RS, S) * (RS * kSetBytes + 4 * NT * 64) + (S > 1 ? RS * kRows * NT * 4 : 0) + 512 + 16 * NT;
    auto* kernel = gemm_tc_kernel<NT, RS, S>;
    const size_t smem = v.smem;
    v.status = attributes.run([kernel, smem] {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess && NT == 128 && RS == 2 && S == 1) {
            // the register shares the warpgroups ask for must fit what the launch gives the CTA, or the asking waits for ever
            cudaFuncAttributes fa;
            e = cudaFuncGetAttributes(&fa, kernel);
            const int have = fa.numRegs * tc_threads(RS);
            const int want = 128 * kRegsLead + 256 * kRegsUnpack + 256 * kRegsEpilogue;
            if (e == cudaSuccess && have < want) e = cudaErrorLaunchOutOfResources;
        }
        return e;
    });
    if (v.status != cudaSuccess) return v;
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    if (v.max_clusters != 0) return v;
    if (S == 1) { v.max_clusters = sm_count; return v; }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(sm_count / S * S));
    cfg.blockDim = dim3(tc_threads(RS));
    cfg.dynamicSmemBytes = v.smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)S; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n < 1) {
        (void)cudaGetLastError();
        n = -1;  // this cluster size cannot be used
    }
    v.max_clusters = n;
    return v;
}

template <int NT, int RS, int S>
cudaError_t launch_variant(TcArgs a, int sm_count, cudaStream_t stream) {
    const TcVariant& v = tc_variant<NT, RS, S>(sm_count);
    if (v.status != cudaSuccess) return v.status;
    const int n_tiles = (int)((a.row_tiles + 8 * RS - 1) / (8 * RS)) * ((a.m + NT - 1) / NT);
    const int n_clusters = v.max_clusters < n_tiles ? v.max_clusters : n_tiles;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(n_clusters * S));
    cfg.blockDim = dim3(tc_threads(RS));
    cfg.dynamicSmemBytes = v.smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = (unsigned)S; attr[1].val.clusterDim.y = 1; attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = S > 1 ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, gemm_tc_kernel<NT, RS, S>, a);
}

// Chunk steps on the busiest CTA when a tile's k range is cut over `s` CTAs (one step charged for the exchange of
// partial sums); a huge number when the cut is not possible.
int64_t tc_split_cost(int s, int max_clusters, int n_tiles, int64_t k_tiles) {
    if (max_clusters < 1) return INT64_MAX;  // (-1: the cluster size is unusable)
    const int64_t cps = (k_tiles + s - 1) / s;
    if (s > 1 && (k_tiles < 2 * s || cps * (s - 1) >= k_tiles)) return INT64_MAX;  // a CTA would be left without chunks
    const int nc = max_clusters < n_tiles ? max_clusters : n_tiles;
    return (int64_t)((n_tiles + nc - 1) / nc) * (cps + (s > 1 ? 1 : 0));
}

cudaError_t launch_product(TcArgs a, int nt, int sm_count, cudaStream_t stream) {
    const int tok_blocks = (a.m + nt - 1) / nt;
    const int n_tiles = (int)((a.row_tiles + 7) / 8) * tok_blocks;          // tiles of 128 rows
    const int n_tiles2 = (int)((a.row_tiles + 15) / 16) * tok_blocks;       // tiles of 256 rows
    if (nt == 128) {
        // 256-row tiles halve the activation traffic per weight; 128-row tiles when there is too little work for them
        return 2 * n_tiles2 >= sm_count ? launch_variant<128, 2, 1>(a, sm_count, stream) : launch_variant<128, 1, 1>(a, sm_count, stream);
    }
    // 64 tokens at most.  More 128-row tiles than SMs: 256-row tiles.  Fewer than half: cut k over a cluster so that
    // one wave of CTAs covers the product.
    if (n_tiles > sm_count) return launch_variant<64, 2, 1>(a, sm_count, stream);
    int best = 1;
    int64_t best_cost = tc_split_cost(1, sm_count, n_tiles, a.k_tiles);
    if (n_tiles * 2 <= sm_count) {
        const int64_t c2 = tc_split_cost(2, tc_variant<64, 1, 2>(sm_count).max_clusters, n_tiles, a.k_tiles);
        const int64_t c4 = tc_split_cost(4, tc_variant<64, 1, 4>(sm_count).max_clusters, n_tiles, a.k_tiles);
        const int64_t c8 = tc_split_cost(8, tc_variant<64, 1, 8>(sm_count).max_clusters, n_tiles, a.k_tiles);
        if (c2 < best_cost) { best = 2; best_cost = c2; }
        if (c4 < best_cost) { best = 4; best_cost = c4; }
        if (c8 < best_cost) { best = 8; best_cost = c8; }
    }
    switch (best) {
        case 2: return launch_variant<64, 1, 2>(a, sm_count, stream);
        case 4: return launch_variant<64, 1, 4>(a, sm_count, stream);
        case 8: return launch_variant<64, 1, 8>(a, sm_count, stream);
        default: return launch_variant<64, 1, 1>(a, sm_count, stream);
    }
}

}  // namespace

int gemm_tc_kernels(const LinearDev& lin, int64_t m, int sm_count) {
    (void)m; (void)sm_count;
    return lin.w.n_bases;  // one launch per basis; a k split is reduced inside the launch
}

size_t gemm_tc_act_bytes(int64_t m, int64_t k_tiles) {
    const int64_t nt = m <= 64 ? 64 : 128;
    return (size_t)((m + nt - 1) / nt * k_tiles * 4 * nt * 64);
}

cudaError_t launch_gemm_tc(const LinearDev& lin, const void* x, int64_t x_stride, int64_t m, int8_t* qtc, float* sx,
                           int32_t* qsum, void* out, int64_t out_stride, int epilogue, unsigned int* err, int sm_count,
                           cudaStream_t stream, bool prequantised, bt_dtype x_dtype) {
    if (lin.w.n_bases != 1 && epilogue == EPI_BF16) return cudaErrorInvalidValue;
    if (epilogue != EPI_I32 && epilogue != EPI_F32 && epilogue != EPI_F32_ACCUM && epilogue != EPI_BF16)
        return cudaErrorInvalidValue;  // (the SiLU*up epilogue exists in the streaming kernel only)
    const int nt = m <= 64 ? 64 : 128;
    const int k = (int)lin.w.k_in, kts = (int)lin.w.k_tiles;
    cudaError_t e = cudaSuccess;
    if (prequantised) {
    } else if (x_dtype == BT_BF16) {
        e = launch_row_quant_bf16(reinterpret_cast<const __nv_bfloat16*>(x), x_stride, (int)m, k, sx, qsum, stream, qtc, kts);
    } else {
        // f32 rows: the row kernel of the decode step (identity transform); rows of a partly filled token block
        // keep whatever they held, their output columns are never stored
        e = launch_row_quant(PRE_NONE, reinterpret_cast<const float*>(x), x_stride, nullptr, 0.0f, (int)m, k, nullptr, 0, sx, qsum,
                             nullptr, stream, qtc, kts);
    }
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
        e = launch_product(a, nt, sm_count, stream);
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace bt
