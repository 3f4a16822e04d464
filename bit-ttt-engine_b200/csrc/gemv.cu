// Decode-time ternary product for 1..8 tokens: y[m, n] = sum_k q[m, k] * t[n, k].
//
// Stands in for the inner loops of BitLinearCpu::forward (kernels/cpu.rs:73-124,134-239)
// and the never-launched bit_linear_forward kernel (kernels/bit_op.cu:4-45).
//
// HBM-bound: every weight byte is read exactly once per launch.  Structure:
//   * one persistent CTA per SM; CTA c owns row tiles c, c+G, c+2G, ... (16 rows each);
//   * a producer thread streams the tiles of a row tile (contiguous in the tiled layout)
//     into a shared-memory ring with 1-D bulk async copies that complete on mbarriers -
//     8 KB per stage, as many stages as shared memory allows, so tens of KB per SM are
//     in flight independent of what the math warps are doing;
//   * 8 math warps split each stage along K (one 1 KB tile each).  A lane's two 16-byte
//     chunks are already the A-operand slots of mma.m16n8k32 (u8 x s8 -> s32): one AND
//     per register isolates field r of every byte as an unsigned multiple of 4^r, so the
//     unpack costs one integer instruction per four weights and the four field
//     positions accumulate into four accumulator sets that are shifted back at the end;
//   * the int8 activations sit in shared memory, byte-transposed in groups of 16 so that
//     the B-operand registers match the field order of the A registers;
//   * after the last stage of a row tile the 8 warps reduce through shared memory and
//     128 threads run the epilogue (subtract sum_k q to undo the +1 weight offset, scale,
//     store).  Integer accumulation makes the result independent of the split.
#include "bt_common.cuh"
#include "bt_ptx.cuh"

namespace bt {

namespace {

constexpr int kMathWarps = 8;
constexpr int kMathThreads = kMathWarps * 32;
constexpr int kThreads = kMathThreads + 32;  // + producer warp
constexpr int kStageTiles = 8;
constexpr int kStageBytes = kStageTiles * kTileBytes;
constexpr int kRedBytes = 2 * kMathWarps * 4 * 32 * 4;
constexpr int kMaxStages = 16;
constexpr unsigned kErrGemvTimeout = 0x47454d56u;  // 'GEMV'

__device__ __forceinline__ uint4 lds128(const void* p) { return *reinterpret_cast<const uint4*>(p); }

__global__ void __launch_bounds__(kThreads, 1) gemv_kernel(GemvArgs a, int nstages, int act_stride) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* ring = smem;
    uint8_t* acts = ring + (size_t)nstages * kStageBytes;
    int* red = reinterpret_cast<int*>(acts + (size_t)a.m * act_stride);
    uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(red) + kRedBytes);
    uint64_t* empty = full + kMaxStages;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t stages_per_rt = (a.k_tiles + kStageTiles - 1) / kStageTiles;
    const int64_t my_rts = (a.row_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x;
    const int64_t total_iters = my_rts * stages_per_rt;

    if (threadIdx.x == 0) {
        for (int s = 0; s < nstages; ++s) {
            ptx::mbar_init(&full[s], 1);
            ptx::mbar_init(&empty[s], kMathWarps);
        }
        ptx::mbar_fence_init();
    }
    __syncthreads();

    if (warp == kMathWarps) {
        // ---------------- producer: weights do not depend on earlier kernels ----------------
        if (lane == 0) {
            bool ok = true;
            for (int64_t it = 0; it < total_iters; ++it) {
                const int slot = (int)(it % nstages);
                const int64_t use = it / nstages;
                if (use > 0) ok &= ptx::mbar_wait_bounded(&empty[slot], (uint32_t)((use - 1) & 1));
                const int64_t rt = blockIdx.x + (it / stages_per_rt) * gridDim.x;
                const int64_t kt0 = (it % stages_per_rt) * kStageTiles;
                const int64_t nt = a.k_tiles - kt0 < kStageTiles ? a.k_tiles - kt0 : kStageTiles;
                const uint32_t bytes = (uint32_t)(nt * kTileBytes);
                ptx::mbar_arrive_expect_tx(&full[slot], bytes);
                ptx::bulk_g2s(ring + (size_t)slot * kStageBytes,
                              a.tiles + (rt * a.k_tiles + kt0) * kTileBytes, bytes, &full[slot]);
                if (it + 1 == nstages || it + 1 == total_iters) ptx::pdl_launch_dependents();
            }
            if (!ok) atomicExch(a.err, kErrGemvTimeout);
        }
        return;
    }

    // ---------------- math warps ----------------
    ptx::pdl_wait();  // activations come from the previous kernel of the stream
    const int tid = threadIdx.x;
    const int g = lane >> 2, t = lane & 3;

    // Stage the int8 activations: for every group of 16 consecutive inputs, byte r of word
    // b (input 4b + r) moves to byte b of word r, and word r of the four 16-groups of a
    // lane's 64-input chunk are stored side by side: offset = kt*256 + r*64 + t*16 + i*4.
    {
        const int groups = (int)(a.k_tiles * (kTileK / 16));
        for (int n = 0; n < a.m; ++n) {
            const uint4* src = reinterpret_cast<const uint4*>(a.q + (int64_t)n * a.q_stride);
            uint8_t* dst = acts + (size_t)n * act_stride;
            for (int j = tid; j < groups; j += kMathThreads) {
                const uint4 v = src[j];
                const uint32_t in[4] = {v.x, v.y, v.z, v.w};
                uint32_t out[4];
                ptx::transpose4x4(in, out);
                const int kt = j >> 4, tt = (j >> 2) & 3, i = j & 3;
                uint8_t* p = dst + kt * kTileK + tt * 16 + i * 4;
#pragma unroll
                for (int r = 0; r < 4; ++r) *reinterpret_cast<uint32_t*>(p + r * 64) = out[r];
            }
        }
    }
    ptx::named_bar_sync(1, kMathThreads);

    int acc[4][4];
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[r][j] = 0;

    const uint8_t* my_acts = acts + (size_t)g * act_stride + t * 16;
    const bool has_token = g < a.m;
    bool ok = true;
    int buf = 0;

    for (int64_t it = 0; it < total_iters; ++it) {
        const int slot = (int)(it % nstages);
        const uint32_t parity = (uint32_t)((it / nstages) & 1);
        const int64_t sk = it % stages_per_rt;
        const int64_t kt = sk * kStageTiles + warp;
        ok &= ptx::mbar_wait_bounded(&full[slot], parity);
        if (kt < a.k_tiles) {
            const uint8_t* tile = ring + (size_t)slot * kStageBytes + warp * kTileBytes;
            const uint4 w4 = lds128(tile + lane * 16);
            const uint4 v4 = lds128(tile + 512 + lane * 16);
            const uint32_t W[4] = {w4.x, w4.y, w4.z, w4.w};
            const uint32_t V[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                uint4 b4 = make_uint4(0, 0, 0, 0);
                if (has_token) b4 = lds128(my_acts + kt * kTileK + r * 64);
                const uint32_t mask = 0x03030303u << (2 * r);
                ptx::mma_u8s8(acc[r], W[0] & mask, V[0] & mask, W[2] & mask, V[2] & mask, b4.x, b4.z);
                ptx::mma_u8s8(acc[r], W[1] & mask, V[1] & mask, W[3] & mask, V[3] & mask, b4.y, b4.w);
            }
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&empty[slot]);

        if (sk == stages_per_rt - 1) {
            // row tile complete: fold the four field positions, reduce over warps, store
            int* my_red = red + buf * (kMathWarps * 128) + warp * 128;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int v = acc[0][j] + (acc[1][j] >> 2) + (acc[2][j] >> 4) + (acc[3][j] >> 6);
                my_red[j * 32 + lane] = v;
                acc[0][j] = acc[1][j] = acc[2][j] = acc[3][j] = 0;
            }
            ptx::named_bar_sync(1, kMathThreads);
            if (tid < 128) {
                const int j = tid >> 5, l = tid & 31;
                int sum = 0;
#pragma unroll
                for (int w = 0; w < kMathWarps; ++w) sum += red[buf * (kMathWarps * 128) + w * 128 + j * 32 + l];
                const int64_t rt = blockIdx.x + (it / stages_per_rt) * gridDim.x;
                const int64_t row = rt * kTileRows + (l >> 2) + ((j & 2) ? 8 : 0);
                const int token = 2 * (l & 3) + (j & 1);
                if (token < a.m && row < a.n_out) {
                    const int accv = sum - a.qsum[token];
                    const int64_t o = (int64_t)token * a.out_stride + row;
                    if (a.epilogue == EPI_I32) {
                        reinterpret_cast<int32_t*>(a.out)[o] = accv;
                    } else {
                        const float y = __fmul_rn(__fmul_rn((float)accv, a.sw), a.sx[token]);
                        if (a.epilogue == EPI_F32) reinterpret_cast<float*>(a.out)[o] = y;
                        else if (a.epilogue == EPI_F32_ACCUM) reinterpret_cast<float*>(a.out)[o] = __fadd_rn(reinterpret_cast<float*>(a.out)[o], y);
                        else reinterpret_cast<__nv_bfloat16*>(a.out)[o] = __float2bfloat16_rn(y);
                    }
                }
            }
            buf ^= 1;
        }
    }
    if (!ok) {
        atomicExch(a.err, kErrGemvTimeout);
        // give copies still in flight a bounded chance to land before the CTA retires
        for (int s = 0; s < nstages; ++s) {
            const int64_t uses = (total_iters - s + nstages - 1) / nstages;
            if (uses > 0) ptx::mbar_wait_bounded(&full[s], (uint32_t)((uses - 1) & 1));
        }
    }
}

}  // namespace

cudaError_t launch_gemv(const GemvArgs& a, int sm_count, cudaStream_t stream) {
    if (a.m < 1 || a.m > 8) return cudaErrorInvalidValue;
    const int act_stride = (int)(a.k_tiles * kTileK + 64);
    const size_t fixed = (size_t)a.m * act_stride + kRedBytes + 2 * kMaxStages * sizeof(uint64_t);
    const size_t budget = 200 * 1024;
    if (fixed + 2 * kStageBytes > budget) return cudaErrorInvalidConfiguration;
    int nstages = (int)((budget - fixed) / kStageBytes);
    if (nstages > kMaxStages) nstages = kMaxStages;
    const int64_t stages_per_rt = (a.k_tiles + kStageTiles - 1) / kStageTiles;
    int grid = (int)(a.row_tiles < sm_count ? a.row_tiles : sm_count);
    const int64_t max_iters = ((a.row_tiles + grid - 1) / grid) * stages_per_rt;
    if (nstages > max_iters) nstages = (int)max_iters;
    if (nstages < 1) nstages = 1;
    const size_t smem = (size_t)nstages * kStageBytes + fixed;
    static thread_local size_t configured = 0;
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget);
        if (e != cudaSuccess) return e;
        configured = budget;
    }
    gemv_kernel<<<grid, kThreads, smem, stream>>>(a, nstages, act_stride);
    return cudaGetLastError();
}

}  // namespace bt
