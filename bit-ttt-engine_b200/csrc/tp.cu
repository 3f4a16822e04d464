// Tensor parallelism over the GPUs of one node (no counterpart in the reference, which is
// single-GPU: model/llama.rs:43,404 hard-code device 0).  One process per GPU; q|k|v and
// gate|up are split by output rows (column-parallel), o_proj and down_proj by input columns
// (row-parallel).  A row-parallel projection is made exact with respect to the single-GPU
// result by (i) an all-reduce(max) of the per-token max|x| before quantising, so that every
// rank quantises with the same scale, and (ii) an all-reduce(sum) of the int32 accumulators
// before the scale epilogue: integer sums do not depend on the order of the ranks.
//
// The collectives go through NCCL, looked up at run time in the process (the library has no
// link-time dependency on it): ncclAllReduce is stream-ordered and can be captured into
// the decode step's CUDA graph.
//
// Decode moves a few KB per exchange, so two NCCL calls per projection cost far more than the
// data: when the ranks have exchanged CUDA IPC handles of their inboxes (tp_peer_*), the two
// all-reduces run as two small kernels of this library over NVLink peer memory instead.  Every
// rank PUSHES its values into each peer's inbox (plain stores to peer memory), publishes a
// per-source epoch flag with release semantics at system scope, waits - with a bound - for the
// flags of all sources in its own inbox, and reduces locally; the integer sum is fused with
// the scale epilogue and the residual add.  Two inbox slots alternate (o_proj / down_proj), so
// a rank that runs ahead never overwrites values a slower rank has not read yet: it cannot
// reach the same slot again without the slower rank's contribution to the exchanges between.
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include <new>

#include "bt_handles.cuh"
#include "bt_ptx.cuh"

namespace bt {

namespace {

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;  // optional
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    bool ok = false;
};

NcclApi* nccl_api() {
    static NcclApi api;
    static bool tried = false;
    if (tried) return api.ok ? &api : nullptr;
    tried = true;
    // the copy already loaded into the process (e.g. by PyTorch) wins; otherwise the system's
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return nullptr;
    api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
    api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
    api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
    api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(dlsym(h, "ncclAllReduce"));
    api.GetErrorString = reinterpret_cast<decltype(api.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
    api.AllGather = reinterpret_cast<decltype(api.AllGather)>(dlsym(h, "ncclAllGather"));
    api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.GetErrorString;
    return api.ok ? &api : nullptr;
}

// h[m, n] += ((float)acc[m, n] * sw) * (absmax[m] / 127): the scale epilogue of a
// row-parallel projection after its accumulators were summed over the ranks.
__global__ void tp_residual_kernel(const int32_t* __restrict__ acc, const unsigned int* __restrict__ absmax,
                                   float sw, int n, float* __restrict__ h) {
    ptx::pdl_wait();
    ptx::pdl_launch_dependents();
    const int m = blockIdx.y;
    const float sx = __fdiv_rn(__uint_as_float(absmax[m]), 127.0f);
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < n; c += gridDim.x * blockDim.x) {
        const int64_t o = (int64_t)m * n + c;
        h[o] = __fadd_rn(h[o], __fmul_rn(__fmul_rn((float)acc[o], sw), sx));
    }
}


// ---------------------------------------------------------------------------------------
// peer-memory exchange
// ---------------------------------------------------------------------------------------
constexpr int kTpMaxRanks = 8;
constexpr unsigned kErrTpTimeout = 0x54505754u;  // 'TPWT'

// Inbox layout (identical on every rank): for slot s in {0, 1} and source rank r
//   acc  [s][r][max_batch * hidden] int32
//   amax [s][r][max_batch] u32 (rows padded to 16 entries)
//   flag [s][kind][r] u64 epochs (kind 0: amax published)
//   cflag [s][r][cta] u64 epochs: CTA `cta` of rank r's sum kernel has pushed its slice of acc
struct TpLayout {
    int size, max_batch, hidden;
    __host__ __device__ size_t acc_elems() const { return (size_t)max_batch * hidden; }
    __host__ __device__ size_t acc_off(int s, int r) const { return ((size_t)(s * size + r) * acc_elems()) * 4; }
    __host__ __device__ size_t amax_base() const { return (size_t)2 * size * acc_elems() * 4; }
    __host__ __device__ size_t amax_off(int s, int r) const { return amax_base() + (size_t)(s * size + r) * 16 * 4; }
    __host__ __device__ size_t flag_base() const { return amax_base() + (size_t)2 * size * 16 * 4; }
    __host__ __device__ size_t flag_off(int s, int kind, int r) const { return flag_base() + (size_t)((s * 2 + kind) * size + r) * 8; }
    // per-CTA epochs of the sum exchange: [s][r][16 CTAs]
    __host__ __device__ size_t cflag_base() const { return flag_base() + (size_t)2 * 2 * size * 8; }
    __host__ __device__ size_t cflag_off(int s, int r, int cta) const { return cflag_base() + (size_t)((s * size + r) * 16 + cta) * 8; }
    __host__ __device__ size_t bytes() const { return cflag_base() + (size_t)2 * size * 16 * 8; }
};

struct TpView {
    TpLayout lay;
    int rank;
    uint8_t* inbox[kTpMaxRanks];       // every rank's inbox as mapped into this process (own included)
    unsigned long long* epoch;         // local, [2 slots]: exchanges done on the slot
    unsigned long long wait_ns;        // how long a kernel waits for its peers before it gives up
    unsigned int* done;                // local, [2 slots]: CTAs of the running sum kernel that have pushed
    unsigned int* err;
};

__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
// Waits until the cell holds epoch e or later.  The wait is bounded in time (globaltimer, the
// limit is set from the host) and is skipped altogether once any kernel has recorded an error on
// this device: after one rank has gone missing the rest of the step drains quickly instead of
// paying the limit at every exchange.
__device__ __forceinline__ bool wait_epoch(const TpView& v, const unsigned long long* f, unsigned long long e) {
    if (ld_acquire_sys(f) >= e) return true;
    if (*reinterpret_cast<volatile unsigned int*>(v.err) != 0u) return false;
    const unsigned long long t0 = ptx::globaltimer();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; ++i)
            if (ld_acquire_sys(f) >= e) return true;
        if (ptx::globaltimer() - t0 > v.wait_ns) return false;
    }
}
// waits until source rank `src` has published epoch e on (slot, kind) of this rank's inbox
__device__ __forceinline__ bool wait_sources(const TpView& v, int slot, int kind, unsigned long long e, int src) {
    return wait_epoch(v, reinterpret_cast<const unsigned long long*>(v.inbox[v.rank] + v.lay.flag_off(slot, kind, src)), e);
}

// all-reduce(max) of the per-token max|x| cells: one CTA
__global__ void __launch_bounds__(256) tp_max_exchange_kernel(TpView v, int slot, unsigned int* amax_cell, int batch) {
    __shared__ int ok_s;
    const int tid = threadIdx.x, R = v.lay.size;
    ptx::pdl_wait();               // the cells belong to the kernel before this one until here
    ptx::pdl_launch_dependents();  // the product that follows may start fetching its weights during the exchange
    const unsigned long long e = v.epoch[slot] + 1;
    if (tid == 0) ok_s = 1;
    for (int i = tid; i < batch * R; i += blockDim.x) {
        const int p = i / batch, tok = i % batch;
        reinterpret_cast<unsigned int*>(v.inbox[p] + v.lay.amax_off(slot, v.rank))[tok] = amax_cell[tok];
    }
    __threadfence_system();
    __syncthreads();
    if (tid < R) {
        st_release_sys(reinterpret_cast<unsigned long long*>(v.inbox[tid] + v.lay.flag_off(slot, 0, v.rank)), e);
        if (!wait_sources(v, slot, 0, e, tid)) ok_s = 0;
    }
    __syncthreads();
    if (tid < batch) {
        unsigned int mx = 0;  // bit patterns of non-negative floats order like the floats
        for (int r = 0; r < R; ++r)
            mx = max(mx, __ldcg(reinterpret_cast<const unsigned int*>(v.inbox[v.rank] + v.lay.amax_off(slot, r)) + tid));
        amax_cell[tid] = mx;
    }
    if (tid == 0) {
        v.epoch[slot] = e;  // the sum kernel that follows on this slot uses the same epoch
        if (!ok_s) atomicExch(v.err, kErrTpTimeout);
    }
}

// all-reduce(sum) of the int32 accumulators fused with the scale epilogue and the residual:
// h[m, n] += ((float)sum_r acc_r[m, n] * sw) * (absmax[m] / 127)
__global__ void __launch_bounds__(256) tp_sum_residual_kernel(TpView v, int slot, const int32_t* __restrict__ acc,
                                                              const unsigned int* __restrict__ amax_cell, float sw,
                                                              int batch, int n, float* __restrict__ h) {
    __shared__ int ok_s;
    const int tid = threadIdx.x, R = v.lay.size;
    ptx::pdl_wait();               // acc and the epoch belong to earlier kernels until here
    ptx::pdl_launch_dependents();
    const unsigned long long e = v.epoch[slot];  // set by the max exchange just before
    const int total4 = batch * n / 4;            // n is a multiple of 16
    const int per_cta = (total4 + gridDim.x - 1) / gridDim.x;
    const int i0 = blockIdx.x * per_cta, i1 = min(total4, i0 + per_cta);
    if (tid == 0) ok_s = 1;
    for (int i = i0 + tid; i < i1; i += blockDim.x) {
        const int4 val = reinterpret_cast<const int4*>(acc)[i];
        for (int p = 0; p < R; ++p) reinterpret_cast<int4*>(v.inbox[p] + v.lay.acc_off(slot, v.rank))[i] = val;
    }
    // CTA c of every rank owns the same slice: it publishes its own epoch cell at every peer and
    // waits for the peers' cells of the same slice.  The barrier orders the CTA's pushes before the
    // fence of the publishing threads (fences are cumulative).
    __syncthreads();
    if (tid < R) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<unsigned long long*>(v.inbox[tid] + v.lay.cflag_off(slot, v.rank, blockIdx.x)), e);
        const unsigned long long* f = reinterpret_cast<const unsigned long long*>(v.inbox[v.rank] + v.lay.cflag_off(slot, tid, blockIdx.x));
        if (!wait_epoch(v, f, e)) ok_s = 0;
    }
    __syncthreads();
    if (!ok_s) {
        // a peer never arrived: its cells are stale, so h is left as it was (the step's result is
        // invalid either way; the host sees BT_ERR_TIMEOUT and must reset all ranks)
        if (tid == 0) atomicExch(v.err, kErrTpTimeout);
        return;
    }
    for (int i = i0 + tid; i < i1; i += blockDim.x) {
        int4 sum = make_int4(0, 0, 0, 0);
        for (int r = 0; r < R; ++r) {
            const int4 a4 = __ldcg(reinterpret_cast<const int4*>(v.inbox[v.rank] + v.lay.acc_off(slot, r)) + i);
            sum.x += a4.x; sum.y += a4.y; sum.z += a4.z; sum.w += a4.w;
        }
        const int m = (4 * i) / n;
        const float sx = __fdiv_rn(__uint_as_float(amax_cell[m]), 127.0f);
        float4 hv = reinterpret_cast<float4*>(h)[i];
        hv.x = __fadd_rn(hv.x, __fmul_rn(__fmul_rn((float)sum.x, sw), sx));
        hv.y = __fadd_rn(hv.y, __fmul_rn(__fmul_rn((float)sum.y, sw), sx));
        hv.z = __fadd_rn(hv.z, __fmul_rn(__fmul_rn((float)sum.z, sw), sx));
        hv.w = __fadd_rn(hv.w, __fmul_rn(__fmul_rn((float)sum.w, sw), sx));
        reinterpret_cast<float4*>(h)[i] = hv;
    }
}

}  // namespace

bt_status tp_unique_id(void* out128) {
    NcclApi* api = nccl_api();
    if (!api) return set_error(BT_ERR_NCCL, "NCCL (libnccl.so.2) could not be loaded");
    ncclUniqueId id;
    ncclResult_t r = api->GetUniqueId(&id);
    if (r != ncclSuccess) return set_error(BT_ERR_NCCL, "ncclGetUniqueId: %s", api->GetErrorString(r));
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId size");
    memcpy(out128, &id, 128);
    return BT_OK;
}

bt_status tp_comm_init(void** comm, const void* id128, int rank, int size) {
    NcclApi* api = nccl_api();
    if (!api) return set_error(BT_ERR_NCCL, "NCCL (libnccl.so.2) could not be loaded");
    ncclUniqueId id;
    memcpy(&id, id128, 128);
    ncclComm_t c = nullptr;
    ncclResult_t r = api->CommInitRank(&c, size, id, rank);
    if (r != ncclSuccess) return set_error(BT_ERR_NCCL, "ncclCommInitRank: %s", api->GetErrorString(r));
    *comm = c;
    return BT_OK;
}

void tp_comm_destroy(void* comm) {
    NcclApi* api = nccl_api();
    if (api && comm) api->CommDestroy(reinterpret_cast<ncclComm_t>(comm));
}

bt_status tp_allreduce_max_f32(void* comm, float* buf, size_t count, cudaStream_t s) {
    NcclApi* api = nccl_api();
    ncclResult_t r = api->AllReduce(buf, buf, count, ncclFloat32, ncclMax, reinterpret_cast<ncclComm_t>(comm), s);
    if (r != ncclSuccess) return set_error(BT_ERR_NCCL, "ncclAllReduce(max): %s", api->GetErrorString(r));
    return BT_OK;
}

bt_status tp_allreduce_sum_i32(void* comm, int32_t* buf, size_t count, cudaStream_t s) {
    NcclApi* api = nccl_api();
    ncclResult_t r = api->AllReduce(buf, buf, count, ncclInt32, ncclSum, reinterpret_cast<ncclComm_t>(comm), s);
    if (r != ncclSuccess) return set_error(BT_ERR_NCCL, "ncclAllReduce(sum): %s", api->GetErrorString(r));
    return BT_OK;
}

bool tp_allgather_available() {
    NcclApi* api = nccl_api();
    return api && api->AllGather;
}

// In-place all-gather of `count` floats per rank: rank r's part lies at buf + r * count on every rank.
bt_status tp_allgather_f32(void* comm, float* buf, size_t count, int rank, cudaStream_t s) {
    NcclApi* api = nccl_api();
    if (!api || !api->AllGather) return set_error(BT_ERR_NCCL, "ncclAllGather is not available");
    ncclResult_t r = api->AllGather(buf + (size_t)rank * count, buf, count, ncclFloat32, reinterpret_cast<ncclComm_t>(comm), s);
    if (r != ncclSuccess) return set_error(BT_ERR_NCCL, "ncclAllGather: %s", api->GetErrorString(r));
    return BT_OK;
}

// full[b][r * vl + j] = parts[r][b][j]: the vocabulary slices of the ranks (rank r computed rows r * vl .. of the
// head, n_r = min(vl, vocab - r * vl) of them, stored [batch][n_r] at parts + r * batch * vl) side by side.
__global__ void tp_logits_rows_kernel(const float* __restrict__ parts, int tp, int batch, int64_t vl, int64_t vocab,
                                      float* __restrict__ full) {
    const int b = blockIdx.y;
    for (int64_t v = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; v < vocab; v += (int64_t)gridDim.x * blockDim.x) {
        const int r = (int)(v / vl);
        const int64_t n_r = vocab - r * vl < vl ? vocab - r * vl : vl;
        full[(int64_t)b * vocab + v] = parts[((int64_t)r * batch) * vl + (int64_t)b * n_r + (v - r * vl)];
    }
}

cudaError_t launch_tp_logits_rows(const float* parts, int tp, int batch, int64_t vl, int64_t vocab, float* full, cudaStream_t s) {
    tp_logits_rows_kernel<<<dim3(148, batch), 256, 0, s>>>(parts, tp, batch, vl, vocab, full);
    return cudaGetLastError();
}

// ---------------------------------------------------------------------------------------
// peer-memory exchange: host side
// ---------------------------------------------------------------------------------------
struct TpPeer {
    TpView view{};
    uint8_t* local = nullptr;
    bool opened[kTpMaxRanks] = {false};
    bool ready = false;
};

bt_status tp_peer_create(void** out, int rank, int size, int max_batch, int hidden, unsigned int* err) {
    if (size < 2 || size > kTpMaxRanks || rank < 0 || rank >= size || max_batch < 1 || max_batch > 16 || hidden % 16 != 0)
        return set_error(BT_ERR_ARG, "tp_peer_create: size %d (2..8), rank %d, max_batch %d (1..16) or hidden %d unsupported",
                         size, rank, max_batch, hidden);
    TpPeer* p = new (std::nothrow) TpPeer();
    if (!p) return set_error(BT_ERR_NOMEM, "host allocation failed");
    p->view.lay = TpLayout{size, max_batch, hidden};
    p->view.rank = rank;
    p->view.err = err;
    p->view.wait_ns = 5000000000ull;  // 5 s: longer than any host-side stall between two ranks' launches
    // plain cudaMalloc memory: IPC handles cannot be taken from pool allocations
    cudaError_t e = cudaMalloc(reinterpret_cast<void**>(&p->local), p->view.lay.bytes());
    if (e == cudaSuccess) e = cudaMemset(p->local, 0, p->view.lay.bytes());
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&p->view.epoch), 2 * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMemset(p->view.epoch, 0, 2 * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void**>(&p->view.done), 2 * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaMemset(p->view.done, 0, 2 * sizeof(unsigned int));
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(p->local); cudaFree(p->view.epoch); cudaFree(p->view.done);
        delete p;
        return set_error(BT_ERR_CUDA, "tp_peer_create: %s", cudaGetErrorString(e));
    }
    p->view.inbox[rank] = p->local;
    *out = p;
    return BT_OK;
}

bt_status tp_peer_export(void* peer, void* handle64_out) {
    TpPeer* p = reinterpret_cast<TpPeer*>(peer);
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, p->local);
    if (e != cudaSuccess) return set_error(BT_ERR_CUDA, "cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
    memcpy(handle64_out, &h, 64);
    return BT_OK;
}

bt_status tp_peer_import(void* peer, const void* handles) {
    TpPeer* p = reinterpret_cast<TpPeer*>(peer);
    if (p->ready) return BT_OK;
    for (int r = 0; r < p->view.lay.size; ++r) {
        if (r == p->view.rank) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, reinterpret_cast<const uint8_t*>(handles) + 64 * r, 64);
        void* mapped = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&mapped, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) return set_error(BT_ERR_CUDA, "cudaIpcOpenMemHandle(rank %d): %s", r, cudaGetErrorString(e));
        p->view.inbox[r] = reinterpret_cast<uint8_t*>(mapped);
        p->opened[r] = true;
    }
    p->ready = true;
    return BT_OK;
}

void tp_peer_set_wait(void* peer, unsigned long long ns) {
    if (peer) reinterpret_cast<TpPeer*>(peer)->view.wait_ns = ns;
}

// Back to epoch 0: clears the epoch counters and every flag of the local inbox.  All ranks have to
// do this between the same two steps (the peers' next flags start from 1 again).
cudaError_t tp_peer_reset(void* peer) {
    TpPeer* p = reinterpret_cast<TpPeer*>(peer);
    if (!p) return cudaSuccess;
    const TpLayout& lay = p->view.lay;
    cudaError_t e = cudaMemset(p->local + lay.flag_base(), 0, lay.bytes() - lay.flag_base());
    if (e == cudaSuccess) e = cudaMemset(p->view.epoch, 0, 2 * sizeof(unsigned long long));
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    return e;
}

bool tp_peer_ready(const void* peer) { return peer && reinterpret_cast<const TpPeer*>(peer)->ready; }

void tp_peer_destroy(void* peer) {
    TpPeer* p = reinterpret_cast<TpPeer*>(peer);
    if (!p) return;
    for (int r = 0; r < kTpMaxRanks; ++r)
        if (p->opened[r]) cudaIpcCloseMemHandle(p->view.inbox[r]);
    cudaFree(p->local);
    cudaFree(p->view.epoch);
    cudaFree(p->view.done);
    delete p;
}

cudaError_t launch_tp_peer_max(void* peer, int slot, unsigned int* amax_cell, int batch, cudaStream_t s) {
    TpPeer* p = reinterpret_cast<TpPeer*>(peer);
    return launch_pdl(tp_max_exchange_kernel, dim3(1), dim3(256), 0, s, true, p->view, slot, amax_cell, batch);
}

cudaError_t launch_tp_peer_sum_residual(void* peer, int slot, const int32_t* acc, const unsigned int* amax_cell, float sw,
                                        int batch, int n, float* h, cudaStream_t s) {
    TpPeer* p = reinterpret_cast<TpPeer*>(peer);
    const int total4 = batch * n / 4;
    int grid = (total4 + 1023) / 1024;
    grid = grid < 1 ? 1 : (grid > 16 ? 16 : grid);
    return launch_pdl(tp_sum_residual_kernel, dim3(grid), dim3(256), 0, s, true, p->view, slot, acc, amax_cell, sw, batch, n, h);
}

cudaError_t launch_tp_residual(const int32_t* acc, const unsigned int* absmax, float sw, int m, int n, float* h,
                               cudaStream_t s, bool pdl) {
    dim3 grid((n + 1023) / 1024 < 16 ? (n + 1023) / 1024 : 16, m);
    return launch_pdl(tp_residual_kernel, grid, dim3(256), 0, s, pdl, acc, absmax, sw, n, h);
}

}  // namespace bt
