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
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include "bt_handles.cuh"
#include "bt_ptx.cuh"

namespace bt {

namespace {

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
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

cudaError_t launch_tp_residual(const int32_t* acc, const unsigned int* absmax, float sw, int m, int n, float* h,
                               cudaStream_t s, bool pdl) {
    dim3 grid((n + 1023) / 1024 < 16 ? (n + 1023) / 1024 : 16, m);
    return launch_pdl(tp_residual_kernel, grid, dim3(256), 0, s, pdl, acc, absmax, sw, n, h);
}

}  // namespace bt
