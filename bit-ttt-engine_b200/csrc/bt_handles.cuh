// Definitions of the opaque handle types shared between the C-ABI translation units.
#pragma once

#include <mutex>

#include "bt_model.cuh"

struct bt_workspace {
    int device = 0;
    uint8_t* base = nullptr;
    size_t bytes = 0;
};

struct bt_linear {
    int device = 0;
    bt::TiledWeights w;
    uint8_t* tiles = nullptr;
    float* scale_tiles = nullptr;  // device [n_bases][row_tiles]
    float scales[8] = {0};
    bt_workspace* own_ws = nullptr;
    std::mutex ws_mu;
    bt::LinearDev dev() const {
        bt::LinearDev d;
        d.w = w;
        d.scale_tiles = scale_tiles;
        return d;
    }
};

struct bt_kv_cache {
    int device = 0;
    int64_t batch = 0, n_kv = 0, head_dim = 0, max_seq = 0;
    bt::KvCacheView view{};
    float* inv_freq = nullptr;   // device [head_dim/2], built for inv_freq_theta
    double inv_freq_theta = 0.0;
    float* rope_cos = nullptr;   // device [max_seq, head_dim/2] for inv_freq_theta
    float* rope_sin = nullptr;
    int max_heads = 0;
};

namespace bt {
// Gate and up projections of a SwiGLU block as ONE BitLinear whose row tiles hold 8 gate
// rows followed by the 8 matching up rows, so that the product's epilogue sees gate[j] and
// up[j] in the same thread and can emit silu(gate)*up directly (EPI_SWIGLU).
bt_status create_gate_up(bt_linear** out, const uint8_t* gate_packed_host, const uint8_t* up_packed_host,
                         int64_t rows, int64_t k_in, int n_bases, const float* gate_scales, const float* up_scales,
                         int device);
}  // namespace bt

namespace bt {
// tensor-parallel plumbing (tp.cu)
bt_status tp_unique_id(void* out128);
bt_status tp_comm_init(void** comm, const void* id128, int rank, int size);
void tp_comm_destroy(void* comm);
bt_status tp_allreduce_max_f32(void* comm, float* buf, size_t count, cudaStream_t s);
bt_status tp_allreduce_sum_i32(void* comm, int32_t* buf, size_t count, cudaStream_t s);
bool tp_allgather_available();
bt_status tp_allgather_f32(void* comm, float* buf, size_t count, int rank, cudaStream_t s);
cudaError_t launch_tp_logits_rows(const float* parts, int tp, int batch, int64_t vl, int64_t vocab, float* full, cudaStream_t s);
cudaError_t launch_tp_residual(const int32_t* acc, const unsigned int* absmax, float sw, int m, int n, float* h,
                               cudaStream_t s, bool pdl);
// exchange over NVLink peer memory (CUDA IPC between the ranks' processes) instead of NCCL
bt_status tp_peer_create(void** out, int rank, int size, int max_batch, int hidden, unsigned int* err);
bt_status tp_peer_export(void* peer, void* handle64_out);
bt_status tp_peer_import(void* peer, const void* handles /* [size][64] */);
bool tp_peer_ready(const void* peer);
void tp_peer_set_wait(void* peer, unsigned long long ns);
cudaError_t tp_peer_reset(void* peer);
void tp_peer_destroy(void* peer);
cudaError_t launch_tp_peer_max(void* peer, int slot, unsigned int* amax_cell, int batch, cudaStream_t s);
cudaError_t launch_tp_peer_sum_residual(void* peer, int slot, const int32_t* acc, const unsigned int* amax_cell, float sw,
                                        int batch, int n, float* h, cudaStream_t s);
}  // namespace bt
