// extern "C" entry points for the TTT fast-weight update, the Q8 KV cache and decode
// attention.
#include <math.h>

#include <new>
#include <vector>

#include "bt_handles.cuh"

using namespace bt;

namespace bt {

// inv_freq[i] = 1 / theta^(2i/hd) evaluated in f64, cast to f32
// (RotaryEmbedding::new, layers/attention.rs:19-22).
cudaError_t upload_inv_freq(float* dev, int head_dim, double theta) {
    std::vector<float> host((size_t)head_dim / 2);
    for (int i = 0; i < head_dim / 2; ++i)
        host[(size_t)i] = (float)(1.0 / pow(theta, (double)(2 * i) / (double)head_dim));
    return cudaMemcpy(dev, host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice);
}

}  // namespace bt

extern "C" bt_status bt_ttt_update(float* w_state_dev, const float* feat_dev, int64_t batch, int64_t t_len,
                                   int64_t d, float inner_lr, int64_t chunk, float* z_dev, int device,
                                   void* stream) {
    if (!w_state_dev || !feat_dev || !z_dev) return set_error(BT_ERR_ARG, "bt_ttt_update: null pointer");
    if (batch < 0 || t_len < 0 || d < 1 || d > 1024)
        return set_error(BT_ERR_SHAPE, "bt_ttt_update: bad shape batch=%lld t_len=%lld d=%lld (d must be 1..1024)",
                         (long long)batch, (long long)t_len, (long long)d);
    if (chunk < 1 || chunk > 64 || chunk * d * 4 > 200 * 1024)
        return set_error(BT_ERR_ARG, "bt_ttt_update: chunk %lld unsupported for d=%lld (1..64, chunk*d*4 <= 200 KiB)",
                         (long long)chunk, (long long)d);
    if (batch == 0 || t_len == 0) return BT_OK;
    DeviceGuard guard(device);
    if (!guard.ok) return set_error(BT_ERR_DEVICE, "cannot select device %d", device);
    BT_CUDA_TRY(launch_ttt_chunk(w_state_dev, feat_dev, (int)batch, (int)t_len, (int)d, inner_lr, (int)chunk, z_dev,
                                 reinterpret_cast<cudaStream_t>(stream)));
    return BT_OK;
}

extern "C" bt_status bt_kv_create(bt_kv_cache** out, int64_t batch, int64_t n_kv_heads, int64_t head_dim,
                                  int64_t max_seq_len, int device) {
    if (!out) return set_error(BT_ERR_ARG, "bt_kv_create: null out pointer");
    *out = nullptr;
    if (batch < 1 || n_kv_heads < 1 || max_seq_len < 1)
        return set_error(BT_ERR_SHAPE, "bt_kv_create: bad shape");
    if (head_dim % 32 != 0 || head_dim < 32 || head_dim > 128)
        return set_error(BT_ERR_SHAPE, "bt_kv_create: head_dim %lld must be 32, 64, 96 or 128", (long long)head_dim);
    if (bt_device_count() <= device || device < 0) return set_error(BT_ERR_DEVICE, "bt_kv_create: no CUDA device %d", device);
    DeviceGuard guard(device);
    if (!guard.ok) return set_error(BT_ERR_DEVICE, "cannot select device %d", device);
    bt_kv_cache* c = new (std::nothrow) bt_kv_cache();
    if (!c) return set_error(BT_ERR_NOMEM, "host allocation failed");
    c->device = device;
    c->batch = batch; c->n_kv = n_kv_heads; c->head_dim = head_dim; c->max_seq = max_seq_len;
    const size_t rows = (size_t)batch * n_kv_heads * max_seq_len;
    c->max_heads = (int)n_kv_heads * 8;
    cudaError_t e = cudaMalloc(&c->view.k_q, rows * head_dim);
    if (e == cudaSuccess) e = cudaMalloc(&c->view.v_q, rows * head_dim);
    if (e == cudaSuccess) e = cudaMalloc(&c->view.k_s, rows * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&c->view.v_s, rows * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&c->inv_freq, (size_t)head_dim / 2 * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&c->rope_cos, (size_t)max_seq_len * (head_dim / 2) * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&c->rope_sin, (size_t)max_seq_len * (head_dim / 2) * sizeof(float));
    c->view.max_seq = (int)max_seq_len;
    if (e != cudaSuccess) {
        bt_kv_destroy(c);
        return set_error(BT_ERR_NOMEM, "bt_kv_create: %s", cudaGetErrorString(e));
    }
    *out = c;
    return bt_kv_reset(c);
}

extern "C" bt_status bt_kv_reset(bt_kv_cache* c) {
    if (!c) return set_error(BT_ERR_ARG, "bt_kv_reset: null handle");
    DeviceGuard guard(c->device);
    const size_t rows = (size_t)c->batch * c->n_kv * c->max_seq;
    BT_CUDA_TRY(cudaMemset(c->view.k_q, 128, rows * c->head_dim));
    BT_CUDA_TRY(cudaMemset(c->view.v_q, 128, rows * c->head_dim));
    BT_CUDA_TRY(cudaMemset(c->view.k_s, 0, rows * sizeof(float)));
    BT_CUDA_TRY(cudaMemset(c->view.v_s, 0, rows * sizeof(float)));
    return BT_OK;
}

extern "C" bt_status bt_kv_destroy(bt_kv_cache* c) {
    if (!c) return BT_OK;
    DeviceGuard guard(c->device);
    cudaFree(c->view.k_q); cudaFree(c->view.v_q); cudaFree(c->view.k_s); cudaFree(c->view.v_s);
    cudaFree(c->inv_freq); cudaFree(c->rope_cos); cudaFree(c->rope_sin);
    delete c;
    return BT_OK;
}

extern "C" bt_status bt_kv_export(bt_kv_cache* c, int64_t b, int64_t t_len, uint8_t* k_q_host, float* k_s_host,
                                  uint8_t* v_q_host, float* v_s_host) {
    if (!c) return set_error(BT_ERR_ARG, "bt_kv_export: null handle");
    if (b < 0 || b >= c->batch || t_len < 0 || t_len > c->max_seq)
        return set_error(BT_ERR_SHAPE, "bt_kv_export: sequence %lld / length %lld out of range", (long long)b, (long long)t_len);
    DeviceGuard guard(c->device);
    BT_CUDA_TRY(cudaDeviceSynchronize());
    for (int64_t h = 0; h < c->n_kv; ++h) {
        const size_t row0 = ((size_t)b * c->n_kv + h) * c->max_seq;
        const size_t o = (size_t)h * t_len;
        if (k_q_host) BT_CUDA_TRY(cudaMemcpy(k_q_host + o * c->head_dim, c->view.k_q + row0 * c->head_dim, (size_t)t_len * c->head_dim, cudaMemcpyDeviceToHost));
        if (v_q_host) BT_CUDA_TRY(cudaMemcpy(v_q_host + o * c->head_dim, c->view.v_q + row0 * c->head_dim, (size_t)t_len * c->head_dim, cudaMemcpyDeviceToHost));
        if (k_s_host) BT_CUDA_TRY(cudaMemcpy(k_s_host + o, c->view.k_s + row0, (size_t)t_len * sizeof(float), cudaMemcpyDeviceToHost));
        if (v_s_host) BT_CUDA_TRY(cudaMemcpy(v_s_host + o, c->view.v_s + row0, (size_t)t_len * sizeof(float), cudaMemcpyDeviceToHost));
    }
    return BT_OK;
}

extern "C" bt_status bt_kv_import(bt_kv_cache* c, int64_t b, int64_t t_len, const uint8_t* k_q_host, const float* k_s_host,
                                  const uint8_t* v_q_host, const float* v_s_host) {
    if (!c) return set_error(BT_ERR_ARG, "bt_kv_import: null handle");
    if (b < 0 || b >= c->batch || t_len < 0 || t_len > c->max_seq)
        return set_error(BT_ERR_SHAPE, "bt_kv_import: sequence %lld / length %lld out of range", (long long)b, (long long)t_len);
    DeviceGuard guard(c->device);
    BT_CUDA_TRY(cudaDeviceSynchronize());
    for (int64_t h = 0; h < c->n_kv; ++h) {
        const size_t row0 = ((size_t)b * c->n_kv + h) * c->max_seq;
        const size_t o = (size_t)h * t_len;
        if (k_q_host) BT_CUDA_TRY(cudaMemcpy(c->view.k_q + row0 * c->head_dim, k_q_host + o * c->head_dim, (size_t)t_len * c->head_dim, cudaMemcpyHostToDevice));
        if (v_q_host) BT_CUDA_TRY(cudaMemcpy(c->view.v_q + row0 * c->head_dim, v_q_host + o * c->head_dim, (size_t)t_len * c->head_dim, cudaMemcpyHostToDevice));
        if (k_s_host) BT_CUDA_TRY(cudaMemcpy(c->view.k_s + row0, k_s_host + o, (size_t)t_len * sizeof(float), cudaMemcpyHostToDevice));
        if (v_s_host) BT_CUDA_TRY(cudaMemcpy(c->view.v_s + row0, v_s_host + o, (size_t)t_len * sizeof(float), cudaMemcpyHostToDevice));
    }
    return BT_OK;
}

extern "C" bt_status bt_kv_append(bt_kv_cache* c, const float* k_dev, const float* v_dev, const int32_t* pos_dev,
                                  int64_t batch, void* stream) {
    if (!c || !k_dev || !v_dev || !pos_dev) return set_error(BT_ERR_ARG, "bt_kv_append: null pointer");
    if (batch < 1 || batch > c->batch) return set_error(BT_ERR_SHAPE, "bt_kv_append: batch %lld exceeds the cache's %lld", (long long)batch, (long long)c->batch);
    DeviceGuard guard(c->device);
    if (!guard.ok) return set_error(BT_ERR_DEVICE, "cannot select device %d", c->device);
    BT_CUDA_TRY(launch_kv_append(c->view, k_dev, v_dev, pos_dev, (int)batch, (int)c->n_kv, (int)c->head_dim,
                                 reinterpret_cast<cudaStream_t>(stream)));
    return BT_OK;
}

extern "C" bt_status bt_attn_decode(bt_kv_cache* c, const float* qkv_dev, const int32_t* pos_dev, int64_t batch,
                                    int64_t n_heads, double rope_theta, float* out_dev, void* stream) {
    if (!c || !qkv_dev || !pos_dev || !out_dev) return set_error(BT_ERR_ARG, "bt_attn_decode: null pointer");
    if (batch < 1 || batch > c->batch) return set_error(BT_ERR_SHAPE, "bt_attn_decode: batch %lld exceeds the cache's %lld", (long long)batch, (long long)c->batch);
    const int64_t rep = n_heads / c->n_kv;
    if (n_heads % c->n_kv != 0 || !(rep == 1 || rep == 2 || rep == 4 || rep == 8) || n_heads > c->max_heads)
        return set_error(BT_ERR_SHAPE, "bt_attn_decode: %lld query heads over %lld KV heads unsupported (group size 1, 2, 4 or 8)", (long long)n_heads, (long long)c->n_kv);
    DeviceGuard guard(c->device);
    if (!guard.ok) return set_error(BT_ERR_DEVICE, "cannot select device %d", c->device);
    if (c->inv_freq_theta != rope_theta) {
        BT_CUDA_TRY(cudaDeviceSynchronize());
        BT_CUDA_TRY(upload_inv_freq(c->inv_freq, (int)c->head_dim, rope_theta));
        BT_CUDA_TRY(launch_rope_tables(c->inv_freq, (int)c->max_seq, (int)c->head_dim / 2, c->rope_cos, c->rope_sin, 0));
        BT_CUDA_TRY(cudaDeviceSynchronize());
        c->inv_freq_theta = rope_theta;
    }
    AttnArgs a;
    a.qkv = qkv_dev;
    a.cache = c->view;
    a.pos = pos_dev;
    a.rope_cos = c->rope_cos;
    a.rope_sin = c->rope_sin;
    a.out = out_dev;
    a.batch = (int)batch; a.n_heads = (int)n_heads; a.n_kv = (int)c->n_kv; a.head_dim = (int)c->head_dim; a.q_rows = 1;
    a.sm_count = device_sm_count(c->device);
    attn_plan(batch, c->n_kv, c->max_seq, a.sm_count, (int)rep, &a.splits, &a.span);
    a.scaling = (float)(1.0 / sqrt((double)c->head_dim));  // layers/attention.rs:114
    a.absmax_out = nullptr;
    a.pdl = false;
    BT_CUDA_TRY(launch_attn_decode(a, reinterpret_cast<cudaStream_t>(stream)));
    return BT_OK;
}
