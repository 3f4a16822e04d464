// bitttt.hpp - C++ face of the C ABI in bitttt.h, with the class and method names of the
// reference engine (crates/rust_engine/src; RE below), so that host code written against the
// reference reads the same: PackedTensor::pack / unpack, BitLinear::load / precompute_packed /
// forward, AdaptiveBitLinear, TTTLayer::forward_update / forward_chunkwise, QuantizedKVCache::
// append / reset, BitLlama::forward_one.  Header only; every call goes through libbitttt_b200.so.
// Failures throw bitttt::Error carrying the status code and the library's message.
#ifndef BITTTT_HPP
#define BITTTT_HPP

#include <cstdint>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "bitttt.h"

namespace bitttt {

struct Error : std::runtime_error {
    bt_status status;
    Error(bt_status s, const std::string& msg) : std::runtime_error(msg), status(s) {}
};
inline void check(bt_status s) {
    if (s != BT_OK) throw Error(s, bt_last_error());
}

// RE/kernels/packing.rs:15-21
struct PackedTensor {
    std::vector<uint8_t> data;  // 4 weights per byte, row-major [out, in/4]
    float scale = 0.0f;
    std::vector<int64_t> shape;
    int64_t num_elem = 0;

    // PackedTensor::pack, RE/kernels/packing.rs:50-105
    static PackedTensor pack(const float* w, int64_t out_features, int64_t in_features) {
        PackedTensor p;
        p.num_elem = out_features * in_features;
        p.shape = {out_features, in_features};
        p.data.resize(static_cast<size_t>((p.num_elem + 3) / 4));
        check(bt_pack_ternary(w, p.num_elem, p.data.data(), &p.scale));
        return p;
    }
    // PackedTensor::new, RE/kernels/packing.rs:25-47
    static PackedTensor from_bytes(std::vector<uint8_t> bytes, std::vector<int64_t> shape, float scale) {
        PackedTensor p;
        p.data = std::move(bytes);
        p.shape = std::move(shape);
        p.scale = scale;
        p.num_elem = 1;
        for (int64_t d : p.shape) p.num_elem *= d;
        return p;
    }
    // PackedTensor::unpack, RE/kernels/packing.rs:108-133
    std::vector<float> unpack() const {
        std::vector<float> out(static_cast<size_t>(num_elem));
        check(bt_unpack_ternary(data.data(), num_elem, scale, out.data()));
        return out;
    }
};

// RE/layers/bit_linear.rs:13-96 (one basis) and RE/layers/adaptive_linear.rs:40-161 (several bases)
class BitLinear {
public:
    int64_t in_features = 0, out_features = 0;
    PackedTensor packed_params;  // empty for AdaptiveBitLinear handles built from a converted checkpoint

    BitLinear() = default;
    BitLinear(const BitLinear&) = delete;
    BitLinear& operator=(const BitLinear&) = delete;
    BitLinear(BitLinear&& o) noexcept { *this = std::move(o); }
    BitLinear& operator=(BitLinear&& o) noexcept {
        std::swap(h_, o.h_);
        std::swap(in_features, o.in_features);
        std::swap(out_features, o.out_features);
        std::swap(packed_params, o.packed_params);
        std::swap(weight_, o.weight_);
        return *this;
    }
    ~BitLinear() { if (h_) bt_linear_destroy(h_); }

    // BitLinear::load (RE/layers/bit_linear.rs:24-41): keeps the dense f32 weight until it is packed
    static BitLinear load(int64_t in_dim, int64_t out_dim, const float* weight, int device) {
        BitLinear l;
        l.in_features = in_dim;
        l.out_features = out_dim;
        l.device_ = device;
        l.weight_.assign(weight, weight + in_dim * out_dim);
        return l;
    }
    // BitLinear::precompute_packed (RE/layers/bit_linear.rs:44-50)
    void precompute_packed() {
        if (weight_.empty()) throw Error(BT_ERR_ARG, "precompute_packed: no dense weight loaded");
        packed_params = PackedTensor::pack(weight_.data(), out_features, in_features);
        check(bt_linear_create(&h_, packed_params.data.data(), out_features, in_features, 1, &packed_params.scale, device_));
        weight_.clear();
    }
    // AdaptiveBitLinear::load (RE/layers/adaptive_linear.rs:40-129): `weight_packed` [out, in/4, n_bases] + `scales`
    static BitLinear from_packed(const uint8_t* weight_packed, const float* scales, int n_bases, int64_t out_dim, int64_t in_dim,
                                 int device) {
        BitLinear l;
        l.in_features = in_dim;
        l.out_features = out_dim;
        l.device_ = device;
        check(bt_linear_create(&l.h_, weight_packed, out_dim, in_dim, n_bases, scales, device));
        return l;
    }
    // BitLinear::forward (RE/layers/bit_linear.rs:52-96) on device buffers: x [m, in_features] -> y [m, out_features]
    void forward(const void* x_dev, int64_t m, bt_dtype x_dtype, void* y_dev, bt_dtype y_dtype, void* stream = nullptr,
                 bt_workspace* ws = nullptr) const {
        if (!h_) throw Error(BT_ERR_ARG, "BitLinear::forward: weights are not packed; call precompute_packed()");
        check(bt_linear_forward(h_, ws, x_dev, m, in_features, x_dtype, y_dev, y_dtype, stream));
    }
    bt_linear* handle() const { return h_; }

private:
    bt_linear* h_ = nullptr;
    int device_ = 0;
    std::vector<float> weight_;
};
using AdaptiveBitLinear = BitLinear;

// The state update of TTTLayer (RE/layers/ttt.rs:48-119) between its down and up projections.
struct TTTLayer {
    // forward_update: one token per sequence; w_state [batch, d, d] updated in place, z = prediction with the old state
    static void forward_update(float* w_state_dev, const float* feat_dev, int64_t batch, int64_t d, float inner_lr, float* z_dev,
                               int device, void* stream = nullptr) {
        check(bt_ttt_update(w_state_dev, feat_dev, batch, 1, d, inner_lr, 1, z_dev, device, stream));
    }
    // forward_chunkwise: t_len tokens per sequence, one gradient step per `chunk_size` tokens
    static void forward_chunkwise(float* w_state_dev, const float* feat_dev, int64_t batch, int64_t t_len, int64_t d, float inner_lr,
                                  int64_t chunk_size, float* z_dev, int device, void* stream = nullptr) {
        check(bt_ttt_update(w_state_dev, feat_dev, batch, t_len, d, inner_lr, chunk_size, z_dev, device, stream));
    }
};

// RE/layers/kv_cache.rs:14-128
class QuantizedKVCache {
public:
    QuantizedKVCache(int64_t max_seq_len, int64_t batch, int64_t n_kv_heads, int64_t head_dim, int device) {
        check(bt_kv_create(&h_, batch, n_kv_heads, head_dim, max_seq_len, device));
    }
    QuantizedKVCache(const QuantizedKVCache&) = delete;
    QuantizedKVCache& operator=(const QuantizedKVCache&) = delete;
    ~QuantizedKVCache() { if (h_) bt_kv_destroy(h_); }
    void reset() { check(bt_kv_reset(h_)); }
    // append (:50-92): k, v [batch, n_kv_heads, head_dim] f32 on the device, keys already rotated
    void append(const float* k_dev, const float* v_dev, const int32_t* pos_dev, int64_t batch, void* stream = nullptr) {
        check(bt_kv_append(h_, k_dev, v_dev, pos_dev, batch, stream));
    }
    // RoPE + append + attention of one new token per sequence (BitAttention::forward, RE/layers/attention.rs:166-217)
    void attend(const float* qkv_dev, const int32_t* pos_dev, int64_t batch, int64_t n_heads, double rope_theta, float* out_dev,
                void* stream = nullptr) {
        check(bt_attn_decode(h_, qkv_dev, pos_dev, batch, n_heads, rope_theta, out_dev, stream));
    }
    bt_kv_cache* handle() const { return h_; }

private:
    bt_kv_cache* h_ = nullptr;
};

// RE/model/llama.rs:17-272 (the decode path): weights are handed over tensor by tensor, then finalize()
class BitLlama {
public:
    BitLlama(const bt_model_config& cfg, int device) { check(bt_model_create(&h_, &cfg, device)); }
    BitLlama(const BitLlama&) = delete;
    BitLlama& operator=(const BitLlama&) = delete;
    ~BitLlama() { if (h_) bt_model_destroy(h_); }
    void set_linear(int layer, bt_weight_kind kind, const uint8_t* packed, int64_t n_out, int64_t k_in, int n_bases, const float* scales) {
        check(bt_model_set_linear_bases(h_, layer, kind, packed, n_out, k_in, n_bases, scales));
    }
    void set_tensor(bt_tensor_kind kind, int layer, const float* data, int64_t n_elem, bt_dtype storage = BT_BF16) {
        check(bt_model_set_tensor_typed(h_, kind, layer, data, n_elem, storage));
    }
    void finalize() { check(bt_model_finalize(h_)); }
    void reset_kv_cache() { check(bt_model_reset(h_)); }  // RE/model/llama.rs:179-188
    int current_pos() const { return bt_model_pos(h_); }
    // forward_one (RE/model/llama.rs:201-272): host ids in; logits [batch, vocab] (optional) and greedy ids (optional) out
    void forward_one(const int32_t* tokens, int batch, float* logits, int32_t* next) { check(bt_model_forward_one(h_, tokens, batch, logits, next)); }
    // the CLI's prefill loop (RE/model/llama.rs:495-498) as one batched call
    void prefill(const int32_t* tokens, int batch, int n_tokens, float* logits, int32_t* next, int ttt_chunk = 1) {
        check(bt_model_prefill(h_, tokens, batch, n_tokens, ttt_chunk, logits, next));
    }
    bt_model* handle() const { return h_; }

private:
    bt_model* h_ = nullptr;
};

}  // namespace bitttt

#endif  // BITTTT_HPP
