// Launchers of the kernels that make up one decode step besides the ternary products.
#pragma once

#include "bt_common.cuh"

namespace bt {

enum RowPre : int { PRE_NONE = 0, PRE_RMSNORM = 1, PRE_SWIGLU = 2 };

// Also clears `n_clear` words at `clear` (the per-step absmax cells).
cudaError_t launch_embed(const int32_t* tokens, const __nv_bfloat16* table, int batch, int hidden,
                         int vocab, float* h, cudaStream_t stream, unsigned int* clear = nullptr,
                         int n_clear = 0, bool pdl = false, bool f16 = false);  // f16: the table holds IEEE halves, not bf16

// Row transform (none | RMSNorm | silu(gate)*up) + per-token absmax int8 quantisation.
// x: [batch, x_stride] f32 (PRE_SWIGLU: gate and up interleaved in groups of 8 rows, 2k values); q rows of q_stride
// bytes (multiple of 4, zero-filled beyond k; q may be null); v_out optional [batch, k]
// transformed row; qtc optional: the same int8 values in the tensor-core product's activation
// layout (k_tiles = padded k / 256), so that launch_gemm_tc can skip its own quantiser.
cudaError_t launch_row_quant(int pre, const float* x, int64_t x_stride, const float* w, float eps,
                             int batch, int k, int8_t* q, int64_t q_stride, float* s, int32_t* qsum,
                             float* v_out, cudaStream_t stream, int8_t* qtc = nullptr, int k_tiles = 0,
                             const unsigned int* amax_in = nullptr, unsigned int* amax_out = nullptr);

// h[i] += y[i], i < n
cudaError_t launch_residual_add(float* h, const float* y, int64_t n, cudaStream_t stream);

cudaError_t launch_argmax(const float* logits, int batch, int vocab, int32_t* out, cudaStream_t stream);

// Final RMSNorm fused into the dense lm_head, plus per-CTA arg-max candidates:
// logits[b, :] = lm_head . rmsnorm(h[b, :]); cand_val/cand_idx [batch, *n_cand].
cudaError_t launch_lm_head_fused(const __nv_bfloat16* w, const float* h, const float* norm_w, float eps,
                                 int batch, int hidden, int64_t vocab, float* logits, float* cand_val,
                                 int32_t* cand_idx, int* n_cand, int sm_count, cudaStream_t stream, bool pdl,
                                 bool f16 = false);  // f16: w holds IEEE halves, not bf16
// Reduces the candidates to the greedy pick per token and advances the positions.
cudaError_t launch_pick(const float* cand_val, const int32_t* cand_idx, int n_cand, int batch, int32_t* out,
                        int32_t* pos, int n_pos, cudaStream_t stream, bool pdl);
int lm_head_max_candidates(int sm_count);

// Tensor-core lm_head for batches above 8 (tcgen05, bf16 x (bf16 hi + bf16 lo), f32 accumulate).
size_t lm_head_tc_weight_bytes(int64_t vocab, int hidden);
size_t lm_head_tc_act_bytes(int hidden);
cudaError_t launch_lm_retile(const __nv_bfloat16* w, int64_t vocab, int hidden, void* tiles, cudaStream_t stream);
cudaError_t launch_lm_head_tc(const void* wtiles, const float* h, const float* norm_w, float eps, int batch, int hidden,
                              int64_t vocab, void* btiles, float* logits, unsigned int* err, int sm_count,
                              cudaStream_t stream, bool w_f16 = false);  // w_f16: the weight tiles hold IEEE halves

// Q8 KV cache of one layer: u8 data [batch, n_kv, max_seq, head_dim] and f32 scales
// [batch, n_kv, max_seq] for K and V (layers/kv_cache.rs:14-24).
struct KvCacheView {
    uint8_t* k_q;
    uint8_t* v_q;
    float* k_s;
    float* v_s;
    int max_seq;
};

// Fused decode attention for one new token per sequence: RoPE on q and k at position
// pos[b], Q8 append of k and v, attention of the n_heads queries over positions
// 0..pos[b] of the quantised cache, output [batch, n_heads*head_dim] f32.
// qkv: [batch, (n_heads + 2 n_kv) * head_dim] f32 laid out q | k | v.
struct AttnArgs {
    const float* qkv;
    KvCacheView cache;
    const int32_t* pos;      // [batch] position of the new token
    const float* rope_cos;   // [max_seq, head_dim/2] f32 tables (RotaryEmbedding::new, attention.rs:15-41)
    const float* rope_sin;
    float* out;              // [batch, n_heads*head_dim]
    int batch, n_heads, n_kv, head_dim;
    int q_rows;              // new tokens per sequence: 1 = decode; more = prefill (their K/V rows already appended,
                             // qkv / out rows ordered [sequence][token], pos[b] = position of the first new token)
    int sm_count;            // SMs of the device
    int splits;              // spans per sequence (grid.y) = CTAs of one thread-block cluster
    int span;                // positions per span, multiple of 32
    float scaling;
    unsigned int* absmax_out;  // optional [batch]: running max|out| (bits) via atomicMax
    bool pdl;                  // launch with programmatic stream serialisation
};
cudaError_t launch_attn_decode(const AttnArgs& a, cudaStream_t stream);
cudaError_t launch_row_quant_bf16(const __nv_bfloat16* x, int64_t x_stride, int batch, int k, float* s, int32_t* qsum,
                                  cudaStream_t stream, int8_t* qtc, int k_tiles);
// Spans per (sequence, KV head) and positions per span for a cache of max_seq positions; rep = query
// heads per KV head (selects the kernel instance whose cluster limit applies).
void attn_plan(int64_t batch, int64_t n_kv, int64_t max_seq, int sm_count, int rep, int* splits, int* span);
// Prefill: RoPE + Q8 append of the keys and values of q_rows new tokens per sequence (qkv rows [b][i]) at
// positions pos[b] + i.
cudaError_t launch_kv_append_rows(const KvCacheView& cache, const float* qkv, const int32_t* pos, const float* rope_cos,
                                  const float* rope_sin, int batch, int q_rows, int n_heads, int n_kv, int hd,
                                  cudaStream_t stream);
// QuantizedKVCache::append for one token per sequence: k, v [batch, n_kv, head_dim] f32 (already rotated)
// are quantised into row pos[b] of the cache.
cudaError_t launch_kv_append(const KvCacheView& cache, const float* k, const float* v, const int32_t* pos, int batch,
                             int n_kv, int hd, cudaStream_t stream);
// cos/sin tables for positions 0..max_seq-1: freq = f32(pos) * inv_freq (f32 product), cos/sin
// evaluated in f64 and rounded to f32.
cudaError_t launch_rope_tables(const float* inv_freq, int max_seq, int half, float* cos_t, float* sin_t,
                               cudaStream_t stream);

// TTT fast-weight step (layers/ttt.rs:52-68) for `batch` independent states:
// w: [batch, d, d] f32 updated in place, feat: [batch, d], z_out: [batch, d].
cudaError_t launch_ttt_step(float* w, const float* feat, int batch, int d, float lr, float* z_out,
                            cudaStream_t stream, unsigned int* absmax_out = nullptr, bool pdl = false);
// Chunked form (layers/ttt.rs:88-113): feats [batch, t_len, d], z_out [batch, t_len, d].
cudaError_t launch_ttt_chunk(float* w, const float* feats, int batch, int t_len, int d, float lr,
                             int chunk, float* z_out, cudaStream_t stream, unsigned int* absmax_out = nullptr,
                             bool pdl = false);

}  // namespace bt
