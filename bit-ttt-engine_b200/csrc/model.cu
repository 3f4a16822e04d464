// bt_model: one decode step of the reference's BitLlama (model/llama.rs:201-272,
// model/block.rs:87-134) as a fixed sequence of this library's kernels on one stream,
// replayed as a CUDA graph once captured.  Host code here only owns buffers and order;
// all arithmetic is in the kernels.
#include <string.h>

#include <new>
#include <vector>

#include "bt_handles.cuh"

using namespace bt;

__global__ void set_pos_kernel(int32_t* pos, int n, int value) {
    if (threadIdx.x < n) pos[threadIdx.x] = value;
}

namespace bt {
cudaError_t upload_inv_freq(float* dev, int head_dim, double theta);

__global__ void advance_pos_kernel(int32_t* pos, int n) {
    if (threadIdx.x < n) pos[threadIdx.x] += 1;
}
// f32 -> the 16-bit storage type of the dense tables: bf16, or IEEE half (same 2 bytes per element)
__global__ void f32_to_16bit_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, int64_t n, bool f16) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        if (f16) reinterpret_cast<__half*>(out)[i] = __float2half_rn(in[i]);
        else out[i] = __float2bfloat16_rn(in[i]);
    }
}
}  // namespace bt

namespace {

constexpr float kRmsEps = 1e-5f;  // model/block.rs:10, model/llama.rs:13

struct HostLinear {
    std::vector<uint8_t> packed;  // [n_out, k_in/4, n_bases]
    int64_t n_out = 0, k_in = 0;
    int n_bases = 1;
    float scales[8] = {0};
    bool set = false;
};

struct Layer {
    HostLinear host[9];
    bt_linear* qkv = nullptr;
    bt_linear* o = nullptr;
    bt_linear* gate_up_il = nullptr;   // gate/up interleaved by 8 rows (fused SwiGLU epilogue; SwiGLU row kernel)
    bt_linear* down = nullptr;
    bt_linear* ttt_down = nullptr;
    bt_linear* ttt_up = nullptr;
    float* norm1 = nullptr;
    float* norm2 = nullptr;
    bt_kv_cache* kv = nullptr;
    float* w_state = nullptr;  // [max_batch, d, d]
};

}  // namespace

struct bt_model {
    bt_model_config cfg{};
    int device = 0;
    int sm_count = 0;
    int head_dim = 0, d_small = 0, qkv_dim = 0;
    int tp = 1;                      // tensor-parallel degree
    int nh_l = 0, nkv_l = 0, i_l = 0;  // this rank's query heads, KV heads, MLP columns
    void* comm = nullptr;            // NCCL communicator when tp > 1
    void* peer = nullptr;            // peer-memory exchange (CUDA IPC inboxes) when the ranks have set it up
    int32_t* acc_i32 = nullptr;      // [max_batch, hidden] accumulators of a row-parallel projection
    bool finalized = false;
    bool multi_basis = false;        // a projection has several bases: the step runs quantiser and product kernels separately
    std::vector<Layer> layers;
    __nv_bfloat16* embed = nullptr;   // 16-bit storage: bf16, or IEEE half when embed_f16
    __nv_bfloat16* lm_head = nullptr;
    bool embed_f16 = false, head_f16 = false;
    float* norm_f = nullptr;
    float* inv_freq = nullptr;
    float* rope_cos = nullptr;   // [max_pos, head_dim/2]
    float* rope_sin = nullptr;
    // activations
    int32_t* tokens = nullptr;
    int32_t* pos = nullptr;
    float* h = nullptr;
    int8_t* q = nullptr;
    int64_t q_stride = 0;
    float* sx = nullptr;
    int32_t* qsum = nullptr;
    float* qkv = nullptr;
    float* att = nullptr;
    float* gu = nullptr;
    float* feat = nullptr;
    float* z = nullptr;
    float* xn = nullptr;
    float* logits = nullptr;
    int32_t* next = nullptr;
    float* act = nullptr;            // [max_batch, intermediate] silu(gate)*up
    float* xt = nullptr;             // [max_batch, max(hidden, intermediate)] transformed rows (batches above 8)
    int8_t* qtc = nullptr;           // activations in the tensor-core product's layout (batches above 8)
    void* lm_tiles = nullptr;        // lm_head in tensor-core tile order (batches above 8, hidden % 64 == 0)
    void* lm_btiles = nullptr;       // normalised hidden states as bf16 hi|lo tiles
    float* lm_gather = nullptr;      // tensor parallelism: the ranks' vocabulary slices of the logits, [tp][batch][vl]
    int64_t vl = 0;                  // rows of the head per rank (multiple of 128)
    unsigned int* absmax = nullptr;  // [num_layers][2][max_batch] max|x| cells of the fused path
    float* cand_val = nullptr;
    int32_t* cand_idx = nullptr;
    int32_t* tokens_pinned = nullptr;
    int32_t* next_pinned = nullptr;
    float* trace = nullptr;          // inspection aid: per-layer intermediate tensors of a step (caller's device buffer)
    int trace_rows = 0;              // rows per tensor the trace buffer was sized for
    // prefill scratch (allocated at the first bt_model_prefill, for pf_rows = sequences x tokens of a chunk)
    int pf_rows = 0;
    int32_t* pf_tokens = nullptr;
    float* pf_h = nullptr;
    float* pf_qkv = nullptr;
    float* pf_att = nullptr;
    float* pf_gu = nullptr;
    float* pf_act = nullptr;         // silu(gate)*up rows, only while a trace is recorded
    int pf_act_rows = 0;
    int8_t* pf_qtc = nullptr;
    float* pf_sx = nullptr;
    int32_t* pf_qsum = nullptr;
    std::vector<int32_t> pf_host;
    unsigned int* err_pinned = nullptr;  // tensor parallel: the device error word as read after a step
    int host_pos = 0;
    int64_t ternary_bytes = 0;
    cudaStream_t stream = nullptr;
    cudaGraphExec_t graphs[65] = {nullptr};
};

namespace {

template <typename T>
cudaError_t dev_alloc(T** p, size_t count) { return cudaMalloc(reinterpret_cast<void**>(p), count * sizeof(T)); }

// One BitLinear from 1..3 projections that share their input, stacked along the output rows; every part in the
// checkpoint layout [rows, k_in/4, n_bases] with its own scale per basis (the parts agree on n_bases).
bt_status make_linear(bt_model* m, HostLinear** parts, int n_parts, bt_linear** out) {
    int64_t rows_total = 0;
    for (int i = 0; i < n_parts; ++i) {
        if (!parts[i]->set) return set_error(BT_ERR_ARG, "bt_model_finalize: a projection weight was never set");
        if (parts[i]->k_in != parts[0]->k_in) return set_error(BT_ERR_SHAPE, "bt_model_finalize: fused projections disagree on in_features");
        if (parts[i]->n_bases != parts[0]->n_bases) return set_error(BT_ERR_SHAPE, "bt_model_finalize: fused projections disagree on the number of bases");
        if (n_parts > 1 && parts[i]->n_out % kTileRows != 0)
            return set_error(BT_ERR_ALIGN, "bt_model_finalize: a fused projection has %lld rows (need a multiple of 16)", (long long)parts[i]->n_out);
        rows_total += parts[i]->n_out;
    }
    const int nb = parts[0]->n_bases;
    const size_t row_bytes = (size_t)(parts[0]->k_in / 4) * nb;
    bt_status st;
    if (n_parts == 1) {
        st = bt_linear_create(out, parts[0]->packed.data(), rows_total, parts[0]->k_in, nb, parts[0]->scales, m->device);
    } else {
        std::vector<uint8_t> cat((size_t)rows_total * row_bytes);
        size_t off = 0;
        for (int i = 0; i < n_parts; ++i) {
            memcpy(cat.data() + off, parts[i]->packed.data(), (size_t)parts[i]->n_out * row_bytes);
            off += (size_t)parts[i]->n_out * row_bytes;
        }
        st = bt_linear_create(out, cat.data(), rows_total, parts[0]->k_in, nb, parts[0]->scales, m->device);
        if (st == BT_OK) {
            // one weight scale per (basis, half row tile): every part brings its own
            const int64_t rt2 = (*out)->w.row_tiles * 2;
            std::vector<float> host((size_t)nb * rt2);
            for (int b = 0; b < nb; ++b) {
                int64_t r = 0;
                for (int i = 0; i < n_parts; ++i)
                    for (int64_t k = 0; k < parts[i]->n_out / kTileRows * 2; ++k) host[(size_t)b * rt2 + r++] = parts[i]->scales[b];
            }
            cudaError_t e = cudaMemcpy((*out)->scale_tiles, host.data(), host.size() * sizeof(float), cudaMemcpyHostToDevice);
            if (e != cudaSuccess) return set_error(BT_ERR_CUDA, "bt_model_finalize: %s", cudaGetErrorString(e));
        }
    }
    if (st != BT_OK) return st;
    m->ternary_bytes += (*out)->w.basis_stride() * nb;
    for (int i = 0; i < n_parts; ++i) { parts[i]->packed.clear(); parts[i]->packed.shrink_to_fit(); }
    return BT_OK;
}

// One decode step for up to 8 sequences with the quantisers folded into the product
// kernels and every launch allowed to start early (programmatic dependent launch):
// per block  [norm1+quant+q|k|v]  [attention]  [combine]  [quant+o_proj+residual]
//            [norm2+quant+gate|up+SiLU*up]  [quant+down+residual].
// Three to eight sequences: the fused product would repeat its per-CTA quantisation prologue for
// every token in every CTA (3 us per token for the 14336 inputs of down_proj), so the rows are
// quantised once by a kernel of their own (one CTA per row) and the product reads them.
constexpr int kSplitQuantBatch = 3;
bt_status quant_then_product(bt_model* m, bt_linear* lin, int pre, const float* x, int64_t x_stride, const float* w,
                             int k, int batch, void* out, int64_t out_stride, int epilogue, unsigned int* absmax_out,
                             unsigned int* err, cudaStream_t s) {
    const int64_t qs = ((int64_t)k + kTileK - 1) / kTileK * kTileK;
    BT_CUDA_TRY(launch_row_quant(pre, x, x_stride, w, kRmsEps, batch, k, m->q, qs, m->sx, m->qsum, nullptr, s));
    BT_CUDA_TRY(linear_product_q(lin->dev(), m->q, qs, m->qsum, m->sx, batch, out, out_stride, epilogue, absmax_out, err,
                                 m->sm_count, s));
    return BT_OK;
}

// Trace layout: [layer][h_in | qkv | att | h_mid | act | h_out], every part [max_batch, width] f32.
// arch ttt: the "qkv" part holds the down-projected features and "att" the TTT prediction z.
enum TraceSlot { TR_H_IN = 0, TR_QKV, TR_ATT, TR_H_MID, TR_ACT, TR_H_OUT, TR_SLOTS };
void trace_widths(const bt_model* m, int64_t (&w)[TR_SLOTS]) {
    const int64_t H = m->cfg.hidden_dim;
    w[TR_H_IN] = H;
    w[TR_QKV] = m->cfg.arch == 1 ? m->qkv_dim : m->d_small;
    w[TR_ATT] = m->cfg.arch == 1 ? (int64_t)m->nh_l * m->head_dim : m->d_small;
    w[TR_H_MID] = H;
    w[TR_ACT] = m->i_l;
    w[TR_H_OUT] = H;
}
int64_t trace_layer_floats(const bt_model* m, int rows) {
    int64_t w[TR_SLOTS], n = 0;
    trace_widths(m, w);
    for (int i = 0; i < TR_SLOTS; ++i) n += w[i] * rows;
    return n;
}
cudaError_t trace_copy(const bt_model* m, int layer, int slot, const float* src, int rows, cudaStream_t s) {
    if (!m->trace) return cudaSuccess;
    if (rows > m->trace_rows) return cudaErrorInvalidValue;
    int64_t w[TR_SLOTS], off = 0;
    trace_widths(m, w);
    for (int i = 0; i < slot; ++i) off += w[i] * m->trace_rows;
    float* dst = m->trace + (int64_t)layer * trace_layer_floats(m, m->trace_rows) + off;
    return cudaMemcpyAsync(dst, src, (size_t)rows * w[slot] * sizeof(float), cudaMemcpyDeviceToDevice, s);
}

bt_status enqueue_head(bt_model* m, int batch, cudaStream_t s, bool fused_launches);

bt_status enqueue_step_fused(bt_model* m, int batch, cudaStream_t s) {
    const bt_model_config& c = m->cfg;
    const int H = c.hidden_dim, I = m->i_l, B = c.max_batch;
    const int att_dim = m->nh_l * m->head_dim;  // this rank's attention output width
    unsigned int* err = device_error_word(m->device);
    const int sm = m->sm_count;
    const bool split_quant = m->tp == 1 && c.arch == 1 && batch >= kSplitQuantBatch;
    bt_status qst;
    BT_CUDA_TRY(launch_embed(m->tokens, m->embed, batch, H, c.vocab_size, m->h, s, m->absmax, c.num_layers * 2 * B, true, m->embed_f16));
    for (int li = 0; li < c.num_layers; ++li) {
        Layer& L = m->layers[(size_t)li];
        unsigned int* amax_core = m->absmax + ((size_t)li * 2 + 0) * B;
        unsigned int* amax_mlp = m->absmax + ((size_t)li * 2 + 1) * B;
        FusedIn norm1{PRO_RMSNORM, m->h, H, L.norm1, kRmsEps, nullptr};
        BT_CUDA_TRY(trace_copy(m, li, TR_H_IN, m->h, batch, s));
        if (c.arch == 0) {
            BT_CUDA_TRY(linear_product_fused(L.ttt_down->dev(), norm1, batch, m->feat, m->d_small, EPI_F32, nullptr, err, sm, s));
            BT_CUDA_TRY(trace_copy(m, li, TR_QKV, m->feat, batch, s));
            BT_CUDA_TRY(launch_ttt_step(L.w_state, m->feat, batch, m->d_small, c.inner_lr, m->z, s, amax_core, true));
            BT_CUDA_TRY(trace_copy(m, li, TR_ATT, m->z, batch, s));
            FusedIn zin{PRO_ABSMAX, m->z, m->d_small, nullptr, 0.f, amax_core};
            BT_CUDA_TRY(linear_product_fused(L.ttt_up->dev(), zin, batch, m->h, H, EPI_F32_ACCUM, nullptr, err, sm, s));
        } else {
            if (split_quant) {
                if ((qst = quant_then_product(m, L.qkv, PRE_RMSNORM, m->h, H, L.norm1, H, batch, m->qkv, m->qkv_dim, EPI_F32, nullptr, err, s)) != BT_OK) return qst;
            } else {
                BT_CUDA_TRY(linear_product_fused(L.qkv->dev(), norm1, batch, m->qkv, m->qkv_dim, EPI_F32, nullptr, err, sm, s));
            }
            AttnArgs a;
            a.qkv = m->qkv;
            a.cache = L.kv->view;
            a.pos = m->pos;
            a.rope_cos = m->rope_cos;
            a.rope_sin = m->rope_sin;
            a.out = m->att;
            a.batch = batch; a.n_heads = m->nh_l; a.n_kv = m->nkv_l; a.head_dim = m->head_dim; a.q_rows = 1;
            a.sm_count = sm;
            attn_plan(batch, m->nkv_l, c.max_position_embeddings, sm, m->nh_l / m->nkv_l, &a.splits, &a.span);
            a.scaling = (float)(1.0 / sqrt((double)m->head_dim));
            a.absmax_out = amax_core;
            a.pdl = true;
            BT_CUDA_TRY(trace_copy(m, li, TR_QKV, m->qkv, batch, s));
            BT_CUDA_TRY(launch_attn_decode(a, s));
            BT_CUDA_TRY(trace_copy(m, li, TR_ATT, m->att, batch, s));
            FusedIn ain{PRO_ABSMAX, m->att, att_dim, nullptr, 0.f, amax_core};
            if (m->tp > 1 && tp_peer_ready(m->peer)) {
                // row-parallel over NVLink peer memory: max of the quantisation scale, then the integer
                // sum fused with the scale epilogue and the residual
                BT_CUDA_TRY(launch_tp_peer_max(m->peer, 0, amax_core, batch, s));
                BT_CUDA_TRY(linear_product_fused(L.o->dev(), ain, batch, m->acc_i32, H, EPI_I32, nullptr, err, sm, s));
                BT_CUDA_TRY(launch_tp_peer_sum_residual(m->peer, 0, m->acc_i32, amax_core, L.o->scales[0], batch, H, m->h, s));
            } else if (m->tp > 1) {
                // row-parallel: same quantisation scale on every rank, integer sum over the ranks
                bt_status st = tp_allreduce_max_f32(m->comm, reinterpret_cast<float*>(amax_core), (size_t)batch, s);
                if (st != BT_OK) return st;
                BT_CUDA_TRY(linear_product_fused(L.o->dev(), ain, batch, m->acc_i32, H, EPI_I32, nullptr, err, sm, s));
                if ((st = tp_allreduce_sum_i32(m->comm, m->acc_i32, (size_t)batch * H, s)) != BT_OK) return st;
                BT_CUDA_TRY(launch_tp_residual(m->acc_i32, amax_core, L.o->scales[0], batch, H, m->h, s, true));
            } else if (split_quant) {
                if ((qst = quant_then_product(m, L.o, PRE_NONE, m->att, att_dim, nullptr, att_dim, batch, m->h, H, EPI_F32_ACCUM, nullptr, err, s)) != BT_OK) return qst;
            } else {
                BT_CUDA_TRY(linear_product_fused(L.o->dev(), ain, batch, m->h, H, EPI_F32_ACCUM, nullptr, err, sm, s));
            }
        }
        FusedIn norm2{PRO_RMSNORM, m->h, H, L.norm2, kRmsEps, nullptr};
        BT_CUDA_TRY(trace_copy(m, li, TR_H_MID, m->h, batch, s));
        if (split_quant) {
            if ((qst = quant_then_product(m, L.gate_up_il, PRE_RMSNORM, m->h, H, L.norm2, H, batch, m->act, I, EPI_SWIGLU, amax_mlp, err, s)) != BT_OK) return qst;
        } else {
            BT_CUDA_TRY(linear_product_fused(L.gate_up_il->dev(), norm2, batch, m->act, I, EPI_SWIGLU, amax_mlp, err, sm, s));
        }
        FusedIn din{PRO_ABSMAX, m->act, I, nullptr, 0.f, amax_mlp};
        BT_CUDA_TRY(trace_copy(m, li, TR_ACT, m->act, batch, s));
        if (m->tp > 1 && tp_peer_ready(m->peer)) {
            BT_CUDA_TRY(launch_tp_peer_max(m->peer, 1, amax_mlp, batch, s));
            BT_CUDA_TRY(linear_product_fused(L.down->dev(), din, batch, m->acc_i32, H, EPI_I32, nullptr, err, sm, s));
            BT_CUDA_TRY(launch_tp_peer_sum_residual(m->peer, 1, m->acc_i32, amax_mlp, L.down->scales[0], batch, H, m->h, s));
        } else if (m->tp > 1) {
            bt_status st = tp_allreduce_max_f32(m->comm, reinterpret_cast<float*>(amax_mlp), (size_t)batch, s);
            if (st != BT_OK) return st;
            BT_CUDA_TRY(linear_product_fused(L.down->dev(), din, batch, m->acc_i32, H, EPI_I32, nullptr, err, sm, s));
            if ((st = tp_allreduce_sum_i32(m->comm, m->acc_i32, (size_t)batch * H, s)) != BT_OK) return st;
            BT_CUDA_TRY(launch_tp_residual(m->acc_i32, amax_mlp, L.down->scales[0], batch, H, m->h, s, true));
        } else if (split_quant) {
            if ((qst = quant_then_product(m, L.down, PRE_NONE, m->act, I, nullptr, I, batch, m->h, H, EPI_F32_ACCUM, nullptr, err, s)) != BT_OK) return qst;
        } else {
            BT_CUDA_TRY(linear_product_fused(L.down->dev(), din, batch, m->h, H, EPI_F32_ACCUM, nullptr, err, sm, s));
        }
        BT_CUDA_TRY(trace_copy(m, li, TR_H_OUT, m->h, batch, s));
    }
    return enqueue_head(m, batch, s, true);
}

// logits = lm_head(norm(h))  (model/llama.rs:256-266), greedy pick, position advance.  Under tensor parallelism with
// an NCCL communicator every rank computes the vocabulary rows rank * vl .. (the weights stay replicated in memory,
// the reading and the arithmetic are split), the slices are all-gathered and every rank picks from the full row.
bt_status enqueue_head(bt_model* m, int batch, cudaStream_t s, bool fused_launches) {
    const bt_model_config& c = m->cfg;
    const int H = c.hidden_dim, B = c.max_batch;
    unsigned int* err = device_error_word(m->device);
    const int sm = m->sm_count;
    const bool tc = m->lm_tiles && batch > 8;
    if (m->tp > 1 && m->comm && m->lm_gather) {
        const int64_t v0 = (int64_t)c.tp_rank * m->vl;
        const int64_t n_loc = c.vocab_size - v0 < m->vl ? c.vocab_size - v0 : m->vl;
        float* mine = m->lm_gather + (size_t)c.tp_rank * batch * m->vl;
        if (n_loc > 0) {
            if (tc) {
                const uint8_t* tiles = reinterpret_cast<const uint8_t*>(m->lm_tiles) + lm_head_tc_weight_bytes(v0, H);
                BT_CUDA_TRY(launch_lm_head_tc(tiles, m->h, m->norm_f, kRmsEps, batch, H, n_loc, m->lm_btiles, mine, err, sm, s, m->head_f16));
            } else {
                int n_cand = 0;
                BT_CUDA_TRY(launch_lm_head_fused(m->lm_head + (size_t)v0 * H, m->h, m->norm_f, kRmsEps, batch, H, n_loc, mine,
                                                 m->cand_val, m->cand_idx, &n_cand, sm, s, fused_launches, m->head_f16));
            }
        }
        bt_status st = tp_allgather_f32(m->comm, m->lm_gather, (size_t)batch * m->vl, c.tp_rank, s);
        if (st != BT_OK) return st;
        BT_CUDA_TRY(launch_tp_logits_rows(m->lm_gather, m->tp, batch, m->vl, c.vocab_size, m->logits, s));
        BT_CUDA_TRY(launch_argmax(m->logits, batch, c.vocab_size, m->next, s));
        advance_pos_kernel<<<1, 64, 0, s>>>(m->pos, B);
        BT_CUDA_TRY(cudaGetLastError());
        return BT_OK;
    }
    if (tc) {
        BT_CUDA_TRY(launch_lm_head_tc(m->lm_tiles, m->h, m->norm_f, kRmsEps, batch, H, c.vocab_size, m->lm_btiles, m->logits,
                                      err, sm, s, m->head_f16));
        BT_CUDA_TRY(launch_argmax(m->logits, batch, c.vocab_size, m->next, s));
        advance_pos_kernel<<<1, 64, 0, s>>>(m->pos, B);
        BT_CUDA_TRY(cudaGetLastError());
        return BT_OK;
    }
    int n_cand = 0;
    BT_CUDA_TRY(launch_lm_head_fused(m->lm_head, m->h, m->norm_f, kRmsEps, batch, H, c.vocab_size, m->logits,
                                     m->cand_val, m->cand_idx, &n_cand, sm, s, fused_launches, m->head_f16));
    BT_CUDA_TRY(launch_pick(m->cand_val, m->cand_idx, n_cand, batch, m->next, m->pos, B, s, fused_launches));
    return BT_OK;
}

// One decode step for more than 8 sequences: row transforms (RMSNorm, SiLU*up) as separate
// kernels, every projection on the tensor-core product (tcgen05), which quantises its input.
bt_status enqueue_step(bt_model* m, int batch, cudaStream_t s) {
    const bt_model_config& c = m->cfg;
    const int H = c.hidden_dim, I = m->i_l, B = c.max_batch;
    unsigned int* err = device_error_word(m->device);
    const int sm = m->sm_count;
    const int kt_h = (H + kTileK - 1) / kTileK, kt_i = (I + kTileK - 1) / kTileK;
    const int att_dim = m->nh_l * m->head_dim;
    const int kt_att = (att_dim + kTileK - 1) / kTileK;
    // Tensor parallelism at these batch sizes: q|k|v and gate|up hold this rank's rows, o_proj and down_proj this
    // rank's input columns.  Their input is quantised with the maximum over all ranks (all-reduce max of the
    // per-token absmax), their int32 accumulators are summed over the ranks (all-reduce sum) before the scale
    // epilogue: the hidden state stays bit-identical to one GPU.  Both collectives go through NCCL here.
    const bool tp = m->tp > 1;
    if (tp && !m->comm) return set_error(BT_ERR_NCCL, "tensor-parallel steps of more than 8 sequences need bt_model_tp_init (NCCL)");
    auto row_parallel = [&](bt_linear* lin, const float* x, int k, int k_tiles, unsigned int* amax) -> bt_status {
        bt_status st = tp_allreduce_max_f32(m->comm, reinterpret_cast<float*>(amax), (size_t)batch, s);
        if (st != BT_OK) return st;
        BT_CUDA_TRY(launch_row_quant(PRE_NONE, x, k, nullptr, 0.f, batch, k, nullptr, 0, m->sx, m->qsum, nullptr, s, m->qtc, k_tiles, amax));
        BT_CUDA_TRY(launch_gemm_tc(lin->dev(), nullptr, k, batch, m->qtc, m->sx, m->qsum, m->acc_i32, H, EPI_I32, err, sm, s, true));
        if ((st = tp_allreduce_sum_i32(m->comm, m->acc_i32, (size_t)batch * H, s)) != BT_OK) return st;
        BT_CUDA_TRY(launch_tp_residual(m->acc_i32, amax, lin->scales[0], batch, H, m->h, s, false));
        return BT_OK;
    };
    BT_CUDA_TRY(launch_embed(m->tokens, m->embed, batch, H, c.vocab_size, m->h, s, m->absmax, c.num_layers * 2 * B, false, m->embed_f16));
    for (int li = 0; li < c.num_layers; ++li) {
        Layer& L = m->layers[(size_t)li];
        unsigned int* amax_core = m->absmax + ((size_t)li * 2 + 0) * B;
        unsigned int* amax_mlp = m->absmax + ((size_t)li * 2 + 1) * B;
        // x_norm = norm1(x)  (model/block.rs:98)
        //   (the row kernels write the int8 activations straight in the tensor-core product's layout)
        BT_CUDA_TRY(trace_copy(m, li, TR_H_IN, m->h, batch, s));
        BT_CUDA_TRY(launch_row_quant(PRE_RMSNORM, m->h, H, L.norm1, kRmsEps, batch, H, nullptr, 0, m->sx, m->qsum, nullptr, s, m->qtc, kt_h));
        if (c.arch == 0) {
            // TTTLayer::forward_update (layers/ttt.rs:48-74)
            BT_CUDA_TRY(launch_gemm_tc(L.ttt_down->dev(), nullptr, H, batch, m->qtc, m->sx, m->qsum, m->feat, m->d_small, EPI_F32, err, sm, s, true));
            BT_CUDA_TRY(trace_copy(m, li, TR_QKV, m->feat, batch, s));
            BT_CUDA_TRY(launch_ttt_step(L.w_state, m->feat, batch, m->d_small, c.inner_lr, m->z, s));
            BT_CUDA_TRY(trace_copy(m, li, TR_ATT, m->z, batch, s));
            BT_CUDA_TRY(launch_gemm_tc(L.ttt_up->dev(), m->z, m->d_small, batch, m->qtc, m->sx, m->qsum, m->h, H, EPI_F32_ACCUM, err, sm, s));
        } else {
            // BitAttention::forward (layers/attention.rs:149-225), seq_len 1
            BT_CUDA_TRY(launch_gemm_tc(L.qkv->dev(), nullptr, H, batch, m->qtc, m->sx, m->qsum, m->qkv, m->qkv_dim, EPI_F32, err, sm, s, true));
            AttnArgs a;
            a.qkv = m->qkv;
            a.cache = L.kv->view;
            a.pos = m->pos;
            a.rope_cos = m->rope_cos;
            a.rope_sin = m->rope_sin;
            a.out = m->att;
            a.batch = batch; a.n_heads = m->nh_l; a.n_kv = m->nkv_l; a.head_dim = m->head_dim; a.q_rows = 1;
            a.sm_count = sm;
            attn_plan(batch, m->nkv_l, c.max_position_embeddings, sm, m->nh_l / m->nkv_l, &a.splits, &a.span);
            a.scaling = (float)(1.0 / sqrt((double)m->head_dim));
            a.absmax_out = tp ? amax_core : nullptr;
            a.pdl = true;
            BT_CUDA_TRY(trace_copy(m, li, TR_QKV, m->qkv, batch, s));
            BT_CUDA_TRY(launch_attn_decode(a, s));
            BT_CUDA_TRY(trace_copy(m, li, TR_ATT, m->att, batch, s));
            if (tp) {
                bt_status st = row_parallel(L.o, m->att, att_dim, kt_att, amax_core);
                if (st != BT_OK) return st;
            } else {
                BT_CUDA_TRY(launch_gemm_tc(L.o->dev(), m->att, att_dim, batch, m->qtc, m->sx, m->qsum, m->h, H, EPI_F32_ACCUM, err, sm, s));
            }
        }
        // x = x + mlp(norm2(x))  (model/block.rs:119-131, layers/swiglu.rs:29-35)
        BT_CUDA_TRY(trace_copy(m, li, TR_H_MID, m->h, batch, s));
        BT_CUDA_TRY(launch_row_quant(PRE_RMSNORM, m->h, H, L.norm2, kRmsEps, batch, H, nullptr, 0, m->sx, m->qsum, nullptr, s, m->qtc, kt_h));
        BT_CUDA_TRY(launch_gemm_tc(L.gate_up_il->dev(), nullptr, H, batch, m->qtc, m->sx, m->qsum, m->gu, 2 * I, EPI_F32, err, sm, s, true));
        if (tp) {
            // silu(gate) * up of this rank's columns and their maximum, then the row-parallel product
            BT_CUDA_TRY(launch_row_quant(PRE_SWIGLU, m->gu, 2 * I, nullptr, 0.f, batch, I, nullptr, 0, m->sx, m->qsum, m->act, s, nullptr, 0, nullptr, amax_mlp));
            BT_CUDA_TRY(trace_copy(m, li, TR_ACT, m->act, batch, s));
            bt_status st = row_parallel(L.down, m->act, I, kt_i, amax_mlp);
            if (st != BT_OK) return st;
        } else {
            BT_CUDA_TRY(launch_row_quant(PRE_SWIGLU, m->gu, 2 * I, nullptr, 0.f, batch, I, nullptr, 0, m->sx, m->qsum, m->trace ? m->act : nullptr, s, m->qtc, kt_i));
            BT_CUDA_TRY(trace_copy(m, li, TR_ACT, m->act, batch, s));
            BT_CUDA_TRY(launch_gemm_tc(L.down->dev(), nullptr, I, batch, m->qtc, m->sx, m->qsum, m->h, H, EPI_F32_ACCUM, err, sm, s, true));
        }
        BT_CUDA_TRY(trace_copy(m, li, TR_H_OUT, m->h, batch, s));
    }
    return enqueue_head(m, batch, s, false);
}

// One decode step with every stage as its own kernel: row transform + quantiser, then the product of every
// basis (streaming kernel up to 8 sequences, tensor-core kernel above), the bases summed in basis order before
// the residual is added (AdaptiveBitLinear: y = x . (sum_b scale_b T_b)^T, layers/adaptive_linear.rs:86-161).
// Used for models with several bases per projection; any batch size.
bt_status enqueue_step_generic(bt_model* m, int batch, cudaStream_t s) {
    const bt_model_config& c = m->cfg;
    const int H = c.hidden_dim, I = m->i_l, B = c.max_batch;
    unsigned int* err = device_error_word(m->device);
    const int sm = m->sm_count;
    const bool tc = batch > 8;
    auto quant = [&](int pre, const float* x, int64_t x_stride, const float* w, int k, float* v_out) -> bt_status {
        const int64_t qs = ((int64_t)k + kTileK - 1) / kTileK * kTileK;
        BT_CUDA_TRY(launch_row_quant(pre, x, x_stride, w, kRmsEps, batch, k, tc ? nullptr : m->q, tc ? 0 : qs, m->sx, m->qsum, v_out, s,
                                     tc ? m->qtc : nullptr, (int)(qs / kTileK)));
        return BT_OK;
    };
    auto product = [&](bt_linear* lin, float* out, int64_t out_stride) -> bt_status {
        const int64_t qs = lin->w.k_pad();
        if (tc)
            BT_CUDA_TRY(launch_gemm_tc(lin->dev(), nullptr, lin->w.k_in, batch, m->qtc, m->sx, m->qsum, out, out_stride, EPI_F32, err, sm, s, true));
        else
            BT_CUDA_TRY(linear_product(lin->dev(), m->q, qs, m->qsum, m->sx, batch, out, out_stride, EPI_F32, err, sm, s));
        return BT_OK;
    };
    bt_status st;
    float* tmp = m->xn;  // [max_batch, hidden]
    BT_CUDA_TRY(launch_embed(m->tokens, m->embed, batch, H, c.vocab_size, m->h, s, m->absmax, c.num_layers * 2 * B, false, m->embed_f16));
    for (int li = 0; li < c.num_layers; ++li) {
        Layer& L = m->layers[(size_t)li];
        BT_CUDA_TRY(trace_copy(m, li, TR_H_IN, m->h, batch, s));
        if ((st = quant(PRE_RMSNORM, m->h, H, L.norm1, H, nullptr)) != BT_OK) return st;
        if (c.arch == 0) {
            if ((st = product(L.ttt_down, m->feat, m->d_small)) != BT_OK) return st;
            BT_CUDA_TRY(trace_copy(m, li, TR_QKV, m->feat, batch, s));
            BT_CUDA_TRY(launch_ttt_step(L.w_state, m->feat, batch, m->d_small, c.inner_lr, m->z, s));
            BT_CUDA_TRY(trace_copy(m, li, TR_ATT, m->z, batch, s));
            if ((st = quant(PRE_NONE, m->z, m->d_small, nullptr, m->d_small, nullptr)) != BT_OK) return st;
            if ((st = product(L.ttt_up, tmp, H)) != BT_OK) return st;
        } else {
            if ((st = product(L.qkv, m->qkv, m->qkv_dim)) != BT_OK) return st;
            BT_CUDA_TRY(trace_copy(m, li, TR_QKV, m->qkv, batch, s));
            AttnArgs a;
            a.qkv = m->qkv;
            a.cache = L.kv->view;
            a.pos = m->pos;
            a.rope_cos = m->rope_cos;
            a.rope_sin = m->rope_sin;
            a.out = m->att;
            a.batch = batch; a.n_heads = m->nh_l; a.n_kv = m->nkv_l; a.head_dim = m->head_dim; a.q_rows = 1;
            a.sm_count = sm;
            attn_plan(batch, m->nkv_l, c.max_position_embeddings, sm, m->nh_l / m->nkv_l, &a.splits, &a.span);
            a.scaling = (float)(1.0 / sqrt((double)m->head_dim));
            a.absmax_out = nullptr;
            a.pdl = false;
            BT_CUDA_TRY(launch_attn_decode(a, s));
            BT_CUDA_TRY(trace_copy(m, li, TR_ATT, m->att, batch, s));
            const int att_dim = m->nh_l * m->head_dim;
            if ((st = quant(PRE_NONE, m->att, att_dim, nullptr, att_dim, nullptr)) != BT_OK) return st;
            if ((st = product(L.o, tmp, H)) != BT_OK) return st;
        }
        BT_CUDA_TRY(launch_residual_add(m->h, tmp, (int64_t)batch * H, s));
        BT_CUDA_TRY(trace_copy(m, li, TR_H_MID, m->h, batch, s));
        if ((st = quant(PRE_RMSNORM, m->h, H, L.norm2, H, nullptr)) != BT_OK) return st;
        if ((st = product(L.gate_up_il, m->gu, 2 * I)) != BT_OK) return st;
        if ((st = quant(PRE_SWIGLU, m->gu, 2 * I, nullptr, I, m->act)) != BT_OK) return st;
        BT_CUDA_TRY(trace_copy(m, li, TR_ACT, m->act, batch, s));
        if ((st = product(L.down, tmp, H)) != BT_OK) return st;
        BT_CUDA_TRY(launch_residual_add(m->h, tmp, (int64_t)batch * H, s));
        BT_CUDA_TRY(trace_copy(m, li, TR_H_OUT, m->h, batch, s));
    }
    return enqueue_head(m, batch, s, false);
}

}  // namespace

extern "C" bt_status bt_model_create(bt_model** out, const bt_model_config* cfg, int device) {
    if (!out || !cfg) return set_error(BT_ERR_ARG, "bt_model_create: null pointer");
    *out = nullptr;
    const bt_model_config& c = *cfg;
    if (c.arch != 0 && c.arch != 1) return set_error(BT_ERR_ARG, "bt_model_create: arch must be 0 (ttt) or 1 (llama)");
    if (c.vocab_size < 1 || c.hidden_dim < 4 || c.num_layers < 1 || c.intermediate_dim < 4)
        return set_error(BT_ERR_SHAPE, "bt_model_create: bad dimensions");
    if (c.hidden_dim % 16 != 0 || c.intermediate_dim % 16 != 0)
        return set_error(BT_ERR_ALIGN, "bt_model_create: hidden_dim and intermediate_dim must be multiples of 16");
    if (c.max_batch < 1 || c.max_batch > 64) return set_error(BT_ERR_ARG, "bt_model_create: max_batch must be 1..64");
    if (c.arch == 1) {
        if (c.n_heads < 1 || c.n_kv_heads < 1 || c.hidden_dim % c.n_heads != 0 || c.n_heads % c.n_kv_heads != 0)
            return set_error(BT_ERR_SHAPE, "bt_model_create: heads do not divide hidden_dim / each other");
        const int hd = c.hidden_dim / c.n_heads;
        if (hd % 32 != 0 || hd > 128) return set_error(BT_ERR_SHAPE, "bt_model_create: head_dim %d unsupported (32..128, multiple of 32)", hd);
        { const int rep = c.n_heads / c.n_kv_heads; if (!(rep == 1 || rep == 2 || rep == 4 || rep == 8)) return set_error(BT_ERR_SHAPE, "bt_model_create: query heads per KV head must be 1, 2, 4 or 8"); }
        if (c.max_position_embeddings < 1) return set_error(BT_ERR_ARG, "bt_model_create: max_position_embeddings < 1");
    } else if ((c.hidden_dim / 4) % 16 != 0 || c.hidden_dim / 4 > 1024) {
        return set_error(BT_ERR_SHAPE, "bt_model_create: d_small = hidden_dim/4 must be a multiple of 16 and <= 1024");
    }
    if (bt_device_count() <= device || device < 0) return set_error(BT_ERR_DEVICE, "bt_model_create: no CUDA device %d", device);
    DeviceGuard guard(device);
    if (!guard.ok || !device_error_word(device)) return set_error(BT_ERR_DEVICE, "bt_model_create: cannot use device %d", device);
    bt_model* m = new (std::nothrow) bt_model();
    if (!m) return set_error(BT_ERR_NOMEM, "host allocation failed");
    const int tp = c.tp_size > 1 ? c.tp_size : 1;
    if (tp > 1) {
        if (c.arch != 1) { delete m; return set_error(BT_ERR_ARG, "bt_model_create: tensor parallelism needs arch llama"); }
        if (c.tp_rank < 0 || c.tp_rank >= tp || c.n_kv_heads % tp != 0 || c.n_heads % tp != 0 ||
            c.intermediate_dim % (16 * tp) != 0) {
            delete m;
            return set_error(BT_ERR_SHAPE, "bt_model_create: tp_size %d must divide n_kv_heads, n_heads and intermediate_dim/16 "
                                           "(rank in range)", tp);
        }
    }
    m->cfg = c;
    m->tp = tp;
    m->device = device;
    m->sm_count = device_sm_count(device);
    m->head_dim = c.arch == 1 ? c.hidden_dim / c.n_heads : 0;
    m->d_small = c.hidden_dim / 4;  // layers/ttt.rs:29
    m->nh_l = c.arch == 1 ? c.n_heads / tp : 0;
    m->nkv_l = c.arch == 1 ? c.n_kv_heads / tp : 0;
    m->i_l = c.intermediate_dim / tp;
    m->qkv_dim = c.arch == 1 ? (m->nh_l + 2 * m->nkv_l) * m->head_dim : 0;
    m->layers.resize((size_t)c.num_layers);
    *out = m;
    return BT_OK;
}

extern "C" bt_status bt_model_set_linear_bases(bt_model* m, int layer, bt_weight_kind kind, const uint8_t* packed_host,
                                               int64_t n_out, int64_t k_in, int n_bases, const float* scales_host) {
    if (!m || !packed_host || !scales_host) return set_error(BT_ERR_ARG, "bt_model_set_linear: null pointer");
    if (m->finalized) return set_error(BT_ERR_ARG, "bt_model_set_linear: model already finalized");
    if (layer < 0 || layer >= m->cfg.num_layers || (int)kind < 0 || (int)kind > 8)
        return set_error(BT_ERR_ARG, "bt_model_set_linear: layer %d / kind %d out of range", layer, (int)kind);
    if (n_bases < 1 || n_bases > 8) return set_error(BT_ERR_ARG, "bt_model_set_linear: n_bases %d outside 1..8", n_bases);
    if (n_bases > 1 && m->tp > 1) return set_error(BT_ERR_ARG, "bt_model_set_linear: tensor-parallel models take one basis per projection");
    const bt_model_config& c = m->cfg;
    const int64_t H = c.hidden_dim, I = m->i_l, hd = m->head_dim, d = m->d_small;
    int64_t en = 0, ek = 0;
    switch (kind) {
        case BT_W_Q: en = m->nh_l * hd; ek = H; break;
        case BT_W_K: case BT_W_V: en = m->nkv_l * hd; ek = H; break;
        case BT_W_O: en = H; ek = m->nh_l * hd; break;
        case BT_W_GATE: case BT_W_UP: en = I; ek = H; break;
        case BT_W_DOWN: en = H; ek = I; break;
        case BT_W_TTT_DOWN: en = d; ek = H; break;
        case BT_W_TTT_UP: en = H; ek = d; break;
    }
    if (n_out != en || k_in != ek)
        return set_error(BT_ERR_SHAPE, "bt_model_set_linear: weight [%lld, %lld] given, [%lld, %lld] expected",
                         (long long)n_out, (long long)k_in, (long long)en, (long long)ek);
    HostLinear& hl = m->layers[(size_t)layer].host[(int)kind];
    hl.packed.assign(packed_host, packed_host + (size_t)n_out * (size_t)(k_in / 4) * (size_t)n_bases);
    hl.n_out = n_out; hl.k_in = k_in; hl.n_bases = n_bases; hl.set = true;
    for (int b = 0; b < n_bases; ++b) hl.scales[b] = scales_host[b];
    if (n_bases > 1) m->multi_basis = true;
    return BT_OK;
}

extern "C" bt_status bt_model_set_linear(bt_model* m, int layer, bt_weight_kind kind, const uint8_t* packed_host,
                                         int64_t n_out, int64_t k_in, float scale) {
    return bt_model_set_linear_bases(m, layer, kind, packed_host, n_out, k_in, 1, &scale);
}

extern "C" bt_status bt_model_set_tensor(bt_model* m, bt_tensor_kind kind, int layer, const float* data, int64_t n_elem) {
    return bt_model_set_tensor_typed(m, kind, layer, data, n_elem, BT_BF16);
}

extern "C" bt_status bt_model_set_tensor_typed(bt_model* m, bt_tensor_kind kind, int layer, const float* data, int64_t n_elem,
                                               bt_dtype storage) {
    if (!m || !data) return set_error(BT_ERR_ARG, "bt_model_set_tensor: null pointer");
    if (storage != BT_BF16 && storage != BT_F16) return set_error(BT_ERR_ARG, "bt_model_set_tensor: storage must be BT_BF16 or BT_F16");
    if (m->finalized) return set_error(BT_ERR_ARG, "bt_model_set_tensor: model already finalized");
    const bt_model_config& c = m->cfg;
    DeviceGuard guard(m->device);
    const int64_t H = c.hidden_dim, VH = (int64_t)c.vocab_size * H;
    if (kind == BT_T_EMBED || kind == BT_T_LM_HEAD) {
        if (n_elem != VH) return set_error(BT_ERR_SHAPE, "bt_model_set_tensor: %lld elements given, %lld expected", (long long)n_elem, (long long)VH);
        __nv_bfloat16** dst = kind == BT_T_EMBED ? &m->embed : &m->lm_head;
        (kind == BT_T_EMBED ? m->embed_f16 : m->head_f16) = storage == BT_F16;
        if (!*dst) BT_CUDA_TRY(dev_alloc(dst, (size_t)VH));
        // staged through a bounded f32 buffer, converted on the device
        const int64_t chunk = 16 << 20;
        float* tmp = nullptr;
        BT_CUDA_TRY(dev_alloc(&tmp, (size_t)(VH < chunk ? VH : chunk)));
        for (int64_t off = 0; off < VH; off += chunk) {
            const int64_t n = VH - off < chunk ? VH - off : chunk;
            cudaError_t e = cudaMemcpy(tmp, data + off, (size_t)n * sizeof(float), cudaMemcpyHostToDevice);
            if (e == cudaSuccess) {
                f32_to_16bit_kernel<<<1184, 256>>>(tmp, *dst + off, n, storage == BT_F16);
                e = cudaDeviceSynchronize();
            }
            if (e != cudaSuccess) { cudaFree(tmp); return set_error(BT_ERR_CUDA, "bt_model_set_tensor: %s", cudaGetErrorString(e)); }
        }
        cudaFree(tmp);
        return BT_OK;
    }
    if (n_elem != H) return set_error(BT_ERR_SHAPE, "bt_model_set_tensor: norm weight has %lld elements, %lld expected", (long long)n_elem, (long long)H);
    float** dst = nullptr;
    if (kind == BT_T_NORM_F) dst = &m->norm_f;
    else {
        if (layer < 0 || layer >= c.num_layers) return set_error(BT_ERR_ARG, "bt_model_set_tensor: layer %d out of range", layer);
        dst = kind == BT_T_NORM1 ? &m->layers[(size_t)layer].norm1 : &m->layers[(size_t)layer].norm2;
    }
    if (!*dst) BT_CUDA_TRY(dev_alloc(dst, (size_t)H));
    BT_CUDA_TRY(cudaMemcpy(*dst, data, (size_t)H * sizeof(float), cudaMemcpyHostToDevice));
    return BT_OK;
}

extern "C" bt_status bt_model_finalize(bt_model* m) {
    if (!m) return set_error(BT_ERR_ARG, "bt_model_finalize: null handle");
    if (m->finalized) return BT_OK;
    const bt_model_config& c = m->cfg;
    DeviceGuard guard(m->device);
    if (!m->embed || !m->lm_head || !m->norm_f) return set_error(BT_ERR_ARG, "bt_model_finalize: embedding, lm_head or final norm missing");
    const int B = c.max_batch, H = c.hidden_dim, I = m->i_l;
    for (auto& L : m->layers) {
        if (!L.norm1 || !L.norm2) return set_error(BT_ERR_ARG, "bt_model_finalize: a layer norm weight is missing");
        bt_status st;
        if (c.arch == 1) {
            HostLinear* qkv[3] = {&L.host[BT_W_Q], &L.host[BT_W_K], &L.host[BT_W_V]};
            if ((st = make_linear(m, qkv, 3, &L.qkv)) != BT_OK) return st;
            HostLinear* o[1] = {&L.host[BT_W_O]};
            if ((st = make_linear(m, o, 1, &L.o)) != BT_OK) return st;
            if ((st = bt_kv_create(&L.kv, B, m->nkv_l, m->head_dim, c.max_position_embeddings, m->device)) != BT_OK) return st;
        } else {
            HostLinear* dn[1] = {&L.host[BT_W_TTT_DOWN]};
            if ((st = make_linear(m, dn, 1, &L.ttt_down)) != BT_OK) return st;
            HostLinear* up[1] = {&L.host[BT_W_TTT_UP]};
            if ((st = make_linear(m, up, 1, &L.ttt_up)) != BT_OK) return st;
            BT_CUDA_TRY(dev_alloc(&L.w_state, (size_t)B * m->d_small * m->d_small));
        }
        HostLinear* gu[2] = {&L.host[BT_W_GATE], &L.host[BT_W_UP]};
        if (!gu[0]->set || !gu[1]->set) return set_error(BT_ERR_ARG, "bt_model_finalize: a projection weight was never set");
        if (gu[0]->n_bases != gu[1]->n_bases) return set_error(BT_ERR_SHAPE, "bt_model_finalize: gate and up projections disagree on the number of bases");
        if ((st = create_gate_up(&L.gate_up_il, gu[0]->packed.data(), gu[1]->packed.data(), gu[0]->n_out, gu[0]->k_in,
                                 gu[0]->n_bases, gu[0]->scales, gu[1]->scales, m->device)) != BT_OK) return st;
        m->ternary_bytes += L.gate_up_il->w.basis_stride() * gu[0]->n_bases;
        for (HostLinear* hl : gu) { hl->packed.clear(); hl->packed.shrink_to_fit(); }
        HostLinear* dn[1] = {&L.host[BT_W_DOWN]};
        if ((st = make_linear(m, dn, 1, &L.down)) != BT_OK) return st;
    }
    int64_t kmax = H > I ? H : I;
    m->q_stride = (kmax + kTileK - 1) / kTileK * kTileK;
    BT_CUDA_TRY(dev_alloc(&m->tokens, (size_t)B));
    BT_CUDA_TRY(dev_alloc(&m->pos, (size_t)B));
    BT_CUDA_TRY(dev_alloc(&m->h, (size_t)B * H));
    BT_CUDA_TRY(dev_alloc(&m->q, (size_t)B * m->q_stride));
    BT_CUDA_TRY(dev_alloc(&m->sx, (size_t)B));
    BT_CUDA_TRY(dev_alloc(&m->qsum, (size_t)B));
    BT_CUDA_TRY(dev_alloc(&m->gu, (size_t)B * 2 * I));
    BT_CUDA_TRY(dev_alloc(&m->xn, (size_t)B * H));
    BT_CUDA_TRY(dev_alloc(&m->act, (size_t)B * I));
    if (B > 8) {
        BT_CUDA_TRY(dev_alloc(&m->xt, (size_t)B * (H > I ? H : I)));
        BT_CUDA_TRY(dev_alloc(&m->qtc, gemm_tc_act_bytes(B, (kmax + kTileK - 1) / kTileK)));
        if (H % 64 == 0) {
            BT_CUDA_TRY(cudaMalloc(&m->lm_tiles, lm_head_tc_weight_bytes(c.vocab_size, H)));
            BT_CUDA_TRY(cudaMalloc(&m->lm_btiles, lm_head_tc_act_bytes(H)));
            BT_CUDA_TRY(launch_lm_retile(m->lm_head, c.vocab_size, H, m->lm_tiles, 0));
            BT_CUDA_TRY(cudaDeviceSynchronize());
        }
    }
    BT_CUDA_TRY(dev_alloc(&m->absmax, (size_t)c.num_layers * 2 * B));
    BT_CUDA_TRY(cudaMemset(m->absmax, 0, (size_t)c.num_layers * 2 * B * sizeof(unsigned int)));
    BT_CUDA_TRY(dev_alloc(&m->cand_val, (size_t)B * lm_head_max_candidates(m->sm_count)));
    BT_CUDA_TRY(dev_alloc(&m->cand_idx, (size_t)B * lm_head_max_candidates(m->sm_count)));
    BT_CUDA_TRY(dev_alloc(&m->logits, (size_t)B * c.vocab_size));
    BT_CUDA_TRY(dev_alloc(&m->next, (size_t)B));
    if (c.arch == 1) {
        BT_CUDA_TRY(dev_alloc(&m->qkv, (size_t)B * m->qkv_dim));
        BT_CUDA_TRY(dev_alloc(&m->att, (size_t)B * H));
        BT_CUDA_TRY(dev_alloc(&m->inv_freq, (size_t)m->head_dim / 2));
        BT_CUDA_TRY(upload_inv_freq(m->inv_freq, m->head_dim, c.rope_theta));
        BT_CUDA_TRY(dev_alloc(&m->rope_cos, (size_t)c.max_position_embeddings * (m->head_dim / 2)));
        BT_CUDA_TRY(dev_alloc(&m->rope_sin, (size_t)c.max_position_embeddings * (m->head_dim / 2)));
        BT_CUDA_TRY(launch_rope_tables(m->inv_freq, c.max_position_embeddings, m->head_dim / 2, m->rope_cos, m->rope_sin, 0));
        BT_CUDA_TRY(cudaDeviceSynchronize());
        if (m->tp > 1) BT_CUDA_TRY(dev_alloc(&m->acc_i32, (size_t)B * H));
        if (m->tp > 1 && tp_allgather_available()) {
            m->vl = ((c.vocab_size + m->tp - 1) / m->tp + 127) / 128 * 128;
            BT_CUDA_TRY(dev_alloc(&m->lm_gather, (size_t)m->tp * B * m->vl));
        }
    } else {
        BT_CUDA_TRY(dev_alloc(&m->feat, (size_t)B * m->d_small));
        BT_CUDA_TRY(dev_alloc(&m->z, (size_t)B * m->d_small));
    }
    BT_CUDA_TRY(cudaMallocHost(reinterpret_cast<void**>(&m->tokens_pinned), (size_t)B * sizeof(int32_t)));
    BT_CUDA_TRY(cudaMallocHost(reinterpret_cast<void**>(&m->next_pinned), (size_t)B * sizeof(int32_t)));
    BT_CUDA_TRY(cudaMallocHost(reinterpret_cast<void**>(&m->err_pinned), sizeof(unsigned int)));
    *m->err_pinned = 0;
    BT_CUDA_TRY(cudaStreamCreateWithFlags(&m->stream, cudaStreamNonBlocking));
    m->finalized = true;
    return bt_model_reset(m);
}

extern "C" bt_status bt_model_destroy(bt_model* m) {
    if (!m) return BT_OK;
    DeviceGuard guard(m->device);
    cudaDeviceSynchronize();
    for (auto& g : m->graphs)
        if (g && g != reinterpret_cast<cudaGraphExec_t>(uintptr_t(1))) cudaGraphExecDestroy(g);  // 1 = "ran eagerly once" sentinel
    for (auto& L : m->layers) {
        bt_linear_destroy(L.qkv); bt_linear_destroy(L.o); bt_linear_destroy(L.gate_up_il); bt_linear_destroy(L.down);
        bt_linear_destroy(L.ttt_down); bt_linear_destroy(L.ttt_up);
        bt_kv_destroy(L.kv);
        cudaFree(L.norm1); cudaFree(L.norm2); cudaFree(L.w_state);
    }
    void* bufs[] = {m->embed, m->lm_head, m->norm_f, m->inv_freq, m->tokens, m->pos, m->h, m->q, m->sx, m->qsum,
                    m->qkv, m->att, m->gu, m->feat, m->z, m->xn, m->logits, m->next, m->act, m->absmax, m->cand_val, m->cand_idx, m->rope_cos, m->rope_sin, m->acc_i32, m->xt, m->qtc, m->lm_tiles, m->lm_btiles, m->lm_gather};
    for (void* p : bufs) cudaFree(p);
    for (void* p : {(void*)m->pf_tokens, (void*)m->pf_h, (void*)m->pf_qkv, (void*)m->pf_att, (void*)m->pf_gu, (void*)m->pf_qtc,
                    (void*)m->pf_sx, (void*)m->pf_qsum, (void*)m->pf_act}) cudaFree(p);
    if (m->tokens_pinned) cudaFreeHost(m->tokens_pinned);
    if (m->next_pinned) cudaFreeHost(m->next_pinned);
    if (m->err_pinned) cudaFreeHost(m->err_pinned);
    if (m->stream) cudaStreamDestroy(m->stream);
    if (m->comm) tp_comm_destroy(m->comm);
    if (m->peer) tp_peer_destroy(m->peer);
    delete m;
    return BT_OK;
}

extern "C" bt_status bt_model_reset(bt_model* m) {
    if (!m || !m->finalized) return set_error(BT_ERR_ARG, "bt_model_reset: model not finalized");
    DeviceGuard guard(m->device);
    BT_CUDA_TRY(cudaDeviceSynchronize());
    for (auto& L : m->layers) {
        if (L.kv) { bt_status st = bt_kv_reset(L.kv); if (st != BT_OK) return st; }
        if (L.w_state) BT_CUDA_TRY(cudaMemset(L.w_state, 0, (size_t)m->cfg.max_batch * m->d_small * m->d_small * sizeof(float)));
    }
    BT_CUDA_TRY(cudaMemset(m->pos, 0, (size_t)m->cfg.max_batch * sizeof(int32_t)));
    BT_CUDA_TRY(cudaDeviceSynchronize());  // the clears are done before a step on another stream can start
    m->host_pos = 0;
    return BT_OK;
}

// After a timed-out exchange the ranks' epoch counters no longer agree.  Every rank calls this while no rank has a
// step in flight (host barrier before) and starts its next step only when all ranks are through (host barrier after).
extern "C" bt_status bt_model_tp_resync(bt_model* m) {
    if (!m || !m->finalized) return set_error(BT_ERR_ARG, "bt_model_tp_resync: model not finalized");
    DeviceGuard guard(m->device);
    BT_CUDA_TRY(cudaDeviceSynchronize());
    if (m->peer) BT_CUDA_TRY(tp_peer_reset(m->peer));
    return BT_OK;
}

namespace {

bt_status enqueue_any(bt_model* m, int batch, cudaStream_t s) {
    if (m->multi_basis) return enqueue_step_generic(m, batch, s);
    return batch <= 8 ? enqueue_step_fused(m, batch, s) : enqueue_step(m, batch, s);
}

bt_status run_step(bt_model* m, int batch, cudaStream_t s) {
    if (m->tp > 1 && !m->comm && !tp_peer_ready(m->peer))
        return set_error(BT_ERR_NCCL, "tensor-parallel model used before bt_model_tp_init / bt_model_tp_peer_import");
    if (m->cfg.arch == 1 && m->host_pos >= m->cfg.max_position_embeddings)
        return set_error(BT_ERR_SHAPE, "position %d reaches max_position_embeddings %d", m->host_pos, m->cfg.max_position_embeddings);
    // first call at a batch size runs eagerly (it also sets kernel attributes); the second
    // is captured into a graph that later calls replay
    static_assert(sizeof(m->graphs) / sizeof(m->graphs[0]) == 65, "graph table");
    cudaGraphExec_t& exec = m->graphs[batch];
    const uintptr_t marker = 1;  // "ran eagerly once" sentinel stored in the table
    if (m->trace) {
        // inspection: launch by launch with the copies into the trace buffer in between (never captured)
        bt_status st = enqueue_any(m, batch, s);
        if (st != BT_OK) return st;
    } else if (exec == nullptr) {
        bt_status st = enqueue_any(m, batch, s);
        if (st != BT_OK) return st;
        exec = reinterpret_cast<cudaGraphExec_t>(marker);
    } else if (exec == reinterpret_cast<cudaGraphExec_t>(marker)) {
        cudaGraph_t graph = nullptr;
        // captured on the model's own stream (the legacy default stream cannot capture),
        // launched on the caller's
        cudaStream_t cs = m->stream;
        BT_CUDA_TRY(cudaStreamBeginCapture(cs, cudaStreamCaptureModeThreadLocal));
        bt_status st = enqueue_any(m, batch, cs);
        cudaError_t e = cudaStreamEndCapture(cs, &graph);
        if (st != BT_OK) { if (graph) cudaGraphDestroy(graph); return st; }
        if (e != cudaSuccess) return set_error(BT_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
        cudaGraphExec_t ge = nullptr;
        e = cudaGraphInstantiate(&ge, graph, 0);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) return set_error(BT_ERR_CUDA, "graph instantiate failed: %s", cudaGetErrorString(e));
        exec = ge;
        BT_CUDA_TRY(cudaGraphLaunch(exec, s));
    } else {
        BT_CUDA_TRY(cudaGraphLaunch(exec, s));
    }
    m->host_pos += 1;
    return BT_OK;
}

}  // namespace

extern "C" bt_status bt_model_step_dev(bt_model* m, const int32_t* tokens_dev, int batch, void* stream) {
    if (!m || !m->finalized || !tokens_dev) return set_error(BT_ERR_ARG, "bt_model_step_dev: null pointer or model not finalized");
    if (batch < 1 || batch > m->cfg.max_batch) return set_error(BT_ERR_SHAPE, "bt_model_step_dev: batch %d outside 1..%d", batch, m->cfg.max_batch);
    DeviceGuard guard(m->device);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    BT_CUDA_TRY(cudaMemcpyAsync(m->tokens, tokens_dev, (size_t)batch * sizeof(int32_t), cudaMemcpyDeviceToDevice, s));
    return run_step(m, batch, s);
}

extern "C" bt_status bt_model_forward_one(bt_model* m, const int32_t* tokens_host, int batch, float* logits_host,
                                          int32_t* next_host) {
    if (!m || !m->finalized || !tokens_host) return set_error(BT_ERR_ARG, "bt_model_forward_one: null pointer or model not finalized");
    if (batch < 1 || batch > m->cfg.max_batch) return set_error(BT_ERR_SHAPE, "bt_model_forward_one: batch %d outside 1..%d", batch, m->cfg.max_batch);
    DeviceGuard guard(m->device);
    cudaStream_t s = m->stream;
    memcpy(m->tokens_pinned, tokens_host, (size_t)batch * sizeof(int32_t));
    BT_CUDA_TRY(cudaMemcpyAsync(m->tokens, m->tokens_pinned, (size_t)batch * sizeof(int32_t), cudaMemcpyHostToDevice, s));
    bt_status st = run_step(m, batch, s);
    if (st != BT_OK) return st;
    if (logits_host)
        BT_CUDA_TRY(cudaMemcpyAsync(logits_host, m->logits, (size_t)batch * m->cfg.vocab_size * sizeof(float), cudaMemcpyDeviceToHost, s));
    BT_CUDA_TRY(cudaMemcpyAsync(m->next_pinned, m->next, (size_t)batch * sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    unsigned int* err_word = m->tp > 1 ? device_error_word(m->device) : nullptr;
    if (err_word) BT_CUDA_TRY(cudaMemcpyAsync(m->err_pinned, err_word, sizeof(unsigned int), cudaMemcpyDeviceToHost, s));
    BT_CUDA_TRY(cudaStreamSynchronize(s));
    if (err_word && *m->err_pinned != 0) {
        // a peer never arrived at an exchange: the hidden state of this step is not valid
        const unsigned int tag = *m->err_pinned;
        BT_CUDA_TRY(cudaMemsetAsync(err_word, 0, sizeof(unsigned int), s));
        BT_CUDA_TRY(cudaStreamSynchronize(s));
        *m->err_pinned = 0;
        return set_error(BT_ERR_TIMEOUT, "bt_model_forward_one: a tensor-parallel exchange timed out (kernel tag 0x%08x); "
                                         "reset every rank (bt_model_reset) before the next step", tag);
    }
    if (next_host) memcpy(next_host, m->next_pinned, (size_t)batch * sizeof(int32_t));
    return BT_OK;
}


namespace {

constexpr int kPrefillRowsMax = 2048;  // rows (sequences x tokens) one prefill chunk works on

bt_status prefill_buffers(bt_model* m, int rows) {
    if (rows <= m->pf_rows) return BT_OK;
    const bt_model_config& c = m->cfg;
    const int64_t H = c.hidden_dim, I = m->i_l;
    const int64_t qw = c.arch == 1 ? m->qkv_dim : m->d_small;  // q|k|v, or the TTT features and predictions (two slots)
    BT_CUDA_TRY(cudaDeviceSynchronize());
    for (void* p : {(void*)m->pf_tokens, (void*)m->pf_h, (void*)m->pf_qkv, (void*)m->pf_att, (void*)m->pf_gu, (void*)m->pf_qtc,
                    (void*)m->pf_sx, (void*)m->pf_qsum}) cudaFree(p);
    m->pf_rows = 0;
    const int64_t kmax = H > I ? H : I;
    BT_CUDA_TRY(dev_alloc(&m->pf_tokens, (size_t)rows));
    BT_CUDA_TRY(dev_alloc(&m->pf_h, (size_t)rows * H));
    BT_CUDA_TRY(dev_alloc(&m->pf_qkv, (size_t)rows * qw));
    BT_CUDA_TRY(dev_alloc(&m->pf_att, (size_t)rows * H));
    BT_CUDA_TRY(dev_alloc(&m->pf_gu, (size_t)rows * 2 * I));
    BT_CUDA_TRY(cudaMalloc(reinterpret_cast<void**>(&m->pf_qtc), gemm_tc_act_bytes(rows, (kmax + kTileK - 1) / kTileK)));
    BT_CUDA_TRY(dev_alloc(&m->pf_sx, (size_t)rows));
    BT_CUDA_TRY(dev_alloc(&m->pf_qsum, (size_t)rows));
    m->pf_rows = rows;
    return BT_OK;
}

// One chunk of a prefill: n new tokens for each of `batch` sequences (rows ordered [sequence][token]), all
// sequences at position `past`.  Every projection runs on the tensor-core product over all rows at once; K/V
// rows are appended for the whole chunk, then every token attends causally over the cache
// (model/block.rs:87-134 applied to a [batch, n, hidden] input, cache semantics of model/llama.rs:495-498).
bt_status enqueue_prefill_chunk(bt_model* m, int batch, int n, int past, int ttt_chunk, cudaStream_t s) {
    const bt_model_config& c = m->cfg;
    const int H = c.hidden_dim, I = m->i_l, M = batch * n;
    unsigned int* err = device_error_word(m->device);
    const int sm = m->sm_count;
    const int kt_h = (H + kTileK - 1) / kTileK, kt_i = (I + kTileK - 1) / kTileK;
    BT_CUDA_TRY(launch_embed(m->pf_tokens, m->embed, M, H, c.vocab_size, m->pf_h, s, nullptr, 0, false, m->embed_f16));
    for (int li = 0; li < c.num_layers; ++li) {
        Layer& L = m->layers[(size_t)li];
        BT_CUDA_TRY(trace_copy(m, li, TR_H_IN, m->pf_h, M, s));
        BT_CUDA_TRY(launch_row_quant(PRE_RMSNORM, m->pf_h, H, L.norm1, kRmsEps, M, H, nullptr, 0, m->pf_sx, m->pf_qsum, nullptr, s, m->pf_qtc, kt_h));
        if (c.arch == 0) {
            // TTTLayer::forward_chunkwise (layers/ttt.rs:80-119); ttt_chunk = 1 is the token-by-token update
            float* feat = m->pf_qkv;
            float* z = m->pf_att;
            BT_CUDA_TRY(launch_gemm_tc(L.ttt_down->dev(), nullptr, H, M, m->pf_qtc, m->pf_sx, m->pf_qsum, feat, m->d_small, EPI_F32, err, sm, s, true));
            BT_CUDA_TRY(trace_copy(m, li, TR_QKV, feat, M, s));
            BT_CUDA_TRY(launch_ttt_chunk(L.w_state, feat, batch, n, m->d_small, c.inner_lr, ttt_chunk, z, s));
            BT_CUDA_TRY(trace_copy(m, li, TR_ATT, z, M, s));
            if (m->multi_basis) {  // the bases are summed first, then the residual is added (the order the layer defines)
                BT_CUDA_TRY(launch_gemm_tc(L.ttt_up->dev(), z, m->d_small, M, m->pf_qtc, m->pf_sx, m->pf_qsum, m->pf_gu, H, EPI_F32, err, sm, s));
                BT_CUDA_TRY(launch_residual_add(m->pf_h, m->pf_gu, (int64_t)M * H, s));
            } else {
                BT_CUDA_TRY(launch_gemm_tc(L.ttt_up->dev(), z, m->d_small, M, m->pf_qtc, m->pf_sx, m->pf_qsum, m->pf_h, H, EPI_F32_ACCUM, err, sm, s));
            }
        } else {
            BT_CUDA_TRY(launch_gemm_tc(L.qkv->dev(), nullptr, H, M, m->pf_qtc, m->pf_sx, m->pf_qsum, m->pf_qkv, m->qkv_dim, EPI_F32, err, sm, s, true));
            BT_CUDA_TRY(trace_copy(m, li, TR_QKV, m->pf_qkv, M, s));
            BT_CUDA_TRY(launch_kv_append_rows(L.kv->view, m->pf_qkv, m->pos, m->rope_cos, m->rope_sin, batch, n, m->nh_l, m->nkv_l, m->head_dim, s));
            AttnArgs a;
            a.qkv = m->pf_qkv;
            a.cache = L.kv->view;
            a.pos = m->pos;
            a.rope_cos = m->rope_cos;
            a.rope_sin = m->rope_sin;
            a.out = m->pf_att;
            a.batch = batch; a.n_heads = m->nh_l; a.n_kv = m->nkv_l; a.head_dim = m->head_dim; a.q_rows = n;
            a.sm_count = sm;
            a.splits = 1;
            a.span = (c.max_position_embeddings + 31) / 32 * 32;
            a.scaling = (float)(1.0 / sqrt((double)m->head_dim));
            a.absmax_out = nullptr;
            a.pdl = false;
            if (n == 1) attn_plan(batch, m->nkv_l, c.max_position_embeddings, sm, m->nh_l / m->nkv_l, &a.splits, &a.span);
            BT_CUDA_TRY(launch_attn_decode(a, s));
            BT_CUDA_TRY(trace_copy(m, li, TR_ATT, m->pf_att, M, s));
            if (m->multi_basis) {
                BT_CUDA_TRY(launch_gemm_tc(L.o->dev(), m->pf_att, m->nh_l * m->head_dim, M, m->pf_qtc, m->pf_sx, m->pf_qsum, m->pf_gu, H, EPI_F32, err, sm, s));
                BT_CUDA_TRY(launch_residual_add(m->pf_h, m->pf_gu, (int64_t)M * H, s));
            } else {
                BT_CUDA_TRY(launch_gemm_tc(L.o->dev(), m->pf_att, m->nh_l * m->head_dim, M, m->pf_qtc, m->pf_sx, m->pf_qsum, m->pf_h, H, EPI_F32_ACCUM, err, sm, s));
            }
        }
        BT_CUDA_TRY(trace_copy(m, li, TR_H_MID, m->pf_h, M, s));
        BT_CUDA_TRY(launch_row_quant(PRE_RMSNORM, m->pf_h, H, L.norm2, kRmsEps, M, H, nullptr, 0, m->pf_sx, m->pf_qsum, nullptr, s, m->pf_qtc, kt_h));
        BT_CUDA_TRY(launch_gemm_tc(L.gate_up_il->dev(), nullptr, H, M, m->pf_qtc, m->pf_sx, m->pf_qsum, m->pf_gu, 2 * I, EPI_F32, err, sm, s, true));
        BT_CUDA_TRY(launch_row_quant(PRE_SWIGLU, m->pf_gu, 2 * I, nullptr, 0.f, M, I, nullptr, 0, m->pf_sx, m->pf_qsum,
                                     m->trace ? m->pf_act : nullptr, s, m->pf_qtc, kt_i));
        if (m->trace) BT_CUDA_TRY(trace_copy(m, li, TR_ACT, m->pf_act, M, s));
        if (m->multi_basis) {
            BT_CUDA_TRY(launch_gemm_tc(L.down->dev(), nullptr, I, M, m->pf_qtc, m->pf_sx, m->pf_qsum, m->pf_att, H, EPI_F32, err, sm, s, true));
            BT_CUDA_TRY(launch_residual_add(m->pf_h, m->pf_att, (int64_t)M * H, s));
        } else {
            BT_CUDA_TRY(launch_gemm_tc(L.down->dev(), nullptr, I, M, m->pf_qtc, m->pf_sx, m->pf_qsum, m->pf_h, H, EPI_F32_ACCUM, err, sm, s, true));
        }
        BT_CUDA_TRY(trace_copy(m, li, TR_H_OUT, m->pf_h, M, s));
    }
    (void)past;
    return BT_OK;
}

}  // namespace

extern "C" bt_status bt_model_prefill(bt_model* m, const int32_t* tokens_host, int batch, int n_tokens, int ttt_chunk,
                                      float* logits_host, int32_t* next_host) {
    if (!m || !m->finalized || !tokens_host) return set_error(BT_ERR_ARG, "bt_model_prefill: null pointer or model not finalized");
    if (batch < 1 || batch > m->cfg.max_batch) return set_error(BT_ERR_SHAPE, "bt_model_prefill: batch %d outside 1..%d", batch, m->cfg.max_batch);
    if (n_tokens < 1) return set_error(BT_ERR_SHAPE, "bt_model_prefill: no tokens");
    if (m->tp > 1) return set_error(BT_ERR_ARG, "bt_model_prefill: tensor-parallel models prefill token by token (bt_model_forward_one)");
    if (ttt_chunk < 1 || ttt_chunk > 64) return set_error(BT_ERR_ARG, "bt_model_prefill: ttt_chunk %d outside 1..64", ttt_chunk);
    const bt_model_config& c = m->cfg;
    if (c.arch == 1 && m->host_pos + n_tokens > c.max_position_embeddings)
        return set_error(BT_ERR_SHAPE, "position %d reaches max_position_embeddings %d", m->host_pos + n_tokens, c.max_position_embeddings);
    DeviceGuard guard(m->device);
    cudaStream_t s = m->stream;
    // tokens per sequence and chunk: as many as keep sequences x tokens within the scratch (a TTT chunk is never cut)
    int per = kPrefillRowsMax / batch;
    if (per < 1) per = 1;
    if (per > n_tokens) per = n_tokens;
    if (c.arch == 0 && per < n_tokens && per > ttt_chunk) per -= per % ttt_chunk;
    if (m->trace && (int64_t)batch * per > m->trace_rows) per = m->trace_rows / batch;
    if (per < 1) return set_error(BT_ERR_NOMEM, "bt_model_prefill: the trace buffer holds fewer rows than sequences");
    bt_status st = prefill_buffers(m, batch * per);
    if (st != BT_OK) return st;
    if (m->trace && m->pf_act_rows < batch * per) {
        BT_CUDA_TRY(cudaDeviceSynchronize());
        cudaFree(m->pf_act);
        m->pf_act = nullptr;
        BT_CUDA_TRY(dev_alloc(&m->pf_act, (size_t)batch * per * m->i_l));
        m->pf_act_rows = batch * per;
    }
    const int H = c.hidden_dim, past0 = m->host_pos;
    int last_n = 0;
    for (int c0 = 0; c0 < n_tokens; c0 += per) {
        const int n = n_tokens - c0 < per ? n_tokens - c0 : per;
        m->pf_host.resize((size_t)batch * n);
        for (int b = 0; b < batch; ++b)
            for (int i = 0; i < n; ++i) m->pf_host[(size_t)b * n + i] = tokens_host[(size_t)b * n_tokens + c0 + i];
        BT_CUDA_TRY(cudaMemcpyAsync(m->pf_tokens, m->pf_host.data(), (size_t)batch * n * sizeof(int32_t), cudaMemcpyHostToDevice, s));
        set_pos_kernel<<<1, 64, 0, s>>>(m->pos, c.max_batch, past0 + c0);
        BT_CUDA_TRY(cudaGetLastError());
        if ((st = enqueue_prefill_chunk(m, batch, n, past0 + c0, ttt_chunk, s)) != BT_OK) return st;
        BT_CUDA_TRY(cudaStreamSynchronize(s));  // pf_host is reused by the next chunk
        last_n = n;
    }
    // logits of the last token of every sequence: its hidden state moves into the decode buffers
    BT_CUDA_TRY(cudaMemcpy2DAsync(m->h, (size_t)H * sizeof(float), m->pf_h + (size_t)(last_n - 1) * H, (size_t)last_n * H * sizeof(float),
                                  (size_t)H * sizeof(float), (size_t)batch, cudaMemcpyDeviceToDevice, s));
    if (m->lm_tiles && batch > 8) {
        BT_CUDA_TRY(launch_lm_head_tc(m->lm_tiles, m->h, m->norm_f, kRmsEps, batch, H, c.vocab_size, m->lm_btiles, m->logits,
                                      device_error_word(m->device), m->sm_count, s, m->head_f16));
        BT_CUDA_TRY(launch_argmax(m->logits, batch, c.vocab_size, m->next, s));
    } else {
        int n_cand = 0;
        BT_CUDA_TRY(launch_lm_head_fused(m->lm_head, m->h, m->norm_f, kRmsEps, batch, H, c.vocab_size, m->logits,
                                         m->cand_val, m->cand_idx, &n_cand, m->sm_count, s, false, m->head_f16));
        BT_CUDA_TRY(launch_pick(m->cand_val, m->cand_idx, n_cand, batch, m->next, m->pos, 0, s, false));
    }
    set_pos_kernel<<<1, 64, 0, s>>>(m->pos, c.max_batch, past0 + n_tokens);
    BT_CUDA_TRY(cudaGetLastError());
    m->host_pos = past0 + n_tokens;
    if (logits_host)
        BT_CUDA_TRY(cudaMemcpyAsync(logits_host, m->logits, (size_t)batch * c.vocab_size * sizeof(float), cudaMemcpyDeviceToHost, s));
    BT_CUDA_TRY(cudaMemcpyAsync(m->next_pinned, m->next, (size_t)batch * sizeof(int32_t), cudaMemcpyDeviceToHost, s));
    BT_CUDA_TRY(cudaStreamSynchronize(s));
    if (next_host) memcpy(next_host, m->next_pinned, (size_t)batch * sizeof(int32_t));
    return BT_OK;
}

extern "C" const float* bt_model_logits(bt_model* m) { return m ? m->logits : nullptr; }
extern "C" const int32_t* bt_model_next(bt_model* m) { return m ? m->next : nullptr; }
extern "C" int bt_model_pos(const bt_model* m) { return m ? m->host_pos : -1; }
extern "C" float* bt_model_ttt_state(bt_model* m, int layer) {
    if (!m || layer < 0 || layer >= (int)m->layers.size()) return nullptr;
    return m->layers[(size_t)layer].w_state;
}
extern "C" bt_kv_cache* bt_model_kv_cache(bt_model* m, int layer) {
    if (!m || layer < 0 || layer >= (int)m->layers.size()) return nullptr;
    return m->layers[(size_t)layer].kv;
}
extern "C" int64_t bt_model_trace_floats(const bt_model* m, int rows) {
    return (m && m->finalized && rows > 0) ? trace_layer_floats(m, rows) * m->cfg.num_layers : 0;
}
extern "C" bt_status bt_model_set_trace(bt_model* m, float* trace_dev, int rows) {
    if (!m || !m->finalized) return set_error(BT_ERR_ARG, "bt_model_set_trace: model not finalized");
    if (trace_dev && rows < m->cfg.max_batch) return set_error(BT_ERR_ARG, "bt_model_set_trace: rows %d below max_batch %d", rows, m->cfg.max_batch);
    DeviceGuard guard(m->device);
    BT_CUDA_TRY(cudaDeviceSynchronize());
    m->trace = trace_dev;
    m->trace_rows = trace_dev ? rows : 0;
    return BT_OK;
}
extern "C" int64_t bt_model_ternary_bytes(const bt_model* m) { return m ? m->ternary_bytes : 0; }

extern "C" bt_status bt_model_enqueue_products(bt_model* m, int batch, int as_in_step, void* stream, int* n_launches) {
    if (!m || !m->finalized) return set_error(BT_ERR_ARG, "bt_model_enqueue_products: model not finalized");
    if (batch < 1 || batch > m->cfg.max_batch) return set_error(BT_ERR_SHAPE, "batch %d outside 1..%d", batch, m->cfg.max_batch);
    DeviceGuard guard(m->device);
    cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
    unsigned int* err = device_error_word(m->device);
    const bt_model_config& c = m->cfg;
    const int groups = (batch + 7) / 8;
    int launches = 0;
    const bool fused = as_in_step && batch < kSplitQuantBatch && c.arch == 1 && m->tp == 1;
    // outputs go to the gate/up buffer (the largest activation buffer), never to h
    for (size_t li = 0; li < m->layers.size(); ++li) {
        Layer& L = m->layers[li];
        if (fused) {
            // the launches of enqueue_step_fused, prologues and epilogues included, on whatever the
            // activation buffers hold; the SwiGLU epilogue's absmax goes to a cell nobody reads
            unsigned int* amax = m->absmax + (li * 2) * (size_t)c.max_batch;
            FusedIn norm1{PRO_RMSNORM, m->h, c.hidden_dim, L.norm1, kRmsEps, nullptr};
            BT_CUDA_TRY(linear_product_fused(L.qkv->dev(), norm1, batch, m->gu, m->qkv_dim, EPI_F32, nullptr, err, m->sm_count, s));
            FusedIn ain{PRO_ABSMAX, m->att, m->nh_l * m->head_dim, nullptr, 0.f, amax};
            BT_CUDA_TRY(linear_product_fused(L.o->dev(), ain, batch, m->gu, c.hidden_dim, EPI_F32_ACCUM, nullptr, err, m->sm_count, s));
            FusedIn norm2{PRO_RMSNORM, m->h, c.hidden_dim, L.norm2, kRmsEps, nullptr};
            BT_CUDA_TRY(linear_product_fused(L.gate_up_il->dev(), norm2, batch, m->gu, m->i_l, EPI_SWIGLU, amax, err, m->sm_count, s));
            FusedIn din{PRO_ABSMAX, m->act, m->i_l, nullptr, 0.f, amax};
            BT_CUDA_TRY(linear_product_fused(L.down->dev(), din, batch, m->gu, c.hidden_dim, EPI_F32_ACCUM, nullptr, err, m->sm_count, s));
            launches += 4;
            continue;
        }
        bt_linear* seq[4] = {c.arch == 1 ? L.qkv : L.ttt_down, c.arch == 1 ? L.o : L.ttt_up,
                             L.gate_up_il, L.down};
        for (bt_linear* lin : seq) {
            if (batch > 8) {
                // tensor-core product on whatever the transformed-row buffer holds (quantiser included)
                BT_CUDA_TRY(launch_gemm_tc(lin->dev(), m->xt, lin->w.k_in, batch, m->qtc, m->sx, m->qsum, m->gu,
                                           lin->w.n_out, EPI_F32, err, m->sm_count, s));
                launches += 1 + gemm_tc_kernels(lin->dev(), batch, m->sm_count);
            } else {
                BT_CUDA_TRY(linear_product(lin->dev(), m->q, m->q_stride, m->qsum, m->sx, batch, m->gu, lin->w.n_out,
                                           EPI_F32, err, m->sm_count, s));
                launches += groups;
            }
        }
    }
    if (n_launches) *n_launches = launches;
    return BT_OK;
}

extern "C" int bt_model_launches_per_step(const bt_model* m, int batch) {
    if (!m) return 0;
    // kernels of this library only: NCCL's own kernels (all-reduce, all-gather) are not counted
    const bool split_head = m->tp > 1 && m->comm && m->lm_gather;  // the head's rows cut over the ranks
    if (batch <= 8) {
        // fused path: per layer 4 products + attention or TTT update; tensor parallel: + 2 scale epilogues after the
        // NCCL all-reduces, or + 2 max-exchange and 2 sum-exchange kernels over peer memory;
        // embedding, lm_head per 4 tokens, pick (split head: gathered-rows copy, arg-max, position advance instead)
        int per_layer = 4 + 1 + (m->tp > 1 ? (tp_peer_ready(m->peer) ? 4 : 2) : 0);
        if (m->tp == 1 && m->cfg.arch == 1 && batch >= kSplitQuantBatch) per_layer += 4;  // a quantiser kernel in front of every product
        return m->cfg.num_layers * per_layer + 1 + (batch + 3) / 4 + (split_head ? 3 : 1);
    }
    // batches above 8: per layer 3 row kernels (norm1, norm2, SiLU*up, quantiser included), the quantiser of the
    // attention / TTT output, 4 tensor-core products, attention or TTT update; tensor parallel: each of the two
    // row-parallel projections also has its scale-and-residual kernel, and SiLU*up and the quantiser of its result
    // are two kernels; embedding; lm_head (tensor-core: prepare + product; else per 8 tokens) + pick pair, or with a
    // split head the gathered-rows copy, arg-max and position advance
    const Layer& L = m->layers[0];
    const bt_linear* seq[4] = {m->cfg.arch == 1 ? L.qkv : L.ttt_down, m->cfg.arch == 1 ? L.o : L.ttt_up, L.gate_up_il, L.down};
    int per_layer = 3 + 1 + 1 + (m->tp > 1 ? 3 : 0);
    for (const bt_linear* lin : seq) per_layer += gemm_tc_kernels(lin->dev(), batch, m->sm_count);
    const int head = m->lm_tiles ? 2 : (batch + 7) / 8;
    return m->cfg.num_layers * per_layer + 1 + head + (split_head ? 3 : (m->lm_tiles ? 2 : 1));
}


extern "C" bt_status bt_model_seek(bt_model* m, int pos) {
    if (!m || !m->finalized) return set_error(BT_ERR_ARG, "bt_model_seek: model not finalized");
    if (pos < 0 || (m->cfg.arch == 1 && pos >= m->cfg.max_position_embeddings))
        return set_error(BT_ERR_SHAPE, "bt_model_seek: position %d outside [0, %d)", pos, m->cfg.max_position_embeddings);
    DeviceGuard guard(m->device);
    BT_CUDA_TRY(cudaDeviceSynchronize());
    set_pos_kernel<<<1, 64>>>(m->pos, m->cfg.max_batch, pos);
    BT_CUDA_TRY(cudaDeviceSynchronize());
    m->host_pos = pos;
    return BT_OK;
}

extern "C" bt_status bt_tp_unique_id(uint8_t* id128_out) {
    if (!id128_out) return set_error(BT_ERR_ARG, "bt_tp_unique_id: null pointer");
    return tp_unique_id(id128_out);
}

extern "C" bt_status bt_model_tp_peer_export(bt_model* m, uint8_t* handle64_out) {
    if (!m || !m->finalized || !handle64_out) return set_error(BT_ERR_ARG, "bt_model_tp_peer_export: null pointer or model not finalized");
    if (m->tp <= 1) return set_error(BT_ERR_ARG, "bt_model_tp_peer_export: the model is not tensor-parallel");
    DeviceGuard guard(m->device);
    if (!m->peer) {
        bt_status st = tp_peer_create(&m->peer, m->cfg.tp_rank, m->tp, m->cfg.max_batch < 8 ? m->cfg.max_batch : 8,  // steps of up to 8 sequences use it
                                      m->cfg.hidden_dim, device_error_word(m->device));
        if (st != BT_OK) return st;
    }
    return tp_peer_export(m->peer, handle64_out);
}

extern "C" bt_status bt_model_tp_peer_import(bt_model* m, const uint8_t* handles) {
    if (!m || !m->finalized || !m->peer)
        return set_error(BT_ERR_ARG, "bt_model_tp_peer_import: null pointer, model not finalized or bt_model_tp_peer_export not called");
    DeviceGuard guard(m->device);
    if (!handles) {  // back to NCCL (e.g. another rank could not map the inboxes)
        BT_CUDA_TRY(cudaDeviceSynchronize());
        for (auto& g : m->graphs) {
            if (g && g != reinterpret_cast<cudaGraphExec_t>(uintptr_t(1))) cudaGraphExecDestroy(g);
            g = nullptr;
        }
        tp_peer_destroy(m->peer);
        m->peer = nullptr;
        return BT_OK;
    }
    BT_CUDA_TRY(cudaDeviceSynchronize());
    // graphs captured with the NCCL path must not be replayed after the switch
    for (auto& g : m->graphs) {
        if (g && g != reinterpret_cast<cudaGraphExec_t>(uintptr_t(1))) cudaGraphExecDestroy(g);
        g = nullptr;
    }
    return tp_peer_import(m->peer, handles);
}

namespace {
void drop_graphs(bt_model* m) {
    for (auto& g : m->graphs) {
        if (g && g != reinterpret_cast<cudaGraphExec_t>(uintptr_t(1))) cudaGraphExecDestroy(g);
        g = nullptr;
    }
}
}  // namespace

extern "C" bt_status bt_model_tp_set_timeout(bt_model* m, int milliseconds) {
    if (!m || !m->finalized || !m->peer) return set_error(BT_ERR_ARG, "bt_model_tp_set_timeout: no peer-memory exchange on this model");
    if (milliseconds < 1) return set_error(BT_ERR_ARG, "bt_model_tp_set_timeout: %d ms", milliseconds);
    DeviceGuard guard(m->device);
    BT_CUDA_TRY(cudaDeviceSynchronize());
    drop_graphs(m);  // the limit travels as a kernel argument of the captured launches
    tp_peer_set_wait(m->peer, (unsigned long long)milliseconds * 1000000ull);
    return BT_OK;
}

extern "C" bt_status bt_model_tp_destroy(bt_model* m) {
    if (!m) return BT_OK;
    DeviceGuard guard(m->device);
    BT_CUDA_TRY(cudaDeviceSynchronize());
    drop_graphs(m);
    if (m->peer) { tp_peer_destroy(m->peer); m->peer = nullptr; }
    if (m->comm) { tp_comm_destroy(m->comm); m->comm = nullptr; }
    return BT_OK;
}

extern "C" bt_status bt_model_tp_init(bt_model* m, const uint8_t* id128) {
    if (!m || !m->finalized || !id128) return set_error(BT_ERR_ARG, "bt_model_tp_init: null pointer or model not finalized");
    if (m->tp <= 1) return BT_OK;
    if (m->comm) return BT_OK;
    DeviceGuard guard(m->device);
    return tp_comm_init(&m->comm, id128, m->cfg.tp_rank, m->tp);
}
