/*
 * bitttt.h - C ABI of the B200 (sm_100a) BitLinear inference library.
 *
 * Plain pointers and sizes only; every entry point returns a bt_status (0 = ok,
 * negative = error) and never aborts or traps.  bt_last_error() gives the message of
 * the calling thread's last failure, with the reference's wording for shape errors.
 *
 * Each declaration names the interface of Bit-TTT-Engine that it stands in for
 * (paths relative to the reference project root, RE = crates/rust_engine/src).
 *
 * Pointers named *_dev are CUDA device pointers on the handle's device; *_host are
 * host pointers.  `stream` is a cudaStream_t passed as void* (NULL = default stream).
 * Calls are asynchronous on that stream unless stated otherwise.
 */
#ifndef BITTTT_H
#define BITTTT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int bt_status;
enum {
    BT_OK = 0,
    BT_ERR_SHAPE = -1,   /* dimension mismatch (reference: "Shape mismatch: Input [..] vs Weight [..]") */
    BT_ERR_ALIGN = -2,   /* K % 4 != 0, misaligned pointer */
    BT_ERR_DEVICE = -3,  /* no CUDA device / wrong device */
    BT_ERR_CUDA = -4,    /* a CUDA runtime call failed */
    BT_ERR_NCCL = -5,
    BT_ERR_TIMEOUT = -6, /* a bounded device-side wait ran out */
    BT_ERR_NOMEM = -7,
    BT_ERR_ARG = -8      /* null pointer, unsupported dtype or option */
};

typedef enum { BT_F32 = 0, BT_BF16 = 1, BT_I8 = 2, BT_I32 = 3, BT_F16 = 4 } bt_dtype;

/* Message of the calling thread's last failed call ("" if none). */
const char* bt_last_error(void);
/* Library version, major*10000 + minor*100 + patch. */
int bt_version(void);
/* Number of CUDA devices visible (0 if none); never fails. */
int bt_device_count(void);
/* Synchronises `device` and reports a sticky device-side error (bounded wait that ran
 * out) recorded by any kernel of this library since the last call. */
bt_status bt_device_check(int device);

/* ---- packing (host) ----------------------------------------------------------------- */

/* PackedTensor::pack, RE/kernels/packing.rs:50-105: scale = mean|w| + 1e-6,
 * q = clamp(round(w/scale),-1,1), 2-bit codes 00/01/10 = 0/+1/-1, four per byte, LSB
 * first.  out_host holds ceil(n_elem/4) bytes. */
bt_status bt_pack_ternary(const float* w_host, int64_t n_elem, uint8_t* out_host, float* scale_out);
/* PackedTensor::unpack, RE/kernels/packing.rs:108-133. */
bt_status bt_unpack_ternary(const uint8_t* packed_host, int64_t n_elem, float scale, float* out_host);

/* Reader for the legacy one-byte-per-weight layout of tools/conversion/convert_adaptive.py:43-83
 * ([n_out, k_in/4, n_bases, 4] int8, the input of adaptive_gemm_n3_kernel_f32,
 * RE/kernels/adaptive_bit_op.cu:74-161): rewrites it as the 2-bit layout [n_out, k_in/4, n_bases]
 * (n_out * k_in/4 * n_bases bytes) that bt_linear_create accepts, so that such a checkpoint streams
 * 2 bits per weight and basis instead of 8.  Values other than -1 / 0 / +1 give BT_ERR_ARG. */
bt_status bt_convert_l3_to_l2(const int8_t* l3_host, int64_t n_out, int64_t k_in, int n_bases,
                              uint8_t* l2_out_host);

/* ---- BitLinear ---------------------------------------------------------------------- */

typedef struct bt_linear bt_linear;

/* Stands in for BitLinear::load + precompute_packed (RE/layers/bit_linear.rs:24-50) and
 * for AdaptiveBitLinear::load (RE/layers/adaptive_linear.rs:40-129).
 * packed_host: the packed bytes exactly as the reference stores them:
 *   n_bases == 1: PackedTensor.data, row-major [n_out, k_in/4] (RE/kernels/packing.rs:15-21);
 *   n_bases  > 1: `weight_packed` of a converted checkpoint, [n_out, k_in/4, n_bases]
 *                 (tools/conversion/convert_llama_v2.py:111-151).
 * scales_host: n_bases floats.  k_in must be a multiple of 4 (BT_ERR_ALIGN otherwise;
 * the reference's packer and kernels disagree for such shapes).  The bytes are copied to
 * `device` once, into the library's own streaming layout; the handle is immutable
 * afterwards and may be used from several host threads at once, each with its own
 * workspace and stream.  Synchronous. */
bt_status bt_linear_create(bt_linear** out, const uint8_t* packed_host, int64_t n_out,
                           int64_t k_in, int n_bases, const float* scales_host, int device);
bt_status bt_linear_destroy(bt_linear* lin);
bt_status bt_linear_dims(const bt_linear* lin, int64_t* n_out, int64_t* k_in, int* n_bases);

/* Scratch memory for forward calls (quantised activations).  One workspace serves one
 * stream at a time.  bytes = 0 picks a size good for m <= 64 at k_in <= 16384. */
typedef struct bt_workspace bt_workspace;
bt_status bt_workspace_create(bt_workspace** out, int device, size_t bytes);
bt_status bt_workspace_destroy(bt_workspace* ws);

/* Stands in for BitLinearCuda::forward / BitLinearCpu::forward
 * (RE/kernels/cuda.rs:21-47, RE/kernels/cpu.rs:17-127) as called from BitLinear::forward
 * (RE/layers/bit_linear.rs:65-85): y[m, n_out] = x[m, k_in] . W^T with per-token absmax
 * int8 quantisation of x in front:  y = sum_b ((float)acc_b * scale_b) * s_x[m].
 * x_dtype: BT_F32 or BT_BF16; y_dtype: BT_F32 or BT_BF16.  x_k must equal the handle's
 * k_in, else BT_ERR_SHAPE with the reference's message.  ws may be NULL: a workspace
 * owned by the handle is then used (allocated on first use; calls on one handle with
 * ws == NULL must not overlap). */
bt_status bt_linear_forward(bt_linear* lin, bt_workspace* ws, const void* x_dev, int64_t m,
                            int64_t x_k, bt_dtype x_dtype, void* y_dev, bt_dtype y_dtype,
                            void* stream);

/* Same product on activations that are already int8 (row-major [m, k_in]).  out_dtype
 * BT_I32: raw integer accumulators sum_k q*t of basis 0, [m, n_out] (the bit-exact
 * check against RE/kernels/cpu.rs:73-124 on integer-valued inputs).  BT_F32: scaled like
 * bt_linear_forward using sx_dev[m]. */
bt_status bt_linear_forward_q(bt_linear* lin, bt_workspace* ws, const int8_t* q_dev,
                              const float* sx_dev, int64_t m, void* out_dev,
                              bt_dtype out_dtype, void* stream);

/* Host-buffer convenience with the reference's calling convention for a CUDA device:
 * x and y live in host memory, as the reference's PackedTensor path moves data over
 * PCIe on every call (RE/kernels/cuda.rs:40-42, RE/kernels/packing.rs:108-133).  f32 in,
 * f32 out.  Synchronous. */
bt_status bt_linear_forward_host(bt_linear* lin, const float* x_host, int64_t m, int64_t x_k,
                                 float* y_host);

/* Per-token absmax int8 quantiser (no counterpart kernel in the reference; defined
 * after QuantizedKVCache::quantize_q8, RE/layers/kv_cache.rs:95-119, without the +128
 * zero point; the BitNet b1.58 form): amax = max|x|, q = clamp(round(x * (127/amax)), -127, 127)
 * with round half away from zero, dequantisation scale s = amax/127, amax == 0 -> q = 0.
 * q_dev [m,k] int8, s_dev [m] f32, qsum_dev [m] int32 (sum_k q, may be NULL). */
bt_status bt_act_quant(const void* x_dev, bt_dtype x_dtype, int64_t m, int64_t k, int8_t* q_dev,
                       float* s_dev, int32_t* qsum_dev, int device, void* stream);


/* Largest activation block bt_linear_forward_noalloc accepts: m * k_pad bytes, where k_pad
 * is k_in rounded up to a multiple of 256 (e.g. 8 tokens x 16384 inputs). */
#define BT_NOALLOC_MAX_ACT_BYTES (128 * 1024)

/* bt_linear_forward for callers that must not allocate device memory.  It has no
 * counterpart in the reference.
 *
 * Some hosts cannot tolerate a cudaMalloc on their inference path: a serving runtime that
 * has already handed every spare byte of the GPU to its own arena (KV cache sized to fit),
 * or a latency-critical loop in which cudaMalloc's implicit device-wide synchronisation
 * would stall other streams.  bt_linear_forward needs scratch for the quantised
 * activations and normally takes it from a bt_workspace (a cudaMalloc at creation) or from
 * a workspace it allocates on first use.  This variant instead keeps that scratch in a
 * fixed array compiled into the library's device image, so the call performs no
 * cudaMalloc / cudaFree and touches no allocator at all.
 *
 * Limits and rules:
 *  - m * k_pad must not exceed BT_NOALLOC_MAX_ACT_BYTES and m must be <= 8; larger requests
 *    fail with BT_ERR_NOMEM and a message, nothing is launched.  With several bases the
 *    output must be BT_F32.
 *  - The array lives once per GPU that loads the library (about 129 KiB of device memory,
 *    held until the process exits) and is shared by every call on that GPU: two calls
 *    whose kernels may overlap (different streams, different threads) race on it.  Issue
 *    these calls on one stream, or order them yourself.
 *  - Nothing in the array needs to start at zero: each call rewrites every byte it later
 *    reads (the quantiser zero-fills the padding up to k_pad).
 *  - The first call on a device looks up the array's device address
 *    (cudaGetSymbolAddress) and, like the first call of any forward entry point, sets the
 *    product kernel's shared-memory attribute (cudaFuncSetAttribute); neither allocates, but
 *    make that first call outside of any stream capture.
 * Same arithmetic, arguments and errors as bt_linear_forward otherwise. */
bt_status bt_linear_forward_noalloc(bt_linear* lin, const void* x_dev, int64_t m, int64_t x_k,
                                    bt_dtype x_dtype, void* y_dev, bt_dtype y_dtype, void* stream);

/* A BitLinear made of several projections that share their input, stacked along the
 * output dimension (q|k|v, gate|up): one launch streams them all.  Each segment is given
 * exactly like bt_linear_create's n_bases == 1 input; seg_rows[i] must be a multiple of
 * 16.  No single call in the reference corresponds to it: it replaces the back-to-back
 * forwards at RE/layers/attention.rs:159-161 and RE/layers/swiglu.rs:30-31. */
bt_status bt_linear_create_fused(bt_linear** out, const uint8_t* const* seg_packed_host,
                                 const int64_t* seg_rows, const float* seg_scales, int n_seg,
                                 int64_t k_in, int device);

/* ---- TTT fast-weight layer ------------------------------------------------------------ */

/* Inner update of TTTLayer::forward_update (RE/layers/ttt.rs:52-68; t_len = 1, chunk = 1)
 * and TTTLayer::forward_chunkwise (RE/layers/ttt.rs:88-113) between the down and up
 * projections: features are L2-normalised (eps 1e-6 added after the sqrt), predicted
 * with the state, and the state takes one gradient step per chunk.
 * w_state_dev [batch, d, d] f32 in/out; feat_dev [batch, t_len, d]; z_dev [batch, t_len, d]
 * receives the predictions made with the pre-update state.  d <= 1024, chunk <= 64. */
bt_status bt_ttt_update(float* w_state_dev, const float* feat_dev, int64_t batch, int64_t t_len,
                        int64_t d, float inner_lr, int64_t chunk, float* z_dev, int device,
                        void* stream);

/* ---- Q8 KV cache + decode attention --------------------------------------------------- */

typedef struct bt_kv_cache bt_kv_cache;

/* QuantizedKVCache::new (RE/layers/kv_cache.rs:26-35) for `batch` sequences: u8 data
 * [batch, n_kv_heads, max_seq_len, head_dim] + f32 scale per (sequence, head, position)
 * for K and V, preallocated (the reference grows it with `cat`, :61-76). */
bt_status bt_kv_create(bt_kv_cache** out, int64_t batch, int64_t n_kv_heads, int64_t head_dim,
                       int64_t max_seq_len, int device);
/* QuantizedKVCache::reset (RE/layers/kv_cache.rs:38-44). */
bt_status bt_kv_reset(bt_kv_cache* cache);
bt_status bt_kv_destroy(bt_kv_cache* cache);
/* Copies position range [0, t_len) of sequence b to host: k_q/v_q [n_kv, t_len, head_dim]
 * u8, k_s/v_s [n_kv, t_len] f32 (any may be NULL).  Synchronous; for tests and state I/O. */
bt_status bt_kv_export(bt_kv_cache* cache, int64_t b, int64_t t_len, uint8_t* k_q_host,
                       float* k_s_host, uint8_t* v_q_host, float* v_s_host);

/* The inverse of bt_kv_export: writes position range [0, t_len) of sequence b from host arrays of the
 * same shapes (any may be NULL).  With bt_kv_export it carries a cache across processes, next to the
 * TTT states of Llama::save_memory / load_memory (RE/model/llama.rs:575-611); bt_model_seek then
 * continues decoding at t_len.  Synchronous. */
bt_status bt_kv_import(bt_kv_cache* cache, int64_t b, int64_t t_len, const uint8_t* k_q_host,
                       const float* k_s_host, const uint8_t* v_q_host, const float* v_s_host);
/* QuantizedKVCache::append (RE/layers/kv_cache.rs:50-92) on its own, one new token per sequence:
 * k_dev, v_dev [batch, n_kv_heads, head_dim] f32 (keys already rotated, as the caller at
 * RE/layers/attention.rs:180-196 passes them) are quantised (RE/layers/kv_cache.rs:95-119) into row
 * pos_dev[b] of sequence b.  Rows with pos outside [0, max_seq_len) are skipped.  Unlike the reference
 * it does not return the dequantised cache: bt_attn_decode reads the cache in place. */
bt_status bt_kv_append(bt_kv_cache* cache, const float* k_dev, const float* v_dev, const int32_t* pos_dev,
                       int64_t batch, void* stream);

/* The attention core of BitAttention::forward for one new token per sequence
 * (RE/layers/attention.rs:166-217 with seq_len == 1): RoPE at pos[b] on q and k
 * (:180-182), QuantizedKVCache::append of k and v (RE/layers/kv_cache.rs:50-92),
 * softmax((q.K^T)/sqrt(head_dim)) . V over positions 0..pos[b] of the dequantised cache,
 * grouped-query sharing of KV heads (:228-239).
 * qkv_dev [batch, (n_heads + 2 n_kv) * head_dim] f32 = q | k | v projections;
 * pos_dev [batch] int32; out_dev [batch, n_heads * head_dim] f32.
 * pos[b] must be < max_seq_len (BT_ERR_SHAPE is not detectable on device: the caller
 * guarantees it, as the reference's RoPE table narrows fail beyond max_position). */
bt_status bt_attn_decode(bt_kv_cache* cache, const float* qkv_dev, const int32_t* pos_dev,
                         int64_t batch, int64_t n_heads, double rope_theta, float* out_dev,
                         void* stream);

/* ---- whole model: one decode step ----------------------------------------------------- */

typedef struct bt_model bt_model;

typedef struct {
    int arch;                     /* 0 = "ttt", 1 = "llama" (RE/model/config.rs:12-18) */
    int vocab_size;
    int hidden_dim;
    int num_layers;
    int n_heads;
    int n_kv_heads;
    int intermediate_dim;
    float inner_lr;
    double rope_theta;            /* default 10000 (RE/model/config.rs:61-63) */
    int max_position_embeddings;  /* default 2048 (RE/model/config.rs:64-66) */
    int max_batch;                /* sequences decoded together, >= 1 */
    int tp_rank;                  /* tensor-parallel rank of this process (0 when tp_size <= 1) */
    int tp_size;                  /* tensor-parallel degree: 0 or 1 = none; else it divides n_kv_heads */
} bt_model_config;

typedef enum {
    BT_W_Q = 0, BT_W_K, BT_W_V, BT_W_O, BT_W_GATE, BT_W_UP, BT_W_DOWN, BT_W_TTT_DOWN, BT_W_TTT_UP
} bt_weight_kind;

typedef enum {
    BT_T_EMBED = 0,   /* [vocab, hidden] */
    BT_T_LM_HEAD,     /* [vocab, hidden], dense (RE/model/llama.rs:23) */
    BT_T_NORM_F,      /* [hidden] */
    BT_T_NORM1,       /* per layer [hidden] */
    BT_T_NORM2
} bt_tensor_kind;

/* BitLlama::load (RE/model/llama.rs:37-158) split into create / set_* / finalize so that
 * the caller owns file parsing.  Weights are given the way a converted checkpoint stores
 * them: ternary projections as packed bytes + scales (one basis here), embeddings, head
 * and norms as f32 host arrays (the engine loads everything as F32, :414-415; embedding
 * and head are kept in bf16 on the device). */
bt_status bt_model_create(bt_model** out, const bt_model_config* cfg, int device);

/* Tensor parallelism (an addition: the reference is single-GPU, RE/model/llama.rs:43,404).
 * One process per GPU.  With tp_size = R > 1 (arch llama only) bt_model_set_linear takes this
 * rank's shard: q/k/v rows of its n_heads/R query and n_kv_heads/R KV heads, gate/up rows
 * [rank*I/R, (rank+1)*I/R), and for o_proj / down_proj the matching input COLUMNS (a
 * [hidden, n_heads/R*head_dim] resp. [hidden, I/R] matrix).  Embedding, norms and lm_head are
 * replicated.  Every rank computes the same hidden state bit for bit, identical to R = 1: the
 * row-parallel projections quantise with the all-reduced max|x| and all-reduce their int32
 * accumulators before scaling.  bt_tp_unique_id gives the 128-byte NCCL id that rank 0
 * creates and hands to the others (any transport); bt_model_tp_init joins the communicator
 * (collective call, after bt_model_finalize, before the first step). */
bt_status bt_tp_unique_id(uint8_t* id128_out);
bt_status bt_model_tp_init(bt_model* m, const uint8_t* id128);
/* Optional, faster exchange for the row-parallel projections (no reference counterpart): the
 * two all-reduces run as kernels of this library over NVLink peer memory instead of NCCL calls.
 * Each rank calls bt_model_tp_peer_export (64-byte CUDA IPC handle of its inbox), the ranks
 * exchange the handles by any transport, and each calls bt_model_tp_peer_import with all
 * tp_size handles in rank order (64 bytes each; its own entry is ignored).  One process per
 * GPU, all on one node with peer access.  Results are bit-identical to the NCCL path and to
 * tp_size = 1.  A rank that never arrives makes the others' waits run out (they are bounded in time,
 * 5 s unless bt_model_tp_set_timeout says otherwise): the exchange leaves the hidden state as it was,
 * the remaining exchanges of the step no longer wait, bt_model_forward_one returns BT_ERR_TIMEOUT
 * (callers of bt_model_step_dev see it through bt_device_check at their next synchronisation), and
 * decoding continues only after every rank has called bt_model_reset and bt_model_tp_resync (which
 * restarts the exchange epochs) with a host-side barrier before and after the latter, so that no rank
 * clears flags a faster rank has already written for the next step.  bt_model_tp_peer_import with handles = NULL drops the inbox and returns the model to the
 * NCCL path (all ranks must do the same). */
bt_status bt_model_tp_peer_export(bt_model* m, uint8_t* handle64_out);
bt_status bt_model_tp_peer_import(bt_model* m, const uint8_t* handles);
/* How long an exchange kernel waits for its peers (milliseconds, >= 1).  Drops the captured step graphs. */
bt_status bt_model_tp_set_timeout(bt_model* m, int milliseconds);
/* Restarts the exchange epochs and clears this rank's inbox flags after a timeout; see above for the barriers
 * the host has to put around it.  Not needed in normal operation (bt_model_reset leaves the epochs alone). */
bt_status bt_model_tp_resync(bt_model* m);
/* Leaves tensor parallelism: closes the peer mappings and destroys the communicator (collective in the
 * sense that every rank should do it before any rank's inbox memory goes away).  bt_model_destroy does
 * the same implicitly. */
bt_status bt_model_tp_destroy(bt_model* m);
bt_status bt_model_set_linear(bt_model* m, int layer, bt_weight_kind kind, const uint8_t* packed_host,
                              int64_t n_out, int64_t k_in, float scale);
/* The same for a projection with several bases, as the converter writes them by default (NumBases = 3,
 * tools/conversion/convert_llama_v2.py:169): packed_host [n_out, k_in/4, n_bases], scales_host [n_bases]
 * (AdaptiveBitLinear::load, RE/layers/adaptive_linear.rs:40-129; the reference rebuilds a dense f32 matrix from
 * them, this library streams every basis as 2-bit tiles and adds the per-basis products in basis order).
 * q, k, v of a layer must agree on n_bases, and so must gate and up.  A model with any multi-basis projection
 * runs its decode step with the quantiser and product kernels launched separately.  One basis only on
 * tensor-parallel models. */
bt_status bt_model_set_linear_bases(bt_model* m, int layer, bt_weight_kind kind, const uint8_t* packed_host,
                                    int64_t n_out, int64_t k_in, int n_bases, const float* scales_host);
bt_status bt_model_set_tensor(bt_model* m, bt_tensor_kind kind, int layer, const float* data_host,
                              int64_t n_elem);
/* The same with the 16-bit storage type of the embedding and the lm_head chosen by the caller: BT_BF16 (what
 * bt_model_set_tensor uses) or BT_F16.  A converted checkpoint stores these tensors as IEEE halves
 * (tools/conversion/convert_llama_v2.py:262-283) and the reference widens them to f32 unchanged
 * (RE/model/llama.rs:414-415): with BT_F16 the device tables hold exactly those values at the same 2 bytes per
 * element, whereas bf16 would round them to 8 significand bits.  Norm weights are kept in f32 either way. */
bt_status bt_model_set_tensor_typed(bt_model* m, bt_tensor_kind kind, int layer, const float* data_host,
                                    int64_t n_elem, bt_dtype storage);
bt_status bt_model_finalize(bt_model* m);
bt_status bt_model_destroy(bt_model* m);
/* reset_kv_cache + fresh zero TTT states (RE/model/llama.rs:179-188,161-170). */
bt_status bt_model_reset(bt_model* m);
/* BitLlama::forward_one (RE/model/llama.rs:201-272) for `batch` sequences that are all at
 * the same position: host token ids in, optional host logits [batch, vocab] f32 and/or
 * greedy next ids out (last index among equal maxima, :510-515).  Synchronous. */
bt_status bt_model_forward_one(bt_model* m, const int32_t* tokens_host, int batch,
                               float* logits_host, int32_t* next_host);
/* Same step with everything on the device and no synchronisation: the ids are read from
 * tokens_dev, results stay in the model's buffers (bt_model_logits / bt_model_next). */
bt_status bt_model_step_dev(bt_model* m, const int32_t* tokens_dev, int batch, void* stream);
const float* bt_model_logits(bt_model* m);   /* device [max_batch, vocab] */
const int32_t* bt_model_next(bt_model* m);   /* device [max_batch] */
/* Current position (tokens consumed since the last reset). */
int bt_model_pos(const bt_model* m);
/* State I/O aid: declares that the KV caches already hold `pos` positions (contents as
 * they are in device memory: zero keys/values after a reset, or whatever the caller put
 * there through bt_model_kv_cache) and continues decoding from there.  The reference's
 * counterpart is assigning BitLlama::current_pos together with restored caches
 * (RE/model/llama.rs:35,269). */
bt_status bt_model_seek(bt_model* m, int pos);
/* TTT state of one layer: device pointer [max_batch, d_small, d_small] f32 (NULL for
 * arch llama); KV cache of one layer (NULL for arch ttt). */
float* bt_model_ttt_state(bt_model* m, int layer);
bt_kv_cache* bt_model_kv_cache(bt_model* m, int layer);
/* Batched prefill: n_tokens new tokens for each of `batch` sequences (tokens_host [batch][n_tokens]), all
 * sequences at the current position.  Equivalent to n_tokens calls of bt_model_forward_one - the reference
 * CLI's prefill loop, RE/model/llama.rs:495-498: the Q8 caches end up holding the new positions and every
 * token attends over the dequantised cache up to itself (causal rule of RE/layers/attention.rs:249-262) - but
 * every projection runs once over all rows on the tensor-core product, K/V rows are appended in one pass and
 * attention walks blocks of query positions.  arch ttt: the fast-weight state takes one gradient step per
 * ttt_chunk tokens (TTTLayer::forward_chunkwise, RE/layers/ttt.rs:80-119, as BitLlama::forward_chunkwise
 * applies it, RE/model/llama.rs:275-312); ttt_chunk = 1 is the token-by-token update of forward_one.
 * logits_host [batch, vocab] (optional) and next_host [batch] (optional) are those of the LAST token.
 * Long inputs are worked off in chunks of at most 2048 rows (sequences x tokens).  Synchronous.
 * Not available on tensor-parallel models (BT_ERR_ARG). */
bt_status bt_model_prefill(bt_model* m, const int32_t* tokens_host, int batch, int n_tokens, int ttt_chunk,
                           float* logits_host, int32_t* next_host);

/* Inspection aid: the tensors between the calls of BitLlamaBlock::forward (RE/model/block.rs:87-134).
 * While a trace buffer is set, every decode step runs launch by launch (no graph replay) and copies, per layer,
 *   h_in [rows, hidden] | q|k|v [rows, (n_heads + 2 n_kv) head_dim] | attention output [rows, hidden] |
 *   h after the attention residual | silu(gate)*up [rows, intermediate] | h after the MLP residual
 * into trace_dev ([num_layers] blocks of that layout, every tensor with room for `rows` rows,
 * bt_model_trace_floats(m, rows) floats in all; arch ttt: the down-projected features and the TTT prediction,
 * d_small wide, take the places of q|k|v and the attention output; tensor-parallel models record their local
 * slices).  A decode step fills `batch` rows; bt_model_prefill fills sequences x tokens rows, ordered
 * [sequence][token], and cuts its chunks to fit `rows`.  rows >= max_batch.  The kernels and their
 * arguments are the ones of the normal step.  trace_dev = NULL switches it off.  Synchronises the device. */
int64_t bt_model_trace_floats(const bt_model* m, int rows);
bt_status bt_model_set_trace(bt_model* m, float* trace_dev, int rows);
/* Ternary-weight bytes streamed by one decode step (sum over all BitLinear tiles). */
int64_t bt_model_ternary_bytes(const bt_model* m);
/* Measurement aid (no counterpart in the reference): enqueues only the ternary-product
 * launches of one decode step, in step order, on whatever the activation buffers hold,
 * writing to scratch outputs; model state is not touched.  as_in_step = 0: the plain product
 * on already quantised activations; as_in_step = 1: the launches exactly as the step issues
 * them (for one or two sequences: RMSNorm / absmax quantisation prologues and the SwiGLU and
 * accumulate epilogues inside the product kernel).  *n_launches receives the number of kernel
 * launches enqueued. */
bt_status bt_model_enqueue_products(bt_model* m, int batch, int as_in_step, void* stream, int* n_launches);
/* Kernel launches of one decode step at this batch size. */
int bt_model_launches_per_step(const bt_model* m, int batch);

#ifdef __cplusplus
}
#endif
#endif /* BITTTT_H */
