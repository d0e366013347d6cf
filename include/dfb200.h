/* dfb200 — C ABI of the B200 (sm_100a) int4 decode-step kernels.
 *
 * Plain pointers and sizes only; every pointer is a CUDA device pointer unless its name ends in
 * `_host`. `stream` is a cudaStream_t passed as void* (NULL = the default stream). Every function
 * returns 0 on success and a non-zero code otherwise (1 = CUDA error, 2 = bad argument); the text of
 * the last error of the calling thread is returned by dfb_last_error(). Nothing here aborts, traps
 * or falls back to a CPU path. The library allocates no device memory except CUDA graph objects
 * owned by an engine: all buffers, including scratch, belong to the caller.
 *
 * Each entry point names the interface of LoveManna/deltaforge it stands in for (paths relative to
 * that project's root). bf16 tensors are passed as void*, row-major with the last axis contiguous.
 */
#ifndef DFB200_H
#define DFB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DFB_OK 0
#define DFB_ERR_CUDA 1
#define DFB_ERR_ARG 2

/* Arithmetic of the int4 GEMV: FAST sums x*q per 128-group in fp32 and applies the group scale once
 * (weights are not rounded to bf16); EXACT rounds every dequantised weight to bf16 first, exactly as
 * torch_dequant_gemv_int4 does; FAST_HALF2 is FAST with packed fp16 partial sums. */
#define DFB_MATH_FAST 0
#define DFB_MATH_EXACT 1
#define DFB_MATH_FAST_HALF2 2

#define DFB_PROLOGUE_NONE 0
#define DFB_PROLOGUE_RMSNORM 1  /* x <- rms_norm(x, norm_w, eps), reference.py:92-96 */
#define DFB_PROLOGUE_SILU_MUL 2 /* x <- silu(x) * up, reference.py:692-693 */

#define DFB_EPILOGUE_STORE 0
#define DFB_EPILOGUE_RESIDUAL 1 /* out <- residual + y, reference.py:730,735 */
#define DFB_EPILOGUE_CONV 2     /* columns < conv_dim: causal conv step + SiLU, reference.py:496-510 */

const char* dfb_last_error(void);
int dfb_abi_version(void);

/* ---- int4, group-wise, K-major -------------------------------------------------------------- */

/* Group width along K the format uses for a K-deep weight: 128 when K is a multiple of 256, else one group per half of
 * K; 0 where the format does not exist (odd K, or a half that is not a power of two). group_size_for,
 * src/deltaforge/kernels/quantised_linear.py:193-207. */
int dfb_int4_group_size(int K);

/* weight [N, K] (row-major, bf16 or fp32) -> packed [K/2, N] uint8 + scale [K/group, N] fp32, bit for bit what
 * quantise_int4_k_major returns (src/deltaforge/kernels/tiled_gemv.py:242-278): symmetric, scale = amax(group) / 7
 * (1 for an all-zero group), round half to even, clamp to [-7, 7], stored + 8, row j low nibble / row j + K/2 high. */
int dfb_int4_quantise_k_major(const void* weight, int weight_is_bf16, int N, int K, uint8_t* packed, float* scale,
                              void* stream);

/* packed [K/2, N] uint8 -> signed values [K, N] int8. The integer half of dequantise_int4_k_major,
 * src/deltaforge/kernels/tiled_gemv.py:284-287. */
int dfb_int4_unpack(const uint8_t* packed, int K, int N, int8_t* out, void* stream);

/* packed + scale [K/group, N] -> bf16 weight [K, N] = bf16(fp32(value) * fp32(scale)).
 * dequantise_int4_k_major followed by the cast in torch_dequant_gemv_int4:
 * src/deltaforge/kernels/tiled_gemv.py:281-288, src/deltaforge/kernels/visible_int4_head.py:198. */
int dfb_int4_dequant(const uint8_t* packed, const void* scale, int scale_is_bf16, int K, int N, int group,
                     void* out_bf16, void* stream);

typedef struct dfb_gemv_desc {
  const void* x; /* bf16 [rows, K] */
  int64_t x_stride;
  int32_t rows;
  const uint8_t* packed; /* [K/2, N] */
  const void* scale;     /* [K/group, N], fp32 or bf16 */
  int32_t scale_is_bf16;
  int32_t K, N, group;
  int32_t prologue;
  const void* norm_w; /* bf16 [K] */
  float eps;
  const void* up; /* bf16 [rows, K] */
  int64_t up_stride;
  int32_t epilogue;
  void* out; /* bf16 [rows, N] */
  int64_t out_stride;
  const void* residual; /* bf16 [rows, N]; may alias out */
  int64_t residual_stride;
  void* conv_state;   /* bf16 [rows, conv_dim, 3], oldest tap first, updated in place */
  const void* conv_w; /* bf16 [conv_dim, 4] */
  int32_t conv_dim;
  void* scratch; /* dfb_int4_gemv_scratch_bytes() bytes; zero it once before first use */
  size_t scratch_bytes;
  int32_t math;
  int32_t force_tiled; /* 1: use the register-tiled kernel even where the streaming (TMA) kernel applies */
  const void* packed_k8; /* optional: the weight re-packed by dfb_int4_repack_k8; enables the streaming kernel */
  const void* packed_mma; /* optional: the weight and its scales re-packed by dfb_int4_repack_mma (pair = 0); with one
                           * activation row and FAST arithmetic the integer tensor-core GEMV runs on it */
} dfb_gemv_desc;

/* Re-pack a K-major int4 weight for the streaming GEMV: packed [K/2, N] bytes -> out [K/8, N] uint32,
 * word (kb, n) = the eight nibbles (still value + 8) of column n for rows 8kb .. 8kb+7, nibble i = row
 * 8kb + i. Same values as quantise_int4_k_major produces (src/deltaforge/kernels/tiled_gemv.py:242-278),
 * another order; done once at install time. */
int dfb_int4_repack_k8(const uint8_t* packed, int K, int N, void* out, void* stream);

/* Re-pack a K-major int4 weight AND its scales for the one-row GEMV on the integer tensor-core instruction
 * (mma.sync m16n8k32): tiles of 256 columns (128 where N < 4096), one contiguous unit per (tile, 128-row group) holding
 * the group's words in the order the instruction's operand fragments are read, then the unit's scales. Same values
 * and scales as quantise_int4_k_major produces (src/deltaforge/kernels/tiled_gemv.py:242-278); columns beyond N are
 * stored as zeros. pair = 1 lays a gate_proj|up_proj matrix (N = 2 * intermediate) out so that a tile holds 128 gate
 * columns and the up columns of the same channels (the decode engine fuses SwiGLU on that form). K % 128 == 0.
 * `out` takes dfb_int4_repack_mma_bytes() bytes, 16-byte aligned. */
size_t dfb_int4_repack_mma_bytes(int K, int N, int pair, int scale_is_bf16);
int dfb_int4_repack_mma(const uint8_t* packed, const void* scale, int scale_is_bf16, int K, int N, int pair, void* out,
                        void* stream);

/* Scratch for one GEMV problem: split-K partial sums, one arrival counter per column tile, and in the
 * last 256 bytes a status word (int32, 0 = ok) that the streaming kernel sets if one of its bounded
 * waits gives up. Zero the scratch once before the first launch; every launch leaves the counters zero. */
size_t dfb_int4_gemv_scratch_bytes(int rows, int K, int N, int group);

/* y = x @ dequant(W), with optional fused prologue and epilogue. Stands in for the op
 * deltaforge::tiled_gemv_int4(x, packed, scale, group_size) (src/deltaforge/kernels/tiled_gemv.py:
 * 915-958) and torch_dequant_gemv_int4 (src/deltaforge/kernels/visible_int4_head.py:187-199); with
 * the prologue/epilogue it also absorbs RMSNorm.forward (src/deltaforge/reference.py:92-96), the
 * residual adds of DecoderLayer.forward (:730, :735), SwiGLUMLP's silu*up (:692-693) and the causal
 * conv decode step (src/deltaforge/kernels/inline_causal_conv.py:98-129). */
int dfb_int4_gemv(const dfb_gemv_desc* desc, void* stream);

/* The same GEMV for callers that hold no device scratch: the split-K partial sums and arrival counters
 * live in a device array that is part of the library image, so the call allocates nothing, on the host
 * or the device. This entry point has no counterpart in the reference (its Triton GEMV takes its
 * scratch from torch's allocator). It always runs the register-tiled split-K kernel, and serves only
 * the group-128 layout (K % 256 == 0, N % 8 == 0); `scratch`, `scratch_bytes`, `force_tiled` and
 * `packed_k8` of the descriptor are ignored. The built-in scratch holds
 * dfb_int4_gemv_static_max_partials_bytes() (2 MiB) of partial sums, rows * (K/256) * N * 4 bytes per
 * problem, and 4096 column-tile counters: every layer projection of the 4B decode step at one row
 * fits, the LM head does not, and a problem beyond either limit is refused with DFB_ERR_ARG and a
 * message that names both sizes. The first call on each device looks the array's address up (the
 * device must be current); make that first call before any stream capture begins. Each call clears its
 * counters in stream order before the launch. There is one array per device: two calls whose
 * execution may overlap (different streams, or different host threads on different streams) race on
 * it and give wrong sums, so callers serialise them on one stream. */
size_t dfb_int4_gemv_static_max_partials_bytes(void);
int dfb_int4_gemv_static(const dfb_gemv_desc* desc, void* stream);

/* ---- elementwise ops with the reference's op contracts --------------------------------------- */

/* deltaforge::rms_norm, src/deltaforge/kernels/fused_rmsnorm_residual.py:201-226. */
int dfb_rms_norm(const void* x, const void* weight, float eps, int rows, int n, void* out, void* stream);
/* deltaforge::add_rms_norm -> (resid_out = residual + x, out = rms_norm(resid_out)), :164-193. */
int dfb_add_rms_norm(const void* x, const void* residual, const void* weight, float eps, int rows, int n,
                     void* resid_out, void* out, void* stream);
/* deltaforge::silu_mul, src/deltaforge/kernels/fused_swiglu.py:51-74. */
int dfb_silu_mul(const void* gate, const void* up, int64_t n, void* out, void* stream);
/* deltaforge::partial_rope: x (batch, heads, seq, d), cos/sin (batch, seq, rotary_dim).
 * src/deltaforge/kernels/fused_rope.py:97-150. */
int dfb_partial_rope(const void* x, const void* cos, const void* sin, int batch, int heads, int seq, int d,
                     int rotary_dim, void* out, void* stream);
/* deltaforge::fused_causal_conv_step: x (B, C), conv_cache (B, C, 3) updated in place, weight (C, 4).
 * src/deltaforge/kernels/fused_causal_conv.py:136-176. */
int dfb_causal_conv_step(const void* x, void* conv_cache, const void* weight, int batch, int channels, void* out,
                         void* stream);

/* ---- Gated DeltaNet ---------------------------------------------------------------------------- */

/* deltaforge::delta_rule_step(state, q, k, v, g, beta) -> (out, new_state); all fp32, q and k already
 * normalised. src/deltaforge/kernels/gated_delta_step.py:109-177. */
int dfb_delta_rule_step(const float* state, const float* q, const float* k, const float* v, const float* g,
                        const float* beta, int batch, int heads, int dk, int dv, float* out, float* state_out,
                        void* stream);

typedef struct dfb_deltanet_desc {
  int32_t batch, num_k_heads, num_v_heads, dk, dv;
  const void* q; /* bf16, post-conv, [Hk*dk] per sequence */
  const void* k;
  const void* v; /* [Hv*dv] */
  const void* z; /* [Hv*dv] */
  const void* b; /* [Hv] */
  const void* a; /* [Hv] */
  int64_t row_stride;
  const float* a_log;
  const float* dt_bias;
  const float* norm_w;
  int32_t norm_w_is_bf16; /* the model holds the norm weight in bf16: round weight*normed to bf16 */
  float eps;
  float* state; /* [batch, Hv, dk, dv], in place */
  void* out;    /* bf16 [batch, Hv*dv] */
  int64_t out_stride;
} dfb_deltanet_desc;

/* Everything of GatedDeltaNet.forward between the conv and out_proj for one token:
 * src/deltaforge/reference.py:518-549 (l2norm :403-404, recurrence :450-458, GatedRMSNorm :115-121). */
int dfb_deltanet_step(const dfb_deltanet_desc* desc, void* stream);

/* ---- decode attention ---------------------------------------------------------------------------- */

typedef struct dfb_attn_desc {
  int32_t batch, hq, hkv, d;
  const void* q; /* bf16 */
  int64_t q_stride, qh_stride;
  const void* kcache; /* bf16 [batch, hkv, max_seq, d] */
  const void* vcache;
  int64_t kv_batch_stride, kv_head_stride;
  int32_t key_len;
  const int32_t* pos; /* optional device scalar: key_len = *pos + 1 */
  float scale;
  int32_t splits;
  void* scratch; /* dfb_attn_scratch_bytes(); zero once */
  size_t scratch_bytes;
  const void* gate; /* optional bf16 gate logits */
  int64_t gate_stride, gateh_stride;
  int32_t gate_is_swish;
  void* out; /* bf16 [batch, hq*d] */
  int64_t out_stride;
} dfb_attn_desc;

size_t dfb_attn_scratch_bytes(int batch, int hq, int hkv, int d, int splits);

/* deltaforge::gqa_decode_attention(q, k, v, scale) (src/deltaforge/kernels/gqa_decode.py:138-199) when
 * splits == 1 and deltaforge::split_kv_decode_attention(q, k, v, scale, splits)
 * (src/deltaforge/kernels/flash_decode_splitkv.py:177-256) otherwise; with `gate` it also applies
 * apply_output_gate (src/deltaforge/reference.py:558-568, :675-676). */
int dfb_attn_decode(const dfb_attn_desc* desc, void* stream);

typedef struct dfb_attn_prep_desc {
  int32_t batch, hq, hkv, d, rotary_dim;
  const void* proj; /* bf16 [batch, hq*(2d or d) + 2*hkv*d] */
  int64_t proj_stride;
  const void* q_norm_w;
  const void* k_norm_w;
  float eps;
  const float* inv_freq; /* [rotary_dim/2], as the model holds it */
  const int32_t* pos;    /* device scalar */
  void* q_out;           /* bf16 [batch, hq, d] */
  void* kcache;
  void* vcache;
  int64_t kv_batch_stride, kv_head_stride;
  int32_t attn_output_gate;
  int32_t max_seq; /* rows per head of the cache; the caller keeps *pos below it */
} dfb_attn_prep_desc;

/* q_norm / k_norm, partial RoPE at *pos and the KV-cache write of GatedAttention.forward:
 * src/deltaforge/reference.py:632-650. */
int dfb_attn_prep(const dfb_attn_prep_desc* desc, void* stream);

typedef struct dfb_attn_step_desc {
  int32_t batch, hq, hkv, d, rotary_dim;
  const void* proj; /* bf16 [batch, hq*(2d or d) + 2*hkv*d]: per head query(|gate), then keys, then values */
  int64_t proj_stride;
  const void* q_norm_w;
  const void* k_norm_w;
  float eps;
  const float* inv_freq;
  const int32_t* pos; /* device scalar: tokens already cached; the new token is row *pos */
  void* kcache;       /* bf16 [batch, hkv, max_seq, d] */
  void* vcache;
  int64_t kv_batch_stride, kv_head_stride;
  int32_t max_seq;
  int32_t attn_output_gate, gate_is_swish;
  float scale;
  int32_t splits;       /* power of two; ceil(max_seq / splits) <= 160 */
  int32_t cluster_size; /* 1..8 dividing splits, with splits / cluster_size <= 16; 0 = min(splits, 4) */
  void* scratch;        /* dfb_attn_scratch_bytes(batch, hq, hkv, d, splits); zero once */
  size_t scratch_bytes;
  void* out; /* bf16 [batch, hq*d] */
  int64_t out_stride;
  int32_t* status; /* optional device word, set non-zero if the bounded wait on the staging copies gives up */
} dfb_attn_step_desc;

/* dfb_attn_prep followed by dfb_attn_decode with the output gate, in one launch: everything of
 * GatedAttention.forward between q/k/v_proj and o_proj for one new token (src/deltaforge/reference.py:
 * 621-676). Takes head_dim 256 and 1, 2 or 4 query heads per KV head. */
int dfb_attn_step(const dfb_attn_step_desc* desc, void* stream);

/* ---- whole decode step ------------------------------------------------------------------------- */

typedef struct dfb_linear {
  const uint8_t* packed;
  const void* scale;
  int32_t scale_is_bf16;
  int32_t K, N, group;
  const void* packed_k8; /* optional re-packed copy (dfb_int4_repack_k8) */
  const void* packed_mma; /* optional re-packed copy with scales (dfb_int4_repack_mma); batch-1 steps prefer it */
  int32_t mma_pair;       /* packed_mma was made with pair = 1 (the gate_up projection) */
} dfb_linear;

#define DFB_LAYER_DELTANET 0
#define DFB_LAYER_ATTENTION 1

typedef struct dfb_layer_desc {
  int32_t kind;
  const void* input_norm_w; /* bf16 [hidden] */
  const void* post_norm_w;
  dfb_linear in_proj;  /* DeltaNet: in_proj_qkv|z|b|a along N; attention: q_proj|k_proj|v_proj */
  dfb_linear out_proj; /* out_proj / o_proj */
  dfb_linear gate_up;  /* gate_proj|up_proj */
  dfb_linear down;
  const void* conv_w; /* bf16 [conv_dim, 4] */
  const float* a_log;
  const float* dt_bias;
  const float* gnorm_w;
  int32_t gnorm_w_is_bf16;
  void* conv_state; /* bf16 [batch, conv_dim, 3] */
  float* recurrent; /* [batch, Hv, dk, dv] */
  const void* q_norm_w;
  const void* k_norm_w;
  void* kcache; /* bf16 [batch, hkv, max_seq, d] */
  void* vcache;
} dfb_layer_desc;

typedef struct dfb_model_desc {
  int32_t hidden, intermediate, vocab, num_layers, batch, max_seq;
  int32_t hq, hkv, head_dim, rotary_dim, attn_output_gate, gate_is_swish;
  int32_t lin_k_heads, lin_v_heads, lin_dk, lin_dv;
  float eps;
  const float* inv_freq;
  const void* embed; /* bf16 [vocab, hidden] */
  const void* final_norm_w;
  dfb_linear head;
  const dfb_layer_desc* layers_host; /* host array of num_layers entries, copied at creation */
  int64_t* tokens;  /* [batch]: input token of the step, overwritten with the greedy next token */
  int64_t* history; /* optional [max_seq, batch]: history[p] = token chosen after position p */
  int32_t* pos;     /* device scalar: tokens already in the cache; the step advances it */
  void* logits;     /* bf16 [batch, vocab] */
  void* workspace;  /* dfb_engine_workspace_bytes(); zero once before creation */
  size_t workspace_bytes;
  int32_t attn_splits;
  int32_t math;
  /* Tensor parallelism: > 1 says this engine holds one rank's shard (its heads, its slice of the MLP and of
   * the vocabulary; all shapes above are the local ones). The projections that end each half of a layer are
   * sharded along K: they leave fp32 partial sums [batch, hidden] in dfb_engine_partial_buffer() instead of
   * adding into the residual stream, the caller adds that buffer across ranks (an all-reduce on the same
   * stream) between dfb_engine_step_segment() calls, and picks the token across the vocabulary shards itself. */
  int32_t tp_size;
  int32_t tp_rank;
  /* Optional, with tp_size > 1: host array of tp_size device pointers, entry r = rank r's exchange buffer of
   * dfb_engine_tp_exchange_bytes() zeroed bytes, each mapped into this process (peer access over NVLink; entry
   * tp_rank is this rank's own). With it the ranks exchange inside the kernels: the K-sharded projections
   * store their fp32 partial sums, tagged with an epoch, straight into every rank's buffer, the next kernel
   * waits (bounded, reporting through the status word) for all ranks' words, adds them in rank order and adds
   * the result to the residual stream; the token is picked across shards the same way. No collective library
   * call remains, dfb_engine_step / capture / replay / decode_host work as for one GPU, and every rank must
   * run the same number of steps. One rank per GPU: kernels of different ranks wait on one another. Every
   * engine starts its epoch counter at 1, so the buffers must be zero when the engines are created (words left
   * by an earlier engine would carry valid-looking tags), and a model may have at most 127 layers (254
   * exchanges per token). A wait gives up after about two seconds and sets status 50; the ranks' hosts must
   * therefore start a step within that time of one another (a barrier before the first launch). */
  void* const* tp_peer_slots;
} dfb_model_desc;

size_t dfb_engine_workspace_bytes(const dfb_model_desc* desc);

/* One engine = one model replica's decode step: ReferenceModel.forward at seq_len 1 plus the argmax of
 * greedy_decode (src/deltaforge/reference.py:779-817, src/deltaforge/model.py:141-147). */
int dfb_engine_create(const dfb_model_desc* desc, void** engine_out);
int dfb_engine_destroy(void* engine);
/* Enqueue the kernels of one step on `stream` (no graph). */
int dfb_engine_step(void* engine, void* stream);
/* Tensor-parallel engines: a step is dfb_engine_num_segments() = 2 * layers + 1 segments (embedding + first half
 * of layer 0; second half of layer l; first half of layer l + 1; ...; LM head). Every segment but the first
 * starts by adding the (all-reduced) partial buffer to the residual stream. */
int dfb_engine_num_segments(void* engine);
int dfb_engine_step_segment(void* engine, int segment, void* stream);
void* dfb_engine_partial_buffer(void* engine);
/* Bytes of one rank's exchange buffer for tp_peer_slots. */
size_t dfb_engine_tp_exchange_bytes(int batch, int hidden, int tp_size);
/* Capture one step into a CUDA graph (the position is read from device memory, so one graph serves
 * every token; the reference re-records per step, src/deltaforge/kernels/static_cache.py:62-74). */
int dfb_engine_capture(void* engine, void* stream);
/* Launch the captured step `steps` times back to back (greedy: each step consumes the token the
 * previous one produced). */
int dfb_engine_replay(void* engine, int steps, void* stream);
/* Serving-style loop with host buffers: per step copy the input token host->device, run the graph,
 * copy the chosen token device->host and wait for it. tokens_host holds [batch] input tokens on
 * entry; out_host receives [steps, batch]. Both should be pinned for the copies to be asynchronous. */
int dfb_engine_decode_host(void* engine, const int64_t* tokens_host, int steps, int64_t* out_host, void* stream);
/* Wait for `stream` and read the engine's status word: 0, or the code a kernel recorded when one of its
 * bounded waits (on a shared-memory barrier fed by asynchronous copies) gave up instead of hanging. */
int dfb_engine_status(void* engine, int* status_host, void* stream);
/* How far ahead the kernels of a batch-1 step ask the L2 cache for weights: every launch requests, a slice
 * per CTA, the int4 words and scales of the projection `distance` GEMVs after the one it runs (or precedes),
 * so HBM keeps streaming while the kernels work through their dependent latencies. 0 (the default) switches it
 * off: under programmatic dependent launch the next kernel's own copies are normally in flight already, and on
 * B200 the extra requests cost 1.5 to 3 % of the step. Takes effect for steps enqueued or captured afterwards. No counterpart in the reference
 * (its kernels rely on the hardware's own prefetching, src/deltaforge/kernels/tiled_gemv.py:452-454). */
int dfb_engine_set_prefetch_distance(void* engine, int distance);
/* Profiling of the graph-of-kernels step: with `buffer` (device memory, max_launches * ctas_per_launch * 8
 * int64, zeroed by the caller) set, one thread of every CTA of launch number l of a step stores %globaltimer
 * (ns) at buffer[(l * ctas_per_launch + cta) * 8 + mark]; marks: 0 kernel entry, 1 the wait for the previous
 * kernel returned, 2 activation ready in shared memory, 3 dot products done (all weights arrived), 4 the first
 * unit of weights done, 5 cluster barrier passed, 6 exit, 7 this CTA's copies (and prefetches) issued. NULL switches it
 * off. Applies to steps enqueued or captured afterwards. */
int dfb_engine_set_trace(void* engine, int64_t* buffer, int max_launches, int ctas_per_launch);
/* Number of kernel launches in one step. */
int dfb_engine_launches_per_step(void* engine);

#ifdef __cplusplus
}
#endif

#endif /* DFB200_H */
