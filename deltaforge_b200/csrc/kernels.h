// Host-side launch interface of the decode-step kernels. Internal to the library: the public
// surface is the C ABI in include/dfb200.h, whose entry points fill these structs.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace dfb {

typedef __nv_bfloat16 bf16;

// Optional timeline of one launch (profiling): see trace_mark() in common.cuh. buf == nullptr: off.
constexpr int TRACE_PHASES = 8;
struct Trace {
  long long* buf;
  int slot;  // index of the launch within the step
  int ctas;  // CTAs recorded per launch
};

// PRO_ATTN_MERGE (engine-internal, cluster kernel only): the activation is the gated attention output, formed on the
// fly from the partial results the split-KV attention step left per slice cluster (see AttnMerge)
enum Prologue { PRO_NONE = 0, PRO_RMSNORM = 1, PRO_SILU_MUL = 2, PRO_ATTN_MERGE = 3 };

// The last step of split-KV attention, done by its consumer: head h's output is sum_c w_c acc[h][c][:] / sum_c w_c l[h][c]
// with w_c = exp(m[h][c] - max_c m[h][c]), rounded to bf16, then multiplied by the bf16 output gate, which the attention
// step left already activated (src/deltaforge/reference.py:558-568, :675-676). acc [heads, nclusters, d] fp32,
// ml [heads, nclusters, 2] = (m, l).
struct AttnMerge {
  const float* acc;
  const float* ml;
  int nclusters;  // 1..8
  int d;          // head dim (a multiple of 128)
  const bf16* gate;  // optional activated gate, bf16(sigmoid(logit)): element (h, i) at gate[h * gateh_stride + i]
  long gateh_stride;
};
// EPI_PARTIAL_F32 (engine-internal, tensor parallelism): `out` is an fp32 buffer that receives the unrounded sum
// EPI_PARTIAL_PEER (engine-internal): the unrounded sum goes, tagged with an epoch, straight into a slot of every
// rank's exchange buffer (peer stores over NVLink); see TpPeer
// EPI_SWIGLU (engine-internal, cluster kernel only): the matrix is gate_proj|up_proj along N; `out` receives the N/2
// values bf16(bf16(silu(gate)) * up) of SwiGLUMLP instead of the N projections
enum Epilogue { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_CONV = 2, EPI_PARTIAL_F32 = 3, EPI_PARTIAL_PEER = 4, EPI_SWIGLU = 5 };

// Where the K-sharded projections of a tensor-parallel rank leave their partial sums when the ranks exchange
// them by peer stores: slots[r] is rank r's exchange buffer (8-byte words {fp32 bits, epoch}); this rank
// writes word word_off + row * N + n of every rank's buffer. The epoch is *epoch_ctr * 256 + epoch_off.
constexpr int TP_MAX = 8;
struct TpPeer {
  unsigned long long* slots[TP_MAX];
  int tp_size;
  const unsigned* epoch_ctr;
  int epoch_off;
  long word_off;
};
// MATH_FAST sums x*q per scale group and applies the fp32 scale once per group (the weight is
// never rounded to bf16); MATH_EXACT rounds every dequantised weight to bf16 before the product,
// as the reference's expression does.
enum Math { MATH_FAST = 0, MATH_EXACT = 1, MATH_FAST_HALF2 = 2 };

struct GemvParams {
  // activation, [rows, K] bf16
  const bf16* x;
  long x_stride;
  int rows;
  // weight: packed [K/2, N] uint8 (low nibble row j, high nibble row j + K/2), scale [K/group, N]
  const uint8_t* packed;
  const uint32_t* packed_k8;  // optional re-packed copy [K/8, N] words for the streaming kernel
  const unsigned char* packed_mma;  // optional copy in the tensor-core GEMV's unit order (launch_int4_repack_mma), scales included
  int mma_pair;                     // that copy pairs gate_proj and up_proj columns (made for EPI_SWIGLU)
  const void* scale;
  int scale_bf16;  // 0: fp32 scales, 1: bf16 scales
  int K, N, group;
  // prologue
  int prologue;
  const bf16* norm_w;  // PRO_RMSNORM: x <- bf16(x * rsqrt(mean(x^2) + eps) * (1 + norm_w))
  float eps;
  const bf16* up;  // PRO_SILU_MUL: x <- bf16(bf16(silu(x)) * up)
  long up_stride;
  // epilogue
  int epilogue;
  bf16* out;  // [rows, N]
  long out_stride;
  const bf16* residual;  // EPI_RESIDUAL: out <- bf16(residual + bf16(y)); may alias out
  long res_stride;
  bf16* conv_state;  // EPI_CONV: columns < conv_dim go through the 4-tap conv + SiLU, [rows, conv_dim, 3]
  const bf16* conv_w;  // [conv_dim, 4]
  int conv_dim;
  int conv_state_settled;  // 1: no kernel still in flight on the stream writes conv_state (it may be read before the dependency wait)
  // scratch: split-K partial sums [rows, K/256, N] fp32 and one arrival counter per column tile
  float* partials;
  unsigned* counters;
  int math;
  int* status;      // device word the streaming kernel sets if one of its bounded waits gives up
  int force_tiled;  // 1: never take the streaming (TMA) path
  // Sum-of-squares hand-off between a GEMV that writes the residual stream and the RMSNorm-prologue GEMV
  // that reads it: the producer (cluster kernel) stores the sum of squares of each output tile, the
  // consumer adds ss_count of them instead of reducing the whole row again. Optional, either may be null.
  float* ss_out;
  const float* ss_in;
  int ss_count;
  TpPeer peer;  // EPI_PARTIAL_PEER only
  // Optional: up to two byte ranges (the words and the scales of the GEMV that follows in the step) that the
  // CTAs of this launch ask the L2 to fetch, a slice each, once their own loads are issued.
// up to three small arrays a LATER kernel of the stream reads first thing after its dependency wait (norm weights, rotary
  // frequencies): one CTA of this launch asks the L2 for them, so that the later kernel finds them there
  const void* touch_ptr[3];
  int touch_bytes[3];
    const void* pf_ptr[2];
  size_t pf_bytes[2];
  Trace trace;
  AttnMerge merge;  // PRO_ATTN_MERGE only
};

// Bytes of scratch the split-K path needs for a problem, and the number of counters.
size_t gemv_partials_bytes(int rows, int K, int N, int group);
size_t gemv_counter_count(int rows, int K, int N, int group);
int launch_gemv(const GemvParams& p, cudaStream_t stream);
// streaming (TMA ring, persistent CTAs, programmatic dependent launch) variant for one activation row
bool stream_path_ok(const GemvParams& p);
int stream_max_slots(int K, int N);
size_t stream_partials_bytes(int K, int N);
size_t stream_counter_count(int K, int N);
int stream_configure();
// one-cluster-per-tile variant for layer-sized matrices (same re-packed weight, no global scratch)
bool cluster_path_ok(const GemvParams& p);
int cluster_configure();
int launch_gemv_cluster(const GemvParams& p, int* status, cudaStream_t stream);
int launch_gemv_stream(const GemvParams& p, int* status, cudaStream_t stream);
// one activation row on the integer tensor-core instruction (mma.sync m16n8k32), on its own re-packed copy of the weight
bool mma_path_ok(const GemvParams& p);
int mma_configure();
int mma_tile_width(int N);
size_t mma_repack_bytes(int K, int N, int pair, int scale_bf16);
int launch_int4_repack_mma(const uint8_t* packed, const void* scale, int scale_bf16, int K, int N, int pair, void* out, cudaStream_t stream);
int launch_gemv_mma(const GemvParams& p, int* status, cudaStream_t stream);
// tensor-core (tcgen05) variant for 8..128 activation rows, on the re-packed weight
bool tc_path_ok(const GemvParams& p);
int tc_configure();
int launch_gemm_tc(const GemvParams& p, int* status, cudaStream_t stream);
// packed [K/2, N] bytes -> [K/8, N] words, word (kb, n) = the nibbles of column n, rows 8kb .. 8kb+7
int launch_int4_repack_k8(const uint8_t* packed, int K, int N, uint32_t* out, cudaStream_t stream);

// weight [N, K] (bf16 or fp32) -> packed [K/2, N] + scale [K/group, N] fp32, the reference's K-major int4 format
int launch_int4_quantise(const void* weight, int weight_is_bf16, int N, int K, int group, uint8_t* packed, float* scale,
                         cudaStream_t stream);
int launch_int4_unpack(const uint8_t* packed, int K, int N, int8_t* out, cudaStream_t stream);
int launch_int4_dequant(const uint8_t* packed, const void* scale, int scale_bf16, int K, int N, int group, bf16* out,
                        cudaStream_t stream);

struct DeltaNetParams {
  int batch;
  int num_k_heads, num_v_heads, dk, dv;  // dk == dv == 128 on the fast path
  // post-conv activations, one row per sequence: q [Hk*dk], k [Hk*dk], v [Hv*dv] (bf16)
  const bf16* q;
  const bf16* k;
  const bf16* v;
  const bf16* z;  // gate of the output norm, [Hv*dv]
  const bf16* b;  // [Hv] beta logits
  const bf16* a;  // [Hv] decay logits
  long row_stride;  // elements between sequences for q,k,v,z,b,a (they share one projection row)
  const float* a_log;    // [Hv]
  const float* dt_bias;  // [Hv]
  const float* norm_w;   // [dv]
  int norm_w_bf16;       // round norm_w * normed to bf16 (the weight is held in bf16 by the model)
  float eps;
  float* state;  // [batch, Hv, dk, dv] fp32, updated in place
  bf16* out;     // [batch, Hv*dv]
  long out_stride;
  const void* pf_ptr[2];  // as in GemvParams
  size_t pf_bytes[2];
  Trace trace;
};
int launch_deltanet_step(const DeltaNetParams& p, cudaStream_t stream);

struct DeltaRuleParams {  // the bare recurrence on pre-normalised q,k (fp32 in, fp32 out)
  int batch, heads, dk, dv;
  const float* state;
  const float* q;
  const float* k;
  const float* v;
  const float* g;
  const float* beta;
  float* out;
  float* state_out;
};
int launch_delta_rule_step(const DeltaRuleParams& p, cudaStream_t stream);

struct AttnParams {
  int batch, hq, hkv, d;  // d == 256 on the fast path
  const bf16* q;          // [batch, hq, d] (q_stride between sequences, qh_stride between heads)
  long q_stride, qh_stride;
  const bf16* kcache;  // [batch, hkv, max_seq, d]
  const bf16* vcache;
  long kv_batch_stride, kv_head_stride;  // elements; rows are d apart
  int key_len;                            // used when pos == nullptr
  const int* pos;                         // device scalar: key_len = *pos + 1
  float scale;
  int splits;
  float* part_acc;  // [batch, hq, splits, d]
  float* part_ml;   // [batch, hq, splits, 2]
  unsigned* counters;  // [batch * hkv]
  const bf16* gate;    // optional output-gate logits, one d-vector per query head
  long gate_stride, gateh_stride;  // elements between sequences / between heads
  int gate_swish;
  bf16* out;  // [batch, hq*d]
  long out_stride;
};
int launch_attn_decode(const AttnParams& p, cudaStream_t stream);
// tensor-core (mma.sync) variant for many sequences or long caches; launch_attn_decode picks it when it applies
bool attn_mma_ok(const AttnParams& p);
int launch_attn_decode_mma(const AttnParams& p, int* status, cudaStream_t stream);

struct AttnPrepParams {  // q/k RMSNorm + partial RoPE + KV-cache write for the new token
  int batch, hq, hkv, d, rotary_dim;
  const bf16* proj;  // [batch, hq*2*d (query|gate per head) + hkv*d (k) + hkv*d (v)]
  long proj_stride;
  const bf16* q_norm_w;
  const bf16* k_norm_w;
  float eps;
  const float* inv_freq;  // [rotary_dim/2]
  const int* pos;          // device scalar position
  bf16* q_out;             // [batch, hq, d]
  bf16* kcache;
  bf16* vcache;
  long kv_batch_stride, kv_head_stride;
  int attn_output_gate;
  int max_seq;  // rows per head in the cache; a position beyond it is not written
};
int launch_attn_prep(const AttnPrepParams& p, cudaStream_t stream);

struct AttnStepParams {  // prep + split-KV decode + merge + gate in one launch (head_dim 256)
  int batch, hq, hkv, d, rotary_dim;
  const bf16* proj;  // [batch, hq*(2d or d) + 2*hkv*d]: per head query(|gate), then keys, then values
  long proj_stride;
  const bf16* q_norm_w;
  const bf16* k_norm_w;
  float eps;
  const float* inv_freq;
  const int* pos;  // device scalar: tokens already cached; the new token goes to row *pos
  bf16* kcache;
  bf16* vcache;
  long kv_batch_stride, kv_head_stride;
  int max_seq;
  int attn_output_gate, gate_swish;
  float scale;
  int splits;        // power of two, grid.x
  int cluster_size;  // min(splits, 8)
  float* part_acc;   // [batch, hq, splits / cluster_size, d]
  float* part_ml;    // [batch, hq, splits / cluster_size, 2]
  unsigned* counters;  // [batch * hkv]
  bf16* out;  // [batch, hq*d]
  long out_stride;
  int* status;  // device word set if the bounded wait on the staging copies gives up
  // 1: with more than one cluster of slices per KV head, leave the per-cluster partial results (part_acc, part_ml) for the
  // consumer to merge (PRO_ATTN_MERGE of the output projection) instead of merging them here by the last cluster to arrive;
  // `out` is then not written and `counters` not used
  int defer_merge;
  const void* pf_ptr[2];  // as in GemvParams
  size_t pf_bytes[2];
  Trace trace;
};
bool attn_step_ok(int d, int hq, int hkv, int rotary_dim, int splits, int max_seq);
int attn_step_configure();
int launch_attn_step(const AttnStepParams& p, cudaStream_t stream);

int launch_rms_norm(const bf16* x, const bf16* w, float eps, int rows, int n, bf16* out, cudaStream_t s);
int launch_add_rms_norm(const bf16* x, const bf16* res, const bf16* w, float eps, int rows, int n, bf16* resid_out,
                        bf16* out, cudaStream_t s);
int launch_silu_mul(const bf16* gate, const bf16* up, long n, bf16* out, cudaStream_t s);
int launch_partial_rope(const bf16* x, const bf16* cos, const bf16* sin, int batch, int heads, int seq, int d, int rd,
                        bf16* out, cudaStream_t s);
int launch_causal_conv_step(const bf16* x, bf16* cache, const bf16* w, int batch, int channels, bf16* out,
                            cudaStream_t s);
// gate and up are rows of one buffer (in_stride apart), out is [rows, n] contiguous
int launch_silu_mul_rows(const bf16* gate, const bf16* up, long in_stride, int rows, int n, bf16* out, cudaStream_t s);
// conv + SiLU in place on the first `channels` entries of every row of x; cache [rows, channels, 3]
int launch_causal_conv_rows(bf16* x, long x_stride, bf16* cache, const bf16* w, int rows, int channels, cudaStream_t s);
// Row gather; when ss_out is given (batch 1) also stores the row's sum of squares in ss_out[0] and zeros ss_out[1..ss_count).
int launch_embed(const bf16* table, const int64_t* tokens, int batch, int hidden, bf16* out, float* ss_out, int ss_count,
                 cudaStream_t s);
// Column-tile width the cluster GEMV uses for an N-column matrix (the granularity of ss_out).
int cluster_tile_width(int N);
// out[b] = argmax; optionally hist[*pos, b] = argmax. scratch_val/idx: [batch, 64]; counter: [batch], zeroed once.
int launch_argmax(const bf16* logits, int batch, int n, long stride, int64_t* out, int64_t* hist, const int* pos,
                  float* scratch_val, int* scratch_idx, unsigned* counter, cudaStream_t s);
// Opt the kernels with large dynamic shared memory in; call once before stream capture.
int configure_kernels();
int launch_advance(int* pos, int by, cudaStream_t s);
// h <- bf16(h + bf16(sum)) over n elements: the residual add after an all-reduce of fp32 partial sums
int launch_add_partial(bf16* h, const float* sum, long n, cudaStream_t s);
// The receiving side of the peer exchange: wait (bounded) for the tp words of every element to carry the epoch,
// add them in rank order, round to bf16 and add to the residual stream. slots: this rank's own buffer.
int launch_tp_reduce(bf16* h, const unsigned long long* slots, int tp_size, long n, long word_off, const unsigned* epoch_ctr,
                     int epoch_off, int* status, const Trace& trace, cudaStream_t s);
// Greedy pick across vocabulary shards by peer exchange of (best logit, global index); tokens holds the local index on entry.
int launch_tp_pick(const bf16* logits, int vocab_local, int batch, int tp_rank, const TpPeer& peer, const unsigned long long* my_slots,
                   int64_t* tokens, int64_t* hist, const int* pos, int* status, cudaStream_t s);
int launch_bump(unsigned* counter, cudaStream_t s);

}  // namespace dfb

