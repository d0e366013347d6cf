// C entry points of libdfb200: argument checks, descriptor -> kernel-parameter translation, errors.
#include <stdarg.h>
#include <stdio.h>

#include "../../include/dfb200.h"
#include "common.cuh"
#include "kernels.h"

namespace dfb {

static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

int check_launch(const char* what) {
  const cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return DFB_OK;
  set_error("%s: %s", what, cudaGetErrorString(e));
  return DFB_ERR_CUDA;
}

static int bad(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return DFB_ERR_ARG;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int check_int4_shape(int K, int N, int group) {
  if (K <= 0 || K % 2) return bad("int4 packing needs an even, positive K, got %d", K);
  if (N <= 0) return bad("N must be positive, got %d", N);
  if (group <= 0 || (K / 2) % group) return bad("group %d must divide K/2 = %d", group, K / 2);
  return DFB_OK;
}

}  // namespace dfb

using namespace dfb;

extern "C" {

const char* dfb_last_error(void) { return g_error; }
int dfb_abi_version(void) { return 1; }

int dfb_int4_group_size(int K) {
  if (K <= 0 || K % 2) return 0;
  const int group = K % 256 == 0 ? 128 : K / 2;
  return (group & (group - 1)) ? 0 : group;
}

int dfb_int4_quantise_k_major(const void* weight, int weight_is_bf16, int N, int K, uint8_t* packed, float* scale, void* stream) {
  if (!weight || !packed || !scale) return bad("dfb_int4_quantise_k_major: null pointer");
  if (N <= 0 || K <= 0) return bad("dfb_int4_quantise_k_major: bad shape N=%d K=%d", N, K);
  const int group = dfb_int4_group_size(K);
  if (group == 0) return bad("dfb_int4_quantise_k_major: K=%d is odd, or half of it is not a power of two where K is not a multiple of 256", K);
  return launch_int4_quantise(weight, weight_is_bf16, N, K, group, packed, scale, (cudaStream_t)stream);
}

int dfb_int4_unpack(const uint8_t* packed, int K, int N, int8_t* out, void* stream) {
  if (!packed || !out) return bad("dfb_int4_unpack: null pointer");
  if (K <= 0 || K % 2 || N <= 0) return bad("dfb_int4_unpack: bad shape K=%d N=%d", K, N);
  return launch_int4_unpack(packed, K, N, out, (cudaStream_t)stream);
}

int dfb_int4_dequant(const uint8_t* packed, const void* scale, int scale_is_bf16, int K, int N, int group,
                     void* out_bf16, void* stream) {
  if (!packed || !scale || !out_bf16) return bad("dfb_int4_dequant: null pointer");
  if (int rc = check_int4_shape(K, N, group)) return rc;
  return launch_int4_dequant(packed, scale, scale_is_bf16, K, N, group, (bf16*)out_bf16, (cudaStream_t)stream);
}

int dfb_int4_repack_k8(const uint8_t* packed, int K, int N, void* out, void* stream) {
  if (!packed || !out) return bad("dfb_int4_repack_k8: null pointer");
  if (K <= 0 || K % 8 || N <= 0) return bad("dfb_int4_repack_k8: K must be a positive multiple of 8, got K=%d N=%d", K, N);
  return launch_int4_repack_k8(packed, K, N, (uint32_t*)out, (cudaStream_t)stream);
}

size_t dfb_int4_repack_mma_bytes(int K, int N, int pair, int scale_is_bf16) {
  if (K <= 0 || K % 128 || N <= 0 || (pair && N % 2)) return 0;
  return mma_repack_bytes(K, N, pair, scale_is_bf16);
}

int dfb_int4_repack_mma(const uint8_t* packed, const void* scale, int scale_is_bf16, int K, int N, int pair, void* out, void* stream) {
  if (!packed || !scale || !out) return bad("dfb_int4_repack_mma: null pointer");
  if (K <= 0 || K % 128 || N <= 0 || (pair && N % 2))
    return bad("dfb_int4_repack_mma: K must be a positive multiple of 128 and N positive (even for a gate|up pair), got K=%d N=%d", K, N);
  return launch_int4_repack_mma(packed, scale, scale_is_bf16, K, N, pair, out, (cudaStream_t)stream);
}

size_t dfb_int4_gemv_scratch_bytes(int rows, int K, int N, int group) {
  if (rows <= 0 || K <= 0 || N <= 0) return 0;
  const size_t body = align_up(gemv_partials_bytes(rows, K, N, group), 256) + align_up(gemv_counter_count(rows, K, N, group) * 4, 256);
  return body ? body + 256 : 0;  // the last 256 bytes start with the status word
}

int dfb_int4_gemv(const dfb_gemv_desc* d, void* stream) {
  if (!d) return bad("dfb_int4_gemv: null descriptor");
  if (d->rows < 0) return bad("dfb_int4_gemv: negative row count");
  if (d->rows == 0) return DFB_OK;
  if (!d->x || !d->packed || !d->scale || !d->out) return bad("dfb_int4_gemv: null tensor pointer");
  if (int rc = check_int4_shape(d->K, d->N, d->group)) return rc;
  if (d->prologue == DFB_PROLOGUE_RMSNORM && !d->norm_w) return bad("dfb_int4_gemv: RMSNorm prologue without a weight");
  if (d->prologue == DFB_PROLOGUE_SILU_MUL && !d->up) return bad("dfb_int4_gemv: SiLU-mul prologue without `up`");
  if (d->prologue < 0 || d->prologue > 2) return bad("dfb_int4_gemv: unknown prologue %d", d->prologue);
  if (d->epilogue == DFB_EPILOGUE_RESIDUAL && !d->residual) return bad("dfb_int4_gemv: residual epilogue without a residual");
  if (d->epilogue == DFB_EPILOGUE_CONV && (!d->conv_state || !d->conv_w || d->conv_dim < 0 || d->conv_dim > d->N))
    return bad("dfb_int4_gemv: conv epilogue needs conv_state, conv_w and 0 <= conv_dim <= N");
  if (d->epilogue < 0 || d->epilogue > 2) return bad("dfb_int4_gemv: unknown epilogue %d", d->epilogue);
  if (d->math < 0 || d->math > 2) return bad("dfb_int4_gemv: unknown math mode %d", d->math);
  const size_t need = dfb_int4_gemv_scratch_bytes(d->rows, d->K, d->N, d->group);
  if (need && (!d->scratch || d->scratch_bytes < need))
    return bad("dfb_int4_gemv: scratch of %zu bytes required, got %zu", need, d->scratch ? d->scratch_bytes : (size_t)0);
  GemvParams p = {};
  p.x = (const bf16*)d->x;
  p.x_stride = d->x_stride;
  p.rows = d->rows;
  p.packed = d->packed;
  p.scale = d->scale;
  p.scale_bf16 = d->scale_is_bf16;
  p.K = d->K;
  p.N = d->N;
  p.group = d->group;
  p.prologue = d->prologue;
  p.norm_w = (const bf16*)d->norm_w;
  p.eps = d->eps;
  p.up = (const bf16*)d->up;
  p.up_stride = d->up_stride;
  p.epilogue = d->epilogue;
  p.out = (bf16*)d->out;
  p.out_stride = d->out_stride;
  p.residual = (const bf16*)d->residual;
  p.res_stride = d->residual_stride;
  p.conv_state = (bf16*)d->conv_state;
  p.conv_w = (const bf16*)d->conv_w;
  p.conv_dim = d->conv_dim;
  p.math = d->math;
  p.packed_mma = (const unsigned char*)d->packed_mma;
  if (need) {
    p.partials = (float*)d->scratch;
    p.counters = (unsigned*)((char*)d->scratch + align_up(gemv_partials_bytes(d->rows, d->K, d->N, d->group), 256));
    p.status = (int*)((char*)d->scratch + need - 256);
  }
  p.force_tiled = d->force_tiled;
  p.packed_k8 = (const uint32_t*)d->packed_k8;
  return launch_gemv(p, (cudaStream_t)stream);
}

int dfb_rms_norm(const void* x, const void* weight, float eps, int rows, int n, void* out, void* stream) {
  if (!x || !weight || !out) return bad("dfb_rms_norm: null pointer");
  if (rows < 0 || n <= 0) return bad("dfb_rms_norm: bad shape rows=%d n=%d", rows, n);
  return launch_rms_norm((const bf16*)x, (const bf16*)weight, eps, rows, n, (bf16*)out, (cudaStream_t)stream);
}

int dfb_add_rms_norm(const void* x, const void* residual, const void* weight, float eps, int rows, int n,
                     void* resid_out, void* out, void* stream) {
  if (!x || !residual || !weight || !resid_out || !out) return bad("dfb_add_rms_norm: null pointer");
  if (rows < 0 || n <= 0) return bad("dfb_add_rms_norm: bad shape rows=%d n=%d", rows, n);
  return launch_add_rms_norm((const bf16*)x, (const bf16*)residual, (const bf16*)weight, eps, rows, n, (bf16*)resid_out,
                             (bf16*)out, (cudaStream_t)stream);
}

int dfb_silu_mul(const void* gate, const void* up, int64_t n, void* out, void* stream) {
  if (!gate || !up || !out) return bad("dfb_silu_mul: null pointer");
  if (n < 0) return bad("dfb_silu_mul: negative length");
  return launch_silu_mul((const bf16*)gate, (const bf16*)up, (long)n, (bf16*)out, (cudaStream_t)stream);
}

int dfb_partial_rope(const void* x, const void* cos, const void* sin, int batch, int heads, int seq, int d,
                     int rotary_dim, void* out, void* stream) {
  if (!x || !cos || !sin || !out) return bad("dfb_partial_rope: null pointer");
  if (rotary_dim % 2) return bad("rotary_dim must be even to rotate in halves, got %d", rotary_dim);
  if (rotary_dim > d) return bad("rotary_dim %d exceeds head_dim %d", rotary_dim, d);
  return launch_partial_rope((const bf16*)x, (const bf16*)cos, (const bf16*)sin, batch, heads, seq, d, rotary_dim,
                             (bf16*)out, (cudaStream_t)stream);
}

int dfb_causal_conv_step(const void* x, void* conv_cache, const void* weight, int batch, int channels, void* out,
                         void* stream) {
  if (!x || !conv_cache || !weight || !out) return bad("dfb_causal_conv_step: null pointer");
  return launch_causal_conv_step((const bf16*)x, (bf16*)conv_cache, (const bf16*)weight, batch, channels, (bf16*)out,
                                 (cudaStream_t)stream);
}

int dfb_delta_rule_step(const float* state, const float* q, const float* k, const float* v, const float* g,
                        const float* beta, int batch, int heads, int dk, int dv, float* out, float* state_out,
                        void* stream) {
  if (!state || !q || !k || !v || !g || !beta || !out || !state_out) return bad("dfb_delta_rule_step: null pointer");
  DeltaRuleParams p = {batch, heads, dk, dv, state, q, k, v, g, beta, out, state_out};
  return launch_delta_rule_step(p, (cudaStream_t)stream);
}

int dfb_deltanet_step(const dfb_deltanet_desc* d, void* stream) {
  if (!d) return bad("dfb_deltanet_step: null descriptor");
  if (!d->q || !d->k || !d->v || !d->z || !d->b || !d->a || !d->a_log || !d->dt_bias || !d->norm_w || !d->state || !d->out)
    return bad("dfb_deltanet_step: null tensor pointer");
  DeltaNetParams p = {};
  p.batch = d->batch;
  p.num_k_heads = d->num_k_heads;
  p.num_v_heads = d->num_v_heads;
  p.dk = d->dk;
  p.dv = d->dv;
  p.q = (const bf16*)d->q;
  p.k = (const bf16*)d->k;
  p.v = (const bf16*)d->v;
  p.z = (const bf16*)d->z;
  p.b = (const bf16*)d->b;
  p.a = (const bf16*)d->a;
  p.row_stride = d->row_stride;
  p.a_log = d->a_log;
  p.dt_bias = d->dt_bias;
  p.norm_w = d->norm_w;
  p.norm_w_bf16 = d->norm_w_is_bf16;
  p.eps = d->eps;
  p.state = d->state;
  p.out = (bf16*)d->out;
  p.out_stride = d->out_stride;
  return launch_deltanet_step(p, (cudaStream_t)stream);
}

size_t dfb_attn_scratch_bytes(int batch, int hq, int hkv, int d, int splits) {
  if (splits <= 1) return 0;
  return align_up((size_t)batch * hq * splits * d * 4, 256) + align_up((size_t)batch * hq * splits * 2 * 4, 256) +
         align_up((size_t)batch * hkv * 4, 256);
}

int dfb_attn_decode(const dfb_attn_desc* d, void* stream) {
  if (!d) return bad("dfb_attn_decode: null descriptor");
  if (!d->q || !d->kcache || !d->vcache || !d->out) return bad("dfb_attn_decode: null tensor pointer");
  if (d->hkv <= 0 || d->hq % d->hkv) return bad("%d query heads do not divide into %d KV heads", d->hq, d->hkv);
  if (!d->pos && d->key_len < 1) return bad("cannot attend over an empty KV cache");
  if (d->splits < 1) return bad("splits must be at least 1, got %d", d->splits);
  const size_t need = dfb_attn_scratch_bytes(d->batch, d->hq, d->hkv, d->d, d->splits);
  if (need && (!d->scratch || d->scratch_bytes < need))
    return bad("dfb_attn_decode: scratch of %zu bytes required for %d splits", need, d->splits);
  AttnParams p = {};
  p.batch = d->batch;
  p.hq = d->hq;
  p.hkv = d->hkv;
  p.d = d->d;
  p.q = (const bf16*)d->q;
  p.q_stride = d->q_stride;
  p.qh_stride = d->qh_stride;
  p.kcache = (const bf16*)d->kcache;
  p.vcache = (const bf16*)d->vcache;
  p.kv_batch_stride = d->kv_batch_stride;
  p.kv_head_stride = d->kv_head_stride;
  p.key_len = d->key_len;
  p.pos = d->pos;
  p.scale = d->scale;
  p.splits = d->splits;
  if (need) {
    char* s = (char*)d->scratch;
    p.part_acc = (float*)s;
    s += align_up((size_t)d->batch * d->hq * d->splits * d->d * 4, 256);
    p.part_ml = (float*)s;
    s += align_up((size_t)d->batch * d->hq * d->splits * 2 * 4, 256);
    p.counters = (unsigned*)s;
  }
  p.gate = (const bf16*)d->gate;
  p.gate_stride = d->gate_stride;
  p.gateh_stride = d->gateh_stride;
  p.gate_swish = d->gate_is_swish;
  p.out = (bf16*)d->out;
  p.out_stride = d->out_stride;
  return launch_attn_decode(p, (cudaStream_t)stream);
}

int dfb_attn_step(const dfb_attn_step_desc* d, void* stream) {
  if (!d) return bad("dfb_attn_step: null descriptor");
  if (!d->proj || !d->q_norm_w || !d->k_norm_w || !d->inv_freq || !d->pos || !d->kcache || !d->vcache || !d->out)
    return bad("dfb_attn_step: null tensor pointer");
  const int cs = d->cluster_size > 0 ? d->cluster_size : (d->splits < 4 ? d->splits : 4);
  if (cs < 1 || cs > 8 || d->splits % cs) return bad("dfb_attn_step: cluster size %d does not divide %d slices", cs, d->splits);
  if (!attn_step_ok(d->d, d->hq, d->hkv, d->rotary_dim, d->splits, d->max_seq))
    return bad("dfb_attn_step: unsupported shape (d=%d, hq=%d, hkv=%d, rotary=%d, splits=%d, max_seq=%d)", d->d, d->hq, d->hkv,
               d->rotary_dim, d->splits, d->max_seq);
  const size_t need = dfb_attn_scratch_bytes(d->batch, d->hq, d->hkv, d->d, d->splits);
  if (need && (!d->scratch || d->scratch_bytes < need)) return bad("dfb_attn_step: scratch of %zu bytes required", need);
  AttnStepParams p = {};
  p.batch = d->batch;
  p.hq = d->hq;
  p.hkv = d->hkv;
  p.d = d->d;
  p.rotary_dim = d->rotary_dim;
  p.proj = (const bf16*)d->proj;
  p.proj_stride = d->proj_stride;
  p.q_norm_w = (const bf16*)d->q_norm_w;
  p.k_norm_w = (const bf16*)d->k_norm_w;
  p.eps = d->eps;
  p.inv_freq = d->inv_freq;
  p.pos = d->pos;
  p.kcache = (bf16*)d->kcache;
  p.vcache = (bf16*)d->vcache;
  p.kv_batch_stride = d->kv_batch_stride;
  p.kv_head_stride = d->kv_head_stride;
  p.max_seq = d->max_seq;
  p.attn_output_gate = d->attn_output_gate;
  p.gate_swish = d->gate_is_swish;
  p.scale = d->scale;
  p.splits = d->splits;
  p.cluster_size = cs;
  if (need) {
    char* s = (char*)d->scratch;
    p.part_acc = (float*)s;
    s += align_up((size_t)d->batch * d->hq * d->splits * d->d * 4, 256);
    p.part_ml = (float*)s;
    s += align_up((size_t)d->batch * d->hq * d->splits * 2 * 4, 256);
    p.counters = (unsigned*)s;
  }
  p.out = (bf16*)d->out;
  p.out_stride = d->out_stride;
  p.status = d->status;
  static OncePerDevice once;
  const int configured = once.run(attn_step_configure);
  if (configured) return configured;
  return launch_attn_step(p, (cudaStream_t)stream);
}

int dfb_attn_prep(const dfb_attn_prep_desc* d, void* stream) {
  if (!d) return bad("dfb_attn_prep: null descriptor");
  if (!d->proj || !d->q_norm_w || !d->k_norm_w || !d->inv_freq || !d->pos || !d->q_out || !d->kcache || !d->vcache)
    return bad("dfb_attn_prep: null tensor pointer");
  AttnPrepParams p = {};
  p.batch = d->batch;
  p.hq = d->hq;
  p.hkv = d->hkv;
  p.d = d->d;
  p.rotary_dim = d->rotary_dim;
  p.proj = (const bf16*)d->proj;
  p.proj_stride = d->proj_stride;
  p.q_norm_w = (const bf16*)d->q_norm_w;
  p.k_norm_w = (const bf16*)d->k_norm_w;
  p.eps = d->eps;
  p.inv_freq = d->inv_freq;
  p.pos = d->pos;
  p.q_out = (bf16*)d->q_out;
  p.kcache = (bf16*)d->kcache;
  p.vcache = (bf16*)d->vcache;
  p.kv_batch_stride = d->kv_batch_stride;
  p.kv_head_stride = d->kv_head_stride;
  p.attn_output_gate = d->attn_output_gate;
  p.max_seq = d->max_seq;
  return launch_attn_prep(p, (cudaStream_t)stream);
}

}  // extern "C"
