// Gated DeltaNet decode step, sm_100a.
//
// deltanet_fused_kernel does, for one token and one value head per cluster, everything between the
// causal conv and out_proj of the reference's GatedDeltaNet.forward (src/deltaforge/reference.py:
// 518-549): L2-norm of q and k and the 1/sqrt(dk) query scale (:403-404, :435-437), beta =
// sigmoid(b) and g = -exp(A_log) * softplus(a + dt_bias) (:528-532), the recurrence
//   S <- S * exp(g);  r = S^T k;  delta = (v - r) * beta;  S <- S + k delta^T;  o = S^T q   (:450-458)
// and the gated RMSNorm with the z gate (:115-121). It replaces the reference's Triton step
// (src/deltaforge/kernels/gated_delta_step.py:50-106) and the elementwise ops around it.
//
// The fp32 state [Hv, dk, dv] is read once and written once, in place. A cluster of dv/32 CTAs
// owns one value head; each CTA holds a dk x 32 slab of the state in registers (lane = value
// column, each warp a band of key rows), so both reductions over dk and the rank-1 update happen
// without touching memory again. The only thing a head needs across its CTAs is the sum of squares
// for the output norm, which the CTAs exchange through distributed shared memory.
//
// Bytes per launch: 2 * Hv*dk*dv*4 (state read + write) + the q/k/v/z/b/a row and the output row.
#include <cooperative_groups.h>

#include "common.cuh"
#include "kernels.h"

namespace cg = cooperative_groups;

namespace dfb {

namespace {

constexpr int VB = 32;       // value columns per CTA (one per lane)
constexpr int DN_WARPS = 8;  // key rows are split over 8 warps
constexpr int MAX_DK = 128;
constexpr int RPT = MAX_DK / DN_WARPS;  // state rows per thread

struct CoreOut {
  float o;  // read-out for this thread's value column (valid in every warp)
};

// The recurrence on a dk x 32 slab. `s` holds rows warp*RPT + i of column `col`; qn/kn are the
// normalised query/key in shared memory; red is [2][DN_WARPS][VB] scratch.
__device__ __forceinline__ float delta_core(float (&s)[RPT], int dk, bool col_ok, const float* qn, const float* kn,
                                            float vval, float decay, float beta, float* red) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float r = 0.f;
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int k = warp * RPT + i;
    s[i] = __fmul_rn(s[i], decay);
    if (k < dk) r = fmaf(s[i], kn[k], r);
  }
  red[warp * VB + lane] = r;
  __syncthreads();
  r = 0.f;
#pragma unroll
  for (int w = 0; w < DN_WARPS; ++w) r += red[w * VB + lane];
  const float delta = __fmul_rn(__fsub_rn(vval, r), beta);
  float o = 0.f;
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int k = warp * RPT + i;
    if (k < dk) {
      s[i] = __fadd_rn(s[i], __fmul_rn(kn[k], delta));
      o = fmaf(s[i], qn[k], o);
    }
  }
  red[(DN_WARPS + warp) * VB + lane] = o;
  __syncthreads();
  o = 0.f;
#pragma unroll
  for (int w = 0; w < DN_WARPS; ++w) o += red[(DN_WARPS + w) * VB + lane];
  (void)col_ok;
  return o;
}

__global__ void __launch_bounds__(DN_WARPS * 32) deltanet_fused_kernel(const DeltaNetParams p) {
  __shared__ float qn[MAX_DK], kn[MAX_DK];
  __shared__ float red[2 * DN_WARPS * VB];
  __shared__ float wred[DN_WARPS];
  __shared__ float gates[2];
  __shared__ float cluster_ss[8];  // sums of squares of the head's column blocks, one slot per cluster rank

  cg::cluster_group cluster = cg::this_cluster();
  const int nvb = (p.dv + VB - 1) / VB;  // == cluster size
  const int hv = blockIdx.x / nvb, vb = blockIdx.x % nvb, b = blockIdx.y;
  const int hk = hv / (p.num_v_heads / p.num_k_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
  const int col = vb * VB + lane;
  const bool col_ok = col < p.dv;
  const int dk = p.dk, dv = p.dv;

  // Under programmatic dependent launch this kernel may start while the projection GEMV before it is
  // still running: let the next kernel start its own prefetch, and touch nothing the GEMV writes
  // until griddepcontrol.wait below. The recurrent state is only ever written by this kernel.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int cta = blockIdx.y * gridDim.x + blockIdx.x, nctas = gridDim.x * gridDim.y;
  if (t == 0) trace_mark(p.trace, cta, 0);
  // 1. The state slab goes in flight first; nothing below depends on it until delta_core.
  float* S = p.state + ((long)(b * p.num_v_heads + hv) * dk) * dv;
  float s[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int k = warp * RPT + i;
    s[i] = (col_ok && k < dk) ? __ldcs(S + (long)k * dv + col) : 0.f;
  }
  if (t == 32) {  // a slice of the weights a later GEMV of the step reads, into the L2
#pragma unroll
    for (int i = 0; i < 2; ++i)
      if (p.pf_ptr[i] != nullptr)
        l2_prefetch_range(p.pf_ptr[i], p.pf_bytes[i] * (size_t)cta / nctas, p.pf_bytes[i] * (size_t)(cta + 1) / nctas);
  }

  // constants of the layer (never written by a kernel): in flight before the wait
  const float nw = col_ok ? p.norm_w[col] : 0.f;
  const float a_log = p.a_log[hv], dt_bias = p.dt_bias[hv];

  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (t == 0) trace_mark(p.trace, cta, 1);
  // 2. Everything the projection before this kernel wrote goes in flight together (one round trip to the L2, not
  // three): this thread's q or k element, its value and gate, and the two gate logits of the head.
  const long row = (long)b * p.row_stride;
  const bool is_k = t >= MAX_DK;
  const int j = is_k ? t - MAX_DK : t;
  float x = 0.f;
  if (j < dk) x = bf2f((is_k ? p.k : p.q)[row + (long)hk * dk + j]);
  const float vval = col_ok ? bf2f(p.v[row + (long)hv * dv + col]) : 0.f;
  const float zval = col_ok ? bf2f(p.z[row + (long)hv * dv + col]) : 0.f;
  const float b_logit = bf2f(p.b[row + hv]), a_logit = bf2f(p.a[row + hv]);
  // q, k of the key head: fp32, L2-normalised, query scaled by 1/sqrt(dk).
  {
    const float ss = warp_sum(x * x);
    if (lane == 0) wred[warp] = ss;
    if (t == DN_WARPS * 32 - 1) {  // the gates, by a thread of the last warp while the sums of squares are gathered
      const float beta = round_bf16(sigmoid_f(b_logit));
      const float g = __fmul_rn(-expf(a_log), softplus_f(__fadd_rn(a_logit, dt_bias)));
      gates[0] = beta;
      gates[1] = expf(g);
    }
    __syncthreads();
    float tot = 0.f;
    const int w0 = is_k ? DN_WARPS / 2 : 0;
#pragma unroll
    for (int w = 0; w < DN_WARPS / 2; ++w) tot += wred[w0 + w];
    float xn = __fmul_rn(x, rsqrt_2step(__fadd_rn(tot, 1e-6f)));
    if (!is_k) xn = __fdiv_rn(xn, sqrtf((float)dk));
    if (j < dk) (is_k ? kn : qn)[j] = xn;
  }
  __syncthreads();
  if (t == 0) trace_mark(p.trace, cta, 2);

  // 3. Recurrence; the updated slab goes straight back.
  const float o = delta_core(s, dk, col_ok, qn, kn, vval, gates[1], gates[0], red);
  if (t == 0) trace_mark(p.trace, cta, 3);
  // (the updated slab is stored after the cluster exchange below: the barrier's release would otherwise wait for
  // these 2 MB of stores to be acknowledged before the head's sum of squares could be read)

  // 4. Gated RMSNorm over the head's dv outputs: the CTAs of the cluster swap their sums of squares.
  const float ob = col_ok ? round_bf16(o) : 0.f;
  // Each CTA pushes its sum into slot [its rank] of every CTA of the cluster, so that after one
  // cluster barrier everybody reads only its own shared memory and may leave at once.
  if (warp == 0) {
    const float ss = warp_sum(ob * ob);
    if (lane < nvb) *cluster.map_shared_rank(&cluster_ss[vb], lane) = ss;
  }
  const float sz = silu_f(zval);  // needs nothing from the other CTAs: evaluated while their sums arrive
  cluster.sync();
  if (t == 0) trace_mark(p.trace, cta, 5);
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int k = warp * RPT + i;
    if (col_ok && k < dk) __stcs(S + (long)k * dv + col, s[i]);
  }
  float tot = 0.f;
  for (int rk = 0; rk < nvb; ++rk) tot += cluster_ss[rk];
  if (warp == 0 && col_ok) {
    const float rstd = rsqrt_2step(__fadd_rn(__fdiv_rn(tot, (float)dv), p.eps));
    const float nrm = round_bf16(__fmul_rn(ob, rstd));
    float y = __fmul_rn(nw, nrm);
    if (p.norm_w_bf16) y = round_bf16(y);
    y = __fmul_rn(y, sz);
    p.out[(long)b * p.out_stride + (long)hv * dv + col] = f2bf(y);
  }
  if (t == 0) trace_mark(p.trace, cta, 6);
}

// Many sequences: one CTA owns a whole value head (all dv <= 128 columns, 64 state values per thread), so the
// head's sum of squares stays inside the CTA and the grid needs no clusters: with 32 sequences the clustered
// kernel above launches 1024 clusters of four small CTAs per layer and spends most of its time scheduling them.
constexpr int HB_COLS = 4;  // column groups of 32 per thread: dv <= 128
__global__ void __launch_bounds__(DN_WARPS * 32, 2) deltanet_head_kernel(const DeltaNetParams p) {
  __shared__ float qn[MAX_DK], kn[MAX_DK];
  __shared__ float red[2 * DN_WARPS * HB_COLS * VB];
  __shared__ float wred[DN_WARPS];
  __shared__ float gates[2];
  const int hv = blockIdx.x, b = blockIdx.y;
  const int hk = hv / (p.num_v_heads / p.num_k_heads);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
  const int dk = p.dk, dv = p.dv;
  pdl_launch_dependents();
  // the state of the head goes in flight first; nothing below depends on it until the recurrence
  float* S = p.state + ((long)(b * p.num_v_heads + hv) * dk) * dv;
  float s[HB_COLS][RPT];
#pragma unroll
  for (int c = 0; c < HB_COLS; ++c)
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int k = warp * RPT + i, col = c * VB + lane;
      s[c][i] = (col < dv && k < dk) ? __ldcs(S + (long)k * dv + col) : 0.f;
    }
  pdl_wait();
  const long row = (long)b * p.row_stride;
  {
    const bool is_k = t >= MAX_DK;
    const int j = is_k ? t - MAX_DK : t;
    float x = 0.f;
    if (j < dk) x = bf2f((is_k ? p.k : p.q)[row + (long)hk * dk + j]);
    const float ss = warp_sum(x * x);
    if (lane == 0) wred[warp] = ss;
    __syncthreads();
    float tot = 0.f;
    const int w0 = is_k ? DN_WARPS / 2 : 0;
#pragma unroll
    for (int w = 0; w < DN_WARPS / 2; ++w) tot += wred[w0 + w];
    float xn = __fmul_rn(x, rsqrt_2step(__fadd_rn(tot, 1e-6f)));
    if (!is_k) xn = __fdiv_rn(xn, sqrtf((float)dk));
    if (j < dk) (is_k ? kn : qn)[j] = xn;
    if (t == 0) {
      const float beta = round_bf16(sigmoid_f(bf2f(p.b[row + hv])));
      const float g = __fmul_rn(-expf(p.a_log[hv]), softplus_f(__fadd_rn(bf2f(p.a[row + hv]), p.dt_bias[hv])));
      gates[0] = beta;
      gates[1] = expf(g);
    }
  }
  float vval[HB_COLS], zval[HB_COLS];
#pragma unroll
  for (int c = 0; c < HB_COLS; ++c) {
    const int col = c * VB + lane;
    vval[c] = col < dv ? bf2f(p.v[row + (long)hv * dv + col]) : 0.f;
    zval[c] = col < dv ? bf2f(p.z[row + (long)hv * dv + col]) : 0.f;
  }
  __syncthreads();
  const float decay = gates[1], beta = gates[0];
  // r = S^T k on the decayed state, all four column groups in one pass and one barrier
#pragma unroll
  for (int c = 0; c < HB_COLS; ++c) {
    float r = 0.f;
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int k = warp * RPT + i;
      s[c][i] = __fmul_rn(s[c][i], decay);
      if (k < dk) r = fmaf(s[c][i], kn[k], r);
    }
    red[(warp * HB_COLS + c) * VB + lane] = r;
  }
  __syncthreads();
  float o[HB_COLS];
#pragma unroll
  for (int c = 0; c < HB_COLS; ++c) {
    float r = 0.f;
#pragma unroll
    for (int w = 0; w < DN_WARPS; ++w) r += red[(w * HB_COLS + c) * VB + lane];
    const float delta = __fmul_rn(__fsub_rn(vval[c], r), beta);
    float oc = 0.f;
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int k = warp * RPT + i;
      if (k < dk) {
        s[c][i] = __fadd_rn(s[c][i], __fmul_rn(kn[k], delta));
        oc = fmaf(s[c][i], qn[k], oc);
      }
    }
    red[((DN_WARPS + warp) * HB_COLS + c) * VB + lane] = oc;
  }
  __syncthreads();
  // the updated state goes straight back
#pragma unroll
  for (int c = 0; c < HB_COLS; ++c)
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
      const int k = warp * RPT + i, col = c * VB + lane;
      if (col < dv && k < dk) __stcs(S + (long)k * dv + col, s[c][i]);
    }
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < HB_COLS; ++c) {
    float oc = 0.f;
#pragma unroll
    for (int w = 0; w < DN_WARPS; ++w) oc += red[((DN_WARPS + w) * HB_COLS + c) * VB + lane];
    o[c] = (c * VB + lane) < dv ? round_bf16(oc) : 0.f;
    ss = fmaf(o[c], o[c], ss);
  }
  if (warp != 0) return;
  // gated RMSNorm over the head's dv outputs (src/deltaforge/reference.py:115-121): every warp holds all of them
  const float tot = warp_sum(ss);
  const float rstd = rsqrt_2step(__fadd_rn(__fdiv_rn(tot, (float)dv), p.eps));
#pragma unroll
  for (int c = 0; c < HB_COLS; ++c) {
    const int col = c * VB + lane;
    if (col >= dv) continue;
    const float nrm = round_bf16(__fmul_rn(o[c], rstd));
    float y = __fmul_rn(p.norm_w[col], nrm);
    if (p.norm_w_bf16) y = round_bf16(y);
    y = __fmul_rn(y, silu_f(zval[c]));
    p.out[(long)b * p.out_stride + (long)hv * dv + col] = f2bf(y);
  }
}

// The bare recurrence with the reference op's contract (src/deltaforge/kernels/gated_delta_step.py:
// 109-177): q, k already normalised, everything fp32, new state written to a separate tensor.
__global__ void __launch_bounds__(DN_WARPS * 32) delta_rule_kernel(const DeltaRuleParams p) {
  __shared__ float qn[MAX_DK], kn[MAX_DK];
  __shared__ float red[2 * DN_WARPS * VB];
  const int nvb = (p.dv + VB - 1) / VB;
  const int h = blockIdx.x / nvb, vb = blockIdx.x % nvb, b = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
  const int col = vb * VB + lane;
  const bool col_ok = col < p.dv;
  const long bh = (long)b * p.heads + h;
  const float* S = p.state + bh * p.dk * p.dv;
  float s[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int k = warp * RPT + i;
    s[i] = (col_ok && k < p.dk) ? S[(long)k * p.dv + col] : 0.f;
  }
  if (t < p.dk) qn[t] = p.q[bh * p.dk + t];
  if (t >= MAX_DK && t - MAX_DK < p.dk) kn[t - MAX_DK] = p.k[bh * p.dk + t - MAX_DK];
  __syncthreads();
  const float vval = col_ok ? p.v[bh * p.dv + col] : 0.f;
  const float o = delta_core(s, p.dk, col_ok, qn, kn, vval, expf(p.g[bh]), p.beta[bh], red);
  float* So = p.state_out + bh * p.dk * p.dv;
#pragma unroll
  for (int i = 0; i < RPT; ++i) {
    const int k = warp * RPT + i;
    if (col_ok && k < p.dk) So[(long)k * p.dv + col] = s[i];
  }
  if (warp == 0 && col_ok) p.out[bh * p.dv + col] = o;
}

}  // namespace

int deltanet_configure() {
  cudaError_t e = prefer_max_shared(deltanet_fused_kernel);
  if (e == cudaSuccess) e = prefer_max_shared(deltanet_head_kernel);
  if (e == cudaSuccess) e = prefer_max_shared(delta_rule_kernel);
  return e == cudaSuccess ? 0 : check_launch("deltanet step: shared-memory carve-out");
}

int launch_deltanet_step(const DeltaNetParams& p, cudaStream_t stream) {
  if (p.batch <= 0) return 0;
  if (p.dk > MAX_DK || p.dv > 8 * VB || p.dk < 1 || p.dv < 1) {
    set_error("deltanet step: key dim %d (max %d) or value dim %d (max %d) unsupported", p.dk, MAX_DK, p.dv, 8 * VB);
    return 2;
  }
  if (p.num_k_heads < 1 || p.num_v_heads % p.num_k_heads) {
    set_error("deltanet step: %d value heads do not divide into %d key heads", p.num_v_heads, p.num_k_heads);
    return 2;
  }
  if (p.batch >= 4 && p.dv <= HB_COLS * VB) {  // many sequences: a CTA per (head, sequence), no clusters
    if (launch_pdl(deltanet_head_kernel, dim3(p.num_v_heads, p.batch), dim3(DN_WARPS * 32), 0, stream, p) != cudaSuccess)
      return check_launch("deltanet step (per head)");
    return check_launch("deltanet step (per head)");
  }
  const int nvb = (p.dv + VB - 1) / VB;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.num_v_heads * nvb, p.batch, 1);
  cfg.blockDim = dim3(DN_WARPS * 32, 1, 1);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = nvb;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  cudaError_t e = cudaLaunchKernelEx(&cfg, deltanet_fused_kernel, p);
  if (e != cudaSuccess) {
    set_error("deltanet step: launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  return check_launch("deltanet step");
}

int launch_delta_rule_step(const DeltaRuleParams& p, cudaStream_t stream) {
  if (p.batch <= 0 || p.heads <= 0) return 0;
  if (p.dk > MAX_DK || p.dk < 1 || p.dv < 1) {
    set_error("delta rule step: key dim %d unsupported (max %d)", p.dk, MAX_DK);
    return 2;
  }
  const int nvb = (p.dv + VB - 1) / VB;
  delta_rule_kernel<<<dim3(p.heads * nvb, p.batch), DN_WARPS * 32, 0, stream>>>(p);
  return check_launch("delta rule step");
}

}  // namespace dfb
