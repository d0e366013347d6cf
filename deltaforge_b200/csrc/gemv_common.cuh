// Prologue and epilogue arithmetic shared by the int4 GEMV kernels.
#pragma once

#include "common.cuh"
#include "kernels.h"

namespace dfb {

__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & mask) | orv
  return r;
}

// d = a * b + c with a, b fp16 (the selected half of `pair`, and x) and c, d fp32: the product of two
// fp16 numbers is exact in fp32, so this is one rounding, like an fp32 FMA on converted operands.
__device__ __forceinline__ float fma_f16(uint32_t pair, int hi, unsigned short x, float c) {
  unsigned short a = hi ? (unsigned short)(pair >> 16) : (unsigned short)(pair & 0xffffu);
  float d;
  asm("fma.rn.f32.f16 %0, %1, %2, %3;" : "=f"(d) : "h"(a), "h"(x), "f"(c));
  return d;
}

// Value of activation element k of row r after the prologue, as the bf16 the reference would hold.
__device__ __forceinline__ float prologue_value(const GemvParams& p, int r, int k, float rstd) {
  float xv = bf2f(p.x[(long)r * p.x_stride + k]);
  if (p.prologue == PRO_RMSNORM) {
    float v = __fmul_rn(xv, rstd);
    v = __fmul_rn(v, __fadd_rn(1.0f, bf2f(p.norm_w[k])));
    return round_bf16(v);
  }
  if (p.prologue == PRO_SILU_MUL) {
    float s = round_bf16(silu_f(xv));
    return round_bf16(__fmul_rn(s, bf2f(p.up[(long)r * p.up_stride + k])));
  }
  return xv;
}

// The same arithmetic on values already loaded: xv the activation, wv the norm weight (PRO_RMSNORM) or `up`
// (PRO_SILU_MUL), both as the fp32 of their bf16.
__device__ __forceinline__ float prologue_apply(int prologue, float xv, float wv, float rstd) {
  if (prologue == PRO_RMSNORM) {
    float v = __fmul_rn(xv, rstd);
    v = __fmul_rn(v, __fadd_rn(1.0f, wv));
    return round_bf16(v);
  }
  if (prologue == PRO_SILU_MUL) {
    float s = round_bf16(silu_f(xv));
    return round_bf16(__fmul_rn(s, wv));
  }
  return xv;
}

// PRO_ATTN_MERGE: the four activation values k .. k+3 (k a multiple of 4) of the gated attention output. All loads
// (every cluster's (m, l) pair and its four partial sums) are issued before anything is computed: one round trip.
__device__ __forceinline__ void attn_merge_values(const AttnMerge& a, int k, float (&v)[4]) {
  constexpr int MAXC = 8;  // cluster_path_ok() admits at most this many
  const int h = k / a.d, i = k % a.d;
  const float2* ml = (const float2*)(a.ml + (long)h * a.nclusters * 2);
  const float* acc = a.acc + (long)h * a.nclusters * a.d + i;
  float2 mlv[MAXC];
  float4 pa[MAXC];
  uint2 graw = make_uint2(0u, 0u);
  if (a.gate) graw = *(const uint2*)(a.gate + (long)h * a.gateh_stride + i);
  // volatile loads keep their order among themselves: all sixteen are issued before the first value is used. (Left to
  // the compiler's schedule they went cluster by cluster: one trip to the L2 per cluster, 0.35 us each.)
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {
    mlv[c] = make_float2(-INFINITY, 0.f);
    pa[c] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (c < a.nclusters) {
      asm volatile("ld.global.cg.v2.f32 {%0, %1}, [%2];" : "=f"(mlv[c].x), "=f"(mlv[c].y) : "l"(ml + c));
      asm volatile("ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(pa[c].x), "=f"(pa[c].y), "=f"(pa[c].z), "=f"(pa[c].w)
                   : "l"(acc + (long)c * a.d));
    }
  }
  float mg = -INFINITY;
#pragma unroll
  for (int c = 0; c < MAXC; ++c) mg = fmaxf(mg, mlv[c].x);
  float o[4] = {0.f, 0.f, 0.f, 0.f}, l = 0.f;
#pragma unroll
  for (int c = 0; c < MAXC; ++c) {  // fixed order: the same bits every run
    const float w = (mlv[c].x == -INFINITY) ? 0.f : __expf(mlv[c].x - mg);
    l = fmaf(w, mlv[c].y, l);
    o[0] = fmaf(w, pa[c].x, o[0]), o[1] = fmaf(w, pa[c].y, o[1]), o[2] = fmaf(w, pa[c].z, o[2]), o[3] = fmaf(w, pa[c].w, o[3]);
  }
  const float gl[4] = {__uint_as_float(graw.x << 16), __uint_as_float(graw.x & 0xffff0000u), __uint_as_float(graw.y << 16),
                       __uint_as_float(graw.y & 0xffff0000u)};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float y = round_bf16(__fdiv_rn(o[j], l));
    if (a.gate) y = round_bf16(__fmul_rn(y, gl[j]));
    v[j] = y;
  }
}

__device__ __forceinline__ float load_scale(const GemvParams& p, long idx) {
  return p.scale_bf16 ? bf2f(((const bf16*)p.scale)[idx]) : ((const float*)p.scale)[idx];
}

// What the epilogue of output element (r, n) reads besides the sum: loaded early, so that the loads are in
// flight while the dot products run, and handed to epilogue_store_pre().
struct EpiPre {
  float res;             // EPI_RESIDUAL: the residual stream's value
  float h0, h1, h2;      // EPI_CONV: the three older taps of the channel's history
  float w0, w1, w2, w3;  // EPI_CONV: the channel's conv weights
};
__device__ __forceinline__ EpiPre epilogue_preload(const GemvParams& p, int r, int n) {
  EpiPre e = {};
  if (p.epilogue == EPI_RESIDUAL) {
    e.res = bf2f(p.residual[(long)r * p.res_stride + n]);
  } else if (p.epilogue == EPI_CONV && n < p.conv_dim) {
    const bf16* st = p.conv_state + ((long)r * p.conv_dim + n) * 3;
    const bf16* w = p.conv_w + (long)n * 4;
    e.h0 = bf2f(st[0]), e.h1 = bf2f(st[1]), e.h2 = bf2f(st[2]);
    e.w0 = bf2f(w[0]), e.w1 = bf2f(w[1]), e.w2 = bf2f(w[2]), e.w3 = bf2f(w[3]);
  }
  return e;
}

// Output element (r, n) from its fp32 sum; returns the value stored (as fp32).
__device__ __forceinline__ float epilogue_store_pre(const GemvParams& p, int r, int n, float sum, const EpiPre& pre) {
  if (!DFB_IN_BOUNDS(r >= 0 && r < p.rows && n >= 0 && n < p.N, p.status, 1)) return 0.f;
  if (p.epilogue == EPI_PARTIAL_PEER) {
    // one 8-byte store per rank: the value and the epoch arrive together, the receiver needs no fence
    const unsigned epoch = *p.peer.epoch_ctr * 256u + (unsigned)p.peer.epoch_off;
    const unsigned long long w = ((unsigned long long)epoch << 32) | __float_as_uint(sum);
    const long at = p.peer.word_off + (long)r * p.N + n;
    for (int k = 0; k < p.peer.tp_size; ++k)
      asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p.peer.slots[k] + at), "l"(w) : "memory");
    return sum;
  }
  if (p.epilogue == EPI_PARTIAL_F32) {
    ((float*)p.out)[(long)r * p.out_stride + n] = sum;
    return sum;
  }
  bf16 y = f2bf(sum);
  if (p.epilogue == EPI_RESIDUAL) {
    const bf16 o = f2bf(__fadd_rn(pre.res, bf2f(y)));
    p.out[(long)r * p.out_stride + n] = o;
    return bf2f(o);
  }
  if (p.epilogue == EPI_CONV && n < p.conv_dim) {
    // 4-tap depthwise causal conv decode step (src/deltaforge/kernels/inline_causal_conv.py:111-129):
    // fp32 products summed left to right, rounded to bf16, then SiLU; history [h0,h1,h2] <- [h1,h2,x].
    bf16* st = p.conv_state + ((long)r * p.conv_dim + n) * 3;
    const float xv = bf2f(y);
    float acc = __fmul_rn(pre.h0, pre.w0);
    acc = __fadd_rn(acc, __fmul_rn(pre.h1, pre.w1));
    acc = __fadd_rn(acc, __fmul_rn(pre.h2, pre.w2));
    acc = __fadd_rn(acc, __fmul_rn(xv, pre.w3));
    float a = round_bf16(acc);
    const bf16 o = f2bf(silu_f(a));
    p.out[(long)r * p.out_stride + n] = o;
    st[0] = f2bf(pre.h1);
    st[1] = f2bf(pre.h2);
    st[2] = y;
    return bf2f(o);
  }
  p.out[(long)r * p.out_stride + n] = y;
  return bf2f(y);
}
__device__ __forceinline__ float epilogue_store(const GemvParams& p, int r, int n, float sum) {
  return epilogue_store_pre(p, r, n, sum, epilogue_preload(p, r, n));
}

}  // namespace dfb
