// Single-token attention for the gated full-attention layers, sm_100a.
//
// attn_prep_kernel: per-head RMSNorm of query and key, partial RoPE at the current position, and the
// KV-cache write of the new token (src/deltaforge/reference.py:621-650; RoPE tables :189-200, rotation
// :137-149). attn_decode_kernel: split-KV flash-decode on the unexpanded GQA cache with the output
// gate fused into the merge (reference.py:655-676). They replace the reference's Triton kernels
// _gqa_decode_kernel (src/deltaforge/kernels/gqa_decode.py:67-135), _split_kv_partial_kernel /
// _split_kv_merge_kernel (src/deltaforge/kernels/flash_decode_splitkv.py:51-174) and
// _partial_rope_kernel (src/deltaforge/kernels/fused_rope.py:43-94).
//
// One CTA scans one slice of the keys of one KV head for all query heads of its group, so each K/V
// row is read from HBM once per KV head, not once per query head. A warp takes every 8th key of the
// slice; a lane holds 8 of the 256 head dims (one 16-byte load per row). Scores, running max, sum and
// the weighted values are fp32 (like the reference's own decode kernels). The 8 warps of a CTA are
// merged in shared memory, slices are merged by the last CTA to arrive for the KV head: per query
// head one warp reduces (max, sum) over the slices with shuffles, then every thread rescales its
// head dim. The position comes from device memory, so one captured launch serves every token.
//
// Bytes per launch: 2 * batch * hkv * key_len * d * 2 (K and V once) + partials.
#include "common.cuh"
#include "kernels.h"

namespace dfb {

namespace {

constexpr int AW = 8;          // warps per CTA
constexpr int MAX_GROUP = 8;   // query heads per KV head
constexpr int MAX_SPLITS = 128;

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

template <int GROUPS>
__global__ void __launch_bounds__(AW * 32) attn_decode_kernel(const AttnParams p) {
  // d == 256: lane l owns dims [8l, 8l+8).
  constexpr int D = 256;
  extern __shared__ float sm[];
  float* q_s = sm;                         // [GROUPS][D]
  float* acc_s = q_s + GROUPS * D;         // [AW][GROUPS][D]
  float* ml_s = acc_s + AW * GROUPS * D;   // [AW][GROUPS][2]
  float* wgt_s = ml_s + AW * GROUPS * 2;   // [GROUPS][MAX_SPLITS] merge weights
  __shared__ int s_last;

  pdl_launch_dependents();
  pdl_wait();  // q, the new K/V row and the position come from the kernels before this one
  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
  const int L = p.pos ? (*p.pos + 1) : p.key_len;
  const int S = p.splits;
  const int chunk = (L + S - 1) / S;
  const int k_begin = split * chunk, k_end = min(L, k_begin + chunk);

  // queries of this KV head's group, fp32, pre-multiplied by the softmax scale
  for (int i = t; i < GROUPS * D; i += AW * 32) {
    const int g = i / D, dd = i % D;
    q_s[i] = bf2f(p.q[(long)b * p.q_stride + (long)(hk * GROUPS + g) * p.qh_stride + dd]) * p.scale;
  }
  __syncthreads();
  float qr[GROUPS][8];
#pragma unroll
  for (int g = 0; g < GROUPS; ++g)
#pragma unroll
    for (int i = 0; i < 8; ++i) qr[g][i] = q_s[g * D + lane * 8 + i];

  const uint64_t pol = make_evict_first_policy();
  const bf16* kbase = p.kcache + (long)b * p.kv_batch_stride + (long)hk * p.kv_head_stride + lane * 8;
  const bf16* vbase = p.vcache + (long)b * p.kv_batch_stride + (long)hk * p.kv_head_stride + lane * 8;

  float m[GROUPS], l[GROUPS], acc[GROUPS][8];
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
  }

  // two keys per iteration so four 16-byte loads are in flight per lane
  for (int k0 = k_begin + warp * 2; k0 < k_end; k0 += AW * 2) {
    const bool two = (k0 + 1) < k_end;
    const uint4 ka = ldg_stream_u4(kbase + (long)k0 * D, pol);
    const uint4 va = ldg_stream_u4(vbase + (long)k0 * D, pol);
    uint4 kb = ka, vb = va;
    if (two) {
      kb = ldg_stream_u4(kbase + (long)(k0 + 1) * D, pol);
      vb = ldg_stream_u4(vbase + (long)(k0 + 1) * D, pol);
    }
    float kf[2][8], vf[2][8];
    unpack8(ka, kf[0]);
    unpack8(kb, kf[1]);
    unpack8(va, vf[0]);
    unpack8(vb, vf[1]);
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
      float s0 = 0.f, s1 = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        s0 = fmaf(qr[g][i], kf[0][i], s0);
        s1 = fmaf(qr[g][i], kf[1][i], s1);
      }
      s0 = warp_sum(s0);
      s1 = two ? warp_sum(s1) : -INFINITY;
      const float mn = fmaxf(m[g], fmaxf(s0, s1));
      const float corr = __expf(m[g] - mn), p0 = __expf(s0 - mn), p1 = __expf(s1 - mn);
      l[g] = l[g] * corr + p0 + p1;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[g][i] = acc[g][i] * corr + p0 * vf[0][i] + p1 * vf[1][i];
      m[g] = mn;
    }
  }

  // merge the 8 warps
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
#pragma unroll
    for (int i = 0; i < 8; ++i) acc_s[(warp * GROUPS + g) * D + lane * 8 + i] = acc[g][i];
    if (lane == 0) {
      ml_s[(warp * GROUPS + g) * 2] = m[g];
      ml_s[(warp * GROUPS + g) * 2 + 1] = l[g];
    }
  }
  __syncthreads();
  float o[GROUPS], lt[GROUPS], mt[GROUPS];  // thread t owns head dim t
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    float mg = -INFINITY;
#pragma unroll
    for (int w = 0; w < AW; ++w) mg = fmaxf(mg, ml_s[(w * GROUPS + g) * 2]);
    float lg = 0.f, og = 0.f;
#pragma unroll
    for (int w = 0; w < AW; ++w) {
      const float mw = ml_s[(w * GROUPS + g) * 2];
      const float sc = (mw == -INFINITY) ? 0.f : __expf(mw - mg);
      lg += ml_s[(w * GROUPS + g) * 2 + 1] * sc;
      og += acc_s[(w * GROUPS + g) * D + t] * sc;
    }
    o[g] = og;
    lt[g] = lg;
    mt[g] = mg;
  }

  const int hq0 = hk * GROUPS;
  if (S > 1) {
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
      const long ph = ((long)b * p.hq + hq0 + g) * S + split;
      __stcg(&p.part_acc[ph * D + t], o[g]);
      if (t == 0) {
        __stcg(&p.part_ml[ph * 2], mt[g]);
        __stcg(&p.part_ml[ph * 2 + 1], lt[g]);
      }
    }
    __threadfence();
    __syncthreads();
    if (t == 0) {
      unsigned* ctr = &p.counters[b * p.hkv + hk];
      const unsigned old = atomicAdd(ctr, 1u);
      s_last = (old == (unsigned)(S - 1));
      if (s_last) *ctr = 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // log-sum-exp combine over the slices: warp g reduces head g's (max, sum) with shuffles.
    for (int g = warp; g < GROUPS; g += AW) {
      const long ph = ((long)b * p.hq + hq0 + g) * S;
      float mloc = -INFINITY;
      for (int s = lane; s < S; s += 32) mloc = fmaxf(mloc, __ldcg(&p.part_ml[(ph + s) * 2]));
      const float mg = warp_max(mloc);
      float lloc = 0.f;
      for (int s = lane; s < S; s += 32) {
        const float ms = __ldcg(&p.part_ml[(ph + s) * 2]);
        const float sc = (ms == -INFINITY) ? 0.f : __expf(ms - mg);
        wgt_s[g * MAX_SPLITS + s] = sc;
        lloc += __ldcg(&p.part_ml[(ph + s) * 2 + 1]) * sc;
      }
      const float lg = warp_sum(lloc);
      const float inv = 1.f / lg;
      for (int s = lane; s < S; s += 32) wgt_s[g * MAX_SPLITS + s] *= inv;
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
      const long ph = ((long)b * p.hq + hq0 + g) * S;
      float og = 0.f;
      for (int s = 0; s < S; ++s) og = fmaf(wgt_s[g * MAX_SPLITS + s], __ldcg(&p.part_acc[(ph + s) * D + t]), og);
      o[g] = og;
      lt[g] = 1.f;
    }
  }

  // normalise, output gate (reference.py:558-568, :675-676), store
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    float y = round_bf16(o[g] / lt[g]);
    if (p.gate) {
      const float gv = bf2f(p.gate[(long)b * p.gate_stride + (long)(hq0 + g) * p.gateh_stride + t]);
      const float gg = round_bf16(p.gate_swish ? silu_f(gv) : sigmoid_f(gv));
      y = round_bf16(__fmul_rn(y, gg));
    }
    p.out[(long)b * p.out_stride + (long)(hq0 + g) * D + t] = f2bf(y);
  }
}

// Any head_dim and group size: one CTA of 128 threads per (query head, batch), one pass, no splits.
__global__ void __launch_bounds__(128) attn_decode_generic_kernel(const AttnParams p) {
  extern __shared__ float sm[];  // [d] query, [L] scores
  pdl_launch_dependents();
  pdl_wait();
  const int hq = blockIdx.x, b = blockIdx.y, t = threadIdx.x;
  const int groups = p.hq / p.hkv, hk = hq / groups, d = p.d;
  const int L = p.pos ? (*p.pos + 1) : p.key_len;
  float* q_s = sm;
  float* sc = sm + d;
  __shared__ float redm[4];
  for (int i = t; i < d; i += 128) q_s[i] = bf2f(p.q[(long)b * p.q_stride + (long)hq * p.qh_stride + i]) * p.scale;
  __syncthreads();
  const bf16* kb = p.kcache + (long)b * p.kv_batch_stride + (long)hk * p.kv_head_stride;
  const bf16* vb = p.vcache + (long)b * p.kv_batch_stride + (long)hk * p.kv_head_stride;
  float mloc = -INFINITY;
  for (int k = t; k < L; k += 128) {
    float s = 0.f;
    for (int i = 0; i < d; ++i) s = fmaf(q_s[i], bf2f(kb[(long)k * d + i]), s);
    sc[k] = s;
    mloc = fmaxf(mloc, s);
  }
  mloc = warp_max(mloc);
  if ((t & 31) == 0) redm[t >> 5] = mloc;
  __syncthreads();
  const float mg = fmaxf(fmaxf(redm[0], redm[1]), fmaxf(redm[2], redm[3]));
  __syncthreads();
  float lloc = 0.f;
  for (int k = t; k < L; k += 128) {
    const float e = expf(sc[k] - mg);
    sc[k] = e;
    lloc += e;
  }
  lloc = warp_sum(lloc);
  if ((t & 31) == 0) redm[t >> 5] = lloc;
  __syncthreads();
  const float lg = redm[0] + redm[1] + redm[2] + redm[3];
  for (int i = t; i < d; i += 128) {
    float o = 0.f;
    for (int k = 0; k < L; ++k) o = fmaf(sc[k], bf2f(vb[(long)k * d + i]), o);
    float y = round_bf16(o / lg);
    if (p.gate) {
      const float gv = bf2f(p.gate[(long)b * p.gate_stride + (long)hq * p.gateh_stride + i]);
      const float gg = round_bf16(p.gate_swish ? silu_f(gv) : sigmoid_f(gv));
      y = round_bf16(__fmul_rn(y, gg));
    }
    p.out[(long)b * p.out_stride + (long)hq * d + i] = f2bf(y);
  }
}

// One warp per head row of the fused q|k|v projection.
__global__ void __launch_bounds__(128) attn_prep_kernel(const AttnPrepParams p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  pdl_launch_dependents();
  pdl_wait();  // the projection row comes from the GEMV before this kernel
  const int head = blockIdx.x * 4 + warp, b = blockIdx.y;
  const int total = p.hq + 2 * p.hkv;
  if (head >= total) return;
  const int d = p.d, rd = p.rotary_dim, half = rd / 2;
  const int pos = *p.pos;
  if (head >= p.hq && p.max_seq > 0 && pos >= p.max_seq) return;  // never write past the cache
  const int qw = p.attn_output_gate ? 2 * d : d;
  const bf16* src;
  bf16* dst;
  const bf16* nw = nullptr;
  if (head < p.hq) {
    src = p.proj + (long)b * p.proj_stride + (long)head * qw;
    dst = p.q_out + ((long)b * p.hq + head) * d;
    nw = p.q_norm_w;
  } else if (head < p.hq + p.hkv) {
    const int h = head - p.hq;
    src = p.proj + (long)b * p.proj_stride + (long)p.hq * qw + (long)h * d;
    dst = p.kcache + (long)b * p.kv_batch_stride + (long)h * p.kv_head_stride + (long)pos * d;
    nw = p.k_norm_w;
  } else {
    const int h = head - p.hq - p.hkv;
    src = p.proj + (long)b * p.proj_stride + (long)p.hq * qw + (long)(p.hkv + h) * d;
    dst = p.vcache + (long)b * p.kv_batch_stride + (long)h * p.kv_head_stride + (long)pos * d;
  }
  if (nw == nullptr) {  // value head: plain copy
    for (int i = lane; i < d; i += 32) dst[i] = src[i];
    return;
  }
  float ss = 0.f;
  for (int i = lane; i < d; i += 32) {
    const float v = bf2f(src[i]);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  const float rstd = rsqrt_2step(__fadd_rn(__fdiv_rn(ss, (float)d), p.eps));
  for (int i = lane; i < d; i += 32) {
    const float xn = round_bf16(__fmul_rn(__fmul_rn(bf2f(src[i]), rstd), __fadd_rn(1.0f, bf2f(nw[i]))));
    if (i >= rd) {
      dst[i] = f2bf(xn);
      continue;
    }
    // rotate: out = x*cos + rotate_half(x)*sin, every product and the sum rounded to bf16
    const int j = (i < half) ? i + half : i - half;
    const float xo = round_bf16(__fmul_rn(__fmul_rn(bf2f(src[j]), rstd), __fadd_rn(1.0f, bf2f(nw[j]))));
    const float ang = __fmul_rn((float)pos, p.inv_freq[i % half]);
    const float c = round_bf16(cosf(ang)), s = round_bf16(sinf(ang));
    const float a = round_bf16(__fmul_rn(xn, c));
    const float r = round_bf16(__fmul_rn(i < half ? -xo : xo, s));
    dst[i] = f2bf(__fadd_rn(a, r));
  }
}

template <int GROUPS>
size_t fast_smem() {
  return (size_t)(GROUPS * 256 + AW * GROUPS * 256 + AW * GROUPS * 2 + GROUPS * MAX_SPLITS) * sizeof(float);
}
template <int GROUPS>
cudaError_t configure_groups() {
  return cudaFuncSetAttribute(attn_decode_kernel<GROUPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fast_smem<GROUPS>());
}

template <int GROUPS>
int launch_fast(const AttnParams& p, cudaStream_t stream) {
  const size_t smem = fast_smem<GROUPS>();
  if (launch_pdl(attn_decode_kernel<GROUPS>, dim3(p.splits, p.hkv, p.batch), dim3(AW * 32), smem, stream, p) != cudaSuccess)
    return check_launch("attention decode");
  return check_launch("attention decode");
}

}  // namespace

int attn_configure() {
  cudaError_t e = configure_groups<1>();
  if (e == cudaSuccess) e = configure_groups<2>();
  if (e == cudaSuccess) e = configure_groups<4>();
  if (e == cudaSuccess) e = configure_groups<8>();
  if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_decode_generic_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  return e == cudaSuccess ? 0 : check_launch("attention decode: shared-memory opt-in");
}

int launch_attn_decode(const AttnParams& p, cudaStream_t stream) {
  if (p.batch <= 0) return 0;
  static OncePerDevice once;
  const int configured = once.run(attn_configure);
  if (configured) return configured;
  if (p.hkv < 1 || p.hq % p.hkv) {
    set_error("attention decode: %d query heads do not divide into %d KV heads", p.hq, p.hkv);
    return 2;
  }
  const int groups = p.hq / p.hkv;
  if (attn_mma_ok(p)) return launch_attn_decode_mma(p, nullptr, stream);
  if (p.d == 256 && (groups == 1 || groups == 2 || groups == 4 || groups == 8) && p.splits >= 1 &&
      p.splits <= MAX_SPLITS) {
    if (p.splits > 1 && (!p.part_acc || !p.part_ml || !p.counters)) {
      set_error("attention decode: split-KV scratch is required for %d splits", p.splits);
      return 2;
    }
    switch (groups) {
      case 1: return launch_fast<1>(p, stream);
      case 2: return launch_fast<2>(p, stream);
      case 4: return launch_fast<4>(p, stream);
      default: return launch_fast<8>(p, stream);
    }
  }
  // With a device-side position, key_len is the capacity of the cache (the most keys there can be).
  if (p.key_len < 1) {
    set_error("attention decode: the generic path needs key_len (or the cache capacity) on the host");
    return 2;
  }
  const size_t smem = (size_t)(p.d + p.key_len) * sizeof(float);
  if (smem > 200 * 1024) {
    set_error("attention decode: generic path limited to %d keys", (int)(200 * 1024 / 4 - p.d));
    return 2;
  }
  if (launch_pdl(attn_decode_generic_kernel, dim3(p.hq, p.batch), dim3(128), smem, stream, p) != cudaSuccess)
    return check_launch("attention decode (generic)");
  return check_launch("attention decode (generic)");
}

int launch_attn_prep(const AttnPrepParams& p, cudaStream_t stream) {
  if (p.batch <= 0) return 0;
  if (p.rotary_dim % 2 || p.rotary_dim > p.d) {
    set_error("attention prep: rotary_dim %d must be even and at most head_dim %d", p.rotary_dim, p.d);
    return 2;
  }
  const int total = p.hq + 2 * p.hkv;
  if (launch_pdl(attn_prep_kernel, dim3((total + 3) / 4, p.batch), dim3(128), 0, stream, p) != cudaSuccess)
    return check_launch("attention prep");
  return check_launch("attention prep");
}

}  // namespace dfb
