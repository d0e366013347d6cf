// The whole attention mixer of a decode step between its two projections, in one launch, sm_100a.
//
// From the fused q(|gate)|k|v projection row to the gated attention output, for one new token:
// q_norm / k_norm, partial RoPE at the device-side position, the KV-cache write, split-KV
// flash-decode over the unexpanded GQA cache, the log-sum-exp merge and the output gate
// (GatedAttention.forward, src/deltaforge/reference.py:621-676). It does the work of attn_prep_kernel
// plus attn_decode_kernel (attn_decode.cu) without the kernel boundary between them and without the
// serial merge of all slices by one CTA:
//
//  * grid (slices, kv heads, batch), clusters of up to 8 slices, at most 160 keys per slice. The rows of
//    a slice that are already in the cache (everything but the new token) are contiguous, so one
//    thread brings K and V of the slice into shared memory with two bulk asynchronous copies, issued
//    before griddepcontrol.wait: they overlap the projection GEMV that runs before this kernel.
//  * After the wait every CTA normalises and rotates the query heads of its KV head itself; the CTA
//    whose slice holds the new position also normalises, rotates and stores the new key and value,
//    and appends that row to its staged slice.
//  * The slice is scanned in three passes over shared memory. Scores: a lane holds 8 of the 256 head dims and forms its
//    part of 32 dot products (8 keys x 4 query heads); one transposing reduction of 31 shuffles finishes all 32, where
//    a reduction per score would take 160. Softmax: one warp per query head finds the slice's maximum and sum. Values:
//    a warp takes every 8th key, a lane 8 head dims. Everything is fp32 (like the reference's own decode kernels). The
//    first form of this kernel reduced every score over the warp with five shuffles and kept a running maximum per
//    warp: 10 000 cycles for 129 keys, nearly all of it shuffle latency.
//  * Warps merge in shared memory; the CTAs of a cluster merge in the first CTA's shared memory
//    through distributed shared memory and one cluster barrier; clusters merge through a small
//    global buffer, finished by the last cluster to arrive.
//
// The wait on the copy barrier is bounded (about two seconds); on a timeout the CTA records a code in
// the status word and carries on with what it has, so that its cluster barrier still completes.
//
// Bytes per launch: 2 * batch * hkv * (pos + 1) * d * 2 (K and V once).
#include "common.cuh"
#include "kernels.h"

namespace dfb {

namespace {

constexpr int AW = 8;  // warps per CTA
constexpr int D = 256;
constexpr int MAX_CS = 8;
constexpr int MAX_KEYS = 160;  // most rows a slice may have (160 KB of staged K and V: one CTA per SM)
constexpr long long WAIT_LIMIT_CYCLES = 4000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void dsmem_store(float* local, uint32_t rank, float v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
__device__ __forceinline__ void bulk_copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t pol) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol)
      : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 256; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - t0 > WAIT_LIMIT_CYCLES) return false;
  }
}
__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __uint_as_float(w[i] << 16);
    f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

// RMSNorm (1 + w) and partial RoPE of one 256-wide head row by one warp, through `row` ([256] floats of
// shared memory); on return row[] holds the bf16 values the reference holds (reference.py:92-96,137-149).
__device__ __noinline__ void norm_rope_row(const bf16* src, const bf16* nw, float eps, const float* inv_freq, int rd, int pos,
                                           float* row) {
  const int lane = threadIdx.x & 31;
  const float f0 = lane < rd / 2 ? inv_freq[lane] : 0.f;  // in flight with the row itself
  float x[8], w[8];
  unpack8(*(const uint4*)(src + lane * 8), x);
  unpack8(*(const uint4*)(nw + lane * 8), w);
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
  ss = warp_sum(ss);
  // 1 / sqrt(ss / 256 + eps) in two correctly rounded steps, as a CPU evaluates it: the division by 256 is exact, so one
  // fused multiply-add rounds where the sum would, and the correctly rounded reciprocal is the correctly rounded 1 / x
  const float rstd = __frcp_rn(__fsqrt_rn(fmaf(ss, 1.0f / (float)D, eps)));
#pragma unroll
  for (int i = 0; i < 8; ++i) row[lane * 8 + i] = round_bf16(__fmul_rn(__fmul_rn(x[i], rstd), __fadd_rn(1.0f, w[i])));
  __syncwarp();
  const int half = rd / 2;
  // out = x*cos + rotate_half(x)*sin, every product and the sum rounded to bf16. Dims d and d + half
  // share an angle and only read each other, so one thread rotates the pair in place.
#pragma unroll 1
  for (int d = lane; d < half; d += 32) {
    const float a = row[d], bb = row[d + half];
    const float ang = __fmul_rn((float)pos, d == lane ? f0 : inv_freq[d]);
    float s, c;
    sincosf(ang, &s, &c);
    c = round_bf16(c), s = round_bf16(s);
    row[d] = round_bf16(__fadd_rn(round_bf16(__fmul_rn(a, c)), round_bf16(__fmul_rn(-bb, s))));
    row[d + half] = round_bf16(__fadd_rn(round_bf16(__fmul_rn(bb, c)), round_bf16(__fmul_rn(a, s))));
  }
  __syncwarp();
}

template <int GROUPS>
__global__ void __launch_bounds__(AW * 32) attn_step_kernel(const AttnStepParams p) {
  extern __shared__ __align__(128) unsigned char smraw[];
  // rows staged per slice: what the cache's capacity can ask for (at least the 32 rows' worth of bytes the warp merge reuses)
  const int cap = max((p.max_seq + (int)gridDim.x - 1) / (int)gridDim.x, AW * GROUPS * 2);
  const int scp = (cap + 31) & ~31;               // score rows are padded to whole warps of keys
  bf16* kst = (bf16*)smraw;                       // [cap][D] staged keys
  bf16* vst = kst + cap * D;                      // [cap][D] staged values
  float* q_s = (float*)(vst + cap * D);           // [GROUPS][D] rotated queries times the softmax scale
  float* rowbuf = q_s + GROUPS * D;               // [2][D] scratch for the new key / value row
  float* sc = rowbuf + 2 * D;                     // [GROUPS][scp] scores of the slice
  float* pj = sc + GROUPS * scp;                  // [scp][GROUPS] exp(score - max): what the value pass reads per key
  float* cl_acc = pj + GROUPS * scp;              // [MAX_CS][GROUPS][D] per-rank sums (used in rank 0)
  float* cl_ml = cl_acc + MAX_CS * GROUPS * D;    // [MAX_CS][GROUPS][2]
  float* wgt = cl_ml + MAX_CS * GROUPS * 2;       // [GROUPS][16] merge weights
  float* wgt_w = wgt + GROUPS * 16;               // [32] rescale weights of the cluster merge
  float* mlt_s = wgt_w + 32;                      // [GROUPS][2] (max, sum) of the slice, then of the cluster
  uint64_t* bar = (uint64_t*)(mlt_s + GROUPS * 2); // copy barrier
  float* acc_s = (float*)smraw;                   // [AW][GROUPS][D], reuses the staged slice after the scan
  __shared__ int s_last;

  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
  const int S = gridDim.x, cs = p.cluster_size;
  const int rank = (int)cluster_rank();
  const int pos = *p.pos;  // written by the previous step's last kernel, long complete
  const int L = pos + 1;
  const int chunk = (L + S - 1) / S;  // <= MAX_KEYS, checked on the host against the cache capacity
  const int k_begin = split * chunk, k_end = min(L, k_begin + chunk);
  // (bounds build: a slice longer than its staging buffer is recorded and scanned as empty; the CTA still takes part in
  // every barrier)
  const bool sane = DFB_IN_BOUNDS(chunk <= max((p.max_seq + S - 1) / S, AW * GROUPS * 2), p.status, 6);
  const bool owns_new = sane && (k_begin <= pos) && (pos < k_end);
  const int n_old = sane ? max(0, (owns_new ? k_end - 1 : k_end) - k_begin) : 0;  // rows already in the cache
  const int n_keys = n_old + (owns_new ? 1 : 0);

  if (t == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bar)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_launch_dependents();
  const int cta = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x, nctas = gridDim.x * gridDim.y * gridDim.z;
  if (t == 0) trace_mark(p.trace, cta, 0);
  if (t == 32) {  // a slice of the weights a later GEMV of the step reads, into the L2
#pragma unroll
    for (int i = 0; i < 2; ++i)
      if (p.pf_ptr[i] != nullptr)
        l2_prefetch_range(p.pf_ptr[i], p.pf_bytes[i] * (size_t)cta / nctas, p.pf_bytes[i] * (size_t)(cta + 1) / nctas);
  }
  if (t == 0 && n_old > 0) {
    // old rows of the slice are contiguous in the cache: two bulk copies, in flight before the wait
    const uint64_t pol = make_evict_first_policy();
    const long off = (long)b * p.kv_batch_stride + (long)hk * p.kv_head_stride + (long)k_begin * D;
    const uint32_t bytes = (uint32_t)n_old * D * 2;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(2 * bytes) : "memory");
    bulk_copy(kst, p.kcache + off, bytes, bar, pol);
    bulk_copy(vst, p.vcache + off, bytes, bar, pol);
  }
  pdl_wait();
  if (t == 0) trace_mark(p.trace, cta, 1);

  // queries of this KV head's group (warps 0..GROUPS-1), new key (warp GROUPS) and value (warp GROUPS+1)
  const int qw = p.attn_output_gate ? 2 * D : D;
  const bf16* proj = p.proj + (long)b * p.proj_stride;
  if (warp < GROUPS) {
    float* row = q_s + warp * D;
    norm_rope_row(proj + (long)(hk * GROUPS + warp) * qw, p.q_norm_w, p.eps, p.inv_freq, p.rotary_dim, pos, row);
#pragma unroll
    for (int i = 0; i < 8; ++i) row[lane * 8 + i] *= p.scale;
  } else if (owns_new && warp == GROUPS) {
    norm_rope_row(proj + (long)p.hq * qw + (long)hk * D, p.k_norm_w, p.eps, p.inv_freq, p.rotary_dim, pos, rowbuf);
    bf16* dst = p.kcache + (long)b * p.kv_batch_stride + (long)hk * p.kv_head_stride + (long)pos * D + lane * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const bf16 v = f2bf(rowbuf[lane * 8 + i]);
      kst[n_old * D + lane * 8 + i] = v;  // the new row joins the staged slice
      if (pos < p.max_seq) dst[i] = v;
    }
  } else if (owns_new && warp == GROUPS + 1) {
    const uint4 raw = *(const uint4*)(proj + (long)p.hq * qw + (long)(p.hkv + hk) * D + lane * 8);
    *(uint4*)(vst + n_old * D + lane * 8) = raw;
    if (pos < p.max_seq)
      *(uint4*)(p.vcache + (long)b * p.kv_batch_stride + (long)hk * p.kv_head_stride + (long)pos * D + lane * 8) = raw;
  }
  // the output-gate logits are needed last: fetch them now
  float gate_v[GROUPS];
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) gate_v[g] = p.attn_output_gate ? bf2f(proj[(long)(hk * GROUPS + g) * qw + D + t]) : 0.f;
  bool ok = true;
  if (n_old > 0) ok = mbar_wait(bar, 0);
  if (!ok && t == 0 && p.status) atomicExch(p.status, 5);
  __syncthreads();
  if (t == 0) trace_mark(p.trace, cta, 2);

  // Pass 1, scores: a lane holds 8 of the 256 head dims (rows are read as they lie, no bank conflicts) and forms its part
  // of the dot products of a batch of keys with every query head of the group: 32 partial sums per lane. One
  // transposing reduction (31 shuffles: at every level a lane sends the half of its values that its partner keeps)
  // leaves lane l with the finished score number l of the batch, instead of five shuffles per score.
  {
    float qr[GROUPS][8];
#pragma unroll
    for (int g = 0; g < GROUPS; ++g)
#pragma unroll
      for (int i = 0; i < 8; ++i) qr[g][i] = q_s[g * D + lane * 8 + i];
    constexpr int KB = 32 / GROUPS;  // keys per batch
#pragma unroll 1
    for (int j0 = warp * KB; j0 < n_keys; j0 += AW * KB) {
      float v[32];
#pragma unroll
      for (int kk = 0; kk < KB; ++kk) {
        float kf[8];
        unpack8(*(const uint4*)(kst + (size_t)min(j0 + kk, n_keys - 1) * D + lane * 8), kf);
#pragma unroll
        for (int g = 0; g < GROUPS; ++g) {
          float a = 0.f;
#pragma unroll
          for (int i = 0; i < 8; ++i) a = fmaf(qr[g][i], kf[i], a);
          v[kk * GROUPS + g] = a;
        }
      }
#pragma unroll
      for (int h = 16; h > 0; h >>= 1) {
        const bool up = (lane & h) != 0;
#pragma unroll
        for (int i = 0; i < h; ++i) {
          const float send = up ? v[i] : v[i + h], keep = up ? v[i + h] : v[i];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, h);
        }
      }
      const int j = j0 + lane / GROUPS;  // lane l holds value number l of the batch: key l / GROUPS, head l % GROUPS
      if (j < n_keys) sc[(lane % GROUPS) * scp + j] = v[0];
    }
  }
  __syncthreads();
  // Pass 2, softmax of the slice: warp g takes query head g
  if (warp < GROUPS) {
    float mx = -INFINITY;
    for (int i = lane; i < n_keys; i += 32) mx = fmaxf(mx, sc[warp * scp + i]);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int i = lane; i < n_keys; i += 32) {
      const float sv = sc[warp * scp + i];
      const float pe = __expf(sv - mx);
      pj[i * GROUPS + warp] = pe;
      sum += pe;
    }
    sum = warp_sum(sum);
    if (lane == 0) {
      mlt_s[warp * 2] = mx;
      mlt_s[warp * 2 + 1] = sum;
    }
  }
  __syncthreads();
  // Pass 3, values: a warp takes every 8th key, a lane 8 of the 256 head dims
  float acc[GROUPS][8];
#pragma unroll
  for (int g = 0; g < GROUPS; ++g)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
#pragma unroll 2
  for (int j = warp; j < n_keys; j += AW) {
    float vf[8];
    unpack8(*(const uint4*)(vst + (size_t)j * D + lane * 8), vf);
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
      const float pe = pj[j * GROUPS + g];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(pe, vf[i], acc[g][i]);
    }
  }
  __syncthreads();  // everyone is done with the staged slice; its memory becomes the warp-merge buffer
  if (t == 0) trace_mark(p.trace, cta, 3);

  // add the 8 warps (one common maximum per slice: no rescaling): afterwards thread t owns head dim t of every query head
#pragma unroll
  for (int g = 0; g < GROUPS; ++g)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc_s[(warp * GROUPS + g) * D + lane * 8 + i] = acc[g][i];
  __syncthreads();
  float o[GROUPS], lt[GROUPS], mt[GROUPS];
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    float og = 0.f;
#pragma unroll
    for (int w = 0; w < AW; ++w) og += acc_s[(w * GROUPS + g) * D + t];
    o[g] = og, lt[g] = mlt_s[g * 2 + 1], mt[g] = mlt_s[g * 2];
  }
  __syncthreads();  // (mlt_s is written again by the cluster merge)

  // With the last merge left to the output projection, one cluster per KV head also leaves the output gate, already
  // activated: bf16(sigmoid(fp32(gate))) (src/deltaforge/reference.py:558-568). It depends on nothing computed here, so
  // it is evaluated now, while the other CTAs of the cluster arrive at the barrier, and not after it on the way out.
  const bool early_gate = p.defer_merge && S / cs > 1 && split / cs == 0 && rank == 0 && p.attn_output_gate;
  if (early_gate) {
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
      const float gv = gate_v[g];
      p.out[(long)b * p.out_stride + (long)(hk * GROUPS + g) * D + t] = f2bf(p.gate_swish ? silu_f(gv) : sigmoid_f(gv));
    }
  }
  // merge the CTAs of the cluster in rank 0, the same way
  if (cs > 1) {
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
      dsmem_store(cl_acc + (rank * GROUPS + g) * D + t, 0, o[g]);
      if (t == 0) {
        dsmem_store(cl_ml + (rank * GROUPS + g) * 2, 0, mt[g]);
        dsmem_store(cl_ml + (rank * GROUPS + g) * 2 + 1, 0, lt[g]);
      }
    }
    cluster_barrier();
    if (t == 0) trace_mark(p.trace, cta, 5);
    if (rank != 0) return;
    if (warp == 0) {  // lane = r * GROUPS + g (cs * GROUPS <= 32)
      const int g = lane % GROUPS, r = lane / GROUPS;
      const bool live = lane < cs * GROUPS;
      float mg = -INFINITY;
      for (int rr = 0; rr < cs; ++rr) mg = fmaxf(mg, cl_ml[(rr * GROUPS + g) * 2]);
      const float mr = live ? cl_ml[(r * GROUPS + g) * 2] : -INFINITY;
      const float e = (mr == -INFINITY) ? 0.f : __expf(mr - mg);
      float lr = live ? cl_ml[(r * GROUPS + g) * 2 + 1] * e : 0.f;
#pragma unroll
      for (int o2 = GROUPS; o2 < 32; o2 <<= 1) lr += __shfl_xor_sync(0xffffffffu, lr, o2);
      if (live) wgt_w[lane] = e;
      if (lane < GROUPS) {
        mlt_s[lane * 2] = mg;
        mlt_s[lane * 2 + 1] = lr;
      }
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
      float og = 0.f;
      for (int r = 0; r < cs; ++r) og = fmaf(cl_acc[(r * GROUPS + g) * D + t], wgt_w[r * GROUPS + g], og);
      o[g] = og, lt[g] = mlt_s[g * 2 + 1], mt[g] = mlt_s[g * 2];
    }
  }

  // merge the clusters through global memory; the last one to arrive finishes
  const int hq0 = hk * GROUPS;
  const int nclusters = S / cs;
  if (nclusters > 1) {
    const int cidx = split / cs;
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
      const long ph = ((long)b * p.hq + hq0 + g) * nclusters + cidx;
      __stcg(&p.part_acc[ph * D + t], o[g]);
      if (t == 0) {
        __stcg(&p.part_ml[ph * 2], mt[g]);
        __stcg(&p.part_ml[ph * 2 + 1], lt[g]);
      }
    }
    if (p.defer_merge) {  // the output projection merges the clusters' partial results while it builds its activation
      // (... and multiplies by the output gate, which one cluster per KV head has left in `out`, see above)
      if (t == 0) trace_mark(p.trace, cta, 6);
      return;
    }
    __threadfence();
    __syncthreads();
    if (t == 0) {
      unsigned* ctr = &p.counters[b * p.hkv + hk];
      const unsigned old = atomicAdd(ctr, 1u);
      s_last = (old == (unsigned)(nclusters - 1));
      if (s_last) *ctr = 0u;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    if (warp < GROUPS) {  // nclusters <= 16: one lane per cluster, the warp finds the common max
      const long ph = ((long)b * p.hq + hq0 + warp) * nclusters + lane;
      const float ms = lane < nclusters ? __ldcg(&p.part_ml[ph * 2]) : -INFINITY;
      const float mg = warp_max(ms);
      if (lane < nclusters) wgt[warp * 16 + lane] = (ms == -INFINITY) ? 0.f : __expf(ms - mg);
    }
    __syncthreads();
#pragma unroll
    for (int g = 0; g < GROUPS; ++g) {
      // all of a head's cluster partials in flight together, then the weighted sum
      const long ph = ((long)b * p.hq + hq0 + g) * nclusters;
      float pa[16], pl[16];
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        pa[c] = c < nclusters ? __ldcg(&p.part_acc[(ph + c) * D + t]) : 0.f;
        pl[c] = c < nclusters ? __ldcg(&p.part_ml[(ph + c) * 2 + 1]) : 0.f;
      }
      float og = 0.f, lg = 0.f;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const float w = c < nclusters ? wgt[g * 16 + c] : 0.f;
        og = fmaf(w, pa[c], og);
        lg = fmaf(w, pl[c], lg);
      }
      o[g] = og, lt[g] = lg;
    }
  }

  // normalise, output gate (reference.py:558-568, :675-676), store
#pragma unroll
  for (int g = 0; g < GROUPS; ++g) {
    float y = round_bf16(o[g] / lt[g]);
    if (p.attn_output_gate) {
      const float gv = gate_v[g];
      const float gg = round_bf16(p.gate_swish ? silu_f(gv) : sigmoid_f(gv));
      y = round_bf16(__fmul_rn(y, gg));
    }
    p.out[(long)b * p.out_stride + (long)(hq0 + g) * D + t] = f2bf(y);
  }
  if (t == 0) trace_mark(p.trace, cta, 6);
}

template <int GROUPS>
size_t step_smem(int max_seq = MAX_KEYS, int splits = 1) {
  const int cap = std::max((max_seq + splits - 1) / splits, AW * GROUPS * 2);
  const int scp = (cap + 31) & ~31;
  const size_t stage = (size_t)2 * cap * D * 2;  // also holds the [AW][GROUPS][D] float warp-merge buffer
  const size_t merge = (size_t)AW * GROUPS * D * 4;
  return std::max(stage, merge) +
         (size_t)(GROUPS * D + 2 * D + 2 * GROUPS * scp + MAX_CS * GROUPS * D + MAX_CS * GROUPS * 2 + GROUPS * 16 + 32 + GROUPS * 2) * 4 + 16 + 128;
}

template <int GROUPS>
int launch_groups(const AttnStepParams& p, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(p.splits, p.hkv, p.batch);
  cfg.blockDim = dim3(AW * 32, 1, 1);
  cfg.dynamicSmemBytes = step_smem<GROUPS>(p.max_seq, p.splits);
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = p.cluster_size;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, attn_step_kernel<GROUPS>, p);
  if (e != cudaSuccess) {
    set_error("attention step: launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  return check_launch("attention step");
}

}  // namespace

// The fused kernel takes head_dim 256, 1/2/4 query heads per KV head, a power-of-two number of slices
// (at most 16 clusters of 8) and at most 160 keys per slice at the cache's capacity.
bool attn_step_ok(int d, int hq, int hkv, int rotary_dim, int splits, int max_seq) {
  if (d != D || hkv < 1 || hq % hkv) return false;
  const int groups = hq / hkv;
  if (!(groups == 1 || groups == 2 || groups == 4)) return false;
  if (rotary_dim % 2 || rotary_dim > D || rotary_dim < 2) return false;
  if (splits < 1 || (splits & (splits - 1)) || splits > MAX_CS * 16) return false;
  return (max_seq + splits - 1) / splits <= MAX_KEYS;
}

int attn_step_configure() {
  cudaError_t e = cudaFuncSetAttribute(attn_step_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)step_smem<1>());
  if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_step_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)step_smem<2>());
  if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_step_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)step_smem<4>());
  if (e == cudaSuccess) e = prefer_max_shared(attn_step_kernel<1>);
  if (e == cudaSuccess) e = prefer_max_shared(attn_step_kernel<2>);
  if (e == cudaSuccess) e = prefer_max_shared(attn_step_kernel<4>);
  return e == cudaSuccess ? 0 : check_launch("attention step: shared-memory opt-in");
}

int launch_attn_step(const AttnStepParams& p, cudaStream_t stream) {
  if (p.batch <= 0) return 0;
  if (!attn_step_ok(p.d, p.hq, p.hkv, p.rotary_dim, p.splits, p.max_seq)) {
    set_error("attention step: unsupported shape (d=%d, hq=%d, hkv=%d, rotary=%d, splits=%d, max_seq=%d)", p.d, p.hq, p.hkv,
              p.rotary_dim, p.splits, p.max_seq);
    return 2;
  }
  if (p.cluster_size < 1 || p.cluster_size > MAX_CS || p.splits % p.cluster_size || p.splits / p.cluster_size > 16) {
    // the last merge keeps one weight per cluster in a 16-entry row of shared memory
    set_error("attention step: %d slices in clusters of %d: need a divisor of at most 8 and at most 16 clusters", p.splits,
              p.cluster_size);
    return 2;
  }
  if (p.splits > p.cluster_size && (!p.part_acc || !p.part_ml || !p.counters)) {
    set_error("attention step: scratch is required to merge %d slices", p.splits);
    return 2;
  }
  switch (p.hq / p.hkv) {
    case 1: return launch_groups<1>(p, stream);
    case 2: return launch_groups<2>(p, stream);
    default: return launch_groups<4>(p, stream);
  }
}

}  // namespace dfb
