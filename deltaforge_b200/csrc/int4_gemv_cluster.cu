// Cluster int4 dequant-GEMV for the per-layer projections of batch-1 decode, sm_100a.
//
// Same function, arithmetic and re-packed weight layout as int4_gemv_stream.cu (the reference's
// group-128 int4 linear, op deltaforge::tiled_gemv_int4, src/deltaforge/kernels/tiled_gemv.py:915-958),
// shaped for matrices of 5 to 25 MB, where the time of a launch is its chain of dependent latencies,
// not its bytes:
//
//  * One thread-block cluster per column tile (256 or 128 columns); the CTAs of the cluster split
//    the tile's 128-row scale groups between them. Each CTA issues the TMA copies of ALL its units
//    (weight words and the group's scale row) at once, before it waits for the previous kernel of
//    the stream (griddepcontrol.wait): there is no ring to recycle, and under programmatic dependent
//    launch the whole matrix is already in shared memory or in flight when the activation arrives.
//  * After the wait: the activation slice of the CTA's groups is quantised to 16-bit integers with a
//    per-group exponent (see int4_gemv_stream.cu), every thread runs four dp4a per 8 nibbles over
//    its 4 columns and its share of the rows, row lanes are added through shared memory, and the
//    CTAs of the cluster hand their column sums to the cluster's first CTA through distributed
//    shared memory. One hardware cluster barrier later that CTA adds them in rank order and applies
//    the epilogue. No global scratch, no atomics, no grid-wide dependency: results are identical run
//    to run.
//
// The wait on each TMA barrier is bounded (about two seconds); a CTA whose wait gives up records a
// code in the status word and still takes part in the cluster barrier, so its cluster never hangs.
//
// Bytes per launch: K*N/2 (words) + K/128*N scale bytes + N*2 output.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>

#include "gemv_common.cuh"

namespace dfb {

namespace {

constexpr int UROWS = 16;      // word rows per unit = one 128-row scale group
constexpr int MAX_CS = 8;      // portable cluster size limit
constexpr long long WAIT_LIMIT_CYCLES = 4000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
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
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar, uint64_t pol) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3}], [%4], %5;"
      ::"r"(smem_u32(dst)), "l"((uint64_t)map), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(pol)
      : "memory");
}
template <int CT>
__device__ __forceinline__ void consumer_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(CT) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// store a float into the shared memory of CTA `rank` of this cluster, at the address `local` has here
__device__ __forceinline__ void dsmem_store(float* local, uint32_t rank, float v) {
  uint32_t remote;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
  asm("dp4a.u32.s32 %0, %1, %2, %0;" : "+r"(c) : "r"(a), "r"(b));
  return c;
}
__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c) {
  asm("dp4a.u32.u32 %0, %1, %2, %0;" : "+r"(c) : "r"(a), "r"(b));
  return c;
}

// Epilogue for column `tile * TNW + t` by the TNW threads that hold the tile's final sums; optionally
// leaves the tile's sum of squares (of the values stored) for the next kernel's RMSNorm.
template <int TNW>
__device__ __forceinline__ void finish_tile(const GemvParams& p, int tile, int t, float v, float* wred, const EpiPre& pre) {
  const int n = tile * TNW + t;
  const float stored = n < p.N ? epilogue_store_pre(p, 0, n, v, pre) : 0.f;
  if (p.ss_out == nullptr) return;
  const float sq = warp_sum(stored * stored);
  if ((t & 31) == 0) wred[t >> 5] = sq;
  asm volatile("bar.sync 2, %0;" ::"n"(TNW) : "memory");
  if (t == 0) {
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < TNW / 32; ++w) tot += wred[w];
    p.ss_out[tile] = tot;
  }
  asm volatile("bar.sync 2, %0;" ::"n"(TNW) : "memory");  // wred is written again by the next tile of this CTA
}

struct ClusterArgs {
  GemvParams p;
  int cs;         // cluster size = CTAs that share the rows of a column tile
  int max_units;  // most groups any CTA of a cluster gets
  int tpc;        // column tiles a cluster works through, one after the other
  int num_tiles;  // ceil(N / TNW)
  int stages;     // ring depth in units (>= max_units when tpc == 1: nothing is recycled then)
  int* status;
};

constexpr int MAX_TPC = 4;

// TNW: columns per tile. CW: consumer warps (8 or 16); one more warp issues the copies.
template <int TNW, int CW>
__global__ void __launch_bounds__(CW * 32 + 32) gemv_cluster_kernel(const __grid_constant__ CUtensorMap wmap,
                                                                    const __grid_constant__ CUtensorMap smap, const ClusterArgs a) {
  constexpr int CT = CW * 32;          // consumer threads
  constexpr int CQ = TNW / 4;          // column quads per tile
  constexpr int RL = CT / CQ;          // row lanes
  constexpr int RPT = UROWS / RL;      // word rows per thread per unit
  static_assert(RL >= 1 && RPT >= 1 && RL * RPT == UROWS, "thread layout must tile a unit");
  constexpr int W_BYTES = UROWS * TNW * 4;
  constexpr int STAGE = W_BYTES + TNW * 4;  // + one scale row (fp32 size; bf16 uses half of it)
  extern __shared__ unsigned char smem_raw[];
  const GemvParams& p = a.p;
  const int G = p.K / 128;
  unsigned char* ring = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);  // stages * STAGE
  unsigned char* xq = ring + (size_t)a.stages * STAGE;             // [max_units*16][16] activation bytes for dp4a
  int* mk = (int*)(xq + (size_t)a.max_units * UROWS * 16);         // [max_units*16] sum of m per word row
  float* fg = (float*)(mk + a.max_units * UROWS);                  // [max_units] 2^e per group
  float* red = fg + ((a.max_units + 3) & ~3);                      // [RL][TNW] row-lane partials
  float* dsm = red + RL * TNW;                                     // [tpc][cs][TNW] column sums from every rank (used in rank 0)
  uint64_t* full = (uint64_t*)(dsm + a.tpc * a.cs * TNW);          // [stages]
  uint64_t* empty = full + a.stages;                               // [stages]
  float* wred = (float*)(empty + a.stages);                        // [16]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
  const int cs = a.cs;
  const int rank = (int)cluster_rank();
  const int cluster = blockIdx.x / cs;
  // Under the SwiGLU epilogue (TNW = 256) a tile is 128 gate_proj columns and the 128 up_proj columns of the same
  // channels, half the matrix further on: two boxes of 128 columns per unit, each laid out [16 rows][128 columns].
  const bool swiglu = p.epilogue == EPI_SWIGLU;
  const int tile0 = cluster * a.tpc;
  const int ntiles = min(a.tpc, a.num_tiles - tile0);  // >= 1: the grid holds no empty cluster
  const int g0 = (int)((long)rank * G / cs), g1 = (int)((long)(rank + 1) * G / cs);
  const int nunits = g1 - g0;
  const int total = ntiles * nunits;
  const uint32_t scale_bytes = p.scale_bf16 ? TNW * 2 : TNW * 4;
  const int cta = blockIdx.x;

  if (t == 0) {
    trace_mark(p.trace, cta, 0);
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], CW);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  bool ok = true;
  EpiPre pre = {};  // epilogue inputs of the cluster's first tile (later tiles of a folded grid load theirs at the end)
  if (warp == CW) {
    // producer: the weights never depend on earlier kernels, so the ring is filled at once; units beyond the
    // ring's depth (several tiles per cluster) follow as the consumers hand stages back
    if (lane == 0) {
      const uint64_t pol = make_evict_first_policy();
      int st = 0, round = 0, i = 0, s = 0;
      for (int j = 0; j < total; ++j) {
        if (round > 0 && !mbar_wait(&empty[st], (round - 1) & 1)) {
          atomicExch(a.status, 6);
          break;
        }
        unsigned char* dst = ring + (size_t)st * STAGE;
        mbar_expect_tx(&full[st], W_BYTES + scale_bytes);
        if (swiglu) {
          const int cg = (tile0 + i) * (TNW / 2), cu = p.N / 2 + cg;
          tma_load_2d(dst, &wmap, cg, (g0 + s) * UROWS, &full[st], pol);
          tma_load_2d(dst + W_BYTES / 2, &wmap, cu, (g0 + s) * UROWS, &full[st], pol);
          tma_load_2d(dst + W_BYTES, &smap, cg, g0 + s, &full[st], pol);
          tma_load_2d(dst + W_BYTES + scale_bytes / 2, &smap, cu, g0 + s, &full[st], pol);
        } else {
          tma_load_2d(dst, &wmap, (tile0 + i) * TNW, (g0 + s) * UROWS, &full[st], pol);
          tma_load_2d(dst + W_BYTES, &smap, (tile0 + i) * TNW, g0 + s, &full[st], pol);
        }
        if (++s == nunits) s = 0, ++i;
        if (++st == a.stages) st = 0, ++round;
        if (j + 1 == min(total, a.stages)) {
          // with this CTA's first copies queued, start the L2 on a slice of what a later GEMV of the step will read
#pragma unroll
          for (int q = 0; q < 2; ++q)
            if (p.pf_ptr[q] != nullptr)
              l2_prefetch_range(p.pf_ptr[q], p.pf_bytes[q] * (size_t)cta / gridDim.x, p.pf_bytes[q] * (size_t)(cta + 1) / gridDim.x);
          trace_mark(p.trace, cta, 7);
        }
      }
    }
    __syncwarp();  // the whole warp takes part in the (aligned) cluster barrier below
  } else {
    asm volatile("griddepcontrol.wait;" ::: "memory");  // the activation comes from the previous kernel
    if (t == 0) trace_mark(p.trace, cta, 1);
    // Everything this CTA reads that an earlier kernel wrote goes in flight at once: the activation values of
    // the first group each warp quantises, and what the epilogue adds to (rank 0 finishes the tiles).
    uint2 xraw = make_uint2(0u, 0u), wraw = make_uint2(0u, 0u);
    if (warp < nunits && p.prologue != PRO_ATTN_MERGE) {
      const int k = (g0 + warp) * 128 + lane * 4;
      xraw = *(const uint2*)(p.x + k);
      if (p.prologue == PRO_RMSNORM) wraw = *(const uint2*)(p.norm_w + k);
      if (p.prologue == PRO_SILU_MUL) wraw = *(const uint2*)(p.up + k);
    }
    if ((cs == 1 || rank == 0) && !swiglu && t < TNW && tile0 * TNW + t < p.N) pre = epilogue_preload(p, 0, tile0 * TNW + t);
    float rstd = 1.f;
    if (p.prologue == PRO_RMSNORM) {
      float tot = 0.f;
      if (p.ss_in) {  // the kernel that wrote x left the sums of squares of its tiles
        for (int i = 0; i < p.ss_count; ++i) tot += p.ss_in[i];
      } else {
        float ss = 0.f;
        for (int k = t; k < p.K; k += CT) {
          const float v = bf2f(p.x[k]);
          ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) wred[warp] = ss;
        consumer_sync<CT>();
#pragma unroll
        for (int w = 0; w < CW; ++w) tot += wred[w];
      }
      rstd = rsqrt_2step(__fadd_rn(__fdiv_rn(tot, (float)p.K), p.eps));
    }
    // one warp per group of this CTA: shared exponent, 16-bit integers, bytes laid out for dp4a
    for (int gl = warp; gl < nunits; gl += CW) {
      const int g = g0 + gl;
      float v[4];
      float amax = 0.f;
      if (gl != warp && p.prologue != PRO_ATTN_MERGE) {  // later groups of this warp (the first one's values are already here)
        const int k = g * 128 + lane * 4;
        xraw = *(const uint2*)(p.x + k);
        if (p.prologue == PRO_RMSNORM) wraw = *(const uint2*)(p.norm_w + k);
        if (p.prologue == PRO_SILU_MUL) wraw = *(const uint2*)(p.up + k);
      }
      const float xr[4] = {__uint_as_float(xraw.x << 16), __uint_as_float(xraw.x & 0xffff0000u), __uint_as_float(xraw.y << 16),
                           __uint_as_float(xraw.y & 0xffff0000u)};
      const float wr[4] = {__uint_as_float(wraw.x << 16), __uint_as_float(wraw.x & 0xffff0000u), __uint_as_float(wraw.y << 16),
                           __uint_as_float(wraw.y & 0xffff0000u)};
      if (p.prologue == PRO_ATTN_MERGE) {
        attn_merge_values(p.merge, g * 128 + lane * 4, v);
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = prologue_apply(p.prologue, xr[i], wr[i], rstd);
      }
#pragma unroll
      for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fabsf(v[i]));
      amax = warp_max(amax);
      int E = amax > 0.f ? (int)((__float_as_uint(amax) >> 23) & 0xff) - 127 : 0;  // amax in [2^E, 2^(E+1))
      E = max(E, -100);
      const float up = __uint_as_float((uint32_t)(127 + 14 - E) << 23);  // 2^(14-E): |x| * up < 2^15
      if (lane == 0) fg[gl] = __uint_as_float((uint32_t)(127 - 14 + E) << 23);
      int msum = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int m = __float2int_rn(v[i] * up);
        msum += m;
        const int kl = lane * 4 + i, kb = kl >> 3, r = kl & 7;
        unsigned char* q = xq + (gl * UROWS + kb) * 16 + (r & 1) * 4 + (r >> 1);
        q[0] = (unsigned char)((m >> 8) & 0xff);
        q[8] = (unsigned char)(m & 0xff);
      }
      msum += __shfl_xor_sync(0xffffffffu, msum, 1);  // lanes 2j, 2j+1 share word row j of the group
      if ((lane & 1) == 0) mk[gl * UROWS + (lane >> 1)] = msum;
    }
    consumer_sync<CT>();
    if (t == 0) trace_mark(p.trace, cta, 2);

    const int rl = t / CQ, cq = t % CQ;
    // where this thread's four columns sit inside a stage: one [16][TNW] block, or (SwiGLU) two [16][TNW/2] blocks
    const int w_row = swiglu ? TNW * 2 : TNW * 4;
    const int w_off = swiglu ? (cq / (CQ / 2)) * (W_BYTES / 2) + (cq % (CQ / 2)) * 16 : cq * 16;
    const int s_quad = swiglu ? (cq / (CQ / 2)) * (CQ / 2) + (cq % (CQ / 2)) : cq;  // scale rows are [gate half | up half] too
    int st = 0, phase = 0;
    for (int i = 0; i < ntiles; ++i) {
      float tot[4] = {0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < nunits; ++s) {
        if (ok) ok = mbar_wait(&full[st], phase);
        if (ok) {
          if (!DFB_IN_BOUNDS(st < a.stages && s < a.max_units && i < a.tpc, a.status, 5)) break;
          const unsigned char* wbase = ring + (size_t)st * STAGE;
          // even rows of a word sit in the low nibbles of its bytes, odd rows in the high nibbles
          int acc_eh[4] = {0, 0, 0, 0}, acc_el[4] = {0, 0, 0, 0};
          int msum = 0;
#pragma unroll
          for (int r = 0; r < RPT; ++r) {
            const int kb = rl + RL * r;
            const uint4 xw = *(const uint4*)(xq + (s * UROWS + kb) * 16);
            const uint4 w4 = *(const uint4*)(wbase + kb * w_row + w_off);
            msum += mk[s * UROWS + kb];
            const uint32_t wv[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const uint32_t ne = wv[q] & 0x0F0F0F0Fu;
              const uint32_t no = (wv[q] >> 4) & 0x0F0F0F0Fu;
              acc_eh[q] = dp4a_us(ne, xw.x, acc_eh[q]);
              acc_eh[q] = dp4a_us(no, xw.y, acc_eh[q]);
              acc_el[q] = dp4a_uu(ne, xw.z, acc_el[q]);
              acc_el[q] = dp4a_uu(no, xw.w, acc_el[q]);
            }
          }
          float sc[4];
          if (p.scale_bf16) {
            const uint2 v = *(const uint2*)(wbase + W_BYTES + s_quad * 8);
            sc[0] = __uint_as_float(v.x << 16), sc[1] = __uint_as_float(v.x & 0xffff0000u);
            sc[2] = __uint_as_float(v.y << 16), sc[3] = __uint_as_float(v.y & 0xffff0000u);
          } else {
            const float4 v = *(const float4*)(wbase + W_BYTES + s_quad * 16);
            sc[0] = v.x, sc[1] = v.y, sc[2] = v.z, sc[3] = v.w;
          }
          const float f = fg[s];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int S = acc_eh[q] * 256 + acc_el[q] - 8 * msum;  // sum over this thread's rows of (nibble - 8) * m, exact
            tot[q] = fmaf((float)S * f, sc[q], tot[q]);
          }
          if (a.stages < total) {  // the stage goes back to the producer (only when units outnumber stages)
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[st]);
          }
        }
        if (++st == a.stages) st = 0, phase ^= 1;
      }
      if (t == 0 && i + 1 == ntiles) trace_mark(p.trace, cta, 3);
      // add the row lanes, then hand this CTA's column sums to rank 0
      if (i > 0) consumer_sync<CT>();  // the previous tile's row-lane sums have been read
      *(float4*)(red + rl * TNW + cq * 4) = make_float4(tot[0], tot[1], tot[2], tot[3]);
      consumer_sync<CT>();
      if (t < TNW) {
        float v = 0.f;
#pragma unroll
        for (int r = 0; r < RL; ++r) v += red[r * TNW + t];
        if (cs == 1 && !swiglu) {
          if (i > 0 && (tile0 + i) * TNW + t < p.N) pre = epilogue_preload(p, 0, (tile0 + i) * TNW + t);
          finish_tile<TNW>(p, tile0 + i, t, v, wred, pre);
        } else {
          dsmem_store(dsm + (i * cs + rank) * TNW + t, 0, v);
        }
      }
    }
    if (!ok && lane == 0) atomicExch(a.status, 4);
  }
  if (cs == 1 && !swiglu) {
    if (t == 0) trace_mark(p.trace, cta, 6);
    return;
  }
  if (cs > 1) cluster_barrier();  // every thread of every CTA of the cluster, the producer warps included
  else __syncthreads();
  if (t == 0) trace_mark(p.trace, cta, 5);
  if (swiglu) {
    // rank 0 holds, per tile, the gate_proj sums of TNW/2 channels (threads 0 .. TNW/2-1) and their up_proj sums (the
    // other half): bf16(silu(g)) * u, rounded as the reference's SwiGLUMLP rounds it (src/deltaforge/reference.py:692-693,
    // src/deltaforge/kernels/fused_swiglu.py:18-22)
    if (rank == 0 && t < TNW) {
      for (int i = 0; i < ntiles; ++i) {
        float v = 0.f;
        for (int r = 0; r < cs; ++r) v += dsm[(i * cs + r) * TNW + t];
        red[t] = v;
        asm volatile("bar.sync 2, %0;" ::"n"(TNW) : "memory");
        const int ch = (tile0 + i) * (TNW / 2) + t;
        if (t < TNW / 2 && ch < p.N / 2) {
          const float sv = round_bf16(silu_f(round_bf16(red[t])));
          p.out[ch] = f2bf(__fmul_rn(sv, round_bf16(red[t + TNW / 2])));
        }
        asm volatile("bar.sync 2, %0;" ::"n"(TNW) : "memory");
      }
    }
  } else if (rank == 0 && t < TNW) {
    for (int i = 0; i < ntiles; ++i) {
      float v = 0.f;
      for (int r = 0; r < cs; ++r) v += dsm[(i * cs + r) * TNW + t];
      if (i > 0 && (tile0 + i) * TNW + t < p.N) pre = epilogue_preload(p, 0, (tile0 + i) * TNW + t);
      finish_tile<TNW>(p, tile0 + i, t, v, wred, pre);
    }
  }
  if (t == 0) trace_mark(p.trace, cta, 6);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &ptr, 12000, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return nullptr;
    return (EncodeTiledFn)ptr;
  }();
  return fn;
}

int pick_cs(int K) {
  const int G = K / 128;
  // Measured on B200: with K = 2560 (20 groups) clusters of 4 with 5 groups per CTA beat clusters of 8
  // (fewer CTAs repeat the prologue, smaller clusters are scheduled sooner); the deeper matrices
  // (K = 4096, 9216) need 8 CTAs per tile to keep a CTA's units within shared memory and the SMs busy.
  if (G <= 24) return std::max(1, std::min(MAX_CS, (G + 2) / 5));
  return MAX_CS;
}

// How a GEMV is cut: clusters of `cs` CTAs share the rows of a tile; a grid that would not be resident in one
// go (more CTAs than about one and a half per SM: its second wave would start only when the first leaves) is
// folded so that every cluster works through `tpc` tiles, its CTAs recycling a ring of `stages` units.
struct ClusterPlan {
  int cs, max_units, tiles, tpc, clusters, stages, cw;
  size_t smem;
};

// Measured on the full-size decode step: sixteen consumer warps cost the second resident CTA per SM (registers) and
// ran a third slower; grids above one and a half CTAs per SM are folded; a ring of about 125 KB (seven 256-column
// stages) was the fastest depth for the folded grids.
constexpr int CONSUMER_WARPS = 8;
constexpr int FOLD_ABOVE_CTAS = 222;
constexpr int RING_BYTES = 125 << 10;
constexpr int MIN_STAGES = 5;
constexpr int SWIGLU_CLUSTER = 2;

template <int TNW>
ClusterPlan plan_cluster(int K, int N, bool swiglu) {
  ClusterPlan c = {};
  const int G = K / 128;
  c.cs = pick_cs(K);
  c.tiles = (N + TNW - 1) / TNW;
  if (swiglu) {
    // a tile pairs TNW/2 gate columns with their up columns; small clusters place well (the CTAs of a cluster must sit
    // in one GPC, and GPCs of 18 or 20 SMs hold only 34 clusters of four single-CTA-per-SM blocks but 74 of two)
    c.cs = std::min(c.cs, SWIGLU_CLUSTER);
    c.tiles = (N / 2 + TNW / 2 - 1) / (TNW / 2);
  }
  c.max_units = (G + c.cs - 1) / c.cs;
  c.cw = CONSUMER_WARPS;
  const int sms = 148;
  const int ctas = c.tiles * c.cs;
  c.tpc = ctas > FOLD_ABOVE_CTAS ? std::min(MAX_TPC, (ctas + sms - 1) / sms) : 1;
  c.clusters = (c.tiles + c.tpc - 1) / c.tpc;
  const size_t stage = (size_t)UROWS * TNW * 4 + TNW * 4;
  // everything resident when it fits in about 100 KB (two CTAs per SM); a ring of stages the consumers recycle otherwise
  const int ring_cap = (int)((size_t)RING_BYTES / stage);
  c.stages = std::min(c.tpc * c.max_units, std::max(MIN_STAGES, ring_cap));
  const int rl = c.cw * 32 / (TNW / 4);
  c.smem = (size_t)c.stages * stage + (size_t)c.max_units * UROWS * 16 + (size_t)c.max_units * UROWS * 4 +
           (size_t)((c.max_units + 3) & ~3) * 4 + (size_t)rl * TNW * 4 + (size_t)c.tpc * c.cs * TNW * 4 + (size_t)c.stages * 16 + 64 + 128;
  return c;
}

template <int TNW, int CW>
int launch_cluster_cfg(const GemvParams& p, const ClusterPlan& c, const CUtensorMap& wmap, const CUtensorMap& smap, int* status,
                       cudaStream_t stream) {
  ClusterArgs a = {};
  a.p = p;
  a.cs = c.cs;
  a.max_units = c.max_units;
  a.tpc = c.tpc;
  a.num_tiles = c.tiles;
  a.stages = c.stages;
  a.status = status;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(c.clusters * c.cs, 1, 1);
  cfg.blockDim = dim3(CW * 32 + 32, 1, 1);
  cfg.dynamicSmemBytes = c.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = c.cs;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_cluster_kernel<TNW, CW>, wmap, smap, a);
  if (e != cudaSuccess) {
    set_error("int4 gemv (cluster): launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  return check_launch("int4 gemv (cluster)");
}

template <int TNW>
int launch_cluster_tnw(const GemvParams& p, int* status, cudaStream_t stream) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) {
    set_error("int4 gemv: cuTensorMapEncodeTiled is not available from this driver");
    return 1;
  }
  CUtensorMap wmap, smap;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)p.N, (cuuint64_t)(p.K / 8)};
    const cuuint64_t strides[1] = {(cuuint64_t)p.N * 4};
    const cuuint32_t box[2] = {(cuuint32_t)(p.epilogue == EPI_SWIGLU ? TNW / 2 : TNW), UROWS};
    const cuuint32_t es[2] = {1, 1};
    const CUresult r = enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, (void*)p.packed_k8, dims, strides, box, es,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      set_error("int4 gemv (cluster): tensor map for the re-packed weight failed (code %d)", (int)r);
      return 1;
    }
  }
  {
    const int esz = p.scale_bf16 ? 2 : 4;
    const cuuint64_t dims[2] = {(cuuint64_t)p.N, (cuuint64_t)(p.K / 128)};
    const cuuint64_t strides[1] = {(cuuint64_t)p.N * esz};
    const cuuint32_t box[2] = {(cuuint32_t)(p.epilogue == EPI_SWIGLU ? TNW / 2 : TNW), 1};
    const cuuint32_t es[2] = {1, 1};
    const CUresult r = enc(&smap, p.scale_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                           (void*)p.scale, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                           CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      set_error("int4 gemv (cluster): tensor map for the scales failed (code %d)", (int)r);
      return 1;
    }
  }
  const ClusterPlan c = plan_cluster<TNW>(p.K, p.N, p.epilogue == EPI_SWIGLU);
  return launch_cluster_cfg<TNW, CONSUMER_WARPS>(p, c, wmap, smap, status, stream);
}

}  // namespace

// Shapes the cluster kernel takes: the same preconditions as the streaming kernel, N a multiple of 4
// for 16-byte rows, and a per-CTA footprint that leaves room for several CTAs per SM.
bool cluster_path_ok(const GemvParams& p) {
  if (!(p.rows == 1 && p.packed_k8 != nullptr && p.group == 128 && p.K % 128 == 0 && p.N % 4 == 0 &&
        ((uintptr_t)p.packed_k8 % 16) == 0 && ((uintptr_t)p.scale % 16) == 0 && p.math == MATH_FAST &&
        ((uintptr_t)p.x % 8) == 0 && (p.prologue != PRO_RMSNORM || ((uintptr_t)p.norm_w % 8) == 0) &&
        (p.prologue != PRO_SILU_MUL || ((uintptr_t)p.up % 8) == 0) &&
        (p.prologue != PRO_ATTN_MERGE || (p.merge.acc && p.merge.ml && p.merge.nclusters >= 1 && p.merge.nclusters <= 8 &&
                                          p.merge.d % 128 == 0 && p.K % p.merge.d == 0 && ((uintptr_t)p.merge.acc % 16) == 0))))
    return false;
  const bool swiglu = p.epilogue == EPI_SWIGLU;
  const int tnw = cluster_tile_width(p.N);
  if (swiglu && (tnw != 256 || p.N % 8 != 0)) return false;  // pairs of 128-column boxes; both halves 16-byte aligned rows
  const ClusterPlan c = tnw == 256 ? plan_cluster<256>(p.K, p.N, swiglu) : plan_cluster<128>(p.K, p.N, swiglu);
  // one tile per cluster: small enough for two CTAs per SM; folded grids run one CTA per SM with a deeper ring
  return c.smem <= (size_t)132 * 1024;
}

int cluster_configure() {
  cudaError_t e = cudaSuccess;
  auto opt_in = [&e](auto kernel) {
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e == cudaSuccess) e = prefer_max_shared(kernel);
  };
  opt_in(gemv_cluster_kernel<256, CONSUMER_WARPS>);
  opt_in(gemv_cluster_kernel<128, CONSUMER_WARPS>);
  if (e != cudaSuccess) return check_launch("int4 gemv (cluster): shared-memory opt-in");
  return 0;
}

int cluster_tile_width(int N) { return N >= 4096 ? 256 : 128; }

int launch_gemv_cluster(const GemvParams& p, int* status, cudaStream_t stream) {
  if (p.N >= 4096) return launch_cluster_tnw<256>(p, status, stream);
  return launch_cluster_tnw<128>(p, status, stream);
}

}  // namespace dfb
