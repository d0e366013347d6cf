// The whole batch-1 decode step as ONE persistent kernel, sm_100a.
//
// Same arithmetic and the same reference lines as the launch sequence in decode_step.cu
// (ReferenceModel.forward at seq_len 1 plus greedy argmax, src/deltaforge/reference.py:779-817,
// src/deltaforge/model.py:141-147); what changes is how the 165 dependent operators of a token are
// scheduled. One CTA per SM stays resident for the whole token (cooperative launch). Each CTA owns a
// fixed slice of the OUTPUT COLUMNS of every int4 projection, over the full K, so no projection needs a
// cross-CTA reduction, and its slices of all projections are laid out at install time as one contiguous
// byte stream in consumption order (scales of a 128-row group, then the group's 16 word rows). A
// producer warp copies that stream through an 8-stage shared-memory ring with bulk asynchronous copies
// and mbarriers and never looks at activations, so the weights of the next operators are already on
// chip while the current operator waits for its input: the HBM stream does not stop at operator
// boundaries. The KV slice of an attention layer travels through the same ring.
//
// Activations cross CTAs through small global buffers of 8-byte words {payload, epoch}: a producer
// writes each word with one 64-bit store, a consumer polls the word until the epoch is the one of the
// producing phase of this token. Data and flag arrive together, so there is no grid barrier, no fence
// and no atomic anywhere; a phase costs one L2 round trip. Epochs grow with every launch, so a buffer
// never has to be cleared. Every poll and every mbarrier wait is bounded: on giving up the CTA records a
// code in the status word, stops consuming, drains its copies in flight and leaves.
//
// Integer GEMV arithmetic is the FAST mode of the other kernels (int16 block floating point activation
// per 128-row group, dp4a on the stored nibbles, zero point through the group's sum, fp32 scale once
// per group); all rounding points outside the GEMV are the reference's.
#include <algorithm>
#include <vector>

#include "../../include/dfb200.h"
#include "common.cuh"
#include "kernels.h"

namespace dfb {

namespace {

typedef unsigned long long u64;

constexpr int CT = 512;            // consumer threads
constexpr int CW = CT / 32;        // consumer warps
constexpr int THREADS = CT + 32;   // + one producer warp
constexpr int STAGE = 20480;       // bytes per ring stage
constexpr int NSTAGE = 8;
constexpr int MAXW = 128;          // widest column block of a projection slice
constexpr int KVU = 16;            // cached keys per ring unit (16 key rows + 16 value rows of 512 bytes)
constexpr int HD = 256;            // attention head dim
constexpr int MAXGQ = 4;           // query heads per KV head
constexpr int MAX_HIDDEN = 4096;
constexpr int MAX_K = 12288;
constexpr int DN_RPT = 128 / CW;   // DeltaNet state rows per thread (the warps split 128 key rows)
constexpr long long WAIT_CYCLES = 1LL << 28;  // ~0.14 s: far beyond any legitimate wait

enum { EPI_P = 0, EPI_CONV = 1, EPI_RES = 2, EPI_SWIGLU = 3, EPI_LOGITS = 4 };
enum { XB_RMS = 0, XB_LL = 1, XB_DN = 2 };

// ---------------------------------------------------------------------------------------------------
// Geometry shared by the host planner, the re-pack kernel, the producer and the consumers.
// ---------------------------------------------------------------------------------------------------

// First element (always even) of CTA c when `total` elements are dealt to P CTAs in pairs.
__host__ __device__ inline int split2(int total, int c, int P) { return 2 * (int)(((long long)(total / 2) * c) / P); }

struct Blocks {
  int nblk, bw;  // number of column blocks and the width of all but the last
};
__host__ __device__ inline Blocks blocks_of(int n, int maxw) {
  Blocks b;
  b.nblk = (n + maxw - 1) / maxw;
  b.bw = b.nblk ? 2 * ((n + 2 * b.nblk - 1) / (2 * b.nblk)) : 0;
  return b;
}
__host__ __device__ inline int group_bytes(int w, int sb) { return ((sb * w + 15) & ~15) + 64 * w; }

// One projection as the persistent kernel sees it. `paired`: N = 2 * items, item i is the pair
// (gate column i, up column items + i) and a CTA's slice keeps both, so SwiGLU happens in its epilogue.
struct ProjGeo {
  int K, N, paired;
};
__host__ __device__ inline int proj_items(const ProjGeo& g) { return g.paired ? g.N / 2 : g.N; }
// Bytes of CTA c's slice of the projection in the stream.
__host__ __device__ inline long long proj_chunk_bytes(const ProjGeo& g, int c, int P, int sb) {
  const int items = proj_items(g);
  const int n = split2(items, c + 1, P) - split2(items, c, P);
  const Blocks bl = blocks_of(n, g.paired ? MAXW / 2 : MAXW);
  long long bytes = 0;
  for (int b = 0; b < bl.nblk; ++b) {
    const int nb = min(bl.bw, n - b * bl.bw);
    if (nb <= 0) break;
    bytes += (long long)(g.K / 128) * group_bytes(g.paired ? 2 * nb : nb, sb);
  }
  return bytes;
}

// A CTA's slice of a projection: first item, item count, column blocks.
struct SliceGeo {
  int items, paired, i0, n, nblk, bw;
};
__host__ __device__ inline SliceGeo slice_geo(int items, int paired, int c, int P) {
  SliceGeo s;
  s.items = items, s.paired = paired;
  s.i0 = split2(items, c, P);
  s.n = split2(items, c + 1, P) - s.i0;
  const Blocks bl = blocks_of(s.n, paired ? MAXW / 2 : MAXW);
  s.nblk = bl.nblk, s.bw = bl.bw;
  return s;
}
constexpr int NGEO = 6;

struct PLayerDev {
  int kind;
  const bf16* in_norm;
  const bf16* post_norm;
  const bf16* conv_w;
  bf16* conv_state;
  const float* a_log;
  const float* dt_bias;
  const float* gnorm_w;
  int gnorm_bf16;
  float* recurrent;
  const bf16* q_norm;
  const bf16* k_norm;
  bf16* kcache;
  bf16* vcache;
  int in_n;  // columns of the fused input projection
};

struct PParams {
  int P;
  int hidden, inter, vocab, layers, max_seq;
  int hq, hkv, rd, gate, gate_swish;
  int hk_lin, hv_lin, dk, dv;
  float eps;
  int sb;  // bytes per scale
  const float* inv_freq;
  const bf16* embed;
  const bf16* final_norm;
  const PLayerDev* L;
  const unsigned char* const* stream_base;  // [P]
  int64_t* tokens;
  int64_t* history;
  int* pos;
  bf16* logits;
  u64 *H, *Pb, *O, *A, *SSQ, *AP, *ARG;
  unsigned* launch_counter;
  int* status;
  long long* trace;  // optional [P][32] device timestamps (ns) of the phases of layer trace_layer, or null
  int trace_layer;
};

// ---------------------------------------------------------------------------------------------------
// Device helpers
// ---------------------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CT) : "memory"); }
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
  asm("dp4a.u32.s32 %0, %1, %2, %0;" : "+r"(c) : "r"(a), "r"(b));
  return c;
}
__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c) {
  asm("dp4a.u32.u32 %0, %1, %2, %0;" : "+r"(c) : "r"(a), "r"(b));
  return c;
}
__device__ __forceinline__ void mbar_init(u64* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(u64* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(u64* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(u64* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void bulk_copy(void* dst, const void* src, uint32_t bytes, u64* bar, uint64_t pol) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol)
      : "memory");
}
__device__ __forceinline__ void ll_store(u64* p, uint32_t payload, uint32_t epoch) {
  const u64 v = ((u64)epoch << 32) | payload;
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ u64 ll_peek(const u64* p) {
  u64 v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  return (uint32_t)__bfloat16_as_ushort(f2bf(a)) | ((uint32_t)__bfloat16_as_ushort(f2bf(b)) << 16);
}
__device__ __forceinline__ float lo_bf16(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float hi_bf16(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// Everything a consumer thread carries around.
struct Ctx {
  const PParams* p;
  int t, warp, lane, c;
  uint32_t base;  // epoch of phase 0 of this launch
  int pos;
  // shared memory
  unsigned char* ring;
  u64* full;
  u64* empty;
  uint4* xq;   // [K/8] activation bytes for dp4a: hi even rows, hi odd, lo even, lo odd
  int* mk;     // [K/8] sum of the eight integers of a word row
  float* fg;   // [K/128] 2^e of the group
  float* un;   // the same memory as xq..fg, as floats, for the attention merge
  float* h_s;  // [hidden] residual stream (bf16 values held as floats)
  float* q_s;  // [4][256] queries; DeltaNet: qn, kn
  float* rowbuf;  // [2][256]
  float* red;     // [1024]
  float* y_s;     // [128]
  float* wred;    // [16]
  volatile int* failed;
  const SliceGeo* geo_s;  // [NGEO] slices of the distinct projection shapes, filled at kernel start
  int it;  // ring units consumed so far
  int tslot;  // diagnostics: first trace slot for the marks inside the current projection phase, or 0
  long long w_ring, w_ll;  // cycles this thread spent waiting for the ring / for other CTAs (diagnostics)
};

__device__ __forceinline__ void mark(Ctx& cx, int idx) {
  if (cx.p->trace && cx.t == 0) {
    long long ns;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(ns));
    cx.p->trace[cx.c * 32 + idx] = ns;
  }
}

// The divisions behind a slice are done once per launch; later uses look the shape up.
__device__ __forceinline__ SliceGeo find_geo(const Ctx& cx, int items, int paired) {
#pragma unroll 1
  for (int i = 0; i < NGEO; ++i)
    if (cx.geo_s[i].items == items && cx.geo_s[i].paired == paired) return cx.geo_s[i];
  return slice_geo(items, paired, cx.c, cx.p->P);
}

__device__ __noinline__ void fail(Ctx& cx, int code) {
  *cx.failed = 1;
  atomicCAS(cx.p->status, 0, code);
}

// Bounded wait on a ring barrier.
__device__ __forceinline__ bool ring_wait(Ctx& cx, u64* bar, uint32_t parity, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*cx.failed) return false;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 128; ++i)
      if (mbar_try_wait(bar, parity)) {
        cx.w_ring += clock64() - t0;
        return true;
      }
    if (*cx.failed) return false;
    if (clock64() - t0 > WAIT_CYCLES) {
      fail(cx, code);
      return false;
    }
  }
}

// Poll one word until it carries `epoch`; 0 after a failure anywhere in the CTA.
__device__ __forceinline__ uint32_t ll_wait(Ctx& cx, const u64* p, uint32_t epoch) {
  u64 v = ll_peek(p);
  if ((uint32_t)(v >> 32) == epoch) return (uint32_t)v;
  if (*cx.failed) return 0u;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      v = ll_peek(p);
      if ((uint32_t)(v >> 32) == epoch) {
        cx.w_ll += clock64() - t0;
        return (uint32_t)v;
      }
      __nanosleep(20);
    }
    if (*cx.failed) return 0u;
    if (clock64() - t0 > WAIT_CYCLES) {
      fail(cx, 20);
      return 0u;
    }
  }
}
// Finish a poll that was started with ll_peek: `raw` is what the first load returned.
__device__ __forceinline__ uint32_t ll_finish(Ctx& cx, const u64* p, uint32_t epoch, u64 raw) {
  if ((uint32_t)(raw >> 32) == epoch) return (uint32_t)raw;
  return ll_wait(cx, p, epoch);
}
// Element `k` (bf16 payloads, two per word) of a buffer.
__device__ __forceinline__ float ll_bf16(Ctx& cx, const u64* buf, int k, uint32_t epoch) {
  const uint32_t w = ll_wait(cx, buf + (k >> 1), epoch);
  return (k & 1) ? hi_bf16(w) : lo_bf16(w);
}

__device__ __forceinline__ float block_sum(Ctx& cx, float v) {
  v = warp_sum(v);
  consumer_sync();  // wred may still be read from the previous use
  if (cx.lane == 0) cx.wred[cx.warp] = v;
  consumer_sync();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < CW; ++w) tot += cx.wred[w];
  return tot;
}

// ---------------------------------------------------------------------------------------------------
// Activation -> int16 block floating point for dp4a (one warp per 128-row group, 4 elements per lane)
// ---------------------------------------------------------------------------------------------------

struct XSrc {
  int kind;
  const bf16* norm_w;  // XB_RMS
  float rstd;          // XB_RMS
  const u64* buf;      // XB_LL / XB_DN: the activation
  uint32_t epoch;
  const u64* zbuf;  // XB_DN: gate logits (the projection buffer), first element z_off
  uint32_t zepoch;
  int z_off;
  const u64* ssq;
  const float* gnorm_w;
  int gnorm_bf16;
};

// KIND selects the source; NB = groups per warp whose loads are in flight together.
template <int KIND, int NB>
__device__ void build_x_t(Ctx& cx, const XSrc& s, int K) {
  const PParams& p = *cx.p;
  const int G = K >> 7;
  unsigned char* xq = (unsigned char*)cx.xq;
  for (int gb0 = cx.warp; gb0 < G; gb0 += CW * NB) {
    u64 ra[NB][2], rz[KIND == XB_DN ? NB : 1][2], rs[KIND == XB_DN ? NB : 1];
    uint2 nw[KIND == XB_RMS ? NB : 1];
#pragma unroll
    for (int j = 0; j < NB; ++j) {
      const int g = gb0 + j * CW;
      const int k = (g < G ? g : gb0) * 128 + cx.lane * 4;
      if (KIND == XB_RMS) {
        nw[j] = *(const uint2*)(s.norm_w + k);
        ra[j][0] = ra[j][1] = 0ull;
      } else {
        ra[j][0] = ll_peek(s.buf + (k >> 1));
        ra[j][1] = ll_peek(s.buf + (k >> 1) + 1);
        if (KIND == XB_DN) {
          rz[j][0] = ll_peek(s.zbuf + ((s.z_off + k) >> 1));
          rz[j][1] = ll_peek(s.zbuf + ((s.z_off + k) >> 1) + 1);
          rs[j] = cx.lane < p.dv / 32 ? ll_peek(s.ssq + (k / p.dv) * (p.dv / 32) + cx.lane) : 0ull;
        }
      }
    }
#pragma unroll
    for (int j = 0; j < NB; ++j) {
      const int g = gb0 + j * CW;
      if (g >= G) break;
      const int k = g * 128 + cx.lane * 4;
      float v[4];
      if (KIND == XB_RMS) {
        const float w[4] = {lo_bf16(nw[j].x), hi_bf16(nw[j].x), lo_bf16(nw[j].y), hi_bf16(nw[j].y)};
#pragma unroll
        for (int i = 0; i < 4; ++i) v[i] = round_bf16(__fmul_rn(__fmul_rn(cx.h_s[k + i], s.rstd), __fadd_rn(1.0f, w[i])));
      } else {
        const uint32_t a = ll_finish(cx, s.buf + (k >> 1), s.epoch, ra[j][0]), b = ll_finish(cx, s.buf + (k >> 1) + 1, s.epoch, ra[j][1]);
        v[0] = lo_bf16(a), v[1] = hi_bf16(a), v[2] = lo_bf16(b), v[3] = hi_bf16(b);
        if (KIND == XB_DN) {
          // Gated RMSNorm of the DeltaNet read-out (src/deltaforge/reference.py:115-121): the head's sum of
          // squares arrives as one partial per 32-column slab, lane i of the warp holds partial i.
          const int nvb = p.dv / 32;
          const float part = cx.lane < nvb ? __uint_as_float(ll_finish(cx, s.ssq + (k / p.dv) * nvb + cx.lane, s.epoch, rs[j])) : 0.f;
          float tot = 0.f;
          for (int i = 0; i < nvb; ++i) tot += __shfl_sync(0xffffffffu, part, i);
          const float rstd = rsqrt_2step(__fadd_rn(__fdiv_rn(tot, (float)p.dv), p.eps));
          const uint32_t za = ll_finish(cx, s.zbuf + ((s.z_off + k) >> 1), s.zepoch, rz[j][0]);
          const uint32_t zb = ll_finish(cx, s.zbuf + ((s.z_off + k) >> 1) + 1, s.zepoch, rz[j][1]);
          const float z[4] = {lo_bf16(za), hi_bf16(za), lo_bf16(zb), hi_bf16(zb)};
          const float4 gw = *(const float4*)(s.gnorm_w + (k % p.dv));  // dv % 4 == 0: the four share a head
          const float gwv[4] = {gw.x, gw.y, gw.z, gw.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float nrm = round_bf16(__fmul_rn(v[i], rstd));
            float y = __fmul_rn(gwv[i], nrm);
            if (s.gnorm_bf16) y = round_bf16(y);
            v[i] = round_bf16(__fmul_rn(y, silu_f(z[i])));
          }
        }
      }
      float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
      amax = warp_max(amax);
      // amax in [2^E, 2^(E+1)) -> |x| * 2^(14-E) < 2^15 (bf16 inputs: at most 32640)
      int E = amax > 0.f ? (int)((__float_as_uint(amax) >> 23) & 0xff) - 127 : 0;
      E = max(E, -100);
      const float up = __uint_as_float((uint32_t)(127 + 14 - E) << 23);
      if (cx.lane == 0) cx.fg[g] = __uint_as_float((uint32_t)(127 - 14 + E) << 23);
      int m[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) m[i] = __float2int_rn(v[i] * up);
      // lane's elements are rows 4*(lane&1) .. +3 of word row g*16 + lane/2: even rows to bytes 0..3 of
      // each half, odd rows to bytes 4..7; high bytes in the first 8 bytes, low bytes in the second 8
      const int kb = g * 16 + (cx.lane >> 1), h = (cx.lane & 1) * 2;
      unsigned char* q = xq + kb * 16;
      *(uint16_t*)(q + h) = (uint16_t)(((m[0] >> 8) & 0xff) | (((m[2] >> 8) & 0xff) << 8));
      *(uint16_t*)(q + 4 + h) = (uint16_t)(((m[1] >> 8) & 0xff) | (((m[3] >> 8) & 0xff) << 8));
      *(uint16_t*)(q + 8 + h) = (uint16_t)((m[0] & 0xff) | ((m[2] & 0xff) << 8));
      *(uint16_t*)(q + 12 + h) = (uint16_t)((m[1] & 0xff) | ((m[3] & 0xff) << 8));
      int msum = m[0] + m[1] + m[2] + m[3];
      msum += __shfl_xor_sync(0xffffffffu, msum, 1);
      if ((cx.lane & 1) == 0) cx.mk[kb] = msum;
    }
  }
  consumer_sync();
}

__device__ void build_x(Ctx& cx, const XSrc& s, int K) {
  if (s.kind == XB_RMS)
    build_x_t<XB_RMS, 2>(cx, s, K);
  else if (s.kind == XB_DN)
    build_x_t<XB_DN, 2>(cx, s, K);
  else
    build_x_t<XB_LL, MAX_K / 128 / CW>(cx, s, K);
}

// ---------------------------------------------------------------------------------------------------
// One column block of a projection slice: w columns (even, <= 128) over the full K, from the ring.
// Thread = (column pair, row lane); row lanes interleave over the unit's word rows. Result in y_s[w].
// ---------------------------------------------------------------------------------------------------

// RPG = word rows of a group per thread: 16 / RPG row lanes share a column pair.
template <int RPG>
__device__ __forceinline__ void gemv_units(Ctx& cx, int G, int w, int gb, int ssec, int gpu, int jp, int q, int glane, int GL,
                                           bool act, float& tot0, float& tot1) {
  constexpr int R = 16 / RPG;
  const int sb = cx.p->sb;
  for (int g0 = 0; g0 < G; g0 += gpu) {
    const int ng = min(gpu, G - g0);
    const int s = cx.it % NSTAGE;
    const bool ok = ring_wait(cx, &cx.full[s], (cx.it / NSTAGE) & 1, 10);
    if (ok && act) {
      const unsigned char* base = cx.ring + (size_t)s * STAGE;
#pragma unroll 1
      for (int gl = glane; gl < ng; gl += GL) {
        const unsigned char* gbase = base + gl * gb;
        const int kb0 = ((g0 + gl) << 4) + q;
        // all loads of the group first, then the arithmetic
        uint2 wv[RPG];
        uint4 xw[RPG];
        int ms = 0;
#pragma unroll
        for (int i = 0; i < RPG; ++i) {
          wv[i] = *(const uint2*)(gbase + ssec + ((q + R * i) * w + 2 * jp) * 4);
          xw[i] = cx.xq[kb0 + R * i];
          ms += cx.mk[kb0 + R * i];
        }
        float s0, s1;
        if (sb == 2) {
          const uint32_t sv = *(const uint32_t*)(gbase + 4 * jp);
          s0 = lo_bf16(sv), s1 = hi_bf16(sv);
        } else {
          const float2 sv = *(const float2*)(gbase + 8 * jp);
          s0 = sv.x, s1 = sv.y;
        }
        const float f = cx.fg[g0 + gl];
        int ah0 = 0, al0 = 0, ah1 = 0, al1 = 0;
#pragma unroll
        for (int i = 0; i < RPG; ++i) {
          const uint32_t e0 = wv[i].x & 0x0F0F0F0Fu, o0 = (wv[i].x >> 4) & 0x0F0F0F0Fu;
          const uint32_t e1 = wv[i].y & 0x0F0F0F0Fu, o1 = (wv[i].y >> 4) & 0x0F0F0F0Fu;
          ah0 = dp4a_us(e0, xw[i].x, ah0);
          ah1 = dp4a_us(e1, xw[i].x, ah1);
          al0 = dp4a_uu(e0, xw[i].z, al0);
          al1 = dp4a_uu(e1, xw[i].z, al1);
          ah0 = dp4a_us(o0, xw[i].y, ah0);
          ah1 = dp4a_us(o1, xw[i].y, ah1);
          al0 = dp4a_uu(o0, xw[i].w, al0);
          al1 = dp4a_uu(o1, xw[i].w, al1);
        }
        tot0 = fmaf((float)(ah0 * 256 + al0 - 8 * ms) * f, s0, tot0);
        tot1 = fmaf((float)(ah1 * 256 + al1 - 8 * ms) * f, s1, tot1);
      }
    }
    __syncwarp();
    if (ok && cx.lane == 0) mbar_arrive(&cx.empty[s]);
    ++cx.it;
  }
}

__device__ void gemv_block(Ctx& cx, int K, int w) {
  const int G = K >> 7;
  const int ssec = (cx.p->sb * w + 15) & ~15;
  const int gb = ssec + 64 * w;
  const int gpu = min(G, STAGE / gb);
  const int np = w >> 1;
  // 16, 8 or 4 row lanes per column pair (a power of two keeps the rows of a group per thread fixed); the
  // threads left over form further "group lanes" that take every GL-th group of a unit
  const int R = np <= 16 ? 16 : (np <= 32 ? 8 : 4);
  const int GL = CT / (np * R);  // >= 2, since np * R <= 256
  const int jp = cx.t % np, ql = cx.t / np;
  const int q = ql % R, glane = ql / R;
  const bool act = glane < GL;
  float tot0 = 0.f, tot1 = 0.f;
  if (R == 16)
    gemv_units<1>(cx, G, w, gb, ssec, gpu, jp, q, glane, GL, act, tot0, tot1);
  else if (R == 8)
    gemv_units<2>(cx, G, w, gb, ssec, gpu, jp, q, glane, GL, act, tot0, tot1);
  else
    gemv_units<4>(cx, G, w, gb, ssec, gpu, jp, q, glane, GL, act, tot0, tot1);
  if (cx.tslot) mark(cx, cx.tslot + 1);
  // (group lane, row lane) -> one value per column, summed in a fixed order
  if (act) {
    cx.red[ql * w + 2 * jp] = tot0;
    cx.red[ql * w + 2 * jp + 1] = tot1;
  }
  consumer_sync();
  if (cx.t < w) {
    float y = 0.f;
    for (int i = 0; i < GL * R; ++i) y += cx.red[i * w + cx.t];
    cx.y_s[cx.t] = y;
  }
  consumer_sync();
  if (cx.tslot) mark(cx, cx.tslot + 2);
}

struct ArgBest {
  float v;
  int i;
};
__device__ __forceinline__ void arg_merge(ArgBest& a, float v, int i) {
  if (v > a.v || (v == a.v && i < a.i)) a.v = v, a.i = i;
}

// 4-tap causal conv + SiLU on a fresh projection output (src/deltaforge/kernels/inline_causal_conv.py:111-129).
__device__ __forceinline__ float conv_silu(float h0, float h1, float h2, float xv, float w0, float w1, float w2, float w3) {
  float acc = __fmul_rn(h0, w0);
  acc = __fadd_rn(acc, __fmul_rn(h1, w1));
  acc = __fadd_rn(acc, __fmul_rn(h2, w2));
  acc = __fadd_rn(acc, __fmul_rn(xv, w3));
  return round_bf16(silu_f(round_bf16(acc)));
}

// A whole projection for this CTA: all its column blocks, each followed by its epilogue.
__device__ void gemv_phase(Ctx& cx, const ProjGeo& g, int epi, uint32_t epoch, const PLayerDev* L, ArgBest* best) {
  const PParams& p = *cx.p;
  const SliceGeo sg = find_geo(cx, proj_items(g), g.paired);
  const int n = sg.n;
  struct {
    int nblk, bw;
  } bl = {sg.nblk, sg.bw};
  for (int b = 0; b < bl.nblk; ++b) {
    const int nb = min(bl.bw, n - b * bl.bw);
    if (nb <= 0) break;
    const int first = sg.i0 + b * bl.bw;  // first item of the block
    const int w = g.paired ? 2 * nb : nb;
    const int e = cx.t;  // epilogue thread e owns items 2e, 2e+1 of the block
    const bool mine = 2 * e < nb;
    const int n0 = first + 2 * e;
    // Conv history and taps do not depend on this token: in flight before the weights are consumed.
    uint32_t st[3] = {0u, 0u, 0u};
    uint4 cw = make_uint4(0u, 0u, 0u, 0u);
    const int conv_dim = 2 * p.hk_lin * p.dk + p.hv_lin * p.dv;
    const bool conv = epi == EPI_CONV && mine && n0 < conv_dim;
    if (conv) {
      const uint32_t* sp = (const uint32_t*)(L->conv_state + (long)n0 * 3);
      st[0] = sp[0], st[1] = sp[1], st[2] = sp[2];
      cw = *(const uint4*)(L->conv_w + (long)n0 * 4);
    }
    if (cx.tslot) mark(cx, cx.tslot);
    gemv_block(cx, g.K, w);
    if (!mine || *cx.failed) continue;
    const float y0 = round_bf16(cx.y_s[2 * e]), y1 = round_bf16(cx.y_s[2 * e + 1]);
    if (epi == EPI_P) {
      ll_store(p.Pb + (n0 >> 1), pack_bf16(y0, y1), epoch);
    } else if (epi == EPI_CONV) {
      if (conv) {
        // history of column n0: bf16 [h0,h1,h2], of n0+1 the next three
        const float a0 = lo_bf16(st[0]), a1 = hi_bf16(st[0]), a2 = lo_bf16(st[1]);
        const float b0 = hi_bf16(st[1]), b1 = lo_bf16(st[2]), b2 = hi_bf16(st[2]);
        const float o0 = conv_silu(a0, a1, a2, y0, lo_bf16(cw.x), hi_bf16(cw.x), lo_bf16(cw.y), hi_bf16(cw.y));
        const float o1 = conv_silu(b0, b1, b2, y1, lo_bf16(cw.z), hi_bf16(cw.z), lo_bf16(cw.w), hi_bf16(cw.w));
        uint32_t* sp = (uint32_t*)(L->conv_state + (long)n0 * 3);
        sp[0] = pack_bf16(a1, a2);
        sp[1] = pack_bf16(y0, b1);
        sp[2] = pack_bf16(b2, y1);
        ll_store(p.Pb + (n0 >> 1), pack_bf16(o0, o1), epoch);
      } else {
        ll_store(p.Pb + (n0 >> 1), pack_bf16(y0, y1), epoch);
      }
    } else if (epi == EPI_RES) {
      const float h0 = round_bf16(__fadd_rn(cx.h_s[n0], y0)), h1 = round_bf16(__fadd_rn(cx.h_s[n0 + 1], y1));
      ll_store(p.H + (n0 >> 1), pack_bf16(h0, h1), epoch);
    } else if (epi == EPI_SWIGLU) {
      // src/deltaforge/reference.py:692-693 with the rounding of src/deltaforge/kernels/fused_swiglu.py:18-22
      const float u0 = round_bf16(cx.y_s[nb + 2 * e]), u1 = round_bf16(cx.y_s[nb + 2 * e + 1]);
      const float a0 = round_bf16(__fmul_rn(round_bf16(silu_f(y0)), u0));
      const float a1 = round_bf16(__fmul_rn(round_bf16(silu_f(y1)), u1));
      ll_store(p.A + (n0 >> 1), pack_bf16(a0, a1), epoch);
    } else {  // EPI_LOGITS
      *(uint32_t*)(p.logits + n0) = pack_bf16(y0, y1);
      arg_merge(*best, y0, n0);
      arg_merge(*best, y1, n0 + 1);
    }
  }
}

// Read the whole residual stream (written by every CTA) into shared memory; returns its sum of squares.
__device__ float gather_h(Ctx& cx, uint32_t epoch) {
  const PParams& p = *cx.p;
  constexpr int NW = MAX_HIDDEN / 2 / CT;  // words per thread, all in flight together
  const int nwords = p.hidden / 2;
  u64 raw[NW];
#pragma unroll
  for (int j = 0; j < NW; ++j) {
    const int i = cx.t + j * CT;
    raw[j] = i < nwords ? ll_peek(p.H + i) : 0ull;
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < NW; ++j) {
    const int i = cx.t + j * CT;
    if (i < nwords) {
      const uint32_t w = ll_finish(cx, p.H + i, epoch, raw[j]);
      const float a = lo_bf16(w), b = hi_bf16(w);
      cx.h_s[2 * i] = a;
      cx.h_s[2 * i + 1] = b;
      ss = fmaf(a, a, ss);
      ss = fmaf(b, b, ss);
    }
  }
  return block_sum(cx, ss);
}

// ---------------------------------------------------------------------------------------------------
// Gated DeltaNet recurrence for one 32-column slab of one value head (src/deltaforge/reference.py:407-461)
// ---------------------------------------------------------------------------------------------------

__device__ void deltanet_phase(Ctx& cx, const PLayerDev& L, uint32_t ep_p, uint32_t ep_o) {
  const PParams& p = *cx.p;
  const int nvb = p.dv / 32, dk = p.dk, dv = p.dv;
  const int kd = p.hk_lin * dk, vd = p.hv_lin * dv;
  float* qn = cx.q_s;
  float* kn = cx.q_s + 128;
  float* gates = cx.q_s + 256;
  for (int piece = cx.c; piece < p.hv_lin * nvb; piece += p.P) {
    const int hv = piece / nvb, vb = piece % nvb;
    const int hk = hv / (p.hv_lin / p.hk_lin);
    const int col = vb * 32 + cx.lane;
    // the state slab goes in flight first: it does not depend on this token's activations
    float* S = L.recurrent + (long)hv * dk * dv;
    float s[DN_RPT];
#pragma unroll
    for (int i = 0; i < DN_RPT; ++i) {
      const int k = cx.warp * DN_RPT + i;
      s[i] = k < dk ? __ldcs(S + (long)k * dv + col) : 0.f;
    }
    // first loads of every word this thread needs, so that their round trips overlap
    // threads 0..127 normalise the query, 128..255 the key; the rest only run the recurrence
    const bool is_k = cx.t >= 128;
    const int j = cx.t < 256 ? (is_k ? cx.t - 128 : cx.t) : dk;
    const int xe = (is_k ? kd : 0) + hk * dk + (j < dk ? j : 0);
    const int ve = 2 * kd + hv * dv + col, be = 2 * kd + 2 * vd + hv, ae = be + p.hv_lin;
    const u64 raw_x = ll_peek(p.Pb + (xe >> 1)), raw_v = ll_peek(p.Pb + (ve >> 1));
    u64 raw_b = 0ull, raw_a = 0ull;
    if (cx.t == 0) raw_b = ll_peek(p.Pb + (be >> 1)), raw_a = ll_peek(p.Pb + (ae >> 1));
    {
      float x = 0.f;
      if (j < dk) {
        const uint32_t w = ll_finish(cx, p.Pb + (xe >> 1), ep_p, raw_x);
        x = (xe & 1) ? hi_bf16(w) : lo_bf16(w);
      }
      const float ss = warp_sum(x * x);
      consumer_sync();
      if (cx.lane == 0) cx.wred[cx.warp] = ss;
      consumer_sync();
      float tot = 0.f;
      const int w0 = is_k ? 4 : 0;
#pragma unroll
      for (int w = 0; w < 4; ++w) tot += cx.wred[w0 + w];
      float xn = __fmul_rn(x, rsqrt_2step(__fadd_rn(tot, 1e-6f)));
      if (!is_k) xn = __fdiv_rn(xn, sqrtf((float)dk));
      if (j < dk) (is_k ? kn : qn)[j] = xn;
      if (cx.t == 0) {
        const uint32_t wb = ll_finish(cx, p.Pb + (be >> 1), ep_p, raw_b), wa = ll_finish(cx, p.Pb + (ae >> 1), ep_p, raw_a);
        const float bv = (be & 1) ? hi_bf16(wb) : lo_bf16(wb), av = (ae & 1) ? hi_bf16(wa) : lo_bf16(wa);
        const float beta = round_bf16(sigmoid_f(bv));
        const float g = __fmul_rn(-expf(L.a_log[hv]), softplus_f(__fadd_rn(av, L.dt_bias[hv])));
        gates[0] = beta;
        gates[1] = expf(g);
      }
    }
    const uint32_t wvv = ll_finish(cx, p.Pb + (ve >> 1), ep_p, raw_v);
    const float vval = (ve & 1) ? hi_bf16(wvv) : lo_bf16(wvv);
    consumer_sync();
    const float decay = gates[1], beta = gates[0];
    float r = 0.f;
#pragma unroll
    for (int i = 0; i < DN_RPT; ++i) {
      const int k = cx.warp * DN_RPT + i;
      s[i] = __fmul_rn(s[i], decay);
      if (k < dk) r = fmaf(s[i], kn[k], r);
    }
    cx.red[cx.warp * 32 + cx.lane] = r;
    consumer_sync();
    r = 0.f;
#pragma unroll
    for (int w = 0; w < CW; ++w) r += cx.red[w * 32 + cx.lane];
    const float delta = __fmul_rn(__fsub_rn(vval, r), beta);
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < DN_RPT; ++i) {
      const int k = cx.warp * DN_RPT + i;
      if (k < dk) {
        s[i] = __fadd_rn(s[i], __fmul_rn(kn[k], delta));
        o = fmaf(s[i], qn[k], o);
      }
    }
    cx.red[(CW + cx.warp) * 32 + cx.lane] = o;
    consumer_sync();
    o = 0.f;
#pragma unroll
    for (int w = 0; w < CW; ++w) o += cx.red[(CW + w) * 32 + cx.lane];
    if (!*cx.failed) {
#pragma unroll
      for (int i = 0; i < DN_RPT; ++i) {
        const int k = cx.warp * DN_RPT + i;
        if (k < dk) __stcs(S + (long)k * dv + col, s[i]);
      }
      if (cx.warp == 0) {
        const float ob = round_bf16(o);
        const float ss = warp_sum(ob * ob);
        const float nb = __shfl_down_sync(0xffffffffu, ob, 1);
        if ((cx.lane & 1) == 0) ll_store(p.O + ((hv * dv + col) >> 1), pack_bf16(ob, nb), ep_o);
        if (cx.lane == 0) ll_store(p.SSQ + hv * nvb + vb, __float_as_uint(ss), ep_o);
      }
    }
    consumer_sync();  // q_s, red are reused by the next piece
  }
}

// ---------------------------------------------------------------------------------------------------
// Gated GQA attention (src/deltaforge/reference.py:610-677): partial pass over a KV slice, then a merge
// ---------------------------------------------------------------------------------------------------

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = lo_bf16(w[i]);
    f[2 * i + 1] = hi_bf16(w[i]);
  }
}

// RMSNorm (1 + w) and partial RoPE of one 256-wide head row (elements src_elem.. of the projection buffer)
// by one warp, through `row`; the values are those a bf16 model holds (reference.py:92-96, :137-149).
__device__ __noinline__ void norm_rope_row(Ctx& cx, int src_elem, uint32_t epoch, const bf16* nw, float* row) {
  const PParams& p = *cx.p;
  const int lane = cx.lane, rd = p.rd;
  const float f0 = lane < rd / 2 ? p.inv_freq[lane] : 0.f;
  float x[8], w[8];
  const u64* src = p.Pb + ((src_elem + lane * 8) >> 1);
  u64 raw[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) raw[i] = ll_peek(src + i);
  unpack8(*(const uint4*)(nw + lane * 8), w);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t v = ll_finish(cx, src + i, epoch, raw[i]);
    x[2 * i] = lo_bf16(v), x[2 * i + 1] = hi_bf16(v);
  }
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) ss = fmaf(x[i], x[i], ss);
  ss = warp_sum(ss);
  const float rstd = rsqrt_2step(__fadd_rn(__fdiv_rn(ss, (float)HD), p.eps));
#pragma unroll
  for (int i = 0; i < 8; ++i) row[lane * 8 + i] = round_bf16(__fmul_rn(__fmul_rn(x[i], rstd), __fadd_rn(1.0f, w[i])));
  __syncwarp();
  const int half = rd / 2;
#pragma unroll 1
  for (int d = lane; d < half; d += 32) {
    const float a = row[d], bb = row[d + half];
    const float ang = __fmul_rn((float)cx.pos, d == lane ? f0 : p.inv_freq[d]);
    float sn, cs;
    sincosf(ang, &sn, &cs);
    cs = round_bf16(cs), sn = round_bf16(sn);
    row[d] = round_bf16(__fadd_rn(round_bf16(__fmul_rn(a, cs)), round_bf16(__fmul_rn(-bb, sn))));
    row[d + half] = round_bf16(__fadd_rn(round_bf16(__fmul_rn(bb, cs)), round_bf16(__fmul_rn(a, sn))));
  }
  __syncwarp();
}

struct KvSlice {
  int active, kvh, ci, nchunk, k_begin, n_old, owns_new;
};
__device__ __forceinline__ KvSlice kv_slice(const PParams& p, int c, int pos) {
  KvSlice s;
  s.nchunk = p.P / p.hkv;
  s.active = c < p.hkv * s.nchunk;
  s.kvh = c / s.nchunk;
  s.ci = c % s.nchunk;
  const int L = pos + 1;
  const int chunk = (L + s.nchunk - 1) / s.nchunk;
  s.k_begin = s.ci * chunk;
  const int k_end = min(L, s.k_begin + chunk);
  s.owns_new = s.active && (s.k_begin <= pos) && (pos < k_end);
  s.n_old = s.active ? max(0, (s.owns_new ? k_end - 1 : k_end) - s.k_begin) : 0;
  return s;
}

__device__ void attn_partial_phase(Ctx& cx, const PLayerDev& L, uint32_t ep_p, uint32_t ep_ap) {
  const PParams& p = *cx.p;
  const KvSlice sl = kv_slice(p, cx.c, cx.pos);
  if (!sl.active) return;
  const int GQ = p.hq / p.hkv;
  const int qw = p.gate ? 2 * HD : HD;
  const float scale = 1.0f / sqrtf((float)HD);
  const int lane = cx.lane, warp = cx.warp;
  float* newk = cx.rowbuf;
  float* newv = cx.rowbuf + HD;
  if (warp < GQ) {
    float* row = cx.q_s + warp * HD;
    norm_rope_row(cx, (sl.kvh * GQ + warp) * qw, ep_p, L.q_norm, row);
#pragma unroll
    for (int i = 0; i < 8; ++i) row[lane * 8 + i] *= scale;
  } else if (sl.owns_new && warp == GQ) {
    norm_rope_row(cx, p.hq * qw + sl.kvh * HD, ep_p, L.k_norm, newk);
    if (cx.pos < p.max_seq && !*cx.failed) {
      bf16* dst = L.kcache + ((long)sl.kvh * p.max_seq + cx.pos) * HD + lane * 8;
      uint4 o;
      o.x = pack_bf16(newk[lane * 8], newk[lane * 8 + 1]);
      o.y = pack_bf16(newk[lane * 8 + 2], newk[lane * 8 + 3]);
      o.z = pack_bf16(newk[lane * 8 + 4], newk[lane * 8 + 5]);
      o.w = pack_bf16(newk[lane * 8 + 6], newk[lane * 8 + 7]);
      *(uint4*)dst = o;
    }
  } else if (sl.owns_new && warp == GQ + 1) {
    const u64* src = p.Pb + ((p.hq * qw + (p.hkv + sl.kvh) * HD + lane * 8) >> 1);
    u64 raw[4];
    uint32_t v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) raw[i] = ll_peek(src + i);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = ll_finish(cx, src + i, ep_p, raw[i]);
#pragma unroll
    for (int i = 0; i < 4; ++i) newv[lane * 8 + 2 * i] = lo_bf16(v[i]), newv[lane * 8 + 2 * i + 1] = hi_bf16(v[i]);
    if (cx.pos < p.max_seq && !*cx.failed)
      *(uint4*)(L.vcache + ((long)sl.kvh * p.max_seq + cx.pos) * HD + lane * 8) = make_uint4(v[0], v[1], v[2], v[3]);
  }
  consumer_sync();

  // (the queries stay in shared memory: with 17 warps a thread has 96 registers)
  float m[MAXGQ], l[MAXGQ], acc[MAXGQ][8];
#pragma unroll
  for (int g = 0; g < MAXGQ; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
  }
  auto one_key = [&](const float (&kf)[8], const float (&vf)[8]) {
#pragma unroll
    for (int g = 0; g < MAXGQ; ++g) {
      if (g >= GQ) break;
      const float4 qa = *(const float4*)(cx.q_s + g * HD + lane * 8), qb = *(const float4*)(cx.q_s + g * HD + lane * 8 + 4);
      float s = qa.x * kf[0];
      s = fmaf(qa.y, kf[1], s), s = fmaf(qa.z, kf[2], s), s = fmaf(qa.w, kf[3], s);
      s = fmaf(qb.x, kf[4], s), s = fmaf(qb.y, kf[5], s), s = fmaf(qb.z, kf[6], s), s = fmaf(qb.w, kf[7], s);
      s = warp_sum(s);
      const float mn = fmaxf(m[g], s);
      const float corr = __expf(m[g] - mn), pe = __expf(s - mn);
      l[g] = l[g] * corr + pe;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[g][i] = acc[g][i] * corr + pe * vf[i];
      m[g] = mn;
    }
  };
  const int nunits = (sl.n_old + KVU - 1) / KVU;
  for (int u = 0; u < nunits; ++u) {
    const int n = min(KVU, sl.n_old - u * KVU);
    const int s = cx.it % NSTAGE;
    const bool ok = ring_wait(cx, &cx.full[s], (cx.it / NSTAGE) & 1, 11);
    if (ok) {
      const bf16* kst = (const bf16*)(cx.ring + (size_t)s * STAGE);
      const bf16* vst = kst + KVU * HD;
      // one key per warp per unit
      if (warp < n) {
        float kf[8], vf[8];
        unpack8(*(const uint4*)(kst + warp * HD + lane * 8), kf);
        unpack8(*(const uint4*)(vst + warp * HD + lane * 8), vf);
        one_key(kf, vf);
      }
    }
    __syncwarp();
    if (ok && lane == 0) mbar_arrive(&cx.empty[s]);
    ++cx.it;
  }
  if (sl.owns_new && warp == 0) {
    float kf[8], vf[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) kf[i] = newk[lane * 8 + i], vf[i] = newv[lane * 8 + i];
    one_key(kf, vf);
  }
  // Merge the warps in two rounds through 32 KB of shared memory: warps 8..15 hand their partial to warps
  // 0..7, then thread (dim, half) merges the remaining eight for the query heads of its half.
  float* acc_s = cx.un;                          // [8][MAXGQ][HD]
  float* ml_s = cx.un + (CW / 2) * MAXGQ * HD;   // [8][MAXGQ][2]
  const int wl = warp & (CW / 2 - 1);
  if (warp >= CW / 2) {
#pragma unroll
    for (int g = 0; g < MAXGQ; ++g) {
      if (g >= GQ) break;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc_s[(wl * MAXGQ + g) * HD + lane * 8 + i] = acc[g][i];
      if (lane == 0) {
        ml_s[(wl * MAXGQ + g) * 2] = m[g];
        ml_s[(wl * MAXGQ + g) * 2 + 1] = l[g];
      }
    }
  }
  consumer_sync();
  if (warp < CW / 2) {
#pragma unroll
    for (int g = 0; g < MAXGQ; ++g) {
      if (g >= GQ) break;
      const float m2 = ml_s[(wl * MAXGQ + g) * 2], l2 = ml_s[(wl * MAXGQ + g) * 2 + 1];
      const float mn = fmaxf(m[g], m2);
      const float c1 = (m[g] == -INFINITY) ? 0.f : __expf(m[g] - mn), c2 = (m2 == -INFINITY) ? 0.f : __expf(m2 - mn);
      l[g] = l[g] * c1 + l2 * c2;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[g][i] = acc[g][i] * c1 + acc_s[(wl * MAXGQ + g) * HD + lane * 8 + i] * c2;
      m[g] = mn;
    }
  }
  consumer_sync();
  if (warp < CW / 2) {
#pragma unroll
    for (int g = 0; g < MAXGQ; ++g) {
      if (g >= GQ) break;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc_s[(wl * MAXGQ + g) * HD + lane * 8 + i] = acc[g][i];
      if (lane == 0) {
        ml_s[(wl * MAXGQ + g) * 2] = m[g];
        ml_s[(wl * MAXGQ + g) * 2 + 1] = l[g];
      }
    }
  }
  consumer_sync();
  if (!*cx.failed) {
    const int d = cx.t & (HD - 1), half = cx.t >> 8;  // CT == 2 * HD
    for (int g = half; g < GQ; g += 2) {
      float mg = -INFINITY;
#pragma unroll
      for (int w = 0; w < CW / 2; ++w) mg = fmaxf(mg, ml_s[(w * MAXGQ + g) * 2]);
      float lg = 0.f, og = 0.f;
#pragma unroll
      for (int w = 0; w < CW / 2; ++w) {
        const float mw = ml_s[(w * MAXGQ + g) * 2];
        const float sc = (mw == -INFINITY) ? 0.f : __expf(mw - mg);
        lg += ml_s[(w * MAXGQ + g) * 2 + 1] * sc;
        og += acc_s[(w * MAXGQ + g) * HD + d] * sc;
      }
      u64* dst = p.AP + ((long)(sl.kvh * GQ + g) * sl.nchunk + sl.ci) * (HD + 2);
      ll_store(dst + 2 + d, __float_as_uint(og), ep_ap);
      if (d == 0) {
        ll_store(dst, __float_as_uint(mg), ep_ap);
        ll_store(dst + 1, __float_as_uint(lg), ep_ap);
      }
    }
  }
  consumer_sync();  // the merge buffer aliases the activation bytes of the next projection
}

// Every CTA merges the partials of its slice of the hq*256 outputs, applies the output gate
// (src/deltaforge/reference.py:558-568, :675-676) and publishes the slice.
__device__ void attn_merge_phase(Ctx& cx, uint32_t ep_p, uint32_t ep_ap, uint32_t ep_o) {
  const PParams& p = *cx.p;
  const SliceGeo mg = find_geo(cx, p.hq * HD, 0);
  const int c0 = mg.i0, n = mg.n;
  const int nchunk = p.P / p.hkv;
  const int qw = p.gate ? 2 * HD : HD;
  const int cl = cx.t & 7;
  for (int b0 = 0; b0 < n; b0 += CT / 8) {
    const int ci_col = b0 + (cx.t >> 3);
    const bool mine = ci_col < n;
    const int col = c0 + (mine ? ci_col : 0);
    const int head = col / HD, d = col % HD;
    float mr = -INFINITY, lr = 0.f, orr = 0.f;
    if (mine) {
      for (int ch = cl; ch < nchunk; ch += 8) {
        const u64* src = p.AP + ((long)head * nchunk + ch) * (HD + 2);
        const float mc = __uint_as_float(ll_wait(cx, src, ep_ap));
        const float lc = __uint_as_float(ll_wait(cx, src + 1, ep_ap));
        const float oc = __uint_as_float(ll_wait(cx, src + 2 + d, ep_ap));
        const float mn = fmaxf(mr, mc);
        const float a = (mr == -INFINITY) ? 0.f : __expf(mr - mn);
        const float bsc = (mc == -INFINITY) ? 0.f : __expf(mc - mn);
        lr = lr * a + lc * bsc;
        orr = orr * a + oc * bsc;
        mr = mn;
      }
    }
    // the 8 chunk lanes of a column are 8 consecutive lanes of a warp
    float mg = mr;
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) mg = fmaxf(mg, __shfl_xor_sync(0xffffffffu, mg, o));
    const float sc = (mr == -INFINITY) ? 0.f : __expf(mr - mg);
    float lg = lr * sc, og = orr * sc;
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
      lg += __shfl_xor_sync(0xffffffffu, lg, o);
      og += __shfl_xor_sync(0xffffffffu, og, o);
    }
    float y = round_bf16(og / lg);
    if (p.gate && mine && cl == 0) {
      const float gv = ll_bf16(cx, p.Pb, head * qw + HD + d, ep_p);
      const float gg = round_bf16(p.gate_swish ? silu_f(gv) : sigmoid_f(gv));
      y = round_bf16(__fmul_rn(y, gg));
    }
    const float ynext = __shfl_down_sync(0xffffffffu, y, 8);  // the next column's result (its lane 0 of 8)
    if (mine && cl == 0 && (ci_col & 1) == 0 && !*cx.failed) ll_store(p.O + (col >> 1), pack_bf16(y, ynext), ep_o);
  }
}

// ---------------------------------------------------------------------------------------------------
// Producer warp (one lane): the weight stream and the KV slices, in consumption order
// ---------------------------------------------------------------------------------------------------

struct Prod {
  Ctx* cx;
  const unsigned char* ptr;
  int it;
  uint64_t pol;
  bool ok;
};
__device__ __forceinline__ bool prod_slot(Prod& pr, int& s) {
  s = pr.it % NSTAGE;
  if (pr.ok && pr.it >= NSTAGE) pr.ok = ring_wait(*pr.cx, &pr.cx->empty[s], ((pr.it / NSTAGE) - 1) & 1, 1);
  return pr.ok;
}
__device__ void produce_proj(Prod& pr, const ProjGeo& g) {
  const PParams& p = *pr.cx->p;
  const SliceGeo sg = find_geo(*pr.cx, proj_items(g), g.paired);
  const int n = sg.n;
  struct {
    int nblk, bw;
  } bl = {sg.nblk, sg.bw};
  const int G = g.K >> 7;
  for (int b = 0; b < bl.nblk; ++b) {
    const int nb = min(bl.bw, n - b * bl.bw);
    if (nb <= 0) break;
    const int gb = group_bytes(g.paired ? 2 * nb : nb, p.sb);
    const int gpu = min(G, STAGE / gb);
    for (int g0 = 0; g0 < G; g0 += gpu) {
      const uint32_t bytes = (uint32_t)(min(gpu, G - g0) * gb);
      int s;
      if (!prod_slot(pr, s)) return;
      mbar_expect_tx(&pr.cx->full[s], bytes);
      bulk_copy(pr.cx->ring + (size_t)s * STAGE, pr.ptr, bytes, &pr.cx->full[s], pr.pol);
      pr.ptr += bytes;
      ++pr.it;
    }
  }
}
__device__ void produce_kv(Prod& pr, const PLayerDev& L) {
  const PParams& p = *pr.cx->p;
  const KvSlice sl = kv_slice(p, pr.cx->c, pr.cx->pos);
  const int nunits = (sl.n_old + KVU - 1) / KVU;
  for (int u = 0; u < nunits; ++u) {
    const int n = min(KVU, sl.n_old - u * KVU);
    const long off = ((long)sl.kvh * p.max_seq + sl.k_begin + u * KVU) * HD;
    const uint32_t bytes = (uint32_t)n * HD * 2;
    int s;
    if (!prod_slot(pr, s)) return;
    unsigned char* dst = pr.cx->ring + (size_t)s * STAGE;
    mbar_expect_tx(&pr.cx->full[s], 2 * bytes);
    bulk_copy(dst, L.kcache + off, bytes, &pr.cx->full[s], pr.pol);
    bulk_copy(dst + KVU * HD * 2, L.vcache + off, bytes, &pr.cx->full[s], pr.pol);
    ++pr.it;
  }
}

__device__ __forceinline__ ProjGeo geo(int K, int N, int paired) {
  ProjGeo g;
  g.K = K, g.N = N, g.paired = paired;
  return g;
}

// ---------------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------------

__global__ void __launch_bounds__(THREADS, 1) pstep_kernel(const __grid_constant__ PParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);
  Ctx cx;
  cx.t = threadIdx.x;
  cx.warp = threadIdx.x >> 5;
  cx.lane = threadIdx.x & 31;
  cx.c = blockIdx.x;
  cx.ring = sm;
  unsigned char* q = sm + (size_t)NSTAGE * STAGE;
  cx.xq = (uint4*)q;
  cx.mk = (int*)(q + (size_t)(MAX_K / 8) * 16);
  cx.fg = (float*)(q + (size_t)(MAX_K / 8) * 20);
  cx.un = (float*)q;
  q += 33280;  // max(activation bytes: MAX_K/8*20 + MAX_K/128*4 = 31104, attention merge: 8*4*256*4 + 256 = 33024)
  cx.h_s = (float*)q;
  q += MAX_HIDDEN * 4;
  cx.q_s = (float*)q;
  q += MAXGQ * HD * 4;
  cx.rowbuf = (float*)q;
  q += 2 * HD * 4;
  cx.red = (float*)q;
  q += 1024 * 4;
  cx.y_s = (float*)q;
  q += MAXW * 4;
  cx.wred = (float*)q;
  q += 16 * 4;
  cx.full = (u64*)q;
  cx.empty = cx.full + NSTAGE;
  q += 2 * NSTAGE * 8;
  cx.failed = (volatile int*)q;
  q += 16;
  SliceGeo* geo_w = (SliceGeo*)q;
  cx.geo_s = geo_w;
  q += NGEO * sizeof(SliceGeo);
  // The parameters and the current layer's table entry are read through pointers by every phase: keep them
  // in shared memory (a generic-address read of a kernel parameter or of the table costs a memory round trip).
  PParams* sp = (PParams*)q;
  q += (sizeof(PParams) + 15) & ~15;
  PLayerDev* ls = (PLayerDev*)q;  // [2], the layer being computed and the next one
  cx.p = sp;
  cx.it = 0;
  cx.w_ring = cx.w_ll = 0;
  cx.tslot = 0;

  if (cx.t == 0) {
    for (int s = 0; s < NSTAGE; ++s) {
      mbar_init(&cx.full[s], 1);
      mbar_init(&cx.empty[s], CW);
    }
    *cx.failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (cx.t >= 32 && cx.t < 32 + (int)(sizeof(PParams) / 4)) ((uint32_t*)sp)[cx.t - 32] = ((const uint32_t*)&p)[cx.t - 32];
  if (cx.t >= 128 && cx.t < 128 + (int)(sizeof(PLayerDev) / 4) && p.layers > 0)
    ((uint32_t*)&ls[0])[cx.t - 128] = ((const uint32_t*)&p.L[0])[cx.t - 128];
  if (cx.t < NGEO) {
    // distinct projection shapes: the two kinds of input projection, hidden-wide outputs, gate|up, the head
    int items = 0, paired = 0;
    if (cx.t < 2) {
      for (int li = 0; li < p.layers; ++li)
        if (p.L[li].kind == cx.t) items = p.L[li].in_n;
    } else if (cx.t == 2) {
      items = p.hidden;
    } else if (cx.t == 3) {
      items = p.inter, paired = 1;
    } else if (cx.t == 4) {
      items = p.vocab;
    } else {
      items = p.hq * HD;  // the attention merge deals its outputs the same way
    }
    geo_w[cx.t] = slice_geo(items, paired, cx.c, p.P);
  }
  __syncthreads();
  cx.base = (*(volatile unsigned*)p.launch_counter) * 1024u;
  cx.pos = *(volatile int*)p.pos;
  const int conv_in_dn = 2 * p.hk_lin * p.dk + 2 * p.hv_lin * p.dv + 2 * p.hv_lin;
  const int attn_in = p.hq * HD * (p.gate ? 2 : 1) + 2 * p.hkv * HD;
  (void)conv_in_dn;
  (void)attn_in;

  if (cx.warp == CW) {
    // ---------------- producer ----------------
    if (cx.lane == 0) {
      Prod pr;
      pr.cx = &cx;
      pr.ptr = p.stream_base[cx.c];
      pr.it = 0;
      pr.pol = make_evict_first_policy();
      pr.ok = true;
      for (int li = 0; li < p.layers && pr.ok; ++li) {
        const PLayerDev& L = p.L[li];
        produce_proj(pr, geo(p.hidden, L.in_n, 0));
        if (L.kind == DFB_LAYER_ATTENTION) produce_kv(pr, L);
        produce_proj(pr, geo(L.kind == DFB_LAYER_ATTENTION ? p.hq * HD : p.hv_lin * p.dv, p.hidden, 0));
        produce_proj(pr, geo(p.hidden, 2 * p.inter, 1));
        produce_proj(pr, geo(p.inter, p.hidden, 0));
      }
      if (pr.ok) produce_proj(pr, geo(p.hidden, p.vocab, 0));
      // Do not leave while copies into this CTA's shared memory may still be in flight: wait (bounded) until
      // the last copy into every stage has landed.
      const int first = pr.it > NSTAGE ? pr.it - NSTAGE : 0;
      for (int i = first; i < pr.it; ++i) {
        const int s = i % NSTAGE;
        const long long t0 = clock64();
        while (!mbar_try_wait(&cx.full[s], (i / NSTAGE) & 1))
          if (clock64() - t0 > WAIT_CYCLES) {
            fail(cx, 2);
            break;
          }
      }
    }
    return;
  }

  // ---------------- consumers ----------------
  uint32_t seq = 0;
  uint32_t ep_h = 0;
  // token embedding (src/deltaforge/reference.py:804): every CTA holds the whole residual stream
  float ss;
  {
    const int64_t tok = p.tokens[0];
    float part = 0.f;
    for (int i = cx.t; i < p.hidden / 2; i += CT) {
      const uint32_t w = *(const uint32_t*)(p.embed + tok * p.hidden + 2 * i);
      const float a = lo_bf16(w), b = hi_bf16(w);
      cx.h_s[2 * i] = a, cx.h_s[2 * i + 1] = b;
      part = fmaf(a, a, part);
      part = fmaf(b, b, part);
    }
    ss = block_sum(cx, part);
  }
  XSrc xs;
  mark(cx, 0);
  for (int li = 0; li < p.layers; ++li) {
    const PLayerDev& L = ls[li & 1];
    if (li + 1 < p.layers && cx.t < (int)(sizeof(PLayerDev) / 4))  // visible long before the next layer starts
      ((uint32_t*)&ls[(li + 1) & 1])[cx.t] = ((const uint32_t*)&p.L[li + 1])[cx.t];
    const bool attn = L.kind == DFB_LAYER_ATTENTION;
    const bool tr = li == p.trace_layer;
    if (tr) mark(cx, 1);
    // input projections, RMSNorm prologue
    xs.kind = XB_RMS;
    xs.norm_w = L.in_norm;
    xs.rstd = rsqrt_2step(__fadd_rn(__fdiv_rn(ss, (float)p.hidden), p.eps));
    build_x(cx, xs, p.hidden);
    if (tr) mark(cx, 2);
    const uint32_t ep_p = cx.base + (++seq);
    cx.tslot = tr ? 22 : 0;
    gemv_phase(cx, geo(p.hidden, L.in_n, 0), attn ? EPI_P : EPI_CONV, ep_p, &L, nullptr);
    cx.tslot = 0;
    if (tr) mark(cx, 3);
    const uint32_t ep_o = cx.base + (++seq);
    int mixw;
    if (attn) {
      const uint32_t ep_ap = cx.base + (++seq);
      attn_partial_phase(cx, L, ep_p, ep_ap);
      if (tr) mark(cx, 15);
      attn_merge_phase(cx, ep_p, ep_ap, ep_o);
      mixw = p.hq * HD;
      xs.kind = XB_LL;
      xs.buf = p.O;
      xs.epoch = ep_o;
    } else {
      deltanet_phase(cx, L, ep_p, ep_o);
      mixw = p.hv_lin * p.dv;
      xs.kind = XB_DN;
      xs.buf = p.O;
      xs.epoch = ep_o;
      xs.zbuf = p.Pb;
      xs.zepoch = ep_p;
      xs.z_off = 2 * p.hk_lin * p.dk + p.hv_lin * p.dv;
      xs.ssq = p.SSQ;
      xs.gnorm_w = L.gnorm_w;
      xs.gnorm_bf16 = L.gnorm_bf16;
    }
    if (tr) mark(cx, 4);
    build_x(cx, xs, mixw);
    if (tr) mark(cx, 5);
    ep_h = cx.base + (++seq);
    cx.tslot = tr ? 26 : 0;
    gemv_phase(cx, geo(mixw, p.hidden, 0), EPI_RES, ep_h, &L, nullptr);
    cx.tslot = 0;
    if (tr) mark(cx, 6);
    ss = gather_h(cx, ep_h);
    if (tr) mark(cx, 7);
    // MLP
    xs.kind = XB_RMS;
    xs.norm_w = L.post_norm;
    xs.rstd = rsqrt_2step(__fadd_rn(__fdiv_rn(ss, (float)p.hidden), p.eps));
    build_x(cx, xs, p.hidden);
    if (tr) mark(cx, 8);
    const uint32_t ep_a = cx.base + (++seq);
    gemv_phase(cx, geo(p.hidden, 2 * p.inter, 1), EPI_SWIGLU, ep_a, &L, nullptr);
    if (tr) mark(cx, 9);
    xs.kind = XB_LL;
    xs.buf = p.A;
    xs.epoch = ep_a;
    build_x(cx, xs, p.inter);
    if (tr) mark(cx, 10);
    ep_h = cx.base + (++seq);
    gemv_phase(cx, geo(p.inter, p.hidden, 0), EPI_RES, ep_h, &L, nullptr);
    if (tr) mark(cx, 11);
    ss = gather_h(cx, ep_h);
    if (tr) mark(cx, 12);
  }
  mark(cx, 16);
  if (p.trace && cx.t == 0) {
    p.trace[cx.c * 32 + 20] = cx.w_ring;
    p.trace[cx.c * 32 + 21] = cx.w_ll;
  }
  // final norm, LM head, greedy pick
  xs.kind = XB_RMS;
  xs.norm_w = p.final_norm;
  xs.rstd = rsqrt_2step(__fadd_rn(__fdiv_rn(ss, (float)p.hidden), p.eps));
  build_x(cx, xs, p.hidden);
  ArgBest best;
  best.v = -INFINITY;
  best.i = 0x7fffffff;
  gemv_phase(cx, geo(p.hidden, p.vocab, 0), EPI_LOGITS, 0, nullptr, &best);
  mark(cx, 17);
  const uint32_t ep_arg = cx.base + (++seq);
  {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) arg_merge(best, __shfl_xor_sync(0xffffffffu, best.v, o), __shfl_xor_sync(0xffffffffu, best.i, o));
    consumer_sync();
    if (cx.lane == 0) {
      cx.red[cx.warp] = best.v;
      cx.red[16 + cx.warp] = __int_as_float(best.i);
    }
    consumer_sync();
    if (cx.t == 0 && !*cx.failed) {
      for (int w = 1; w < CW; ++w) arg_merge(best, cx.red[w], __float_as_int(cx.red[16 + w]));
      ll_store(p.ARG + 2 * cx.c, __float_as_uint(best.v), ep_arg);
      ll_store(p.ARG + 2 * cx.c + 1, (uint32_t)best.i, ep_arg);
    }
  }
  if (cx.c == 0) {
    ArgBest b2;
    b2.v = -INFINITY;
    b2.i = 0x7fffffff;
    for (int i = cx.t; i < p.P; i += CT) {
      const float v = __uint_as_float(ll_wait(cx, p.ARG + 2 * i, ep_arg));
      const int idx = (int)ll_wait(cx, p.ARG + 2 * i + 1, ep_arg);
      arg_merge(b2, v, idx);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) arg_merge(b2, __shfl_xor_sync(0xffffffffu, b2.v, o), __shfl_xor_sync(0xffffffffu, b2.i, o));
    consumer_sync();
    if (cx.lane == 0) {
      cx.red[32 + cx.warp] = b2.v;
      cx.red[48 + cx.warp] = __int_as_float(b2.i);
    }
    consumer_sync();
    if (cx.t == 0) {
      for (int w = 1; w < CW; ++w) arg_merge(b2, cx.red[32 + w], __float_as_int(cx.red[48 + w]));
      if (!*cx.failed) {
        p.tokens[0] = b2.i;
        if (p.history) p.history[cx.pos] = b2.i;
        *p.pos = cx.pos + 1;
      }
      // every CTA has read the counter long ago: its ARG word above depends on all of them
      *p.launch_counter = cx.base / 1024u + 1u;
    }
  }
}

// ---------------------------------------------------------------------------------------------------
// Install-time re-pack: the reference layout (packed [K/2, N] bytes, scale [K/128, N]) -> per-CTA streams
// ---------------------------------------------------------------------------------------------------

__global__ void pstep_repack_kernel(const uint8_t* packed, const void* scale, int sb, ProjGeo g, int P,
                                    unsigned char* const* stream_base, const long long* offsets) {
  const int c = blockIdx.x;
  const int items = proj_items(g);
  const int i0 = split2(items, c, P), n = split2(items, c + 1, P) - i0;
  const Blocks bl = blocks_of(n, g.paired ? MAXW / 2 : MAXW);
  const int G = g.K / 128, half = g.K / 2;
  unsigned char* dst = stream_base[c] + offsets[c];
  for (int b = 0; b < bl.nblk; ++b) {
    const int nb = min(bl.bw, n - b * bl.bw);
    if (nb <= 0) break;
    const int w = g.paired ? 2 * nb : nb;
    const int first = i0 + b * bl.bw;
    const int ssec = (sb * w + 15) & ~15, gb = ssec + 64 * w;
    for (int gi = blockIdx.y; gi < G; gi += gridDim.y) {
      unsigned char* gd = dst + (size_t)gi * gb;
      for (int e = threadIdx.x; e < 17 * w; e += blockDim.x) {
        const int i = e % w, rr = e / w;  // rr == 16: the scale row
        const int col = g.paired ? (i < nb ? first + i : items + first + (i - nb)) : first + i;
        if (rr == 16) {
          if (sb == 2)
            ((uint16_t*)gd)[i] = ((const uint16_t*)scale)[(size_t)gi * g.N + col];
          else
            ((float*)gd)[i] = ((const float*)scale)[(size_t)gi * g.N + col];
        } else {
          const int kb = gi * 16 + rr;
          uint32_t word = 0;
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int r = kb * 8 + j;
            const uint32_t byte = packed[(size_t)(r < half ? r : r - half) * g.N + col];
            word |= (r < half ? (byte & 15u) : (byte >> 4)) << (4 * j);
          }
          ((uint32_t*)(gd + ssec))[rr * w + i] = word;
        }
      }
    }
    dst += (size_t)G * gb;
  }
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int sm_count_now() {
  int dev = 0, v = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  return v;
}

constexpr size_t SMEM_BYTES = (size_t)NSTAGE * STAGE + 33280 + MAX_HIDDEN * 4 + MAXGQ * HD * 4 + 2 * HD * 4 + 1024 * 4 + MAXW * 4 +
                              16 * 4 + 2 * NSTAGE * 8 + 16 + NGEO * sizeof(SliceGeo) + ((sizeof(PParams) + 15) & ~15) +
                              2 * sizeof(PLayerDev) + 128;

struct WsPlan {
  size_t H, Pb, O, A, SSQ, AP, ARG, counter, layers, bases, offsets, trace, total;
};

WsPlan ws_plan(const dfb_model_desc& m, int P) {
  WsPlan w = {};
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off += align_up(bytes, 256);
    return at;
  };
  size_t max_in = 0;
  for (int i = 0; i < m.num_layers; ++i) max_in = std::max(max_in, (size_t)m.layers_host[i].in_proj.N);
  const size_t mixw = std::max((size_t)m.lin_v_heads * m.lin_dv, (size_t)m.hq * m.head_dim);
  const int nchunk = std::max(1, P / std::max(1, m.hkv));
  w.H = take((size_t)m.hidden / 2 * 8);
  w.Pb = take((max_in / 2 + 2) * 8);
  w.O = take((mixw / 2 + 2) * 8);
  w.A = take((size_t)m.intermediate / 2 * 8);
  w.SSQ = take((size_t)std::max(1, m.lin_v_heads) * std::max(1, m.lin_dv / 32) * 8);
  w.AP = take((size_t)m.hq * nchunk * (HD + 2) * 8);
  w.ARG = take((size_t)P * 2 * 8);
  w.counter = take(256);
  w.layers = take((size_t)std::max(1, m.num_layers) * sizeof(PLayerDev));
  w.bases = take((size_t)P * sizeof(void*));
  w.offsets = take((size_t)P * sizeof(long long));
  w.trace = take((size_t)P * 32 * sizeof(long long));
  w.total = off;
  return w;
}

std::vector<ProjGeo> proj_list(const dfb_model_desc& m) {
  std::vector<ProjGeo> v;
  for (int i = 0; i < m.num_layers; ++i) {
    const dfb_layer_desc& L = m.layers_host[i];
    v.push_back({L.in_proj.K, L.in_proj.N, 0});
    v.push_back({L.out_proj.K, L.out_proj.N, 0});
    v.push_back({L.gate_up.K, L.gate_up.N, 1});
    v.push_back({L.down.K, L.down.N, 0});
  }
  v.push_back({m.head.K, m.head.N, 0});
  return v;
}

}  // namespace

struct PStep {
  PParams p;
  int P;
};

bool pstep_eligible(const dfb_model_desc& m) {
  const int P = sm_count_now();
  if (P < 1 || m.batch != 1 || m.math != MATH_FAST) return false;
  if (m.hidden % 128 || m.hidden > MAX_HIDDEN || m.intermediate % 128 || m.intermediate > MAX_K || m.vocab % 2) return false;
  if (m.num_layers * 7 + 4 >= 1024) return false;
  bool any_attn = false, any_dn = false;
  const int sbf = m.head.scale_is_bf16;
  auto lin_ok = [&](const dfb_linear& l) {
    return l.group == 128 && l.K % 128 == 0 && l.K <= MAX_K && l.N % 2 == 0 && l.scale_is_bf16 == sbf && l.packed && l.scale;
  };
  if (!lin_ok(m.head)) return false;
  for (int i = 0; i < m.num_layers; ++i) {
    const dfb_layer_desc& L = m.layers_host[i];
    if (!lin_ok(L.in_proj) || !lin_ok(L.out_proj) || !lin_ok(L.gate_up) || !lin_ok(L.down)) return false;
    (L.kind == DFB_LAYER_ATTENTION ? any_attn : any_dn) = true;
  }
  if (any_attn) {
    if (m.head_dim != HD || m.hkv < 1 || m.hq % m.hkv || m.hq / m.hkv > MAXGQ || m.hkv > P || m.rotary_dim % 2 || m.rotary_dim > HD)
      return false;
  }
  if (any_dn) {
    if (m.lin_dk > 128 || m.lin_dk < 1 || m.lin_dv % 32 || m.lin_dv < 32 || m.lin_k_heads < 1 || m.lin_v_heads % m.lin_k_heads ||
        (m.lin_v_heads * m.lin_dv) % 128 || (2 * m.lin_k_heads * m.lin_dk) % 2 || m.lin_dv % 4)
      return false;
  }
  return true;
}

size_t pstep_workspace_bytes(const dfb_model_desc& m) { return ws_plan(m, std::max(1, sm_count_now())).total; }

size_t pstep_stream_bytes(const dfb_model_desc& m) {
  const int P = std::max(1, sm_count_now());
  const int sb = m.head.scale_is_bf16 ? 2 : 4;
  const std::vector<ProjGeo> ops = proj_list(m);
  size_t total = 0;
  for (int c = 0; c < P; ++c) {
    long long b = 0;
    for (const ProjGeo& g : ops) b += proj_chunk_bytes(g, c, P, sb);
    total += align_up((size_t)b, 128);
  }
  return total + 128;
}

int pstep_create(const dfb_model_desc& m, void* ws, void* stream_mem, size_t stream_bytes, PStep** out, cudaStream_t stream) {
  if (!pstep_eligible(m)) {
    set_error("persistent step: this model shape is not supported (batch 1, group 128, head dim 256, FAST arithmetic only)");
    return DFB_ERR_ARG;
  }
  const int P = sm_count_now();
  if (stream_bytes < pstep_stream_bytes(m) || !stream_mem || ((uintptr_t)stream_mem % 128) != 0) {
    set_error("persistent step: weight stream buffer of %zu bytes (128-byte aligned) required, got %zu", pstep_stream_bytes(m),
              stream_bytes);
    return DFB_ERR_ARG;
  }
  cudaError_t e = cudaFuncSetAttribute(pstep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
  if (e != cudaSuccess) return check_launch("persistent step: shared-memory opt-in");
  int per_sm = 0;
  e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, pstep_kernel, THREADS, SMEM_BYTES);
  if (e != cudaSuccess || per_sm < 1) {
    set_error("persistent step: the kernel does not fit on an SM of this device");
    (void)cudaGetLastError();
    return DFB_ERR_CUDA;
  }
  const WsPlan w = ws_plan(m, P);
  const int sb = m.head.scale_is_bf16 ? 2 : 4;
  char* base = (char*)ws;
  PStep* ps = new (std::nothrow) PStep();
  if (!ps) {
    set_error("persistent step: out of host memory");
    return DFB_ERR_ARG;
  }
  ps->P = P;
  PParams& p = ps->p;
  p = {};
  p.P = P;
  p.hidden = m.hidden, p.inter = m.intermediate, p.vocab = m.vocab, p.layers = m.num_layers, p.max_seq = m.max_seq;
  p.hq = m.hq, p.hkv = m.hkv, p.rd = m.rotary_dim, p.gate = m.attn_output_gate, p.gate_swish = m.gate_is_swish;
  p.hk_lin = m.lin_k_heads, p.hv_lin = m.lin_v_heads, p.dk = m.lin_dk, p.dv = m.lin_dv;
  p.eps = m.eps;
  p.sb = sb;
  p.inv_freq = m.inv_freq;
  p.embed = (const bf16*)m.embed;
  p.final_norm = (const bf16*)m.final_norm_w;
  p.L = (const PLayerDev*)(base + w.layers);
  p.stream_base = (const unsigned char* const*)(base + w.bases);
  p.tokens = m.tokens, p.history = m.history, p.pos = m.pos, p.logits = (bf16*)m.logits;
  p.H = (u64*)(base + w.H), p.Pb = (u64*)(base + w.Pb), p.O = (u64*)(base + w.O), p.A = (u64*)(base + w.A);
  p.SSQ = (u64*)(base + w.SSQ), p.AP = (u64*)(base + w.AP), p.ARG = (u64*)(base + w.ARG);
  p.launch_counter = (unsigned*)(base + w.counter);
  p.status = nullptr;  // set by the caller
  p.trace = nullptr;
  p.trace_layer = -1;

  // device tables
  std::vector<PLayerDev> layers(m.num_layers);
  for (int i = 0; i < m.num_layers; ++i) {
    const dfb_layer_desc& L = m.layers_host[i];
    PLayerDev& d = layers[i];
    d = {};
    d.kind = L.kind;
    d.in_norm = (const bf16*)L.input_norm_w, d.post_norm = (const bf16*)L.post_norm_w;
    d.conv_w = (const bf16*)L.conv_w, d.conv_state = (bf16*)L.conv_state;
    d.a_log = L.a_log, d.dt_bias = L.dt_bias, d.gnorm_w = L.gnorm_w, d.gnorm_bf16 = L.gnorm_w_is_bf16;
    d.recurrent = L.recurrent;
    d.q_norm = (const bf16*)L.q_norm_w, d.k_norm = (const bf16*)L.k_norm_w;
    d.kcache = (bf16*)L.kcache, d.vcache = (bf16*)L.vcache;
    d.in_n = L.in_proj.N;
  }
  const std::vector<ProjGeo> ops = proj_list(m);
  std::vector<unsigned char*> bases(P);
  std::vector<long long> run(P, 0);
  {
    size_t at = 0;
    for (int c = 0; c < P; ++c) {
      bases[c] = (unsigned char*)stream_mem + at;
      long long b = 0;
      for (const ProjGeo& g : ops) b += proj_chunk_bytes(g, c, P, sb);
      at += align_up((size_t)b, 128);
    }
  }
  const unsigned one = 1;
  e = cudaMemcpyAsync(base + w.layers, layers.data(), layers.size() * sizeof(PLayerDev), cudaMemcpyHostToDevice, stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(base + w.bases, bases.data(), (size_t)P * sizeof(void*), cudaMemcpyHostToDevice, stream);
  if (e == cudaSuccess) e = cudaMemcpyAsync(base + w.counter, &one, sizeof(one), cudaMemcpyHostToDevice, stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize(stream);  // the host vectors above go out of scope
  if (e != cudaSuccess) {
    delete ps;
    return check_launch("persistent step: table upload");
  }
  // re-pack every projection in consumption order
  std::vector<const dfb_linear*> lins;
  for (int i = 0; i < m.num_layers; ++i) {
    const dfb_layer_desc& L = m.layers_host[i];
    lins.push_back(&L.in_proj), lins.push_back(&L.out_proj), lins.push_back(&L.gate_up), lins.push_back(&L.down);
  }
  lins.push_back(&m.head);
  for (size_t oi = 0; oi < ops.size(); ++oi) {
    e = cudaMemcpyAsync(base + w.offsets, run.data(), (size_t)P * sizeof(long long), cudaMemcpyHostToDevice, stream);
    if (e != cudaSuccess) break;
    pstep_repack_kernel<<<dim3(P, std::min(ops[oi].K / 128, 16)), 256, 0, stream>>>(lins[oi]->packed, lins[oi]->scale, sb, ops[oi], P,
                                                                                     (unsigned char* const*)(base + w.bases),
                                                                                     (const long long*)(base + w.offsets));
    e = cudaStreamSynchronize(stream);  // `run` is reused as the source of the next upload
    if (e != cudaSuccess) break;
    for (int c = 0; c < P; ++c) run[c] += proj_chunk_bytes(ops[oi], c, P, sb);
  }
  if (e != cudaSuccess || cudaGetLastError() != cudaSuccess) {
    delete ps;
    set_error("persistent step: re-packing the weights failed: %s", cudaGetErrorString(e));
    return DFB_ERR_CUDA;
  }
  *out = ps;
  return DFB_OK;
}

void pstep_set_status(PStep* ps, int* status) { ps->p.status = status; }

// Phase timestamps of one layer (diagnostics): enable with a layer index, read back after a step.
void pstep_set_trace(PStep* ps, void* ws, const dfb_model_desc& m, int layer) {
  const WsPlan w = ws_plan(m, ps->P);
  ps->p.trace = layer >= 0 ? (long long*)((char*)ws + w.trace) : nullptr;
  ps->p.trace_layer = layer;
}
int pstep_read_trace(PStep* ps, long long* out_host, int max_values, cudaStream_t stream) {
  if (!ps->p.trace) return 0;
  const int n = std::min(max_values, ps->P * 32);
  if (cudaMemcpyAsync(out_host, ps->p.trace, (size_t)n * sizeof(long long), cudaMemcpyDeviceToHost, stream) != cudaSuccess ||
      cudaStreamSynchronize(stream) != cudaSuccess)
    return -1;
  return n;
}

void pstep_destroy(PStep* ps) { delete ps; }

int pstep_launch(PStep* ps, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ps->P, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = SMEM_BYTES;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident at once: they wait on one another
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, pstep_kernel, ps->p);
  if (e != cudaSuccess) {
    set_error("persistent step: launch failed: %s", cudaGetErrorString(e));
    return DFB_ERR_CUDA;
  }
  return check_launch("persistent step");
}

}  // namespace dfb
