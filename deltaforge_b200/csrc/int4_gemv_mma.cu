// Cluster int4 dequant-GEMV on the integer tensor-core instruction, for the per-layer projections of batch-1
// decode, sm_100a.
//
// Same function and the same exact-integer arithmetic as int4_gemv_cluster.cu (the reference's group-128 int4 linear,
// op deltaforge::tiled_gemv_int4, src/deltaforge/kernels/tiled_gemv.py:915-958): per 128-row scale group the
// activation is a block of 15-bit integers m with one power-of-two exponent, sum_k (nibble_k - 8) * m_k is formed
// exactly in int32, and exponent and group scale are applied once per group and column in fp32. What changes is who
// multiplies: mma.sync.m16n8k32 (u8 x s8 -> s32) takes 16 columns x 32 rows of weight bytes as its A operand and
// the activation bytes as B, so a warp spends one instruction where the dp4a form spends sixteen. It is used as a
// wide dp4a, not as a matrix product: only three of B's eight columns carry data (the byte-pieces of m).
//
//  * Weight layout (made once at install by int4_repack_mma_kernel from the reference's [K/2, N] bytes): the matrix
//    is cut into tiles of 256 columns and units of (tile, 128-row group); a unit is one contiguous block of
//    16 KB of words in the order the mma A fragments are read (16-column block, pair of 32-row steps, lane, four
//    words) followed by the unit's 256 scales in the order the lanes read them. A unit arrives by ONE bulk copy.
//    Nibbles stay as stored (value + 8): even rows of a word are the low nibbles of its bytes and feed the mma as
//    they are; odd rows are the high nibbles, used unshifted (16 x nibble). The activation bytes make up for it:
//    B holds the three byte-pieces of 16 m against the even rows and the two byte-pieces of m against the odd rows,
//    so column j of the product is piece j of 16 * sum nibble * m.
//    In "pair" mode (gate_proj|up_proj) a tile is 128 gate columns followed by the 128 up columns of the same
//    channels, so the CTA that finishes a tile can apply SwiGLU.
//  * Data movement, prologues and epilogues are those of int4_gemv_cluster.cu: a cluster of CTAs per tile splits the
//    groups, every CTA fills its ring of units before griddepcontrol.wait, column sums go to the cluster's first CTA
//    through distributed shared memory, one cluster barrier, fixed-order sums.
//  * Work split inside a CTA: the tile is cut into chunks of four 16-column blocks; a warp owns one chunk and every
//    second (256-column tiles) or fourth (128-column tiles) unit of it. The four blocks of a unit are four independent
//    chains of mma, so a warp is not waiting on one chain of dependent instructions per unit (a warp that owned two
//    blocks and walked through every unit spent 800 cycles per unit, nearly all of it latency). The warps of a chunk
//    add their column sums through shared memory in warp order. Every unit has an mbarrier of its own (used once), so a
//    warp that reads only some units never meets a barrier phase it skipped.
//  * Measured on B200 for this instruction: one mma.sync.m16n8k32 (u8 x s8) per 8.1 cycles per SM sub-core, 21 cycles
//    of latency; the u4 x s4 form (m16n8k64) is emulated at about 220 cycles and is not used.
//
// Every mbarrier wait is bounded (about two seconds); a CTA whose wait gives up records a code in the status word
// and still takes part in the cluster barrier.
#include <algorithm>
#include <cstdlib>

#include "gemv_common.cuh"

namespace dfb {

namespace {

constexpr int CW = 8;                // consumer warps: TN / 128 blocks of 16 columns each
constexpr int CT = CW * 32;
constexpr int THREADS = CT + 32;     // + the warp that issues the copies
constexpr int QW = CW + 1;           // warps that quantise the activation: all of them
constexpr int XB_BYTES = 16 * 8 * 2 * 4;  // activation bytes of one group: [16 word rows][8 B-columns][2 words]
constexpr int MAX_CS = 8;
constexpr long long WAIT_LIMIT_CYCLES = 4000000000LL;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
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
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t pol) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol)
      : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CT) : "memory"); }
__device__ __forceinline__ void all_sync() { asm volatile("bar.sync 3, %0;" ::"n"(THREADS) : "memory"); }
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
// c += A (16 x 32, unsigned bytes) * B (32 x 8, signed bytes)
__device__ __forceinline__ void imma(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct MmaArgs {
  GemvParams p;
  int cs;         // CTAs of a cluster = shares of the groups of a tile
  int max_units;  // most groups a CTA gets
  int num_tiles;
  int stages;     // ring depth in units
  int unit_bytes; // TN * 64 bytes of words + TN scales
  int* status;
};

// Output column `col` (0 .. TN-1) of tile `tile`: which column of the matrix it is, or -1 beyond N.
template <int TN>
__device__ __forceinline__ int tile_column(int tile, int col, int N, int pair) {
  if (pair) {
    const int ch = tile * (TN / 2) + (col & (TN / 2 - 1));
    if (ch >= N / 2) return -1;
    return col < TN / 2 ? ch : N / 2 + ch;
  }
  const int n = tile * TN + col;
  return n < N ? n : -1;
}

// One group (local index gl) by one warp: v[i] is row 4 * lane + i. Writes the group's exponent factor, integer sum and
// B-fragment bytes. (Two groups at a time per warp, their shuffle chains interleaved, measured slower.)
__device__ __forceinline__ void quantise_group(const float (&v)[4], int gl, float* fg, int* msum, unsigned char* xb, int lane) {
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) amax = fmaxf(amax, fabsf(v[i]));
  // non-negative floats order like their bit patterns: one warp-wide integer maximum instead of five shuffle steps
  const uint32_t abits = __reduce_max_sync(0xffffffffu, __float_as_uint(amax));
  int E = abits != 0u ? (int)((abits >> 23) & 0xff) - 127 : 0;  // amax in [2^E, 2^(E+1))
  E = max(E, -100);
  const float up = __uint_as_float((uint32_t)(127 + 13 - E) << 23);  // 2^(13-E): |x| * up < 2^14
  if (lane == 0) fg[gl] = __uint_as_float((uint32_t)(127 - 13 + E - 4) << 23);  // 2^(E-13) / 16
  // Signed byte-pieces without a carry chain: q = p0 + 256 p1 + 65536 p2 with every p in [-128, 127] is the same as
  // q + 0x808080 in plain unsigned bytes with 128 taken off each, i.e. with each byte's top bit flipped.
  int m[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) m[i] = __float2int_rn(v[i] * up);
  int ms = (m[0] + m[1]) + (m[2] + m[3]);
  // rows 4l+0, 4l+2 (even: the three pieces of 16 m) and 4l+1, 4l+3 (odd: the two pieces of m); byte 3 of each is zero
  const uint32_t t0 = ((uint32_t)(m[0] * 16 + 0x808080) ^ 0x808080u) & 0xffffffu, t2 = ((uint32_t)(m[2] * 16 + 0x808080) ^ 0x808080u) & 0xffffffu;
  const uint32_t u1 = ((uint32_t)(m[1] + 0x8080) ^ 0x8080u) & 0xffffu, u3 = ((uint32_t)(m[3] + 0x8080) ^ 0x8080u) & 0xffffu;
  // this lane's halves (16 bits: two rows each) of the five B words: rows 4l+0, 4l+1 -> byte 0 of the half, rows 4l+2,
  // 4l+3 -> byte 1; even lanes own the low half of the word (rows 0..3 of word row l / 2), odd lanes the high half
  const bool hi = (lane & 1) != 0;
  uint32_t e0 = __byte_perm(t0, t2, hi ? 0x4033 : 0x3340), e1 = __byte_perm(t0, t2, hi ? 0x5133 : 0x3351);
  uint32_t e2 = __byte_perm(t0, t2, hi ? 0x6233 : 0x3362);
  uint32_t o0 = __byte_perm(u1, u3, hi ? 0x4033 : 0x3340), o1 = __byte_perm(u1, u3, hi ? 0x5133 : 0x3351);
  ms = (int)__reduce_add_sync(0xffffffffu, ms);
  if (lane == 0) msum[gl] = ms;
  // lanes 2r and 2r+1 complete each other's words
  e0 |= __shfl_xor_sync(0xffffffffu, e0, 1), e1 |= __shfl_xor_sync(0xffffffffu, e1, 1), e2 |= __shfl_xor_sync(0xffffffffu, e2, 1);
  o0 |= __shfl_xor_sync(0xffffffffu, o0, 1), o1 |= __shfl_xor_sync(0xffffffffu, o1, 1);
  // B column c of word row kb: (b0, b1) at xb[group][kb][c]; columns 3..7 are zero
  uint2* row = (uint2*)(xb + (size_t)gl * XB_BYTES) + (lane >> 1) * 8;
  if ((lane & 1) == 0) {
    row[0] = make_uint2(e0, o0), row[1] = make_uint2(e1, o1), row[2] = make_uint2(e2, 0u), row[3] = make_uint2(0u, 0u);
  } else {
    row[4] = row[5] = row[6] = row[7] = make_uint2(0u, 0u);
  }
}

// TN columns per tile: 256 or 128. MERGE: the instance that serves the attention-merge prologue; it keeps sixteen loads in
// flight per lane and needs more registers than the others, which stay at three CTAs per SM.
template <int TN, bool MERGE = false>
__global__ void __launch_bounds__(THREADS) gemv_mma_kernel(const MmaArgs a) {
  constexpr int CH = TN / 64;              // chunks of four 16-column blocks per tile
  constexpr int W_BYTES = TN / 16 * 1024;  // bytes of words per unit
  extern __shared__ unsigned char smem_raw[];
  const GemvParams& p = a.p;
  const int G = p.K / 128;
  unsigned char* ring = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);  // stages * unit_bytes (unit_bytes % 128 == 0)
  unsigned char* xb = ring + (size_t)a.stages * a.unit_bytes;      // [max_units] activation bytes, XB_BYTES each
  int* msum = (int*)(xb + (size_t)a.max_units * XB_BYTES);         // [max_units] sum of m over the group
  float* fg = (float*)(msum + ((a.max_units + 3) & ~3));           // [max_units] 2^e / 16 per group
  float* dsm = fg + ((a.max_units + 3) & ~3);                      // [cs][TN] column sums from every rank (used in rank 0)
  float* red = dsm + a.cs * TN;                                    // [TN] scratch of the SwiGLU epilogue
  uint64_t* full = (uint64_t*)(red + TN);                          // [max_units] one per unit, each used once: a warp that
                                                                   // reads only some units never meets a phase it skipped
  uint64_t* empty = full + a.max_units;                            // [stages]
  float* wred = (float*)(empty + a.stages);                        // [16]
  float* part = wred + 16;                                         // [CW][64] column sums of every warp's units

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
  const int cs = a.cs;
  const int rank = (int)cluster_rank();
  const int tile = blockIdx.x / cs;
  const bool swiglu = p.epilogue == EPI_SWIGLU;
  const int g0 = (int)((long)rank * G / cs), g1 = (int)((long)(rank + 1) * G / cs);
  const int nunits = g1 - g0;
  const int cta = blockIdx.x;

  if (t == 0) {
    trace_mark(p.trace, cta, 0);
    for (int s = 0; s < a.max_units; ++s) mbar_init(&full[s], 1);
    for (int s = 0; s < a.stages; ++s) mbar_init(&empty[s], CH);  // one arrival per chunk = per warp that reads the unit
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  bool ok = true;
  EpiPre pre = {};
  // producer (lane 0 of the last warp): the weights never depend on earlier kernels; the ring is filled at once, later units
  // follow, after the activation is quantised, as the consumers hand stages back
  const uint64_t pol = make_evict_first_policy();
  const unsigned char* src = p.packed_mma + ((size_t)tile * G + g0) * a.unit_bytes;
  const int first_fill = min(nunits, a.stages);
  if (warp == CW) {
    if (lane == 0) {
      for (int j = 0; j < first_fill; ++j) {
        mbar_expect_tx(&full[j], (uint32_t)a.unit_bytes);
        bulk_load(ring + (size_t)j * a.unit_bytes, src + (size_t)j * a.unit_bytes, (uint32_t)a.unit_bytes, &full[j], pol);
      }
      trace_mark(p.trace, cta, 7);
    }
    if (lane >= 4 && lane <= 5 && p.pf_ptr[lane - 4] != nullptr)  // a slice of a later projection's weights, into the L2
      l2_prefetch_range(p.pf_ptr[lane - 4], p.pf_bytes[lane - 4] * (size_t)cta / gridDim.x, p.pf_bytes[lane - 4] * (size_t)(cta + 1) / gridDim.x);
    if (cta == 0 && lane >= 1 && lane <= 3 && p.touch_ptr[lane - 1] != nullptr) {
      const char* q = (const char*)p.touch_ptr[lane - 1];
      for (int o = 0; o < p.touch_bytes[lane - 1]; o += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(q + o));
    }
    __syncwarp();
  }
  // Every warp, the producer's included, quantises groups of the activation (warp w: groups w, w + 9, ...).
  // What this CTA reads that no kernel of this token writes goes in flight before the wait for the previous kernel: the
  // norm weights of the groups it quantises, and, where the caller says the history was last written before this stream's
  // current work began (the decode engine: one token ago), the conv taps and history its epilogue uses.
  uint2 xraw[2] = {make_uint2(0u, 0u), make_uint2(0u, 0u)}, wraw[2] = {make_uint2(0u, 0u), make_uint2(0u, 0u)};
  const int my_n = t < TN ? tile_column<TN>(tile, t, p.N, 0) : -1;
  const bool finisher = (cs == 1 || rank == 0) && !swiglu && my_n >= 0;
  if (p.prologue == PRO_RMSNORM) {
#pragma unroll
    for (int j = 0; j < 2; ++j)
      if (warp + j * QW < nunits) wraw[j] = *(const uint2*)(p.norm_w + (g0 + warp + j * QW) * 128 + lane * 4);
  }
  const float inv_k = __frcp_rn((float)p.K);
  const bool conv_early = p.epilogue == EPI_CONV && p.conv_state_settled;
  if (finisher && conv_early) pre = epilogue_preload(p, 0, my_n);
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the activation comes from the previous kernel
  if (t == 0) trace_mark(p.trace, cta, 1);
  // Everything this CTA reads that an earlier kernel wrote goes in flight at once.
  // (the first two groups each warp quantises: a CTA holds at most eighteen groups in practice, so this is all of them)
#pragma unroll
  for (int j = 0; j < 2; ++j)
    if (warp + j * QW < nunits && !MERGE) {
      const int k = (g0 + warp + j * QW) * 128 + lane * 4;
      xraw[j] = *(const uint2*)(p.x + k);
      if (p.prologue == PRO_SILU_MUL) wraw[j] = *(const uint2*)(p.up + k);
    }
  if (finisher && !conv_early) pre = epilogue_preload(p, 0, my_n);
  float rstd = 1.f;
  if (p.prologue == PRO_RMSNORM) {
    float tot = 0.f;
    if (p.ss_in && p.ss_count <= 32) {
      // the kernel that wrote x left the sums of squares of its tiles: one load per lane and a shuffle tree (the same
      // tree in every warp of every CTA, so all of them get the same bits), not a chain of dependent loads
      tot = warp_sum(lane < p.ss_count ? p.ss_in[lane] : 0.f);
    } else if (p.ss_in) {
      for (int i = 0; i < p.ss_count; ++i) tot += p.ss_in[i];
    } else {
      float ss = 0.f;
      for (int k = t; k < p.K; k += THREADS) {
        const float v = bf2f(p.x[k]);
        ss = fmaf(v, v, ss);
      }
      ss = warp_sum(ss);
      if (lane == 0) wred[warp] = ss;
      all_sync();
#pragma unroll
      for (int w = 0; w < QW; ++w) tot += wred[w];
    }
    // 1 / sqrt(mean + eps) by the reciprocal-square-root unit and one Newton step (within an ulp of the two correctly
    // rounded steps the slower kernels take; the chain of dependent instructions is a third as long)
    const float y = fmaf(tot, inv_k, p.eps);
    const float r = rsqrtf(y);
    rstd = r * fmaf(-0.5f * y * r, r, 1.5f);
  }
  // One warp per group of this CTA: shared exponent, 15-bit integers m (|m| < 2^14), cut into signed bytes in the order
  // the mma's B fragments are read. Lane l holds rows 4l .. 4l+3 of the group = half of word row l/2.
  for (int gl = warp; gl < nunits; gl += QW) {
    float v[4];
    if (MERGE) {
      attn_merge_values(p.merge, (g0 + gl) * 128 + lane * 4, v);
    } else {
      uint2 xv = gl == warp ? xraw[0] : xraw[1], wv = gl == warp ? wraw[0] : wraw[1];
      if (gl >= warp + 2 * QW) {  // a third group and later: loaded here
        const int k = (g0 + gl) * 128 + lane * 4;
        xv = *(const uint2*)(p.x + k);
        if (p.prologue == PRO_RMSNORM) wv = *(const uint2*)(p.norm_w + k);
        if (p.prologue == PRO_SILU_MUL) wv = *(const uint2*)(p.up + k);
      }
      const float xr[4] = {__uint_as_float(xv.x << 16), __uint_as_float(xv.x & 0xffff0000u), __uint_as_float(xv.y << 16),
                           __uint_as_float(xv.y & 0xffff0000u)};
      const float wr[4] = {__uint_as_float(wv.x << 16), __uint_as_float(wv.x & 0xffff0000u), __uint_as_float(wv.y << 16),
                           __uint_as_float(wv.y & 0xffff0000u)};
#pragma unroll
      for (int i = 0; i < 4; ++i) v[i] = prologue_apply(p.prologue, xr[i], wr[i], rstd);
    }
    quantise_group(v, gl, fg, msum, xb, lane);
  }
  all_sync();
  if (t == 0) trace_mark(p.trace, cta, 2);
  if (warp == CW) {
    if (lane == 0) {  // the units beyond the ring's depth, each as its stage comes back
      int st = first_fill == a.stages ? 0 : first_fill, round = first_fill == a.stages ? 1 : 0;
      for (int j = first_fill; j < nunits; ++j) {
        if (round > 0 && !mbar_wait(&empty[st], (round - 1) & 1)) {
          atomicExch(a.status, 6);
          break;
        }
        mbar_expect_tx(&full[j], (uint32_t)a.unit_bytes);
        bulk_load(ring + (size_t)st * a.unit_bytes, src + (size_t)j * a.unit_bytes, (uint32_t)a.unit_bytes, &full[j], pol);
        if (++st == a.stages) st = 0, ++round;
      }
    }
    __syncwarp();  // the whole warp takes part in the (aligned) cluster barrier below
  } else {
    // The tile is cut into chunks of four 16-column blocks. A warp owns one chunk (warp % CH) and every (CW / CH)-th
    // unit of it, so the four blocks of a unit give it four independent chains of mma and a unit is waited for once per
    // chunk. lane = 4 * gq + tq: rows gq and gq + 8 of the mma, word row tq of every 32-row step.
    const int gq = lane >> 2, tq = lane & 3;
    const int mul0 = tq == 0 ? 1 : (tq == 1 ? 65536 : 0), mul1 = tq == 0 ? 256 : 0;
    const int ch = warp % CH;
    float tot[4][2] = {};
    int st = warp / CH;  // = s mod stages: the first units fit the ring (stages >= CW / CH whenever units outnumber stages)
    for (int s = warp / CH; s < nunits; s += CW / CH, st += CW / CH) {
      while (st >= a.stages) st -= a.stages;
      if (ok) ok = mbar_wait(&full[s], 0);
      if (!ok || !DFB_IN_BOUNDS(st < a.stages && s < a.max_units, a.status, 2)) break;
      const unsigned char* ub = ring + (size_t)st * a.unit_bytes;
      const uint2* xrow = (const uint2*)(xb + (size_t)s * XB_BYTES);
      uint2 bv[4];
#pragma unroll
      for (int ks = 0; ks < 4; ++ks) bv[ks] = xrow[(ks * 4 + tq) * 8 + gq];
      int c[4][4];
#pragma unroll
      for (int b = 0; b < 4; ++b) c[b][0] = c[b][1] = c[b][2] = c[b][3] = 0;
#pragma unroll
      for (int pr = 0; pr < 2; ++pr) {
        uint4 w[4];
#pragma unroll
        for (int b = 0; b < 4; ++b) w[b] = *(const uint4*)(ub + (size_t)(4 * ch + b) * 1024 + (pr * 32 + lane) * 16);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            const uint32_t wa = h ? w[b].z : w[b].x, wb = h ? w[b].w : w[b].y;  // columns gq and gq + 8
            imma(c[b], wa & 0x0F0F0F0Fu, wb & 0x0F0F0F0Fu, wa & 0xF0F0F0F0u, wb & 0xF0F0F0F0u, bv[2 * pr + h].x, bv[2 * pr + h].y);
          }
        }
      }
      const float f = fg[s];
      const int zp = tq == 0 ? 128 * msum[s] : 0;  // the zero point: 16 * 8 * sum m, taken off where piece 0 lives
      const unsigned char* sp = ub + W_BYTES;
#pragma unroll
      for (int b = 0; b < 4; ++b) {
        // scales of columns gq and gq + 8 of this block, stored as the pair this lane reads
        float s0, s1;
        if (p.scale_bf16) {
          const uint32_t v = *(const uint32_t*)(sp + ((4 * ch + b) * 8 + gq) * 4);
          s0 = __uint_as_float(v << 16), s1 = __uint_as_float(v & 0xffff0000u);
        } else {
          const float2 v = *(const float2*)(sp + ((4 * ch + b) * 8 + gq) * 8);
          s0 = v.x, s1 = v.y;
        }
        const int i0 = c[b][0] * mul0 + c[b][1] * mul1 - zp, i1 = c[b][2] * mul0 + c[b][3] * mul1 - zp;
        tot[b][0] = fmaf((float)i0 * f, s0, tot[b][0]);
        tot[b][1] = fmaf((float)i1 * f, s1, tot[b][1]);
      }
      if (a.stages < nunits) {  // the stage goes back to the producer (only when units outnumber stages)
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[st]);
      }
      if (s == 0 && t == 0) trace_mark(p.trace, cta, 4);  // the first unit is done
    }
    if (!ok && lane == 0) atomicExch(a.status, 4);
    if (t == 0) trace_mark(p.trace, cta, 3);
    // pieces 0, 1 sit in lane tq = 0, piece 2 in lane tq = 1: one exchange, then lane tq = 0 owns the column sums of this
    // warp's units; the warps of a chunk are added in warp order, and the CTA's column sums go to the cluster's first CTA
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      tot[b][0] += __shfl_xor_sync(0xffffffffu, tot[b][0], 1);
      tot[b][1] += __shfl_xor_sync(0xffffffffu, tot[b][1], 1);
      if (tq == 0) {
        part[warp * 64 + b * 16 + gq] = tot[b][0];
        part[warp * 64 + b * 16 + gq + 8] = tot[b][1];
      }
    }
    consumer_sync();
    if (t < TN && DFB_IN_BOUNDS(rank < cs, a.status, 3)) {
      float v = 0.f;
#pragma unroll
      for (int w = t / 64; w < CW; w += CH) v += part[w * 64 + (t & 63)];
      dsmem_store(dsm + rank * TN + t, 0, v);
    }
  }
  if (cs > 1) cluster_barrier();  // every thread of every CTA of the cluster, the producer warps included
  else __syncthreads();
  if (t == 0) trace_mark(p.trace, cta, 5);
  if (rank == 0 && t < TN) {
    float v = 0.f;
    for (int r = 0; r < cs; ++r) v += dsm[r * TN + t];
    if (swiglu) {
      // threads 0 .. 127 hold the gate_proj sums of 128 channels, the others their up_proj sums: bf16(silu(g)) * u,
      // rounded as the reference's SwiGLUMLP rounds it (src/deltaforge/reference.py:692-693,
      // src/deltaforge/kernels/fused_swiglu.py:18-22)
      red[t] = v;
      asm volatile("bar.sync 2, %0;" ::"n"(TN) : "memory");
      const int ch = tile * (TN / 2) + t;
      if (t < TN / 2 && ch < p.N / 2 && DFB_IN_BOUNDS(ch >= 0, a.status, 4)) {
        const float sv = round_bf16(silu_f(round_bf16(red[t])));
        p.out[ch] = f2bf(__fmul_rn(sv, round_bf16(red[t + TN / 2])));
      }
    } else {
      const int n = tile * TN + t;
      const float stored = n < p.N ? epilogue_store_pre(p, 0, n, v, pre) : 0.f;
      if (p.ss_out != nullptr) {
        const float sq = warp_sum(stored * stored);
        if ((t & 31) == 0) wred[t >> 5] = sq;
        asm volatile("bar.sync 2, %0;" ::"n"(TN) : "memory");
        if (t == 0) {
          float tot = 0.f;
#pragma unroll
          for (int w = 0; w < TN / 32; ++w) tot += wred[w];
          p.ss_out[tile] = tot;
        }
      }
    }
  }
  if (t == 0) trace_mark(p.trace, cta, 6);
}

// reference layout [K/2, N] bytes (+ scales [K/128, N]) -> units in the order the kernel above reads them
template <int TN>
__global__ void int4_repack_mma_kernel(const uint8_t* packed, const void* scale, int scale_bf16, int K, int N, int pair, int tiles,
                                       unsigned char* out, int unit_bytes) {
  constexpr int W_BYTES = TN / 16 * 1024;
  const int G = K / 128, half = K / 2;
  const long unit = blockIdx.x;  // tile * G + g
  const int tile = (int)(unit / G), g = (int)(unit % G);
  unsigned char* ub = out + unit * (long)unit_bytes;
  // words: [block cb][pair of steps pr][lane][4]
  for (int idx = threadIdx.x; idx < W_BYTES / 4; idx += blockDim.x) {
    const int w = idx & 3, lane = (idx >> 2) & 31, pr = (idx >> 7) & 1, cb = idx >> 8;
    const int col = cb * 16 + (w & 1) * 8 + (lane >> 2);
    const int kb = (2 * pr + (w >> 1)) * 4 + (lane & 3);  // word row inside the group
    const int n = tile_column<TN>(tile, col, N, pair);
    uint32_t word = 0x88888888u;  // value 0 in every nibble: columns beyond N add nothing
    if (n >= 0) {
      word = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int r = g * 128 + kb * 8 + i;
        const uint32_t byte = packed[(size_t)(r < half ? r : r - half) * N + n];
        word |= (r < half ? (byte & 15u) : (byte >> 4)) << (4 * i);
      }
    }
    ((uint32_t*)ub)[idx] = word;
  }
  // scales: [block cb][gq][2] = columns gq and gq + 8 of the block
  for (int idx = threadIdx.x; idx < TN; idx += blockDim.x) {
    const int cb = idx >> 4, gq = (idx >> 1) & 7, hi = idx & 1;
    const int n = tile_column<TN>(tile, cb * 16 + hi * 8 + gq, N, pair);
    if (scale_bf16) {
      ((bf16*)(ub + W_BYTES))[idx] = n >= 0 ? ((const bf16*)scale)[(size_t)g * N + n] : f2bf(0.f);
    } else {
      ((float*)(ub + W_BYTES))[idx] = n >= 0 ? ((const float*)scale)[(size_t)g * N + n] : 0.f;
    }
  }
  (void)tiles;
}

// Tile width for an N-column matrix: 256 for the wide projections, 128 for those back to the hidden size (so that
// their few tiles still make a grid of about one CTA per SM); a gate|up pair is always 128 + 128.
int mma_tn(int N, int pair) { return (pair || N >= 4096) ? 256 : 128; }
int mma_tiles(int N, int pair) {
  const int tn = mma_tn(N, pair);
  return pair ? (N / 2 + tn / 2 - 1) / (tn / 2) : (N + tn - 1) / tn;
}
int mma_unit_bytes(int tn, int scale_bf16) { return tn * 64 + tn * (scale_bf16 ? 2 : 4); }

struct MmaPlan {
  int tn, cs, max_units, tiles, stages, unit_bytes;
  size_t smem;
};

MmaPlan plan_mma(int K, int N, int pair, int scale_bf16) {
  MmaPlan c = {};
  const int G = K / 128;
  c.tn = mma_tn(N, pair);
  c.tiles = mma_tiles(N, pair);
  // The groups of a tile are split over a cluster of up to eight CTAs, as many as keep the grid within about 250 CTAs
  // (one and two thirds per SM: with at most 84 KB of ring each, two fit on an SM beside the CTAs of the kernels before
  // and after, which is what lets every kernel of the chain fetch its weights while its predecessor runs), then as few
  // as give the same number of groups per CTA. Measured on the full-size decode step: gate|up (72 tiles) 3, the input
  // projections (49 and 40 tiles of 20 groups) 5, the 2560-column projections (20 tiles) 8; each of 2, 4 and 6 in
  // place of 3 and 5 was slower, as was a ring of 68, 100 or 125 KB in place of 84.
  const int c_max = std::max(1, std::min({MAX_CS, 250 / std::max(1, c.tiles), G / 2}));
  c.cs = c_max;
  while (c.cs > 1 && (G + c.cs - 2) / (c.cs - 1) == (G + c_max - 1) / c_max) --c.cs;
  c.max_units = (G + c.cs - 1) / c.cs;
  c.unit_bytes = mma_unit_bytes(c.tn, scale_bf16);
  c.stages = std::min(c.max_units, std::max(4, (int)(((size_t)84 << 10) / c.unit_bytes)));
  c.smem = (size_t)c.stages * c.unit_bytes + (size_t)c.max_units * XB_BYTES + (size_t)((c.max_units + 3) & ~3) * 8 +
           (size_t)c.cs * c.tn * 4 + (size_t)c.tn * 4 + (size_t)(c.max_units + c.stages) * 8 + 64 + (size_t)CW * 64 * 4 + 128;
  return c;
}

}  // namespace

size_t mma_repack_bytes(int K, int N, int pair, int scale_bf16) {
  return (size_t)mma_tiles(N, pair) * (K / 128) * mma_unit_bytes(mma_tn(N, pair), scale_bf16);
}

int launch_int4_repack_mma(const uint8_t* packed, const void* scale, int scale_bf16, int K, int N, int pair, void* out,
                           cudaStream_t stream) {
  if (K % 128 != 0 || N <= 0 || (pair && N % 2 != 0)) {
    set_error("int4 repack (mma layout): K must be a multiple of 128 and N positive (even for a gate|up pair), got K=%d N=%d", K, N);
    return 2;
  }
  const int tiles = mma_tiles(N, pair), tn = mma_tn(N, pair);
  const long units = (long)tiles * (K / 128);
  if (tn == 256)
    int4_repack_mma_kernel<256><<<(unsigned)units, 256, 0, stream>>>(packed, scale, scale_bf16, K, N, pair, tiles, (unsigned char*)out,
                                                                       mma_unit_bytes(tn, scale_bf16));
  else
    int4_repack_mma_kernel<128><<<(unsigned)units, 256, 0, stream>>>(packed, scale, scale_bf16, K, N, pair, tiles, (unsigned char*)out,
                                                                       mma_unit_bytes(tn, scale_bf16));
  return check_launch("int4 repack (mma layout)");
}

// One activation row, the re-packed weight, FAST arithmetic; SwiGLU only on a gate|up pair layout and vice versa.
bool mma_path_ok(const GemvParams& p) {
  if (!(p.rows == 1 && p.packed_mma != nullptr && p.group == 128 && p.K % 128 == 0 && p.math == MATH_FAST &&
        ((uintptr_t)p.packed_mma % 16) == 0 && ((uintptr_t)p.x % 8) == 0 &&
        (p.prologue != PRO_RMSNORM || ((uintptr_t)p.norm_w % 8) == 0) && (p.prologue != PRO_SILU_MUL || ((uintptr_t)p.up % 8) == 0) &&
        (p.prologue != PRO_ATTN_MERGE || (p.merge.acc && p.merge.ml && p.merge.nclusters >= 1 && p.merge.nclusters <= 8 &&
                                          p.merge.d % 128 == 0 && p.K % p.merge.d == 0 && ((uintptr_t)p.merge.acc % 16) == 0))))
    return false;
  if ((p.epilogue == EPI_SWIGLU) != (p.mma_pair != 0)) return false;
  const MmaPlan c = plan_mma(p.K, p.N, p.mma_pair, p.scale_bf16);
  return c.smem <= (size_t)150 * 1024;
}

int mma_configure() {
  cudaError_t e = cudaSuccess;
  auto opt_in = [&e](auto kernel) {
    if (e == cudaSuccess) e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
    if (e == cudaSuccess) e = prefer_max_shared(kernel);
  };
  opt_in(gemv_mma_kernel<256>);
  opt_in(gemv_mma_kernel<128>);
  opt_in(gemv_mma_kernel<256, true>);
  opt_in(gemv_mma_kernel<128, true>);
  if (e != cudaSuccess) return check_launch("int4 gemv (mma): shared-memory opt-in");
  return 0;
}

int mma_tile_width(int N) { return mma_tn(N, 0); }

int launch_gemv_mma(const GemvParams& p, int* status, cudaStream_t stream) {
  const MmaPlan c = plan_mma(p.K, p.N, p.mma_pair, p.scale_bf16);
  MmaArgs a = {};
  a.p = p;
  a.cs = c.cs;
  a.max_units = c.max_units;
  a.num_tiles = c.tiles;
  a.stages = c.stages;
  a.unit_bytes = c.unit_bytes;
  a.status = status;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(c.tiles * c.cs, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
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
  cudaError_t e;
  if (p.prologue == PRO_ATTN_MERGE)
    e = c.tn == 256 ? cudaLaunchKernelEx(&cfg, gemv_mma_kernel<256, true>, a) : cudaLaunchKernelEx(&cfg, gemv_mma_kernel<128, true>, a);
  else
    e = c.tn == 256 ? cudaLaunchKernelEx(&cfg, gemv_mma_kernel<256>, a) : cudaLaunchKernelEx(&cfg, gemv_mma_kernel<128>, a);
  if (e != cudaSuccess) {
    set_error("int4 gemv (mma): launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  return check_launch("int4 gemv (mma)");
}

}  // namespace dfb
