// Streaming int4 dequant-GEMV for batch-1 decode, sm_100a: TMA + mbarrier ring, persistent CTAs,
// integer dot products, programmatic dependent launch.
//
// Same function as int4_gemv.cu (the reference's group-128 int4 linear, op deltaforge::tiled_gemv_int4,
// src/deltaforge/kernels/tiled_gemv.py:915-958; values and scales of quantise_int4_k_major, :242-278)
// for one activation row. It reads a re-packed copy of the weight, made once at install time by
// int4_repack_k8_kernel below from the reference's [K/2, N] byte layout: a [K/8, N] array of 32-bit
// words where word (kb, n) holds the eight nibbles of column n for rows 8kb .. 8kb+7 (nibble i = row
// 8kb + i, still value + 8). Scales stay [K/128, N].
//
//  * Arithmetic. Per 128-row scale group the activation (after the RMSNorm / SwiGLU prologue, i.e.
//    the bf16 values the reference multiplies by) is written as 16-bit integers with one shared
//    power-of-two exponent: x_k = m_k * 2^e, exact for every element within 2^-7 of the group's
//    largest and rounded at 2^-16 of it below that. m is split into a signed high byte and an unsigned
//    low byte, so sum_k nibble_k * m_k is four dp4a instructions per 8 nibbles (two byte masks, one
//    shift), exact in int32. The zero point (-8 * sum m), the exponent and the group's fp32 scale are
//    applied once per group and column; groups are summed in fp32. Like the FAST mode of
//    int4_gemv.cu the dequantised weight is never rounded to bf16.
//  * Data movement. The weight is cut into units of 1024 columns x 4 (or 2) word rows (16 or 8 KB);
//    every word row of a unit is 4 KB of contiguous HBM. Units are ordered column tile by column tile
//    and split evenly over one CTA per SM. A producer warp brings each unit in with four 2-D TMA box
//    copies into a ring of stages guarded by full/empty mbarriers; the ring is filled before the
//    kernel waits for its predecessor (griddepcontrol.wait), so under programmatic dependent launch
//    this GEMV's weights stream in while the previous kernel of the step finishes.
//  * 256 consumer threads each own 4 columns for all rows: one 16-byte shared-memory load per word row,
//    no cross-thread reduction. A tile whose rows were split between CTAs is finished by the last
//    CTA to arrive (partials added in fixed slot order), so results are identical run to run.
//
// Every wait on an mbarrier is bounded: after about two seconds the kernel records a code in the
// status word, drains its own copies and returns.
//
// Bytes per launch: K*N/2 (words) + K/128*N scale bytes + N*2 output.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>

#include "gemv_common.cuh"

namespace dfb {

namespace {

constexpr int TNW = 1024;        // columns per tile
constexpr int BOXW = 256;        // columns per TMA box (256 words = 1 KB per row)
constexpr int CTHREADS = 256;    // consumer threads, 4 columns each
constexpr int THREADS = CTHREADS + 32;
constexpr long long WAIT_LIMIT_CYCLES = 4000000000LL;  // about two seconds

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
// Bounded wait: false if the barrier did not complete the phase within the cycle budget.
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
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CTHREADS) : "memory"); }

// unsigned nibble bytes x signed / unsigned activation bytes, accumulated in int32
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
  asm("dp4a.u32.s32 %0, %1, %2, %0;" : "+r"(c) : "r"(a), "r"(b));
  return c;
}
__device__ __forceinline__ int dp4a_uu(uint32_t a, uint32_t b, int c) {
  asm("dp4a.u32.u32 %0, %1, %2, %0;" : "+r"(c) : "r"(a), "r"(b));
  return c;
}

struct StreamArgs {
  GemvParams p;
  int tiles;      // ceil(N / 1024)
  int rbc;        // units per tile = K/8 / RBK
  int units;      // tiles * rbc
  int stages;     // ring depth
  int max_slots;  // partial slots per tile
  int* status;    // device word: 0 ok, else a code from a timed-out wait
};

template <int RBK>  // word rows per unit
__global__ void __launch_bounds__(THREADS) gemv_stream_kernel(const __grid_constant__ CUtensorMap wmap, const StreamArgs a) {
  constexpr int STAGE = RBK * TNW * 4;
  extern __shared__ unsigned char smem_raw[];
  const GemvParams& p = a.p;
  const int kbn = p.K / 8, G = p.K / 128;
  unsigned char* ring = smem_raw + ((128u - (smem_u32(smem_raw) & 127u)) & 127u);  // stages * STAGE
  unsigned char* xq = ring + (size_t)a.stages * STAGE;  // [kbn][16]: hi even rows, hi odd, lo even, lo odd
  int* mk = (int*)(xq + (size_t)kbn * 16);               // [kbn] sum of the eight m of a word row
  float* fg = (float*)(mk + kbn);                        // [G] 2^e of the group
  uint64_t* full = (uint64_t*)(fg + ((G + 1) & ~1));     // [stages]
  uint64_t* empty = full + a.stages;                     // [stages]
  float* wred = (float*)(empty + a.stages);              // [8]
  int* flags = (int*)(wred + 8);                         // [0] last-arriver flag

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
  const int P = gridDim.x, c = blockIdx.x;
  const int u0 = (int)((long)c * a.units / P), u1 = (int)((long)(c + 1) * a.units / P);

  if (t == 0) {
    trace_mark(p.trace, c, 0);
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], CTHREADS / 32);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // Let the next kernel of the stream start its own prefetch as early as possible.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (warp == CTHREADS / 32) {
    // ---------------- producer: the weights do not depend on earlier kernels ----------------
    if (lane == 0) {
      const uint64_t pol = make_evict_first_policy();
      bool ok = true;
      int issued = 0;
      for (int u = u0; u < u1; ++u, ++issued) {
        const int s = issued % a.stages;
        if (issued >= a.stages) ok = mbar_wait(&empty[s], ((issued / a.stages) - 1) & 1);
        if (!ok) break;
        const int tile = u / a.rbc, rb = u % a.rbc;
        unsigned char* dst = ring + (size_t)s * STAGE;
        mbar_expect_tx(&full[s], STAGE);
#pragma unroll
        for (int b = 0; b < TNW / BOXW; ++b)
          tma_load_2d(dst + b * (RBK * BOXW * 4), &wmap, tile * TNW + b * BOXW, rb * RBK, &full[s], pol);
      }
      if (!ok) atomicExch(a.status, 1);
      // Do not leave while copies into this CTA's shared memory may still be in flight.
      const int first = issued > a.stages ? issued - a.stages : 0;
      for (int i = first; i < issued; ++i)
        if (!mbar_wait(&full[i % a.stages], (i / a.stages) & 1)) {
          atomicExch(a.status, 2);
          break;
        }
    }
    return;
  }

  // ---------------- consumers ----------------
  asm volatile("griddepcontrol.wait;" ::: "memory");  // the activation comes from the previous kernel
  if (t == 0) trace_mark(p.trace, c, 1);

  {
    float rstd = 1.f;
    if (p.prologue == PRO_RMSNORM) {
      float tot = 0.f;
      if (p.ss_in) {  // the kernel that wrote x left the sums of squares of its tiles
        for (int i = 0; i < p.ss_count; ++i) tot += p.ss_in[i];
      } else {
        float ss = 0.f;
        for (int k = t; k < p.K; k += CTHREADS) {
          const float v = bf2f(p.x[k]);
          ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) wred[warp] = ss;
        consumer_sync();
#pragma unroll
        for (int w = 0; w < CTHREADS / 32; ++w) tot += wred[w];
      }
      rstd = rsqrt_2step(__fadd_rn(__fdiv_rn(tot, (float)p.K), p.eps));
    }
    for (int kb = t; kb < kbn; kb += CTHREADS) mk[kb] = 0;
    consumer_sync();
    // one warp per group: shared exponent, 16-bit integers, bytes laid out for dp4a
    for (int g = warp; g < G; g += CTHREADS / 32) {
      float v[4];
      float amax = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        v[i] = prologue_value(p, 0, g * 128 + lane * 4 + i, rstd);
        amax = fmaxf(amax, fabsf(v[i]));
      }
      amax = warp_max(amax);
      // amax in [2^E, 2^(E+1)) -> |x| * 2^(14-E) < 2^15
      int E = amax > 0.f ? (int)((__float_as_uint(amax) >> 23) & 0xff) - 127 : 0;
      E = max(E, -100);  // keeps 2^(14-E) finite; groups this small contribute nothing measurable
      const float up = __uint_as_float((uint32_t)(127 + 14 - E) << 23);  // 2^(14-E), exact
      if (lane == 0) fg[g] = __uint_as_float((uint32_t)(127 - 14 + E) << 23);
      int msum = 0;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int m = __float2int_rn(v[i] * up);
        msum += m;
        const int k = g * 128 + lane * 4 + i, kb = k >> 3, r = k & 7;
        unsigned char* q = xq + kb * 16 + (r & 1) * 4 + (r >> 1);
        q[0] = (unsigned char)((m >> 8) & 0xff);
        q[8] = (unsigned char)(m & 0xff);
      }
      msum += __shfl_xor_sync(0xffffffffu, msum, 1);  // lanes 2j, 2j+1 share word row g*16 + j
      if ((lane & 1) == 0) mk[g * 16 + (lane >> 1)] = msum;
    }
    consumer_sync();
  }

  if (t == 0) trace_mark(p.trace, c, 2);
  const int n0 = (t << 2);  // first of this thread's 4 columns inside the tile
  const int box_off = (t >> 6) * (RBK * BOXW * 4) + (t & 63) * 16;
  float tot[4] = {0.f, 0.f, 0.f, 0.f};
  int acc_h[4] = {0, 0, 0, 0}, acc_l[4] = {0, 0, 0, 0};
  int msum = 0;
  float sc[4] = {0.f, 0.f, 0.f, 0.f};
  int sc_group = -1;
  int tile_first_rb = -1;
  bool ok = true;

  // (tile, rb) of the unit, the ring stage and its phase advance by increments: no division in the loop
  int tile = u0 / a.rbc, rb = u0 % a.rbc, s = 0, phase = 0;
  auto advance = [&]() {
    if (++rb == a.rbc) rb = 0, ++tile;
    if (++s == a.stages) s = 0, phase ^= 1;
  };
  for (int u = u0; u < u1; ++u, advance()) {
    const int kb0 = rb * RBK, g = kb0 >> 4;
    const int ncol = tile * TNW + n0;
    if (tile_first_rb < 0) tile_first_rb = rb;
    if (sc_group != g) {  // this group's scales, needed when the group is flushed
      sc_group = g;
      if (ncol < p.N) {  // N % 4 == 0: a thread's 4 columns are inside or outside together
        if (p.scale_bf16) {
          const uint2 v = __ldg((const uint2*)((const bf16*)p.scale + (long)g * p.N + ncol));
          sc[0] = __uint_as_float(v.x << 16), sc[1] = __uint_as_float(v.x & 0xffff0000u);
          sc[2] = __uint_as_float(v.y << 16), sc[3] = __uint_as_float(v.y & 0xffff0000u);
        } else {
          const float4 v = __ldg((const float4*)((const float*)p.scale + (long)g * p.N + ncol));
          sc[0] = v.x, sc[1] = v.y, sc[2] = v.z, sc[3] = v.w;
        }
      }
    }
    ok = mbar_wait(&full[s], phase);
    if (!ok) break;
    const unsigned char* wbase = ring + (size_t)s * STAGE + box_off;
#pragma unroll
    for (int r = 0; r < RBK; ++r) {
      const uint4 xw = *(const uint4*)(xq + (kb0 + r) * 16);
      const uint4 w4 = *(const uint4*)(wbase + r * (BOXW * 4));
      msum += mk[kb0 + r];
      const uint32_t wv[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint32_t ne = wv[q] & 0x0F0F0F0Fu, no = (wv[q] >> 4) & 0x0F0F0F0Fu;
        acc_h[q] = dp4a_us(ne, xw.x, acc_h[q]);
        acc_h[q] = dp4a_us(no, xw.y, acc_h[q]);
        acc_l[q] = dp4a_uu(ne, xw.z, acc_l[q]);
        acc_l[q] = dp4a_uu(no, xw.w, acc_l[q]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty[s]);

    const bool tile_done = (u + 1 == u1) || (rb + 1 == a.rbc);
    const bool group_done = tile_done || (((kb0 + RBK) & 15) == 0);
    if (group_done) {
      const float f = fg[g];
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int S = acc_h[q] * 256 + acc_l[q] - 8 * msum;  // sum (nibble - 8) * m, exact
        tot[q] = fmaf((float)S * f, sc[q], tot[q]);
        acc_h[q] = acc_l[q] = 0;
      }
      msum = 0;
    }
    if (!tile_done) continue;

    const bool whole = (tile_first_rb == 0) && (rb == a.rbc - 1);
    if (whole) {
#pragma unroll
      for (int q = 0; q < 4; ++q)
        if (ncol + q < p.N) epilogue_store(p, 0, ncol + q, tot[q]);
    } else {
      // contributors of this tile are consecutive CTAs c_lo..c_hi; slot = c - c_lo
      const long A = (long)tile * a.rbc, B = A + a.rbc;
      const int c_lo = (int)(((A + 1) * P + a.units - 1) / a.units) - 1;
      const int c_hi = (int)((B * P + a.units - 1) / a.units) - 1;
      const int ncontrib = c_hi - c_lo + 1, slot = c - c_lo;
      float* part = p.partials + ((long)tile * a.max_slots) * TNW;
      __stcg((float4*)(part + (long)slot * TNW + n0), make_float4(tot[0], tot[1], tot[2], tot[3]));
      __threadfence();
      consumer_sync();
      if (t == 0) {
        const unsigned old = atomicAdd(&p.counters[tile], 1u);
        const int last = (old == (unsigned)(ncontrib - 1));
        if (last) p.counters[tile] = 0u;
        flags[0] = last;
      }
      consumer_sync();
      if (flags[0]) {
        __threadfence();
        float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sidx = 0; sidx < ncontrib; ++sidx) {
          const float4 v = __ldcg((const float4*)(part + (long)sidx * TNW + n0));
          sum.x += v.x, sum.y += v.y, sum.z += v.z, sum.w += v.w;
        }
        const float o[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
        for (int q = 0; q < 4; ++q)
          if (ncol + q < p.N) epilogue_store(p, 0, ncol + q, o[q]);
      }
      consumer_sync();  // flags[0] is reused by the next shared tile
    }
    tot[0] = tot[1] = tot[2] = tot[3] = 0.f;
    tile_first_rb = -1;
    sc_group = -1;
  }
  if (!ok && lane == 0) atomicExch(a.status, 3);
  if (t == 0) trace_mark(p.trace, c, 6);
}

// reference layout [K/2, N] bytes (row j low nibble, row j + K/2 high nibble) -> [K/8, N] words
__global__ void int4_repack_k8_kernel(const uint8_t* packed, int K, int N, uint32_t* out) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const long total = (long)(K / 8) * N;
  if (idx >= total) return;
  const int kb = (int)(idx / N), n = (int)(idx % N);
  const int half = K / 2;
  uint32_t w = 0;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = kb * 8 + i;
    const uint32_t byte = packed[(size_t)(r < half ? r : r - half) * N + n];
    const uint32_t nib = r < half ? (byte & 15u) : (byte >> 4);
    w |= nib << (4 * i);
  }
  out[idx] = w;
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

int sm_count() {
  static int n = []() {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      return 0;
    return v;
  }();
  return n;
}

int pick_rbk(int K, int N) {
  // 16 KB units unless that leaves fewer than about four units per SM
  const long units4 = (long)((N + TNW - 1) / TNW) * (K / 32);
  return units4 >= 4L * std::max(sm_count(), 1) ? 4 : 2;
}

size_t smem_needed(int K, int rbk, int stages) {
  const int kbn = K / 8, G = K / 128;
  return (size_t)stages * rbk * TNW * 4 + (size_t)kbn * 16 + (size_t)kbn * 4 + (size_t)((G + 1) & ~1) * 4 + (size_t)stages * 16 +
         8 * 4 + 16 + 128;
}

int pick_stages(int K, int rbk) {
  // Two of these CTAs (this GEMV and the next one prefetching) should fit in one SM's 227 KB.
  const size_t budget = 72 * 1024;  // three CTAs per SM
  int stages = rbk == 4 ? 3 : 6;
  while (stages > 2 && smem_needed(K, rbk, stages) > budget) --stages;
  return stages;
}

template <int RBK>
int launch_stream_rbk(const GemvParams& p, int* status, cudaStream_t stream) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) {
    set_error("int4 gemv: cuTensorMapEncodeTiled is not available from this driver");
    return 1;
  }
  CUtensorMap wmap;
  const cuuint64_t dims[2] = {(cuuint64_t)p.N, (cuuint64_t)(p.K / 8)};
  const cuuint64_t strides[1] = {(cuuint64_t)p.N * 4};
  const cuuint32_t box[2] = {BOXW, (cuuint32_t)RBK};
  const cuuint32_t es[2] = {1, 1};
  const CUresult r = enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, (void*)p.packed_k8, dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error("int4 gemv: tensor map for the re-packed weight failed (code %d)", (int)r);
    return 1;
  }
  StreamArgs a = {};
  a.p = p;
  a.tiles = (p.N + TNW - 1) / TNW;
  a.rbc = (p.K / 8) / RBK;
  a.units = a.tiles * a.rbc;
  a.stages = pick_stages(p.K, RBK);
  // three CTAs per SM: 24 consumer warps hide the shared-memory and dp4a latencies one CTA cannot
  constexpr int CTAS_PER_SM = 3;
  a.status = status;
  a.max_slots = stream_max_slots(p.K, p.N);
  const int P = std::min(sm_count() * CTAS_PER_SM, a.units);
  const size_t smem = smem_needed(p.K, RBK, a.stages);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(P, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_stream_kernel<RBK>, wmap, a);
  if (e != cudaSuccess) {
    set_error("int4 gemv (stream): launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  return check_launch("int4 gemv (stream)");
}

}  // namespace

bool stream_path_ok(const GemvParams& p) {
  return p.rows == 1 && p.packed_k8 != nullptr && p.group == 128 && p.K % 256 == 0 && p.N % 4 == 0 &&
         ((uintptr_t)p.packed_k8 % 16) == 0 && ((uintptr_t)p.scale % 16) == 0 && p.math == MATH_FAST && p.K <= 16384 &&
         sm_count() > 0;
}

int stream_max_slots(int K, int N) {
  const int rbk = pick_rbk(K, N);
  const long rbc = (K / 8) / rbk;
  const long units = (long)((N + TNW - 1) / TNW) * rbc;
  const long P = std::min<long>(8L * std::max(sm_count(), 1), units);  // upper bound on the grid, whatever CTAs/SM is chosen
  const long per_cta = std::max<long>(units / P, 1);
  return (int)std::min<long>(P, rbc / per_cta + 2);
}

size_t stream_partials_bytes(int K, int N) {
  return (size_t)((N + TNW - 1) / TNW) * stream_max_slots(K, N) * TNW * sizeof(float);
}
size_t stream_counter_count(int K, int N) {
  (void)K;
  return (size_t)((N + TNW - 1) / TNW);
}

int stream_configure() {
  cudaError_t e = cudaFuncSetAttribute(gemv_stream_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  if (e == cudaSuccess) e = cudaFuncSetAttribute(gemv_stream_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  if (e == cudaSuccess) e = prefer_max_shared(gemv_stream_kernel<4>);
  if (e == cudaSuccess) e = prefer_max_shared(gemv_stream_kernel<2>);
  if (e != cudaSuccess) return check_launch("int4 gemv (stream): shared-memory opt-in");
  if (!encode_fn()) {
    set_error("int4 gemv (stream): cuTensorMapEncodeTiled is not available from this driver");
    return 1;
  }
  return 0;
}

int launch_gemv_stream(const GemvParams& p, int* status, cudaStream_t stream) {
  if (pick_rbk(p.K, p.N) == 4) return launch_stream_rbk<4>(p, status, stream);
  return launch_stream_rbk<2>(p, status, stream);
}

int launch_int4_repack_k8(const uint8_t* packed, int K, int N, uint32_t* out, cudaStream_t stream) {
  const long total = (long)(K / 8) * N;
  if (total == 0) return 0;
  int4_repack_k8_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(packed, K, N, out);
  return check_launch("int4 repack");
}

}  // namespace dfb
