// Group-wise int4 x bf16 product for 8..128 activation rows on the sm_100a tensor cores (tcgen05 + TMEM).
//
// Same contract as the GEMV kernels (y = x @ dequant(W), src/deltaforge/kernels/visible_int4_head.py:187-199,
// op deltaforge::tiled_gemv_int4 at src/deltaforge/kernels/tiled_gemv.py:915-958) for the row counts where one
// weight tile is shared by enough rows that the arithmetic belongs on the tensor cores (decode batches of 8
// and more). The weight is never materialised in bf16 in global memory: a CTA streams a 128-column slab of
// the re-packed int4 words through shared memory, 8 warps turn each 64-row block into the bf16 values the
// reference holds (bf16(fp32(q) * fp32(scale)), every one bit-identical) and write them as the K-major,
// 128-byte-swizzled A operand of tcgen05.mma; the activation rows are the B operand (TMA, same swizzle), so
// the MMA is M = 128 weight columns x N = rows (padded to 16) x K = 16, and the fp32 accumulator lives in
// TMEM: D[column, row]. One thread issues the MMAs, tcgen05.commit releases the stage to the producer, and
// after the last block the 8 warps read the accumulator back (tcgen05.ld), round to bf16 and store
// (optionally adding a residual), or, under split-K, park fp32 partial sums for the last CTA of the tile.
//
// Bytes per launch: K*N/2 (words) + K/128*N*scale_bytes + rows*K*2 per column tile (L2) + rows*N*2.
// Waits are bounded: a barrier that does not complete sets the status word and the CTA winds down.
#include <cuda.h>

#include <algorithm>

#include "gemv_common.cuh"

namespace dfb {

namespace {

constexpr int TM = 128;            // weight columns per CTA (UMMA M)
constexpr int BK = 64;             // k per block: one 128-byte swizzle row of bf16
constexpr int DQ_WARPS = 8;        // dequant / epilogue warps
constexpr int TC_THREADS = (DQ_WARPS + 2) * 32;
constexpr int A_BYTES = TM * BK * 2;          // 16 KB
constexpr int PK_BYTES = (BK / 8) * TM * 4;   // 4 KB of packed words per block
constexpr long long TC_WAIT_CYCLES = 1LL << 28;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
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
// Bounded wait; on giving up records `code` and raises the CTA-wide flag every other wait checks.
__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity, volatile int* failed, int* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*failed) return false;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 128; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*failed) return false;
    if (clock64() - t0 > TC_WAIT_CYCLES) {
      *failed = 1;
      if (status) atomicCAS(status, 0, code);
      return false;
    }
  }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                   smem_u32(dst)),
               "l"((uint64_t)map), "r"(x), "r"(y), "r"(smem_u32(bar))
               : "memory");
}

// Shared-memory matrix descriptor of a K-major tile whose rows are one 128-byte swizzle span: 8-row groups
// are 1024 bytes apart (stride byte offset), the leading byte offset is unused for this layout.
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);   // start address
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset
  d |= 1ull << 46;                               // descriptor version of sm_100
  d |= 2ull << 61;                               // 128-byte swizzle
  return d;
}
// Instruction descriptor for kind::f16: D fp32, A and B bf16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t umma_idesc_bf16(int n) {
  uint32_t d = 0;
  d |= 1u << 4;                    // D format: f32
  d |= 1u << 7;                    // A format: bf16
  d |= 1u << 10;                   // B format: bf16
  d |= (uint32_t)(n >> 3) << 17;   // N / 8
  d |= (uint32_t)(TM >> 4) << 24;  // M / 16
  return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

struct TcArgs {
  GemvParams p;
  int mt;         // rows padded to a multiple of 16 (UMMA N)
  int tmem_cols;  // power of two >= max(32, mt)
  int stages;
  int splits;     // split-K factor (gridDim.y)
  int kblocks;    // K / 64
  int* status;
};

__global__ void __launch_bounds__(TC_THREADS, 2) int4_gemm_tc_kernel(const __grid_constant__ CUtensorMap wmap,
                                                                     const __grid_constant__ CUtensorMap xmap, const TcArgs a) {
  extern __shared__ unsigned char smem_raw[];
  const GemvParams& p = a.p;
  unsigned char* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  const int b_bytes = a.mt * BK * 2;
  const int stage_bytes = A_BYTES + b_bytes + PK_BYTES;
  unsigned char* tail = sm + (size_t)a.stages * stage_bytes;
  uint64_t* full = (uint64_t*)tail;             // [stages] packed words + activation tile landed
  uint64_t* a_ready = full + a.stages;          // [stages] bf16 A tile written
  uint64_t* freed = a_ready + a.stages;         // [stages] the MMAs reading the stage are done
  uint64_t* acc_ready = freed + a.stages;       // [1]
  uint32_t* tmem_slot = (uint32_t*)(acc_ready + 1);
  volatile int* failed = (volatile int*)(tmem_slot + 1);
  int* s_last = (int*)(tmem_slot + 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
  const int tile = blockIdx.x, split = blockIdx.y;
  const int n0 = tile * TM;
  const int kb0 = (int)((long)split * a.kblocks / a.splits), kb1 = (int)((long)(split + 1) * a.kblocks / a.splits);
  const int nblocks = kb1 - kb0;

  if (t == 0) {
    for (int s = 0; s < a.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&a_ready[s], DQ_WARPS);
      mbar_init(&freed[s], 1);
    }
    mbar_init(acc_ready, 1);
    *failed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == DQ_WARPS + 1) {  // the MMA warp owns the tensor-memory allocation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(a.tmem_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;
  pdl_launch_dependents();  // the next kernel may set itself up; it waits for this grid before it touches its inputs

  if (warp == DQ_WARPS) {
    // ---------------- producer: packed words of the slab and the activation tile of every k block ----------------
    if (lane == 0) {
      // The weights never depend on earlier kernels: the first ring of packed words goes in flight before the wait for the
      // kernel that writes the activation (this kernel is launched with programmatic dependent launch).
      const int pre = min(nblocks, a.stages);
      for (int i = 0; i < pre; ++i) {
        unsigned char* st = sm + (size_t)i * stage_bytes;
        mbar_expect_tx(&full[i], PK_BYTES + b_bytes);
        tma_load_2d(st + A_BYTES + b_bytes, &wmap, n0, (kb0 + i) * (BK / 8), &full[i]);
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i) tma_load_2d(sm + (size_t)i * stage_bytes + A_BYTES, &xmap, (kb0 + i) * BK, 0, &full[i]);
      for (int i = pre; i < nblocks; ++i) {
        const int s = i % a.stages;
        if (!tc_wait(&freed[s], ((i / a.stages) - 1) & 1, failed, a.status, 31)) break;
        unsigned char* st = sm + (size_t)s * stage_bytes;
        mbar_expect_tx(&full[s], PK_BYTES + b_bytes);
        tma_load_2d(st + A_BYTES + b_bytes, &wmap, n0, (kb0 + i) * (BK / 8), &full[s]);
        tma_load_2d(st + A_BYTES, &xmap, (kb0 + i) * BK, 0, &full[s]);
      }
    }
  } else if (warp == DQ_WARPS + 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(a.mt);
      bool ok = true;
      for (int i = 0; i < nblocks && ok; ++i) {
        const int s = i % a.stages;
        const uint32_t par = (i / a.stages) & 1;
        ok = tc_wait(&full[s], par, failed, a.status, 32) && tc_wait(&a_ready[s], par, failed, a.status, 33);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = smem_u32(sm + (size_t)s * stage_bytes), b_addr = a_addr + A_BYTES;
#pragma unroll
        for (int k = 0; k < BK / 16; ++k)
          umma_bf16(tmem_base, umma_desc_sw128(a_addr + k * 32), umma_desc_sw128(b_addr + k * 32), idesc, (i | k) != 0);
        umma_commit(&freed[s]);  // arrives when the MMAs issued so far have finished reading shared memory
      }
      if (ok) umma_commit(acc_ready);
    }
  } else {
    // ---------------- dequant warps: packed words -> the bf16 A tile the reference would hold ----------------
    const int n = t & (TM - 1), half = t >> 7;  // column of the slab; word rows half*4 .. half*4+3 of the block
    const bool col_ok = n0 + n < p.N;
    // a scale group is two k blocks; the next group's scale is requested a group ahead of its use
    const int last_group = (kb1 - 1) >> 1;
    float sc = col_ok && nblocks > 0 ? load_scale(p, (long)(kb0 >> 1) * p.N + n0 + n) : 0.f;
    float sc_next = sc;
    bool ok = true;
    for (int i = 0; i < nblocks; ++i) {
      const int s = i % a.stages;
      const int kb = kb0 + i;
      if (i > 0 && (kb & 1) == 0) sc = sc_next;
      if (i == 0 || (kb & 1) == 0) {
        const int g_next = (kb >> 1) + 1;
        if (col_ok && g_next <= last_group) sc_next = load_scale(p, (long)g_next * p.N + n0 + n);
      }
      ok = tc_wait(&full[s], (i / a.stages) & 1, failed, a.status, 34);
      if (!ok) break;
      unsigned char* st = sm + (size_t)s * stage_bytes;
      const uint32_t* pk = (const uint32_t*)(st + A_BYTES + b_bytes);
      uint32_t w[4];
#pragma unroll
      for (int r = 0; r < 4; ++r) w[r] = pk[(half * 4 + r) * TM + n];
      unsigned char* arow = st + (n >> 3) * 1024 + (n & 7) * 128;
      if (p.scale_bf16) {
        // bf16 scales: (128 + nibble) is a bf16 number whose low mantissa bits are the nibble, minus 136 is
        // exactly nibble - 8, and one bf16 multiply rounds (nibble - 8) * scale once, like the reference's
        // fp32 product followed by the conversion (the product of a 4-bit and an 8-bit mantissa is exact in fp32).
        const __nv_bfloat162 s2 = __float2bfloat162_rn(sc);
        __nv_bfloat162 c136;
        *(uint32_t*)&c136 = 0x43084308u;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          uint32_t v[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {  // nibbles j and j + 4 of the word
            __nv_bfloat162 tq;
            *(uint32_t*)&tq = and_or(w[r] >> (4 * j), 0x000F000Fu, 0x43004300u);
            const __nv_bfloat162 y = __hmul2(__hsub2(tq, c136), s2);
            v[j] = *(const uint32_t*)&y;
          }
          // (k0,k4) (k1,k5) (k2,k6) (k3,k7) -> (k0,k1) (k2,k3) (k4,k5) (k6,k7)
          const uint4 o = make_uint4(__byte_perm(v[0], v[1], 0x5410), __byte_perm(v[2], v[3], 0x5410), __byte_perm(v[0], v[1], 0x7632),
                                     __byte_perm(v[2], v[3], 0x7632));
          const int chunk = (half * 4 + r) ^ (n & 7);
          *(uint4*)(arow + chunk * 16) = o;
        }
      } else {
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          // nibble - 8 as fp32 without an integer conversion: 2^23 + nibble, minus (2^23 + 8)
          const float q0 = __uint_as_float(0x4B000000u | ((w[r] >> (8 * j)) & 15u)) - 8388616.0f;
          const float q1 = __uint_as_float(0x4B000000u | ((w[r] >> (8 * j + 4)) & 15u)) - 8388616.0f;
          const uint32_t lo = __bfloat16_as_ushort(f2bf(__fmul_rn(q0, sc))), hi = __bfloat16_as_ushort(f2bf(__fmul_rn(q1, sc)));
          o[j] = lo | (hi << 16);
        }
        const int chunk = (half * 4 + r) ^ (n & 7);  // 128-byte swizzle: 16-byte chunk index xor row within the 8-row group
        *(uint4*)(arow + chunk * 16) = make_uint4(o[0], o[1], o[2], o[3]);
      }
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the tensor core
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_ready[s]);
    }

    // ---------------- epilogue: accumulator D[column, row] -> y[row, column] ----------------
    if (ok) ok = tc_wait(acc_ready, 0, failed, a.status, 35);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int quarter = warp & 3, chalf = warp >> 2;  // TMEM lanes 32*quarter.., accumulator columns of this half
    const int ncol = n0 + quarter * 32 + lane;
    const int c_begin = chalf * (a.mt / 2), c_end = c_begin + a.mt / 2;
    if (ok) {
      for (int c = c_begin; c < c_end; c += 8) {
        float v[8];
        tmem_ld8(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c, v);
        if (ncol >= p.N) continue;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int m = c + j;
          if (m >= p.rows) break;
          if (a.splits == 1)
            epilogue_store(p, m, ncol, v[j]);
          else
            __stcg(&p.partials[((long)split * p.rows + m) * p.N + ncol], v[j]);
        }
      }
    }
    if (a.splits > 1) {
      // the last CTA of the column tile adds the partial sums in split order and applies the epilogue
      __threadfence();
      asm volatile("bar.sync 1, %0;" ::"n"(DQ_WARPS * 32) : "memory");
      if (t == 0) {
        const unsigned old = atomicAdd(&p.counters[tile], 1u);
        *s_last = (old == (unsigned)(a.splits - 1));
        if (*s_last) p.counters[tile] = 0u;
      }
      asm volatile("bar.sync 1, %0;" ::"n"(DQ_WARPS * 32) : "memory");
      if (*s_last && ok) {
        __threadfence();
        const int col = n0 + (t & (TM - 1));
        if (col < p.N)
          for (int m = t >> 7; m < p.rows; m += 2) {
            // eight partial sums in flight at a time, added in split order
            float sum = 0.f;
            for (int sp0 = 0; sp0 < a.splits; sp0 += 8) {
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j)
                v[j] = sp0 + j < a.splits ? __ldcg(&p.partials[((long)(sp0 + j) * p.rows + m) * p.N + col]) : 0.f;
#pragma unroll
              for (int j = 0; j < 8; ++j) sum += v[j];
            }
            epilogue_store(p, m, col, sum);
          }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == DQ_WARPS + 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(a.tmem_cols) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn tc_encode_fn() {
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

int tc_sm_count() {
  static int n = []() {
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      return 0;
    return v;
  }();
  return n;
}

int tc_splits(const GemvParams& p) {
  const int tiles = (p.N + TM - 1) / TM, kblocks = p.K / BK, sms = std::max(tc_sm_count(), 1);
  // two CTAs per SM (16 dequantising warps), at least four k blocks each, within the split-K scratch (K / 256
  // slabs), and the partial sums (written and read once) may cost at most half of what the weights cost
  const long weight_bytes = (long)p.K * p.N / 2, split_bytes = (long)p.rows * p.N * 8;
  const int by_traffic = (int)std::max<long>(1, weight_bytes / (2 * split_bytes));
  return std::max(1, std::min({(2 * sms) / tiles, kblocks / 4, p.K / 256, by_traffic}));
}

}  // namespace

bool tc_path_ok(const GemvParams& p) {
  return p.rows >= 8 && p.rows <= 128 && p.packed_k8 != nullptr && p.group == 128 && p.K % 128 == 0 && p.N % 4 == 0 &&
         p.x_stride % 8 == 0 && ((uintptr_t)p.x % 16) == 0 && ((uintptr_t)p.packed_k8 % 16) == 0 && p.prologue == PRO_NONE &&
         (p.epilogue == EPI_STORE || p.epilogue == EPI_RESIDUAL) && p.math != MATH_FAST_HALF2 && tc_encode_fn() != nullptr &&
         (tc_splits(p) == 1 || (p.partials != nullptr && p.counters != nullptr));
}

int tc_configure() {
  cudaError_t e = cudaFuncSetAttribute(int4_gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
  return e == cudaSuccess ? 0 : check_launch("int4 gemm (tensor core): shared-memory opt-in");
}

int launch_gemm_tc(const GemvParams& p, int* status, cudaStream_t stream) {
  EncodeTiledFn enc = tc_encode_fn();
  if (!enc) {
    set_error("int4 gemm: cuTensorMapEncodeTiled is not available from this driver");
    return 1;
  }
  TcArgs a = {};
  a.p = p;
  a.mt = (p.rows + 15) / 16 * 16;
  a.tmem_cols = 32;
  while (a.tmem_cols < a.mt) a.tmem_cols *= 2;
  a.kblocks = p.K / BK;
  a.splits = tc_splits(p);
  a.status = status;
  const int stage_bytes = A_BYTES + a.mt * BK * 2 + PK_BYTES;
  a.stages = std::max(2, std::min(4, (104 * 1024) / stage_bytes));  // two CTAs fit an SM
  CUtensorMap wmap, xmap;
  {
    const cuuint64_t dims[2] = {(cuuint64_t)p.N, (cuuint64_t)(p.K / 8)};
    const cuuint64_t strides[1] = {(cuuint64_t)p.N * 4};
    const cuuint32_t box[2] = {TM, BK / 8};
    const cuuint32_t es[2] = {1, 1};
    const CUresult r = enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, (void*)p.packed_k8, dims, strides, box, es,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      set_error("int4 gemm: tensor map for the re-packed weight failed (code %d)", (int)r);
      return 1;
    }
  }
  {
    const cuuint64_t dims[2] = {(cuuint64_t)p.K, (cuuint64_t)p.rows};
    const cuuint64_t strides[1] = {(cuuint64_t)p.x_stride * 2};
    const cuuint32_t box[2] = {BK, (cuuint32_t)a.mt};
    const cuuint32_t es[2] = {1, 1};
    const CUresult r = enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)p.x, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      set_error("int4 gemm: tensor map for the activation failed (code %d)", (int)r);
      return 1;
    }
  }
  const size_t smem = (size_t)a.stages * stage_bytes + (3 * a.stages + 1) * 8 + 64 + 1024;
  dim3 grid((p.N + TM - 1) / TM, a.splits, 1);
  if (launch_pdl(int4_gemm_tc_kernel, grid, dim3(TC_THREADS), smem, stream, wmap, xmap, a) != cudaSuccess)
    return check_launch("int4 gemm (tensor core)");
  return check_launch("int4 gemm (tensor core)");
}

}  // namespace dfb
