// Split-KV decode attention for many sequences or long caches, on the tensor cores (head dim 256).
//
// Same result as deltaforge::split_kv_decode_attention / gqa_decode_attention on the unexpanded cache
// (src/deltaforge/kernels/flash_decode_splitkv.py:177-256, src/deltaforge/kernels/gqa_decode.py:138-199): one
// query token per sequence, (max, sum, accumulator) partials per key slice, log-sum-exp merge, optional
// output gate. The CUDA-core kernel in attn_decode.cu spends about 140 instructions per key (half of them
// the shuffles of four 256-wide dot products), which bounds it near a quarter of the HBM bandwidth once the
// cache is the step's main traffic (32 sequences x 32K tokens). Here the query heads of a KV head are the
// rows of an m16n8k16 tile (rows beyond the group are zero), so a 16-key tile costs 32 MMAs for the scores
// and 32 for P.V, and the probabilities are rounded to bf16 before P.V as in the reference
// (src/deltaforge/reference.py:660-672).
//
// Data path: one producer lane copies 16-key tiles with TMA (four 64-dim x 16-key boxes for the keys, four
// for the values, 128-byte swizzle) into a 12-stage ring, so that the 8x8 matrix loads (ldmatrix, transposed
// for V) are free of bank conflicts; tile t belongs to warp t mod 8, which frees the stage itself. (Copying
// the 32 rows of a tile one by one caps an SM near 12 GB/s: the copy engine is bound by the number of
// copies, not by their bytes.) Waits are bounded and report through the status word.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"

namespace dfb {

namespace {

constexpr int D = 256;
constexpr int MW = 8;                          // compute warps
constexpr int TK = 16;                         // keys per tile
constexpr int BOXB = TK * 128;                 // one box: 16 keys x 64 dims of bf16, 128-byte swizzled
constexpr int TILEB = 8 * BOXB;                // four key boxes, then four value boxes
constexpr int MSTAGES = 12;
constexpr int MMA_THREADS = (MW + 1) * 32;
constexpr int MMA_MAX_SPLITS = 128;
constexpr long long MMA_WAIT_CYCLES = 1LL << 28;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mma_wait(uint64_t* bar, uint32_t parity, volatile int* failed) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*failed) return false;
  const long long t0 = clock64();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 128; ++i)
      if (mbar_try_wait(bar, parity)) return true;
    if (*failed) return false;
    if (clock64() - t0 > MMA_WAIT_CYCLES) {
      *failed = 1;
      return false;
    }
  }
}
__device__ __forceinline__ void tma_box(void* dst, const CUtensorMap* map, int dim0, int key, int head, int seq, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];" ::"r"(
          smem_u32(dst)),
      "l"((uint64_t)map), "r"(dim0), "r"(key), "r"(head), "r"(seq), "r"(smem_u32(bar))
      : "memory");
}
// Byte offset of (row r, 16-byte chunk ch of the 512-byte row) inside a 4-box tile half: box ch / 8, 128-byte swizzle
__device__ __forceinline__ uint32_t swz(int r, int ch) { return (uint32_t)((ch >> 3) * BOXB + r * 128 + (((ch & 7) ^ (r & 7)) << 4)); }
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldsm4_t(uint32_t addr, uint32_t (&r)[4]) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  return (uint32_t)__bfloat16_as_ushort(f2bf(a)) | ((uint32_t)__bfloat16_as_ushort(f2bf(b)) << 16);
}

template <int GROUPS>
__global__ void __launch_bounds__(MMA_THREADS, 1) attn_decode_mma_kernel(const __grid_constant__ CUtensorMap kmap,
                                                                         const __grid_constant__ CUtensorMap vmap, const AttnParams p,
                                                                         int* status) {
  extern __shared__ unsigned char smraw0[];
  unsigned char* smraw = smraw0 + ((1024u - (smem_u32(smraw0) & 1023u)) & 1023u);  // swizzled boxes want 1024-byte alignment
  unsigned char* ring = smraw;                                   // [MSTAGES][TILEB]
  float* acc_s = (float*)smraw;                                  // [MW][GROUPS][D], reuses the ring after the scan
  float* ml_s = (float*)(smraw + (size_t)MSTAGES * TILEB);       // [MW][GROUPS][2]
  float* wgt_s = ml_s + MW * GROUPS * 2;                         // [GROUPS][MMA_MAX_SPLITS]
  uint64_t* full = (uint64_t*)(wgt_s + GROUPS * MMA_MAX_SPLITS); // [MSTAGES]
  uint64_t* empty = full + MSTAGES;                              // [MSTAGES]
  volatile int* failed = (volatile int*)(empty + MSTAGES);
  int* s_last = (int*)(empty + MSTAGES) + 1;
  // tiles the producer has issued so far. A compute warp takes every 8th tile of a 12-stage ring, so it meets a stage only
  // every other round, and a parity wait cannot tell "this round has landed" from "the round before the last has": it waits
  // for the tile to be issued first, after which the stage's barrier is in exactly this round's phase.
  volatile int* issued = (volatile int*)(empty + MSTAGES) + 2;

  const int split = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
  if (t == 0) {
    for (int s = 0; s < MSTAGES; ++s) {
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&full[s])));
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&empty[s])));
    }
    *failed = 0;
    *issued = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_launch_dependents();
  pdl_wait();  // q, the new K/V row and the position come from the kernels before this one
  const int L = p.pos ? (*p.pos + 1) : p.key_len;
  const int S = p.splits;
  const int chunk = (L + S - 1) / S;
  const int k_begin = split * chunk, k_end = min(L, k_begin + chunk);
  const int ntiles = k_end > k_begin ? (k_end - k_begin + TK - 1) / TK : 0;
  const bf16* kbase = p.kcache + (long)b * p.kv_batch_stride + (long)hk * p.kv_head_stride;
  const bf16* vbase = p.vcache + (long)b * p.kv_batch_stride + (long)hk * p.kv_head_stride;

  const int g = lane >> 2, c = lane & 3;  // MMA fragment coordinates: row (query head of the group), column pair
  float mrun = -INFINITY, lrun = 0.f;
  float o[D / 8][2];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = 0.f;

  if (warp == MW) {
    // ---------------- producer: eight boxes per tile ----------------
    if (lane == 0) {
      for (int tl = 0; tl < ntiles; ++tl) {
        const int s = tl % MSTAGES;
        if (tl >= MSTAGES && !mma_wait(&empty[s], ((tl / MSTAGES) - 1) & 1, failed)) break;
        const int key0 = k_begin + tl * TK;
        unsigned char* st = ring + (size_t)s * TILEB;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(&full[s])), "r"(TILEB) : "memory");
#pragma unroll
        for (int bx = 0; bx < 4; ++bx) {
          tma_box(st + bx * BOXB, &kmap, bx * 64, key0, hk, b, &full[s]);
          tma_box(st + (4 + bx) * BOXB, &vmap, bx * 64, key0, hk, b, &full[s]);
        }
        *issued = tl + 1;
      }
    }
  } else {
    // ---------------- compute warps ----------------
    // A fragments of the query tile: row g = query head g of the group (zero beyond it), scaled by the softmax
    // scale (a power of two for head dim 256, so the bf16 values stay exact)
    uint32_t qa[D / 16][2];
    {
      const bf16* qrow = p.q + (long)b * p.q_stride + (long)(hk * GROUPS + (g < GROUPS ? g : 0)) * p.qh_stride;
#pragma unroll
      for (int ks = 0; ks < D / 16; ++ks) {
        const float q0 = bf2f(qrow[16 * ks + 2 * c]) * p.scale, q1 = bf2f(qrow[16 * ks + 2 * c + 1]) * p.scale;
        const float q2 = bf2f(qrow[16 * ks + 8 + 2 * c]) * p.scale, q3 = bf2f(qrow[16 * ks + 8 + 2 * c + 1]) * p.scale;
        qa[ks][0] = g < GROUPS ? pack2(q0, q1) : 0u;
        qa[ks][1] = g < GROUPS ? pack2(q2, q3) : 0u;
      }
    }
    float z[2] = {0.f, 0.f};  // rows 8..15 of every accumulator tile: always zero, shared by all MMAs
    for (int tl = warp; tl < ntiles; tl += MW) {
      const int s = tl % MSTAGES;
      if (*issued <= tl) {  // (the usual case is that the producer is far ahead)
        const long long t0 = clock64();
        while (*issued <= tl && !*failed)
          if (clock64() - t0 > MMA_WAIT_CYCLES) *failed = 1;
        if (*failed) break;
      }
      if (!mma_wait(&full[s], (tl / MSTAGES) & 1, failed)) break;
      unsigned char* st = ring + (size_t)s * TILEB;
      const int key0 = k_begin + tl * TK, n = min(TK, k_end - key0);
      // (rows of a ragged last tile past the live length are cache rows that were never written, or zero
      // fill past the tensor: their scores are masked below and their value rows meet probability zero)
      // scores: S[16 x 16 keys] = Q[16 x 256] K^T, two n-tiles of 8 keys
      float sc[2][4];
#pragma unroll
      for (int nt = 0; nt < 2; ++nt) {
        sc[nt][0] = sc[nt][1] = sc[nt][2] = sc[nt][3] = 0.f;
        const uint32_t kbase_s = smem_u32(st);
        const int krow = nt * 8 + (lane & 7);
#pragma unroll
        for (int kk = 0; kk < D / 32; ++kk) {
          uint32_t kb[4];  // dims 32kk + {0..7, 8..15, 16..23, 24..31} of the 8 keys
          ldsm4(kbase_s + swz(krow, 4 * kk + (lane >> 3)), kb);
          mma_bf16(sc[nt], qa[2 * kk][0], 0u, qa[2 * kk][1], 0u, kb[0], kb[1]);
          mma_bf16(sc[nt], qa[2 * kk + 1][0], 0u, qa[2 * kk + 1][1], 0u, kb[2], kb[3]);
        }
      }
      // online softmax of row g over the 16 keys (columns 2c, 2c+1 of each n-tile are this thread's)
      float sv[4] = {sc[0][0], sc[0][1], sc[1][0], sc[1][1]};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int key = (i >> 1) * 8 + 2 * c + (i & 1);
        if (key >= n) sv[i] = -INFINITY;
      }
      float mx = fmaxf(fmaxf(sv[0], sv[1]), fmaxf(sv[2], sv[3]));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
      const float mn = fmaxf(mrun, mx);  // finite: every tile has at least one key
      const float corr = __expf(mrun - mn);
      float pv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) pv[i] = round_bf16(__expf(sv[i] - mn));  // probabilities as bf16, like the reference
      lrun = lrun * corr + (pv[0] + pv[1]) + (pv[2] + pv[3]);
      mrun = mn;
      const uint32_t pa0 = pack2(pv[0], pv[1]), pa2 = pack2(pv[2], pv[3]);
      // O[16 x 256] = O * corr + P[16 x 16 keys] V[16 keys x 256]
      const uint32_t vbase_s = smem_u32(st + 4 * BOXB);
      const int vrow = (lane & 7) + 8 * ((lane >> 3) & 1);
#pragma unroll
      for (int j2 = 0; j2 < D / 16; ++j2) {
        uint32_t vb[4];  // (keys 0..7, dims 16j2..+7), (keys 8..15, same dims), (keys 0..7, dims +8..15), (keys 8..15, ...)
        ldsm4_t(vbase_s + swz(vrow, 2 * j2 + (lane >> 4)), vb);
        float c0[4] = {o[2 * j2][0] * corr, o[2 * j2][1] * corr, z[0], z[1]};
        float c1[4] = {o[2 * j2 + 1][0] * corr, o[2 * j2 + 1][1] * corr, z[0], z[1]};
        mma_bf16(c0, pa0, 0u, pa2, 0u, vb[0], vb[1]);
        mma_bf16(c1, pa0, 0u, pa2, 0u, vb[2], vb[3]);
        o[2 * j2][0] = c0[0], o[2 * j2][1] = c0[1];
        o[2 * j2 + 1][0] = c1[0], o[2 * j2 + 1][1] = c1[1];
      }
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&empty[s])) : "memory");
    }
    lrun += __shfl_xor_sync(0xffffffffu, lrun, 1);
    lrun += __shfl_xor_sync(0xffffffffu, lrun, 2);
  }
  __syncthreads();  // every tile has been consumed: the ring becomes the warp-merge buffer
  if (warp == MW) {
    if (lane == 0 && *failed && status) atomicCAS(status, 0, 41);
    return;
  }
  if (g < GROUPS) {
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
      acc_s[(warp * GROUPS + g) * D + 8 * j + 2 * c] = o[j][0];
      acc_s[(warp * GROUPS + g) * D + 8 * j + 2 * c + 1] = o[j][1];
    }
    if (c == 0) {
      ml_s[(warp * GROUPS + g) * 2] = mrun;
      ml_s[(warp * GROUPS + g) * 2 + 1] = lrun;
    }
  }
  asm volatile("bar.sync 1, %0;" ::"n"(MW * 32) : "memory");
  float oo[GROUPS], lt[GROUPS], mt[GROUPS];  // thread t owns head dim t
#pragma unroll
  for (int gi = 0; gi < GROUPS; ++gi) {
    float mg = -INFINITY;
#pragma unroll
    for (int w = 0; w < MW; ++w) mg = fmaxf(mg, ml_s[(w * GROUPS + gi) * 2]);
    float lg = 0.f, og = 0.f;
#pragma unroll
    for (int w = 0; w < MW; ++w) {
      const float mw = ml_s[(w * GROUPS + gi) * 2];
      const float scw = (mw == -INFINITY) ? 0.f : __expf(mw - mg);
      lg += ml_s[(w * GROUPS + gi) * 2 + 1] * scw;
      og += acc_s[(w * GROUPS + gi) * D + t] * scw;
    }
    oo[gi] = og, lt[gi] = lg, mt[gi] = mg;
  }
  const int hq0 = hk * GROUPS;
  if (S > 1) {
#pragma unroll
    for (int gi = 0; gi < GROUPS; ++gi) {
      const long ph = ((long)b * p.hq + hq0 + gi) * S + split;
      __stcg(&p.part_acc[ph * D + t], oo[gi]);
      if (t == 0) {
        __stcg(&p.part_ml[ph * 2], mt[gi]);
        __stcg(&p.part_ml[ph * 2 + 1], lt[gi]);
      }
    }
    __threadfence();
    asm volatile("bar.sync 1, %0;" ::"n"(MW * 32) : "memory");
    if (t == 0) {
      unsigned* ctr = &p.counters[b * p.hkv + hk];
      const unsigned old = atomicAdd(ctr, 1u);
      *s_last = (old == (unsigned)(S - 1));
      if (*s_last) *ctr = 0u;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(MW * 32) : "memory");
    if (!*s_last) return;
    __threadfence();
    for (int gi = warp; gi < GROUPS; gi += MW) {  // log-sum-exp weights of the slices, one warp per head
      const long ph = ((long)b * p.hq + hq0 + gi) * S;
      float mloc = -INFINITY;
      for (int s = lane; s < S; s += 32) mloc = fmaxf(mloc, __ldcg(&p.part_ml[(ph + s) * 2]));
      const float mg = warp_max(mloc);
      float lloc = 0.f;
      for (int s = lane; s < S; s += 32) {
        const float ms = __ldcg(&p.part_ml[(ph + s) * 2]);
        const float scw = (ms == -INFINITY) ? 0.f : __expf(ms - mg);
        wgt_s[gi * MMA_MAX_SPLITS + s] = scw;
        lloc += __ldcg(&p.part_ml[(ph + s) * 2 + 1]) * scw;
      }
      const float inv = 1.f / warp_sum(lloc);
      for (int s = lane; s < S; s += 32) wgt_s[gi * MMA_MAX_SPLITS + s] *= inv;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(MW * 32) : "memory");
#pragma unroll
    for (int gi = 0; gi < GROUPS; ++gi) {
      const long ph = ((long)b * p.hq + hq0 + gi) * S;
      float og = 0.f;
      for (int s = 0; s < S; ++s) og = fmaf(wgt_s[gi * MMA_MAX_SPLITS + s], __ldcg(&p.part_acc[(ph + s) * D + t]), og);
      oo[gi] = og;
      lt[gi] = 1.f;
    }
  }
  // normalise, output gate (src/deltaforge/reference.py:558-568, :675-676), store
#pragma unroll
  for (int gi = 0; gi < GROUPS; ++gi) {
    float y = round_bf16(oo[gi] / lt[gi]);
    if (p.gate) {
      const float gv = bf2f(p.gate[(long)b * p.gate_stride + (long)(hq0 + gi) * p.gateh_stride + t]);
      const float gg = round_bf16(p.gate_swish ? silu_f(gv) : sigmoid_f(gv));
      y = round_bf16(__fmul_rn(y, gg));
    }
    p.out[(long)b * p.out_stride + (long)(hq0 + gi) * D + t] = f2bf(y);
  }
}

template <int GROUPS>
size_t mma_smem() {
  return (size_t)MSTAGES * TILEB + (size_t)(MW * GROUPS * 2 + GROUPS * MMA_MAX_SPLITS) * 4 + 2 * MSTAGES * 8 + 32 + 1024;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn mma_encode_fn() {
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

// The cache as a 4-D tensor [sequence][KV head][key][256] with the caller's strides; boxes are 64 dims x 16 keys.
bool encode_cache_map(CUtensorMap* map, const bf16* base, const AttnParams& p) {
  EncodeTiledFn enc = mma_encode_fn();
  if (!enc) return false;
  const cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)p.key_len, (cuuint64_t)p.hkv, (cuuint64_t)p.batch};
  const cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)p.kv_head_stride * 2, (cuuint64_t)p.kv_batch_stride * 2};
  const cuuint32_t box[4] = {64, TK, 1, 1};
  const cuuint32_t es[4] = {1, 1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, (void*)base, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int GROUPS>
int launch_mma(const AttnParams& p, int* status, cudaStream_t stream) {
  static const cudaError_t once =
      cudaFuncSetAttribute(attn_decode_mma_kernel<GROUPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)mma_smem<GROUPS>());
  if (once != cudaSuccess) return check_launch("attention decode (tensor core): shared-memory opt-in");
  CUtensorMap kmap, vmap;
  if (!encode_cache_map(&kmap, p.kcache, p) || !encode_cache_map(&vmap, p.vcache, p)) {
    set_error("attention decode (tensor core): tensor map for the cache failed");
    return 1;
  }
  if (launch_pdl(attn_decode_mma_kernel<GROUPS>, dim3(p.splits, p.hkv, p.batch), dim3(MMA_THREADS), mma_smem<GROUPS>(), stream, kmap, vmap,
                 p, status) != cudaSuccess)
    return check_launch("attention decode (tensor core)");
  return check_launch("attention decode (tensor core)");
}

}  // namespace

// Worth it once the key slices are long enough to amortise the ring: many sequences or long caches.
bool attn_mma_ok(const AttnParams& p) {
  const int groups = p.hkv > 0 ? p.hq / p.hkv : 0;
  const int cap = p.key_len;  // live length, or the cache capacity when the position is on the device
  return p.d == D && (groups == 1 || groups == 2 || groups == 4 || groups == 8) && p.splits >= 1 && p.splits <= MMA_MAX_SPLITS &&
         (p.splits == 1 || (p.part_acc && p.part_ml && p.counters)) && cap / p.splits >= 128 && (p.batch >= 2 || cap >= 16384) &&
         ((uintptr_t)p.kcache % 16) == 0 && ((uintptr_t)p.vcache % 16) == 0 && p.kv_batch_stride % 8 == 0 && p.kv_head_stride % 8 == 0 &&
         mma_encode_fn() != nullptr;
}

int launch_attn_decode_mma(const AttnParams& p, int* status, cudaStream_t stream) {
  switch (p.hq / p.hkv) {
    case 1: return launch_mma<1>(p, status, stream);
    case 2: return launch_mma<2>(p, status, stream);
    case 4: return launch_mma<4>(p, status, stream);
    default: return launch_mma<8>(p, status, stream);
  }
}

}  // namespace dfb
