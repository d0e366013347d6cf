// Group-wise int4 dequant-GEMV for the decode step, sm_100a.
//
// Computes y[r, n] = sum_k x[r, k] * (nibble[k, n] - 8) * scale[k / group, n] on the weight layout
// of the reference's K-major int4 format (src/deltaforge/kernels/tiled_gemv.py:242-288): packed is
// [K/2, N] uint8 with N contiguous, byte [j, n] holds row j in its low nibble and row j + K/2 in
// its high nibble, scale is [K/group, N]. It replaces the reference's Triton GEMV
// (tiled_gemv.py:654-774, op deltaforge::tiled_gemv_int4 at :915-958) and the torch expression
// torch_dequant_gemv_int4 (src/deltaforge/kernels/visible_int4_head.py:187-199).
//
// Fast path (group 128, K % 256 == 0, N % 8 == 0). One CTA of 256 threads owns a tile of 256
// columns by 128 packed rows, i.e. exactly one scale group of the low half and one of the high
// half. Each lane loads 8 bytes per row (a warp row is 256 contiguous bytes), each warp owns 16
// rows, and all 16 loads of a thread are issued before anything else happens, so the whole tile is
// in flight while the CTA builds its slice of the activation vector (with the RMSNorm or SwiGLU
// prologue) in shared memory. Nibbles become fp16 values 1024 + n (or 1024 + 16 n for the high
// nibble) by one logic op per pair, and are multiplied with the fp16 activation by the sm_100
// mixed-precision FMA (f16 x f16 + f32), accumulating in fp32; the 1024 bias and the -8 zero point
// are removed once per group from the activation sum, and the group's fp32 scale is applied once
// per column. Warps are reduced through padded shared memory, split-K partial sums go to an fp32
// scratch buffer, and the last CTA to arrive for a column tile adds them in fixed order (no
// atomics on data, so results are identical run to run) and applies the epilogue: store, residual
// add, or the DeltaNet causal-conv + SiLU step.
//
// Bytes per launch (what the roofline is computed from): K*N/2 packed + K/group*N scale bytes
// + rows*N*2 output; the activation vector is re-read from L2 by every CTA and is not counted.
#include <algorithm>
#include <mutex>

#include "../../include/dfb200.h"
#include "gemv_common.cuh"

namespace dfb {

namespace {

constexpr int TN = 256;             // columns per CTA
constexpr int GROUP_ROWS = 128;     // packed rows per CTA = one scale group per half
constexpr int NWARP = 8;
constexpr int RPW = GROUP_ROWS / NWARP;  // rows per warp
constexpr int PADW = TN + TN / 32;       // padded row of the cross-warp reduction buffer

// rsqrt(mean(x^2) + eps) of row r, computed by the whole CTA (blockDim.x threads, <= 32 warps).
__device__ float cta_rstd(const GemvParams& p, int r, float* warp_scratch) {
  float ss = 0.f;
  for (int k = threadIdx.x; k < p.K; k += blockDim.x) {
    float v = bf2f(p.x[(long)r * p.x_stride + k]);
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) warp_scratch[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += warp_scratch[w];
  return rsqrt_2step(__fadd_rn(__fdiv_rn(tot, (float)p.K), p.eps));
}

template <int ROWS, int MATH>
__global__ void __launch_bounds__(NWARP * 32) gemv_g128_kernel(const GemvParams p) {
  extern __shared__ float smem[];
  float* red = smem;                                  // [ROWS][2][NWARP][PADW]
  float* xs_f = red + ROWS * 2 * NWARP * PADW;        // [ROWS][2][128] activation slice, fp32
  __half* xs_h = (__half*)(xs_f + ROWS * 2 * 128);    // [ROWS][2][128] same, fp16
  float* wsum = (float*)(xs_h + ROWS * 2 * 128);      // [ROWS][NWARP] per-warp activation sums
  float* wscr = wsum + ROWS * NWARP;                  // [NWARP] scratch for the row statistic
  __shared__ int s_last;
  __shared__ float wmaxs[ROWS * NWARP];  // per-warp largest |activation|
  __shared__ float upf[ROWS * 2];        // power of two each half-group's fp16 activations were scaled down by

  const int tile = blockIdx.x, g = blockIdx.y, zb = blockIdx.z;
  const int G = p.K / 256, half = p.K / 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, t = threadIdx.x;
  const int col0 = tile * TN + lane * 8;
  const bool col_ok = col0 < p.N;
  const int row0 = zb * ROWS;

  // 1. Put this thread's 16 x 8 bytes of the weight tile in flight.
  const uint64_t pol = make_evict_first_policy();
  uint2 w[RPW];
  {
    const uint8_t* wp = p.packed + (size_t)(g * GROUP_ROWS + warp * RPW) * p.N + col0;
#pragma unroll
    for (int i = 0; i < RPW; ++i)
      w[i] = col_ok ? ldg_stream_u2(wp + (size_t)i * p.N, pol) : make_uint2(0x88888888u, 0x88888888u);
  }
  float sL[8], sH[8];
  if (MATH == MATH_EXACT) {
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      sL[c] = col_ok ? load_scale(p, (long)g * p.N + col0 + c) : 0.f;
      sH[c] = col_ok ? load_scale(p, (long)(g + G) * p.N + col0 + c) : 0.f;
    }
  }

  // 2. The 128 + 128 activation values this tile multiplies, after the prologue.
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    const int row = row0 + r;
    float v = 0.f;
    if (row < p.rows) {
      float rstd = 1.f;
      if (p.prologue == PRO_RMSNORM) rstd = cta_rstd(p, row, wscr);
      const int kind = t >> 7, j = t & 127;
      v = prologue_value(p, row, kind * half + g * GROUP_ROWS + j, rstd);
    }
    xs_f[r * 256 + t] = v;
    if (MATH == MATH_EXACT) {
      const float s = warp_sum(v);
      if (lane == 0) wsum[r * NWARP + warp] = s;
    } else {
      const float am = warp_max(fabsf(v));
      if (lane == 0) wmaxs[r * NWARP + warp] = am;
    }
  }
  __syncthreads();
  if (MATH != MATH_EXACT) {
    // The fp16 forms keep the activation as fp16. A half-group (128 values) whose largest magnitude reaches 2^14 (2^10
    // in the packed-fp16 form) is scaled down by a power of two first, so that nothing overflows (65504) where the reference's bf16 stays finite;
    // the factor goes back on after the group's sum. Below that nothing is scaled and the bits are what they were.
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int kind = t >> 7;
      float gm = 0.f;
#pragma unroll
      for (int wq = 0; wq < 4; ++wq) gm = fmaxf(gm, wmaxs[r * NWARP + kind * 4 + wq]);
      const int ex = (int)((__float_as_uint(gm) >> 23) & 0xff) - 127;  // gm in [2^ex, 2^(ex+1))
      // (the packed-fp16 form also adds four products of up to 8 |x| in fp16: it needs |x| < 2^10)
      const int top = MATH == MATH_FAST_HALF2 ? 10 : 14;
      const int e = (ex >= top && ex < 128) ? ex - (top - 1) : 0;
      const float down = __uint_as_float((uint32_t)(127 - e) << 23);
      if ((t & 127) == 0) upf[r * 2 + kind] = __uint_as_float((uint32_t)(127 + e) << 23);
      const __half hv = __float2half_rn(xs_f[r * 256 + t] * down);
      xs_h[r * 256 + t] = hv;
      const float s = warp_sum(__half2float(hv));
      if (lane == 0) wsum[r * NWARP + warp] = s;
    }
    __syncthreads();
  }

  // 3. Multiply-accumulate this warp's 16 rows.
  float accL[ROWS][8], accH[ROWS][8];
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
#pragma unroll
    for (int c = 0; c < 8; ++c) accL[r][c] = accH[r][c] = 0.f;

  if (MATH == MATH_FAST) {
    // ROWS == 1: the warp's 16 + 16 fp16 activations sit in registers (four 16-byte broadcast loads).
    uint32_t xl[8], xh[8];
    if (ROWS == 1) {
      const uint4* xl4 = (const uint4*)(xs_h + warp * RPW);
      const uint4* xh4 = (const uint4*)(xs_h + 128 + warp * RPW);
      *(uint4*)&xl[0] = xl4[0];
      *(uint4*)&xl[4] = xl4[1];
      *(uint4*)&xh[0] = xh4[0];
      *(uint4*)&xh[4] = xh4[1];
    }
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
      uint32_t tq[2][4];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t wd = h ? w[i].y : w[i].x;
        const uint32_t w8 = wd >> 8;
        tq[h][0] = and_or(wd, 0x000F000Fu, 0x64006400u);  // bytes 0,2 low nibble : 1024 + n
        tq[h][1] = and_or(wd, 0x00F000F0u, 0x64006400u);  // bytes 0,2 high nibble: 1024 + 16 n
        tq[h][2] = and_or(w8, 0x000F000Fu, 0x64006400u);  // bytes 1,3 low
        tq[h][3] = and_or(w8, 0x00F000F0u, 0x64006400u);  // bytes 1,3 high
      }
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        unsigned short xlo, xhi;
        if (ROWS == 1) {
          xlo = (unsigned short)((i & 1) ? (xl[i >> 1] >> 16) : (xl[i >> 1] & 0xffffu));
          xhi = (unsigned short)((i & 1) ? (xh[i >> 1] >> 16) : (xh[i >> 1] & 0xffffu));
        } else {
          xlo = __half_as_ushort(xs_h[r * 256 + warp * RPW + i]);
          xhi = __half_as_ushort(xs_h[r * 256 + 128 + warp * RPW + i]);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int b = h * 4;
          accL[r][b + 0] = fma_f16(tq[h][0], 0, xlo, accL[r][b + 0]);
          accL[r][b + 2] = fma_f16(tq[h][0], 1, xlo, accL[r][b + 2]);
          accH[r][b + 0] = fma_f16(tq[h][1], 0, xhi, accH[r][b + 0]);
          accH[r][b + 2] = fma_f16(tq[h][1], 1, xhi, accH[r][b + 2]);
          accL[r][b + 1] = fma_f16(tq[h][2], 0, xlo, accL[r][b + 1]);
          accL[r][b + 3] = fma_f16(tq[h][2], 1, xlo, accL[r][b + 3]);
          accH[r][b + 1] = fma_f16(tq[h][3], 0, xhi, accH[r][b + 1]);
          accH[r][b + 3] = fma_f16(tq[h][3], 1, xhi, accH[r][b + 3]);
        }
      }
    }
  } else if (MATH == MATH_FAST_HALF2) {
    // Packed fp16 arithmetic: values are de-biased exactly, multiplied by the duplicated activation
    // and summed in fp16 over 4 rows, then flushed to the fp32 accumulators.
    const __half2 c1032 = __float2half2_rn(1032.f), c16th = __float2half2_rn(0.0625f), c72 = __float2half2_rn(72.f);
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
#pragma unroll
      for (int i0 = 0; i0 < RPW; i0 += 4) {
        __half2 aL[4], aH[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) aL[q] = aH[q] = __float2half2_rn(0.f);
#pragma unroll
        for (int ii = 0; ii < 4; ++ii) {
          const int i = i0 + ii;
          const __half2 xlo = __half2half2(xs_h[r * 256 + warp * RPW + i]);
          const __half2 xhi = __half2half2(xs_h[r * 256 + 128 + warp * RPW + i]);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t wd = h ? w[i].y : w[i].x;
            const uint32_t w8 = wd >> 8;
            uint32_t t0 = and_or(wd, 0x000F000Fu, 0x64006400u), t1 = and_or(wd, 0x00F000F0u, 0x64006400u);
            uint32_t t2 = and_or(w8, 0x000F000Fu, 0x64006400u), t3 = and_or(w8, 0x00F000F0u, 0x64006400u);
            const __half2 q0 = __hsub2(*(__half2*)&t0, c1032), q1 = __hfma2(*(__half2*)&t1, c16th, __hneg2(c72));
            const __half2 q2 = __hsub2(*(__half2*)&t2, c1032), q3 = __hfma2(*(__half2*)&t3, c16th, __hneg2(c72));
            aL[h * 2 + 0] = __hfma2(q0, xlo, aL[h * 2 + 0]);
            aH[h * 2 + 0] = __hfma2(q1, xhi, aH[h * 2 + 0]);
            aL[h * 2 + 1] = __hfma2(q2, xlo, aL[h * 2 + 1]);
            aH[h * 2 + 1] = __hfma2(q3, xhi, aH[h * 2 + 1]);
          }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int b = h * 4;
          accL[r][b + 0] += __low2float(aL[h * 2]);
          accL[r][b + 2] += __high2float(aL[h * 2]);
          accL[r][b + 1] += __low2float(aL[h * 2 + 1]);
          accL[r][b + 3] += __high2float(aL[h * 2 + 1]);
          accH[r][b + 0] += __low2float(aH[h * 2]);
          accH[r][b + 2] += __high2float(aH[h * 2]);
          accH[r][b + 1] += __low2float(aH[h * 2 + 1]);
          accH[r][b + 3] += __high2float(aH[h * 2 + 1]);
        }
      }
    }
  } else {
    // Every weight is dequantised as the reference does it, bf16(fp32(nibble - 8) * fp32 scale),
    // and multiplied with the activation in fp32.
#pragma unroll
    for (int i = 0; i < RPW; ++i) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint32_t byte = ((c < 4 ? w[i].x : w[i].y) >> (8 * (c & 3))) & 0xffu;
        const float wl = round_bf16(__fmul_rn((float)((int)(byte & 15u) - 8), sL[c]));
        const float wh = round_bf16(__fmul_rn((float)((int)(byte >> 4) - 8), sH[c]));
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          accL[r][c] = fmaf(xs_f[r * 256 + warp * RPW + i], wl, accL[r][c]);
          accH[r][c] = fmaf(xs_f[r * 256 + 128 + warp * RPW + i], wh, accH[r][c]);
        }
      }
    }
  }

  // 4. Reduce the 8 warps; column c of this thread goes to padded slot c + c/32 (conflict free both ways).
#pragma unroll
  for (int r = 0; r < ROWS; ++r)
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      const int col = lane * 8 + c, slot = col + (col >> 5);
      red[((r * 2 + 0) * NWARP + warp) * PADW + slot] = accL[r][c];
      red[((r * 2 + 1) * NWARP + warp) * PADW + slot] = accH[r][c];
    }
  __syncthreads();

  const int n = tile * TN + t;
  const int slot = t + (t >> 5);
  float val[ROWS];
  {
    float sl = 1.f, sh = 1.f;
    if (MATH != MATH_EXACT && n < p.N) {
      sl = load_scale(p, (long)g * p.N + n);
      sh = load_scale(p, (long)(g + G) * p.N + n);
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      float vL = 0.f, vH = 0.f, sxL = 0.f, sxH = 0.f;
#pragma unroll
      for (int wq = 0; wq < NWARP; ++wq) {
        vL += red[((r * 2 + 0) * NWARP + wq) * PADW + slot];
        vH += red[((r * 2 + 1) * NWARP + wq) * PADW + slot];
      }
#pragma unroll
      for (int wq = 0; wq < 4; ++wq) {
        sxL += wsum[r * NWARP + wq];
        sxH += wsum[r * NWARP + 4 + wq];
      }
      if (MATH == MATH_FAST) {
        // accL = sum x (1024 + n), accH = sum x (1024 + 16 n); remove the bias and the zero point 8.
        vL = fmaf(-1032.f, sxL, vL);
        vH = fmaf(-72.f, sxH, vH * 0.0625f);
      }
      val[r] = (MATH == MATH_EXACT) ? (vL + vH) : fmaf(sl * upf[r * 2], vL, sh * upf[r * 2 + 1] * vH);
    }
  }

  if (G == 1) {
    if (n < p.N)
#pragma unroll
      for (int r = 0; r < ROWS; ++r)
        if (row0 + r < p.rows) epilogue_store(p, row0 + r, n, val[r]);
    return;
  }

  // 5. Split-K: publish this group's partial, the last CTA of the column tile sums all groups in order.
  if (n < p.N)
#pragma unroll
    for (int r = 0; r < ROWS; ++r)
      if (row0 + r < p.rows) __stcg(&p.partials[((long)(row0 + r) * G + g) * p.N + n], val[r]);
  __threadfence();
  __syncthreads();
  if (t == 0) {
    unsigned* ctr = &p.counters[zb * gridDim.x + tile];
    const unsigned old = atomicAdd(ctr, 1u);
    s_last = (old == (unsigned)(G - 1));
    if (s_last) *ctr = 0u;  // ready for the next launch
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  if (n < p.N)
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      if (row0 + r >= p.rows) break;
      const float* pp = p.partials + (long)(row0 + r) * G * p.N + n;
      float sum = 0.f;
      for (int gg = 0; gg < G; ++gg) sum += __ldcg(pp + (long)gg * p.N);
      epilogue_store(p, row0 + r, n, sum);
    }
}

// Any K (even), any group that divides K/2, any N: one thread per column, weights dequantised as
// the reference does. Used for shapes the fast path does not cover (toy models in the tests).
__global__ void __launch_bounds__(128) gemv_generic_kernel(const GemvParams p) {
  __shared__ float wscr[4];
  const int r = blockIdx.y;
  const int n = blockIdx.x * blockDim.x + threadIdx.x;
  const int half = p.K / 2;
  float rstd = 1.f;
  if (p.prologue == PRO_RMSNORM) rstd = cta_rstd(p, r, wscr);
  if (n >= p.N) return;
  float acc = 0.f;
  for (int j = 0; j < half; ++j) {
    const uint32_t byte = p.packed[(size_t)j * p.N + n];
    const float sl = load_scale(p, (long)(j / p.group) * p.N + n);
    const float sh = load_scale(p, (long)((j + half) / p.group) * p.N + n);
    const float wl = round_bf16(__fmul_rn((float)((int)(byte & 15u) - 8), sl));
    const float wh = round_bf16(__fmul_rn((float)((int)(byte >> 4) - 8), sh));
    acc = fmaf(prologue_value(p, r, j, rstd), wl, acc);
    acc = fmaf(prologue_value(p, r, j + half, rstd), wh, acc);
  }
  epilogue_store(p, r, n, acc);
}

__global__ void int4_unpack_kernel(const uint8_t* packed, int half, int N, int8_t* out) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)half * N) return;
  const uint32_t byte = packed[idx];
  out[idx] = (int8_t)((int)(byte & 15u) - 8);
  out[idx + (long)half * N] = (int8_t)((int)(byte >> 4) - 8);
}

__global__ void int4_dequant_kernel(const uint8_t* packed, const void* scale, int scale_bf16, int half, int N, int group,
                                    bf16* out) {
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)half * N) return;
  const int j = (int)(idx / N), n = (int)(idx % N);
  const uint32_t byte = packed[idx];
  const long il = (long)(j / group) * N + n, ih = (long)((j + half) / group) * N + n;
  const float sl = scale_bf16 ? bf2f(((const bf16*)scale)[il]) : ((const float*)scale)[il];
  const float sh = scale_bf16 ? bf2f(((const bf16*)scale)[ih]) : ((const float*)scale)[ih];
  out[idx] = f2bf(__fmul_rn((float)((int)(byte & 15u) - 8), sl));
  out[idx + (long)half * N] = f2bf(__fmul_rn((float)((int)(byte >> 4) - 8), sh));
}

bool fast_path(const GemvParams& p) {
  return p.group == 128 && p.K % 256 == 0 && p.N % 8 == 0 && ((uintptr_t)p.packed % 8) == 0;
}

template <int ROWS>
size_t smem_bytes() {
  return (size_t)ROWS * 2 * NWARP * PADW * 4 + (size_t)ROWS * 256 * 4 + (size_t)ROWS * 256 * 2 + (size_t)ROWS * NWARP * 4 +
         NWARP * 4;
}

template <int ROWS, int MATH>
int launch_fast(const GemvParams& p, cudaStream_t stream) {
  const size_t smem = smem_bytes<ROWS>();
  dim3 grid((p.N + TN - 1) / TN, p.K / 256, (p.rows + ROWS - 1) / ROWS);
  gemv_g128_kernel<ROWS, MATH><<<grid, NWARP * 32, smem, stream>>>(p);
  return check_launch("int4 gemv");
}

template <int ROWS>
int launch_fast_math(const GemvParams& p, cudaStream_t stream) {
  if (p.math == MATH_EXACT) return launch_fast<ROWS, MATH_EXACT>(p, stream);
  if (p.math == MATH_FAST_HALF2) return launch_fast<ROWS, MATH_FAST_HALF2>(p, stream);
  return launch_fast<ROWS, MATH_FAST>(p, stream);
}

}  // namespace

template <int ROWS>
static int configure_rows() {
  const int smem = (int)smem_bytes<ROWS>();
  cudaError_t e = cudaFuncSetAttribute(gemv_g128_kernel<ROWS, MATH_FAST>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(gemv_g128_kernel<ROWS, MATH_EXACT>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(gemv_g128_kernel<ROWS, MATH_FAST_HALF2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  return e == cudaSuccess ? 0 : check_launch("int4 gemv: shared-memory opt-in");
}

int gemv_configure() {
  if (int rc = stream_configure()) return rc;
  if (int rc = cluster_configure()) return rc;
  if (int rc = mma_configure()) return rc;
  if (int rc = tc_configure()) return rc;
  if (int rc = configure_rows<1>()) return rc;
  if (int rc = configure_rows<2>()) return rc;
  return configure_rows<4>();
}

static int rows_per_cta(int rows) { return rows >= 4 ? 4 : (rows >= 2 ? 2 : 1); }

size_t gemv_partials_bytes(int rows, int K, int N, int group) {
  if (group != 128 || K % 256 != 0 || N % 8 != 0) return 0;
  const size_t tiled = K / 256 < 2 ? 0 : (size_t)rows * (K / 256) * N * sizeof(float);
  const size_t streamed = (rows == 1 && N % 16 == 0) ? stream_partials_bytes(K, N) : 0;
  return std::max(tiled, streamed);
}

size_t gemv_counter_count(int rows, int K, int N, int group) {
  if (group != 128 || K % 256 != 0 || N % 8 != 0) return 0;
  const int rpc = rows_per_cta(rows);
  const size_t tiled = (size_t)((N + TN - 1) / TN) * ((rows + rpc - 1) / rpc);
  return std::max(tiled, stream_counter_count(K, N));
}

int launch_gemv(const GemvParams& p, cudaStream_t stream) {
  if (p.rows <= 0 || p.N <= 0) return 0;
  static OncePerDevice once;
  const int configured = once.run(gemv_configure);
  if (configured) return configured;
  if (!p.force_tiled && p.status && p.rows == 1 && mma_path_ok(p)) return launch_gemv_mma(p, p.status, stream);
  if ((p.epilogue == EPI_SWIGLU || p.prologue == PRO_ATTN_MERGE) && !(!p.force_tiled && p.status && p.N < 65536 && cluster_path_ok(p))) {
    set_error("int4 gemv: the SwiGLU epilogue and the attention-merge prologue exist in the cluster kernel only (one row, "
              "re-packed group-128 weight; SwiGLU: N a multiple of two tiles)");
    return 2;
  }
  // eight rows and more: the weight tile is shared by enough rows for the tensor cores
  if (!p.force_tiled && p.rows >= 8 && tc_path_ok(p)) return launch_gemm_tc(p, p.status, stream);
  if (!p.force_tiled && p.status) {
    // layer-sized matrices: one cluster per column tile; very wide ones (the LM head): persistent streaming
    if (p.N < 65536 && cluster_path_ok(p)) return launch_gemv_cluster(p, p.status, stream);
    if (p.partials && p.counters && stream_path_ok(p)) return launch_gemv_stream(p, p.status, stream);
  }
  if (fast_path(p)) {
    if (p.K / 256 > 1 && (p.partials == nullptr || p.counters == nullptr)) {
      set_error("int4 gemv: split-K scratch (partials, counters) is required for K=%d", p.K);
      return 2;
    }
    switch (rows_per_cta(p.rows)) {
      case 4: return launch_fast_math<4>(p, stream);
      case 2: return launch_fast_math<2>(p, stream);
      default: return launch_fast_math<1>(p, stream);
    }
  }
  dim3 grid((p.N + 127) / 128, p.rows);
  gemv_generic_kernel<<<grid, 128, 0, stream>>>(p);
  return check_launch("int4 gemv (generic)");
}

int launch_int4_unpack(const uint8_t* packed, int K, int N, int8_t* out, cudaStream_t stream) {
  const long total = (long)(K / 2) * N;
  if (total == 0) return 0;
  int4_unpack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(packed, K / 2, N, out);
  return check_launch("int4 unpack");
}

int launch_int4_dequant(const uint8_t* packed, const void* scale, int scale_bf16, int K, int N, int group, bf16* out,
                        cudaStream_t stream) {
  const long total = (long)(K / 2) * N;
  if (total == 0) return 0;
  int4_dequant_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(packed, scale, scale_bf16, K / 2, N, group, out);
  return check_launch("int4 dequant");
}

// ---- split-K GEMV on scratch the library owns (no allocation at call time) -----------------------
//
// The split-K kernel above, with its partial sums and arrival counters in a file-scope device array
// instead of caller memory. The array's address is looked up once per device, on the first call with
// that device current; later calls only clear the counters and launch.
constexpr size_t STATIC_PARTIALS_BYTES = 2u << 20;  // 2 MiB of fp32 partial sums
constexpr size_t STATIC_COUNTERS = 4096;            // arrival counters, one per (column tile, row block)
constexpr size_t STATIC_SCRATCH_BYTES = STATIC_PARTIALS_BYTES + STATIC_COUNTERS * sizeof(unsigned);
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

constexpr int STATIC_MAX_DEVICES = 64;
static void* g_static_ptr[STATIC_MAX_DEVICES];
static std::mutex g_static_mutex;

// Address of this device's copy of the array; looked up on first use (the current device's).
static int static_scratch_for_current_device(void** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return check_launch("static-scratch gemv: cudaGetDevice");
  if (dev < 0 || dev >= STATIC_MAX_DEVICES) {
    set_error("static-scratch gemv: device ordinal %d is beyond the %d this entry point tracks", dev, STATIC_MAX_DEVICES);
    return 2;
  }
  std::lock_guard<std::mutex> lock(g_static_mutex);
  if (g_static_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      set_error("static-scratch gemv: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
      (void)cudaGetLastError();
      return 1;  // DFB_ERR_CUDA
    }
    g_static_ptr[dev] = ptr;
  }
  *out = g_static_ptr[dev];
  return 0;
}

}  // namespace dfb

extern "C" size_t dfb_int4_gemv_static_max_partials_bytes(void) { return dfb::STATIC_PARTIALS_BYTES; }

extern "C" int dfb_int4_gemv_static(const dfb_gemv_desc* d, void* stream) {
  using namespace dfb;
  if (!d) {
    set_error("dfb_int4_gemv_static: null descriptor");
    return 2;
  }
  if (d->rows < 0) {
    set_error("dfb_int4_gemv_static: negative row count");
    return 2;
  }
  if (d->rows == 0) return 0;
  if (!d->x || !d->packed || !d->scale || !d->out) {
    set_error("dfb_int4_gemv_static: null tensor pointer");
    return 2;
  }
  if (int rc = check_int4_shape(d->K, d->N, d->group)) return rc;
  if (d->group != 128 || d->K % 256 != 0 || d->N % 8 != 0 || ((uintptr_t)d->packed % 8) != 0) {
    set_error("dfb_int4_gemv_static: serves the group-128 split-K kernel only (K %% 256 == 0, N %% 8 == 0, packed 8-byte "
              "aligned); got K=%d N=%d group=%d", d->K, d->N, d->group);
    return 2;
  }
  if (d->prologue < 0 || d->prologue > 2 || d->epilogue < 0 || d->epilogue > 2 || d->math < 0 || d->math > 2) {
    set_error("dfb_int4_gemv_static: unknown prologue, epilogue or math mode (%d, %d, %d)", d->prologue, d->epilogue, d->math);
    return 2;
  }
  if ((d->prologue == PRO_RMSNORM && !d->norm_w) || (d->prologue == PRO_SILU_MUL && !d->up) ||
      (d->epilogue == EPI_RESIDUAL && !d->residual) ||
      (d->epilogue == EPI_CONV && (!d->conv_state || !d->conv_w || d->conv_dim < 0 || d->conv_dim > d->N))) {
    set_error("dfb_int4_gemv_static: the chosen prologue or epilogue lacks one of its tensors");
    return 2;
  }
  const int rpc = rows_per_cta(d->rows);
  const size_t partial_bytes = (size_t)d->rows * (d->K / 256) * d->N * sizeof(float);
  const size_t counters = (size_t)((d->N + TN - 1) / TN) * ((d->rows + rpc - 1) / rpc);
  if (partial_bytes > STATIC_PARTIALS_BYTES || counters > STATIC_COUNTERS) {
    set_error("dfb_int4_gemv_static: rows=%d K=%d N=%d needs %zu bytes of partial sums and %zu counters; the built-in "
              "scratch holds %zu bytes and %zu counters -- use dfb_int4_gemv with caller scratch for this size",
              d->rows, d->K, d->N, partial_bytes, counters, (size_t)STATIC_PARTIALS_BYTES, (size_t)STATIC_COUNTERS);
    return 2;
  }
  static OncePerDevice once;
  const int configured = once.run(gemv_configure);
  if (configured) return configured;
  void* base = nullptr;
  if (int rc = static_scratch_for_current_device(&base)) return rc;
  GemvParams p = {};
  p.x = (const bf16*)d->x;
  p.x_stride = d->x_stride;
  p.rows = d->rows;
  p.packed = d->packed;
  p.scale = d->scale;
  p.scale_bf16 = d->scale_is_bf16;
  p.K = d->K;
  p.N = d->N;
  p.group = d->group;
  p.prologue = d->prologue;
  p.norm_w = (const bf16*)d->norm_w;
  p.eps = d->eps;
  p.up = (const bf16*)d->up;
  p.up_stride = d->up_stride;
  p.epilogue = d->epilogue;
  p.out = (bf16*)d->out;
  p.out_stride = d->out_stride;
  p.residual = (const bf16*)d->residual;
  p.res_stride = d->residual_stride;
  p.conv_state = (bf16*)d->conv_state;
  p.conv_w = (const bf16*)d->conv_w;
  p.conv_dim = d->conv_dim;
  p.math = d->math;
  p.partials = (float*)base;
  p.counters = (unsigned*)((char*)base + STATIC_PARTIALS_BYTES);
  p.force_tiled = 1;
  // The last-arriver test counts from zero: clear this launch's counters in stream order. The partial
  // sums need no clearing, every one that is read has been written by this launch.
  if (cudaMemsetAsync(p.counters, 0, counters * sizeof(unsigned), (cudaStream_t)stream) != cudaSuccess)
    return check_launch("dfb_int4_gemv_static: clearing the arrival counters");
  switch (rpc) {
    case 4: return launch_fast_math<4>(p, (cudaStream_t)stream);
    case 2: return launch_fast_math<2>(p, (cudaStream_t)stream);
    default: return launch_fast_math<1>(p, (cudaStream_t)stream);
  }
}
