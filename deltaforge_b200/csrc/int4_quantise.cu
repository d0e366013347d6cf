// Install-time int4 quantiser, sm_100a: a weight [N, K] (bf16 or fp32, row-major) to the reference's K-major format
// in one pass.
//
// Same function as quantise_int4_k_major of the reference (src/deltaforge/kernels/tiled_gemv.py:242-278, the group
// rule of src/deltaforge/kernels/quantised_linear.py:193-207), bit for bit: per (column n, group of rows) the scale is
// amax / 7 in fp32 (1 where the group is all zero), values are round-half-even(w / scale) clamped to [-7, 7] and
// stored offset by 8; byte [j, n] carries row j in its low nibble and row j + K/2 in its high nibble; packed is
// [K/2, N], scale [K/group, N] fp32.
//
// One CTA takes 32 columns (rows of the [N, K] weight) and one group of the lower half together with its partner
// group of the upper half, i.e. exactly the rows whose nibbles share bytes. A warp reads a 128-element run of a
// weight row as one coalesced request, reduces the maximum with shuffles and writes its nibbles into a shared tile
// [128 rows][32 columns]; the tile leaves as 32-byte row segments. Group sizes other than 128 (toy widths: one group
// per half) take a plain one-thread-per-group kernel.
#include "common.cuh"
#include "kernels.h"

namespace dfb {

namespace {

constexpr int QG = 128;    // group size of the fast kernel
constexpr int QCOLS = 32;  // columns (weight rows) per CTA

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <>
__device__ __forceinline__ float to_f32<float>(float v) {
  return v;
}
template <>
__device__ __forceinline__ float to_f32<bf16>(bf16 v) {
  return bf2f(v);
}

__device__ __forceinline__ unsigned nibble_of(float w, float scale) {
  float q = rintf(__fdiv_rn(w, scale));  // round half to even, as torch.round
  q = fminf(fmaxf(q, -7.0f), 7.0f);
  return (unsigned)((int)q + 8);
}

template <typename T>
__global__ void __launch_bounds__(256) int4_quantise_g128_kernel(const T* w, int N, int K, uint8_t* packed, float* scale) {
  __shared__ unsigned char tile[QG][QCOLS];  // packed bytes of 128 row pairs x 32 columns
  const int half = K / 2, G = K / QG;
  const int g = blockIdx.y;  // group of the lower half; its partner is g + G/2
  const int n0 = blockIdx.x * QCOLS;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int c = warp; c < QCOLS; c += 8) {
    const int n = n0 + c;
    if (n >= N) {
      for (int i = 0; i < 4; ++i) tile[lane * 4 + i][c] = 0;
      continue;
    }
    const T* row = w + (size_t)n * K;
    float lo[4], hi[4];
    float alo = 0.f, ahi = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lo[i] = to_f32<T>(row[g * QG + lane * 4 + i]);
      hi[i] = to_f32<T>(row[half + g * QG + lane * 4 + i]);
      alo = fmaxf(alo, fabsf(lo[i]));
      ahi = fmaxf(ahi, fabsf(hi[i]));
    }
    alo = warp_max(alo);
    ahi = warp_max(ahi);
    float slo = __fdiv_rn(alo, 7.0f), shi = __fdiv_rn(ahi, 7.0f);
    if (!(slo > 0.f)) slo = 1.0f;
    if (!(shi > 0.f)) shi = 1.0f;
    if (lane == 0) {
      scale[(size_t)g * N + n] = slo;
      scale[(size_t)(g + G / 2) * N + n] = shi;
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) tile[lane * 4 + i][c] = (unsigned char)(nibble_of(lo[i], slo) | (nibble_of(hi[i], shi) << 4));
  }
  __syncthreads();
  // 128 rows of 32 bytes: two threads per row, 16 bytes each (whole 32-byte segments when N is a multiple of 32)
  const int r = threadIdx.x >> 1, part = threadIdx.x & 1;
  uint8_t* dst = packed + (size_t)(g * QG + r) * N + n0 + part * 16;
  if (n0 + QCOLS <= N && (N % 16) == 0) {
    *(uint4*)dst = *(const uint4*)&tile[r][part * 16];
  } else {
    for (int i = 0; i < 16; ++i)
      if (n0 + part * 16 + i < N) dst[i] = tile[r][part * 16 + i];
  }
}

// any group size: thread (n, g) walks its group of the lower half and the partner group of the upper half
template <typename T>
__global__ void int4_quantise_generic_kernel(const T* w, int N, int K, int group, uint8_t* packed, float* scale) {
  const int half = K / 2, gh = half / group;  // groups per half
  const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long)N * gh) return;
  const int n = (int)(idx % N), g = (int)(idx / N);
  const T* row = w + (size_t)n * K;
  float alo = 0.f, ahi = 0.f;
  for (int i = 0; i < group; ++i) {
    alo = fmaxf(alo, fabsf(to_f32<T>(row[g * group + i])));
    ahi = fmaxf(ahi, fabsf(to_f32<T>(row[half + g * group + i])));
  }
  float slo = __fdiv_rn(alo, 7.0f), shi = __fdiv_rn(ahi, 7.0f);
  if (!(slo > 0.f)) slo = 1.0f;
  if (!(shi > 0.f)) shi = 1.0f;
  scale[(size_t)g * N + n] = slo;
  scale[(size_t)(g + gh) * N + n] = shi;
  for (int i = 0; i < group; ++i) {
    const int j = g * group + i;
    packed[(size_t)j * N + n] =
        (uint8_t)(nibble_of(to_f32<T>(row[j]), slo) | (nibble_of(to_f32<T>(row[half + j]), shi) << 4));
  }
}

template <typename T>
int launch_quantise_t(const T* w, int N, int K, int group, uint8_t* packed, float* scale, cudaStream_t stream) {
  if (group == QG && K % (2 * QG) == 0) {
    dim3 grid((N + QCOLS - 1) / QCOLS, K / QG / 2);
    int4_quantise_g128_kernel<T><<<grid, 256, 0, stream>>>(w, N, K, packed, scale);
  } else {
    const long total = (long)N * (K / 2 / group);
    int4_quantise_generic_kernel<T><<<(unsigned)((total + 127) / 128), 128, 0, stream>>>(w, N, K, group, packed, scale);
  }
  return check_launch("int4 quantise");
}

}  // namespace

int launch_int4_quantise(const void* weight, int weight_is_bf16, int N, int K, int group, uint8_t* packed, float* scale,
                         cudaStream_t stream) {
  if (N <= 0 || K <= 0) return 0;
  if (weight_is_bf16) return launch_quantise_t<bf16>((const bf16*)weight, N, K, group, packed, scale, stream);
  return launch_quantise_t<float>((const float*)weight, N, K, group, packed, scale, stream);
}

}  // namespace dfb
