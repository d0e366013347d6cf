// Shared device helpers for the decode-step kernels (sm_100a).
//
// Rounding helpers mirror the places where the reference's torch expressions round to bf16, so the
// fused kernels can keep those rounding points; see the per-kernel comments for which ones.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "kernels.h"

namespace dfb {

__device__ __forceinline__ float bf2f(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ bf16 f2bf(float v) { return __float2bfloat16_rn(v); }
__device__ __forceinline__ float round_bf16(float v) { return bf2f(f2bf(v)); }

// x / (1 + exp(-x)) with the full-precision exponential, as torch evaluates SiLU in fp32.
__device__ __forceinline__ float silu_f(float x) { return __fdiv_rn(x, __fadd_rn(1.0f, expf(-x))); }
__device__ __forceinline__ float sigmoid_f(float x) { return __fdiv_rn(1.0f, __fadd_rn(1.0f, expf(-x))); }
// 1 / sqrt(x) as two correctly rounded steps, which is how a CPU evaluates rsqrt.
__device__ __forceinline__ float rsqrt_2step(float x) { return __fdiv_rn(1.0f, __fsqrt_rn(x)); }
// log(1 + exp(x)) with torch's threshold of 20 above which softplus is the identity.
__device__ __forceinline__ float softplus_f(float x) { return x > 20.0f ? x : log1pf(expf(x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Streaming loads for data read exactly once per step (weights, KV): no L1 allocation and an
// evict-first L2 policy, so the activations, partial sums and recurrent state keep their L2 lines.
__device__ __forceinline__ uint64_t make_evict_first_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint2 ldg_stream_u2(const void* p, uint64_t pol) {
  uint2 r;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v2.u32 {%0,%1}, [%2], %3;"
               : "=r"(r.x), "=r"(r.y)
               : "l"(p), "l"(pol));
  return r;
}
__device__ __forceinline__ uint4 ldg_stream_u4(const void* p, uint64_t pol) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p), "l"(pol));
  return r;
}

// Programmatic dependent launch: pdl_launch_dependents() lets the next kernel of the stream start its
// own prologue early; pdl_wait() blocks until everything the preceding kernels wrote is visible.
// Without the launch attribute both instructions do nothing.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Ask the L2 to fetch [ptr + begin, ptr + end) from HBM without bringing it to the SM (bytes are rounded
// inwards to 16-byte units, pieces of at most 16 KB). Used to start the weight stream of the NEXT kernel of
// the decode step while this one is still working through its own dependent chain.
__device__ __forceinline__ void l2_prefetch_range(const void* ptr, size_t begin, size_t end) {
  const char* a = (const char*)ptr + ((begin + 15) & ~(size_t)15);
  const char* e = (const char*)ptr + (end & ~(size_t)15);
  while (a < e) {
    const size_t left = (size_t)(e - a);
    const uint32_t n = left > 16384 ? 16384u : (uint32_t)left;
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(a), "r"(n) : "memory");
    a += n;
  }
}

// Optional per-launch timeline for profiling the chain of dependent kernels: when `buf` is set, one thread of
// each CTA stores the global nanosecond timer at up to TRACE_PHASES marks, at
// buf[(slot * ctas + cta) * TRACE_PHASES + phase]. CTAs beyond `ctas` record nothing.
__device__ __forceinline__ void trace_mark(const Trace& tr, int cta, int phase) {
  if (tr.buf != nullptr && cta < tr.ctas) {
    long long ns;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
    tr.buf[((long)tr.slot * tr.ctas + cta) * TRACE_PHASES + phase] = ns;
  }
}

// Bounds build (nvcc -DDFB_BOUNDS, `python -m deltaforge_b200.build --bounds`): the kernels check the indices of
// their stores and of their shared-memory tiles against the extents and, instead of making the access, record
// code 60 + site in the status word the launch was given. The checks compile to nothing in the normal build. It
// stands in for a memory checker on machines where none can be run.
#ifdef DFB_BOUNDS
#define DFB_IN_BOUNDS(cond, status_ptr, site) dfb_in_bounds((cond), (status_ptr), (site))
__device__ __forceinline__ bool dfb_in_bounds(bool ok, int* status, int site) {
  if (!ok && status != nullptr) atomicCAS(status, 0, 60 + site);
  return ok;
}
#else
#define DFB_IN_BOUNDS(cond, status_ptr, site) true
#endif

// Error reporting shared by the C entry points (defined in abi.cu).
void set_error(const char* fmt, ...);
int check_launch(const char* what);
int check_int4_shape(int K, int N, int group);  // 0, or DFB_ERR_ARG with the message set

// Kernel attributes (the opt-in to large dynamic shared memory, the carve-out preference) belong to the device
// that is current when they are set, so set-up that a process would otherwise run once has to run once per
// device: run(fn) calls fn the first time it is reached with a given device current and returns fn's code
// (0 afterwards; a failed fn is tried again on the next call).
struct OncePerDevice {
  static constexpr int MAX_DEVICES = 64;
  std::mutex mu;
  bool done[MAX_DEVICES] = {};
  int run(int (*fn)()) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return fn();
    std::lock_guard<std::mutex> lock(mu);
    if (done[dev]) return 0;
    const int rc = fn();
    done[dev] = rc == 0;
    return rc;
  }
};

// Ask for the largest shared-memory carve-out for a kernel. Every kernel of the decode step does,
// including those that use almost none: if consecutive kernels asked for different L1/shared splits
// the SMs would have to drain and re-partition between them.
template <typename K>
inline cudaError_t prefer_max_shared(K kernel) {
  return cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

// Launch with the programmatic-stream-serialization attribute (the kernel must call pdl_wait()
// before it reads or writes anything an earlier kernel of the stream touches).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

}  // namespace dfb
