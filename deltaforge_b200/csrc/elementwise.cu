// Small elementwise kernels of the decode step, sm_100a: the standalone forms of operations that the
// fused kernels otherwise absorb. Each keeps the rounding points of the reference op it stands for.
#include "common.cuh"
#include "kernels.h"

namespace dfb {

namespace {

// y = bf16(x * rsqrt(mean(x^2) + eps) * (1 + w)); optionally x = bf16(x + residual) first.
// src/deltaforge/reference.py:92-96; src/deltaforge/kernels/fused_rmsnorm_residual.py:56-111.
__global__ void __launch_bounds__(256) rms_norm_kernel(const bf16* x, const bf16* res, const bf16* w, float eps, int n,
                                                       bf16* resid_out, bf16* out) {
  __shared__ float wred[8];
  pdl_launch_dependents();
  pdl_wait();  // launched with programmatic dependent launch: everything it reads comes from the kernel before it
  const long row = blockIdx.x;
  const bf16* xr = x + row * n;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += 256) {
    float v = bf2f(xr[i]);
    if (res) {
      v = round_bf16(__fadd_rn(bf2f(res[row * n + i]), v));
      resid_out[row * n + i] = f2bf(v);
    }
    ss = fmaf(v, v, ss);
  }
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) wred[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += wred[i];
  const float rstd = rsqrt_2step(__fadd_rn(__fdiv_rn(tot, (float)n), eps));
  for (int i = threadIdx.x; i < n; i += 256) {
    const float v = res ? bf2f(resid_out[row * n + i]) : bf2f(xr[i]);
    out[row * n + i] = f2bf(__fmul_rn(__fmul_rn(v, rstd), __fadd_rn(1.0f, bf2f(w[i]))));
  }
}

// bf16(bf16(silu(gate)) * up). src/deltaforge/kernels/fused_swiglu.py:18-22, :37-48.
__global__ void silu_mul_kernel(const bf16* gate, const bf16* up, long n, bf16* out) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float s = round_bf16(silu_f(bf2f(gate[i])));
  out[i] = f2bf(__fmul_rn(s, bf2f(up[i])));
}

// x (batch, heads, seq, d), cos/sin (batch, seq, rd). src/deltaforge/reference.py:137-149.
__global__ void partial_rope_kernel(const bf16* x, const bf16* cs, const bf16* sn, int heads, int seq, int d, int rd,
                                    bf16* out) {
  const long rowi = blockIdx.x;  // (b * heads + h) * seq + s
  const int s = (int)(rowi % seq);
  const int b = (int)(rowi / ((long)heads * seq));
  const bf16* xr = x + rowi * d;
  const bf16* c = cs + ((long)b * seq + s) * rd;
  const bf16* sv = sn + ((long)b * seq + s) * rd;
  const int half = rd / 2;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    if (i >= rd) {
      out[rowi * d + i] = xr[i];
      continue;
    }
    const float xo = (i < half) ? -bf2f(xr[i + half]) : bf2f(xr[i - half]);
    const float a = round_bf16(__fmul_rn(bf2f(xr[i]), bf2f(c[i])));
    const float r = round_bf16(__fmul_rn(xo, bf2f(sv[i])));
    out[rowi * d + i] = f2bf(__fadd_rn(a, r));
  }
}

// x (B, C), cache (B, C, 3) oldest first, w (C, 4). src/deltaforge/kernels/inline_causal_conv.py:98-129.
__global__ void causal_conv_step_kernel(const bf16* x, bf16* cache, const bf16* w, int channels, long total, bf16* out) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const int c = (int)(i % channels);
  bf16* st = cache + i * 3;
  const bf16* wc = w + (long)c * 4;
  const bf16 xv = x[i];
  float acc = __fmul_rn(bf2f(st[0]), bf2f(wc[0]));
  acc = __fadd_rn(acc, __fmul_rn(bf2f(st[1]), bf2f(wc[1])));
  acc = __fadd_rn(acc, __fmul_rn(bf2f(st[2]), bf2f(wc[2])));
  acc = __fadd_rn(acc, __fmul_rn(bf2f(xv), bf2f(wc[3])));
  out[i] = f2bf(silu_f(round_bf16(acc)));
  st[0] = st[1];
  st[1] = st[2];
  st[2] = xv;
}

// Row-strided forms for the batched decode step: gate | up live side by side in one projection row, and
// the conv runs in place on the leading channels of the input-projection row.
__global__ void silu_mul_rows_kernel(const bf16* gate, const bf16* up, long in_stride, int n, long total, bf16* out) {
  pdl_launch_dependents();
  pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long r = i / n, c = i % n;
  const float s = round_bf16(silu_f(bf2f(gate[r * in_stride + c])));
  out[i] = f2bf(__fmul_rn(s, bf2f(up[r * in_stride + c])));
}

__global__ void causal_conv_rows_kernel(bf16* x, long x_stride, bf16* cache, const bf16* w, int channels, long total) {
  pdl_launch_dependents();
  pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long r = i / channels;
  const int c = (int)(i % channels);
  bf16* st = cache + i * 3;
  const bf16* wc = w + (long)c * 4;
  bf16* xp = x + r * x_stride + c;
  const bf16 xv = *xp;
  float acc = __fmul_rn(bf2f(st[0]), bf2f(wc[0]));
  acc = __fadd_rn(acc, __fmul_rn(bf2f(st[1]), bf2f(wc[1])));
  acc = __fadd_rn(acc, __fmul_rn(bf2f(st[2]), bf2f(wc[2])));
  acc = __fadd_rn(acc, __fmul_rn(bf2f(xv), bf2f(wc[3])));
  *xp = f2bf(silu_f(round_bf16(acc)));
  st[0] = st[1];
  st[1] = st[2];
  st[2] = xv;
}

// Residual add of a projection whose fp32 partial sums were added across ranks: the sum is rounded to bf16
// (what the unsharded projection would have returned), then added to the stream (src/deltaforge/reference.py:730,735).
__global__ void add_partial_kernel(bf16* h, const float* sum, long n) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  h[i] = f2bf(__fadd_rn(bf2f(h[i]), round_bf16(sum[i])));
}

__device__ __forceinline__ unsigned long long ld_sys_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
// Poll one exchange word until it carries `epoch`. The limit is the seconds scale of the other bounded waits
// (about two seconds: ordinary host skew between the ranks' launches must not trip it); a wait that runs out
// records code 50, and once the status word is set every later wait gives up at once, so a step whose peer
// never arrives costs one limit, not one per kernel.
constexpr long long TP_WAIT_LIMIT_CYCLES = 4000000000LL;
__device__ __forceinline__ bool tp_wait_word(const unsigned long long* p, unsigned epoch, float& value, int* status) {
  unsigned long long v = ld_sys_u64(p);
  if ((unsigned)(v >> 32) != epoch) {
    const long long t0 = clock64();
    for (;;) {
      v = ld_sys_u64(p);
      if ((unsigned)(v >> 32) == epoch) break;
      if (clock64() - t0 > TP_WAIT_LIMIT_CYCLES || (status && *(volatile int*)status != 0)) {
        if (status) atomicCAS(status, 0, 50);
        value = 0.f;
        return false;
      }
      __nanosleep(40);
    }
  }
  value = __uint_as_float((unsigned)v);
  return true;
}

__global__ void tp_reduce_kernel(bf16* h, const unsigned long long* slots, int tp_size, long n, long word_off, const unsigned* epoch_ctr,
                                 int epoch_off, int* status, Trace trace) {
  // Launched with programmatic dependent launch: the projection after this kernel starts at once and streams
  // its weights while the words from the peers are still arriving.
  pdl_launch_dependents();
  if (threadIdx.x == 0) trace_mark(trace, blockIdx.x, 0);
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  // the epoch counter was bumped by the last kernel of the previous token, long complete
  const unsigned epoch = *epoch_ctr * 256u + (unsigned)epoch_off;
  float sum = 0.f;
  bool ok = true;
  if (i < n) {
    for (int r = 0; r < tp_size; ++r) {  // rank order: every rank adds the same numbers in the same order
      float v;
      ok = tp_wait_word(slots + word_off + (long)r * n + i, epoch, v, status) && ok;
      sum += v;
    }
  }
  if (threadIdx.x == 0) trace_mark(trace, blockIdx.x, 1);
  pdl_wait();  // the residual stream belongs to the kernels before this one
  if (i < n && ok) h[i] = f2bf(__fadd_rn(bf2f(h[i]), round_bf16(sum)));
  if (threadIdx.x == 0) trace_mark(trace, blockIdx.x, 6);
}

__global__ void tp_pick_kernel(const bf16* logits, int vocab_local, int batch, int tp_rank, TpPeer peer, const unsigned long long* my_slots,
                               int64_t* tokens, int64_t* hist, const int* pos, int* status) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= batch) return;
  const unsigned epoch = *peer.epoch_ctr * 256u + (unsigned)peer.epoch_off;
  const int local = (int)tokens[b];
  const float best = bf2f(logits[(long)b * vocab_local + local]);
  const unsigned gidx = (unsigned)(local + tp_rank * vocab_local);
  const unsigned long long wv = ((unsigned long long)epoch << 32) | __float_as_uint(best);
  const unsigned long long wi = ((unsigned long long)epoch << 32) | gidx;
  const long at = peer.word_off + ((long)tp_rank * batch + b) * 2;
  for (int k = 0; k < peer.tp_size; ++k) {
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(peer.slots[k] + at), "l"(wv) : "memory");
    asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(peer.slots[k] + at + 1), "l"(wi) : "memory");
  }
  float top = -INFINITY;
  unsigned pick = 0xffffffffu;
  bool ok = true;
  for (int r = 0; r < peer.tp_size; ++r) {
    float v, fi;
    const unsigned long long* src = my_slots + peer.word_off + ((long)r * batch + b) * 2;
    ok = tp_wait_word(src, epoch, v, status) && ok;
    ok = tp_wait_word(src + 1, epoch, fi, status) && ok;
    const unsigned idx = __float_as_uint(fi);
    if (v > top || (v == top && idx < pick)) top = v, pick = idx;
  }
  if (!ok) {
    tokens[b] = -1;  // no valid pick: a token no vocabulary holds (the embedding gather reads it as a zero row)
    return;
  }
  tokens[b] = pick;
  if (hist) hist[(long)(*pos) * batch + b] = pick;
}

__global__ void bump_kernel(unsigned* counter) { *counter += 1u; }

// Row gather of the embedding table (src/deltaforge/reference.py:804).
__global__ void __launch_bounds__(128) embed_kernel(const bf16* table, const int64_t* tokens, int hidden, bf16* out, float* ss_out,
                                                    int ss_count) {
  __shared__ float wred[4];
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.x;
  const int64_t tok = tokens[b];
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const bf16 v = tok >= 0 ? table[tok * hidden + i] : f2bf(0.f);  // negative: the mark of a failed token pick
    out[(long)b * hidden + i] = v;
    ss = fmaf(bf2f(v), bf2f(v), ss);
  }
  if (ss_out == nullptr || b != 0) return;
  // sum of squares of the row, in the form the RMSNorm-prologue GEMV after this kernel reads it
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) wred[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x == 0) ss_out[0] = (wred[0] + wred[1]) + (wred[2] + wred[3]);
  for (int i = 1 + threadIdx.x; i < ss_count; i += blockDim.x) ss_out[i] = 0.f;
}

// argmax over a row of logits, first index on ties (what torch.argmax returns on the reference's CPU
// path, src/deltaforge/model.py:142). Blocks reduce strided chunks, the last block to arrive reduces
// the per-block results.
constexpr int AM_BLOCKS = 64;
__device__ __forceinline__ void argmax_merge(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) {
    v = ov;
    i = oi;
  }
}
__global__ void __launch_bounds__(256) argmax_kernel(const bf16* logits, int n, long stride, int64_t* out, int64_t* hist,
                                                     const int* pos, float* sval, int* sidx, unsigned* counter) {
  __shared__ float bv[8];
  __shared__ int bi[8];
  __shared__ int s_last;
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.y;
  const bf16* row = logits + (long)b * stride;
  float v = -INFINITY;
  int idx = 0x7fffffff;
  for (int i = blockIdx.x * 256 + threadIdx.x; i < n; i += AM_BLOCKS * 256) argmax_merge(v, idx, bf2f(row[i]), i);
  auto block_reduce = [&]() {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
      argmax_merge(v, idx, ov, oi);
    }
    if ((threadIdx.x & 31) == 0) {
      bv[threadIdx.x >> 5] = v;
      bi[threadIdx.x >> 5] = idx;
    }
    __syncthreads();
    if (threadIdx.x == 0)
      for (int w = 1; w < 8; ++w) argmax_merge(v, idx, bv[w], bi[w]);
  };
  block_reduce();
  if (threadIdx.x == 0) {
    __stcg(&sval[b * AM_BLOCKS + blockIdx.x], v);
    __stcg(&sidx[b * AM_BLOCKS + blockIdx.x], idx);
    __threadfence();
    const unsigned old = atomicAdd(&counter[b], 1u);
    s_last = (old == AM_BLOCKS - 1);
    if (s_last) counter[b] = 0u;
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  v = -INFINITY;
  idx = 0x7fffffff;
  if (threadIdx.x < AM_BLOCKS) {
    v = __ldcg(&sval[b * AM_BLOCKS + threadIdx.x]);
    idx = __ldcg(&sidx[b * AM_BLOCKS + threadIdx.x]);
  }
  __syncthreads();
  block_reduce();
  if (threadIdx.x == 0) {
    out[b] = idx;
    if (hist) hist[(long)(*pos) * gridDim.y + b] = idx;
  }
}

__global__ void advance_kernel(int* pos, int by) {
  pdl_wait();  // the argmax before this kernel still reads the position
  *pos += by;
}

}  // namespace

int launch_rms_norm(const bf16* x, const bf16* w, float eps, int rows, int n, bf16* out, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (launch_pdl(rms_norm_kernel, dim3(rows), dim3(256), 0, s, x, (const bf16*)nullptr, w, eps, n, (bf16*)nullptr, out) != cudaSuccess)
    return check_launch("rms_norm");
  return check_launch("rms_norm");
}

int launch_add_rms_norm(const bf16* x, const bf16* res, const bf16* w, float eps, int rows, int n, bf16* resid_out,
                        bf16* out, cudaStream_t s) {
  if (rows <= 0) return 0;
  if (launch_pdl(rms_norm_kernel, dim3(rows), dim3(256), 0, s, x, res, w, eps, n, resid_out, out) != cudaSuccess)
    return check_launch("add_rms_norm");
  return check_launch("add_rms_norm");
}

int launch_silu_mul(const bf16* gate, const bf16* up, long n, bf16* out, cudaStream_t s) {
  if (n <= 0) return 0;
  silu_mul_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(gate, up, n, out);
  return check_launch("silu_mul");
}

int launch_partial_rope(const bf16* x, const bf16* cos, const bf16* sin, int batch, int heads, int seq, int d, int rd,
                        bf16* out, cudaStream_t s) {
  const long rows = (long)batch * heads * seq;
  if (rows <= 0) return 0;
  partial_rope_kernel<<<(unsigned)rows, 128, 0, s>>>(x, cos, sin, heads, seq, d, rd, out);
  return check_launch("partial_rope");
}

int launch_causal_conv_step(const bf16* x, bf16* cache, const bf16* w, int batch, int channels, bf16* out,
                            cudaStream_t s) {
  const long total = (long)batch * channels;
  if (total <= 0) return 0;
  causal_conv_step_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(x, cache, w, channels, total, out);
  return check_launch("causal_conv_step");
}

int launch_silu_mul_rows(const bf16* gate, const bf16* up, long in_stride, int rows, int n, bf16* out, cudaStream_t s) {
  const long total = (long)rows * n;
  if (total <= 0) return 0;
  if (launch_pdl(silu_mul_rows_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, gate, up, in_stride, n, total, out) != cudaSuccess)
    return check_launch("silu_mul (rows)");
  return check_launch("silu_mul (rows)");
}

int launch_causal_conv_rows(bf16* x, long x_stride, bf16* cache, const bf16* w, int rows, int channels, cudaStream_t s) {
  const long total = (long)rows * channels;
  if (total <= 0) return 0;
  if (launch_pdl(causal_conv_rows_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, s, x, x_stride, cache, w, channels, total) != cudaSuccess)
    return check_launch("causal conv (rows)");
  return check_launch("causal_conv_step (rows)");
}

int launch_add_partial(bf16* h, const float* sum, long n, cudaStream_t s) {
  if (n <= 0) return 0;
  add_partial_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(h, sum, n);
  return check_launch("add_partial");
}

int launch_tp_reduce(bf16* h, const unsigned long long* slots, int tp_size, long n, long word_off, const unsigned* epoch_ctr,
                     int epoch_off, int* status, const Trace& trace, cudaStream_t s) {
  if (n <= 0) return 0;
  const cudaError_t e = launch_pdl(tp_reduce_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, h, slots, tp_size, n, word_off,
                                   epoch_ctr, epoch_off, status, trace);
  if (e != cudaSuccess) {
    set_error("tp_reduce: launch failed: %s", cudaGetErrorString(e));
    return 1;
  }
  return check_launch("tp_reduce");
}

int launch_tp_pick(const bf16* logits, int vocab_local, int batch, int tp_rank, const TpPeer& peer, const unsigned long long* my_slots,
                   int64_t* tokens, int64_t* hist, const int* pos, int* status, cudaStream_t s) {
  if (batch <= 0) return 0;
  tp_pick_kernel<<<(batch + 63) / 64, 64, 0, s>>>(logits, vocab_local, batch, tp_rank, peer, my_slots, tokens, hist, pos, status);
  return check_launch("tp_pick");
}

int launch_bump(unsigned* counter, cudaStream_t s) {
  bump_kernel<<<1, 1, 0, s>>>(counter);
  return check_launch("bump");
}

int elementwise_configure() {
  cudaError_t e = prefer_max_shared(embed_kernel);
  if (e == cudaSuccess) e = prefer_max_shared(argmax_kernel);
  if (e == cudaSuccess) e = prefer_max_shared(advance_kernel);
  return e == cudaSuccess ? 0 : check_launch("elementwise: shared-memory carve-out");
}

int launch_embed(const bf16* table, const int64_t* tokens, int batch, int hidden, bf16* out, float* ss_out, int ss_count,
                 cudaStream_t s) {
  if (batch <= 0) return 0;
  if (launch_pdl(embed_kernel, dim3(batch), dim3(128), 0, s, table, tokens, hidden, out, ss_out, ss_count) != cudaSuccess)
    return check_launch("embed");
  return check_launch("embed");
}

int launch_argmax(const bf16* logits, int batch, int n, long stride, int64_t* out, int64_t* hist, const int* pos,
                  float* scratch_val, int* scratch_idx, unsigned* counter, cudaStream_t s) {
  if (batch <= 0) return 0;
  if (launch_pdl(argmax_kernel, dim3(AM_BLOCKS, batch), dim3(256), 0, s, logits, n, stride, out, hist, pos, scratch_val, scratch_idx,
                 counter) != cudaSuccess)
    return check_launch("argmax");
  return check_launch("argmax");
}

int launch_advance(int* pos, int by, cudaStream_t s) {
  if (launch_pdl(advance_kernel, dim3(1), dim3(1), 0, s, pos, by) != cudaSuccess) return check_launch("advance");
  return check_launch("advance");
}

}  // namespace dfb
