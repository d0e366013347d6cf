// The whole single-token decode step as one launch sequence, captured into one CUDA graph.
//
// Stands in for ReferenceModel.forward at seq_len 1 plus the argmax of greedy_decode
// (src/deltaforge/reference.py:779-817, src/deltaforge/model.py:141-147). Five launches per layer:
//   1. RMSNorm-prologue int4 GEMV over the concatenated input projections
//      (DeltaNet: in_proj_qkv|z|b|a with the causal conv + SiLU in the epilogue; attention: q|k|v)
//   2. DeltaNet step, or attention prep (norms, RoPE, KV write) + split-KV decode (2 launches)
//   3. out_proj / o_proj GEMV with the residual add in the epilogue
//   4. RMSNorm-prologue GEMV over gate_proj|up_proj
//   5. SwiGLU-prologue down_proj GEMV with the residual add in the epilogue
// then the final-norm-prologue LM-head GEMV and the argmax. The position lives in device memory and
// is advanced by the last node, so the same graph replays for every token.
#include <new>
#include <vector>

#include "../../include/dfb200.h"
#include "common.cuh"
#include "kernels.h"

namespace dfb {

int gemv_configure();
int attn_configure();
int deltanet_configure();
int elementwise_configure();

int configure_kernels() {
  if (int rc = gemv_configure()) return rc;
  if (int rc = attn_step_configure()) return rc;
  if (int rc = deltanet_configure()) return rc;
  if (int rc = elementwise_configure()) return rc;
  return attn_configure();
}

namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

struct Workspace {
  size_t h, proj, mix, qout, gu, partials, counters, attn, am_val, am_idx, am_ctr, status, h_ss, xn, ar, epoch, total;
};

size_t linear_partials(const dfb_linear& l, int rows) { return gemv_partials_bytes(rows, l.K, l.N, l.group); }
size_t linear_counters(const dfb_linear& l, int rows) { return gemv_counter_count(rows, l.K, l.N, l.group) * 4; }

Workspace plan(const dfb_model_desc& m) {
  Workspace w = {};
  const size_t B = (size_t)m.batch;
  size_t max_proj = 0, max_part = 0, max_ctr = 0;
  auto visit = [&](const dfb_linear& l) {
    max_part = std::max(max_part, linear_partials(l, m.batch));
    max_ctr = std::max(max_ctr, linear_counters(l, m.batch));
  };
  for (int i = 0; i < m.num_layers; ++i) {
    const dfb_layer_desc& L = m.layers_host[i];
    max_proj = std::max(max_proj, (size_t)L.in_proj.N);
    visit(L.in_proj);
    visit(L.out_proj);
    visit(L.gate_up);
    visit(L.down);
  }
  visit(m.head);
  const size_t mixw = std::max((size_t)m.lin_v_heads * m.lin_dv, (size_t)m.hq * m.head_dim);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    const size_t at = off;
    off += align_up(bytes, 256);
    return at;
  };
  w.h = take(B * m.hidden * 2);
  w.proj = take(B * max_proj * 2);
  w.mix = take(B * mixw * 2);
  w.qout = take(B * m.hq * m.head_dim * 2);
  w.gu = take(B * 2 * m.intermediate * 2);
  w.partials = take(max_part);
  w.counters = take(max_ctr);
  w.attn = take(dfb_attn_scratch_bytes(m.batch, m.hq, m.hkv, m.head_dim, m.attn_splits));
  w.am_val = take(B * 64 * 4);
  w.am_idx = take(B * 64 * 4);
  w.am_ctr = take(B * 4);
  w.status = take(256);
  w.h_ss = take(256 * 4);
  // batches of eight and more: the normalised / gated activation the tensor-core product reads
  w.xn = take(m.batch >= 8 ? B * std::max(std::max((size_t)m.hidden, (size_t)m.intermediate), mixw) * 2 : 0);
  w.ar = take(m.tp_size > 1 ? B * m.hidden * 4 : 0);
  w.epoch = take(m.tp_size > 1 ? 256 : 0);
  w.total = off;
  return w;
}

struct Engine {
  dfb_model_desc m;
  std::vector<dfb_layer_desc> layers;
  Workspace ws;
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  int launches = 0;
  bool ss_valid = false;  // the residual stream's per-tile sums of squares in h_ss are current
  unsigned long long* peer_slots[TP_MAX] = {};  // tensor parallelism by peer stores: every rank's exchange buffer
  TpPeer cur_peer = {};                          // where the next EPI_PARTIAL_PEER projection writes
  const void* next_touch[3] = {nullptr, nullptr, nullptr};  // small arrays the next projection asks the L2 for (then cleared)
  int next_touch_bytes[3] = {0, 0, 0};
  AttnMerge cur_merge = {};                      // what the next PRO_ATTN_MERGE projection reads
  // The projections of one step in launch order, and which of them the next GEMV launch is: every kernel of
  // the batch-1 step asks the L2 for the weights of the projection `pf_dist` GEMVs ahead (0: off).
  std::vector<const dfb_linear*> order;
  int cursor = 0;
  int pf_dist = 0;  // measured: with programmatic dependent launch the next kernel's own copies already run ahead
  Trace trace = {};      // optional timeline buffer (dfb_engine_set_trace)
  int trace_launches = 0;

  char* at(size_t off) const { return (char*)m.workspace + off; }

  void plan_order() {
    order.clear();
    for (int i = 0; i < m.num_layers; ++i) {
      order.push_back(&layers[i].in_proj);
      order.push_back(&layers[i].out_proj);
      order.push_back(&layers[i].gate_up);
      order.push_back(&layers[i].down);
    }
    order.push_back(&m.head);
  }
  // Prefetch target for a launch that runs while GEMV number `idx` (of `order`) is the one to come `pf_dist`
  // projections later. Only layer-sized weights: the LM head is 300 MB and streams at full rate by itself.
  void aim_prefetch(const void** ptr, size_t* bytes, int idx) const {
    ptr[0] = ptr[1] = nullptr;
    bytes[0] = bytes[1] = 0;
    if (pf_dist <= 0 || m.batch != 1 || m.tp_size > 1 || idx < 0 || idx >= (int)order.size()) return;
    const dfb_linear& l = *order[idx];
    const size_t wbytes = (size_t)l.K * l.N / 2;
    if (wbytes > ((size_t)48 << 20)) return;
    if (l.packed_mma) {  // the copy the tensor-core GEMV reads: words and scales in one buffer
      ptr[0] = l.packed_mma;
      bytes[0] = mma_repack_bytes(l.K, l.N, l.mma_pair, l.scale_is_bf16);
      return;
    }
    if (!l.packed_k8) return;
    ptr[0] = l.packed_k8;
    bytes[0] = wbytes;
    ptr[1] = l.scale;
    bytes[1] = (size_t)(l.K / l.group) * l.N * (l.scale_is_bf16 ? 2 : 4);
  }
  Trace launch_trace() const {
    Trace t = trace;
    t.slot = launches;
    if (launches >= trace_launches) t.buf = nullptr;
    return t;
  }

  int gemv(const dfb_linear& l, const bf16* x, long x_stride, int prologue, const void* norm_w, const bf16* up,
           long up_stride, int epilogue, bf16* out, long out_stride, const dfb_layer_desc* conv_layer, cudaStream_t s) {
    if (m.batch >= 8 && l.packed_k8 && m.math != MATH_FAST_HALF2 && epilogue != EPI_PARTIAL_F32 && epilogue != EPI_PARTIAL_PEER) {
      // Tensor-core path: prologue and the conv epilogue run as their own small kernels around the product.
      GemvParams q = {};
      q.x = x;
      q.x_stride = x_stride;
      if (prologue == PRO_RMSNORM) {
        if (x_stride != l.K) {
          set_error("engine: RMSNorm prologue expects contiguous rows");
          return DFB_ERR_ARG;
        }
        if (int rc = launch_rms_norm(x, (const bf16*)norm_w, m.eps, m.batch, l.K, (bf16*)at(ws.xn), s)) return rc;
        ++launches;
        q.x = (const bf16*)at(ws.xn);
        q.x_stride = l.K;
      } else if (prologue == PRO_SILU_MUL) {
        if (int rc = launch_silu_mul_rows(x, up, x_stride, m.batch, l.K, (bf16*)at(ws.xn), s)) return rc;
        ++launches;
        q.x = (const bf16*)at(ws.xn);
        q.x_stride = l.K;
      }
      q.rows = m.batch;
      q.packed = l.packed;
      q.packed_k8 = (const uint32_t*)l.packed_k8;
      q.scale = l.scale;
      q.scale_bf16 = l.scale_is_bf16;
      q.K = l.K, q.N = l.N, q.group = l.group;
      q.prologue = PRO_NONE;
      q.epilogue = epilogue == EPI_RESIDUAL ? EPI_RESIDUAL : EPI_STORE;
      q.out = out, q.out_stride = out_stride;
      q.residual = out, q.res_stride = out_stride;
      q.partials = (float*)at(ws.partials);
      q.counters = (unsigned*)at(ws.counters);
      q.math = m.math;
      q.status = (int*)at(ws.status);
      if (tc_path_ok(q)) {
        ss_valid = false;
        ++launches;
        if (int rc = launch_gemv(q, s)) return rc;
        if (conv_layer) {
          ++launches;
          return launch_causal_conv_rows(out, out_stride, (bf16*)conv_layer->conv_state, (const bf16*)conv_layer->conv_w, m.batch,
                                         2 * m.lin_k_heads * m.lin_dk + m.lin_v_heads * m.lin_dv, s);
        }
        return 0;
      }
    }
    const bool x_is_h = (const void*)x == (const void*)at(ws.h);
    GemvParams p = {};
    p.x = x;
    p.x_stride = x_stride;
    p.rows = m.batch;
    p.packed = l.packed;
    p.packed_k8 = (const uint32_t*)l.packed_k8;
    // the gate|up pair layout serves the SwiGLU epilogue only; every other copy serves every other epilogue
    if (l.packed_mma && (l.mma_pair != 0) == (epilogue == EPI_SWIGLU)) {
      p.packed_mma = (const unsigned char*)l.packed_mma;
      p.mma_pair = l.mma_pair;
    }
    p.scale = l.scale;
    p.scale_bf16 = l.scale_is_bf16;
    p.K = l.K;
    p.N = l.N;
    p.group = l.group;
    p.prologue = prologue;
    p.norm_w = (const bf16*)norm_w;
    p.eps = m.eps;
    p.up = up;
    p.up_stride = up_stride;
    p.epilogue = epilogue;
    p.out = out;
    p.out_stride = out_stride;
    p.residual = out;
    p.res_stride = out_stride;
    if (conv_layer) {
      p.conv_state = (bf16*)conv_layer->conv_state;
      p.conv_w = (const bf16*)conv_layer->conv_w;
      p.conv_dim = 2 * m.lin_k_heads * m.lin_dk + m.lin_v_heads * m.lin_dv;
      p.conv_state_settled = 1;  // written by this projection of the previous token, a whole graph launch ago
    }
    p.partials = (float*)at(ws.partials);
    p.counters = (unsigned*)at(ws.counters);
    p.math = m.math;
    p.status = (int*)at(ws.status);
    if (epilogue == EPI_PARTIAL_PEER) p.peer = cur_peer;
    for (int i = 0; i < 3; ++i) {
      p.touch_ptr[i] = next_touch[i], p.touch_bytes[i] = next_touch_bytes[i];
      next_touch[i] = nullptr, next_touch_bytes[i] = 0;
    }
    if (prologue == PRO_ATTN_MERGE) p.merge = cur_merge;
    aim_prefetch(p.pf_ptr, p.pf_bytes, cursor + pf_dist);
    ++cursor;
    p.trace = launch_trace();
    // Sum-of-squares hand-off along the residual stream (batch 1, cluster kernel on both sides).
    const int h_tiles = (m.hidden + cluster_tile_width(m.hidden) - 1) / cluster_tile_width(m.hidden);
    if (prologue == PRO_RMSNORM && x_is_h && ss_valid) {
      p.ss_in = (const float*)at(ws.h_ss);
      p.ss_count = h_tiles;
    }
    if (epilogue == EPI_RESIDUAL) {
      ss_valid = m.batch == 1 && h_tiles <= 256 && l.N < 65536 && (mma_path_ok(p) || cluster_path_ok(p));
      if (ss_valid) p.ss_out = (float*)at(ws.h_ss);
    }
    ++launches;
    return launch_gemv(p, s);
  }

  // ---- the token mixers ------------------------------------------------------------------------------------
  int mixer_deltanet(const dfb_layer_desc& L, bf16* proj, long pstride, bf16* mix, cudaStream_t s) {
    const int kd = m.lin_k_heads * m.lin_dk, vd = m.lin_v_heads * m.lin_dv;
    DeltaNetParams d = {};
    d.batch = m.batch;
    d.num_k_heads = m.lin_k_heads;
    d.num_v_heads = m.lin_v_heads;
    d.dk = m.lin_dk;
    d.dv = m.lin_dv;
    d.q = proj;
    d.k = proj + kd;
    d.v = proj + 2 * kd;
    d.z = proj + 2 * kd + vd;
    d.b = proj + 2 * kd + 2 * vd;
    d.a = proj + 2 * kd + 2 * vd + m.lin_v_heads;
    d.row_stride = pstride;
    d.a_log = L.a_log;
    d.dt_bias = L.dt_bias;
    d.norm_w = L.gnorm_w;
    d.norm_w_bf16 = L.gnorm_w_is_bf16;
    d.eps = m.eps;
    d.state = L.recurrent;
    d.out = mix;
    d.out_stride = vd;
    aim_prefetch(d.pf_ptr, d.pf_bytes, cursor + pf_dist - 1);
    d.trace = launch_trace();
    ++launches;
    return launch_deltanet_step(d, s);
  }

  // Batch 1, one GPU: when the fused attention step cuts the cache into more than one cluster of slices, the clusters'
  // partial results are merged by the output projection while it builds its activation, not by a last-arriver
  // protocol through global memory at the end of the attention kernel.
  int attn_cluster_size() const {
    // small clusters schedule sooner; at most 8 clusters per KV head, so that the output projection can merge them
    // (up to 16 where the last cluster to arrive merges: 128 slices of a long cache)
    int c = std::min(m.attn_splits, 4);
    while (c < 8 && m.attn_splits / c > 8) c *= 2;
    return c;
  }
  bool attn_defer_merge(const dfb_layer_desc& L) const {
    if (m.batch != 1 || tp() || m.math != MATH_FAST || !(L.out_proj.packed_k8 || L.out_proj.packed_mma)) return false;
    if (!attn_step_ok(m.head_dim, m.hq, m.hkv, m.rotary_dim, m.attn_splits, m.max_seq)) return false;
    const int ncl = m.attn_splits / attn_cluster_size();
    if (ncl < 2 || ncl > 8) return false;
    GemvParams q = {};
    q.rows = 1;
    q.packed_k8 = (const uint32_t*)L.out_proj.packed_k8;
    if (L.out_proj.packed_mma && !L.out_proj.mma_pair) q.packed_mma = (const unsigned char*)L.out_proj.packed_mma;
    q.scale_bf16 = L.out_proj.scale_is_bf16;
    q.scale = L.out_proj.scale;
    q.K = L.out_proj.K, q.N = L.out_proj.N, q.group = L.out_proj.group;
    q.prologue = PRO_ATTN_MERGE;
    q.epilogue = EPI_RESIDUAL;
    q.math = MATH_FAST;
    q.x = (const bf16*)at(ws.mix);
    q.merge.acc = (const float*)at(ws.attn);
    q.merge.ml = q.merge.acc;
    q.merge.nclusters = ncl;
    q.merge.d = m.head_dim;
    return mma_path_ok(q) || (q.packed_k8 && cluster_path_ok(q));
  }

  int mixer_attention(const dfb_layer_desc& L, bf16* proj, long pstride, bf16* mix, bf16* qout, cudaStream_t s) {
    const int d_ = m.head_dim;
    const long kvb = (long)m.hkv * m.max_seq * d_, kvh = (long)m.max_seq * d_;
    // One or two sequences: the fused single-launch kernel (latency matters). More: its 160-key staging leaves
    // one CTA per SM alternating between copying and computing, and the two-kernel path with the tensor-core
    // decode streams the cache several times faster.
    if (m.batch <= 2 && attn_step_ok(d_, m.hq, m.hkv, m.rotary_dim, m.attn_splits, m.max_seq)) {
      // norms, RoPE, KV write, split-KV decode, merge and gate in one launch
      AttnStepParams q = {};
      q.batch = m.batch;
      q.hq = m.hq;
      q.hkv = m.hkv;
      q.d = d_;
      q.rotary_dim = m.rotary_dim;
      q.proj = proj;
      q.proj_stride = pstride;
      q.q_norm_w = (const bf16*)L.q_norm_w;
      q.k_norm_w = (const bf16*)L.k_norm_w;
      q.eps = m.eps;
      q.inv_freq = m.inv_freq;
      q.pos = m.pos;
      q.kcache = (bf16*)L.kcache;
      q.vcache = (bf16*)L.vcache;
      q.kv_batch_stride = kvb;
      q.kv_head_stride = kvh;
      q.max_seq = m.max_seq;
      q.attn_output_gate = m.attn_output_gate;
      q.gate_swish = m.gate_is_swish;
      q.scale = 1.0f / sqrtf((float)d_);
      q.splits = m.attn_splits;
      // these CTAs fill an SM each: small clusters schedule sooner; the last merge takes at most 16 clusters,
      // so the longest caches of a one-KV-head shard (128 slices) use clusters of 8
      q.cluster_size = attn_cluster_size();
      if (m.attn_splits > 1) {
        char* sc = at(ws.attn);
        q.part_acc = (float*)sc;
        sc += align_up((size_t)m.batch * m.hq * m.attn_splits * d_ * 4, 256);
        q.part_ml = (float*)sc;
        sc += align_up((size_t)m.batch * m.hq * m.attn_splits * 2 * 4, 256);
        q.counters = (unsigned*)sc;
      }
      q.defer_merge = attn_defer_merge(L) ? 1 : 0;
      if (q.defer_merge) {
        cur_merge = {};
        cur_merge.acc = q.part_acc;
        cur_merge.ml = q.part_ml;
        cur_merge.nclusters = m.attn_splits / q.cluster_size;
        cur_merge.d = d_;
        if (m.attn_output_gate) {  // the attention step leaves the activated gate where its output would have gone
          cur_merge.gate = mix;
          cur_merge.gateh_stride = d_;
        }
      }
      q.out = mix;
      q.out_stride = (long)m.hq * d_;
      q.status = (int*)at(ws.status);
      aim_prefetch(q.pf_ptr, q.pf_bytes, cursor + pf_dist - 1);
      q.trace = launch_trace();
      ++launches;
      return launch_attn_step(q, s);
    }
    AttnPrepParams pp = {};
    pp.batch = m.batch;
    pp.hq = m.hq;
    pp.hkv = m.hkv;
    pp.d = d_;
    pp.rotary_dim = m.rotary_dim;
    pp.proj = proj;
    pp.proj_stride = pstride;
    pp.q_norm_w = (const bf16*)L.q_norm_w;
    pp.k_norm_w = (const bf16*)L.k_norm_w;
    pp.eps = m.eps;
    pp.inv_freq = m.inv_freq;
    pp.pos = m.pos;
    pp.q_out = qout;
    pp.kcache = (bf16*)L.kcache;
    pp.vcache = (bf16*)L.vcache;
    pp.kv_batch_stride = kvb;
    pp.kv_head_stride = kvh;
    pp.attn_output_gate = m.attn_output_gate;
    pp.max_seq = m.max_seq;
    ++launches;
    if (int rc = launch_attn_prep(pp, s)) return rc;
    AttnParams a = {};
    a.batch = m.batch;
    a.hq = m.hq;
    a.hkv = m.hkv;
    a.d = d_;
    a.q = qout;
    a.q_stride = (long)m.hq * d_;
    a.qh_stride = d_;
    a.kcache = (const bf16*)L.kcache;
    a.vcache = (const bf16*)L.vcache;
    a.kv_batch_stride = kvb;
    a.kv_head_stride = kvh;
    a.pos = m.pos;
    a.key_len = m.max_seq;  // capacity; the live length is *pos + 1
    a.scale = 1.0f / sqrtf((float)d_);
    a.splits = m.attn_splits;
    if (m.attn_splits > 1) {
      char* sc = at(ws.attn);
      a.part_acc = (float*)sc;
      sc += align_up((size_t)m.batch * m.hq * m.attn_splits * d_ * 4, 256);
      a.part_ml = (float*)sc;
      sc += align_up((size_t)m.batch * m.hq * m.attn_splits * 2 * 4, 256);
      a.counters = (unsigned*)sc;
    }
    if (m.attn_output_gate) {
      a.gate = proj + d_;
      a.gate_stride = pstride;
      a.gateh_stride = 2 * d_;
      a.gate_swish = m.gate_is_swish;
    }
    a.out = mix;
    a.out_stride = (long)m.hq * d_;
    ++launches;
    return launch_attn_decode(a, s);
  }

  // ---- the step, in halves of a layer ----------------------------------------------------------------------
  // With tensor parallelism (tp_size > 1) the K-sharded projections at the end of each half leave fp32 partial
  // sums in the `ar` buffer instead of adding into the residual stream; the caller all-reduces that buffer
  // between segments and the next segment starts with the residual add.
  bool tp() const { return m.tp_size > 1; }
  bool peer() const { return tp() && peer_slots[0] != nullptr; }
  long bh() const { return (long)m.batch * m.hidden; }
  // all-reduce number `a` of the step (0 .. 2 * layers - 1) alternates between two slot sets
  void aim_peer(int a) {
    cur_peer = {};
    for (int r = 0; r < m.tp_size; ++r) cur_peer.slots[r] = peer_slots[r];
    cur_peer.tp_size = m.tp_size;
    cur_peer.epoch_ctr = (const unsigned*)at(ws.epoch);
    cur_peer.epoch_off = a;
    cur_peer.word_off = ((long)(a & 1) * m.tp_size + m.tp_rank) * bh();
  }
  int num_segments() const { return tp() ? 2 * m.num_layers + 1 : 1; }

  int first_half(int i, cudaStream_t s) {  // input projections, token mixer, output projection
    const dfb_layer_desc& L = layers[i];
    bf16* h = (bf16*)at(ws.h);
    bf16* proj = (bf16*)at(ws.proj);
    bf16* mix = (bf16*)at(ws.mix);
    const int H = m.hidden;
    const long pstride = L.in_proj.N;
    const bool dn = L.kind == DFB_LAYER_DELTANET;
    if (!dn) {
      // the attention step reads its norm weights and rotary frequencies first thing after its wait, eight times per token:
      // they are not in the L2 by then unless somebody asks for them; the projection before it does
      next_touch[0] = L.q_norm_w, next_touch_bytes[0] = m.head_dim * 2;
      next_touch[1] = L.k_norm_w, next_touch_bytes[1] = m.head_dim * 2;
      next_touch[2] = m.inv_freq, next_touch_bytes[2] = m.rotary_dim / 2 * 4;
    }
    int rc = gemv(L.in_proj, h, H, PRO_RMSNORM, L.input_norm_w, nullptr, 0, dn ? EPI_CONV : EPI_STORE, proj, pstride, dn ? &L : nullptr, s);
    if (rc) return rc;
    rc = dn ? mixer_deltanet(L, proj, pstride, mix, s) : mixer_attention(L, proj, pstride, mix, (bf16*)at(ws.qout), s);
    if (rc) return rc;
    const long mixw = dn ? (long)m.lin_v_heads * m.lin_dv : (long)m.hq * m.head_dim;
    if (peer()) {
      aim_peer(2 * i);
      return gemv(L.out_proj, mix, mixw, PRO_NONE, nullptr, nullptr, 0, EPI_PARTIAL_PEER, (bf16*)at(ws.ar), H, nullptr, s);
    }
    if (tp()) return gemv(L.out_proj, mix, mixw, PRO_NONE, nullptr, nullptr, 0, EPI_PARTIAL_F32, (bf16*)at(ws.ar), H, nullptr, s);
    const int pro = (!dn && attn_defer_merge(L)) ? PRO_ATTN_MERGE : PRO_NONE;
    return gemv(L.out_proj, mix, mixw, pro, nullptr, nullptr, 0, EPI_RESIDUAL, h, H, nullptr, s);
  }

  bool swiglu_in_gate_up(const dfb_layer_desc& L) const {
    if (m.batch != 1 || m.math != MATH_FAST || !(L.gate_up.packed_k8 || L.gate_up.packed_mma)) return false;
    GemvParams q = {};
    q.rows = 1;
    q.packed_k8 = (const uint32_t*)L.gate_up.packed_k8;
    if (L.gate_up.packed_mma && L.gate_up.mma_pair) {
      q.packed_mma = (const unsigned char*)L.gate_up.packed_mma;
      q.mma_pair = 1;
    }
    q.scale_bf16 = L.gate_up.scale_is_bf16;
    q.scale = L.gate_up.scale;
    q.K = L.gate_up.K, q.N = L.gate_up.N, q.group = L.gate_up.group;
    q.prologue = PRO_RMSNORM;
    q.epilogue = EPI_SWIGLU;
    q.math = MATH_FAST;
    q.x = (const bf16*)at(ws.h);
    q.norm_w = (const bf16*)L.post_norm_w;
    return mma_path_ok(q) || (q.packed_k8 && cluster_path_ok(q));
  }

  int second_half(int i, cudaStream_t s) {  // SwiGLU MLP
    const dfb_layer_desc& L = layers[i];
    bf16* h = (bf16*)at(ws.h);
    bf16* gu = (bf16*)at(ws.gu);
    const int H = m.hidden, I = m.intermediate;
    // Where the kernel can, gate|up leaves bf16(silu(gate)) * up directly (a cluster holds a gate tile and the up tile of
    // the same channels) and the down projection reads it as it is; otherwise down applies SwiGLU in its prologue.
    const bool fused = swiglu_in_gate_up(L);
    int rc = fused ? gemv(L.gate_up, h, H, PRO_RMSNORM, L.post_norm_w, nullptr, 0, EPI_SWIGLU, gu, I, nullptr, s)
                   : gemv(L.gate_up, h, H, PRO_RMSNORM, L.post_norm_w, nullptr, 0, EPI_STORE, gu, 2L * I, nullptr, s);
    if (rc) return rc;
    const long xs = fused ? I : 2L * I;
    const int pro = fused ? PRO_NONE : PRO_SILU_MUL;
    const bf16* up = fused ? nullptr : gu + I;
    if (peer()) {
      aim_peer(2 * i + 1);
      return gemv(L.down, gu, xs, pro, nullptr, up, xs, EPI_PARTIAL_PEER, (bf16*)at(ws.ar), H, nullptr, s);
    }
    if (tp()) return gemv(L.down, gu, xs, pro, nullptr, up, xs, EPI_PARTIAL_F32, (bf16*)at(ws.ar), H, nullptr, s);
    return gemv(L.down, gu, xs, pro, nullptr, up, xs, EPI_RESIDUAL, h, H, nullptr, s);
  }

  int head_and_pick(cudaStream_t s) {
    bf16* h = (bf16*)at(ws.h);
    int rc = gemv(m.head, h, m.hidden, PRO_RMSNORM, m.final_norm_w, nullptr, 0, EPI_STORE, (bf16*)m.logits, m.vocab, nullptr, s);
    if (rc) return rc;
    if (peer()) {
      // each rank's best logit, then the pick across the vocabulary shards by peer exchange
      rc = launch_argmax((const bf16*)m.logits, m.batch, m.vocab, m.vocab, m.tokens, nullptr, m.pos, (float*)at(ws.am_val),
                         (int*)at(ws.am_idx), (unsigned*)at(ws.am_ctr), s);
      ++launches;
      if (rc) return rc;
      TpPeer pk = {};
      for (int r = 0; r < m.tp_size; ++r) pk.slots[r] = peer_slots[r];
      pk.tp_size = m.tp_size;
      pk.epoch_ctr = (const unsigned*)at(ws.epoch);
      pk.epoch_off = 255;
      pk.word_off = 2L * m.tp_size * bh();
      rc = launch_tp_pick((const bf16*)m.logits, m.vocab, m.batch, m.tp_rank, pk, peer_slots[m.tp_rank], m.tokens, m.history, m.pos,
                          (int*)at(ws.status), s);
      ++launches;
      if (rc) return rc;
      rc = launch_advance(m.pos, 1, s);
      ++launches;
      if (rc) return rc;
      ++launches;
      return launch_bump((unsigned*)at(ws.epoch), s);
    }
    if (!tp()) {  // with a sharded vocabulary the caller picks the token across ranks
      rc = launch_argmax((const bf16*)m.logits, m.batch, m.vocab, m.vocab, m.tokens, m.history, m.pos, (float*)at(ws.am_val),
                         (int*)at(ws.am_idx), (unsigned*)at(ws.am_ctr), s);
      ++launches;
      if (rc) return rc;
    }
    rc = launch_advance(m.pos, 1, s);
    ++launches;
    return rc;
  }

  int embed(cudaStream_t s) {
    const int H = m.hidden;
    const int h_tiles = (H + cluster_tile_width(H) - 1) / cluster_tile_width(H);
    ss_valid = m.batch == 1 && h_tiles <= 256 && !tp();
    ++launches;
    return launch_embed((const bf16*)m.embed, m.tokens, m.batch, H, (bf16*)at(ws.h), ss_valid ? (float*)at(ws.h_ss) : nullptr, h_tiles, s);
  }

  int add_partial(int seg, cudaStream_t s) {
    ss_valid = false;
    if (peer()) {
      const int a = seg - 1;  // the all-reduce that ended the previous segment
      const Trace tr = launch_trace();
      ++launches;
      return launch_tp_reduce((bf16*)at(ws.h), peer_slots[m.tp_rank], m.tp_size, bh(), (long)(a & 1) * m.tp_size * bh(),
                              (const unsigned*)at(ws.epoch), a, (int*)at(ws.status), tr, s);
    }
    ++launches;
    return launch_add_partial((bf16*)at(ws.h), (const float*)at(ws.ar), (long)m.batch * m.hidden, s);
  }

  // Segment `seg` of a tensor-parallel step: 0 = embedding + first half of layer 0; 2l+1 = second half of
  // layer l; 2l+2 = first half of layer l+1; the last = head. Every segment but the first begins with the
  // residual add of the all-reduced buffer.
  int step_segment(int seg, cudaStream_t s) {
    if (!tp() || seg < 0 || seg >= num_segments()) {
      set_error("engine: segment %d of %d (tensor-parallel engines only)", seg, num_segments());
      return DFB_ERR_ARG;
    }
    if (seg == 0) launches = cursor = 0;
    if (seg == 0) {
      if (int rc = embed(s)) return rc;
    } else {
      if (int rc = add_partial(seg, s)) return rc;
    }
    if (seg == 2 * m.num_layers) return head_and_pick(s);
    if (seg & 1) return second_half(seg / 2, s);
    return first_half(seg / 2, s);
  }

  int step(cudaStream_t s) {
    if (peer()) {  // the ranks exchange by peer stores inside the kernels: the whole step is one launch sequence
      for (int seg = 0; seg < num_segments(); ++seg)
        if (int rc = step_segment(seg, s)) return rc;
      return 0;
    }
    if (tp()) {
      set_error("engine: a tensor-parallel step is run segment by segment, with an all-reduce of the partial buffer in between");
      return DFB_ERR_ARG;
    }
    launches = 0;
    cursor = 0;
    if (int rc = embed(s)) return rc;
    for (int i = 0; i < m.num_layers; ++i) {
      if (int rc = first_half(i, s)) return rc;
      if (int rc = second_half(i, s)) return rc;
    }
    return head_and_pick(s);
  }
};

int validate(const dfb_model_desc& m) {
  if (m.batch < 1 || m.num_layers < 0 || m.hidden < 1 || m.vocab < 1) {
    set_error("engine: bad model shape");
    return DFB_ERR_ARG;
  }
  if (!m.embed || !m.final_norm_w || !m.tokens || !m.pos || !m.logits || !m.workspace || !m.inv_freq ||
      (m.num_layers && !m.layers_host)) {
    set_error("engine: null pointer in the model description");
    return DFB_ERR_ARG;
  }
  if (m.tp_size > 1 && m.tp_peer_slots && 2 * m.num_layers > 254) {
    // the exchange tag is epoch * 256 + (index of the exchange within the token), 255 being the token pick
    set_error("engine: the peer exchange tags at most 254 exchanges per token; %d layers need %d", m.num_layers, 2 * m.num_layers);
    return DFB_ERR_ARG;
  }
  if (m.head.K != m.hidden || m.head.N != m.vocab) {
    set_error("engine: LM head is %dx%d, expected %dx%d", m.head.N, m.head.K, m.vocab, m.hidden);
    return DFB_ERR_ARG;
  }
  const int conv_dim = 2 * m.lin_k_heads * m.lin_dk + m.lin_v_heads * m.lin_dv;
  for (int i = 0; i < m.num_layers; ++i) {
    const dfb_layer_desc& L = m.layers_host[i];
    int want_in, want_mix;
    if (L.kind == DFB_LAYER_DELTANET) {
      want_in = conv_dim + m.lin_v_heads * m.lin_dv + 2 * m.lin_v_heads;
      want_mix = m.lin_v_heads * m.lin_dv;
      if (!L.conv_w || !L.a_log || !L.dt_bias || !L.gnorm_w || !L.conv_state || !L.recurrent) {
        set_error("engine: layer %d (DeltaNet) has a null pointer", i);
        return DFB_ERR_ARG;
      }
    } else if (L.kind == DFB_LAYER_ATTENTION) {
      want_in = m.hq * m.head_dim * (m.attn_output_gate ? 2 : 1) + 2 * m.hkv * m.head_dim;
      want_mix = m.hq * m.head_dim;
      if (!L.q_norm_w || !L.k_norm_w || !L.kcache || !L.vcache) {
        set_error("engine: layer %d (attention) has a null pointer", i);
        return DFB_ERR_ARG;
      }
    } else {
      set_error("engine: layer %d has unknown kind %d", i, L.kind);
      return DFB_ERR_ARG;
    }
    if (L.in_proj.K != m.hidden || L.in_proj.N != want_in || L.out_proj.K != want_mix || L.out_proj.N != m.hidden ||
        L.gate_up.K != m.hidden || L.gate_up.N != 2 * m.intermediate || L.down.K != m.intermediate ||
        L.down.N != m.hidden) {
      set_error("engine: layer %d has a projection of the wrong shape", i);
      return DFB_ERR_ARG;
    }
    if (!L.input_norm_w || !L.post_norm_w) {
      set_error("engine: layer %d lacks a norm weight", i);
      return DFB_ERR_ARG;
    }
  }
  return DFB_OK;
}

}  // namespace
}  // namespace dfb

using namespace dfb;

extern "C" {

size_t dfb_engine_workspace_bytes(const dfb_model_desc* desc) {
  if (!desc || (desc->num_layers && !desc->layers_host)) return 0;
  return plan(*desc).total;
}

int dfb_engine_create(const dfb_model_desc* desc, void** engine_out) {
  if (!desc || !engine_out) {
    set_error("dfb_engine_create: null argument");
    return DFB_ERR_ARG;
  }
  if (int rc = validate(*desc)) return rc;
  const Workspace w = plan(*desc);
  if (desc->workspace_bytes < w.total) {
    set_error("engine: workspace of %zu bytes required, got %zu", w.total, desc->workspace_bytes);
    return DFB_ERR_ARG;
  }
  if (int rc = configure_kernels()) return rc;
  Engine* e = new (std::nothrow) Engine();
  if (!e) {
    set_error("engine: out of host memory");
    return DFB_ERR_ARG;
  }
  e->m = *desc;
  e->layers.assign(desc->layers_host, desc->layers_host + desc->num_layers);
  e->m.layers_host = e->layers.data();
  e->ws = w;
  e->plan_order();
  if (desc->tp_size > 1) {
    if (desc->tp_size > TP_MAX || desc->tp_rank < 0 || desc->tp_rank >= desc->tp_size) {
      set_error("engine: tensor-parallel rank %d of %d (at most %d ranks)", desc->tp_rank, desc->tp_size, TP_MAX);
      delete e;
      return DFB_ERR_ARG;
    }
    const unsigned one = 1;
    if (cudaMemcpy(e->at(w.epoch), &one, sizeof(one), cudaMemcpyHostToDevice) != cudaSuccess) {
      delete e;
      return check_launch("engine: epoch counter");
    }
    if (desc->tp_peer_slots)
      for (int r = 0; r < desc->tp_size; ++r) {
        e->peer_slots[r] = (unsigned long long*)desc->tp_peer_slots[r];
        if (!e->peer_slots[r] || ((uintptr_t)e->peer_slots[r] % 8) != 0) {
          set_error("engine: exchange buffer of rank %d is null or misaligned", r);
          delete e;
          return DFB_ERR_ARG;
        }
      }
    e->m.tp_peer_slots = nullptr;  // copied; the caller's array need not outlive creation
  }
  *engine_out = e;
  return DFB_OK;
}

int dfb_engine_destroy(void* engine) {
  Engine* e = (Engine*)engine;
  if (!e) return DFB_OK;
  if (e->exec) cudaGraphExecDestroy(e->exec);
  if (e->graph) cudaGraphDestroy(e->graph);
  delete e;
  return DFB_OK;
}

int dfb_engine_step(void* engine, void* stream) {
  if (!engine) {
    set_error("dfb_engine_step: null engine");
    return DFB_ERR_ARG;
  }
  return ((Engine*)engine)->step((cudaStream_t)stream);
}

size_t dfb_engine_tp_exchange_bytes(int batch, int hidden, int tp_size) {
  if (batch < 1 || hidden < 1 || tp_size < 2) return 0;
  return ((size_t)2 * tp_size * batch * hidden + (size_t)tp_size * batch * 2) * 8;
}

int dfb_engine_num_segments(void* engine) { return engine ? ((Engine*)engine)->num_segments() : 0; }

int dfb_engine_step_segment(void* engine, int segment, void* stream) {
  if (!engine) {
    set_error("dfb_engine_step_segment: null engine");
    return DFB_ERR_ARG;
  }
  return ((Engine*)engine)->step_segment(segment, (cudaStream_t)stream);
}

void* dfb_engine_partial_buffer(void* engine) {
  Engine* e = (Engine*)engine;
  return e && e->tp() ? (void*)e->at(e->ws.ar) : nullptr;
}

int dfb_engine_capture(void* engine, void* stream) {
  Engine* e = (Engine*)engine;
  if (!e) {
    set_error("dfb_engine_capture: null engine");
    return DFB_ERR_ARG;
  }
  if (e->exec) {
    cudaGraphExecDestroy(e->exec);
    e->exec = nullptr;
  }
  if (e->graph) {
    cudaGraphDestroy(e->graph);
    e->graph = nullptr;
  }
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t ce = cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal);
  if (ce != cudaSuccess) {
    set_error("engine: cannot begin stream capture: %s", cudaGetErrorString(ce));
    return DFB_ERR_CUDA;
  }
  const int rc = e->step(s);
  ce = cudaStreamEndCapture(s, &e->graph);
  if (rc) return rc;
  if (ce != cudaSuccess) {
    set_error("engine: stream capture failed: %s", cudaGetErrorString(ce));
    return DFB_ERR_CUDA;
  }
  ce = cudaGraphInstantiate(&e->exec, e->graph, 0);
  if (ce != cudaSuccess) {
    set_error("engine: graph instantiation failed: %s", cudaGetErrorString(ce));
    return DFB_ERR_CUDA;
  }
  return DFB_OK;
}

int dfb_engine_replay(void* engine, int steps, void* stream) {
  Engine* e = (Engine*)engine;
  if (!e || !e->exec) {
    set_error("dfb_engine_replay: no captured graph");
    return DFB_ERR_ARG;
  }
  for (int i = 0; i < steps; ++i) {
    const cudaError_t ce = cudaGraphLaunch(e->exec, (cudaStream_t)stream);
    if (ce != cudaSuccess) {
      set_error("engine: graph launch failed: %s", cudaGetErrorString(ce));
      return DFB_ERR_CUDA;
    }
  }
  return DFB_OK;
}

int dfb_engine_decode_host(void* engine, const int64_t* tokens_host, int steps, int64_t* out_host, void* stream) {
  Engine* e = (Engine*)engine;
  if (!e || !e->exec) {
    set_error("dfb_engine_decode_host: no captured graph");
    return DFB_ERR_ARG;
  }
  if (!tokens_host || !out_host) {
    set_error("dfb_engine_decode_host: null host buffer");
    return DFB_ERR_ARG;
  }
  cudaStream_t s = (cudaStream_t)stream;
  const size_t bytes = (size_t)e->m.batch * sizeof(int64_t);
  const int64_t* src = tokens_host;
  for (int i = 0; i < steps; ++i) {
    cudaError_t ce = cudaMemcpyAsync(e->m.tokens, src, bytes, cudaMemcpyHostToDevice, s);
    if (ce == cudaSuccess) ce = cudaGraphLaunch(e->exec, s);
    int64_t* dst = out_host + (size_t)i * e->m.batch;
    if (ce == cudaSuccess) ce = cudaMemcpyAsync(dst, e->m.tokens, bytes, cudaMemcpyDeviceToHost, s);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(s);
    if (ce != cudaSuccess) {
      set_error("engine: decode step %d failed: %s", i, cudaGetErrorString(ce));
      return DFB_ERR_CUDA;
    }
    src = dst;
  }
  return DFB_OK;
}

int dfb_engine_status(void* engine, int* status_host, void* stream) {
  Engine* e = (Engine*)engine;
  if (!e || !status_host) {
    set_error("dfb_engine_status: null argument");
    return DFB_ERR_ARG;
  }
  cudaError_t ce = cudaMemcpyAsync(status_host, e->at(e->ws.status), sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize((cudaStream_t)stream);
  if (ce != cudaSuccess) {
    set_error("engine: reading the status word failed: %s", cudaGetErrorString(ce));
    return DFB_ERR_CUDA;
  }
  return DFB_OK;
}

int dfb_engine_set_prefetch_distance(void* engine, int distance) {
  Engine* e = (Engine*)engine;
  if (!e || distance < 0 || distance > 8) {
    set_error("dfb_engine_set_prefetch_distance: null engine or distance outside 0..8");
    return DFB_ERR_ARG;
  }
  e->pf_dist = distance;
  return DFB_OK;
}

int dfb_engine_set_trace(void* engine, int64_t* buffer, int max_launches, int ctas_per_launch) {
  Engine* e = (Engine*)engine;
  if (!e || max_launches < 0 || ctas_per_launch < 0 || (buffer && (max_launches == 0 || ctas_per_launch == 0))) {
    set_error("dfb_engine_set_trace: null engine or bad sizes");
    return DFB_ERR_ARG;
  }
  e->trace.buf = (long long*)buffer;
  e->trace.ctas = ctas_per_launch;
  e->trace_launches = buffer ? max_launches : 0;
  return DFB_OK;
}

int dfb_engine_launches_per_step(void* engine) { return engine ? ((Engine*)engine)->launches : 0; }

}  // extern "C"
