// forward.cu — the forward pass of one engine step as a sequence of sm_100a kernels on one
// stream (what TransformerModel.ForwardWithCache does per sequence in the reference,
// purego/tensor/generic_model.go:276-480, here for a ragged batch of T new tokens):
// embedding -> per layer [norm -> fused QKV GEMM -> RoPE + paged KV append -> paged
// attention -> O GEMM -> norm -> FFN / MoE] -> final norm of the last token of each sequence
// -> LM head on those rows only -> on-device argmax / temperature sampling.
// Residual adds are folded into the following norm kernel; GEMMs emit fp32 split-K partials
// that the consumer kernel sums.
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <vector>

#include "common.cuh"
#include "forward_ops.h"
#include "handle.h"

namespace nvllm {


// ------------------------------------------------------------------ workspace
void free_workspace(nvllm_handle* h) {
  Workspace& w = h->ws;
  h->drop_graphs();  // the captured decode steps hold these pointers
  void* ptrs[] = {w.tp_buf, w.x, w.xn, w.xn_f32, w.ws_a, w.ws_b, w.ws_c, w.q, w.attn_out, w.hbuf, w.xn_last,
                  w.xb, w.ssq, w.chain_ctr, w.lat_cq, w.lat_gate, w.lat_o, w.dl_qkv, w.dl_bg, w.dl_o, w.m_xbc, w.m_dt, w.m_y, w.m_yn, w.logits_p, w.logits, w.attn_ws, w.out_tokens, w.amax, w.amax_ticket, w.topk_idx, w.topk_w,
                  w.sort.counts, w.sort.offsets, w.sort.cursor, w.sort.sorted_pair, w.sort.pair_row,
                  w.sort.a_rows, w.sort.tile_expert, w.sort.tile_row0, w.sort.tile_rows,
                  w.sort.n_tiles, w.moe_Y, w.moe_y, w.moe_xs, w.lr_qkw, w.lr_v, w.lr_o, w.att_gate, w.sh_gate, w.mx_in,
                  w.m2_xbc, w.m2_dtx, w.m2_decay, w.v_first, w.side_g, w.att_split, w.att_split_cnt};
  for (void* p : ptrs)
    if (p) cudaFree(p);
  for (auto& r : h->ropes) {
    if (r.cosT) cudaFree(r.cosT);
    if (r.sinT) cudaFree(r.sinT);
    r.cosT = r.sinT = nullptr;
  }
  int keep = w.n_cap_out;
  w = Workspace();
  w.n_cap_out = keep;
  h->ws_bytes = 0;
}

int ensure_workspace(nvllm_handle* h, int T, int n) {
  Workspace& w = h->ws;
  if (T <= w.T_cap && n <= w.n_cap) return NVLLM_OK;
  NV_CHECK(h, cudaStreamSynchronize(h->stream));
  int Tc = std::max(T, w.T_cap), nc = std::max(n, w.n_cap);
  free_workspace(h);
  w.T_cap = Tc;
  w.n_cap = nc;
  const size_t H = h->H, asz = dt_size(h->adt);
  const size_t rows = std::max(Tc, 512);  // room for split-K slices of skinny GEMMs
  uint64_t* acc = &h->ws_bytes;
  auto A = [&](void** p, size_t bytes) -> cudaError_t {
    *p = nullptr;
    if (!bytes) return cudaSuccess;
    bytes = (bytes + 255) / 256 * 256;
    cudaError_t e = cudaMalloc(p, bytes);
    if (e == cudaSuccess) *acc += bytes;
    return e;
  };
#define WS(ptr, bytes)                                                                    \
  {                                                                                       \
    cudaError_t _e = A((void**)&(ptr), (bytes));                                          \
    if (_e != cudaSuccess) {                                                              \
      free_workspace(h);                                                                  \
      return set_err(h, NVLLM_ERR_NOMEM, "workspace for %d tokens: %s", Tc,               \
                     cudaGetErrorString(_e));                                             \
    }                                                                                     \
  }
  WS(w.x, Tc * H * 4);
  WS(w.xn, Tc * H * asz);
  size_t a_cols = std::max(h->qkv_cols, h->moe ? 0 : h->w1_cols);
  if (h->n_mamba) a_cols = std::max(a_cols, (size_t)h->m_P);
  w.ws_a_floats = rows * a_cols;
  if (h->moe) w.ws_a_floats = std::max(w.ws_a_floats, (size_t)Tc * h->topk * 2 * h->F);
  w.ws_b_floats = rows * H;
  WS(w.ws_a, w.ws_a_floats * 4);
  WS(w.ws_b, w.ws_b_floats * 4);
  if (h->parallel) WS(w.ws_c, w.ws_b_floats * 4);
  WS(w.q, (size_t)Tc * h->q_cols * asz);
  WS(w.attn_out, (size_t)Tc * h->q_cols * asz);
  WS(w.hbuf, h->moe ? (size_t)Tc * h->topk * h->F * asz : (size_t)Tc * h->F * asz);
  WS(w.xn_last, nc * H * asz);
  WS(w.chain_ctr, 256);
  if (h->n_mamba) {
    WS(w.m_xbc, (size_t)Tc * h->m_conv * 4);
    WS(w.m_dt, (size_t)Tc * h->m_nh * 4);
    WS(w.m_y, (size_t)Tc * h->m_E * 4);
    WS(w.m_yn, (size_t)Tc * h->m_E * asz);
  }
  if (cudaMemsetAsync(w.chain_ctr, 0, 256, h->stream) != cudaSuccess)
    return set_err(h, NVLLM_ERR_CUDA, "memset(chain counters) failed");
  if (h->fold) {
    WS(w.xb, Tc * H * 2);
    WS(w.ssq, (size_t)ceil_div(h->H, 128) * Tc * 4);
  }
  if (h->layered) {
    size_t cq = 0, heads = 0, ol = 0;
    for (auto& y : h->ll) {
      cq = std::max(cq, (size_t)y.q_rank_p);
      heads = std::max(heads, (size_t)y.s.heads);
      ol = std::max(ol, (size_t)y.ovr_p);
    }
    WS(w.lat_cq, Tc * cq * asz);
    WS(w.lat_gate, Tc * heads * 4);
    WS(w.lat_o, Tc * ol * asz);
    size_t dch = 0, dhv = 0, dh = 0;
    for (auto& y : h->ll)
      if (y.s.mixer == NVLLM_MIXER_DELTA) {
        dch = std::max(dch, (size_t)y.conv_ch);
        dhv = std::max(dhv, (size_t)y.s.heads * y.s.vdim);
        dh = std::max(dh, (size_t)y.s.heads);
      }
    WS(w.dl_qkv, Tc * dch * 4);
    WS(w.dl_bg, Tc * 2 * dh * 4);
    WS(w.dl_o, Tc * dhv * 4);
    size_t lhd = 0, lhv = 0, agate = 0, m2ch = 0, m2in = 0, m2h = 0, vfirst = 0, split_g = 0, split_v = 0;
    bool tmix = false, shared = false;
    for (auto& y : h->ll) {
      const nvllm_layer_spec& s = y.s;
      if (s.mixer == NVLLM_MIXER_MAMBA2) {
        lhv = std::max(lhv, (size_t)s.heads * s.vdim);
        m2ch = std::max(m2ch, (size_t)y.conv_ch);
        m2in = std::max(m2in, (size_t)s.heads * s.vdim);
        m2h = std::max(m2h, (size_t)s.heads);
      } else if (s.mixer == NVLLM_MIXER_ATTENTION) {
        if (s.head_gate) agate = std::max(agate, (size_t)s.heads);
        if (s.v_mix) vfirst = std::max(vfirst, (size_t)s.kv_heads * s.vdim);
        split_g = std::max(split_g, (size_t)s.kv_heads);
        split_v = std::max(split_v, (size_t)s.vdim);
      } else if (s.mixer == NVLLM_MIXER_GLA) {
        lhd = std::max(lhd, (size_t)s.heads * s.dim);
        lhv = std::max(lhv, (size_t)s.heads * s.vdim);
      } else if (s.mixer == NVLLM_MIXER_ATTN_TMIX) {
        lhd = std::max(lhd, (size_t)s.heads2 * s.dim2);
        lhv = std::max(lhv, (size_t)s.heads2 * s.dim2);
        agate = std::max(agate, (size_t)s.heads * s.vdim);
        tmix = true;
      }
      shared = shared || s.shared_ff > 0;
    }
    WS(w.lr_qkw, Tc * 3 * lhd * 4);
    WS(w.lr_v, Tc * lhv * 4);
    WS(w.lr_o, Tc * lhv * 4);
    WS(w.att_gate, Tc * agate * 4);
    WS(w.m2_xbc, Tc * m2ch * 4);
    WS(w.m2_dtx, Tc * m2in * 4);
    WS(w.m2_decay, Tc * m2h * 4);
    WS(w.v_first, Tc * vfirst * 4);
    WS(w.side_g, Tc * (size_t)h->side_p * asz);
    if (split_g) {  // decode steps have one row per sequence: nc sequences at most
      const size_t pairs = (size_t)nc * split_g;
      WS(w.att_split, pairs * WINATTN_MAX_SPLIT * 16 * (split_v + 2) * 4);
      WS(w.att_split_cnt, pairs * 4);
      NV_CHECK(h, cudaMemsetAsync(w.att_split_cnt, 0, pairs * 4, h->stream));
      w.att_split_pairs = (int)pairs;
    }
    if (h->mixer_conv && !h->moe) WS(w.xn_f32, Tc * H * 4);
    if (tmix) WS(w.mx_in, (size_t)5 * Tc * H * asz);
    if (shared) WS(w.sh_gate, (size_t)Tc * 4);
    for (auto& r : h->ropes) {
      WS(r.cosT, (size_t)Tc * (r.dims / 2) * 4);
      WS(r.sinT, (size_t)Tc * (r.dims / 2) * 4);
    }
  }
  if (h->tp > 1) WS(w.tp_buf, Tc * H * 4);
  // tp > 1: this rank's LM-head slice is Vl wide and the gathered logits are [tp][n][Vl]
  const size_t lcols = h->tp > 1 ? (size_t)h->Vl : (size_t)h->ldl;
  w.logits_p_floats = (size_t)std::max(nc, 64) * lcols;
  WS(w.logits_p, w.logits_p_floats * 4);
  WS(w.logits, (size_t)nc * lcols * h->tp * 4);
  w.attn_ws_floats = (size_t)nc * h->nh * 32 * (h->hd + 2);
  WS(w.attn_ws, w.attn_ws_floats * 4);
  WS(w.out_tokens, (size_t)nc * 4);
  WS(w.amax, (size_t)nc * 8);
  WS(w.amax_ticket, (size_t)nc * 4);
  if (cudaMemsetAsync(w.amax, 0, (size_t)nc * 8, h->stream) != cudaSuccess ||
      cudaMemsetAsync(w.amax_ticket, 0, (size_t)nc * 4, h->stream) != cudaSuccess)
    return set_err(h, NVLLM_ERR_CUDA, "memset(argmax scratch) failed");
  if (h->moe) {
    const size_t P = (size_t)Tc * h->topk;
    w.max_tiles = (int)(P / 32 + h->E);  // token tiles are >= 32 rows
    WS(w.xn_f32, Tc * H * 4);
    WS(w.topk_idx, P * 4);
    // A routed layer's norm kernel combines the previous routed layer's experts (reading that
    // layer's weights, k_prev per row) while it writes its own (k per row): with k != k_prev the
    // rows of different CTAs would overlap in one buffer, so consecutive routed layers alternate.
    w.topk_pairs = P;
    WS(w.topk_w, 2 * P * 4);
    WS(w.sort.counts, h->E * 4);
    WS(w.sort.offsets, (h->E + 1) * 4);
    WS(w.sort.cursor, h->E * 4);
    WS(w.sort.sorted_pair, P * 4);
    WS(w.sort.pair_row, P * 4);
    WS(w.sort.a_rows, P * 4);
    WS(w.sort.tile_expert, w.max_tiles * 4);
    WS(w.sort.tile_row0, w.max_tiles * 4);
    WS(w.sort.tile_rows, w.max_tiles * 4);
    WS(w.sort.n_tiles, 4);
    WS(w.moe_Y, P * H * 4);
    if (h->adt == DT_BF16) WS(w.moe_xs, P * H * 2);
    WS(w.moe_y, Tc * H * 4);
  }
#undef WS
  return NVLLM_OK;
}

// ------------------------------------------------------------------ profiling
constexpr int PROF_AGG_CAP = 1 << 18;  // launches per profiled window (32 B each)
static int prof_agg_reset(nvllm_handle* h) {
  std::vector<unsigned long long> init((size_t)PROF_AGG_CAP * 4);
  for (size_t i = 0; i < init.size(); i += 4) {
    init[i] = init[i + 1] = ~0ull;
    init[i + 2] = init[i + 3] = 0ull;
  }
  NV_CHECK(h, cudaMemcpy(h->prof_agg, init.data(), init.size() * 8, cudaMemcpyHostToDevice));
  trace_agg_set(h->prof_agg, PROF_AGG_CAP);
  return NVLLM_OK;
}
int prof_collect(nvllm_handle* h) {
  if (h->prof_open.empty()) return NVLLM_OK;
  NV_CHECK(h, cudaStreamSynchronize(h->stream));
  if (h->profile == 2) {
    const int nseq = std::min(trace_seq(), PROF_AGG_CAP);
    std::vector<unsigned long long> agg((size_t)nseq * 4);
    if (nseq) NV_CHECK(h, cudaMemcpy(agg.data(), h->prof_agg, agg.size() * 8, cudaMemcpyDeviceToHost));
    unsigned long long prev_exit = 0;
    for (auto& r : h->prof_open) {
      unsigned long long first = ~0ull, exit = 0;
      for (int sq = r.seq0; sq < r.seq1 && sq < nseq; sq++) {
        const unsigned long long* a = &agg[(size_t)sq * 4];
        if (a[2] == 0) continue;  // the launch had no traced CTA
        first = std::min(first, a[1] != ~0ull ? a[1] : a[0]);
        exit = std::max(exit, a[2]);
      }
      h->prof[r.cls].bytes += r.bytes;
      h->prof[r.cls].impl_bytes += r.impl;
      h->prof[r.cls].flops += r.flops;
      h->prof[r.cls].launches += 1;
      if (exit == 0) continue;  // un-instrumented kernel: its time goes to the next record
      const unsigned long long start = prev_exit ? prev_exit : first;
      if (exit > start) h->prof[r.cls].ms += (double)(exit - start) * 1e-6;
      prev_exit = std::max(prev_exit, exit);
    }
    h->prof_open.clear();
    return prof_agg_reset(h);
  }
  for (auto& r : h->prof_open) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, r.e0, r.e1) == cudaSuccess) {
      h->prof[r.cls].ms += ms;
      h->prof[r.cls].bytes += r.bytes;
      h->prof[r.cls].impl_bytes += r.impl;
      h->prof[r.cls].flops += r.flops;
      h->prof[r.cls].launches += 1;
    }
    h->prof_pool.push_back(r.e0);
    h->prof_pool.push_back(r.e1);
  }
  h->prof_open.clear();
  return NVLLM_OK;
}

// Tensor parallel: the pending row-parallel GEMM results are this rank's partial sums.  Fold
// them (split-K slices, multipliers, rank-0 biases) into one [T, H] buffer, sum it over the
// ranks and hand it to the norm as a single finished addend.
static int tp_reduce_pending(nvllm_handle* h, Pending* p1, Pending* p2, int T) {
  if (h->tp <= 1) return NVLLM_OK;
  Pending* a = (p1 && p1->p) ? p1 : nullptr;
  Pending* b = (p2 && p2->p) ? p2 : nullptr;
  if (!a) { a = b; b = nullptr; }
  if (!a) return NVLLM_OK;
  Workspace& w = h->ws;
  // large (prefill) messages travel as bf16 in bf16 mode: half the bytes of the exposed
  // all-reduce; the sum over ranks of the per-rank addends is rounded once more, the residual
  // stream itself stays fp32.  NVLLM_TP_BF16=0 keeps fp32 on the wire.
  static const bool wire_bf16_ok = !(getenv("NVLLM_TP_BF16") && atoi(getenv("NVLLM_TP_BF16")) == 0);
  // the peer-memory kernel keeps one flag / epoch state per handle: the two chunks of a pipelined
  // prefill must not use it concurrently
  const bool p2p = h->pipe_role == 0 && tp_p2p_fits(h, (size_t)T * h->H);
  const bool wire_bf16 = !p2p && wire_bf16_ok && h->adt == DT_BF16 && ((size_t)T * h->H % 8) == 0;
  {
    const double n = (double)T * h->H * 4;
    ProfScope ps(h, NVLLM_K_COMM, (wire_bf16 ? 0.5 : 1.0) * n, 0, n * (a->S + (b ? b->S : 0) + 1));  // bytes on the wire per rank
    if (p2p) {
      // one kernel: partial sums + all-reduce over NVLink peer memory (tp.cu)
      LAUNCH(h, launch_tp_allreduce_p2p(h, T, h->H, a->p, a->S, a->stride, a->m, a->bias,
                                        b ? b->p : nullptr, b ? b->S : 0, b ? b->stride : 0,
                                        b ? b->m : 0.f, b ? b->bias : nullptr, w.tp_buf));
    } else {
      LAUNCH(h, launch_tp_partial(h->stream, T, h->H, a->p, a->S, a->stride, a->m, a->bias,
                                  b ? b->p : nullptr, b ? b->S : 0, b ? b->stride : 0,
                                  b ? b->m : 0.f, b ? b->bias : nullptr, w.tp_buf, wire_bf16));
      int rc = tp_all_reduce(h, w.tp_buf, (size_t)T * h->H, wire_bf16);
      if (rc) return rc;
      h->launches++;
    }
  }
  if (p1) *p1 = Pending();
  if (p2) *p2 = Pending();
  Pending& o = p1 ? *p1 : *p2;
  o.p = w.tp_buf; o.S = 1; o.stride = 0; o.m = 1.f; o.bias = nullptr;
  o.bf16 = wire_bf16;
  return NVLLM_OK;
}

// ------------------------------------------------------------------ forward pass
// Inputs are the device arrays of h->lay (already on the device).
int forward_step(nvllm_handle* h) {
  if (h->layered) return forward_step_layered(h);
  const StepLayout& L = h->lay;
  Workspace& w = h->ws;
  const bool is_prefill = L.prefill;
  const int T = L.T, n = L.n, H = h->H;
  // rows through the final norm and the LM head: each sequence's last one, then the rows whose
  // logits were asked for on top (nvllm_request_logits; single-GPU handles only)
  const int n_out = (h->tp == 1 && L.n_out > n) ? L.n_out : n;
  const int32_t* d = L.d;
  const int* d_tokens = d + L.tokens;
  const int* d_pos = d + L.positions;
  const int* d_slots = d + L.slots;
  const nvllm_config& c = h->cfg;
  cudaStream_t st = h->stream;
  const double asz = dt_size(h->adt), kvsz = dt_size(h->kvdt);
  int rc;

  {
    ProfScope ps(h, NVLLM_K_EMBED, (double)T * H * (4 + dt_size(h->wdt)), 0);
    LAUNCH(h, launch_embed(st, h->wdt, d_tokens, d_pos, h->wte, h->wpe, c.max_seq_len,
                           c.embedding_multiplier, w.x, T, H, h->fold ? w.xb : nullptr,
                           h->fold ? w.ssq : nullptr, h->fold ? h->layers[0].attn_norm_w : nullptr));
  }
  // Folded RMSNorm (h->fold): while `xb_parts` > 0, w.xb holds bf16(x) of the CURRENT residual
  // stream and w.ssq its row sums of squares in xb_parts column-tile slices — the next GEMM
  // that would read a normed activation reads w.xb instead and the norm kernel is not launched.
  // read per step (not cached): the parity tests switch it between runs
  const char* chain_env = getenv("NVLLM_CHAIN");
  const bool chain_on = !(chain_env && atoi(chain_env) == 0);
  // Steps of <= 8 rows (GEMV shapes): the FFN activation is built inside the W2 GEMV — one
  // launch per layer less on a chain of ~100 dependent launches.  NVLLM_GEMV_PRE=0 keeps the
  // stand-alone activation kernel (read per step: the parity tests switch it).
  const char* gpre_env = getenv("NVLLM_GEMV_PRE");
  const bool gpre_act = !(gpre_env && atoi(gpre_env) == 0) && T <= 8 && !h->moe;
  int xb_parts = h->fold ? 1 : 0;
  const int h_tiles = ceil_div(H, 128);
  // generic_model.go:359-365: res + rm * x when ResidualMultiplier != 0, else plain add
  const float m_res = (c.residual_multiplier != 0.f) ? c.residual_multiplier : 1.f;
  // generic_model.go:405-416 (parallel block): both multipliers or neither
  const bool par_scaled = c.attention_multiplier != 0.f && c.residual_multiplier != 0.f;
  Pending p1, p2;
  const size_t kv_layer_bytes = h->kv_layer_elems * dt_size(h->kvdt);

  AttnArgs at{};
  // the attention kernels index rows of the WHOLE step (cu_q + q0): a chunk's view of the
  // workspace starts view_r0 rows in
  at.q = (char*)w.q - (size_t)h->view_r0 * h->q_cols * dt_size(h->adt);
  at.out = (char*)w.attn_out - (size_t)h->view_r0 * h->q_cols * dt_size(h->adt);
  at.qdt = h->adt; at.kvdt = h->kvdt;
  at.n_seqs = n; at.nh = h->nh; at.nkv = h->nkv; at.hd = h->hd; at.scale = h->attn_scale;
  at.block_tables = d + L.block_tables; at.max_blocks = L.max_blocks;
  at.cu_q = d + L.cu_q; at.seq_start = d + L.seq_start;
  at.tile_seq = d + L.tile_seq; at.tile_q0 = d + L.tile_q0; at.n_qtiles = L.n_qtiles;
  at.seq_len = d + L.seq_len;
  at.ws = w.attn_ws;
  at.pool_blocks = h->num_blocks;
  at.total_rows = h->view_T > 0 ? h->view_T : T;
  at.sm_count = h->sm_count;
  if (!is_prefill)
    at.n_splits = attn_decode_splits(h->adt, h->kvdt, n, h->nh, h->nkv, h->hd, L.max_len, h->sm_count);
  const double qo_bytes = 2.0 * T * h->q_cols * asz;
  const double attn_flops = 4.0 * h->nh * h->hd * L.attn_pairs;
  // algorithmic: every K/V row of the contexts once (+ the new rows appended by a fused decode
  // prologue); implementation: Q / O staging (and the QKV partials a fused prologue sums)
  const double attn_bytes = 2.0 * L.sum_len * h->nkv * h->hd * kvsz;

  for (int l = 0; l < h->L; l++) {
    const LayerW& lw = h->layers[l];
    if (!h->is_mamba.empty() && h->is_mamba[l]) {
      // ---- Mamba2 sub-block (generic_model.go:162-181, mamba2.go:72-207): norm -> in_proj GEMM
      // -> conv + SiLU + softplus -> selective scan -> gate + RMS norm -> out_proj GEMM, whose
      // result is added to the residual stream by the next norm like an attention output
      if ((rc = run_norm(h, w.x, &p1, &p2, lw.attn_norm_w, lw.attn_norm_b, w.xn, nullptr, nullptr, T)))
        return rc;
      Pending pr;
      if ((rc = run_gemm(h, w.xn, H, lw.m_in_proj, T, h->m_P, H, 1.f, w.ws_a, w.ws_a_floats, h->m_P, &pr)))
        return rc;
      MambaArgs ma{};
      ma.T = T; ma.n_seqs = n;
      ma.nh = h->m_nh; ma.hd = h->m_hd; ma.N = h->m_N; ma.G = h->m_G; ma.K = h->m_K; ma.E = h->m_E;
      ma.conv = h->m_conv; ma.P = h->m_P;
      ma.proj = pr.p; ma.S = pr.S; ma.stride = pr.stride;
      ma.conv_w = lw.m_conv_w; ma.conv_b = lw.m_conv_b; ma.dt_bias = lw.m_dt_bias; ma.a_log = lw.m_a_log;
      ma.d_skip = lw.m_d; ma.norm_w = lw.m_norm;
      ma.xbc = w.m_xbc; ma.dt = w.m_dt; ma.y = w.m_y;
      ma.cu_q = d + L.cu_q; ma.positions = d_pos; ma.block_tables = d + L.block_tables;
      ma.max_blocks = L.max_blocks;
      ma.ssm_pool = h->ssm_pool; ma.n_mamba = h->n_mamba; ma.layer = h->mamba_idx[l];
      {
        const double state_bytes = 2.0 * n * h->m_nh * h->m_hd * h->m_N * 4;  // SSM state in + out
        ProfScope ps(h, NVLLM_K_MISC, (double)T * (h->m_P * 4.0 + h->m_E * asz) + state_bytes, 0,
                     (double)T * (h->m_conv + h->m_nh + 2.0 * h->m_E) * 4 + (double)T * h->m_P * 4 * (pr.S - 1));
        LAUNCH(h, launch_mamba_conv(st, ma));
        LAUNCH(h, launch_mamba_scan(st, ma));
        LAUNCH(h, launch_mamba_gate_norm(st, ma, h->adt, w.m_yn));
      }
      if ((rc = run_gemm(h, w.m_yn, h->m_E, lw.m_out_proj, T, H, h->m_E, 1.f, w.ws_b, w.ws_b_floats, H, &p1)))
        return rc;
      p1.bias = nullptr;
      p1.m = m_res;
    } else {
    // ---- attention sub-block
    if ((rc = tp_reduce_pending(h, &p1, &p2, T))) return rc;
    Pending qkv;
    if (xb_parts > 0 && fold_gemm_ok(h, T, h->qkv_cols, H, H)) {
      RowScale rsc{w.ssq, xb_parts};
      if ((rc = run_gemm(h, w.xb, H, lw.wqkv, T, h->qkv_cols, H, 1.f, w.ws_a, w.ws_a_floats,
                         h->qkv_cols, &qkv, 0, nullptr, 0, nullptr, nullptr, 0, 0.0, &rsc)))
        return rc;
    } else {
      if ((rc = run_norm(h, w.x, &p1, &p2, lw.attn_norm_w, lw.attn_norm_b, w.xn,
                         nullptr, nullptr, T)))
        return rc;
      if ((rc = run_gemm(h, w.xn, H, lw.wqkv, T, h->qkv_cols, H, 1.f, w.ws_a, w.ws_a_floats,
                         h->qkv_cols, &qkv)))
        return rc;
    }
    xb_parts = 0;
    void* kp = (char*)h->kpool + (size_t)l * kv_layer_bytes;
    void* vp = (char*)h->vpool + (size_t)l * kv_layer_bytes;
    const bool fuse_rope = !is_prefill && attn_decode_fuses_rope(h->adt, h->kvdt, h->hd);
    if (fuse_rope) {
      at.qkv_p = qkv.p; at.qkv_S = qkv.S; at.qkv_stride = qkv.stride; at.qkv_ld = h->qkv_cols;
      at.qkv_bias = lw.bqkv;
      at.cosT = h->use_rope ? h->cosT : nullptr;
      at.sinT = h->use_rope ? h->sinT : nullptr;
    } else {
      ProfScope ps(h, NVLLM_K_ROPE_KV,
                   (double)T * h->qkv_cols * 4 + (double)T * h->q_cols * asz +
                       2.0 * T * h->kv_cols * kvsz, 0, (double)T * h->qkv_cols * 4 * (qkv.S - 1));
      LAUNCH(h, launch_rope_kv(st, h->adt, h->kvdt, T, h->nh, h->nkv, h->hd, qkv.p, qkv.S,
                               qkv.stride, lw.bqkv, d_pos, d_slots,
                               h->use_rope ? h->cosT : nullptr, h->use_rope ? h->sinT : nullptr, w.q,
                               kp, vp));
      if (h->pipe_role == 1) NV_CHECK(h, cudaEventRecord(h->pipe_kv[l], st));
    }
    at.kpool = kp;
    at.vpool = vp;
    if (is_prefill) {
      // second chunk: its queries attend the first chunk's keys of this layer
      if (h->pipe_role == 2) NV_CHECK(h, cudaStreamWaitEvent(st, h->pipe_kv[l], 0));
      ProfScope ps(h, NVLLM_K_ATTN_PREFILL, attn_bytes, attn_flops, qo_bytes);
      LAUNCH(h, launch_attn_prefill(st, at));
    } else {
      ProfScope ps(h, NVLLM_K_ATTN_DECODE,
                   attn_bytes + (fuse_rope ? 2.0 * T * h->kv_cols * kvsz : 0.0), attn_flops,
                   fuse_rope ? (double)T * h->qkv_cols * 4 * qkv.S + (double)T * h->q_cols * asz
                             : qo_bytes);
      LAUNCH(h, launch_attn_decode(st, at));
      if (at.n_splits > 1) h->launches++;
    }
    if (resid_gemm_ok(h, T, H, h->q_cols, h->q_cols)) {
      Resid rd{m_res, lw.bo, 0, lw.ffn_norm_w};
      if ((rc = run_gemm(h, w.attn_out, h->q_cols, lw.wo, T, H, h->q_cols, 1.f, w.ws_b,
                         w.ws_b_floats, H, &p1, 0, nullptr, 0, nullptr, nullptr, 0, 0.0, nullptr, &rd)))
        return rc;
      xb_parts = h_tiles;
    } else {
      if ((rc = run_gemm(h, w.attn_out, h->q_cols, lw.wo, T, H, h->q_cols, 1.f, w.ws_b,
                         w.ws_b_floats, H, &p1)))
        return rc;
      p1.bias = lw.bo;
      p1.m = h->parallel ? (par_scaled ? c.attention_multiplier : 1.f) : m_res;
    }
    }  // attention / Mamba2 sub-block
    // ---- feed-forward sub-block
    float* ffn_out = w.ws_b;
    if (h->parallel) {
      ffn_out = w.ws_c;  // FFN reads the same normed input (generic_model.go:395-418)
    } else {
      if ((rc = tp_reduce_pending(h, &p1, nullptr, T))) return rc;
      RouterArgs ra;
      if (h->moe) {
        ra.R = lw.router; ra.E = h->E; ra.k = h->topk;
        ra.topk_idx = w.topk_idx; ra.topk_w = w.topk_w;
      }
      const bool skip_norm = xb_parts > 0 && !h->moe && fold_gemm_ok(h, T, h->w1_cols, H, H);
      if (!skip_norm) {
        if ((rc = run_norm(h, w.x, &p1, nullptr, lw.ffn_norm_w, lw.ffn_norm_b,
                           w.xn, nullptr, nullptr, T, &ra)))
          return rc;
        xb_parts = 0;
      }
    }
    Pending& pf = h->parallel ? p2 : p1;
    if (h->moe) {
      if ((rc = run_moe_ffn(h, T, w.xn, h->E, h->topk, h->F, 0.f, lw.moe_in, lw.moe_out, w.topk_w, &pf))) return rc;
    } else {
      // decode-sized steps: W1 (+ fused activation) and W2 in ONE launch — W2's weight stream
      // starts under W1's epilogues and the launch / drain / release gap between the two
      // GEMMs is gone (gemm_tcgen05.cu, Tc5Chain).  NVLLM_CHAIN=0 keeps two launches.
      const long w1_tiles = ceil_div(h->w1_cols, 128);
      if (chain_on && T > 8 && T <= 128 && xb_parts == 0 && h->wdt == DT_BF16 && h->use_tc5 &&
          tc5_supported(T, h->w1_cols, H) && tc5_supported(T, H, h->F) &&
          (tc5_splits(T, h->w1_cols, H, h->sm_count) == 1 || 2 * w1_tiles >= h->sm_count)) {
        Tc5Args t1{};
        t1.A = w.xn; t1.W = lw.w1; t1.M = T; t1.N = h->w1_cols; t1.K = H; t1.S = 1; t1.alpha = 1.f;
        t1.epi = h->swiglu ? TC5_EPI_SWIGLU : TC5_EPI_GELU; t1.epi_out = w.hbuf; t1.epi_ld = h->F;
        t1.epi_bias = lw.b1;
        Tc5Args t2{};
        t2.A = w.hbuf; t2.W = lw.w2; t2.M = T; t2.N = H; t2.K = h->F; t2.alpha = 1.f;
        t2.out = ffn_out; t2.ldo = H; t2.split_stride = (size_t)T * H; t2.out_capacity = w.ws_b_floats;
        t2.S = tc5_splits(T, H, h->F, h->sm_count);
        while (t2.S > 1 && (size_t)t2.S * T * H > w.ws_b_floats) t2.S--;
        int S2 = 1;
        {
          const double wsz = dt_size(h->wdt);
          ProfScope ps(h, NVLLM_K_GEMM_TC5, ((double)h->w1_cols * H + (double)H * h->F) * wsz,
                       2.0 * T * ((double)h->w1_cols * H + (double)H * h->F),
                       (double)T * H * asz + 2.0 * T * h->F * asz + 4.0 * t2.S * T * H);
          LAUNCH(h, launch_gemm_tc5_chain(st, t1, t2, w.chain_ctr, &S2));
        }
        pf.p = ffn_out; pf.S = S2; pf.stride = (size_t)T * H; pf.bias = lw.b2;
        pf.m = h->parallel ? (par_scaled ? c.residual_multiplier : 1.f) : m_res;
        continue;
      }
      Pending h1;
      RowScale rsc{xb_parts > 0 ? w.ssq : nullptr, xb_parts};
      if ((rc = run_gemm(h, xb_parts > 0 ? w.xb : w.xn, H, lw.w1, T, h->w1_cols, H, 1.f, w.ws_a,
                         w.ws_a_floats, h->w1_cols, &h1, h->swiglu ? TC5_EPI_SWIGLU : TC5_EPI_GELU,
                         w.hbuf, h->F, lw.b1, nullptr, 0, 0.0, &rsc)))
        return rc;
      xb_parts = 0;
      if (h1.S > 0 && gpre_act) {
        GemvPre ga{};
        ga.mode = 2; ga.hp = h1.p; ga.Sh = h1.S; ga.hstride = h1.stride; ga.hld = h->w1_cols;
        ga.hbias = lw.b1; ga.swiglu = h->swiglu ? 1 : 0;
        if ((rc = run_gemm(h, w.hbuf, h->F, lw.w2, T, H, h->F, 1.f, ffn_out, w.ws_b_floats, H, &pf, 0,
                           nullptr, 0, nullptr, nullptr, 0, 0.0, nullptr, nullptr, &ga)))
          return rc;
        pf.bias = lw.b2;
        pf.m = h->parallel ? (par_scaled ? c.residual_multiplier : 1.f) : m_res;
        continue;
      }
      if (h1.S > 0) {
        ProfScope ps(h, NVLLM_K_ACT, (double)T * h->w1_cols * 4 + (double)T * h->F * asz, 0,
                     (double)T * h->w1_cols * 4 * (h1.S - 1));
        LAUNCH(h, launch_act(st, h->adt, T, h->F, h1.p, h1.S, h1.stride, lw.b1, h->swiglu ? 1 : 0,
                             w.hbuf));
      }
      if (!h->parallel && resid_gemm_ok(h, T, H, h->F, h->F)) {
        // the next reader of x is layer l + 1's attention norm (the final norm reads fp32 x)
        Resid rd{m_res, lw.b2, 1, l + 1 < h->L ? h->layers[l + 1].attn_norm_w : nullptr};
        if ((rc = run_gemm(h, w.hbuf, h->F, lw.w2, T, H, h->F, 1.f, ffn_out, w.ws_b_floats, H, &pf, 0,
                           nullptr, 0, nullptr, nullptr, 0, 0.0, nullptr, &rd)))
          return rc;
        xb_parts = h_tiles;
      } else {
        if ((rc = run_gemm(h, w.hbuf, h->F, lw.w2, T, H, h->F, 1.f, ffn_out, w.ws_b_floats, H, &pf)))
          return rc;
        pf.bias = lw.b2;
      }
    }
    if (pf.p) pf.m = h->parallel ? (par_scaled ? c.residual_multiplier : 1.f) : m_res;
  }
  if (h->skip_head) return NVLLM_OK;  // no sequence ends in this chunk: its last residual update is never read
  // final norm on the last token of each sequence only (the reference norms and projects all
  // T rows, generic_model.go:464-470, then keeps row T-1, :595-604)
  if ((rc = tp_reduce_pending(h, &p1, &p2, T))) return rc;
  if ((rc = run_norm(h, w.x, &p1, &p2, h->lnf_w, h->lnf_b, w.xn_last, nullptr, d + L.last_row, n_out)))
    return rc;
  const float alpha = (c.logits_scaling != 0.f) ? 1.0f / c.logits_scaling : 1.f;
  Pending lg;
  const float* logits = nullptr;
  int vsplit = 0;
  if (h->tp > 1) {
    // vocabulary-parallel LM head: this rank's Vl_valid rows -> slot `rank` of [tp][n][Vl],
    // then one all-gather; every rank samples the same token from the same gathered logits
    const int Vl = h->Vl;
    float* slot = w.logits + (size_t)h->rank * n * Vl;
    if (h->Vl_valid > 0) {
      if ((rc = run_gemm(h, w.xn_last, H, h->lm_head, n, h->Vl_valid, H, alpha, w.logits_p,
                         w.logits_p_floats, Vl, &lg)))
        return rc;
      ProfScope ps(h, NVLLM_K_MISC, (double)n * Vl * 4 * (lg.S + 1), 0);
      LAUNCH(h, launch_reduce_partials(st, lg.p, lg.S, lg.stride, (size_t)n * Vl, slot));
    }
    {
      ProfScope ps(h, NVLLM_K_COMM, (double)n * Vl * 4 * h->tp, 0);
      if ((rc = tp_all_gather_f32(h, w.logits, (size_t)n * Vl))) return rc;
      h->launches++;
    }
    logits = w.logits;
    vsplit = Vl;
  } else {
    if ((rc = run_gemm(h, w.xn_last, H, h->lm_head, n_out, h->V, H, alpha, w.logits_p,
                       w.logits_p_floats, h->ldl, &lg, 0, nullptr, 0, nullptr, nullptr, 0,
                       (double)n_out * h->V * 4)))
      return rc;
    logits = lg.p;
    if (lg.S > 1) {
      ProfScope ps(h, NVLLM_K_MISC, 0, 0, (double)n_out * h->ldl * 4 * (lg.S + 1));
      LAUNCH(h, launch_reduce_partials(st, lg.p, lg.S, lg.stride, (size_t)n_out * h->ldl, w.logits));
      logits = w.logits;
    }
  }
  const float* d_temp = reinterpret_cast<const float*>(d + L.temperature);
  const float* d_uni = reinterpret_cast<const float*>(d + L.uniforms);
  {
    ProfScope ps(h, NVLLM_K_SAMPLE, (double)n * h->V * 4, 0);
    LAUNCH(h, launch_sample(st, logits, h->ldl, h->V, n, d_temp, d_uni, w.out_tokens, w.amax,
                            w.amax_ticket, vsplit));
    if (h->filters_active() && h->hist_n == n) {
      // TensorModelRunner's sampler (tensor_model_runner.go:92-94): the rows with
      // temperature > 0 are redrawn with the repetition penalty / top-k / top-p applied
      LAUNCH(h, launch_sample_filtered(st, logits, h->ldl, h->V, n, vsplit, d_temp, d_uni,
                                       h->d_hist + (n + 1), h->d_hist, h->top_p, h->top_k,
                                       h->rep_penalty, h->d_probs, w.out_tokens));
    }
  }
  h->ws.logits_final = logits;
  return NVLLM_OK;
}

// Tensor-parallel prefill of ONE long sequence as two token chunks in flight at once: chunk A
// (rows [0, r0)) on the handle's stream and communicator, chunk B (rows [r0, T)) on stream2 with
// the duplicate communicator.  Each chunk is a complete forward pass over its rows — causal
// attention only needs the earlier chunk's K / V of the same layer, handed over by one event
// per layer — so B's GEMMs run while A's per-layer all-reduce is on the wire and vice versa
// (SURVEY.md 8e / hard part 3: "token-chunk pipelining").  The persistent GEMM grids leave 16
// SMs to the collective kernels.  Only B holds the sequence's last token: A skips the head.
// Opt-in: NVLLM_TP_PIPE=1 (read at tp_init; measured slower at tp 2, see tp.cu), threshold
// NVLLM_TP_PIPE_MIN_T.
int forward_step_auto(nvllm_handle* h) {
  const StepLayout L = h->lay;
  static const int min_T = getenv("NVLLM_TP_PIPE_MIN_T") ? atoi(getenv("NVLLM_TP_PIPE_MIN_T")) : 1024;
  const int qtile = attn_prefill_qtile(h->adt, h->kvdt, h->hd);
  const int ts = L.n_qtiles / 2, r0 = ts * qtile;
  if (!(h->tp > 1 && h->nccl2 && L.prefill && L.n == 1 && !h->profile && !h->moe && L.T >= min_T &&
        ts >= 1 && r0 < L.T && (r0 % 8) == 0))
    return forward_step(h);
  const Workspace W0 = h->ws;
  cudaStream_t s0 = h->stream;
  static bool said = false;
  if (!said && getenv("NVLLM_TP_DEBUG")) {
    said = true;
    fprintf(stderr, "[nvllm] rank %d/%d: two-chunk prefill pipeline, rows [0, %d) + [%d, %d)\n", h->rank,
            h->tp, r0, r0, L.T);
  }
  NV_CHECK(h, cudaEventRecord(h->pipe_fork, s0));
  NV_CHECK(h, cudaStreamWaitEvent(h->stream2, h->pipe_fork, 0));
  const size_t asz = dt_size(h->adt);
  int rc = NVLLM_OK;
  for (int role = 1; role <= 2 && rc == NVLLM_OK; role++) {
    const int rb = role == 1 ? 0 : r0, Tc = role == 1 ? r0 : L.T - r0;
    Workspace v = W0;
    v.x = W0.x + (size_t)rb * h->H;
    v.xn = (char*)W0.xn + (size_t)rb * h->H * asz;
    v.q = (char*)W0.q + (size_t)rb * h->q_cols * asz;
    v.attn_out = (char*)W0.attn_out + (size_t)rb * h->q_cols * asz;
    v.hbuf = (char*)W0.hbuf + (size_t)rb * h->F * asz;
    if (W0.tp_buf) v.tp_buf = W0.tp_buf + (size_t)rb * h->H;
    // split-K partial buffers: one half each
    v.ws_a_floats = W0.ws_a_floats / 2;
    v.ws_b_floats = W0.ws_b_floats / 2;
    if (role == 2) {
      v.ws_a = W0.ws_a + v.ws_a_floats;
      v.ws_b = W0.ws_b + v.ws_b_floats;
      if (W0.ws_c) v.ws_c = W0.ws_c + v.ws_b_floats;
    }
    StepLayout Lv = L;
    Lv.T = Tc;
    Lv.tokens += rb;
    Lv.positions += rb;
    Lv.slots += rb;
    Lv.tile_seq += role == 1 ? 0 : ts;
    Lv.tile_q0 += role == 1 ? 0 : ts;
    Lv.n_qtiles = role == 1 ? ts : L.n_qtiles - ts;
    h->ws = v;
    h->lay = Lv;
    h->stream = role == 1 ? s0 : h->stream2;
    h->pipe_role = role;
    h->view_r0 = rb;
    h->view_T = L.T;
    h->skip_head = role == 1;
    h->gemm_max_ctas = std::max(1, h->sm_count - 16);
    rc = forward_step(h);
    const float* lf = h->ws.logits_final;
    h->ws = W0;
    h->ws.logits_final = lf;
  }
  h->lay = L;
  h->stream = s0;
  h->pipe_role = 0;
  h->view_r0 = 0;
  h->view_T = 0;
  h->skip_head = false;
  h->gemm_max_ctas = 0;
  if (rc) return rc;
  NV_CHECK(h, cudaEventRecord(h->pipe_join, h->stream2));
  NV_CHECK(h, cudaStreamWaitEvent(s0, h->pipe_join, 0));
  return NVLLM_OK;
}

}  // namespace nvllm

using namespace nvllm;

extern "C" int nvllm_set_profile(nvllm_handle* h, int enabled) {
  if (!h) return NVLLM_ERR_INVALID;
  NV_CHECK(h, cudaSetDevice(h->dev));
  if (enabled < 0 || enabled > 2) return set_err(h, NVLLM_ERR_INVALID, "profile mode %d", enabled);
  int rc = prof_collect(h);
  if (rc) return rc;
  memset(h->prof, 0, sizeof h->prof);
  if (h->profile == 2 && enabled != 2) trace_agg_set(nullptr, 0);
  if (enabled == 2) {
    if (!h->prof_agg) NV_CHECK(h, cudaMalloc((void**)&h->prof_agg, (size_t)PROF_AGG_CAP * 32));
    h->profile = 2;
    return prof_agg_reset(h);
  }
  h->profile = enabled;
  return NVLLM_OK;
}

extern "C" int nvllm_get_profile(nvllm_handle* h, nvllm_profile_entry* out) {
  if (!h || !out) return NVLLM_ERR_INVALID;
  NV_CHECK(h, cudaSetDevice(h->dev));
  int rc = prof_collect(h);
  if (rc) return rc;
  memcpy(out, h->prof, sizeof h->prof);
  return NVLLM_OK;
}
