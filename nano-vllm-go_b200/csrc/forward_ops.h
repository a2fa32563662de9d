// forward_ops.h — the launch glue shared by the forward passes (forward.cu, forward_layered.cu):
// profiling scopes, pending residual addends, and the GEMM / norm / mixture-of-experts launch
// helpers that pick the kernel for a shape and do the byte / flop accounting.
#pragma once
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <vector>

#include "common.cuh"
#include "handle.h"

namespace nvllm {

static cudaEvent_t prof_event(nvllm_handle* h) {
  if (!h->prof_pool.empty()) {
    cudaEvent_t e = h->prof_pool.back();
    h->prof_pool.pop_back();
    return e;
  }
  cudaEvent_t e = nullptr;
  cudaEventCreate(&e);
  return e;
}
// Two instruments behind nvllm_set_profile:
//  mode 1  CUDA events around every launch.  Serialises the chain (no programmatic-dependent-
//          launch overlap, no graph replay): per-launch times are an upper bound.  The only mode
//          that sees the NCCL calls of a tensor-parallel step.
//  mode 2  device timeline: every kernel records min(entry) / min(dependency released) /
//          max(exit) of its CTAs in %globaltimer ns (Trace::agg); launches stay back to back on
//          the stream with their PDL edges, exactly as in a real step.  A launch is charged the
//          time between its predecessor's last exit and its own last exit, so the classes add up
//          to the device time of the profiled window.
// `bytes` are ALGORITHMIC bytes only (weights, K/V, logits, one pass over each activation the
// reference's dataflow has); `impl` are the extra bytes of this implementation (split-K
// partials, staged activations).
struct ProfScope {
  nvllm_handle* h;
  int idx = -1;
  ProfScope(nvllm_handle* hh, int cls, double bytes, double flops, double impl = 0.0) : h(hh) {
    h->cur_cls = cls;
    if (!h->profile) return;
    nvllm_handle::ProfRec r{cls, bytes, flops, nullptr, nullptr, impl, 0, 0};
    if (h->profile == 2) {
      r.seq0 = trace_seq();
    } else {
      r.e0 = prof_event(h);
      r.e1 = prof_event(h);
      cudaEventRecord(r.e0, h->stream);
    }
    idx = (int)h->prof_open.size();
    h->prof_open.push_back(r);
  }
  ~ProfScope() {
    if (idx < 0) return;
    if (h->profile == 2) h->prof_open[idx].seq1 = trace_seq();
    else cudaEventRecord(h->prof_open[idx].e1, h->stream);
  }
};
// ------------------------------------------------------------------ kernel glue
struct Pending {  // a GEMM result still to be added to the residual stream
  const float* p = nullptr;
  int S = 0;
  size_t stride = 0;
  float m = 1.f;
  const float* bias = nullptr;
  bool bf16 = false;  // p is one bf16 slice (all-reduced over the tensor-parallel ranks)
  // mixture-of-experts: p holds the expert outputs by sorted row; the addend of token r is
  // sum_s comb_w[r, s] * p[comb_rows[r, s], :]  (fused into the consuming norm kernel)
  const int* comb_rows = nullptr;
  const float* comb_w = nullptr;
  int comb_k = 0;
};

// Folded RMSNorm, consumer side: the GEMM reads the un-normalised bf16 residual stream and scales
// accumulator row m by 1 / sqrt(sum_p ssq[p][m] / H + eps)
struct RowScale {
  const float* ssq = nullptr;
  int parts = 0;
};
// Folded RMSNorm, producer side: the GEMM's epilogue performs the residual update
// x += m * (acc + bias) and leaves bf16(x) + the row sums of squares for the next consumer
struct Resid {
  float m = 1.f;
  const float* bias = nullptr;
  int site = 0;  // 0 = attention output projection, 1 = FFN down projection (counter sets)
  const float* g = nullptr;  // weight of the norm that reads x next (folded into the bf16 copy)
};

struct RouterArgs {  // expert routing fused into the FFN norm of a MoE layer
  const float* R = nullptr;
  int E = 0, k = 0;
  int* topk_idx = nullptr;
  float* topk_w = nullptr;
  RouteOpts opts{};
};

#define LAUNCH(h, expr)                                                                       \
  do {                                                                                        \
    if (((h)->skip_mask >> (h)->cur_cls) & 1) break; /* NVLLM_SKIP timing ablation */         \
    cudaError_t _e = (expr);                                                                  \
    (h)->launches++;                                                                          \
    if (_e != cudaSuccess)                                                                    \
      return set_err(h, NVLLM_ERR_CUDA, "%s: %s (%s:%d)", #expr, cudaGetErrorString(_e),      \
                     __FILE__, __LINE__);                                                     \
  } while (0)

// C = A @ W^T into fp32 split-K partials at `out`
// epi != 0 asks for the FFN activation to be fused into the GEMM epilogue (bf16 hidden state
// written to epi_out); granted only on the tcgen05 path when the GEMM needs no split-K, in
// which case res->S comes back 0 (no partials to reduce).
static int run_gemm(nvllm_handle* h, const void* A, int lda, const void* W, int M, int N, int K,
                    float alpha, float* out, size_t cap, int ldo, Pending* res, int epi = 0,
                    void* epi_out = nullptr, int epi_ld = 0, const float* epi_bias = nullptr,
                    const void* pf_ptr = nullptr, size_t pf_bytes = 0, double alg_out = 0.0,
                    const RowScale* rs = nullptr, const Resid* rd = nullptr,
                    const GemvPre* gp = nullptr) {
  res->p = out;
  res->stride = (size_t)M * ldo;
  const double flops = 2.0 * M * N * K;
  // algorithmic: the weights once (+ the logits the LM head must produce, alg_out);
  // implementation: the staged activations and the fp32 split-K partials
  const double io = (double)N * K * dt_size(h->wdt) + alg_out;
  const double a_in = (double)M * K * dt_size(h->adt) - alg_out;
  if (M <= 8) {
    GemmArgs g{};
    g.A = A; g.adt = h->adt; g.lda = lda; g.W = W; g.wdt = h->wdt;
    g.M = M; g.N = N; g.K = K; g.out = out; g.ldo = ldo; g.split_stride = res->stride;
    g.alpha = alpha; g.out_capacity = cap;
    // a fused pre-stage reads what the activation kernel would have read
    double pre_alg = 0.0, pre_impl = 0.0;
    if (gp && gp->mode == 2) {
      pre_alg = (double)M * gp->hld * 4 - (double)M * K * dt_size(h->adt);
      pre_impl = (double)M * gp->hld * 4 * (gp->Sh - 1);
    }
    ProfScope ps(h, NVLLM_K_GEMV, io + pre_alg, flops, a_in + pre_impl + 4.0 * gemv_splits(M, N, K) * M * N);
    LAUNCH(h, launch_gemv(h->stream, g, gp));
    res->S = g.S;
    return NVLLM_OK;
  }
  if (h->wdt == DT_BF16 && h->use_tc5 && lda == K && tc5_supported(M, N, K)) {
    Tc5Args t{};
    t.A = A; t.W = W; t.M = M; t.N = N; t.K = K; t.out = out; t.ldo = ldo;
    t.split_stride = res->stride; t.alpha = alpha; t.out_capacity = cap;
    t.S = tc5_splits(M, N, K, h->sm_count);
    t.max_ctas = h->gemm_max_ctas;
    if (rs && rs->ssq) {
      t.rs_ssq = rs->ssq; t.rs_parts = rs->parts; t.rs_ld = h->ws.T_cap;
      t.rs_inv_h = 1.0f / (float)h->H; t.rs_eps = h->cfg.norm_eps;
    }
    if (rd) {
      // x += m (A W^T + bias) inside the GEMM; nothing is left pending for a norm kernel
      // split-K shapes (decode batches): the k-splits of a tile are one thread-block cluster and
      // meet in shared memory — no partials in global memory either way
      t.S = tc5_resid_splits(M, N, K, h->sm_count);
      t.epi = TC5_EPI_RESID;
      t.res_x = h->ws.x; t.res_xb = h->ws.xb; t.res_ssq = h->ws.ssq; t.res_ssq_ld = h->ws.T_cap;
      t.res_bias = rd->bias; t.res_m = rd->m; t.res_g = rd->g;
      ProfScope ps(h, NVLLM_K_GEMM_TC5, io + (double)M * N * 4 * 2, flops, a_in + (double)M * N * 2);
      LAUNCH(h, launch_gemm_tc5(h->stream, t, nullptr));
      *res = Pending();
      return NVLLM_OK;
    }
    if (M <= 128) {  // weight-streaming regime: warm L2 with the next big matrix
      t.pf_ptr = pf_ptr;
      t.pf_bytes = pf_bytes;
    }
    const long tiles = (long)ceil_div(N, 128) * ceil_div(M, tc5_box_rows_act(M));
    if (epi && (t.S == 1 || 2 * tiles >= h->sm_count)) {
      t.S = 1;
      t.epi = epi; t.epi_out = epi_out; t.epi_ld = epi_ld; t.epi_bias = epi_bias;
      t.glu_limit = h->glu_limit_cur;
      const double obytes = (double)M * epi_ld * 2;
      ProfScope ps(h, NVLLM_K_GEMM_TC5, io, flops, a_in + obytes);
      LAUNCH(h, launch_gemm_tc5(h->stream, t, nullptr));
      res->S = 0;
      return NVLLM_OK;
    }
    while (t.S > 1 && (size_t)t.S * M * ldo > cap) t.S--;
    ProfScope ps(h, NVLLM_K_GEMM_TC5, io, flops, a_in + 4.0 * t.S * M * N);
    LAUNCH(h, launch_gemm_tc5(h->stream, t, &res->S));
    return NVLLM_OK;
  }
  GemmArgs g{};
  g.A = A; g.adt = h->adt; g.lda = lda; g.W = W; g.wdt = h->wdt;
  g.M = M; g.N = N; g.K = K; g.out = out; g.ldo = ldo; g.split_stride = res->stride;
  g.alpha = alpha; g.out_capacity = cap;
  ProfScope ps(h, NVLLM_K_GEMM_SIMT, io, flops, a_in + 4.0 * M * N);
  LAUNCH(h, launch_gemm_simt(h->stream, g));
  res->S = g.S;
  return NVLLM_OK;
}

// can (M, N, K) with this activation stride take the tcgen05 path (and with it the folded-norm
// epilogues)?
static bool fold_gemm_ok(const nvllm_handle* h, int M, int N, int K, int lda) {
  return h->fold && M > 8 && h->wdt == DT_BF16 && h->use_tc5 && lda == K && tc5_supported(M, N, K);
}
static bool resid_gemm_ok(const nvllm_handle* h, int M, int N, int K, int lda) {
  if (!fold_gemm_ok(h, M, N, K, lda) || N != h->H) return false;
  const int S = tc5_resid_splits(M, N, K, h->sm_count);
  if (S <= 1) return S == 1 && tc5_splits(M, N, K, h->sm_count) == 1;
  // Split-K shapes (decode batches) can run the k-splits of an output tile as one thread-block
  // cluster that reduces through distributed shared memory and finishes the residual update
  // itself (gemm_tcgen05.cu) — no norm kernel behind the O and W2 GEMMs.  Parity-green, but
  // measured SLOWER on cfg2 decode (1150 -> 1195 us/step, DESIGN.md "rejected"): B200 places at
  // most 15 clusters of 8 such CTAs (16 tiles need a second wave) so the split drops to 6 = 96
  // CTAs streaming the weights instead of 128, and the in-cluster exchange + reduce costs more
  // than the norm launch it removes.  Opt-in: NVLLM_RESID_CLUSTER=1 (read per step).
  const char* ce = getenv("NVLLM_RESID_CLUSTER");
  return ce && atoi(ce) != 0;
}

static int run_norm(nvllm_handle* h, float* x, Pending* p1, Pending* p2, const float* w,
                    const float* b, void* y, float* y_f32, const int* row_idx, int n_rows,
                    const RouterArgs* route = nullptr, bool centered = false, const float* row_m2 = nullptr) {
  NormArgs a{};
  a.centered = centered ? 1 : 0;
  a.x = x;
  // algorithmic: x in, y out, and (when a GEMM result is pending) that result once + x back
  double bytes = (double)n_rows * h->H * (4 + dt_size(h->adt)), impl = 0.0;
  if (p1 && p1->p) {
    a.p1 = p1->p; a.S1 = p1->S; a.stride1 = p1->stride; a.m1 = p1->m; a.bias1 = p1->bias;
    a.p1_bf16 = p1->bf16 ? 1 : 0;
    a.comb_rows = p1->comb_rows; a.comb_w = p1->comb_w; a.comb_k = p1->comb_k;
    bytes += (double)n_rows * h->H * 4 * 2;
    impl += (double)n_rows * h->H * 4 * ((p1->comb_rows ? p1->comb_k : p1->S) - 1);
  }
  if (route && route->R) {
    a.router = route->R; a.E = route->E; a.topk = route->k;
    a.topk_idx = route->topk_idx; a.topk_w = route->topk_w; a.route = route->opts;
    bytes += (double)route->E * h->H * 4;
  }
  if (p2 && p2->p && p2->comb_rows)
    return set_err(h, NVLLM_ERR_INVALID, "MoE layers in a parallel block are not supported");
  if (p2 && p2->p) {
    a.p2 = p2->p; a.S2 = p2->S; a.stride2 = p2->stride; a.m2 = p2->m; a.bias2 = p2->bias;
    a.row_m2 = row_m2;
    bytes += (double)n_rows * h->H * 4;
    impl += (double)n_rows * h->H * 4 * (p2->S - 1);
  }
  a.w = w; a.b = b; a.eps = h->cfg.norm_eps; a.y = y; a.ydt = h->adt; a.y_f32 = y_f32;
  a.row_idx = row_idx; a.n_rows = n_rows; a.H = h->H;
  a.row_bias = row_idx ? h->view_r0 : 0;  // row_idx holds rows of the whole step
  a.groups = h->norm_groups;  // > 1: RMS norm in equal parts of the row (layered pre-norm models)
  ProfScope ps(h, NVLLM_K_NORM, bytes, 0, impl);
  LAUNCH(h, launch_norm(h->stream, a));
  if (p1) *p1 = Pending();
  if (p2) *p2 = Pending();
  return NVLLM_OK;
}

// Mixture-of-experts feed-forward of T routed tokens (the routing itself ran inside the norm
// kernel that produced xn): group the (token, slot) pairs by expert, two grouped GEMMs with the
// gated unit between them.  E experts of inner size I, k per token; glu_limit > 0 selects the
// clamped gated unit; topk_w holds this layer's routing weights.  Leaves the expert outputs
// pending in *pf (combined by the next norm).  act = 2: experts W_down relu(W_up x)^2 — moe_in
// stacks [I, H] matrices instead of interleaved [2 I, H] ones.
static int run_moe_ffn(nvllm_handle* h, int T, const void* xn, int E, int k, int I, float glu_limit,
                       const void* moe_in, const void* moe_out, const float* topk_w,
                       Pending* pf, int act = 1) {
  const int H = h->H;
  const int P = T * k;
  Workspace& w = h->ws;
  cudaStream_t st = h->stream;
  const double asz = dt_size(h->adt);
  // bf16 mode: grouped tcgen05 GEMMs over the expert-sorted rows; fp32 parity mode (and
  // shapes TMA cannot address): the SIMT fp32 tiles
  const int N1 = act == 2 ? I : 2 * I;  // columns of the experts' first projection
  const bool tc = h->adt == DT_BF16 && h->wdt == DT_BF16 && tc5_supported(P, N1, H) &&
                  tc5_supported(P, H, I) && (I % 8) == 0;
  const int tile = tc ? tc5_group_tile((P + E - 1) / E) : 64;
  // the routing itself (softmax, top-k) ran inside the FFN norm kernel above
  const bool sg = tc && moe_sort_gather_fits(T, k, E, H);
  {
    ProfScope ps(h, NVLLM_K_MOE_ROUTE, (double)P * 4 * 4 + (sg ? (double)P * H * 2 * 2 : 0.0), 0);
    if (sg)
      LAUNCH(h, launch_moe_sort_gather(st, w.topk_idx, T, k, E, w.sort, w.max_tiles, tile, H,
                                       xn, w.moe_xs));
    else
      LAUNCH(h, launch_moe_sort(st, w.topk_idx, T, k, E, w.sort, w.max_tiles, tile));
  }
  const double wsz = dt_size(h->wdt);
  const int e_touched = std::min(E, P);
  if (tc) {
    if (!sg) {
      ProfScope ps(h, NVLLM_K_MOE_MISC, (double)P * H * 2 * 2, 0);
      LAUNCH(h, launch_moe_gather(st, P, H, xn, w.sort.a_rows, w.moe_xs));
    }
    Tc5Args t{};
    t.A = w.moe_xs; t.W = moe_in; t.M = P; t.N = N1; t.K = H;
    t.S = 1; t.alpha = 1.f; t.epi = act == 2 ? TC5_EPI_RELU2 : TC5_EPI_SWIGLU; t.glu_limit = glu_limit; t.epi_out = w.hbuf; t.epi_ld = I;
    t.g_experts = E; t.g_tile = tile; t.g_max_tiles = w.max_tiles;
    t.g_tile_expert = w.sort.tile_expert; t.g_tile_row0 = w.sort.tile_row0;
    t.g_tile_rows = w.sort.tile_rows; t.g_n_tiles = w.sort.n_tiles;
    {
      ProfScope ps(h, NVLLM_K_MOE_GEMM, (double)e_touched * N1 * H * wsz, 2.0 * P * N1 * H,
                   (double)P * H * asz + (double)P * I * asz);
      LAUNCH(h, launch_gemm_tc5(st, t, nullptr));
    }
    Tc5Args t2 = t;
    t2.A = w.hbuf; t2.W = moe_out; t2.N = H; t2.K = I;
    t2.epi = TC5_EPI_PARTIAL; t2.epi_out = nullptr; t2.out = w.moe_Y; t2.ldo = H;
    t2.split_stride = 0; t2.out_capacity = 0;
    {
      ProfScope ps(h, NVLLM_K_MOE_GEMM, (double)e_touched * H * I * wsz, 2.0 * P * H * I,
                   (double)P * I * asz + (double)P * H * 4);
      LAUNCH(h, launch_gemm_tc5(st, t2, nullptr));
    }
  } else {
    GemmArgs g{};
    g.A = xn; g.adt = h->adt; g.lda = H; g.W = moe_in; g.wdt = h->wdt;
    g.M = P; g.N = N1; g.K = H; g.out = w.ws_a; g.ldo = N1; g.alpha = 1.f;
    g.a_rows = w.sort.a_rows; g.tile_expert = w.sort.tile_expert; g.tile_row0 = w.sort.tile_row0;
    g.tile_rows = w.sort.tile_rows; g.n_tiles = w.sort.n_tiles;
    g.expert_stride = (size_t)N1 * H; g.max_tiles = w.max_tiles;
    {
      ProfScope ps(h, NVLLM_K_MOE_GEMM,
                   (double)e_touched * N1 * H * wsz + (double)P * H * asz + (double)P * N1 * 4,
                   2.0 * P * N1 * H);
      LAUNCH(h, launch_gemm_simt(st, g));
    }
    {
      ProfScope ps(h, NVLLM_K_MOE_MISC, (double)P * (N1 * 4 + I * asz), 0);
      if (act == 2) LAUNCH(h, launch_act(st, h->adt, P, I, w.ws_a, 1, 0, nullptr, 2, w.hbuf));
      else LAUNCH(h, launch_moe_glu(st, h->adt, P, I, w.ws_a, w.hbuf, glu_limit));
    }
    GemmArgs g2{};
    g2.A = w.hbuf; g2.adt = h->adt; g2.lda = I; g2.W = moe_out; g2.wdt = h->wdt;
    g2.M = P; g2.N = H; g2.K = I; g2.out = w.moe_Y; g2.ldo = H; g2.alpha = 1.f;
    g2.tile_expert = w.sort.tile_expert; g2.tile_row0 = w.sort.tile_row0;
    g2.tile_rows = w.sort.tile_rows; g2.n_tiles = w.sort.n_tiles;
    g2.expert_stride = (size_t)H * I; g2.max_tiles = w.max_tiles;
    {
      ProfScope ps(h, NVLLM_K_MOE_GEMM,
                   (double)e_touched * H * I * wsz + (double)P * I * asz + (double)P * H * 4,
                   2.0 * P * H * I);
      LAUNCH(h, launch_gemm_simt(st, g2));
    }
  }
  // the weighted combine (moe.go:116-118) happens inside the norm kernel that consumes pf
  pf->p = w.moe_Y; pf->S = 1; pf->stride = 0; pf->bias = nullptr;
  pf->comb_rows = w.sort.pair_row; pf->comb_w = topk_w; pf->comb_k = k;
  return NVLLM_OK;
}

}  // namespace nvllm
