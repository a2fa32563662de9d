// forward_layered.cu — models whose configuration lists their layers one by one
// (nvllm_create_layered): handle set-up, tensors by checkpoint name, the cache pools and the
// forward pass of one engine step.
//
// Two block styles on the fp32 residual stream x (nvllm_layered_config::block_style):
//   parallel, pre-norm:      h = LayerNorm(x) (weight only);  x += mixer(h) + feed_forward(h)
//   sequential, post-norm:   x += RMSNorm(mixer(x));  x += RMSNorm(feed_forward(x))  — the
//     sublayers read x itself (kept beside the fp32 stream in the activation dtype), the norm
//     kernel normalises the pending sublayer result and adds it (NormArgs::post).  Mixers of
//     this style: sliding-window attention (attention_window.cu) and the gated delta rule
//     (delta.cu); feed-forward W_down relu(W_up x)^2.  Positions enter once, as sinusoids
//     added to the scaled embedding; the head may be the embedding table itself.
//   sequential, pre-norm:    x += mixer(RMSNorm(x));  x += feed_forward(RMSNorm(x)); a run of layers
//     may repeat with the same weights, every pass with caches and state of its own and a learned
//     vector added to x at its start.  Mixers of this style: gated linear attention (linrec.cu) and
//     "attention + time mixing" — grouped-query attention whose q / k / v pass a short convolution
//     (attention_window.cu: whole-row norms, interpolated rotation, score cap, chunked mask, output
//     gate) beside time mixing with a token shift (linrec.cu), their outputs summed with two scales.
//     Feed-forward: a mixture of squared-ReLU experts chosen by sigmoid scores, the weight on the
//     expert's input, plus an always-on expert with a per-token gate.
// Mixer "latent attention" (attention_latent.cu): one fused input projection [W_dq | W_dkv | W_g]
// of h, RMS-normed latents, the query up projection with W_uk folded in, the absorbed-query
// attention over the paged latent cache (per-head sigmoid gate applied to its result), the output
// projection with W_uv folded in.  A layer with
// kv_from = j has no W_dkv and reads layer j's cache rows (written earlier in the same step).
// Feed-forward: none, a dense clamped gated unit, or a group-limited top-k mixture of such
// units (the routing runs inside the norm kernel, the expert GEMMs are the grouped ones the
// other MoE models use).  The two sublayer results stay pending as split-K partials and are
// added to x by the next layer's norm kernel, as everywhere in this library.
#include <math.h>

#include <string>

#include "forward_ops.h"

namespace nvllm {

static size_t up8(size_t a) { return (a + 7) / 8 * 8; }
static size_t wire_size(int api_dt) { return api_dt == NVLLM_DT_F32 ? 4 : 2; }

void layered_free(nvllm_handle* h) {
  auto F = [](void* p) {
    if (p) cudaFree(p);
  };
  for (auto& y : h->ll) {
    F(y.norm_w); F(y.w_in); F(y.dq_norm); F(y.dkv_norm); F(y.w_uq); F(y.w_uk); F(y.w_uv); F(y.w_o); F(y.w_q); F(y.w_ov);
    F(y.w1); F(y.w2); F(y.router); F(y.moe_in); F(y.moe_out);
    F(y.post1_w); F(y.post2_w); F(y.conv_w); F(y.a_log); F(y.dt_bias); F(y.onorm_w);
    F(y.bias_in); F(y.o_bias); F(y.qnorm_w); F(y.knorm_w); F(y.lr_w2); F(y.lr_b); F(y.mu); F(y.bonus);
    F(y.w_in2); F(y.w_o2); F(y.sh_gate);
    F(y.sink_w); F(y.head_temp); F(y.vmix); F(y.conv_b); F(y.d_skip); F(y.route_corr); F(y.canon_w);
    F(y.side_gate); F(y.side_proj); F(y.side_norm);
  }
  F(h->embed_norm_w);
  h->embed_norm_w = nullptr;
  F(h->side_embed);
  h->side_embed = nullptr;
  h->runs.clear();
  F(h->loop_step);
  h->loop_step = nullptr;
  h->ll.clear();
  for (void* p : h->lat_pools) F(p);
  h->lat_pools.clear();
  for (void* p : h->win_kpools) F(p);
  for (void* p : h->win_vpools) F(p);
  h->win_kpools.clear();
  h->win_vpools.clear();
  F(h->pos_freq);
  h->pos_freq = nullptr;
  F(h->state_pool);
  h->state_pool = nullptr;
  for (auto& r : h->ropes) {
    F(r.inv_freq); F(r.cosT); F(r.sinT);
  }
  h->ropes.clear();
}

// ------------------------------------------------------------------ tensors by name
namespace {
struct Dst {
  void* p = nullptr;     // destination base
  int ddt = DT_F32;      // destination dtype
  int64_t rows = 0, cols = 0;  // expected shape ([rows] when cols == 0)
  int ld = 0;            // destination row stride (elements)
  int row_mul = 1, row_add = 0;
  float add = 0.f;       // vectors: constant added to every element (norm weights stored around zero)
};
__global__ void add_const_kernel(float* p, size_t n, float c) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) p[i] += c;
}
}  // namespace

static bool parse_layer_name(const std::string& name, int* layer, std::string* rest) {
  if (name.size() < 3 || name[0] != 'l' || name[1] < '0' || name[1] > '9') return false;
  size_t i = 1;
  int v = 0;
  while (i < name.size() && name[i] >= '0' && name[i] <= '9') v = v * 10 + (name[i++] - '0');
  if (i >= name.size() || name[i] != '.') return false;
  *layer = v;
  *rest = name.substr(i + 1);
  return true;
}

int layered_set_weight(nvllm_handle* h, const char* cname, int dtype, const void* host,
                       const int64_t* shape, int ndim) {
  if (!h->layered) return set_err(h, NVLLM_ERR_STATE, "named weights belong to handles of nvllm_create_layered");
  if (h->finalized) return set_err(h, NVLLM_ERR_STATE, "set_named_weight after finalize");
  if (!cname || !host || (!shape && ndim > 0) || ndim < 0 || ndim > 2) return set_err(h, NVLLM_ERR_INVALID, "bad named weight");
  const int64_t one_el = 1;
  if (ndim == 0) {  // a single number: handled as a vector of one
    shape = &one_el;
    ndim = 1;
  }
  if (dtype < 0 || dtype > 2) return set_err(h, NVLLM_ERR_INVALID, "bad dtype %d", dtype);
  NV_CHECK(h, cudaSetDevice(h->dev));
  const std::string name(cname);
  const int W = h->H, wdt = h->wdt;
  const size_t wsz = dt_size(wdt);
  Dst d;
  auto vec = [&](float* p, int64_t n) { d.p = p; d.ddt = DT_F32; d.rows = n; d.cols = 0; };
  auto mat = [&](void* p, int64_t rows, int64_t cols, int ld, size_t row0 = 0, int mul = 1, int add = 0) {
    d.p = (char*)p + row0 * (size_t)ld * wsz; d.ddt = wdt; d.rows = rows; d.cols = cols; d.ld = ld;
    d.row_mul = mul; d.row_add = add;
  };
  int l = -1;
  std::string rest;
  const float noff = h->norm_offset;
  if (name == "embed") mat(h->wte, h->V, W, W);
  else if (name == "head" && h->lm_head_owned) mat(h->lm_head, h->V, W, W);
  else if (name == "final.norm") { vec(h->lnf_w, W); d.add = noff; }
  else if (name == "embed.norm" && h->embed_norm_w) vec(h->embed_norm_w, W);
  else if (name == "side.embed" && h->side_embed) mat(h->side_embed, h->V, (int64_t)h->L * h->side_dim, h->L * h->side_dim);
  else if (name == "loop.step" && h->loop_step) {
    mat(h->loop_step, h->loop_times, W, W);
    d.ddt = DT_F32; d.p = h->loop_step;
  } else if (parse_layer_name(name, &l, &rest) && l < h->L &&
             (h->ll[l].s.mixer == NVLLM_MIXER_ATTENTION || h->ll[l].s.mixer == NVLLM_MIXER_MAMBA2)) {
    // sequential pre-norm blocks: attention with options / Mamba-2, mixture of gated experts, the
    // convolution on the mixer's input and the per-layer token input
    ListedLayer& y = h->ll[l];
    const nvllm_layer_spec& s = y.s;
    auto f32mat = [&](float* p, int64_t rows, int64_t cols) { mat(p, rows, cols, (int)cols); d.ddt = DT_F32; d.p = p; };
    const int hv = s.heads * s.vdim;
    if (rest == "norm1") vec(y.post1_w, W);
    else if (rest == "norm2" && s.mlp != NVLLM_MLP_NONE) vec(y.post2_w, W);
    else if (rest == "canon1" && y.canon_w) f32mat(y.canon_w, W, h->mixer_conv);
    else if (rest == "side.gate" && y.side_gate) mat(y.side_gate, h->side_dim, W, W);
    else if (rest == "side.proj" && y.side_proj) mat(y.side_proj, W, h->side_dim, h->side_p);
    else if (rest == "side.norm" && y.side_norm) vec(y.side_norm, W);
    else if (rest == "mix.o") mat(y.w_o, W, hv, y.ov_p);
    else if (s.mixer == NVLLM_MIXER_ATTENTION) {
      if (rest == "mix.q") mat(y.w_in, y.n_q, W, W, 0);
      else if (rest == "mix.k") mat(y.w_in, y.n_k, W, W, y.n_q);
      else if (rest == "mix.v") mat(y.w_in, y.n_v, W, W, y.n_q + y.n_k);
      else if (rest == "mix.g" && s.head_gate) mat(y.w_in, s.heads, W, W, y.n_q + y.n_k + y.n_v);
      else if (rest == "mix.q.norm" && s.qk_norm == 3) vec(y.qnorm_w, s.dim);
      else if (rest == "mix.k.norm" && s.qk_norm == 3) vec(y.knorm_w, s.dim);
      else if (rest == "mix.vmix" && s.v_mix) vec(y.vmix, 1);
      else if (rest == "mix.sink" && s.sink_learned) vec(y.sink_w, s.heads);
      else if (rest == "mix.temp" && s.head_temp) vec(y.head_temp, s.heads);
    } else {
      if (rest == "mix.in") mat(y.w_in, y.n_in, W, W);
      else if (rest == "mix.conv") f32mat(y.conv_w, y.conv_ch, s.conv);
      else if (rest == "mix.conv.b") vec(y.conv_b, y.conv_ch);
      else if (rest == "mix.dt_bias") vec(y.dt_bias, s.heads);
      else if (rest == "mix.A_log") vec(y.a_log, s.heads);
      else if (rest == "mix.D") vec(y.d_skip, s.heads);
      else if (rest == "mix.norm") vec(y.onorm_w, hv);
    }
    if (!d.p && s.mlp == NVLLM_MLP_MOE) {
      if (rest == "mlp.router") f32mat(y.router, s.experts, W);
      else if (rest == "mlp.correction" && s.route_correction) vec(y.route_corr, s.experts);
      else if (rest.compare(0, 5, "mlp.e") == 0) {
        size_t i = 5;
        int e = 0;
        while (i < rest.size() && rest[i] >= '0' && rest[i] <= '9') e = e * 10 + (rest[i++] - '0');
        const std::string part = i < rest.size() ? rest.substr(i) : "";
        if (i == 5 || e >= s.experts) return set_err(h, NVLLM_ERR_INVALID, "unknown tensor %s", cname);
        if (part == ".gate") mat(y.moe_in, s.ff, W, W, (size_t)e * 2 * y.ff_p, 2, 0);
        else if (part == ".up") mat(y.moe_in, s.ff, W, W, (size_t)e * 2 * y.ff_p, 2, 1);
        else if (part == ".down") mat(y.moe_out, W, s.ff, y.ff_p, (size_t)e * W);
      }
    }
  } else if (parse_layer_name(name, &l, &rest) && l < h->L &&
             (h->ll[l].s.mixer == NVLLM_MIXER_GLA || h->ll[l].s.mixer == NVLLM_MIXER_ATTN_TMIX)) {
    // sequential pre-norm blocks: gated linear attention / attention + time mixing, mixture of experts
    ListedLayer& y = h->ll[l];
    const nvllm_layer_spec& s = y.s;
    auto f32mat = [&](float* p, int64_t rows, int64_t cols) { mat(p, rows, cols, (int)cols); d.ddt = DT_F32; d.p = p; };
    if (rest == "norm1") vec(y.post1_w, W);
    else if (rest == "norm2" && s.mlp != NVLLM_MLP_NONE) vec(y.post2_w, W);
    else if (s.mixer == NVLLM_MIXER_GLA) {
      const int hd = s.heads * s.dim, hv = s.heads * s.vdim;
      if (rest == "mix.q") mat(y.w_in, hd, W, W, 0);
      else if (rest == "mix.k") mat(y.w_in, hd, W, W, hd);
      else if (rest == "mix.v") mat(y.w_in, hv, W, W, 2 * hd);
      else if (rest == "mix.g") mat(y.w_in, hv, W, W, 2 * hd + hv);
      else if (rest == "mix.a1") mat(y.w_in, s.lowrank, W, W, 2 * hd + 2 * hv);
      else if (rest == "mix.a2") f32mat(y.lr_w2, hd, s.lowrank);
      else if (rest == "mix.a2.b") vec(y.lr_b, hd);
      else if (rest == "mix.norm") vec(y.onorm_w, s.vdim);
      else if (rest == "mix.o") mat(y.w_o, W, hv, y.ov_p);
    } else {
      const int hv = s.heads * s.vdim, hd2 = s.heads2 * s.dim2, nch = y.n_q + y.n_k + y.n_v;
      if (rest == "mix.left.q") mat(y.w_in, y.n_q, W, W, 0);
      else if (rest == "mix.left.k") mat(y.w_in, y.n_k, W, W, y.n_q);
      else if (rest == "mix.left.v") mat(y.w_in, y.n_v, W, W, y.n_q + y.n_k);
      else if (rest == "mix.left.g" && s.out_gate) mat(y.w_in, hv, W, W, nch);
      else if (rest == "mix.left.q.b" && s.proj_bias) vec(y.bias_in, y.n_q);
      else if (rest == "mix.left.k.b" && s.proj_bias) vec(y.bias_in + y.n_q, y.n_k);
      else if (rest == "mix.left.v.b" && s.proj_bias) vec(y.bias_in + y.n_q + y.n_k, y.n_v);
      else if (rest == "mix.left.o.b" && s.proj_bias) vec(y.o_bias, W);
      else if (rest == "mix.left.q.norm") vec(y.qnorm_w, y.n_q);
      else if (rest == "mix.left.k.norm") vec(y.knorm_w, y.n_k);
      else if (rest == "mix.left.q.conv") f32mat(y.conv_w, y.n_q, s.conv);
      else if (rest == "mix.left.k.conv") f32mat(y.conv_w + (size_t)y.n_q * s.conv, y.n_k, s.conv);
      else if (rest == "mix.left.v.conv") f32mat(y.conv_w + (size_t)(y.n_q + y.n_k) * s.conv, y.n_v, s.conv);
      else if (rest == "mix.left.o") mat(y.w_o, W, hv, y.ov_p);
      else if (rest == "mix.right.r") mat(y.w_in2, hd2, W, W, y.seg2[0]);
      else if (rest == "mix.right.k") mat(y.w_in2, hd2, W, W, y.seg2[1]);
      else if (rest == "mix.right.v") mat(y.w_in2, hd2, W, W, y.seg2[2]);
      else if (rest == "mix.right.g") mat(y.w_in2, hd2, W, W, y.seg2[3]);
      else if (rest == "mix.right.w1") mat(y.w_in2, s.lowrank, W, W, y.seg2[4]);
      else if (rest == "mix.right.w2") f32mat(y.lr_w2, hd2, s.lowrank);
      else if (rest == "mix.right.w0") vec(y.lr_b, hd2);
      else if (rest == "mix.right.u") f32mat(y.bonus, s.heads2, s.dim2);
      else if (rest == "mix.right.norm") vec(y.onorm_w, hd2);
      else if (rest == "mix.right.o") mat(y.w_o2, W, hd2, y.ov2_p);
      else if (rest.compare(0, 13, "mix.right.mu.") == 0 && rest.size() == 14) {
        const char* order = "rkvgw";
        const char* at = strchr(order, rest[13]);
        if (at) vec(y.mu + (size_t)(at - order) * W, W);
      }
    }
    if (!d.p && s.mlp == NVLLM_MLP_MOE) {
      if (rest == "mlp.router") f32mat(y.router, s.experts, W);
      else if (rest == "mlp.shared.up" && s.shared_ff > 0) mat(y.w1, s.shared_ff, W, W);
      else if (rest == "mlp.shared.down" && s.shared_ff > 0) mat(y.w2, W, s.shared_ff, y.sff_p);
      else if (rest == "mlp.shared.sg" && s.shared_ff > 0) f32mat(y.sh_gate, 1, W);
      else if (rest.compare(0, 5, "mlp.e") == 0) {
        size_t i = 5;
        int e = 0;
        while (i < rest.size() && rest[i] >= '0' && rest[i] <= '9') e = e * 10 + (rest[i++] - '0');
        const std::string part = i < rest.size() ? rest.substr(i) : "";
        if (i == 5 || e >= s.experts) return set_err(h, NVLLM_ERR_INVALID, "unknown tensor %s", cname);
        if (part == ".up") mat(y.moe_in, s.ff, W, W, (size_t)e * y.ff_p);
        else if (part == ".down") mat(y.moe_out, W, s.ff, y.ff_p, (size_t)e * W);
      }
    }
  } else if (parse_layer_name(name, &l, &rest) && l < h->L && h->ll[l].s.mixer != NVLLM_MIXER_LATENT_ATTENTION) {
    // sequential post-norm blocks: window attention / delta rule mixers, relu^2 feed-forward
    ListedLayer& y = h->ll[l];
    const nvllm_layer_spec& s = y.s;
    const int own = s.kv_from < 0;
    const bool delta = s.mixer == NVLLM_MIXER_DELTA;
    if (rest == "norm1") { vec(y.post1_w, W); d.add = noff; }
    else if (rest == "norm2" && s.mlp != NVLLM_MLP_NONE) { vec(y.post2_w, W); d.add = noff; }
    else if (rest == "mix.q") mat(y.w_in, y.n_q, W, W, 0);
    else if (rest == "mix.k" && (delta || own)) mat(y.w_in, y.n_k, W, W, y.n_q);
    else if (rest == "mix.v" && (delta || own)) mat(y.w_in, y.n_v, W, W, y.n_q + y.n_k);
    else if (rest == "mix.o") mat(y.w_o, W, (int64_t)s.heads * s.vdim, y.ov_p);
    else if (delta && rest == "mix.b") mat(y.w_in, s.heads, W, W, y.conv_ch);
    else if (delta && rest == "mix.a") mat(y.w_in, s.heads, W, W, y.conv_ch + s.heads);
    else if (delta && rest == "mix.g") mat(y.w_in, (int64_t)s.heads * s.vdim, W, W, y.conv_ch + 2 * s.heads);
    else if (delta && rest == "mix.q.conv") { mat(y.conv_w, y.n_q, s.conv, s.conv, 0); d.ddt = DT_F32; d.p = y.conv_w; }
    else if (delta && rest == "mix.k.conv") { mat(y.conv_w, y.n_k, s.conv, s.conv, 0); d.ddt = DT_F32; d.p = y.conv_w + (size_t)y.n_q * s.conv; }
    else if (delta && rest == "mix.v.conv") { mat(y.conv_w, y.n_v, s.conv, s.conv, 0); d.ddt = DT_F32; d.p = y.conv_w + (size_t)(y.n_q + y.n_k) * s.conv; }
    else if (delta && rest == "mix.A_log") vec(y.a_log, s.heads);
    else if (delta && rest == "mix.dt_bias") vec(y.dt_bias, s.heads);
    else if (delta && rest == "mix.norm") vec(y.onorm_w, s.vdim);
    else if (s.mlp == NVLLM_MLP_DENSE && rest == "mlp.up") mat(y.w1, s.ff, W, W);
    else if (s.mlp == NVLLM_MLP_DENSE && rest == "mlp.down") mat(y.w2, W, s.ff, y.ff_p);
  } else if (parse_layer_name(name, &l, &rest) && l < h->L) {
    ListedLayer& y = h->ll[l];
    const nvllm_layer_spec& s = y.s;
    const int own = s.kv_from < 0;
    if (rest == "norm1") vec(y.norm_w, W);
    else if (rest == "mix.dq") mat(y.w_in, s.q_rank, W, W, 0);
    else if (rest == "mix.dkv" && own) mat(y.w_in, y.Dk, W, W, s.q_rank);
    else if (rest == "mix.g") mat(y.w_in, s.heads, W, W, s.q_rank + (own ? y.Dk : 0));
    else if (rest == "mix.dq.norm") vec(y.dq_norm, s.q_rank);
    else if (rest == "mix.dkv.norm" && own) vec(y.dkv_norm, s.kv_rank);
    else if (rest == "mix.uq") mat(y.w_uq, y.q_cols, s.q_rank, y.q_rank_p);
    else if (rest == "mix.uk") mat(y.w_uk, (int64_t)s.heads * s.dim, s.kv_rank, s.kv_rank);
    else if (rest == "mix.uv") mat(y.w_uv, (int64_t)s.heads * s.vdim, s.kv_rank, s.kv_rank);
    else if (rest == "mix.o") mat(y.w_o, W, (int64_t)s.heads * s.vdim, y.ov_p);
    else if (s.mlp == NVLLM_MLP_DENSE && rest == "mlp.gate") mat(y.w1, s.ff, W, W, 0, 2, 0);
    else if (s.mlp == NVLLM_MLP_DENSE && rest == "mlp.up") mat(y.w1, s.ff, W, W, 0, 2, 1);
    else if (s.mlp == NVLLM_MLP_DENSE && rest == "mlp.down") mat(y.w2, W, s.ff, y.ff_p);
    else if (s.mlp == NVLLM_MLP_MOE && rest == "mlp.router") {
      mat(y.router, s.experts, W, W);
      d.ddt = DT_F32;
      d.p = y.router;
    } else if (s.mlp == NVLLM_MLP_MOE && rest.compare(0, 5, "mlp.e") == 0) {
      size_t i = 5;
      int e = 0;
      while (i < rest.size() && rest[i] >= '0' && rest[i] <= '9') e = e * 10 + (rest[i++] - '0');
      const std::string part = i < rest.size() ? rest.substr(i) : "";
      if (i == 5 || e >= s.experts) return set_err(h, NVLLM_ERR_INVALID, "unknown tensor %s", cname);
      if (part == ".gate") mat(y.moe_in, s.ff, W, W, (size_t)e * 2 * y.ff_p, 2, 0);
      else if (part == ".up") mat(y.moe_in, s.ff, W, W, (size_t)e * 2 * y.ff_p, 2, 1);
      else if (part == ".down") mat(y.moe_out, W, s.ff, y.ff_p, (size_t)e * W);
    }
  }
  if (!d.p) return set_err(h, NVLLM_ERR_INVALID, "tensor %s does not belong to this model", cname);
  const bool is_vec = d.cols == 0;
  if ((is_vec && (ndim != 1 || shape[0] != d.rows)) ||
      (!is_vec && (ndim != 2 || shape[0] != d.rows || shape[1] != d.cols)))
    return set_err(h, NVLLM_ERR_INVALID, "tensor %s: shape [%lld%s%lld] where [%lld%s%lld] is expected", cname,
                   (long long)shape[0], ndim > 1 ? ", " : "", ndim > 1 ? (long long)shape[1] : 0LL,
                   (long long)d.rows, is_vec ? "" : ", ", (long long)d.cols);
  const size_t numel = (size_t)d.rows * (is_vec ? 1 : d.cols);
  void* stage = nullptr;
  NV_CHECK(h, cudaMalloc(&stage, numel * wire_size(dtype)));
  cudaError_t e = cudaMemcpyAsync(stage, host, numel * wire_size(dtype), cudaMemcpyHostToDevice, h->stream);
  if (e == cudaSuccess) {
    if (is_vec) {
      e = launch_convert(h->stream, dtype, stage, numel, DT_F32, d.p);
      if (e == cudaSuccess && d.add != 0.f) {
        add_const_kernel<<<(unsigned)((numel + 255) / 256), 256, 0, h->stream>>>((float*)d.p, numel, d.add);
        e = cudaGetLastError();
      }
    } else e = launch_copy_rows(h->stream, dtype, stage, (size_t)d.cols, (int)d.rows, (int)d.cols, d.ddt, d.p,
                              d.ld, d.row_mul, d.row_add);
  }
  if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
  cudaFree(stage);
  if (e != cudaSuccess) return set_err(h, NVLLM_ERR_CUDA, "tensor %s: %s", cname, cudaGetErrorString(e));
  h->named_got.push_back(name);
  return NVLLM_OK;
}

int layered_finalize(nvllm_handle* h) {
  auto got = [&](const std::string& n) {
    for (auto& g : h->named_got)
      if (g == n) return true;
    return false;
  };
  std::vector<std::string> need = {"embed", "final.norm"};
  if (h->lm_head_owned) need.push_back("head");
  if (h->loop_step) need.push_back("loop.step");
  if (h->embed_norm_w) need.push_back("embed.norm");
  if (h->side_embed) need.push_back("side.embed");
  for (int l = 0; l < h->L; l++) {
    const nvllm_layer_spec& s = h->ll[l].s;
    const std::string p = "l" + std::to_string(l) + ".";
    if (s.mixer == NVLLM_MIXER_ATTENTION || s.mixer == NVLLM_MIXER_MAMBA2) {
      need.push_back(p + "norm1");
      need.push_back(p + "mix.o");
      if (s.mixer == NVLLM_MIXER_ATTENTION) {
        for (const char* n : {"mix.q", "mix.k", "mix.v"}) need.push_back(p + n);
        if (s.qk_norm == 3) { need.push_back(p + "mix.q.norm"); need.push_back(p + "mix.k.norm"); }
        if (s.v_mix && !h->ll[l].vmix_first) need.push_back(p + "mix.vmix");
        if (s.sink_learned) need.push_back(p + "mix.sink");
        if (s.head_temp) need.push_back(p + "mix.temp");
        if (s.head_gate) need.push_back(p + "mix.g");
      } else {
        for (const char* n : {"mix.in", "mix.conv", "mix.conv.b", "mix.dt_bias", "mix.A_log", "mix.D", "mix.norm"})
          need.push_back(p + n);
      }
      if (h->ll[l].canon_w) need.push_back(p + "canon1");
      if (h->ll[l].side_gate)
        for (const char* n : {"side.gate", "side.proj", "side.norm"}) need.push_back(p + n);
      if (s.mlp == NVLLM_MLP_MOE) {
        need.push_back(p + "norm2");
        need.push_back(p + "mlp.router");
        if (s.route_correction) need.push_back(p + "mlp.correction");
        for (int e = 0; e < s.experts; e++)
          for (const char* n : {".gate", ".up", ".down"}) need.push_back(p + "mlp.e" + std::to_string(e) + n);
      }
      continue;
    }
    if (s.mixer == NVLLM_MIXER_GLA || s.mixer == NVLLM_MIXER_ATTN_TMIX) {
      need.push_back(p + "norm1");
      if (s.mixer == NVLLM_MIXER_GLA) {
        for (const char* n : {"mix.q", "mix.k", "mix.v", "mix.g", "mix.a1", "mix.a2", "mix.a2.b", "mix.norm", "mix.o"})
          need.push_back(p + n);
      } else {
        for (const char* n : {"mix.left.q", "mix.left.k", "mix.left.v", "mix.left.q.norm", "mix.left.k.norm",
                              "mix.left.q.conv", "mix.left.k.conv", "mix.left.v.conv", "mix.left.o", "mix.right.r",
                              "mix.right.k", "mix.right.v", "mix.right.g", "mix.right.w1", "mix.right.w2", "mix.right.w0",
                              "mix.right.u", "mix.right.norm", "mix.right.o", "mix.right.mu.r", "mix.right.mu.k",
                              "mix.right.mu.v", "mix.right.mu.g", "mix.right.mu.w"})
          need.push_back(p + n);
        if (s.out_gate) need.push_back(p + "mix.left.g");
        if (s.proj_bias)
          for (const char* n : {"mix.left.q.b", "mix.left.k.b", "mix.left.v.b", "mix.left.o.b"}) need.push_back(p + n);
      }
      if (s.mlp == NVLLM_MLP_MOE) {
        need.push_back(p + "norm2");
        need.push_back(p + "mlp.router");
        for (int e = 0; e < s.experts; e++)
          for (const char* n : {".up", ".down"}) need.push_back(p + "mlp.e" + std::to_string(e) + n);
        if (s.shared_ff > 0)
          for (const char* n : {"mlp.shared.up", "mlp.shared.down", "mlp.shared.sg"}) need.push_back(p + n);
      }
      continue;
    }
    if (s.mixer != NVLLM_MIXER_LATENT_ATTENTION) {
      for (const char* n : {"norm1", "mix.q", "mix.o"}) need.push_back(p + n);
      if (s.mixer == NVLLM_MIXER_DELTA) {
        for (const char* n : {"mix.k", "mix.v", "mix.q.conv", "mix.k.conv", "mix.v.conv", "mix.b", "mix.a", "mix.A_log",
                              "mix.dt_bias", "mix.norm", "mix.g"})
          need.push_back(p + n);
      } else if (s.kv_from < 0) {
        need.push_back(p + "mix.k");
        need.push_back(p + "mix.v");
      }
      if (s.mlp == NVLLM_MLP_DENSE)
        for (const char* n : {"norm2", "mlp.up", "mlp.down"}) need.push_back(p + n);
      continue;
    }
    for (const char* n : {"norm1", "mix.dq", "mix.dq.norm", "mix.uq", "mix.uk", "mix.uv", "mix.g", "mix.o"})
      need.push_back(p + n);
    if (s.kv_from < 0) {
      need.push_back(p + "mix.dkv");
      need.push_back(p + "mix.dkv.norm");
    }
    if (s.mlp == NVLLM_MLP_DENSE)
      for (const char* n : {"mlp.gate", "mlp.up", "mlp.down"}) need.push_back(p + n);
    if (s.mlp == NVLLM_MLP_MOE) {
      need.push_back(p + "mlp.router");
      for (int e = 0; e < s.experts; e++)
        for (const char* n : {".gate", ".up", ".down"}) need.push_back(p + "mlp.e" + std::to_string(e) + n);
    }
  }
  for (auto& n : need)
    if (!got(n)) return set_err(h, NVLLM_ERR_INVALID, "missing tensor %s", n.c_str());
  // fold the per-head key / value up projections into the query and output projections
  // (attention_latent.cu), then drop the four tensors as loaded
  for (int l = 0; l < h->L; l++) {
    ListedLayer& y = h->ll[l];
    const nvllm_layer_spec& s = y.s;
    if (s.mixer != NVLLM_MIXER_LATENT_ATTENTION) continue;
    cudaError_t e = launch_latent_fold(h->stream, h->wdt, y.w_uq, y.w_uk, y.w_q, y.w_o, y.w_uv, y.w_ov, h->H, s.heads,
                                       s.dim, s.rot_dim, s.vdim, s.kv_rank, s.q_rank, y.q_rank_p, y.ov_p, y.ovr_p);
    if (e == cudaSuccess) e = cudaStreamSynchronize(h->stream);
    if (e != cudaSuccess) return set_err(h, NVLLM_ERR_CUDA, "folding layer %d: %s", l, cudaGetErrorString(e));
    const size_t wsz = dt_size(h->wdt);
    const size_t freed = ((size_t)y.q_cols * y.q_rank_p + (size_t)s.heads * s.dim * s.kv_rank +
                          (size_t)s.heads * s.vdim * s.kv_rank + (size_t)h->H * y.ov_p) * wsz;
    for (void** p : {&y.w_uq, &y.w_uk, &y.w_uv, &y.w_o}) {
      cudaFree(*p);
      *p = nullptr;
    }
    h->weight_bytes -= std::min<uint64_t>(h->weight_bytes, freed);
  }
  // cache pools: one per layer with its own down projection, rows [c | rotated key part]
  h->lat_pools.assign(h->L, nullptr);
  // (pre-norm blocks: one K / V pool per EXECUTION of an attention layer, see LayerRun)
  const size_t n_pools = std::max((size_t)h->L, h->runs.size());
  h->win_kpools.assign(n_pools, nullptr);
  h->win_vpools.assign(n_pools, nullptr);
  for (size_t r = 0; r < h->runs.size(); r++) {
    const ListedLayer& y = h->ll[h->runs[r].layer];
    if (y.s.mixer != NVLLM_MIXER_ATTN_TMIX && y.s.mixer != NVLLM_MIXER_ATTENTION) continue;
    const size_t rows = (size_t)h->num_blocks * y.s.kv_heads * KV_BLOCK;
    const size_t kb = rows * y.s.dim * dt_size(h->kvdt), vb = rows * y.s.vdim * dt_size(h->kvdt);
    cudaError_t e = cudaMalloc(&h->win_kpools[r], kb);
    if (e == cudaSuccess) e = cudaMalloc(&h->win_vpools[r], vb);
    if (e != cudaSuccess)
      return set_err(h, NVLLM_ERR_NOMEM, "K / V cache of %d blocks does not fit: %s", h->num_blocks, cudaGetErrorString(e));
    NV_CHECK(h, cudaMemsetAsync(h->win_kpools[r], 0, kb, h->stream));
    NV_CHECK(h, cudaMemsetAsync(h->win_vpools[r], 0, vb, h->stream));
    h->kv_bytes += kb + vb;
  }
  for (int l = 0; l < h->L; l++) {
    ListedLayer& y = h->ll[l];
    if (y.s.mixer != NVLLM_MIXER_WINDOW_ATTENTION || y.s.kv_from >= 0) continue;
    // K [blocks][kv_heads][256][dim], V [blocks][kv_heads][256][vdim]
    const size_t rows = (size_t)h->num_blocks * y.s.kv_heads * KV_BLOCK;
    const size_t kb = rows * y.s.dim * dt_size(h->kvdt), vb = rows * y.s.vdim * dt_size(h->kvdt);
    cudaError_t e = cudaMalloc(&h->win_kpools[l], kb);
    if (e == cudaSuccess) e = cudaMalloc(&h->win_vpools[l], vb);
    if (e != cudaSuccess)
      return set_err(h, NVLLM_ERR_NOMEM, "K / V cache of %d blocks does not fit: %s", h->num_blocks, cudaGetErrorString(e));
    NV_CHECK(h, cudaMemsetAsync(h->win_kpools[l], 0, kb, h->stream));
    NV_CHECK(h, cudaMemsetAsync(h->win_vpools[l], 0, vb, h->stream));
    h->kv_bytes += kb + vb;
  }
  if (h->state_slot_floats) {
    const size_t bytes = (size_t)h->num_state_slots * h->state_slot_floats * 4;
    cudaError_t e = cudaMalloc((void**)&h->state_pool, bytes);
    if (e != cudaSuccess)
      return set_err(h, NVLLM_ERR_NOMEM, "recurrent state of %d slots does not fit: %s", h->num_state_slots, cudaGetErrorString(e));
    NV_CHECK(h, cudaMemsetAsync(h->state_pool, 0, bytes, h->stream));
    h->kv_bytes += bytes;
  }
  if (h->position_kind == NVLLM_LPOS_SINUSOIDAL) {
    const int half = h->H / 2;
    std::vector<double> f(half);
    for (int i = 0; i < half; i++) f[i] = pow(10000.0, -2.0 * (double)i / (double)h->H);
    NV_CHECK(h, cudaMalloc((void**)&h->pos_freq, (size_t)half * 8));
    NV_CHECK(h, cudaMemcpy(h->pos_freq, f.data(), (size_t)half * 8, cudaMemcpyHostToDevice));
  }
  for (int l = 0; l < h->L; l++) {
    ListedLayer& y = h->ll[l];
    if (y.s.mixer != NVLLM_MIXER_LATENT_ATTENTION || y.s.kv_from >= 0) continue;
    const size_t bytes = (size_t)h->num_blocks * KV_BLOCK * y.Dk * dt_size(h->kvdt);
    cudaError_t e = cudaMalloc(&h->lat_pools[l], bytes);
    if (e != cudaSuccess)
      return set_err(h, NVLLM_ERR_NOMEM, "latent cache of %d blocks does not fit: %s", h->num_blocks,
                     cudaGetErrorString(e));
    NV_CHECK(h, cudaMemsetAsync(h->lat_pools[l], 0, bytes, h->stream));
    h->kv_bytes += bytes;
  }
  // rotation frequencies base^(-2i/dims), in double
  for (auto& r : h->ropes) {
    const int half = r.dims / 2;
    std::vector<double> f(half);
    for (int i = 0; i < half; i++) f[i] = pow(r.base, -2.0 * (double)i / (double)r.dims);
    if (r.factor > 0 && r.piecewise) {
      for (int i = 0; i < half; i++) {
        const double wl = 2.0 * M_PI / f[i];
        if (wl < r.original / r.fast) continue;
        if (wl > r.original / r.slow) f[i] = f[i] / r.factor;
        else {
          const double sm = (r.original / wl - r.slow) / (r.fast - r.slow);
          f[i] = (1.0 - sm) * f[i] / r.factor + sm * f[i];
        }
      }
    } else if (r.factor > 0) {
      // entry at which a wavelength of original / turns is reached
      auto at = [&](double turns) { return r.dims * log(r.original / (2.0 * M_PI * turns)) / (2.0 * log(r.base)); };
      const double lo = std::max(floor(at(r.fast)), 0.0), hi = std::min(ceil(at(r.slow)), (double)r.dims - 1.0);
      for (int i = 0; i < half; i++) {
        const double ramp = std::min(std::max(((double)i - lo) / std::max(hi - lo, 0.001), 0.0), 1.0);
        f[i] = f[i] / r.factor * ramp + f[i] * (1.0 - ramp);
      }
      r.mult = 0.1 * log(r.factor) + 1.0;
    }
    NV_CHECK(h, cudaMalloc((void**)&r.inv_freq, (size_t)half * 8));
    NV_CHECK(h, cudaMemcpy(r.inv_freq, f.data(), (size_t)half * 8, cudaMemcpyHostToDevice));
  }
  NV_CHECK(h, cudaStreamSynchronize(h->stream));
  h->finalized = true;
  return NVLLM_OK;
}


// ------------------------------------------------------------------ sequential post-norm blocks
// x += w * rmsnorm(pending sublayer result); xn = x in the activation dtype (what the next
// sublayer reads)
static int run_postnorm(nvllm_handle* h, Pending* p, const float* w, int T, bool want_y = true) {
  NormArgs a{};
  a.post = 1;
  a.x = h->ws.x;
  a.p1 = p->p; a.S1 = p->S; a.stride1 = p->stride; a.m1 = 1.f;
  a.w = w; a.eps = h->cfg.norm_eps; a.y = want_y ? h->ws.xn : nullptr; a.ydt = h->adt;
  a.n_rows = T; a.H = h->H;
  ProfScope ps(h, NVLLM_K_NORM, (double)T * h->H * (4 * 3 + dt_size(h->adt)), 0, (double)T * h->H * 4 * (p->S - 1));
  LAUNCH(h, launch_norm(h->stream, a));
  *p = Pending();
  return NVLLM_OK;
}

static int mixer_window_attention(nvllm_handle* h, const ListedLayer& y, Pending* out) {
  const StepLayout& L = h->lay;
  Workspace& w = h->ws;
  const nvllm_layer_spec& s = y.s;
  const int T = L.T, H = h->H;
  const int32_t* d = L.d;
  const double asz = dt_size(h->adt), kvsz = dt_size(h->kvdt);
  const int own = s.kv_from < 0;
  int rc;
  Pending pin;
  if ((rc = run_gemm(h, w.xn, H, y.w_in, T, y.n_in, H, 1.f, w.ws_a, w.ws_a_floats, y.n_in, &pin))) return rc;
  WinAttnArgs a{};
  a.T = T; a.n_seqs = L.n; a.H = s.heads; a.G = s.kv_heads; a.dim = s.dim; a.vdim = s.vdim;
  a.window = s.window; a.sink = s.sink; a.qk_norm = s.qk_norm; a.own_kv = own;
  a.eps = h->cfg.norm_eps; a.scale = s.scale;
  a.in_p = pin.p; a.in_S = pin.S; a.in_stride = pin.stride; a.in_ld = y.n_in;
  a.slots = d + L.slots;
  a.kpool = h->win_kpools[y.pool]; a.vpool = h->win_vpools[y.pool];
  a.q = w.q; a.out = w.attn_out; a.o_ld = y.ov_p;
  a.block_tables = d + L.block_tables; a.max_blocks = L.max_blocks;
  a.cu_q = d + L.cu_q; a.seq_start = d + L.seq_start; a.seq_len = d + L.seq_len;
  if (L.prefill) {
    a.tile_seq = d + L.tile_seq; a.tile_q0 = d + L.tile_q0; a.n_tiles = L.n_qtiles; a.qtile = h->attn_qtile;
  } else {
    a.n_tiles = L.n; a.qtile = 1;
  }
  {
    ProfScope ps(h, NVLLM_K_ROPE_KV,
                 (double)T * y.n_in * 4 + (double)T * (s.heads * s.dim * asz + own * s.kv_heads * (s.dim + s.vdim) * kvsz), 0,
                 (double)T * y.n_in * 4 * (pin.S - 1));
    LAUNCH(h, launch_winattn_prep(h->stream, h->adt, h->kvdt, a));
  }
  {
    // algorithmic: the window's K / V rows of every sequence once per step; flops over the visible pairs
    const double win = s.window > 0 ? s.window : 1e30;
    const double keys = std::min((double)L.sum_len, (double)L.n * (win - 1) + (double)T);
    const double pairs = std::min(L.attn_pairs, (double)T * win);
    ProfScope ps(h, L.prefill ? NVLLM_K_ATTN_PREFILL : NVLLM_K_ATTN_DECODE, keys * s.kv_heads * (s.dim + s.vdim) * kvsz,
                 2.0 * s.heads * (s.dim + s.vdim) * pairs, (double)T * (s.heads * s.dim + y.ov_p) * asz);
    LAUNCH(h, launch_winattn(h->stream, h->adt, h->kvdt, a));
  }
  return run_gemm(h, w.attn_out, y.ov_p, y.w_o, T, H, y.ov_p, 1.f, w.ws_b, w.ws_b_floats, H, out);
}

static int mixer_delta(nvllm_handle* h, const ListedLayer& y, Pending* out) {
  const StepLayout& L = h->lay;
  Workspace& w = h->ws;
  const nvllm_layer_spec& s = y.s;
  const int T = L.T, H = h->H;
  const int32_t* d = L.d;
  const double asz = dt_size(h->adt);
  int rc;
  Pending pin;
  if ((rc = run_gemm(h, w.xn, H, y.w_in, T, y.n_in, H, 1.f, w.ws_a, w.ws_a_floats, y.n_in, &pin))) return rc;
  DeltaArgs a{};
  a.T = T; a.n_seqs = L.n; a.H = s.heads; a.G = s.kv_heads; a.dim = s.dim; a.vdim = s.vdim; a.taps = s.conv;
  a.n_q = y.n_q; a.n_k = y.n_k; a.n_v = y.n_v; a.conv_ch = y.conv_ch;
  a.eps = h->cfg.norm_eps;
  a.fast_act = h->adt == DT_BF16;
  a.in_p = pin.p; a.in_S = pin.S; a.in_stride = pin.stride; a.in_ld = y.n_in;
  a.conv_w = y.conv_w; a.a_log = y.a_log; a.dt_bias = y.dt_bias; a.onorm_w = y.onorm_w;
  a.cu_q = d + L.cu_q; a.positions = d + L.positions; a.state_slots = d + L.state_slots;
  a.state_pool = h->state_pool; a.slot_floats = h->state_slot_floats; a.state_off = y.state_off; a.tail_off = y.tail_off;
  a.qkv = w.dl_qkv; a.bg = w.dl_bg; a.o = w.dl_o;
  a.out = w.attn_out; a.o_ld = y.ov_p;
  const double hv = (double)s.heads * s.vdim;
  {
    ProfScope ps(h, NVLLM_K_RECUR, (double)T * (y.conv_ch + 2 * s.heads) * 8, 0,
                 (double)T * y.n_in * 4 * (pin.S - 1) + (double)T * y.conv_ch * 4 * (s.conv - 1));
    LAUNCH(h, launch_delta_prep(h->stream, a));
  }
  {
    // algorithmic: every sequence's state once in and once out, the token inputs once, the read-outs once
    const double state = (double)L.n * s.heads * s.dim * s.vdim * 4 * 2;
    ProfScope ps(h, NVLLM_K_RECUR, state + (double)T * (y.conv_ch + 2 * s.heads + hv) * 4, 6.0 * T * hv * s.dim);
    LAUNCH(h, launch_delta_scan(h->stream, a));
  }
  {
    ProfScope ps(h, NVLLM_K_RECUR, (double)T * hv * (4 + 4 + asz), 0, (double)T * hv * 4 * (pin.S - 1));
    LAUNCH(h, launch_delta_out(h->stream, h->adt, a));
  }
  return run_gemm(h, w.attn_out, y.ov_p, y.w_o, T, H, y.ov_p, 1.f, w.ws_b, w.ws_b_floats, H, out);
}

// W_down act(W_up x), act = relu^2: the activation rides in the up projection's epilogue (tcgen05,
// no split-K), in the down projection's GEMV pre-stage (steps of <= 8 rows) or in its own kernel
static int ffn_dense_unary(nvllm_handle* h, const ListedLayer& y, Pending* out) {
  Workspace& w = h->ws;
  const int T = h->lay.T, H = h->H, ff = y.ff_p;
  const double asz = dt_size(h->adt);
  int rc;
  Pending h1;
  if ((rc = run_gemm(h, w.xn, H, y.w1, T, ff, H, 1.f, w.ws_a, w.ws_a_floats, ff, &h1, TC5_EPI_RELU2, w.hbuf, ff, nullptr)))
    return rc;
  const char* gpre_env = getenv("NVLLM_GEMV_PRE");
  if (h1.S > 0 && T <= 8 && !(gpre_env && atoi(gpre_env) == 0)) {
    GemvPre ga{};
    ga.mode = 2; ga.hp = h1.p; ga.Sh = h1.S; ga.hstride = h1.stride; ga.hld = ff; ga.swiglu = 2;
    return run_gemm(h, w.hbuf, ff, y.w2, T, H, ff, 1.f, w.ws_b, w.ws_b_floats, H, out, 0, nullptr, 0, nullptr, nullptr, 0,
                    0.0, nullptr, nullptr, &ga);
  }
  if (h1.S > 0) {
    ProfScope ps(h, NVLLM_K_ACT, (double)T * ff * (4 + asz), 0, (double)T * ff * 4 * (h1.S - 1));
    LAUNCH(h, launch_act(h->stream, h->adt, T, ff, h1.p, h1.S, h1.stride, nullptr, 2, w.hbuf));
  }
  return run_gemm(h, w.hbuf, ff, y.w2, T, H, ff, 1.f, w.ws_b, w.ws_b_floats, H, out);
}

static int forward_layers_postnorm(nvllm_handle* h) {
  const int T = h->lay.T;
  int rc;
  for (int l = 0; l < h->L; l++) {
    const ListedLayer& y = h->ll[l];
    Pending pm;
    if (y.s.mixer == NVLLM_MIXER_WINDOW_ATTENTION) rc = mixer_window_attention(h, y, &pm);
    else if (y.s.mixer == NVLLM_MIXER_DELTA) rc = mixer_delta(h, y, &pm);
    else rc = set_err(h, NVLLM_ERR_INVALID, "layer %d: this mixer has no sequential post-norm form", l);
    if (rc) return rc;
    if ((rc = run_postnorm(h, &pm, y.post1_w, T))) return rc;
    if (y.s.mlp == NVLLM_MLP_DENSE) {
      Pending pf;
      if ((rc = ffn_dense_unary(h, y, &pf))) return rc;
      if ((rc = run_postnorm(h, &pf, y.post2_w, T))) return rc;
    }
  }
  return NVLLM_OK;
}

// ------------------------------------------------------------------ sequential pre-norm blocks
static LinSeg seg_of(const Pending& p, int ld, int col) {
  LinSeg g;
  g.p = p.p + col; g.S = p.S; g.stride = p.stride; g.ld = ld;
  return g;
}

// x += pending sublayer results (+ the vector that opens a pass); xn = RMSNorm(x) * w.  With `moe`
// the kernel also routes the normed row and computes the always-on expert's gate.
// f32_out: the normed row goes out in fp32 (to xn_f32) instead of the activation dtype — the input of the
// convolution that precedes a mixer.  plain: no norm, xn = the updated x itself.
static int run_prenorm(nvllm_handle* h, Pending* p1, Pending* p2, const float* row_m2, const float* xadd, const float* w,
                       const ListedLayer* moe, int T, bool f32_out = false, bool plain = false) {
  Workspace& ws = h->ws;
  NormArgs a{};
  a.x = ws.x;
  a.groups = h->norm_groups;
  a.plain = plain ? 1 : 0;
  double bytes = (double)T * h->H * (4 + dt_size(h->adt)), impl = 0.0;
  if (p1->p) {
    a.p1 = p1->p; a.S1 = p1->S; a.stride1 = p1->stride; a.m1 = p1->m; a.bias1 = p1->bias;
    a.comb_rows = p1->comb_rows; a.comb_w = p1->comb_w; a.comb_k = p1->comb_k;
    bytes += (double)T * h->H * 8;
    impl += (double)T * h->H * 4 * ((p1->comb_rows ? p1->comb_k : p1->S) - 1);
  }
  if (p2->p) {
    a.p2 = p2->p; a.S2 = p2->S; a.stride2 = p2->stride; a.m2 = p2->m; a.bias2 = p2->bias;
    a.row_m2 = row_m2;
    bytes += (double)T * h->H * 4;
    impl += (double)T * h->H * 4 * (p2->S - 1);
  }
  a.xadd = xadd;
  a.w = w; a.eps = h->cfg.norm_eps; a.y = ws.xn; a.ydt = h->adt;
  if (f32_out) { a.y = nullptr; a.y_f32 = ws.xn_f32; }
  a.n_rows = T; a.H = h->H;
  if (moe) {
    const nvllm_layer_spec& s = moe->s;
    a.router = moe->router; a.E = s.experts; a.topk = s.top;
    a.topk_idx = ws.topk_idx; a.topk_w = ws.topk_w;
    a.route = RouteOpts{s.groups, s.keep_groups, s.route_norm ? 0 : 1, 1.f, s.route_sigmoid, s.weight_on_input,
                        s.route_correction ? moe->route_corr : nullptr, s.group_top2};
    if (s.shared_ff > 0) { a.gate_w = moe->sh_gate; a.gate_out = ws.sh_gate; }
    bytes += (double)s.experts * h->H * 4;
  }
  ProfScope ps(h, NVLLM_K_NORM, bytes, 0, impl);
  LAUNCH(h, launch_norm(h->stream, a));
  *p1 = Pending();
  *p2 = Pending();
  return NVLLM_OK;
}

static void linrec_common(nvllm_handle* h, LinRecArgs* a, const LayerRun& r) {
  const StepLayout& L = h->lay;
  const int32_t* d = L.d;
  a->T = L.T; a->n_seqs = L.n;
  a->eps = h->cfg.norm_eps;
  a->cu_q = d + L.cu_q; a->positions = d + L.positions; a->state_slots = d + L.state_slots;
  a->state_pool = h->state_pool; a->slot_floats = h->state_slot_floats; a->state_off = r.state_off;
  a->qkw = h->ws.lr_qkw; a->vv = h->ws.lr_v; a->o = h->ws.lr_o;
  a->out = h->ws.attn_out;
}
// prep, scan and gated norm of a linear recurrence; the caller has filled the segments
static int run_linrec(nvllm_handle* h, const LinRecArgs& a, double in_cols, int in_S) {
  const int T = a.T;
  const double hd = (double)a.H * a.dim, hv = (double)a.H * a.vdim, asz = dt_size(h->adt);
  if (linrec_decode_fused_ok(a)) {
    // one row per sequence: the three kernels as one launch; algorithmic bytes: the state in and out, the row's inputs, the read-out
    ProfScope ps(h, NVLLM_K_RECUR, (double)a.n_seqs * hd * a.vdim * 8 + (double)T * (in_cols * 4 + hv * asz) + hd * a.rank * 4,
                 4.0 * T * hv * a.dim + 2.0 * T * hd * a.rank, (double)T * in_cols * 4 * (in_S - 1));
    LAUNCH(h, launch_linrec_decode(h->stream, h->adt, a));
    return NVLLM_OK;
  }
  {
    ProfScope ps(h, NVLLM_K_RECUR, (double)T * (in_cols * 4 + (3 * hd + hv) * 4) + hd * a.rank * 4, 2.0 * T * hd * a.rank,
                 (double)T * in_cols * 4 * (in_S - 1));
    LAUNCH(h, launch_linrec_prep(h->stream, a));
  }
  {
    // algorithmic: every sequence's state once in and once out, the token inputs once, the read-outs once
    const double state = (double)a.n_seqs * hd * a.vdim * 4 * 2;
    ProfScope ps(h, NVLLM_K_RECUR, state + (double)T * (3 * hd + 2 * hv) * 4, 4.0 * T * hv * a.dim);
    LAUNCH(h, launch_linrec_scan(h->stream, a));
  }
  {
    ProfScope ps(h, NVLLM_K_RECUR, (double)T * hv * (4 + 4 + asz), 0, (double)T * hv * 4 * (a.gate.S - 1));
    LAUNCH(h, launch_linrec_out(h->stream, h->adt, a));
  }
  return NVLLM_OK;
}

static int mixer_gla(nvllm_handle* h, const ListedLayer& y, const LayerRun& r, Pending* out) {
  Workspace& w = h->ws;
  const nvllm_layer_spec& s = y.s;
  const int T = h->lay.T, H = h->H;
  const int hd = s.heads * s.dim, hv = s.heads * s.vdim;
  int rc;
  Pending pin;
  if ((rc = run_gemm(h, w.xn, H, y.w_in, T, y.n_in, H, 1.f, w.ws_a, w.ws_a_floats, y.n_in, &pin))) return rc;
  LinRecArgs a{};
  linrec_common(h, &a, r);
  a.H = s.heads; a.dim = s.dim; a.vdim = s.vdim; a.tmix = 0;
  a.tau = s.tau; a.qmul = 1.0f / sqrtf((float)s.dim);
  a.q = seg_of(pin, y.n_in, 0); a.k = seg_of(pin, y.n_in, hd); a.v = seg_of(pin, y.n_in, 2 * hd);
  a.gate = seg_of(pin, y.n_in, 2 * hd + hv); a.lr = seg_of(pin, y.n_in, 2 * hd + 2 * hv);
  a.rank = s.lowrank; a.w2 = y.lr_w2; a.w2b = y.lr_b;
  a.onorm_w = y.onorm_w; a.onorm_ld = 0;
  a.o_ld = y.ov_p;
  if ((rc = run_linrec(h, a, y.n_in, pin.S))) return rc;
  return run_gemm(h, w.attn_out, y.ov_p, y.w_o, T, H, y.ov_p, 1.f, w.ws_b, w.ws_b_floats, H, out);
}

// Two mixers on the same normed input: *pa = attention (its scale and output bias ride in the
// pending addend), *pb = time mixing.
static int mixer_attn_tmix(nvllm_handle* h, const ListedLayer& y, const LayerRun& r, int run_idx, Pending* pa, Pending* pb) {
  const StepLayout& L = h->lay;
  Workspace& w = h->ws;
  const nvllm_layer_spec& s = y.s;
  const int T = L.T, H = h->H;
  const int32_t* d = L.d;
  const double asz = dt_size(h->adt), kvsz = dt_size(h->kvdt);
  const size_t wsz = dt_size(h->wdt);
  int rc;
  // ---- attention side
  Pending pin;
  if ((rc = run_gemm(h, w.xn, H, y.w_in, T, y.n_in, H, 1.f, w.ws_a, w.ws_a_floats, y.n_in, &pin))) return rc;
  WinAttnArgs a{};
  a.T = T; a.n_seqs = L.n; a.H = s.heads; a.G = s.kv_heads; a.dim = s.dim; a.vdim = s.vdim;
  a.window = s.window; a.chunk = s.chunk; a.softcap = s.softcap; a.sink = s.sink; a.qk_norm = s.qk_norm; a.own_kv = 1;
  a.eps = h->cfg.norm_eps; a.scale = s.scale;
  a.in_p = pin.p; a.in_S = pin.S; a.in_stride = pin.stride; a.in_ld = y.n_in;
  a.slots = d + L.slots;
  a.kpool = h->win_kpools[run_idx]; a.vpool = h->win_vpools[run_idx];
  a.q = w.q; a.out = w.attn_out; a.o_ld = y.ov_p;
  a.block_tables = d + L.block_tables; a.max_blocks = L.max_blocks;
  a.cu_q = d + L.cu_q; a.seq_start = d + L.seq_start; a.seq_len = d + L.seq_len;
  if (s.out_gate) { a.gate = w.att_gate; a.gate_ld = s.heads * s.vdim; }
  if (L.prefill) {
    a.tile_seq = d + L.tile_seq; a.tile_q0 = d + L.tile_q0; a.n_tiles = L.n_qtiles; a.qtile = h->attn_qtile;
  } else {
    a.n_tiles = L.n; a.qtile = 1;
  }
  ConvAttnPrep c{};
  c.taps = s.conv; c.conv_w = y.conv_w; c.bias = s.proj_bias ? y.bias_in : nullptr;
  c.qnorm_w = y.qnorm_w; c.knorm_w = y.knorm_w;
  if (y.rope >= 0) {
    const RopeTable& rt = h->ropes[y.rope];
    c.rot_half = s.rot_dims / 2; c.cosT = rt.cosT; c.sinT = rt.sinT;
  }
  c.positions = d + L.positions; c.state_slots = d + L.state_slots;
  c.state_pool = h->state_pool; c.slot_floats = h->state_slot_floats; c.tail_off = r.tail_off;
  c.gate_out = s.out_gate ? w.att_gate : nullptr; c.gate_ld = a.gate_ld;
  {
    ProfScope ps(h, NVLLM_K_ROPE_KV,
                 (double)T * y.n_in * 4 + (double)T * (y.n_q * asz + (y.n_k + y.n_v) * kvsz + (s.out_gate ? a.gate_ld * 4.0 : 0.0)), 0,
                 (double)T * y.n_in * 4 * (pin.S - 1) + (double)T * y.conv_ch * 4 * (s.conv - 1));
    LAUNCH(h, launch_winattn_prep_conv(h->stream, h->adt, h->kvdt, a, c));
  }
  {
    // algorithmic: the visible K / V rows of every sequence once per step; flops over the visible pairs
    const double span = s.chunk > 0 ? s.chunk : (s.window > 0 ? s.window : 1e30);
    const double keys = std::min((double)L.sum_len, (double)L.n * (span - 1) + (double)T);
    const double pairs = std::min(L.attn_pairs, (double)T * (s.chunk > 0 ? (span + 1) / 2 : span));
    ProfScope ps(h, L.prefill ? NVLLM_K_ATTN_PREFILL : NVLLM_K_ATTN_DECODE, keys * s.kv_heads * (s.dim + s.vdim) * kvsz,
                 2.0 * s.heads * (s.dim + s.vdim) * pairs, (double)T * (s.heads * s.dim + y.ov_p) * asz);
    LAUNCH(h, launch_winattn(h->stream, h->adt, h->kvdt, a));
  }
  if ((rc = run_gemm(h, w.attn_out, y.ov_p, y.w_o, T, H, y.ov_p, 1.f, w.ws_b, w.ws_b_floats, H, pa))) return rc;
  pa->m = s.mix_scale;
  pa->bias = s.proj_bias ? y.o_bias : nullptr;
  // ---- time mixing side: the five shifted inputs, a projection each into one row of partials
  {
    ProfScope ps(h, NVLLM_K_RECUR, (double)T * H * asz * 6 + 5.0 * H * 4, 0);
    LAUNCH(h, launch_token_shift(h->stream, h->adt, T, L.n, H, 5, w.xn, y.mu, d + L.cu_q, d + L.positions, d + L.state_slots,
                                 h->state_pool, h->state_slot_floats, r.shift_off, w.mx_in));
  }
  // the slot's tails move on: the attention side's convolution inputs (still in ws_a) and the token shift's last row
  {
    TailJob jobs[2];
    int nj = 0;
    if (s.conv > 1) {
      TailJob& j = jobs[nj++];
      j.seg = seg_of(pin, y.n_in, 0); j.bias = c.bias; j.act = nullptr;
      j.channels = y.conv_ch; j.taps = s.conv; j.tail_off = r.tail_off;
    }
    TailJob& j = jobs[nj++];
    j.seg = LinSeg{nullptr, 0, 0, 0}; j.bias = nullptr; j.act = w.xn;
    j.channels = H; j.taps = 2; j.tail_off = r.shift_off;
    ProfScope ps(h, NVLLM_K_RECUR, (double)L.n * ((s.conv - 1) * y.conv_ch + H) * 8, 0);
    LAUNCH(h, launch_roll_tails(h->stream, h->adt, L.n, jobs, nj, d + L.cu_q, d + L.positions, d + L.state_slots,
                                h->state_pool, h->state_slot_floats));
  }
  const int hd2 = s.heads2 * s.dim2;
  Pending seg[5];
  for (int i = 0; i < 5; i++) {
    const int n = i < 4 ? hd2 : s.lowrank;
    const char* A = (const char*)w.mx_in + (size_t)i * T * H * (size_t)asz;
    const char* Wt = (const char*)y.w_in2 + (size_t)y.seg2[i] * H * wsz;
    if ((rc = run_gemm(h, A, H, Wt, T, n, H, 1.f, w.ws_a + y.seg2[i], w.ws_a_floats - y.seg2[i], y.n_in2, &seg[i]))) return rc;
  }
  LinRecArgs b{};
  linrec_common(h, &b, r);
  b.H = s.heads2; b.dim = s.dim2; b.vdim = s.dim2; b.tmix = 1;
  b.tau = 1.f; b.qmul = 1.f;
  b.q = seg_of(seg[0], y.n_in2, 0); b.k = seg_of(seg[1], y.n_in2, 0); b.v = seg_of(seg[2], y.n_in2, 0);
  b.gate = seg_of(seg[3], y.n_in2, 0); b.lr = seg_of(seg[4], y.n_in2, 0);
  b.rank = s.lowrank; b.w2 = y.lr_w2; b.w2b = y.lr_b; b.bonus = y.bonus;
  b.onorm_w = y.onorm_w; b.onorm_ld = s.dim2;
  b.o_ld = y.ov2_p;
  if ((rc = run_linrec(h, b, y.n_in2, seg[0].S))) return rc;
  if ((rc = run_gemm(h, w.attn_out, y.ov2_p, y.w_o2, T, H, y.ov2_p, 1.f, w.ws_c, w.ws_b_floats, H, pb))) return rc;
  pb->m = s.mix2_scale;
  return NVLLM_OK;
}

// Mixture of squared-ReLU experts (+ the always-on expert): *p1 = the experts' outputs, combined
// by the next norm kernel with the squared scores; *p2 = the always-on expert, times its gate there.
static int ffn_moe_relu2(nvllm_handle* h, const ListedLayer& y, Pending* p1, Pending* p2) {
  Workspace& w = h->ws;
  const nvllm_layer_spec& s = y.s;
  const int T = h->lay.T, H = h->H;
  const double asz = dt_size(h->adt);
  int rc;
  if ((rc = run_moe_ffn(h, T, w.xn, s.experts, s.top, y.ff_p, 0.f, y.moe_in, y.moe_out, w.topk_w, p1, 2))) return rc;
  if (s.shared_ff <= 0) return NVLLM_OK;
  const int ff = y.sff_p;
  Pending h1;
  if ((rc = run_gemm(h, w.xn, H, y.w1, T, ff, H, 1.f, w.ws_a, w.ws_a_floats, ff, &h1, TC5_EPI_RELU2, w.hbuf, ff, nullptr)))
    return rc;
  // steps of <= 8 rows: the activation is built inside the down projection's GEMV (one launch less)
  const char* gpre_env = getenv("NVLLM_GEMV_PRE");
  if (h1.S > 0 && T <= 8 && !(gpre_env && atoi(gpre_env) == 0)) {
    GemvPre ga{};
    ga.mode = 2; ga.hp = h1.p; ga.Sh = h1.S; ga.hstride = h1.stride; ga.hld = ff; ga.swiglu = 2;
    return run_gemm(h, w.hbuf, ff, y.w2, T, H, ff, 1.f, w.ws_b, w.ws_b_floats, H, p2, 0, nullptr, 0, nullptr, nullptr, 0,
                    0.0, nullptr, nullptr, &ga);
  }
  if (h1.S > 0) {
    ProfScope ps(h, NVLLM_K_ACT, (double)T * ff * (4 + asz), 0, (double)T * ff * 4 * (h1.S - 1));
    LAUNCH(h, launch_act(h->stream, h->adt, T, ff, h1.p, h1.S, h1.stride, nullptr, 2, w.hbuf));
  }
  return run_gemm(h, w.hbuf, ff, y.w2, T, H, ff, 1.f, w.ws_b, w.ws_b_floats, H, p2);
}

// Prefill steps of an attention layer whose keys and values have one size, 64 or 128, in bf16, and whose scores are
// neither capped nor biased by the distance (a sink and head gates are fine) run on the tcgen05 kernel
// (attention_tc5.cu, 128 queries per tile); everything else on the window kernels (attention_window.cu)
static bool attention_on_tc5(const nvllm_handle* h, const nvllm_layer_spec& s) {
  return h->adt == DT_BF16 && h->kvdt == DT_BF16 && s.dim == s.vdim && (s.dim == 64 || s.dim == 128) &&
         s.softcap == 0.f && s.dist_slope == 0.f && attn_prefill_tc5_enabled();
}

// Grouped-query attention over the whole cached prefix with the options of the spec
static int mixer_attention(nvllm_handle* h, const ListedLayer& y, int run_idx, Pending* out) {
  const StepLayout& L = h->lay;
  Workspace& w = h->ws;
  const nvllm_layer_spec& s = y.s;
  const int T = L.T, H = h->H;
  const int32_t* d = L.d;
  const double asz = dt_size(h->adt), kvsz = dt_size(h->kvdt);
  int rc;
  Pending pin;
  if ((rc = run_gemm(h, w.xn, H, y.w_in, T, y.n_in, H, 1.f, w.ws_a, w.ws_a_floats, y.n_in, &pin))) return rc;
  WinAttnArgs a{};
  a.T = T; a.n_seqs = L.n; a.H = s.heads; a.G = s.kv_heads; a.dim = s.dim; a.vdim = s.vdim;
  a.softcap = s.softcap; a.sink = s.sink; a.qk_norm = s.qk_norm; a.own_kv = 1;
  a.eps = h->cfg.norm_eps; a.scale = s.scale;
  a.in_p = pin.p; a.in_S = pin.S; a.in_stride = pin.stride; a.in_ld = y.n_in;
  a.slots = d + L.slots;
  a.kpool = h->win_kpools[run_idx]; a.vpool = h->win_vpools[run_idx];
  a.q = w.q; a.out = w.attn_out; a.o_ld = y.ov_p;
  a.block_tables = d + L.block_tables; a.max_blocks = L.max_blocks;
  a.cu_q = d + L.cu_q; a.seq_start = d + L.seq_start; a.seq_len = d + L.seq_len;
  a.qnorm_w = y.qnorm_w; a.knorm_w = y.knorm_w;
  if (y.rope >= 0) {
    const RopeTable& rt = h->ropes[y.rope];
    a.rot_half = s.rot_dims / 2; a.rot_pairs = s.rot_pairs; a.cosT = rt.cosT; a.sinT = rt.sinT;
  }
  a.positions = d + L.positions;
  a.qtemp_coef = s.qtemp_coef; a.qtemp_every = s.qtemp_every;
  a.head_scale = s.head_temp ? y.head_temp : nullptr;
  if (s.v_mix) {
    a.vfirst = w.v_first; a.vfirst_write = y.vmix_first;
    a.vmix = y.vmix_first ? nullptr : y.vmix;
  }
  if (s.head_gate) { a.gate_out = w.att_gate; a.gate = w.att_gate; a.gate_ld = s.heads; a.gate_head = 1; }
  a.slope_exp = s.dist_slope;
  a.sink_w = s.sink_learned ? y.sink_w : nullptr;
  if (L.prefill) {
    a.tile_seq = d + L.tile_seq; a.tile_q0 = d + L.tile_q0; a.n_tiles = L.n_qtiles; a.qtile = h->attn_qtile;
  } else {
    a.n_tiles = L.n; a.qtile = 1;
    // no window bounds the context: few sequences with long contexts would leave most SMs without a CTA, so the
    // keys of a (sequence, key / value head) pair are cut into ranges.  The count depends on the number of
    // sequences only (a captured step replays with the same grid whatever the lengths have become)
    const int pairs = L.n * s.kv_heads;
    if (pairs <= w.att_split_pairs && pairs < 2 * h->sm_count) {
      a.n_split = std::min(WINATTN_MAX_SPLIT, std::max(1, 2 * h->sm_count / pairs));
      a.split_ws = w.att_split; a.split_cnt = w.att_split_cnt;
    }
  }
  {
    ProfScope ps(h, NVLLM_K_ROPE_KV,
                 (double)T * y.n_in * 4 + (double)T * (y.n_q * asz + (y.n_k + y.n_v) * kvsz), 0,
                 (double)T * y.n_in * 4 * (pin.S - 1));
    LAUNCH(h, launch_winattn_prep(h->stream, h->adt, h->kvdt, a));
  }
  {
    // algorithmic: the K / V rows of every context once per step; flops over the visible pairs
    ProfScope ps(h, L.prefill ? NVLLM_K_ATTN_PREFILL : NVLLM_K_ATTN_DECODE,
                 (double)L.sum_len * s.kv_heads * (s.dim + s.vdim) * kvsz, 2.0 * s.heads * (s.dim + s.vdim) * L.attn_pairs,
                 (double)T * (s.heads * s.dim + y.ov_p) * asz);
    if (L.prefill && h->attn_qtile == 128 && attention_on_tc5(h, s)) {
      AttnArgs t{};
      t.q = w.q; t.out = w.attn_out; t.qdt = h->adt; t.kvdt = h->kvdt;
      t.kpool = a.kpool; t.vpool = a.vpool;
      t.n_seqs = L.n; t.nh = s.heads; t.nkv = s.kv_heads; t.hd = s.dim; t.scale = s.scale;
      t.block_tables = a.block_tables; t.max_blocks = a.max_blocks;
      t.cu_q = a.cu_q; t.seq_start = a.seq_start; t.seq_len = a.seq_len;
      t.tile_seq = a.tile_seq; t.tile_q0 = a.tile_q0; t.n_qtiles = L.n_qtiles;
      t.pool_blocks = h->num_blocks; t.total_rows = T; t.sm_count = h->sm_count;
      t.sink = s.sink; t.sink_w = a.sink_w;
      t.head_gate = s.head_gate ? w.att_gate : nullptr; t.gate_ld = s.heads;
      LAUNCH(h, launch_attn_prefill_tc5(h->stream, t));
    } else {
      LAUNCH(h, launch_winattn(h->stream, h->adt, h->kvdt, a));
    }
  }
  return run_gemm(h, w.attn_out, y.ov_p, y.w_o, T, H, y.ov_p, 1.f, w.ws_b, w.ws_b_floats, H, out);
}

// Mamba-2 between its two projections: convolution / step sizes / decays (mamba.cu), the scan of
// linrec.cu (k = B, q = C of the head's group, v = dt x, one decay per token and head), D skip + gate +
// grouped norm (mamba.cu).  *pin_out: the input projection's partials (the convolution's inputs, for the tail).
static int mixer_mamba2(nvllm_handle* h, const ListedLayer& y, const LayerRun& r, Pending* pin_out, Pending* out) {
  const StepLayout& L = h->lay;
  Workspace& w = h->ws;
  const nvllm_layer_spec& s = y.s;
  const int T = L.T, H = h->H;
  const int32_t* d = L.d;
  const double asz = dt_size(h->adt);
  const int inner = s.heads * s.vdim, gn = s.ssm_groups * s.state, ch = y.conv_ch;
  int rc;
  Pending pin;
  if ((rc = run_gemm(h, w.xn, H, y.w_in, T, y.n_in, H, 1.f, w.ws_a, w.ws_a_floats, y.n_in, &pin))) return rc;
  *pin_out = pin;
  Mamba2SlotArgs m{};
  m.T = T; m.n_seqs = L.n; m.heads = s.heads; m.vdim = s.vdim; m.N = s.state; m.G = s.ssm_groups; m.taps = s.conv;
  m.norm_groups = s.norm_groups; m.eps = h->cfg.norm_eps; m.fast_act = h->adt == DT_BF16;
  m.in_p = pin.p; m.in_S = pin.S; m.in_stride = pin.stride; m.in_ld = y.n_in;
  m.conv_w = y.conv_w; m.conv_b = y.conv_b; m.dt_bias = y.dt_bias; m.a_log = y.a_log; m.d_skip = y.d_skip; m.norm_w = y.onorm_w;
  m.cu_q = d + L.cu_q; m.positions = d + L.positions; m.state_slots = d + L.state_slots;
  m.state_pool = h->state_pool; m.slot_floats = h->state_slot_floats; m.tail_off = r.tail_off;
  m.xbc = w.m2_xbc; m.dtx = w.m2_dtx; m.decay = w.m2_decay; m.o = w.lr_o;
  m.out = w.attn_out; m.o_ld = y.ov_p;
  m.state_off = r.state_off;
  if (mamba2_slot_decode_ok(m)) {
    // one row per sequence: convolution, step sizes and the recurrence as one launch.  Algorithmic bytes: every
    // sequence's state once in and once out, the row's inputs, the read-outs
    {
      ProfScope ps(h, NVLLM_K_RECUR, (double)L.n * inner * s.state * 8 + (double)T * ((ch + s.heads) * 4 + 2.0 * inner * 4),
                   4.0 * T * inner * s.state, (double)T * y.n_in * 4 * (pin.S - 1) + (double)T * ch * 4 * (s.conv - 1));
      LAUNCH(h, launch_mamba2_slot_decode(h->stream, m, w.lr_o));
    }
    {
      ProfScope ps(h, NVLLM_K_RECUR, (double)T * inner * (4 + 4 + 4 + asz), 0, (double)T * inner * 4 * (pin.S - 1));
      LAUNCH(h, launch_mamba2_slot_out(h->stream, h->adt, m));
    }
    return run_gemm(h, w.attn_out, y.ov_p, y.w_o, T, H, y.ov_p, 1.f, w.ws_b, w.ws_b_floats, H, out);
  }
  {
    ProfScope ps(h, NVLLM_K_RECUR, (double)T * ((ch + s.heads) * 4 + (ch + inner + s.heads) * 4), 0,
                 (double)T * y.n_in * 4 * (pin.S - 1) + (double)T * ch * 4 * (s.conv - 1));
    LAUNCH(h, launch_mamba2_slot_prep(h->stream, m));
  }
  LinRecArgs b{};
  linrec_common(h, &b, r);
  b.H = s.heads; b.dim = s.state; b.vdim = s.vdim; b.tmix = 0; b.tau = 1.f; b.qmul = 1.f;
  b.q = LinSeg{w.m2_xbc + inner + gn, 1, 0, ch};
  b.k = LinSeg{w.m2_xbc + inner, 1, 0, ch};
  b.v = LinSeg{w.m2_dtx, 1, 0, inner};
  b.qk_div = s.heads / s.ssm_groups;
  b.decay_p = w.m2_decay; b.decay_ld = s.heads;
  {
    // algorithmic: every sequence's state once in and once out, the token inputs once, the read-outs once
    const double state = (double)L.n * inner * s.state * 4 * 2;
    ProfScope ps(h, NVLLM_K_RECUR, state + (double)T * (2.0 * gn + 2.0 * inner + s.heads) * 4, 4.0 * T * inner * s.state);
    LAUNCH(h, launch_linrec_scan(h->stream, b));
  }
  {
    ProfScope ps(h, NVLLM_K_RECUR, (double)T * inner * (4 + 4 + 4 + asz), 0, (double)T * inner * 4 * (pin.S - 1));
    LAUNCH(h, launch_mamba2_slot_out(h->stream, h->adt, m));
  }
  return run_gemm(h, w.attn_out, y.ov_p, y.w_o, T, H, y.ov_p, 1.f, w.ws_b, w.ws_b_floats, H, out);
}

// Per-layer token input after the feed-forward: x += rmsnorm(W_proj (gelu_tanh(W_gate x) * e)) * w, e = the
// token's entries of this layer's part of the side table.  The pending results join x first (the
// gate reads the updated stream itself, not a normed copy).
static int token_side_input(nvllm_handle* h, const ListedLayer& y, int layer, Pending* p1, Pending* p2, const float* row_m2) {
  const StepLayout& L = h->lay;
  Workspace& w = h->ws;
  const int T = L.T, H = h->H, sp = h->side_p;
  int rc;
  if ((rc = run_prenorm(h, p1, p2, row_m2, nullptr, nullptr, nullptr, T, false, true))) return rc;
  Pending pg;
  if ((rc = run_gemm(h, w.xn, H, y.side_gate, T, sp, H, 1.f, w.ws_a, w.ws_a_floats, sp, &pg))) return rc;
  {
    ProfScope ps(h, NVLLM_K_ACT, (double)T * sp * (4 + dt_size(h->wdt) + dt_size(h->adt)), 0, (double)T * sp * 4 * (pg.S - 1));
    LAUNCH(h, launch_token_gate(h->stream, h->adt, h->wdt, T, h->side_dim, pg.p, pg.S, pg.stride, sp, L.d + L.tokens,
                                h->side_embed, h->L * h->side_dim, layer * h->side_dim, w.side_g, sp));
  }
  Pending pp;
  if ((rc = run_gemm(h, w.side_g, sp, y.side_proj, T, H, sp, 1.f, w.ws_b, w.ws_b_floats, H, &pp))) return rc;
  return run_postnorm(h, &pp, y.side_norm, T, false);
}

// *row_m2_out: per-row multiplier of the second addend still pending at the end (or null)
static int forward_layers_prenorm(nvllm_handle* h, Pending* p1, Pending* p2, const float** row_m2_out) {
  const int T = h->lay.T;
  const float* row_m2 = nullptr;  // per-row multiplier of the pending second addend
  int rc;
  for (size_t ri = 0; ri < h->runs.size(); ri++) {
    const LayerRun& r = h->runs[ri];
    const ListedLayer& y = h->ll[r.layer];
    const float* xadd = r.pass_start >= 0 ? h->loop_step + (size_t)r.pass_start * h->H : nullptr;
    const bool conv_in = y.canon_w != nullptr;  // the mixer reads h + conv(h)
    if ((rc = run_prenorm(h, p1, p2, row_m2, xadd, y.post1_w, nullptr, T, conv_in))) return rc;
    row_m2 = nullptr;
    const StepLayout& L = h->lay;
    const int32_t* d = L.d;
    if (conv_in) {
      ProfScope ps(h, NVLLM_K_RECUR, (double)T * h->H * (4 + dt_size(h->adt)), 2.0 * T * h->H * h->mixer_conv,
                   (double)T * h->H * 4 * (h->mixer_conv - 1));
      LAUNCH(h, launch_mixer_conv(h->stream, h->adt, T, L.n, h->H, h->mixer_conv, h->ws.xn_f32, y.canon_w, d + L.cu_q,
                                  d + L.positions, d + L.state_slots, h->state_pool, h->state_slot_floats, r.canon_off,
                                  h->ws.xn));
    }
    Pending pa, pb, pin;
    if (y.s.mixer == NVLLM_MIXER_GLA) rc = mixer_gla(h, y, r, &pa);
    else if (y.s.mixer == NVLLM_MIXER_ATTENTION) rc = mixer_attention(h, y, (int)ri, &pa);
    else if (y.s.mixer == NVLLM_MIXER_MAMBA2) rc = mixer_mamba2(h, y, r, &pin, &pa);
    else rc = mixer_attn_tmix(h, y, r, (int)ri, &pa, &pb);
    if (rc) return rc;
    if (conv_in || y.s.mixer == NVLLM_MIXER_MAMBA2) {
      // the slot's tails move on: the normed rows the mixer's convolution read (still in xn_f32) and Mamba-2's
      // convolution inputs (still in ws_a: the output projection wrote elsewhere)
      TailJob jobs[2];
      int nj = 0;
      double bytes = 0;
      if (conv_in) {
        TailJob& j = jobs[nj++];
        j.seg = LinSeg{h->ws.xn_f32, 1, 0, h->H}; j.bias = nullptr; j.act = nullptr;
        j.channels = h->H; j.taps = h->mixer_conv; j.tail_off = r.canon_off;
        bytes += (double)L.n * (h->mixer_conv - 1) * h->H * 8;
      }
      if (y.s.mixer == NVLLM_MIXER_MAMBA2 && y.s.conv > 1) {
        TailJob& j = jobs[nj++];
        j.seg = seg_of(pin, y.n_in, y.s.heads * y.s.vdim); j.bias = nullptr; j.act = nullptr;
        j.channels = y.conv_ch; j.taps = y.s.conv; j.tail_off = r.tail_off;
        bytes += (double)L.n * (y.s.conv - 1) * y.conv_ch * 8;
      }
      if (nj) {
        ProfScope ps(h, NVLLM_K_RECUR, bytes, 0);
        LAUNCH(h, launch_roll_tails(h->stream, h->adt, L.n, jobs, nj, d + L.cu_q, d + L.positions, d + L.state_slots,
                                    h->state_pool, h->state_slot_floats));
      }
    }
    if (y.s.mlp == NVLLM_MLP_MOE && y.s.act == NVLLM_FFN_SWIGLU) {
      if ((rc = run_prenorm(h, &pa, &pb, nullptr, nullptr, y.post2_w, &y, T))) return rc;
      if ((rc = run_moe_ffn(h, T, h->ws.xn, y.s.experts, y.s.top, y.ff_p, 0.f, y.moe_in, y.moe_out, h->ws.topk_w, p1))) return rc;
    } else if (y.s.mlp == NVLLM_MLP_MOE) {
      if ((rc = run_prenorm(h, &pa, &pb, nullptr, nullptr, y.post2_w, &y, T))) return rc;
      if ((rc = ffn_moe_relu2(h, y, p1, p2))) return rc;
      row_m2 = p2->p ? h->ws.sh_gate : nullptr;
    } else {
      *p1 = pa;
      *p2 = pb;
    }
    if (y.side_gate) {
      if ((rc = token_side_input(h, y, r.layer, p1, p2, row_m2))) return rc;
      row_m2 = nullptr;
    }
  }
  h->glu_limit_cur = 0.f;
  *row_m2_out = row_m2;
  return NVLLM_OK;
}

// ------------------------------------------------------------------ forward pass
int forward_step_layered(nvllm_handle* h) {
  const StepLayout& L = h->lay;
  Workspace& w = h->ws;
  const int T = L.T, n = L.n, n_out = L.n_out > 0 ? L.n_out : L.n, H = h->H;
  const int32_t* d = L.d;
  const int* d_pos = d + L.positions;
  cudaStream_t st = h->stream;
  const double asz = dt_size(h->adt), kvsz = dt_size(h->kvdt), wsz = dt_size(h->wdt);
  int rc;
  {
    ProfScope ps(h, NVLLM_K_EMBED, (double)T * H * (4 + wsz), 0);
    const bool seq_style = h->block_style == NVLLM_LBLOCK_SEQUENTIAL_POSTNORM;
    LAUNCH(h, launch_embed(st, h->wdt, d + L.tokens, d_pos, h->wte, nullptr, 0, h->cfg.embedding_multiplier,
                           w.x, T, H, nullptr, nullptr, nullptr, h->pos_freq, seq_style ? w.xn : nullptr));
  }
  if (h->embed_norm_w) {  // the embedding is normed in place: x <- norm(x) * w
    NormArgs a{};
    a.x = w.x; a.w = h->embed_norm_w; a.eps = h->cfg.norm_eps; a.y = nullptr; a.ydt = h->adt; a.y_f32 = w.x;
    a.n_rows = T; a.H = H; a.groups = h->norm_groups;
    ProfScope ps(h, NVLLM_K_NORM, (double)T * H * 8, 0);
    LAUNCH(h, launch_norm(st, a));
  }
  for (auto& r : h->ropes) {
    ProfScope ps(h, NVLLM_K_MISC, (double)T * r.dims * 4, 0);
    LAUNCH(h, launch_rope_table(st, d_pos, T, r.dims / 2, r.inv_freq, r.cosT, r.sinT, r.mult));
  }
  Pending p1, p2;
  int routed = 0;  // routed layers so far: picks the half of topk_w this layer writes
  const float* row_m2 = nullptr;
  if (h->block_style == NVLLM_LBLOCK_SEQUENTIAL_POSTNORM) {
    if ((rc = forward_layers_postnorm(h))) return rc;
  } else if (h->block_style == NVLLM_LBLOCK_SEQUENTIAL_PRENORM) {
    if ((rc = forward_layers_prenorm(h, &p1, &p2, &row_m2))) return rc;
  } else
  for (int l = 0; l < h->L; l++) {
    const ListedLayer& y = h->ll[l];
    const nvllm_layer_spec& s = y.s;
    RouterArgs ra;
    float* topk_w = w.topk_w;
    if (s.mlp == NVLLM_MLP_MOE) {
      topk_w += (size_t)(routed++ & 1) * w.topk_pairs;
      ra.R = y.router; ra.E = s.experts; ra.k = s.top;
      ra.topk_idx = w.topk_idx; ra.topk_w = topk_w;
      ra.opts = RouteOpts{s.groups, s.keep_groups, 1, s.router_scale};
    }
    if ((rc = run_norm(h, w.x, &p1, &p2, y.norm_w, nullptr, w.xn, nullptr, nullptr, T,
                       s.mlp == NVLLM_MLP_MOE ? &ra : nullptr, true)))
      return rc;
    // ---- mixer: latent attention
    const int own = s.kv_from < 0;
    Pending pin;
    if ((rc = run_gemm(h, w.xn, H, y.w_in, T, y.n_in, H, 1.f, w.ws_a, w.ws_a_floats, y.n_in, &pin))) return rc;
    const RopeTable& rt = h->ropes[y.rope];
    LatentArgs a{};
    a.T = T; a.H = s.heads; a.dim = s.dim; a.rot = s.rot_dim; a.rot_dims = s.rot_dims; a.vdim = s.vdim;
    a.R = s.kv_rank; a.q_rank = s.q_rank; a.q_rank_p = y.q_rank_p; a.o_ld = y.ovr_p; a.own_kv = own;
    a.eps = h->cfg.norm_eps; a.scale = s.scale;
    a.in_p = pin.p; a.in_S = pin.S; a.in_stride = pin.stride; a.in_ld = y.n_in;
    a.dq_norm = y.dq_norm; a.dkv_norm = y.dkv_norm;
    a.cosT = rt.cosT; a.sinT = rt.sinT;
    a.slots = d + L.slots;
    a.pool = h->lat_pools[y.pool];
    a.cq = w.lat_cq; a.gate = w.lat_gate;
    a.qabs = w.q;
    a.block_tables = d + L.block_tables; a.max_blocks = L.max_blocks;
    a.cu_q = d + L.cu_q; a.seq_start = d + L.seq_start; a.seq_len = d + L.seq_len;
    a.olat = w.lat_o;
    a.split_ws = w.attn_ws;
    a.sm_count = h->sm_count;
    if (L.prefill) {
      a.tile_seq = d + L.tile_seq; a.tile_q0 = d + L.tile_q0; a.n_tiles = L.n_qtiles;
      a.qtile = LAT_QTILE; a.n_splits = 1;
    } else {
      a.n_tiles = n; a.qtile = 1;
      a.n_splits = latent_attn_splits(n, s.heads, L.max_len, h->sm_count);
      while (a.n_splits > 1 && (size_t)T * s.heads * a.n_splits * (s.kv_rank + 2) > w.attn_ws_floats) a.n_splits--;
    }
    {
      ProfScope ps(h, NVLLM_K_ROPE_KV, (double)T * y.n_in * 4 + (double)T * (y.q_rank_p * asz + own * y.Dk * kvsz), 0,
                   (double)T * y.n_in * 4 * (pin.S - 1));
      LAUNCH(h, launch_latent_prep(st, h->adt, h->kvdt, a));
    }
    const int qn = s.heads * y.Dk;
    Pending pq;
    if ((rc = run_gemm(h, w.lat_cq, y.q_rank_p, y.w_q, T, qn, y.q_rank_p, 1.f, w.ws_a, w.ws_a_floats, qn, &pq)))
      return rc;
    a.q_p = pq.p; a.q_S = pq.S; a.q_stride = pq.stride; a.q_ld = qn;
    {
      ProfScope ps(h, NVLLM_K_ROPE_KV, (double)T * qn * (4 + asz), 0, (double)T * qn * 4 * (pq.S - 1));
      LAUNCH(h, launch_latent_q(st, h->adt, a));
    }
    {
      // algorithmic: every cached row of the contexts once; flops: scores over Dk, sums over R
      const double bytes = (double)L.sum_len * y.Dk * kvsz;
      const double flops = 2.0 * s.heads * (y.Dk + s.kv_rank) * L.attn_pairs;
      ProfScope ps(h, L.prefill ? NVLLM_K_ATTN_PREFILL : NVLLM_K_ATTN_DECODE, bytes, flops,
                   (double)T * (qn + y.ovr_p) * asz);
      LAUNCH(h, launch_latent_attn(st, h->adt, h->kvdt, a));
      if (a.n_splits > 1) h->launches++;
    }
    Pending pa;
    if ((rc = run_gemm(h, w.lat_o, y.ovr_p, y.w_ov, T, H, y.ovr_p, 1.f, w.ws_b, w.ws_b_floats, H, &pa))) return rc;
    // ---- feed-forward on the same normed input
    Pending pm;
    if (s.mlp == NVLLM_MLP_DENSE) {
      const int ff = y.ff_p;  // padded with zero rows / columns: the gated unit of (0, 0) is 0
      Pending h1;
      h->glu_limit_cur = s.limit;
      rc = run_gemm(h, w.xn, H, y.w1, T, 2 * ff, H, 1.f, w.ws_a, w.ws_a_floats, 2 * ff, &h1, TC5_EPI_SWIGLU,
                    w.hbuf, ff, nullptr);
      h->glu_limit_cur = 0.f;
      if (rc) return rc;
      // steps of <= 8 rows: the gated unit is built inside the down projection's GEMV (one launch less)
      const char* gpre_env = getenv("NVLLM_GEMV_PRE");
      if (h1.S > 0 && T <= 8 && !(gpre_env && atoi(gpre_env) == 0)) {
        GemvPre ga{};
        ga.mode = 2; ga.hp = h1.p; ga.Sh = h1.S; ga.hstride = h1.stride; ga.hld = 2 * ff;
        ga.swiglu = 1; ga.glu_limit = s.limit;
        if ((rc = run_gemm(h, w.hbuf, ff, y.w2, T, H, ff, 1.f, w.ws_c, w.ws_b_floats, H, &pm, 0, nullptr, 0,
                           nullptr, nullptr, 0, 0.0, nullptr, nullptr, &ga)))
          return rc;
      } else {
        if (h1.S > 0) {
          ProfScope ps(h, NVLLM_K_ACT, (double)T * 2 * ff * 4 + (double)T * ff * asz, 0,
                       (double)T * 2 * ff * 4 * (h1.S - 1));
          LAUNCH(h, launch_act(st, h->adt, T, ff, h1.p, h1.S, h1.stride, nullptr, 1, w.hbuf, s.limit));
        }
        if ((rc = run_gemm(h, w.hbuf, ff, y.w2, T, H, ff, 1.f, w.ws_c, w.ws_b_floats, H, &pm))) return rc;
      }
    } else if (s.mlp == NVLLM_MLP_MOE) {
      if ((rc = run_moe_ffn(h, T, w.xn, s.experts, s.top, y.ff_p, s.limit, y.moe_in, y.moe_out, topk_w, &pm))) return rc;
    }
    if (pm.p) {
      p1 = pm;  // the expert combine can only be the first addend of the norm kernel
      p2 = pa;
    } else {
      p1 = pa;
      p2 = Pending();
    }
  }
  // final norm + LM head on the rows that were asked for: each sequence's last, then the extra ones
  if ((rc = run_norm(h, w.x, &p1, &p2, h->lnf_w, nullptr, w.xn_last, nullptr, d + L.last_row, n_out, nullptr,
                     h->block_style == NVLLM_LBLOCK_PARALLEL_PRENORM, row_m2)))
    return rc;
  Pending lg;
  if ((rc = run_gemm(h, w.xn_last, H, h->lm_head, n_out, h->V, H, h->logit_scale != 0.f ? h->logit_scale : 1.f, w.logits_p,
                     w.logits_p_floats, h->ldl, &lg, 0,
                     nullptr, 0, nullptr, nullptr, 0, (double)n_out * h->V * 4)))
    return rc;
  {
    ProfScope ps(h, NVLLM_K_MISC, (double)n_out * h->ldl * 8, 0, (double)n_out * h->ldl * 4 * (lg.S - 1));
    LAUNCH(h, launch_softcap(st, lg.p, lg.S, lg.stride, (size_t)n_out * h->ldl, h->logit_softcap, w.logits));
  }
  const float* d_temp = reinterpret_cast<const float*>(d + L.temperature);
  const float* d_uni = reinterpret_cast<const float*>(d + L.uniforms);
  {
    ProfScope ps(h, NVLLM_K_SAMPLE, (double)n * h->V * 4, 0);
    LAUNCH(h, launch_sample(st, w.logits, h->ldl, h->V, n, d_temp, d_uni, w.out_tokens, w.amax, w.amax_ticket, 0));
    if (h->filters_active() && h->hist_n == n)
      LAUNCH(h, launch_sample_filtered(st, w.logits, h->ldl, h->V, n, 0, d_temp, d_uni, h->d_hist + (n + 1),
                                       h->d_hist, h->top_p, h->top_k, h->rep_penalty, h->d_probs, w.out_tokens));
  }
  h->ws.logits_final = w.logits;
  return NVLLM_OK;
}

}  // namespace nvllm

using namespace nvllm;

extern "C" int nvllm_create_layered(const nvllm_layered_config* c, const nvllm_layer_spec* layers,
                                    nvllm_handle** out) {
  if (!c || !layers || !out) return set_err(nullptr, NVLLM_ERR_INVALID, "null argument");
  *out = nullptr;
  if (c->abi_version != NVLLM_ABI_VERSION)
    return set_err(nullptr, NVLLM_ERR_INVALID, "abi_version %d != %d", c->abi_version, NVLLM_ABI_VERSION);
  auto bad = [&](int l, const char* what) {
    return set_err(nullptr, NVLLM_ERR_INVALID, "invalid config (layer %d): %s", l, what);
  };
  if (c->vocab_size <= 0 || c->hidden <= 0 || c->num_layers <= 0) return bad(-1, "non-positive dimension");
  if (c->hidden % 8) return bad(-1, "width must be a multiple of 8");
  if (c->precision != NVLLM_PREC_FP32 && c->precision != NVLLM_PREC_BF16) return bad(-1, "precision");
  const bool pre_style = c->block_style == NVLLM_LBLOCK_SEQUENTIAL_PRENORM;
  const bool has_loop = c->loop_times >= 1 && c->loop_stop > c->loop_start;
  if (has_loop && (!pre_style || c->loop_start < 0 || c->loop_stop > c->num_layers))
    return bad(-1, "a repeated run of layers needs the sequential pre-norm block style and 0 <= start < stop <= layers");
  if ((c->norm_groups > 1 || c->embed_norm || c->mixer_conv > 1 || c->side_dim > 0) && !pre_style)
    return bad(-1, "grouped norms, a normed embedding, the convolution on the mixers' input and the per-layer token input need the sequential pre-norm block style");
  if (c->norm_groups > 64 || (c->norm_groups > 1 && c->hidden % c->norm_groups)) return bad(-1, "norm groups must divide the width (at most 64)");
  if (c->mixer_conv < 0 || c->mixer_conv > 8) return bad(-1, "convolution on the mixers' input: at most 8 taps");
  if (c->side_dim < 0) return bad(-1, "negative side_dim");
  int vmix_first = -1;
  for (int l = 0; l < c->num_layers; l++) {
    const nvllm_layer_spec& s = layers[l];
    const bool seq_style = c->block_style == NVLLM_LBLOCK_SEQUENTIAL_POSTNORM;
    if (s.mixer == NVLLM_MIXER_ATTENTION || s.mixer == NVLLM_MIXER_MAMBA2) {
      if (!pre_style) return bad(l, "attention with options / Mamba-2 need the sequential pre-norm block style");
      if (s.heads <= 0 || s.vdim <= 0) return bad(l, "non-positive mixer size");
      if (s.mixer == NVLLM_MIXER_ATTENTION) {
        if (s.kv_heads <= 0 || s.dim <= 0 || s.heads % s.kv_heads) return bad(l, "heads must be a multiple of kv_heads");
        if (s.vdim > 512 || s.dim > 1024) return bad(l, "attention: dim <= 1024, vdim <= 512");
        if (s.qk_norm != 0 && s.qk_norm != 1 && s.qk_norm != 3) return bad(l, "attention: qk_norm 0, 1 (per head) or 3 (per head, weighted)");
        if (s.rot_dims < 0 || s.rot_dims > s.dim || (s.rot_dims & 1)) return bad(l, "rotated entries must be even and <= dim");
        if (s.rot_piecewise && !(s.rot_factor > 0.f && s.rot_fast != s.rot_slow)) return bad(l, "piecewise frequency scaling: factor > 0, two different bounds");
        if (s.qtemp_coef > 0.f && s.qtemp_every <= 0) return bad(l, "query temperature: a positive step");
        if (s.sink_learned && !s.sink) return bad(l, "a learned sink needs sink = 1");
        if (s.v_mix) {
          if (vmix_first < 0) vmix_first = l;
          else if (layers[vmix_first].kv_heads != s.kv_heads || layers[vmix_first].vdim != s.vdim)
            return bad(l, "layers that mix values must have the first such layer's kv_heads and vdim");
        }
      } else {
        if (s.state <= 0 || s.state > LINREC_MAX_DIM) return bad(l, "Mamba-2: 0 < state <= 256");
        if (s.ssm_groups <= 0 || s.heads % s.ssm_groups) return bad(l, "Mamba-2: heads must be a multiple of the groups");
        if (s.heads > 256) return bad(l, "Mamba-2: at most 256 heads");
        if (s.norm_groups <= 0 || s.norm_groups > 64 || (s.heads * s.vdim) % s.norm_groups) return bad(l, "Mamba-2: norm groups must divide heads * vdim (at most 64)");
        if (s.conv < 1 || s.conv > 8) return bad(l, "convolution taps 1..8");
      }
      if (s.mlp != NVLLM_MLP_NONE && s.mlp != NVLLM_MLP_MOE) return bad(l, "pre-norm blocks: feed-forward none or mixture of experts");
      if (s.mlp == NVLLM_MLP_MOE) {
        if (s.act != NVLLM_FFN_SWIGLU) return bad(l, "these blocks take gated experts W_down (silu(W_gate h) * W_up h)");
        if (s.ff <= 0 || s.experts <= 0 || s.experts > 256 || s.top <= 0 || s.top > 32 || s.top > s.experts)
          return bad(l, "ff > 0, experts 1..256, top 1..32");
        const int g = s.groups > 0 ? s.groups : 1, keep = s.groups > 0 ? s.keep_groups : 1;
        if (s.experts % g || keep <= 0 || keep > g || keep * (s.experts / g) < s.top)
          return bad(l, "expert groups must divide the experts and the kept groups must hold `top` experts");
      }
      continue;
    }
    if (s.mixer == NVLLM_MIXER_GLA || s.mixer == NVLLM_MIXER_ATTN_TMIX) {
      if (!pre_style) return bad(l, "gated linear attention / attention + time mixing need the sequential pre-norm block style");
      if (s.heads <= 0 || s.dim <= 0 || s.vdim <= 0 || s.lowrank <= 0) return bad(l, "non-positive mixer size");
      if (s.mixer == NVLLM_MIXER_GLA) {
        if (s.dim > LINREC_MAX_DIM) return bad(l, "gated linear attention: dim <= 256");
        if (!(s.tau > 0.f)) return bad(l, "gated linear attention: tau must be positive");
      } else {
        if (s.kv_heads <= 0 || s.heads % s.kv_heads) return bad(l, "heads must be a multiple of kv_heads");
        if (s.heads2 <= 0 || s.dim2 <= 0 || s.dim2 > LINREC_MAX_DIM) return bad(l, "time mixing: heads2 > 0, 0 < dim2 <= 256");
        if (s.conv < 1 || s.conv > 8) return bad(l, "convolution taps 1..8");
        if (s.vdim > 512 || s.dim > 1024) return bad(l, "attention: dim <= 1024, vdim <= 512");
        if (s.rot_dims < 0 || s.rot_dims > s.dim || (s.rot_dims & 1)) return bad(l, "rotated entries must be even and <= dim");
        if (s.chunk < 0 || s.window < 0 || (s.chunk > 0 && s.window > 0)) return bad(l, "a chunked mask or a window, not both");
        if (s.qk_norm != 2) return bad(l, "attention + time mixing: qk_norm = 2 (whole-row norms with weights)");
      }
      if (s.mlp != NVLLM_MLP_NONE && s.mlp != NVLLM_MLP_MOE) return bad(l, "pre-norm blocks: feed-forward none or mixture of experts");
      if (s.mlp == NVLLM_MLP_MOE) {
        if (s.act != NVLLM_FFN_RELU2 || !s.route_sigmoid || !s.weight_on_input)
          return bad(l, "pre-norm blocks: squared-ReLU experts chosen by sigmoid scores, weight on the input");
        if (s.ff <= 0 || s.experts <= 0 || s.experts > 256 || s.top <= 0 || s.top > 32 || s.top > s.experts || s.shared_ff < 0)
          return bad(l, "ff > 0, experts 1..256, top 1..32");
      }
      continue;
    }
    if (pre_style) return bad(l, "this mixer has no sequential pre-norm form");
    if (s.mixer == NVLLM_MIXER_WINDOW_ATTENTION || s.mixer == NVLLM_MIXER_DELTA) {
      if (!seq_style) return bad(l, "window attention / delta rule mixers need the sequential post-norm block style");
      if (s.heads <= 0 || s.kv_heads <= 0 || s.dim <= 0 || s.vdim <= 0) return bad(l, "non-positive mixer size");
      if (s.heads % s.kv_heads) return bad(l, "heads must be a multiple of kv_heads");
      if (s.mixer == NVLLM_MIXER_DELTA) {
        if (s.conv < 1 || s.conv > 8) return bad(l, "convolution taps 1..8");
        if (s.dim > 512 || s.vdim > 4096 || s.heads > 256) return bad(l, "delta rule: dim <= 512, vdim <= 4096, heads <= 256");
        if (s.kv_from >= 0) return bad(l, "a delta rule layer has no cache to borrow");
      } else {
        if (s.window < 0) return bad(l, "negative window");
        if (s.vdim > 512 || s.dim > 1024) return bad(l, "window attention: dim <= 1024, vdim <= 512");
        if (s.kv_from >= 0) {
          if (s.kv_from >= l) return bad(l, "kv_from must name an earlier layer");
          const nvllm_layer_spec& j = layers[s.kv_from];
          if (j.mixer != NVLLM_MIXER_WINDOW_ATTENTION || j.kv_from >= 0)
            return bad(l, "kv_from must name an attention layer with projections of its own");
          if (j.kv_heads != s.kv_heads || j.dim != s.dim || j.vdim != s.vdim) return bad(l, "kv_from layer has other cache sizes");
        }
      }
      if (s.mlp != NVLLM_MLP_NONE && s.mlp != NVLLM_MLP_DENSE) return bad(l, "unknown feed-forward kind");
      if (s.mlp == NVLLM_MLP_DENSE && (s.ff <= 0 || s.act != NVLLM_FFN_RELU2)) return bad(l, "dense feed-forward: ff > 0, squared-ReLU activation");
      continue;
    }
    if (s.mixer != NVLLM_MIXER_LATENT_ATTENTION) return bad(l, "unknown mixer kind");
    if (seq_style) return bad(l, "latent attention needs the parallel pre-norm block style");
    if (s.heads <= 0 || s.dim <= 0 || s.rot_dim <= 0 || s.vdim <= 0 || s.kv_rank <= 0 || s.q_rank <= 0)
      return bad(l, "non-positive mixer size");
    if (s.kv_rank > 512) return bad(l, "kv_rank above 512");
    if (s.rot_dims < 2 || s.rot_dims > s.rot_dim || (s.rot_dims & 1)) return bad(l, "rotated entries must be even and <= rot_dim");
    if (s.kv_from >= 0) {
      if (s.kv_from >= l) return bad(l, "kv_from must name an earlier layer");
      const nvllm_layer_spec& j = layers[s.kv_from];
      if (j.kv_from >= 0) return bad(l, "kv_from must name a layer with its own down projection");
      if (j.kv_rank != s.kv_rank || j.rot_dim != s.rot_dim) return bad(l, "kv_from layer has other cache sizes");
    }
    if (s.mlp < NVLLM_MLP_NONE || s.mlp > NVLLM_MLP_MOE) return bad(l, "unknown feed-forward kind");
    if (s.mlp != NVLLM_MLP_NONE && s.ff <= 0) return bad(l, "ff must be positive");
    if (s.mlp != NVLLM_MLP_NONE && !(s.limit > 0.f)) return bad(l, "limit must be positive");
    if (s.mlp == NVLLM_MLP_MOE) {
      if (s.experts <= 0 || s.experts > 256 || s.top <= 0 || s.top > 32 || s.top > s.experts)
        return bad(l, "experts 1..256, top 1..32");
      const int g = s.groups > 0 ? s.groups : 1, keep = s.groups > 0 ? s.keep_groups : 1;
      if (s.experts % g || keep <= 0 || keep > g || keep * (s.experts / g) < s.top)
        return bad(l, "expert groups must divide the experts and the kept groups must hold `top` experts");
    }
  }
  cudaError_t e = cudaSetDevice(c->device);
  if (e != cudaSuccess)
    return set_err(nullptr, NVLLM_ERR_CUDA, "cudaSetDevice(%d): %s (no CPU fallback exists)", c->device,
                   cudaGetErrorString(e));
  cudaDeviceProp prop;
  e = cudaGetDeviceProperties(&prop, c->device);
  if (e != cudaSuccess) return set_err(nullptr, NVLLM_ERR_CUDA, "cudaGetDeviceProperties: %s", cudaGetErrorString(e));
  if (prop.major != 10)
    return set_err(nullptr, NVLLM_ERR_CUDA, "device %d is sm_%d%d; this library contains sm_100a code only",
                   c->device, prop.major, prop.minor);
  if (const char* env = getenv("NVLLM_PDL")) set_pdl_enabled(atoi(env) != 0);
  nvllm_handle* h = new nvllm_handle();
  h->layered = true;
  nvllm_config& g = h->cfg;  // what nvllm_get_config reports; the uniform fields describe layer 0
  g.abi_version = NVLLM_ABI_VERSION;
  g.vocab_size = c->vocab_size; g.hidden = c->hidden; g.num_layers = c->num_layers;
  g.num_heads = layers[0].heads; g.num_kv_heads = 1; g.head_dim = layers[0].dim + layers[0].rot_dim;
  g.max_seq_len = 1 << 30;
  g.attention_type = NVLLM_ATTN_MQA; g.norm_type = NVLLM_NORM_LAYER; g.position_type = NVLLM_POS_ROPE;
  g.activation_type = NVLLM_ACT_SWIGLU; g.block_style = NVLLM_BLOCK_PARALLEL;
  if (c->block_style == NVLLM_LBLOCK_SEQUENTIAL_POSTNORM) {
    g.num_kv_heads = layers[0].kv_heads; g.head_dim = layers[0].dim;
    g.attention_type = NVLLM_ATTN_GQA; g.norm_type = NVLLM_NORM_RMS; g.position_type = NVLLM_POS_NONE;
    g.activation_type = NVLLM_ACT_GELU; g.block_style = NVLLM_BLOCK_SEQUENTIAL;
    g.tied_embedding = c->tied_head;
  }
  g.norm_eps = c->norm_eps; g.embedding_multiplier = c->embedding_scale;
  g.precision = c->precision;
  g.num_kv_blocks = c->num_kv_blocks > 0 ? c->num_kv_blocks : 1024;
  g.max_num_seqs = c->max_num_seqs > 0 ? c->max_num_seqs : 512;
  g.max_batched_tokens = c->max_batched_tokens > 0 ? c->max_batched_tokens : 16384;
  g.tp_size = 1; g.device = c->device;
  h->dev = c->device;
  h->sm_count = prop.multiProcessorCount;
  h->wdt = h->adt = h->kvdt = (c->precision == NVLLM_PREC_BF16) ? DT_BF16 : DT_F32;
  h->H = c->hidden; h->V = c->vocab_size; h->L = c->num_layers;
  h->ldl = (int)up8(h->V); h->Vl = h->ldl; h->Vl_valid = h->V;
  h->parallel = true;
  h->num_blocks = g.num_kv_blocks;
  h->logit_softcap = c->logit_softcap;
  h->block_style = c->block_style;
  h->position_kind = c->position;
  h->norm_offset = c->norm_offset;
  h->norm_groups = c->norm_groups > 1 ? c->norm_groups : 0;
  h->mixer_conv = c->mixer_conv > 1 ? c->mixer_conv : 0;
  h->side_dim = c->side_dim;
  h->side_p = (int)up8((size_t)c->side_dim);
  h->logit_scale = c->logit_scale;
  if (pre_style) {
    g.num_kv_heads = layers[0].kv_heads > 0 ? layers[0].kv_heads : layers[0].heads; g.head_dim = layers[0].dim;
    g.attention_type = NVLLM_ATTN_GQA; g.norm_type = NVLLM_NORM_RMS; g.position_type = NVLLM_POS_ROPE;
    g.activation_type = NVLLM_ACT_GELU; g.block_style = NVLLM_BLOCK_SEQUENTIAL;
    if (has_loop) {
      h->loop_start = c->loop_start; h->loop_stop = c->loop_stop; h->loop_times = c->loop_times;
    }
  }
  h->num_state_slots = c->num_state_slots > 0 ? c->num_state_slots : g.max_num_seqs;
  h->spec_enabled = 0;  // the speculative next step is keyed on the uniform models' shapes
  if (const char* env = getenv("NVLLM_SKIP")) h->skip_mask = (unsigned)strtoul(env, nullptr, 0);
  auto fail = [&](cudaError_t ce, const char* what) {
    int code = (ce == cudaErrorMemoryAllocation) ? NVLLM_ERR_NOMEM : NVLLM_ERR_CUDA;
    set_err(nullptr, code, "%s: %s", what, cudaGetErrorString(ce));
    nvllm_destroy(h);
    return code;
  };
  if ((e = cudaStreamCreateWithFlags(&h->stream, cudaStreamNonBlocking)) != cudaSuccess) return fail(e, "cudaStreamCreate");
  if ((e = cudaEventCreate(&h->ev0)) != cudaSuccess) return fail(e, "cudaEventCreate");
  if ((e = cudaEventCreate(&h->ev1)) != cudaSuccess) return fail(e, "cudaEventCreate");
  const int W = h->H;
  const size_t wsz = dt_size(h->wdt);
  // zero-filled: inner extents are padded to 8 and the padding must stay zero
  auto alloc = [&](void** p, size_t bytes) -> cudaError_t {
    bytes = (bytes + 255) / 256 * 256;
    cudaError_t ce = cudaMalloc(p, bytes);
    if (ce == cudaSuccess) ce = cudaMemsetAsync(*p, 0, bytes, h->stream);
    if (ce == cudaSuccess) h->weight_bytes += bytes;
    return ce;
  };
#define AL(ptr, bytes) \
  if ((e = alloc((void**)&(ptr), (size_t)(bytes))) != cudaSuccess) return fail(e, "cudaMalloc(weights)");
  AL(h->wte, (size_t)h->V * W * wsz);
  if (c->tied_head) {
    h->lm_head = h->wte;  // [V, W] is already K-contiguous: the table itself is the head
  } else {
    AL(h->lm_head, (size_t)h->V * W * wsz);
    h->lm_head_owned = true;
  }
  AL(h->lnf_w, (size_t)W * 4);
  if (c->embed_norm) AL(h->embed_norm_w, (size_t)W * 4);
  if (h->side_dim > 0) AL(h->side_embed, (size_t)h->V * h->L * h->side_dim * wsz);
  h->ll.resize(h->L);
  int qkv_cols = 0, q_cols = 0, win_qtile = 0;
  for (int l = 0; l < h->L; l++) {
    ListedLayer& y = h->ll[l];
    y.s = layers[l];
    const nvllm_layer_spec& s = y.s;
    if (pre_style && h->mixer_conv) AL(y.canon_w, (size_t)W * h->mixer_conv * 4);
    if (pre_style && h->side_dim > 0) {
      AL(y.side_gate, (size_t)h->side_p * W * wsz);
      AL(y.side_proj, (size_t)W * h->side_p * wsz);
      AL(y.side_norm, (size_t)W * 4);
      qkv_cols = std::max(qkv_cols, h->side_p);
    }
    if (s.mixer == NVLLM_MIXER_ATTENTION || s.mixer == NVLLM_MIXER_MAMBA2) {
      const int hv = s.heads * s.vdim;
      y.ov_p = (int)up8((size_t)hv);
      y.ff_p = (int)up8((size_t)std::max(s.ff, 0));
      AL(y.post1_w, (size_t)W * 4);
      if (s.mixer == NVLLM_MIXER_ATTENTION) {
        y.n_q = s.heads * s.dim; y.n_k = s.kv_heads * s.dim; y.n_v = s.kv_heads * s.vdim;
        y.n_in = y.n_q + y.n_k + y.n_v + (s.head_gate ? s.heads : 0);  // Q | K | V | head gates
        AL(y.w_in, (size_t)y.n_in * W * wsz);
        if (s.qk_norm == 3) {
          AL(y.qnorm_w, (size_t)s.dim * 4);
          AL(y.knorm_w, (size_t)s.dim * 4);
        }
        if (s.v_mix) {
          AL(y.vmix, 4);
          y.vmix_first = l == vmix_first;
        }
        if (s.sink_learned) AL(y.sink_w, (size_t)s.heads * 4);
        if (s.head_temp) AL(y.head_temp, (size_t)s.heads * 4);
        if (s.rot_dims > 0) {
          for (size_t r = 0; r < h->ropes.size(); r++) {
            const RopeTable& t = h->ropes[r];
            if (t.base == (double)s.rot_base && t.dims == s.rot_dims && t.factor == (double)s.rot_factor &&
                t.original == (double)s.rot_original && t.fast == (double)s.rot_fast && t.slow == (double)s.rot_slow &&
                t.piecewise == (s.rot_piecewise != 0))
              y.rope = (int)r;
          }
          if (y.rope < 0) {
            RopeTable rt;
            rt.base = s.rot_base; rt.dims = s.rot_dims;
            rt.factor = s.rot_factor; rt.original = s.rot_original; rt.fast = s.rot_fast; rt.slow = s.rot_slow;
            rt.piecewise = s.rot_piecewise != 0;
            y.rope = (int)h->ropes.size();
            h->ropes.push_back(rt);
          }
        }
        // (a model whose attention layers all fit the tcgen05 kernel gets its tiles of 128 queries)
        const int qt = attention_on_tc5(h, s) ? 128 : winattn_qtile(h->adt, h->kvdt, s.dim, s.vdim);
        win_qtile = win_qtile ? std::min(win_qtile, qt) : qt;
        q_cols = std::max(q_cols, std::max(y.n_q, y.ov_p));
      } else {
        const int gn = s.ssm_groups * s.state;
        y.conv_ch = hv + 2 * gn;
        y.n_in = 2 * hv + 2 * gn + s.heads;  // z | x | B | C | dt
        AL(y.w_in, (size_t)y.n_in * W * wsz);
        AL(y.conv_w, (size_t)y.conv_ch * s.conv * 4);
        AL(y.conv_b, (size_t)y.conv_ch * 4);
        AL(y.dt_bias, (size_t)s.heads * 4);
        AL(y.a_log, (size_t)s.heads * 4);
        AL(y.d_skip, (size_t)s.heads * 4);
        AL(y.onorm_w, (size_t)hv * 4);
        q_cols = std::max(q_cols, y.ov_p);
      }
      AL(y.w_o, (size_t)W * y.ov_p * wsz);
      if (s.mlp == NVLLM_MLP_MOE) {
        AL(y.post2_w, (size_t)W * 4);
        AL(y.router, (size_t)s.experts * W * 4);
        if (s.route_correction) AL(y.route_corr, (size_t)s.experts * 4);
        AL(y.moe_in, (size_t)s.experts * 2 * y.ff_p * W * wsz);
        AL(y.moe_out, (size_t)s.experts * W * y.ff_p * wsz);
        h->moe = true;
        h->E = std::max(h->E, s.experts);
        h->topk = std::max(h->topk, s.top);
        h->F = std::max(h->F, y.ff_p);
      }
      qkv_cols = std::max(qkv_cols, y.n_in);
      h->nh = std::max(h->nh, s.heads);
      h->hd = std::max(h->hd, s.vdim);
      continue;
    }
    if (s.mixer == NVLLM_MIXER_GLA || s.mixer == NVLLM_MIXER_ATTN_TMIX) {
      const int hd = s.heads * s.dim, hv = s.heads * s.vdim;
      y.ov_p = (int)up8((size_t)hv);
      y.ff_p = (int)up8((size_t)std::max(s.ff, 0));
      AL(y.post1_w, (size_t)W * 4);
      if (s.mixer == NVLLM_MIXER_GLA) {
        y.n_in = 2 * hd + 2 * hv + s.lowrank;  // q | k | v | gate | decay inner
        AL(y.w_in, (size_t)y.n_in * W * wsz);
        AL(y.lr_w2, (size_t)hd * s.lowrank * 4);
        AL(y.lr_b, (size_t)hd * 4);
        AL(y.onorm_w, (size_t)s.vdim * 4);
        q_cols = std::max(q_cols, y.ov_p);
      } else {
        const int hd2 = s.heads2 * s.dim2;
        y.n_q = hd; y.n_k = s.kv_heads * s.dim; y.n_v = s.kv_heads * s.vdim;
        y.conv_ch = y.n_q + y.n_k + y.n_v;
        y.n_in = y.conv_ch + (s.out_gate ? hv : 0);  // Q | K | V | gate
        AL(y.w_in, (size_t)y.n_in * W * wsz);
        AL(y.bias_in, (size_t)y.n_in * 4);
        AL(y.o_bias, (size_t)W * 4);
        AL(y.qnorm_w, (size_t)y.n_q * 4);
        AL(y.knorm_w, (size_t)y.n_k * 4);
        AL(y.conv_w, (size_t)y.conv_ch * s.conv * 4);
        // time mixing: five projections, each on its own input, into one row of partials
        int off = 0;
        for (int i = 0; i < 5; i++) {
          y.seg2[i] = off;
          off += (int)up8((size_t)(i < 4 ? hd2 : s.lowrank));
        }
        y.n_in2 = off;
        y.ov2_p = (int)up8((size_t)hd2);
        AL(y.w_in2, (size_t)y.n_in2 * W * wsz);
        AL(y.w_o2, (size_t)W * y.ov2_p * wsz);
        AL(y.lr_w2, (size_t)hd2 * s.lowrank * 4);
        AL(y.lr_b, (size_t)hd2 * 4);
        AL(y.mu, (size_t)5 * W * 4);
        AL(y.bonus, (size_t)hd2 * 4);
        AL(y.onorm_w, (size_t)hd2 * 4);
        if (s.rot_dims > 0) {
          for (size_t r = 0; r < h->ropes.size(); r++) {
            const RopeTable& t = h->ropes[r];
            if (t.base == (double)s.rot_base && t.dims == s.rot_dims && t.factor == (double)s.rot_factor &&
                t.original == (double)s.rot_original && t.fast == (double)s.rot_fast && t.slow == (double)s.rot_slow)
              y.rope = (int)r;
          }
          if (y.rope < 0) {
            RopeTable rt;
            rt.base = s.rot_base; rt.dims = s.rot_dims;
            rt.factor = s.rot_factor; rt.original = s.rot_original; rt.fast = s.rot_fast; rt.slow = s.rot_slow;
            y.rope = (int)h->ropes.size();
            h->ropes.push_back(rt);
          }
        }
        const int qt = winattn_qtile(h->adt, h->kvdt, s.dim, s.vdim);
        win_qtile = win_qtile ? std::min(win_qtile, qt) : qt;
        qkv_cols = std::max(qkv_cols, y.n_in2);
        q_cols = std::max(q_cols, std::max(y.n_q, std::max(y.ov_p, y.ov2_p)));
        h->nh = std::max(h->nh, s.heads2);
      }
      AL(y.w_o, (size_t)W * y.ov_p * wsz);
      if (s.mlp == NVLLM_MLP_MOE) {
        AL(y.post2_w, (size_t)W * 4);
        AL(y.router, (size_t)s.experts * W * 4);
        AL(y.moe_in, (size_t)s.experts * y.ff_p * W * wsz);
        AL(y.moe_out, (size_t)s.experts * W * y.ff_p * wsz);
        h->moe = true;
        h->E = std::max(h->E, s.experts);
        h->topk = std::max(h->topk, s.top);
        h->F = std::max(h->F, y.ff_p);
        if (s.shared_ff > 0) {
          y.sff_p = (int)up8((size_t)s.shared_ff);
          AL(y.w1, (size_t)y.sff_p * W * wsz);
          AL(y.w2, (size_t)W * y.sff_p * wsz);
          AL(y.sh_gate, (size_t)W * 4);
          h->F = std::max(h->F, y.sff_p);
          qkv_cols = std::max(qkv_cols, y.sff_p);
        }
      }
      qkv_cols = std::max(qkv_cols, y.n_in);
      h->nh = std::max(h->nh, s.heads);
      h->hd = std::max(h->hd, s.vdim);
      continue;
    }
    if (s.mixer != NVLLM_MIXER_LATENT_ATTENTION) {
      const bool delta = s.mixer == NVLLM_MIXER_DELTA;
      const int own = s.kv_from < 0;
      y.ov_p = (int)up8((size_t)s.heads * s.vdim);
      y.ff_p = (int)up8((size_t)std::max(s.ff, 0));
      y.pool = own ? l : s.kv_from;
      if (delta) {
        y.n_q = y.n_k = s.kv_heads * s.dim;
        y.n_v = s.heads * s.vdim;
        y.conv_ch = y.n_q + y.n_k + y.n_v;
        y.n_in = y.conv_ch + 2 * s.heads + s.heads * s.vdim;  // q | k | v | beta | decay | gate
        y.state_off = h->state_slot_floats;
        y.tail_off = y.state_off + (size_t)s.heads * s.dim * s.vdim;
        h->state_slot_floats = y.tail_off + (size_t)(s.conv - 1) * y.conv_ch;
        AL(y.conv_w, (size_t)y.conv_ch * s.conv * 4);
        AL(y.a_log, (size_t)s.heads * 4);
        AL(y.dt_bias, (size_t)s.heads * 4);
        AL(y.onorm_w, (size_t)s.vdim * 4);
      } else {
        y.n_q = s.heads * s.dim;
        y.n_k = own ? s.kv_heads * s.dim : 0;
        y.n_v = own ? s.kv_heads * s.vdim : 0;
        y.n_in = y.n_q + y.n_k + y.n_v;
        // every prefill tile list of the step is built for one query-tile size: the smallest any layer wants
        const int qt = winattn_qtile(h->adt, h->kvdt, s.dim, s.vdim);
        win_qtile = win_qtile ? std::min(win_qtile, qt) : qt;
      }
      AL(y.post1_w, (size_t)W * 4);
      AL(y.w_in, (size_t)y.n_in * W * wsz);
      AL(y.w_o, (size_t)W * y.ov_p * wsz);
      if (s.mlp == NVLLM_MLP_DENSE) {
        AL(y.post2_w, (size_t)W * 4);
        AL(y.w1, (size_t)y.ff_p * W * wsz);
        AL(y.w2, (size_t)W * y.ff_p * wsz);
        h->F = std::max(h->F, y.ff_p);
      }
      qkv_cols = std::max(qkv_cols, std::max(y.n_in, y.ff_p));
      q_cols = std::max(q_cols, std::max(y.n_q, y.ov_p));
      h->nh = std::max(h->nh, s.heads);
      h->hd = std::max(h->hd, s.vdim);
      continue;
    }
    y.Dk = s.kv_rank + s.rot_dim;
    y.n_in = s.q_rank + (s.kv_from < 0 ? y.Dk : 0) + s.heads;
    y.q_cols = s.heads * (s.dim + s.rot_dim);
    y.q_rank_p = (int)up8(s.q_rank);
    y.ov_p = (int)up8((size_t)s.heads * s.vdim);
    y.ovr_p = (int)up8((size_t)s.heads * s.kv_rank);
    y.ff_p = (int)up8((size_t)std::max(s.ff, 0));
    y.pool = s.kv_from < 0 ? l : s.kv_from;
    for (size_t r = 0; r < h->ropes.size(); r++)
      if (h->ropes[r].base == (double)s.rot_base && h->ropes[r].dims == s.rot_dims) y.rope = (int)r;
    if (y.rope < 0) {
      RopeTable rt;
      rt.base = s.rot_base;
      rt.dims = s.rot_dims;
      y.rope = (int)h->ropes.size();
      h->ropes.push_back(rt);
    }
    AL(y.norm_w, (size_t)W * 4);
    AL(y.w_in, (size_t)y.n_in * W * wsz);
    AL(y.dq_norm, (size_t)s.q_rank * 4);
    if (s.kv_from < 0) AL(y.dkv_norm, (size_t)s.kv_rank * 4);
    AL(y.w_uq, (size_t)y.q_cols * y.q_rank_p * wsz);
    AL(y.w_uk, (size_t)s.heads * s.dim * s.kv_rank * wsz);
    AL(y.w_uv, (size_t)s.heads * s.vdim * s.kv_rank * wsz);
    AL(y.w_o, (size_t)W * y.ov_p * wsz);
    AL(y.w_q, (size_t)s.heads * y.Dk * y.q_rank_p * wsz);
    AL(y.w_ov, (size_t)W * y.ovr_p * wsz);
    if (s.mlp == NVLLM_MLP_DENSE) {
      AL(y.w1, (size_t)2 * y.ff_p * W * wsz);
      AL(y.w2, (size_t)W * y.ff_p * wsz);
      qkv_cols = std::max(qkv_cols, 2 * y.ff_p);
      h->F = std::max(h->F, y.ff_p);
    } else if (s.mlp == NVLLM_MLP_MOE) {
      AL(y.router, (size_t)s.experts * W * 4);
      AL(y.moe_in, (size_t)s.experts * 2 * y.ff_p * W * wsz);
      AL(y.moe_out, (size_t)s.experts * W * y.ff_p * wsz);
      h->moe = true;
      h->E = std::max(h->E, s.experts);
      h->topk = std::max(h->topk, s.top);
      h->F = std::max(h->F, y.ff_p);
    }
    // extents the shared workspace is sized by (forward.cu ensure_workspace)
    qkv_cols = std::max(qkv_cols, std::max(y.n_in, s.heads * y.Dk));
    q_cols = std::max(q_cols, s.heads * y.Dk);
    h->nh = std::max(h->nh, s.heads);
    h->hd = std::max(h->hd, s.kv_rank);
  }
  if (pre_style) {
    // the executions of a step in order; every one gets its own piece of a state slot
    auto add_run = [&](int l, int pass_start) {
      LayerRun r;
      r.layer = l; r.pass_start = pass_start;
      const nvllm_layer_spec& s = h->ll[l].s;
      // every piece starts on a 16-byte boundary (the kernels read them with 16-byte loads)
      auto up4 = [](size_t n) { return (n + 3) / 4 * 4; };
      r.state_off = up4(h->state_slot_floats);
      if (h->mixer_conv) {  // tail of the convolution on the mixer's input, every layer
        r.canon_off = r.state_off;
        h->state_slot_floats = up4(r.canon_off + (size_t)(h->mixer_conv - 1) * W);
        r.state_off = h->state_slot_floats;
      }
      if (s.mixer == NVLLM_MIXER_ATTENTION) {
        // no state of its own
      } else if (s.mixer == NVLLM_MIXER_MAMBA2) {
        r.tail_off = up4(r.state_off + (size_t)s.heads * s.state * s.vdim);
        h->state_slot_floats = up4(r.tail_off + (size_t)(s.conv - 1) * h->ll[l].conv_ch);
      } else if (s.mixer == NVLLM_MIXER_GLA) {
        h->state_slot_floats = up4(r.state_off + (size_t)s.heads * s.dim * s.vdim);
      } else {
        r.tail_off = up4(r.state_off + (size_t)s.heads2 * s.dim2 * s.dim2);
        r.shift_off = up4(r.tail_off + (size_t)(s.conv - 1) * h->ll[l].conv_ch);
        h->state_slot_floats = up4(r.shift_off + (size_t)W);
      }
      h->runs.push_back(r);
    };
    const bool loop = h->loop_times >= 1 && h->loop_stop > h->loop_start;
    const int a0 = loop ? h->loop_start : 0, a1 = loop ? h->loop_stop : 0;
    for (int l = 0; l < a0; l++) add_run(l, -1);
    for (int t = 0; t < (loop ? h->loop_times : 0); t++)
      for (int l = a0; l < a1; l++) add_run(l, l == a0 ? t : -1);
    for (int l = a1; l < h->L; l++) add_run(l, -1);
    if (loop) AL(h->loop_step, (size_t)h->loop_times * W * 4);
  }
#undef AL
  h->attn_qtile = win_qtile ? win_qtile : latent_attn_qtile();
  h->F = std::max(h->F, 8);
  h->nkv = 1;
  h->qkv_cols = qkv_cols;
  h->q_cols = q_cols;
  h->w1_cols = 0;
  *out = h;
  return NVLLM_OK;
}

extern "C" int nvllm_set_named_weight(nvllm_handle* h, const char* name, int dtype, const void* host_data,
                                      const int64_t* shape, int ndim) {
  if (!h) return NVLLM_ERR_INVALID;
  return layered_set_weight(h, name, dtype, host_data, shape, ndim);
}
