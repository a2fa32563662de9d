// attention_window.cu — grouped-query attention over a sliding window of the paged K / V cache,
// with an optional sink in the softmax, for the layers of a model given as a list
// (nvllm_mixer_kind NVLLM_MIXER_WINDOW_ATTENTION).  Every size is a run-time argument.
//
//   q_h = norm(W_q x)_h, k_g = norm(W_k x)_g, v_g = (W_v x)_g      norm = x / sqrt(mean(x^2) + eps)
//   s_ij = scale * q_i . k_j   for 0 <= i - j < window (window = 0: every j <= i)
//   p_ij = exp(s_ij) / (sink + sum_j exp(s_ij))                    sink = 1: a key of score 0 without a value
//   o_i  = sum_j p_ij v_j;  query head h reads key / value head h / (H / G)
// Options of the same kernels (WinAttnArgs): chunk > 0 replaces the window by a chunked mask — i sees
// j <= i with i / chunk == j / chunk, chunks counted from position 0 of the sequence —, softcap > 0
// caps the score, s <- softcap * tanh(s / softcap), before the mask, and gate multiplies the
// normalised output element by element.  Both masks give every query a contiguous key range
// [first_key(i), i] whose start does not decrease with i, which is all the tile logic relies on.
//
//  * winattn_prep_kernel: epilogue of the fused projection [Q | K | V] — split-K sum, the
//    per-head norms, Q to the activation dtype, K / V rows into the layer's pools at slots[t]
//    (pool layout [block][kv head][256][dim] and [...][vdim], addressed through the block tables
//    like every other cache of the library).  A layer that borrows another layer's cache has no
//    K / V columns and writes nothing.
//  * winattn_kernel: fp32 arithmetic for any dim / vdim.  CTA = (query tile, head), 8 warps;
//    a warp owns two queries of a 16-query sub-tile, its lanes own the keys of a 32-key tile for
//    the scores and vdim / 32 output columns for the weighted sum.  Only the key tiles that a
//    query of the sub-tile can see are read: [first query - window + 1, last query].  The sink
//    is the initial state (max 0, denominator 1) of the running softmax.  Prefill steps come with
//    a tile list; without one every sequence has one query at seq_len - 1 (decode).
//  * winattn_mma_kernel (bf16, dim and vdim multiples of 16): the same on mma.sync m16n8k16,
//    64 queries x one head per CTA, K / V tiles of 64 keys by cp.async (double buffered).
#include <stdlib.h>

#include <algorithm>

#include "common.cuh"
#include "kernels.h"
#include "mma.cuh"

namespace nvllm {

namespace {
// first key position i sees
__device__ __forceinline__ int first_key(const WinAttnArgs& a, int i) {
  if (a.chunk > 0) return i / a.chunk * a.chunk;
  return a.window > 0 ? max(0, i - a.window + 1) : 0;
}
// cap * tanh(s / cap).  FAST (the bf16 kernels): tanh through one fast exponential and one fast
// division; its ABSOLUTE error is about cap * 3e-7 (the exponential's 2 ulp), which is what a
// softmax weight sees, far below the bf16 rounding of the weights.  Otherwise the library tanh.
template <bool FAST>
__device__ __forceinline__ float cap_score(float s, float cap) {
  if (!FAST) return cap * tanhf(s / cap);
  const float x = s * __fdividef(1.0f, cap);  // the reciprocal leaves the loop over the scores
  const float e = __expf(-2.0f * fabsf(x));
  return copysignf(cap * __fdividef(1.0f - e, 1.0f + e), x);
}
__device__ __forceinline__ float sum_slices(const float* __restrict__ p, int S, size_t stride) {
  float acc = 0.f;
  for (int s = 0; s < S; s++) acc += p[(size_t)s * stride];
  return acc;
}
// slope of the distance bias of a head: the score of key j for the query at i loses slope * (i - j)
__device__ __forceinline__ float head_slope(const WinAttnArgs& a, int head) {
  return a.slope_exp > 0.f ? exp2f(-a.slope_exp * (float)(head + 1) / (float)a.H) : 0.f;
}
// score of the sink (a term of the softmax denominator without a key or a value): 0 or learned per head
__device__ __forceinline__ float sink_score(const WinAttnArgs& a, int head) { return a.sink_w ? a.sink_w[head] : 0.f; }
__device__ __forceinline__ const float* gate_row(const WinAttnArgs& a, size_t row, int head, int vdim) {
  return a.gate ? a.gate + row * a.gate_ld + (a.gate_head ? head : head * vdim) : nullptr;
}
}  // namespace

// ------------------------------------------------------------------ projection epilogue
// grid (T, Y), 256 threads; a warp takes one head of the row at a time: H query heads, then (own
// cache only) G key heads and G value heads.  A head of up to 256 entries is read once into
// registers (the split-K slices summed on the way), normed and written; longer heads take two
// passes over the slices.
// WP_MAXV: entries per lane kept in registers
template <typename QT, typename KT, int WP_MAXV>
__global__ void __launch_bounds__(256) winattn_prep_kernel(WinAttnArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int n_qkv = a.H + (a.own_kv ? 2 * a.G : 0);
  const int n_items = n_qkv + (a.gate_out ? 1 : 0);
  const float* row = a.in_p + (size_t)t * a.in_ld;
  const int slot = a.slots[t];
  const int blk = slot / KV_BLOCK, off = slot % KV_BLOCK;
  const int rot = 2 * a.rot_half;
  const float* cs = a.rot_half ? a.cosT + (size_t)t * a.rot_half : nullptr;
  const float* sn = a.rot_half ? a.sinT + (size_t)t * a.rot_half : nullptr;
  // what multiplies every query of the row: grows with the position in steps of qtemp_every
  float qmul = 1.f;
  if (a.qtemp_coef > 0.f && a.qtemp_every > 0)
    qmul = 1.0f + a.qtemp_coef * logf((float)((a.positions[t] + 1) / a.qtemp_every) + 1.0f);
  const float lam = a.vmix ? a.vmix[0] : 0.f;
  for (int it = blockIdx.y * nw + warp; it < n_items; it += gridDim.y * nw) {
    if (it == n_qkv) {  // the heads' gates: sigmoid of the H columns after Q | K | V
      const float* gp = row + (a.H + (a.own_kv ? a.G : 0)) * a.dim + (a.own_kv ? a.G : 0) * a.vdim;
      for (int i = lane; i < a.H; i += 32)
        a.gate_out[(size_t)t * a.H + i] = 1.0f / (1.0f + expf(-sum_slices(gp + i, a.in_S, a.in_stride)));
      continue;
    }
    int col, n, kind;  // 0 = query, 1 = key, 2 = value
    if (it < a.H) { kind = 0; n = a.dim; col = it * a.dim; }
    else if (it < a.H + a.G) { kind = 1; n = a.dim; col = a.H * a.dim + (it - a.H) * a.dim; }
    else { kind = 2; n = a.vdim; col = (a.H + a.G) * a.dim + (it - a.H - a.G) * a.vdim; }
    // the rotation of (i, i + rot_half) pairs reaches across lanes: those heads take the second path
    const bool in_regs = n <= 32 * WP_MAXV && !(rot > 0 && !a.rot_pairs && kind != 2);
    float v[WP_MAXV];
#pragma unroll
    for (int c = 0; c < WP_MAXV; c++) v[c] = 0.f;
    float ss = 0.f;
    if (in_regs) {
#pragma unroll 4
      for (int sl = 0; sl < a.in_S; sl++) {
        const float* p = row + (size_t)sl * a.in_stride + col + lane;
#pragma unroll
        for (int c = 0; c < WP_MAXV; c++)
          if (lane + 32 * c < n) v[c] += p[32 * c];
      }
#pragma unroll
      for (int c = 0; c < WP_MAXV; c++) ss += v[c] * v[c];
    } else {
      for (int i = lane; i < n; i += 32) {
        const float x = sum_slices(row + col + i, a.in_S, a.in_stride);
        ss += x * x;
      }
    }
    // (a rotation leaves the sum of squares as it is: the norm's factor comes from the unrotated entries)
    float inv = 1.f;
    if (kind != 2 && a.qk_norm) inv = 1.0f / sqrtf(warp_sum(ss) / (float)n + a.eps);
    if (kind == 0) inv *= qmul * (a.head_scale ? a.head_scale[it] : 1.f);
    const float* nw_ = (kind == 2 || a.qk_norm != 3) ? nullptr : (kind == 0 ? a.qnorm_w : a.knorm_w);
    float* vf = (kind == 2 && a.vfirst) ? a.vfirst + (size_t)t * a.G * a.vdim + (size_t)(it - a.H - a.G) * a.vdim : nullptr;
    QT* qd = nullptr;
    KT* kd = nullptr;
    if (kind == 0) qd = (QT*)a.q + (size_t)t * a.H * a.dim + col;
    else if (kind == 1) kd = (KT*)a.kpool + (((size_t)blk * a.G + (it - a.H)) * KV_BLOCK + off) * a.dim;
    else kd = (KT*)a.vpool + (((size_t)blk * a.G + (it - a.H - a.G)) * KV_BLOCK + off) * a.vdim;
    if (in_regs) {
#pragma unroll
      for (int c = 0; c < WP_MAXV; c++) {
        const int i = lane + 32 * c;
        float x = v[c];
        if (kind != 2 && rot > 0) {  // pairs (2i, 2i + 1) sit in neighbouring lanes
          const float o = __shfl_xor_sync(0xffffffffu, x, 1);
          if (i < rot && i < n) x = (i & 1) ? x * cs[i >> 1] + o * sn[i >> 1] : x * cs[i >> 1] - o * sn[i >> 1];
        }
        if (i < n) {
          x *= inv;
          if (nw_) x *= nw_[i];
          if (vf) {
            if (a.vfirst_write) vf[i] = x;
            else x = (1.0f - lam) * x + lam * vf[i];
          }
          if (qd) qd[i] = from_f32<QT>(x);
          else kd[i] = from_f32<KT>(x);
        }
      }
    } else {
      for (int i = lane; i < n; i += 32) {
        float x = sum_slices(row + col + i, a.in_S, a.in_stride);
        if (kind != 2 && i < rot) {
          const int ip = a.rot_pairs ? (i ^ 1) : (i < a.rot_half ? i + a.rot_half : i - a.rot_half);
          const int f = a.rot_pairs ? (i >> 1) : (i < a.rot_half ? i : ip);
          const bool first = a.rot_pairs ? !(i & 1) : i < a.rot_half;
          const float o = sum_slices(row + col + ip, a.in_S, a.in_stride);
          x = first ? x * cs[f] - o * sn[f] : x * cs[f] + o * sn[f];
        }
        x *= inv;
        if (nw_) x *= nw_[i];
        if (vf) {
          if (a.vfirst_write) vf[i] = x;
          else x = (1.0f - lam) * x + lam * vf[i];
        }
        if (qd) qd[i] = from_f32<QT>(x);
        else kd[i] = from_f32<KT>(x);
      }
    }
  }
  TRACE_EXIT(tr);
}

cudaError_t launch_winattn_prep(cudaStream_t st, int qdt, int kvdt, const WinAttnArgs& a) {
  if (a.T <= 0) return cudaSuccess;
  if (2 * a.rot_half > a.dim || (a.vfirst && !a.own_kv)) return cudaErrorInvalidValue;
  // few rows (decode): the heads of a row spread over several CTAs
  const int n_items = a.H + (a.own_kv ? 2 * a.G : 0) + (a.gate_out ? 1 : 0);
  const int ny = a.T >= 1024 ? 1 : ceil_div(n_items, 8);
  const dim3 grid(a.T, ny);
  const int big = std::max(a.dim, a.vdim);
  if (qdt == DT_F32 && kvdt == DT_F32) {
    if (big <= 64) (void)launch_k(winattn_prep_kernel<float, float, 2>, grid, dim3(256), 0, st, a, next_trace(30));
    else if (big <= 128) (void)launch_k(winattn_prep_kernel<float, float, 4>, grid, dim3(256), 0, st, a, next_trace(30));
    else (void)launch_k(winattn_prep_kernel<float, float, 8>, grid, dim3(256), 0, st, a, next_trace(30));
  } else if (qdt == DT_BF16 && kvdt == DT_BF16) {
    if (big <= 64) (void)launch_k(winattn_prep_kernel<bf16, bf16, 2>, grid, dim3(256), 0, st, a, next_trace(30));
    else if (big <= 128) (void)launch_k(winattn_prep_kernel<bf16, bf16, 4>, grid, dim3(256), 0, st, a, next_trace(30));
    else (void)launch_k(winattn_prep_kernel<bf16, bf16, 8>, grid, dim3(256), 0, st, a, next_trace(30));
  } else {
    return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

// ------------------------------------------------------------------ projection epilogue with a short convolution
// One CTA per token.  Pass 1: every q / k / v channel's convolution over the last `taps` projected
// rows (this step's rows through the partials, earlier ones through the slot's tail), q and k
// staged in shared memory with their sums of squares, v straight into the pool, the gates'
// sigmoids out.  Pass 2: the two whole-row norms, weights, rotation, Q and K out.
// TAPS > 0: the number of taps at compile time (no predicates around the taps' loads); 0: c.taps <= 8.
template <typename QT, typename KT, int TAPS>
__global__ void __launch_bounds__(1024) winattn_prep_conv_kernel(WinAttnArgs a, ConvAttnPrep c, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  extern __shared__ float qk[];  // [n_q + n_k] convolved
  __shared__ float red[32];
  pdl_wait();
  constexpr int MT = TAPS > 0 ? TAPS : 8;
  const int taps = TAPS > 0 ? TAPS : c.taps;
  const int t = blockIdx.x;
  const int n_q = a.H * a.dim, n_k = a.G * a.dim, n_v = a.G * a.vdim, n_ch = n_q + n_k + n_v;
  // sequence of the row: one row per sequence in a decode step; else every thread tests one
  // sequence's range (one round trip instead of a chain of dependent loads)
  __shared__ int s_seq;
  if (a.T == a.n_seqs) {
    if (threadIdx.x == 0) s_seq = t;
  } else {
    for (int i = threadIdx.x; i < a.n_seqs; i += blockDim.x)
      if (a.cu_q[i] <= t && t < a.cu_q[i + 1]) s_seq = i;
  }
  __syncthreads();
  const int s = s_seq;
  const int r0 = a.cu_q[s];
  const int li = t - r0, pos = c.positions[t];
  const int keep = taps - 1;
  const float* tail = c.state_pool + (size_t)c.state_slots[s] * c.slot_floats + c.tail_off;
  const int slot = a.slots[t];
  const int blk = slot / KV_BLOCK, off = slot % KV_BLOCK;
  // where tap j's input lives is the same for every channel of the row: a row of this step's
  // partials, a row of the slot's tail, or nowhere (before the sequence's start)
  const float* src[MT];
  float bmul[MT];  // 1: the row still wants the projection's bias
#pragma unroll
  for (int j = 0; j < MT; j++) {
    src[j] = nullptr;
    bmul[j] = 0.f;
    if (j < taps) {
      const int back = keep - j;  // input `back` positions before this token
      if (back <= li) { src[j] = a.in_p + (size_t)(t - back) * a.in_ld; bmul[j] = 1.f; }
      else if (back <= pos) src[j] = tail + (size_t)(keep - (back - li)) * n_ch;
    }
  }
  const bool one = a.in_S == 1;
  auto conv_at = [&](int ch) {
    const float b = c.bias ? c.bias[ch] : 0.f;
    float u[MT], wv[MT];
#pragma unroll
    for (int j = 0; j < MT; j++) {  // all the loads first
      u[j] = 0.f;
      wv[j] = j < taps ? c.conv_w[ch * taps + j] : 0.f;
      if (j < taps && src[j]) {
        if (one || bmul[j] == 0.f) u[j] = src[j][ch];  // one slice (or a tail row): nothing to sum
        else u[j] = sum_slices(src[j] + ch, a.in_S, a.in_stride);
      }
    }
    float y = 0.f;
#pragma unroll
    for (int j = 0; j < MT; j++) y = fmaf(wv[j], fmaf(bmul[j], b, u[j]), y);
    return y;
  };
  float ssq = 0.f, ssk = 0.f;
  for (int ch = threadIdx.x; ch < n_q; ch += blockDim.x) {
    const float y = conv_at(ch);
    qk[ch] = y;
    ssq += y * y;
  }
  for (int ch = n_q + threadIdx.x; ch < n_q + n_k; ch += blockDim.x) {
    const float y = conv_at(ch);
    qk[ch] = y;
    ssk += y * y;
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int g = warp; g < a.G; g += nw) {  // values: a warp per head, no division per element
    KT* vd = (KT*)a.vpool + (((size_t)blk * a.G + g) * KV_BLOCK + off) * a.vdim;
    for (int i = lane; i < a.vdim; i += 32) vd[i] = from_f32<KT>(conv_at(n_q + n_k + g * a.vdim + i));
  }
  if (c.gate_out) {
    const int n_g = a.H * a.vdim;
    const float* gp = a.in_p + (size_t)t * a.in_ld + n_ch;
    float* go = c.gate_out + (size_t)t * c.gate_ld;
    for (int i = threadIdx.x; i < n_g; i += blockDim.x) {
      const float z = one ? gp[i] : sum_slices(gp + i, a.in_S, a.in_stride);
      go[i] = 1.0f / (1.0f + expf(-z));
    }
  }
  const float inv_q = 1.0f / sqrtf(block_sum(ssq, red) / (float)n_q + a.eps);
  const float inv_k = 1.0f / sqrtf(block_sum(ssk, red) / (float)n_k + a.eps);
  const float* cs = c.cosT + (size_t)t * c.rot_half;
  const float* sn = c.sinT + (size_t)t * c.rot_half;
  const int rot = 2 * c.rot_half;
  for (int hh = warp; hh < a.H + a.G; hh += nw) {  // a warp per query / key head
    const bool isq = hh < a.H;
    const int base = hh * a.dim;                    // first channel of the head in qk[]
    const float inv = isq ? inv_q : inv_k;
    const float* w = isq ? c.qnorm_w + base : c.knorm_w + (base - n_q);
    const float* x = qk + base;
    QT* qd = isq ? (QT*)a.q + (size_t)t * n_q + base : nullptr;
    KT* kd = isq ? nullptr : (KT*)a.kpool + (((size_t)blk * a.G + (hh - a.H)) * KV_BLOCK + off) * a.dim;
    for (int i = lane; i < a.dim; i += 32) {
      float v = x[i] * inv * w[i];
      if (i < rot) {
        const int ip = i < c.rot_half ? i + c.rot_half : i - c.rot_half;  // the entry it is paired with
        const float o = x[ip] * inv * w[ip];
        const int f = i < c.rot_half ? i : ip;
        v = i < c.rot_half ? v * cs[f] - o * sn[f] : v * cs[f] + o * sn[f];
      }
      if (isq) qd[i] = from_f32<QT>(v);
      else kd[i] = from_f32<KT>(v);
    }
  }
  TRACE_EXIT(tr);
}

template <typename QT, typename KT>
static void winattn_prep_conv_launch(cudaStream_t st, const WinAttnArgs& a, const ConvAttnPrep& c, dim3 block, size_t smem) {
#define WPC(T_)                                                                                                        \
  {                                                                                                                    \
    if (smem > 48 * 1024)                                                                                              \
      cudaFuncSetAttribute(winattn_prep_conv_kernel<QT, KT, T_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    (void)launch_k(winattn_prep_conv_kernel<QT, KT, T_>, dim3(a.T), block, smem, st, a, c, next_trace(38));            \
  }
  if (c.taps == 1) WPC(1)
  else if (c.taps == 2) WPC(2)
  else if (c.taps == 3) WPC(3)
  else if (c.taps == 4) WPC(4)
  else WPC(0)
#undef WPC
}

cudaError_t launch_winattn_prep_conv(cudaStream_t st, int qdt, int kvdt, const WinAttnArgs& a, const ConvAttnPrep& c) {
  if (a.T <= 0) return cudaSuccess;
  if (c.taps < 1 || c.taps > 8 || 2 * c.rot_half > a.dim || !a.own_kv) return cudaErrorInvalidValue;
  const size_t smem = (size_t)(a.H + a.G) * a.dim * sizeof(float);
  // few rows (decode): the row's channels spread over more threads
  const dim3 block(a.T >= 1024 ? 256 : 1024);
  if (qdt == DT_F32 && kvdt == DT_F32) winattn_prep_conv_launch<float, float>(st, a, c, block, smem);
  else if (qdt == DT_BF16 && kvdt == DT_BF16) winattn_prep_conv_launch<bf16, bf16>(st, a, c, block, smem);
  else return cudaErrorInvalidValue;
  return cudaGetLastError();
}

// ------------------------------------------------------------------ attention, fp32 arithmetic
constexpr int WA_KT = 32;  // keys per tile (divides KV_BLOCK)
constexpr int WA_QS = 16;  // queries per sub-tile: 8 warps x 2

template <typename QT, typename KT, int VPL>
__global__ void __launch_bounds__(256) winattn_kernel(WinAttnArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  const int dim = a.dim, vdim = a.vdim;
  const int kld = dim | 1;  // odd row stride: the 32 lanes read 32 different banks
  float* Qs = smem;                   // [WA_QS][dim], scaled
  float* Ks = Qs + WA_QS * dim;       // [WA_KT][kld]
  float* Vs = Ks + WA_KT * kld;       // [WA_KT][vdim]
  const int tile = blockIdx.x, head = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int seq, q0, n_new, row0, qpos0;
  if (a.tile_seq) {
    seq = a.tile_seq[tile];
    q0 = a.tile_q0[tile];
    n_new = a.cu_q[seq + 1] - a.cu_q[seq];
    row0 = a.cu_q[seq] + q0;
    qpos0 = a.seq_start[seq] + q0;
  } else {
    seq = tile; q0 = 0; n_new = 1; row0 = seq;
    qpos0 = a.seq_len[seq] - 1;
  }
  const int nq = min(a.qtile, n_new - q0);
  const int g = head / (a.H / a.G);
  const int* bt = a.block_tables + (size_t)seq * a.max_blocks;
  const KT* kpool = (const KT*)a.kpool;
  const KT* vpool = (const KT*)a.vpool;
  const float m0 = a.sink ? sink_score(a, head) : -INFINITY, l0 = a.sink ? 1.f : 0.f;
  const float slope = head_slope(a, head);

  for (int qb = 0; qb < nq; qb += WA_QS) {
    const int nqs = min(WA_QS, nq - qb);
    __syncthreads();  // the previous sub-tile's Qs / Ks / Vs have been consumed
    for (int i = threadIdx.x; i < nqs * dim; i += blockDim.x) {
      const int qi = i / dim, d = i % dim;
      Qs[i] = to_f32(((const QT*)a.q)[(size_t)(row0 + qb + qi) * a.H * dim + head * dim + d]) * a.scale;
    }
    float m[2], l[2], acc[2][VPL];
#pragma unroll
    for (int qq = 0; qq < 2; qq++) {
      m[qq] = m0;
      l[qq] = l0;
#pragma unroll
      for (int c = 0; c < VPL; c++) acc[qq][c] = 0.f;
    }
    const int p_first = qpos0 + qb, p_last = qpos0 + qb + nqs - 1;
    int k_lo = first_key(a, p_first);
    k_lo = k_lo / WA_KT * WA_KT;
    const int k_hi = p_last + 1;
    for (int k0 = k_lo; k0 < k_hi; k0 += WA_KT) {
      const int nk = min(WA_KT, k_hi - k0);
      const int blk = bt[k0 / KV_BLOCK];
      const size_t kb = (((size_t)blk * a.G + g) * KV_BLOCK + (k0 % KV_BLOCK));
      __syncthreads();
      for (int i = threadIdx.x; i < nk * dim; i += blockDim.x) {
        const int r = i / dim, d = i % dim;
        Ks[r * kld + d] = to_f32(kpool[(kb + r) * dim + d]);
      }
      for (int i = threadIdx.x; i < nk * vdim; i += blockDim.x) Vs[i] = to_f32(vpool[kb * vdim + i]);
      __syncthreads();
#pragma unroll
      for (int qq = 0; qq < 2; qq++) {
        const int qi = warp + 8 * qq;
        if (qi >= nqs) continue;  // warp-uniform
        const int qp = p_first + qi;
        const int j = k0 + lane;
        const bool vis = lane < nk && j <= qp && j >= first_key(a, qp);
        float s = -INFINITY;
        if (vis) {
          const float* qr = Qs + qi * dim;
          const float* kr = Ks + lane * kld;
          float d = 0.f;
          for (int i = 0; i < dim; i++) d = fmaf(qr[i], kr[i], d);
          s = a.softcap > 0.f ? cap_score<sizeof(QT) == 2>(d, a.softcap) : d;
          s -= slope * (float)(qp - j);
        }
        const float cmax = warp_max(s);
        if (cmax == -INFINITY) continue;  // no key of this tile is visible to the query
        const float mn = fmaxf(m[qq], cmax);
        const float corr = (m[qq] == -INFINITY) ? 0.f : expf(m[qq] - mn);
        const float p = vis ? expf(s - mn) : 0.f;
        l[qq] = l[qq] * corr + warp_sum(p);
#pragma unroll
        for (int c = 0; c < VPL; c++) acc[qq][c] *= corr;
        for (int jj = 0; jj < nk; jj++) {
          const float pj = __shfl_sync(0xffffffffu, p, jj);
          if (pj == 0.f) continue;  // warp-uniform
          const float* vr = Vs + jj * vdim;
#pragma unroll
          for (int c = 0; c < VPL; c++) {
            const int col = lane + 32 * c;
            if (col < vdim) acc[qq][c] = fmaf(pj, vr[col], acc[qq][c]);
          }
        }
        m[qq] = mn;
      }
    }
#pragma unroll
    for (int qq = 0; qq < 2; qq++) {
      const int qi = warp + 8 * qq;
      if (qi >= nqs) continue;
      const float inv = 1.0f / l[qq];
      QT* op = (QT*)a.out + (size_t)(row0 + qb + qi) * a.o_ld;
      const float* gt = gate_row(a, (size_t)(row0 + qb + qi), head, vdim);
#pragma unroll
      for (int c = 0; c < VPL; c++) {
        const int col = lane + 32 * c;
        if (col < vdim) op[head * vdim + col] = from_f32<QT>(acc[qq][c] * inv * (gt ? gt[a.gate_head ? 0 : col] : 1.f));
      }
      if (head == 0)  // padding columns of the output projection's input stay zero
        for (int col = a.H * vdim + lane; col < a.o_ld; col += 32) op[col] = from_f32<QT>(0.f);
    }
  }
  TRACE_EXIT(tr);
}

template <typename QT, typename KT>
static cudaError_t winattn_dispatch(cudaStream_t st, const WinAttnArgs& a) {
  const dim3 grid(a.n_tiles, a.H);
  const size_t smem = ((size_t)WA_QS * a.dim + (size_t)WA_KT * (a.dim | 1) + (size_t)WA_KT * a.vdim) * sizeof(float);
  const int vpl = ceil_div(a.vdim, 32);
#define WA(V)                                                                                               \
  {                                                                                                         \
    if (smem > 48 * 1024)                                                                                   \
      cudaFuncSetAttribute(winattn_kernel<QT, KT, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    (void)launch_k(winattn_kernel<QT, KT, V>, grid, dim3(256), smem, st, a, next_trace(31));                \
  }
  if (vpl <= 1) WA(1)
  else if (vpl <= 2) WA(2)
  else if (vpl <= 4) WA(4)
  else if (vpl <= 8) WA(8)
  else if (vpl <= 16) WA(16)
  else return cudaErrorInvalidValue;
#undef WA
  return cudaGetLastError();
}


// ------------------------------------------------------------------ decode: one query per sequence
// CTA = (sequence, head), 4 warps that take the window's 32-key chunks in turn: a lane scores
// its own key (a cached row is contiguous), the chunk's probabilities are then broadcast lane
// by lane for the weighted sum over the value rows (coalesced); the four partial states meet in
// shared memory, where the sink joins once.
template <typename QT, typename KT, int VPL>
__global__ void __launch_bounds__(128) winattn_decode_kernel(WinAttnArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  const int dim = a.dim, vdim = a.vdim;
  float* qs = smem;             // [dim], scaled
  float* part = smem + dim;     // [4][vdim + 2]
  const int seq = blockIdx.x, head = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = head / (a.H / a.G);
  const int qp = a.seq_len[seq] - 1;
  const int k_lo = first_key(a, qp);
  const float slope = head_slope(a, head);
  const int* bt = a.block_tables + (size_t)seq * a.max_blocks;
  const KT* kpool = (const KT*)a.kpool;
  const KT* vpool = (const KT*)a.vpool;
  for (int i = threadIdx.x; i < dim; i += blockDim.x)
    qs[i] = to_f32(((const QT*)a.q)[(size_t)seq * a.H * dim + head * dim + i]) * a.scale;
  __syncthreads();
  float m = -INFINITY, l = 0.f, acc[VPL];
#pragma unroll
  for (int c = 0; c < VPL; c++) acc[c] = 0.f;
  for (int k0 = k_lo + warp * 32; k0 <= qp; k0 += 4 * 32) {
    const int j = k0 + lane;
    const bool vis = j <= qp;
    float s = -INFINITY;
    if (vis) {
      const KT* kr = kpool + (((size_t)bt[j / KV_BLOCK] * a.G + g) * KV_BLOCK + (j % KV_BLOCK)) * dim;
      float d = 0.f;
      for (int i = 0; i < dim; i++) d = fmaf(qs[i], to_f32(kr[i]), d);
      s = a.softcap > 0.f ? cap_score<sizeof(QT) == 2>(d, a.softcap) : d;
      s -= slope * (float)(qp - j);
    }
    const float mn = fmaxf(m, warp_max(s));  // lane 0 of the chunk is always visible
    const float corr = (m == -INFINITY) ? 0.f : expf(m - mn);
    const float p = vis ? expf(s - mn) : 0.f;
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int c = 0; c < VPL; c++) acc[c] *= corr;
    const int nk = min(32, qp + 1 - k0);
    for (int jj = 0; jj < nk; jj++) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int jp = k0 + jj;
      const KT* vr = vpool + (((size_t)bt[jp / KV_BLOCK] * a.G + g) * KV_BLOCK + (jp % KV_BLOCK)) * vdim;
#pragma unroll
      for (int c = 0; c < VPL; c++) {
        const int col = lane + 32 * c;
        if (col < vdim) acc[c] = fmaf(pj, to_f32(vr[col]), acc[c]);
      }
    }
    m = mn;
  }
  float* mine = part + warp * (vdim + 2);
#pragma unroll
  for (int c = 0; c < VPL; c++) {
    const int col = lane + 32 * c;
    if (col < vdim) mine[col] = acc[c];
  }
  if (lane == 0) {
    mine[vdim] = m;
    mine[vdim + 1] = l;
  }
  __syncthreads();
  const float sk = sink_score(a, head);
  float mt = a.sink ? sk : -INFINITY;
  for (int w = 0; w < 4; w++) mt = fmaxf(mt, part[w * (vdim + 2) + vdim]);
  float lt = a.sink ? expf(sk - mt) : 0.f;
  float cw[4];
  for (int w = 0; w < 4; w++) {
    const float mw = part[w * (vdim + 2) + vdim];
    cw[w] = (mw == -INFINITY) ? 0.f : expf(mw - mt);
    lt += part[w * (vdim + 2) + vdim + 1] * cw[w];
  }
  QT* op = (QT*)a.out + (size_t)seq * a.o_ld;
  for (int col = threadIdx.x; col < vdim; col += blockDim.x) {
    float v = 0.f;
    for (int w = 0; w < 4; w++) v += part[w * (vdim + 2) + col] * cw[w];
    if (a.gate) v *= gate_row(a, (size_t)seq, head, vdim)[a.gate_head ? 0 : col];
    op[head * vdim + col] = from_f32<QT>(v / lt);
  }
  if (head == 0)
    for (int col = a.H * vdim + threadIdx.x; col < a.o_ld; col += blockDim.x) op[col] = from_f32<QT>(0.f);
  TRACE_EXIT(tr);
}

// Grouped decode kernel (dim a multiple of 8, vdim = 32 * VPT): CTA = (sequence, key / value head,
// chunk of up to GQMAX query heads of its group), so a cached row is read once for the whole
// group.  A lane scores its own key against all the group's queries with 16-byte loads of the row
// (queries in shared memory, broadcast), then owns VPT neighbouring value columns: a value row
// is one coalesced load for the warp, the lanes' probabilities and row addresses travel by shuffle.
template <int N, typename T>
__device__ __forceinline__ void load_n(const T* p, float (&v)[N]);
template <> __device__ __forceinline__ void load_n<1, float>(const float* p, float (&v)[1]) { v[0] = p[0]; }
template <> __device__ __forceinline__ void load_n<2, float>(const float* p, float (&v)[2]) {
  const float2 x = *reinterpret_cast<const float2*>(p);
  v[0] = x.x; v[1] = x.y;
}
template <> __device__ __forceinline__ void load_n<4, float>(const float* p, float (&v)[4]) {
  const float4 x = *reinterpret_cast<const float4*>(p);
  v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
}
template <> __device__ __forceinline__ void load_n<8, float>(const float* p, float (&v)[8]) { load8(p, v); }
template <> __device__ __forceinline__ void load_n<1, bf16>(const bf16* p, float (&v)[1]) { v[0] = __bfloat162float(p[0]); }
template <> __device__ __forceinline__ void load_n<2, bf16>(const bf16* p, float (&v)[2]) {
  const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
  v[0] = x.x; v[1] = x.y;
}
template <> __device__ __forceinline__ void load_n<4, bf16>(const bf16* p, float (&v)[4]) {
  const uint2 r = *reinterpret_cast<const uint2*>(p);
  const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.x));
  const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r.y));
  v[0] = x.x; v[1] = x.y; v[2] = y.x; v[3] = y.y;
}
template <> __device__ __forceinline__ void load_n<8, bf16>(const bf16* p, float (&v)[8]) { load8(p, v); }

constexpr int WD_WARPS = 8;
template <typename QT, typename KT, int VPT, int GQMAX>
__global__ void __launch_bounds__(256, (GQMAX * VPT <= 16) ? 2 : 1) winattn_decode_group_kernel(WinAttnArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  const int dim = a.dim, vdim = 32 * VPT;
  const int seq = blockIdx.x, g = blockIdx.y;
  const int GQ = a.H / a.G;
  const int gq0 = blockIdx.z * GQMAX;         // first query head of the chunk within the group
  const int gqn = min(GQMAX, GQ - gq0);
  const int h0 = g * GQ + gq0;
  float* qs = smem;                            // [GQMAX][dim], scaled
  float* part = smem + GQMAX * dim;            // [WD_WARPS][GQMAX][vdim + 2]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int qp = a.seq_len[seq] - 1;
  const int k_lo = first_key(a, qp);
  const int* bt = a.block_tables + (size_t)seq * a.max_blocks;
  const KT* kpool = (const KT*)a.kpool;
  const KT* vpool = (const KT*)a.vpool;
  for (int i = threadIdx.x; i < gqn * dim; i += blockDim.x)
    qs[i] = to_f32(((const QT*)a.q)[(size_t)seq * a.H * dim + (size_t)(h0 + i / dim) * dim + i % dim]) * a.scale;
  __syncthreads();
  float m[GQMAX], l[GQMAX], acc[GQMAX][VPT];
#pragma unroll
  for (int q = 0; q < GQMAX; q++) {
    m[q] = -INFINITY;
    l[q] = 0.f;
#pragma unroll
    for (int c = 0; c < VPT; c++) acc[q][c] = 0.f;
  }
  for (int k0 = k_lo + warp * 32; k0 <= qp; k0 += WD_WARPS * 32) {
    const int j = k0 + lane;
    const bool vis = j <= qp;
    const int jc = vis ? j : qp;
    const int rowb = (bt[jc / KV_BLOCK] * a.G + g) * KV_BLOCK + (jc % KV_BLOCK);  // row of the layer's pools
    // the chunk's value rows do not wait for the scores: the first VB of them are requested now,
    // beside the key row, and arrive while the scores and the softmax are computed
    constexpr int VB = (64 / VPT) < 8 ? 8 : ((64 / VPT) > 32 ? 32 : (64 / VPT));  // value rows in flight
    float vv[VB][VPT];
#pragma unroll
    for (int u = 0; u < VB; u++) {
      const int rb = __shfl_sync(0xffffffffu, rowb, u);
      load_n<VPT, KT>(vpool + (size_t)rb * vdim + lane * VPT, vv[u]);
    }
    float s[GQMAX];
#pragma unroll
    for (int q = 0; q < GQMAX; q++) s[q] = 0.f;
    const KT* kr = kpool + (size_t)rowb * dim;
#pragma unroll 4
    for (int i = 0; i < dim; i += 8) {
      float k8[8];
      load8(kr + i, k8);
#pragma unroll
      for (int q = 0; q < GQMAX; q++)
        if (q < gqn) {
          const float4 qa = *reinterpret_cast<const float4*>(qs + q * dim + i);
          const float4 qb = *reinterpret_cast<const float4*>(qs + q * dim + i + 4);
          s[q] = fmaf(k8[0], qa.x, s[q]); s[q] = fmaf(k8[1], qa.y, s[q]);
          s[q] = fmaf(k8[2], qa.z, s[q]); s[q] = fmaf(k8[3], qa.w, s[q]);
          s[q] = fmaf(k8[4], qb.x, s[q]); s[q] = fmaf(k8[5], qb.y, s[q]);
          s[q] = fmaf(k8[6], qb.z, s[q]); s[q] = fmaf(k8[7], qb.w, s[q]);
        }
    }
    float p[GQMAX];
#pragma unroll
    for (int q = 0; q < GQMAX; q++) {
      const float sv = vis ? (a.softcap > 0.f ? cap_score<sizeof(QT) == 2>(s[q], a.softcap) : s[q]) -
                                 head_slope(a, h0 + q) * (float)(qp - j)
                           : -INFINITY;
      const float mn = fmaxf(m[q], warp_max(sv));  // lane 0 of a chunk is always visible
      const float corr = (m[q] == -INFINITY) ? 0.f : expf(m[q] - mn);
      p[q] = vis ? expf(sv - mn) : 0.f;
      l[q] = l[q] * corr + warp_sum(p[q]);
#pragma unroll
      for (int c = 0; c < VPT; c++) acc[q][c] *= corr;
      m[q] = mn;
    }
    // weighted sum over the value rows; lanes past the last key carry probability 0 and a valid
    // (clamped) row
    const int nk = min(32, qp + 1 - k0);
    for (int jj0 = 0; jj0 < nk; jj0 += VB) {
      if (jj0 > 0) {
#pragma unroll
        for (int u = 0; u < VB; u++) {
          const int rb = __shfl_sync(0xffffffffu, rowb, jj0 + u);
          load_n<VPT, KT>(vpool + (size_t)rb * vdim + lane * VPT, vv[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < VB; u++) {
#pragma unroll
        for (int q = 0; q < GQMAX; q++) {
          const float pj = __shfl_sync(0xffffffffu, p[q], jj0 + u);
#pragma unroll
          for (int c = 0; c < VPT; c++) acc[q][c] = fmaf(pj, vv[u][c], acc[q][c]);
        }
      }
    }
  }
  const int ps = vdim + 2;
#pragma unroll
  for (int q = 0; q < GQMAX; q++) {
    float* mine = part + ((size_t)warp * GQMAX + q) * ps;
#pragma unroll
    for (int c = 0; c < VPT; c++) mine[lane * VPT + c] = acc[q][c];
    if (lane == 0) {
      mine[vdim] = m[q];
      mine[vdim + 1] = l[q];
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < gqn * vdim; i += blockDim.x) {
    const int q = i / vdim, col = i % vdim;
    const float sk = sink_score(a, h0 + q);
    float mt = a.sink ? sk : -INFINITY;
    for (int w = 0; w < WD_WARPS; w++) mt = fmaxf(mt, part[((size_t)w * GQMAX + q) * ps + vdim]);
    float lt = a.sink ? expf(sk - mt) : 0.f, v = 0.f;
    for (int w = 0; w < WD_WARPS; w++) {
      const float* pw = part + ((size_t)w * GQMAX + q) * ps;
      const float cw = (pw[vdim] == -INFINITY) ? 0.f : expf(pw[vdim] - mt);
      lt += pw[vdim + 1] * cw;
      v += pw[col] * cw;
    }
    if (a.gate) v *= gate_row(a, (size_t)seq, h0 + q, vdim)[a.gate_head ? 0 : col];
    ((QT*)a.out)[(size_t)seq * a.o_ld + (size_t)(h0 + q) * vdim + col] = from_f32<QT>(v / lt);
  }
  if (g == 0 && blockIdx.z == 0)
    for (int col = a.H * vdim + threadIdx.x; col < a.o_ld; col += blockDim.x)
      ((QT*)a.out)[(size_t)seq * a.o_ld + col] = from_f32<QT>(0.f);
  TRACE_EXIT(tr);
}

template <typename QT, typename KT, int VPT>
static cudaError_t winattn_decode_group_vpt(cudaStream_t st, const WinAttnArgs& a) {
  const int GQ = a.H / a.G;
  const int gmax = GQ <= 1 ? 1 : GQ <= 2 ? 2 : GQ <= 4 ? 4 : 8;
  const dim3 grid(a.n_tiles, a.G, ceil_div(GQ, gmax));
  const size_t smem = ((size_t)gmax * a.dim + WD_WARPS * (size_t)gmax * (a.vdim + 2)) * sizeof(float);
  if (smem > 48 * 1024) return cudaErrorInvalidValue;
  if (gmax == 1) (void)launch_k(winattn_decode_group_kernel<QT, KT, VPT, 1>, grid, dim3(32 * WD_WARPS), smem, st, a, next_trace(33));
  else if (gmax == 2) (void)launch_k(winattn_decode_group_kernel<QT, KT, VPT, 2>, grid, dim3(32 * WD_WARPS), smem, st, a, next_trace(33));
  else if (gmax == 4) (void)launch_k(winattn_decode_group_kernel<QT, KT, VPT, 4>, grid, dim3(32 * WD_WARPS), smem, st, a, next_trace(33));
  else (void)launch_k(winattn_decode_group_kernel<QT, KT, VPT, 8>, grid, dim3(32 * WD_WARPS), smem, st, a, next_trace(33));
  return cudaGetLastError();
}
static bool winattn_decode_group_ok(const WinAttnArgs& a) {
  static const bool on = [] {
    const char* e = getenv("NVLLM_WINATTN_GROUP");
    return e ? atoi(e) != 0 : true;
  }();
  const int vpt = a.vdim / 32;
  const int gmax = std::min(8, a.H / a.G);
  return on && a.dim % 8 == 0 && a.vdim % 32 == 0 && (vpt == 1 || vpt == 2 || vpt == 4 || vpt == 8) &&
         ((size_t)gmax * a.dim + WD_WARPS * (size_t)gmax * (a.vdim + 2)) * sizeof(float) <= 48 * 1024;
}
template <typename QT, typename KT>
static cudaError_t winattn_decode_group(cudaStream_t st, const WinAttnArgs& a) {
  switch (a.vdim / 32) {
    case 1: return winattn_decode_group_vpt<QT, KT, 1>(st, a);
    case 2: return winattn_decode_group_vpt<QT, KT, 2>(st, a);
    case 4: return winattn_decode_group_vpt<QT, KT, 4>(st, a);
    default: return winattn_decode_group_vpt<QT, KT, 8>(st, a);
  }
}

template <typename QT, typename KT>
static cudaError_t winattn_decode_dispatch(cudaStream_t st, const WinAttnArgs& a) {
  const dim3 grid(a.n_tiles, a.H);
  const size_t smem = ((size_t)a.dim + 4 * ((size_t)a.vdim + 2)) * sizeof(float);
  const int vpl = ceil_div(a.vdim, 32);
#define WD(V) (void)launch_k(winattn_decode_kernel<QT, KT, V>, grid, dim3(128), smem, st, a, next_trace(33));
  if (smem > 48 * 1024) return cudaErrorInvalidValue;
  if (vpl <= 1) WD(1)
  else if (vpl <= 2) WD(2)
  else if (vpl <= 4) WD(4)
  else if (vpl <= 8) WD(8)
  else if (vpl <= 16) WD(16)
  else return cudaErrorInvalidValue;
#undef WD
  return cudaGetLastError();
}

// ------------------------------------------------------------------ attention on mma.sync (bf16)
// CTA = 64 queries of one sequence x one head, 4 warps x 16 query rows.  Q [64][DP] and the K / V
// tiles [64][DP] / [64][VP] live in shared memory with rows padded by 8 elements (ldmatrix
// without bank conflicts); DP / VP = dim / vdim (multiples of 16).  S = Q K^T in fp32
// accumulators, masked per element (causal + window), online softmax in the accumulator layout
// (the sink is the initial max 0 / denominator 1), P rounded to bf16 as the A operand of O += P V
// with V read through ldmatrix.trans.  Key tiles outside [first query - window + 1, last query]
// are never loaded; K / V of tile i + 1 arrive by cp.async while tile i is computed.
constexpr int WM_Q = 64, WM_K = 64;

template <int DIM, int VDIM>
__global__ void __launch_bounds__(128) winattn_mma_kernel(WinAttnArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  constexpr int DP = DIM + 8, VP = VDIM + 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);  // [64][DP]
  bf16* Ks = Qs + WM_Q * DP;                      // [2][64][DP]
  bf16* Vs = Ks + 2 * WM_K * DP;                  // [2][64][VP]
  const int tile = blockIdx.x, head = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int seq, q0, n_new, row0, qpos0;
  if (a.tile_seq) {
    seq = a.tile_seq[tile];
    q0 = a.tile_q0[tile];
    n_new = a.cu_q[seq + 1] - a.cu_q[seq];
    row0 = a.cu_q[seq] + q0;
    qpos0 = a.seq_start[seq] + q0;
  } else {
    seq = tile; q0 = 0; n_new = 1; row0 = seq;
    qpos0 = a.seq_len[seq] - 1;
  }
  const int nq = min(WM_Q, n_new - q0);
  const int g = head / (a.H / a.G);
  const int* bt = a.block_tables + (size_t)seq * a.max_blocks;
  const bf16* kpool = (const bf16*)a.kpool;
  const bf16* vpool = (const bf16*)a.vpool;
  const bf16* qg = (const bf16*)a.q + (size_t)row0 * a.H * DIM + head * DIM;

  // Q tile: rows past nq are zero
  for (int i = threadIdx.x; i < WM_Q * (DIM / 8); i += blockDim.x) {
    const int r = i / (DIM / 8), c = i % (DIM / 8);
    const bool ok = r < nq;
    cp_async16(smem_addr(Qs + r * DP + c * 8), ok ? (const void*)(qg + (size_t)r * a.H * DIM + c * 8) : (const void*)qg, ok);
  }
  int k_lo = first_key(a, qpos0);
  k_lo = k_lo / WM_K * WM_K;
  const int k_hi = qpos0 + nq;  // keys [k_lo, k_hi)
  const int n_kt = (k_hi - k_lo + WM_K - 1) / WM_K;
  auto load_kv = [&](int kt, int buf) {
    const int k0 = k_lo + kt * WM_K;
    const int nk = min(WM_K, k_hi - k0);
    const int blk = bt[k0 / KV_BLOCK];
    const size_t kb = (((size_t)blk * a.G + g) * KV_BLOCK + (k0 % KV_BLOCK));
    bf16* kd = Ks + buf * WM_K * DP;
    bf16* vd = Vs + buf * WM_K * VP;
    for (int i = threadIdx.x; i < WM_K * (DIM / 8); i += blockDim.x) {
      const int r = i / (DIM / 8), c = i % (DIM / 8);
      const bool ok = r < nk;
      cp_async16(smem_addr(kd + r * DP + c * 8), ok ? (const void*)(kpool + (kb + r) * DIM + c * 8) : (const void*)kpool, ok);
    }
    for (int i = threadIdx.x; i < WM_K * (VDIM / 8); i += blockDim.x) {
      const int r = i / (VDIM / 8), c = i % (VDIM / 8);
      const bool ok = r < nk;
      cp_async16(smem_addr(vd + r * VP + c * 8), ok ? (const void*)(vpool + (kb + r) * VDIM + c * 8) : (const void*)vpool, ok);
    }
  };
  load_kv(0, 0);
  cp_async_commit();

  const int gid = lane >> 2, tig = lane & 3;
  const int r_lo = warp * 16 + gid, r_hi = r_lo + 8;     // the thread's two query rows in the tile
  const int qp_lo = qpos0 + r_lo, qp_hi = qpos0 + r_hi;  // their positions
  float m_lo, m_hi, l_lo, l_hi;
  m_lo = m_hi = a.sink ? sink_score(a, head) * 1.4426950408889634f : -INFINITY;  // base-2 domain, like the scores
  l_lo = l_hi = a.sink ? 1.f : 0.f;
  const float slope2 = head_slope(a, head) * 1.4426950408889634f;
  float o[VDIM / 8][4];
#pragma unroll
  for (int i = 0; i < VDIM / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const float sc = a.scale * 1.4426950408889634f;  // log2(e): softmax in base 2

  for (int kt = 0; kt < n_kt; kt++) {
    const int buf = kt & 1;
    if (kt + 1 < n_kt) load_kv(kt + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int k0 = k_lo + kt * WM_K;
    const bf16* kd = Ks + buf * WM_K * DP;
    const bf16* vd = Vs + buf * WM_K * VP;
    // does any row of this warp see any key of the tile?
    const int w_qlo = qpos0 + warp * 16, w_qhi = w_qlo + 15;
    const bool warp_sees = warp * 16 < nq && k0 <= w_qhi && k0 + WM_K - 1 >= first_key(a, w_qlo);
    if (warp_sees) {
      float s[WM_K / 8][4];
#pragma unroll
      for (int i = 0; i < WM_K / 8; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < DIM / 16; kk++) {
        uint32_t a0, a1, a2, a3;
        // A fragment (16 query rows x 16 dims): matrices (rows 0-7, k 0-7), (rows 8-15, k 0-7),
        // (rows 0-7, k 8-15), (rows 8-15, k 8-15)
        ldsm_x4(smem_addr(Qs + (warp * 16 + (lane & 15)) * DP + kk * 16 + (lane >> 4) * 8), a0, a1, a2, a3);
#pragma unroll
        for (int nb = 0; nb < WM_K / 16; nb++) {
          // B fragments of two 8-key blocks: K rows are the n index, dims the k index
          uint32_t b0, b1, b2, b3;
          ldsm_x4(smem_addr(kd + (nb * 16 + (lane & 7) + ((lane >> 4) << 3)) * DP + kk * 16 + ((lane >> 3) & 1) * 8),
                  b0, b1, b2, b3);
          mma16816(s[2 * nb], a0, a1, a2, a3, b0, b1);
          mma16816(s[2 * nb + 1], a0, a1, a2, a3, b2, b3);
        }
      }
      // scale (scores live in the base-2 domain: exp2 of a difference is one instruction), mask
      // (only on tiles that some row of the warp sees partly), running max
      const bool interior = k0 + WM_K - 1 <= w_qlo && k0 + WM_K <= k_hi && k0 >= first_key(a, w_qhi);
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
      if (a.softcap > 0.f) {  // the cap works on the scaled score; back to the base-2 domain afterwards
#pragma unroll
        for (int nb = 0; nb < WM_K / 8; nb++)
#pragma unroll
          for (int e = 0; e < 4; e++) s[nb][e] = cap_score<true>(s[nb][e] * a.scale, a.softcap) * (1.4426950408889634f / sc);
      }
      if (interior) {
#pragma unroll
        for (int nb = 0; nb < WM_K / 8; nb++) {
          s[nb][0] *= sc; s[nb][1] *= sc; s[nb][2] *= sc; s[nb][3] *= sc;
          if (slope2 != 0.f) {
            const int j = k0 + nb * 8 + tig * 2;
            s[nb][0] -= slope2 * (float)(qp_lo - j); s[nb][1] -= slope2 * (float)(qp_lo - j - 1);
            s[nb][2] -= slope2 * (float)(qp_hi - j); s[nb][3] -= slope2 * (float)(qp_hi - j - 1);
          }
          mx_lo = fmaxf(mx_lo, fmaxf(s[nb][0], s[nb][1]));
          mx_hi = fmaxf(mx_hi, fmaxf(s[nb][2], s[nb][3]));
        }
      } else {
#pragma unroll
        for (int nb = 0; nb < WM_K / 8; nb++) {
#pragma unroll
          for (int e = 0; e < 4; e++) {
            const int j = k0 + nb * 8 + tig * 2 + (e & 1);
            const int qp = (e & 2) ? qp_hi : qp_lo;
            const bool vis = j <= qp && j < k_hi && j >= first_key(a, qp);
            const float v = vis ? s[nb][e] * sc - slope2 * (float)(qp - j) : -INFINITY;
            s[nb][e] = v;
            if (e & 2) mx_hi = fmaxf(mx_hi, v);
            else mx_lo = fmaxf(mx_lo, v);
          }
        }
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);
      // a row that has seen nothing yet (and has no sink) keeps max -inf: every p below is 0
      const float c_lo = (mn_lo == -INFINITY) ? 1.f : exp2f(m_lo - mn_lo);  // exp2(-inf) = 0
      const float c_hi = (mn_hi == -INFINITY) ? 1.f : exp2f(m_hi - mn_hi);
      const float sub_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo, sub_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi;
      float ps_lo = 0.f, ps_hi = 0.f;
      uint32_t pa[WM_K / 8][2];
#pragma unroll
      for (int nb = 0; nb < WM_K / 8; nb++) {
        const float p0 = exp2f(s[nb][0] - sub_lo), p1 = exp2f(s[nb][1] - sub_lo);  // masked scores are -inf: 0
        const float p2 = exp2f(s[nb][2] - sub_hi), p3 = exp2f(s[nb][3] - sub_hi);
        ps_lo += p0 + p1;
        ps_hi += p2 + p3;
        pa[nb][0] = pack_bf16(p0, p1);
        pa[nb][1] = pack_bf16(p2, p3);
      }
      ps_lo += __shfl_xor_sync(0xffffffffu, ps_lo, 1);
      ps_lo += __shfl_xor_sync(0xffffffffu, ps_lo, 2);
      ps_hi += __shfl_xor_sync(0xffffffffu, ps_hi, 1);
      ps_hi += __shfl_xor_sync(0xffffffffu, ps_hi, 2);
      l_lo = l_lo * c_lo + ps_lo;
      l_hi = l_hi * c_hi + ps_hi;
      m_lo = mn_lo;
      m_hi = mn_hi;
#pragma unroll
      for (int i = 0; i < VDIM / 8; i++) {
        o[i][0] *= c_lo; o[i][1] *= c_lo;
        o[i][2] *= c_hi; o[i][3] *= c_hi;
      }
      // O += P V: P (16 x 64 keys) as A fragments of 16 keys each, V [key][vdim] through ldmatrix.trans
#pragma unroll
      for (int kk = 0; kk < WM_K / 16; kk++) {
        const uint32_t a0 = pa[2 * kk][0], a1 = pa[2 * kk][1], a2 = pa[2 * kk + 1][0], a3 = pa[2 * kk + 1][1];
#pragma unroll
        for (int nb = 0; nb < VDIM / 16; nb++) {
          uint32_t b0, b1, b2, b3;
          // matrices: (keys 0-7, cols 0-7), (keys 8-15, cols 0-7), (keys 0-7, cols 8-15), (keys 8-15, cols 8-15)
          ldsm_x4_t(smem_addr(vd + (kk * 16 + (lane & 15)) * VP + nb * 16 + (lane >> 4) * 8), b0, b1, b2, b3);
          mma16816(o[2 * nb], a0, a1, a2, a3, b0, b1);
          mma16816(o[2 * nb + 1], a0, a1, a2, a3, b2, b3);
        }
      }
    }
    __syncthreads();  // the buffer is free for the load of tile kt + 2
  }
  cp_async_wait<0>();
  const float i_lo = 1.0f / l_lo, i_hi = 1.0f / l_hi;
  bf16* ob = (bf16*)a.out + (size_t)row0 * a.o_ld + head * VDIM;
  const float* gb = gate_row(a, (size_t)row0, head, VDIM);
#pragma unroll
  for (int i = 0; i < VDIM / 8; i++) {
    const int col = i * 8 + tig * 2;
    float g0 = 1.f, g1 = 1.f, g2 = 1.f, g3 = 1.f;
    if (gb && a.gate_head) {
      if (r_lo < nq) g0 = g1 = gb[(size_t)r_lo * a.gate_ld];
      if (r_hi < nq) g2 = g3 = gb[(size_t)r_hi * a.gate_ld];
    } else if (gb) {
      if (r_lo < nq) { g0 = gb[(size_t)r_lo * a.gate_ld + col]; g1 = gb[(size_t)r_lo * a.gate_ld + col + 1]; }
      if (r_hi < nq) { g2 = gb[(size_t)r_hi * a.gate_ld + col]; g3 = gb[(size_t)r_hi * a.gate_ld + col + 1]; }
    }
    if (r_lo < nq) *reinterpret_cast<uint32_t*>(ob + (size_t)r_lo * a.o_ld + col) = pack_bf16(o[i][0] * i_lo * g0, o[i][1] * i_lo * g1);
    if (r_hi < nq) *reinterpret_cast<uint32_t*>(ob + (size_t)r_hi * a.o_ld + col) = pack_bf16(o[i][2] * i_hi * g2, o[i][3] * i_hi * g3);
  }
  if (head == 0) {
    bf16* orow = (bf16*)a.out + (size_t)row0 * a.o_ld;
    const int pad = a.o_ld - a.H * VDIM;
    for (int i = threadIdx.x; i < nq * pad; i += blockDim.x)
      orow[(size_t)(i / pad) * a.o_ld + a.H * VDIM + i % pad] = __float2bfloat16_rn(0.f);
  }
  TRACE_EXIT(tr);
}

// ------------------------------------------------------------------ decode on mma.sync (bf16)
// CTA = (sequence, key / value head), 4 warps.  The 16 rows of the MMA tile are the query heads of
// the group (all at the sequence's last position; rows past the group are zero), so a cached row
// is read once for the whole group.  K / V tiles of 64 keys arrive by cp.async in a ring of three
// (two tiles in flight while one is computed); every warp takes 16 keys of each tile — S = Q K^T
// on its keys, the running softmax in base 2, O += P V — and the four partial states meet in
// shared memory at the end, where the sink joins once.
constexpr int WDM_ST = 3;
constexpr int WDM_MIN_TILES = 4;  // a split range holds at least this many key tiles

template <int DIM, int VDIM>
__global__ void __launch_bounds__(128) winattn_decode_mma_kernel(WinAttnArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  constexpr int DP = DIM + 8, VP = VDIM + 8;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* Qs = reinterpret_cast<bf16*>(smem_raw);  // [16][DP]
  bf16* Ks = Qs + 16 * DP;                        // [WDM_ST][64][DP]
  bf16* Vs = Ks + WDM_ST * WM_K * DP;             // [WDM_ST][64][VP]
  const int seq = blockIdx.x, g = blockIdx.y;
  const int GQ = a.H / a.G, h0 = g * GQ;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int qp = a.seq_len[seq] - 1;
  const int k_lo = first_key(a, qp);
  const int t_lo = k_lo / WM_K * WM_K;
  const int n_kt = (qp + 1 - t_lo + WM_K - 1) / WM_K;
  // the CTA's range of key tiles: all of them, or (long contexts, few sequences) one of n_split ranges of at
  // least WDM_MIN_TILES tiles; a range past the context is empty and hands in an empty state
  const int n_split = a.n_split > 1 ? a.n_split : 1;
  int kt_b = 0, kt_e = n_kt;
  if (n_split > 1) {
    const int per = max(WDM_MIN_TILES, (n_kt + n_split - 1) / n_split);
    kt_b = min(n_kt, (int)blockIdx.z * per);
    kt_e = min(n_kt, kt_b + per);
  }
  const int* bt = a.block_tables + (size_t)seq * a.max_blocks;
  const bf16* kpool = (const bf16*)a.kpool;
  const bf16* vpool = (const bf16*)a.vpool;
  const bf16* qg = (const bf16*)a.q + ((size_t)seq * a.H + h0) * DIM;  // the group's heads are neighbours
  for (int i = threadIdx.x; i < 16 * (DIM / 8); i += blockDim.x) {
    const int r = i / (DIM / 8), c = i % (DIM / 8);
    const bool ok = r < GQ;
    cp_async16(smem_addr(Qs + r * DP + c * 8), ok ? (const void*)(qg + (size_t)r * DIM + c * 8) : (const void*)qg, ok);
  }
  auto load_kv = [&](int kt) {
    const int buf = kt % WDM_ST;
    const int k0 = t_lo + kt * WM_K;
    const int nk = min(WM_K, qp + 1 - k0);
    const size_t kb = (((size_t)bt[k0 / KV_BLOCK] * a.G + g) * KV_BLOCK + (k0 % KV_BLOCK));
    bf16* kd = Ks + buf * WM_K * DP;
    bf16* vd = Vs + buf * WM_K * VP;
    for (int i = threadIdx.x; i < WM_K * (DIM / 8); i += blockDim.x) {
      const int r = i / (DIM / 8), c = i % (DIM / 8);
      const bool ok = r < nk;
      cp_async16(smem_addr(kd + r * DP + c * 8), ok ? (const void*)(kpool + (kb + r) * DIM + c * 8) : (const void*)kpool, ok);
    }
    for (int i = threadIdx.x; i < WM_K * (VDIM / 8); i += blockDim.x) {
      const int r = i / (VDIM / 8), c = i % (VDIM / 8);
      const bool ok = r < nk;
      cp_async16(smem_addr(vd + r * VP + c * 8), ok ? (const void*)(vpool + (kb + r) * VDIM + c * 8) : (const void*)vpool, ok);
    }
  };
  if (kt_b < kt_e) load_kv(kt_b);
  cp_async_commit();
  if (kt_b + 1 < kt_e) load_kv(kt_b + 1);
  cp_async_commit();

  const int gid = lane >> 2, tig = lane & 3;
  const int kb16 = warp * 16;  // the warp's keys inside a tile
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  float o[VDIM / 8][4];
#pragma unroll
  for (int i = 0; i < VDIM / 8; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  uint32_t qa[DIM / 16][4];
  const float sc = a.scale * 1.4426950408889634f;  // log2(e): softmax in base 2
  // the thread's two rows are two heads of the group, each with its own slope
  const float slope_lo = gid < GQ ? head_slope(a, h0 + gid) * 1.4426950408889634f : 0.f;
  const float slope_hi = gid + 8 < GQ ? head_slope(a, h0 + gid + 8) * 1.4426950408889634f : 0.f;

  for (int kt = kt_b; kt < kt_e; kt++) {
    if (kt + 2 < kt_e) load_kv(kt + 2);
    cp_async_commit();
    cp_async_wait<2>();  // tile kt (and, the first time, the queries) has landed
    __syncthreads();
    if (kt == kt_b) {
#pragma unroll
      for (int kk = 0; kk < DIM / 16; kk++)
        ldsm_x4(smem_addr(Qs + (lane & 15) * DP + kk * 16 + (lane >> 4) * 8), qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3]);
    }
    const int k0 = t_lo + kt * WM_K;
    const bf16* kd = Ks + (kt % WDM_ST) * WM_K * DP;
    const bf16* vd = Vs + (kt % WDM_ST) * WM_K * VP;
    const int j0 = k0 + kb16;  // first key of the warp's 16
    if (j0 <= qp && j0 + 15 >= k_lo) {
      float s[2][4];
#pragma unroll
      for (int i = 0; i < 2; i++) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
      for (int kk = 0; kk < DIM / 16; kk++) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(smem_addr(kd + (kb16 + (lane & 7) + ((lane >> 4) << 3)) * DP + kk * 16 + ((lane >> 3) & 1) * 8), b0, b1, b2, b3);
        mma16816(s[0], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b0, b1);
        mma16816(s[1], qa[kk][0], qa[kk][1], qa[kk][2], qa[kk][3], b2, b3);
      }
      float mx_lo = -INFINITY, mx_hi = -INFINITY;
#pragma unroll
      for (int nb = 0; nb < 2; nb++) {
#pragma unroll
        for (int e = 0; e < 4; e++) {
          const int j = j0 + nb * 8 + tig * 2 + (e & 1);
          const float sv = (a.softcap > 0.f ? cap_score<true>(s[nb][e] * a.scale, a.softcap) * 1.4426950408889634f : s[nb][e] * sc) -
                           ((e & 2) ? slope_hi : slope_lo) * (float)(qp - j);
          const float v = (j >= k_lo && j <= qp) ? sv : -INFINITY;  // every row sits at position qp
          s[nb][e] = v;
          if (e & 2) mx_hi = fmaxf(mx_hi, v);
          else mx_lo = fmaxf(mx_lo, v);
        }
      }
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 1));
      mx_lo = fmaxf(mx_lo, __shfl_xor_sync(0xffffffffu, mx_lo, 2));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 1));
      mx_hi = fmaxf(mx_hi, __shfl_xor_sync(0xffffffffu, mx_hi, 2));
      const float mn_lo = fmaxf(m_lo, mx_lo), mn_hi = fmaxf(m_hi, mx_hi);  // finite: at least one key of the 16 is visible
      const float c_lo = exp2f(m_lo - mn_lo), c_hi = exp2f(m_hi - mn_hi);  // exp2(-inf) = 0
      float ps_lo = 0.f, ps_hi = 0.f;
      uint32_t pa[2][2];
#pragma unroll
      for (int nb = 0; nb < 2; nb++) {
        const float p0 = exp2f(s[nb][0] - mn_lo), p1 = exp2f(s[nb][1] - mn_lo);
        const float p2 = exp2f(s[nb][2] - mn_hi), p3 = exp2f(s[nb][3] - mn_hi);
        ps_lo += p0 + p1;
        ps_hi += p2 + p3;
        pa[nb][0] = pack_bf16(p0, p1);
        pa[nb][1] = pack_bf16(p2, p3);
      }
      ps_lo += __shfl_xor_sync(0xffffffffu, ps_lo, 1);
      ps_lo += __shfl_xor_sync(0xffffffffu, ps_lo, 2);
      ps_hi += __shfl_xor_sync(0xffffffffu, ps_hi, 1);
      ps_hi += __shfl_xor_sync(0xffffffffu, ps_hi, 2);
      l_lo = l_lo * c_lo + ps_lo;
      l_hi = l_hi * c_hi + ps_hi;
      m_lo = mn_lo;
      m_hi = mn_hi;
#pragma unroll
      for (int i = 0; i < VDIM / 8; i++) {
        o[i][0] *= c_lo; o[i][1] *= c_lo;
        o[i][2] *= c_hi; o[i][3] *= c_hi;
      }
#pragma unroll
      for (int nb = 0; nb < VDIM / 16; nb++) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(smem_addr(vd + (kb16 + (lane & 15)) * VP + nb * 16 + (lane >> 4) * 8), b0, b1, b2, b3);
        mma16816(o[2 * nb], pa[0][0], pa[0][1], pa[1][0], pa[1][1], b0, b1);
        mma16816(o[2 * nb + 1], pa[0][0], pa[0][1], pa[1][0], pa[1][1], b2, b3);
      }
    }
    __syncthreads();  // the buffer is free for the load of tile kt + 3
  }
  cp_async_wait<0>();
  __syncthreads();
  // the four warps' states meet in the (now free) tile buffers: [4][16][VDIM + 2] floats
  float* mrg = reinterpret_cast<float*>(Ks);
  constexpr int MS = VDIM + 2;
  {
    float* lo = mrg + ((size_t)warp * 16 + gid) * MS;
    float* hi = mrg + ((size_t)warp * 16 + gid + 8) * MS;
#pragma unroll
    for (int i = 0; i < VDIM / 8; i++) {
      const int col = i * 8 + tig * 2;
      lo[col] = o[i][0]; lo[col + 1] = o[i][1];
      hi[col] = o[i][2]; hi[col + 1] = o[i][3];
    }
    if (tig == 0) {
      lo[VDIM] = m_lo; lo[VDIM + 1] = l_lo;
      hi[VDIM] = m_hi; hi[VDIM + 1] = l_hi;
    }
  }
  __syncthreads();
  if (n_split > 1) {
    // the CTA's state (relative to its own maximum, without the sink) goes to its place among the pair's
    // n_split; the CTA that arrives last adds them up.  Nobody waits: the counter only tells who is last.
    __shared__ int is_last;
    const size_t pair = (size_t)seq * a.G + g;
    float* part = a.split_ws + (pair * n_split + blockIdx.z) * 16 * MS;
    for (int i = threadIdx.x; i < GQ * VDIM; i += blockDim.x) {
      const int r = i / VDIM, col = i % VDIM;
      float mt = -INFINITY;
      for (int w = 0; w < 4; w++) mt = fmaxf(mt, mrg[((size_t)w * 16 + r) * MS + VDIM]);
      float lt = 0.f, v = 0.f;
      if (mt > -INFINITY) {
        for (int w = 0; w < 4; w++) {
          const float* pw = mrg + ((size_t)w * 16 + r) * MS;
          const float cw = exp2f(pw[VDIM] - mt);
          lt += pw[VDIM + 1] * cw;
          v += pw[col] * cw;
        }
      }
      part[(size_t)r * MS + col] = v;
      if (col == 0) {
        part[(size_t)r * MS + VDIM] = mt;
        part[(size_t)r * MS + VDIM + 1] = lt;
      }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      const unsigned before = atomicAdd(a.split_cnt + pair, 1u);
      is_last = before == (unsigned)n_split - 1;
      if (is_last) a.split_cnt[pair] = 0;  // every CTA of the pair has arrived: zero again for the next launch
    }
    __syncthreads();
    if (is_last) {
      __threadfence();
      const float* all = a.split_ws + pair * n_split * 16 * MS;
      for (int i = threadIdx.x; i < GQ * VDIM; i += blockDim.x) {
        const int r = i / VDIM, col = i % VDIM;
        const float sk = sink_score(a, h0 + r) * 1.4426950408889634f;
        float mt = a.sink ? sk : -INFINITY;
        for (int z = 0; z < n_split; z++) mt = fmaxf(mt, __ldcg(all + ((size_t)z * 16 + r) * MS + VDIM));
        float lt = a.sink ? exp2f(sk - mt) : 0.f, v = 0.f;
        for (int z = 0; z < n_split; z++) {
          const float* pz = all + ((size_t)z * 16 + r) * MS;
          const float cz = exp2f(__ldcg(pz + VDIM) - mt);  // an empty range has max -inf: weight 0
          lt += __ldcg(pz + VDIM + 1) * cz;
          v += __ldcg(pz + col) * cz;
        }
        if (a.gate) v *= gate_row(a, (size_t)seq, h0 + r, VDIM)[a.gate_head ? 0 : col];
        ((bf16*)a.out)[(size_t)seq * a.o_ld + (size_t)(h0 + r) * VDIM + col] = __float2bfloat16_rn(v / lt);
      }
    }
  } else {
    for (int i = threadIdx.x; i < GQ * VDIM; i += blockDim.x) {
      const int r = i / VDIM, col = i % VDIM;
      const float sk = sink_score(a, h0 + r) * 1.4426950408889634f;
      float mt = a.sink ? sk : -INFINITY;
      for (int w = 0; w < 4; w++) mt = fmaxf(mt, mrg[((size_t)w * 16 + r) * MS + VDIM]);
      float lt = a.sink ? exp2f(sk - mt) : 0.f, v = 0.f;
      for (int w = 0; w < 4; w++) {
        const float* pw = mrg + ((size_t)w * 16 + r) * MS;
        const float cw = exp2f(pw[VDIM] - mt);  // a warp that saw no key has max -inf: weight 0
        lt += pw[VDIM + 1] * cw;
        v += pw[col] * cw;
      }
      if (a.gate) v *= gate_row(a, (size_t)seq, h0 + r, VDIM)[a.gate_head ? 0 : col];
      ((bf16*)a.out)[(size_t)seq * a.o_ld + (size_t)(h0 + r) * VDIM + col] = __float2bfloat16_rn(v / lt);
    }
  }
  if (g == 0 && blockIdx.z == 0)
    for (int col = a.H * VDIM + threadIdx.x; col < a.o_ld; col += blockDim.x)
      ((bf16*)a.out)[(size_t)seq * a.o_ld + col] = __float2bfloat16_rn(0.f);
  TRACE_EXIT(tr);
}

template <int DIM, int VDIM>
static cudaError_t winattn_decode_mma_launch(cudaStream_t st, const WinAttnArgs& a) {
  const size_t tiles = (size_t)WDM_ST * WM_K * ((DIM + 8) + (VDIM + 8)) * 2;
  const size_t merge = (size_t)4 * 16 * (VDIM + 2) * 4;
  const size_t smem = (size_t)16 * (DIM + 8) * 2 + std::max(tiles, merge);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(winattn_decode_mma_kernel<DIM, VDIM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  const int n_split = a.n_split > 1 && a.split_ws && a.split_cnt ? std::min(a.n_split, WINATTN_MAX_SPLIT) : 1;
  WinAttnArgs b = a;
  b.n_split = n_split;
  (void)launch_k(winattn_decode_mma_kernel<DIM, VDIM>, dim3(a.n_tiles, a.G, n_split), dim3(128), smem, st, b, next_trace(37));
  return cudaGetLastError();
}

static bool winattn_mma_on() {
  static const bool on = [] {
    const char* e = getenv("NVLLM_WINATTN_MMA");
    return e ? atoi(e) != 0 : true;
  }();
  return on;
}
// compile-time (dim, vdim) pairs of the mma.sync kernel
static bool winattn_mma_shape(int dim, int vdim) {
  return (dim == 64 && vdim == 64) || (dim == 96 && vdim == 96) || (dim == 128 && vdim == 128) ||
         (dim == 32 && vdim == 32) || (dim == 64 && vdim == 128) || (dim == 128 && vdim == 64);
}
bool winattn_uses_mma(int qdt, int kvdt, int dim, int vdim) {
  return winattn_mma_on() && qdt == DT_BF16 && kvdt == DT_BF16 && winattn_mma_shape(dim, vdim);
}
int winattn_qtile(int qdt, int kvdt, int dim, int vdim) {
  return winattn_uses_mma(qdt, kvdt, dim, vdim) ? WM_Q : WA_QS;
}

template <int DIM, int VDIM>
static cudaError_t winattn_mma_launch(cudaStream_t st, const WinAttnArgs& a) {
  const size_t smem = ((size_t)WM_Q * (DIM + 8) + 2 * (size_t)WM_K * (DIM + 8) + 2 * (size_t)WM_K * (VDIM + 8)) * 2;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(winattn_mma_kernel<DIM, VDIM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  (void)launch_k(winattn_mma_kernel<DIM, VDIM>, dim3(a.n_tiles, a.H), dim3(128), smem, st, a, next_trace(32));
  return cudaGetLastError();
}

cudaError_t launch_winattn(cudaStream_t st, int qdt, int kvdt, const WinAttnArgs& a) {
  if (a.n_tiles <= 0) return cudaSuccess;
  if (a.H % a.G) return cudaErrorInvalidValue;
  if (a.tile_seq == nullptr) {  // decode: one query per sequence
    static const bool dec_mma = !(getenv("NVLLM_WINATTN_DECODE_MMA") && atoi(getenv("NVLLM_WINATTN_DECODE_MMA")) == 0);
    if (dec_mma && winattn_uses_mma(qdt, kvdt, a.dim, a.vdim) && a.H / a.G <= 16) {
      if (a.dim == 64 && a.vdim == 64) return winattn_decode_mma_launch<64, 64>(st, a);
      if (a.dim == 96 && a.vdim == 96) return winattn_decode_mma_launch<96, 96>(st, a);
      if (a.dim == 128 && a.vdim == 128) return winattn_decode_mma_launch<128, 128>(st, a);
      if (a.dim == 32 && a.vdim == 32) return winattn_decode_mma_launch<32, 32>(st, a);
      if (a.dim == 64 && a.vdim == 128) return winattn_decode_mma_launch<64, 128>(st, a);
      if (a.dim == 128 && a.vdim == 64) return winattn_decode_mma_launch<128, 64>(st, a);
    }
    if (winattn_decode_group_ok(a)) {
      if (qdt == DT_F32 && kvdt == DT_F32) return winattn_decode_group<float, float>(st, a);
      if (qdt == DT_BF16 && kvdt == DT_BF16) return winattn_decode_group<bf16, bf16>(st, a);
    }
    if (qdt == DT_F32 && kvdt == DT_F32) return winattn_decode_dispatch<float, float>(st, a);
    if (qdt == DT_BF16 && kvdt == DT_BF16) return winattn_decode_dispatch<bf16, bf16>(st, a);
    return cudaErrorInvalidValue;
  }
  // the mma kernel's tile is 64 queries: prefill steps whose tile list was built for it
  if (winattn_uses_mma(qdt, kvdt, a.dim, a.vdim) && a.qtile == WM_Q && (a.o_ld % 2) == 0) {
    if (a.dim == 64 && a.vdim == 64) return winattn_mma_launch<64, 64>(st, a);
    if (a.dim == 96 && a.vdim == 96) return winattn_mma_launch<96, 96>(st, a);
    if (a.dim == 128 && a.vdim == 128) return winattn_mma_launch<128, 128>(st, a);
    if (a.dim == 32 && a.vdim == 32) return winattn_mma_launch<32, 32>(st, a);
    if (a.dim == 64 && a.vdim == 128) return winattn_mma_launch<64, 128>(st, a);
    if (a.dim == 128 && a.vdim == 64) return winattn_mma_launch<128, 64>(st, a);
  }
  if (qdt == DT_F32 && kvdt == DT_F32) return winattn_dispatch<float, float>(st, a);
  if (qdt == DT_BF16 && kvdt == DT_BF16) return winattn_dispatch<bf16, bf16>(st, a);
  return cudaErrorInvalidValue;
}

}  // namespace nvllm
