// attention_latent.cu — latent ("compressed key/value") attention over the paged pool.
//
// A layer of this kind caches, per token, ONE row shared by all heads: the normed latent
// c [R] followed by the rotated key part k_r [rot]  (Dk = R + rot).  Per head the key is
// [W_uk c | k_r] and the value W_uv c.  The kernels never expand keys or values: with
// q~ = W_uk^T q_n  (absorbed query, R wide) the score is (q~ . c + q_r . k_r) * scale, and the
// head's output is W_uv (sum_j p_j c_j) — i.e. multi-query attention with one latent "kv head"
// whose key row is [c | k_r] and whose value row is the first R entries of the same row.
//
//  latent_prep_kernel     sums the split-K partials of the fused input projection
//                         [W_dq | W_dkv | W_g] h, RMS-norms the query latent, RMS-norms the key
//                         latent and rotates the shared key part into the pool row at slots[t],
//                         and keeps sigmoid(W_g h) per head
//  rope_table_kernel      cos / sin of pos * base^(-2i/dims) for the step's rows (double)
//  latent_fold_*          at load: W_uk folded into the query up projection, W_uv into the output
//                         projection (per head), so that both are plain GEMMs on the tensor cores
//  latent_q_kernel        split-K sum of the folded query projection, rotation of q_r
//  latent_attn_kernel     causal online-softmax attention of (query, head) items against the
//                         latent rows; one warp per item, a CTA's items share each key tile;
//                         optional key splits (decode) merged by latent_combine_kernel
//                         the head's sigmoid gate is applied where the sum is normalised
// All arithmetic is fp32 (double for the angles); QT / KT are the activation / cache dtypes.
#include <stdlib.h>

#include "common.cuh"
#include "kernels.h"
#include "mma.cuh"

namespace nvllm {

constexpr int LAT_WARPS = 8;    // (query, head) items per attention CTA
constexpr int LAT_KT = 32;      // keys per shared-memory tile: one per lane
constexpr int LAT_NACC = 16;    // accumulator registers per lane: R <= 32 * LAT_NACC

// ---------------------------------------------------------------- rope table
__global__ void rope_table_kernel(const int* __restrict__ positions, int T, int half,
                                  const double* __restrict__ inv_freq, float* __restrict__ cosT,
                                  float* __restrict__ sinT, double mult) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * half) return;
  const int t = i / half, j = i % half;
  double s, c;
  sincos((double)positions[t] * inv_freq[j], &s, &c);
  cosT[i] = (float)(c * mult);
  sinT[i] = (float)(s * mult);
}
cudaError_t launch_rope_table(cudaStream_t st, const int* positions, int T, int half,
                              const double* inv_freq, float* cosT, float* sinT, double mult) {
  if (T <= 0 || half <= 0) return cudaSuccess;
  const int n = T * half;
  (void)launch_k(rope_table_kernel, dim3((n + 255) / 256), dim3(256), 0, st, positions, T, half, inv_freq,
                 cosT, sinT, mult);
  return cudaGetLastError();
}

// ---------------------------------------------------------------- input-projection epilogue
template <typename QT, typename KT>
__global__ void __launch_bounds__(256) latent_prep_kernel(LatentArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  extern __shared__ float row[];  // [n_in]
  __shared__ float red[32];
  const int t = blockIdx.x;
  const int n_in = a.q_rank + (a.own_kv ? a.R + a.rot : 0) + a.H;
  pdl_wait();
  if ((n_in & 7) == 0 && (a.in_stride & 7) == 0) {
    for (int i = threadIdx.x * 8; i < n_in; i += blockDim.x * 8) {
      float v[8];
      sum_partials8(a.in_p + (size_t)t * a.in_ld + i, a.in_S, a.in_stride, v);
#pragma unroll
      for (int j = 0; j < 8; j++) row[i + j] = v[j];
    }
  } else {
    for (int i = threadIdx.x; i < n_in; i += blockDim.x) {
      float s = 0.f;
      for (int k = 0; k < a.in_S; k++) s += a.in_p[(size_t)k * a.in_stride + (size_t)t * a.in_ld + i];
      row[i] = s;
    }
  }
  __syncthreads();
  // query latent: c_q = v / sqrt(mean(v^2) + eps) * w
  float ss = 0.f;
  for (int i = threadIdx.x; i < a.q_rank; i += blockDim.x) ss += row[i] * row[i];
  ss = block_sum(ss, red);
  const float inv_q = 1.0f / sqrtf(ss / (float)a.q_rank + a.eps);
  QT* cq = (QT*)a.cq + (size_t)t * a.q_rank_p;
  for (int i = threadIdx.x; i < a.q_rank_p; i += blockDim.x)
    cq[i] = from_f32<QT>(i < a.q_rank ? row[i] * inv_q * a.dq_norm[i] : 0.f);
  if (a.own_kv) {
    const float* v = row + a.q_rank;
    float s2 = 0.f;
    for (int i = threadIdx.x; i < a.R; i += blockDim.x) s2 += v[i] * v[i];
    s2 = block_sum(s2, red);
    const float inv_k = 1.0f / sqrtf(s2 / (float)a.R + a.eps);
    KT* pr = (KT*)a.pool + (size_t)a.slots[t] * (a.R + a.rot);
    for (int i = threadIdx.x; i < a.R; i += blockDim.x) pr[i] = from_f32<KT>(v[i] * inv_k * a.dkv_norm[i]);
    // shared key part: entry i pairs with i + half inside the first rot_dims entries
    const float* kr = v + a.R;
    const int half = a.rot_dims / 2;
    for (int i = threadIdx.x; i < a.rot; i += blockDim.x) {
      float o = kr[i];
      if (i < half) {
        const float c = a.cosT[(size_t)t * half + i], s = a.sinT[(size_t)t * half + i];
        o = kr[i] * c - kr[i + half] * s;
      } else if (i < a.rot_dims) {
        const int j = i - half;
        const float c = a.cosT[(size_t)t * half + j], s = a.sinT[(size_t)t * half + j];
        o = kr[i] * c + kr[j] * s;
      }
      pr[a.R + i] = from_f32<KT>(o);
    }
  }
  const float* g = row + a.q_rank + (a.own_kv ? a.R + a.rot : 0);
  for (int i = threadIdx.x; i < a.H; i += blockDim.x) a.gate[(size_t)t * a.H + i] = 1.0f / (1.0f + expf(-g[i]));
  TRACE_EXIT(tr);
}

cudaError_t launch_latent_prep(cudaStream_t st, int qdt, int kvdt, const LatentArgs& a) {
  if (a.T <= 0) return cudaSuccess;
  const size_t smem = (size_t)(a.q_rank + a.R + a.rot + a.H) * sizeof(float);
  if (qdt == DT_F32 && kvdt == DT_F32)
    (void)launch_k(latent_prep_kernel<float, float>, dim3(a.T), dim3(256), smem, st, a, next_trace(20));
  else if (qdt == DT_BF16 && kvdt == DT_BF16)
    (void)launch_k(latent_prep_kernel<bf16, bf16>, dim3(a.T), dim3(256), smem, st, a, next_trace(20));
  else
    return cudaErrorInvalidValue;
  return cudaGetLastError();
}

// ---------------------------------------------------------------- absorbed query, epilogue
// The query up projection runs with the FOLDED weight (W_uk^T W_uq,n per head, then the rotated
// rows of W_uq; latent_fold_q_kernel), so its output already is [q~ (R) | q_r (rot)] per head.
// This kernel sums the split-K partials, rotates q_r and rounds to the activation dtype.
template <typename QT>
__global__ void __launch_bounds__(256) latent_q_kernel(LatentArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  const int t = blockIdx.x, Dk = a.R + a.rot, n = a.H * Dk, half = a.rot_dims / 2;
  pdl_wait();
  QT* out = (QT*)a.qabs + (size_t)t * n;
  const float* src = a.q_p + (size_t)t * a.q_ld;
  const float* cs = a.cosT + (size_t)t * half;
  const float* sn = a.sinT + (size_t)t * half;
  // absorbed part, 8 entries at a time when the sizes allow (sum of the slices, one rounding)
  const bool vec = (a.R & 7) == 0 && (Dk & 7) == 0 && (a.q_stride & 7) == 0 && (a.q_ld & 7) == 0;
  if (vec) {
    const int vph = a.R / 8;  // vectors per head
    for (int v = threadIdx.x; v < a.H * vph; v += blockDim.x) {
      const int i = (v / vph) * Dk + (v % vph) * 8;
      float acc[8];
      sum_partials8(src + i, a.q_S, a.q_stride, acc);
      store8(out + i, acc);
    }
  }
  for (int i0 = threadIdx.x; i0 < (vec ? a.H * a.rot : n); i0 += blockDim.x) {
    const int i = vec ? (i0 / a.rot) * Dk + a.R + i0 % a.rot : i0;
    const int d = i % Dk - a.R;  // index inside the rotated part (negative: absorbed part)
    float v = 0.f, pair = 0.f;
    const int j = d < 0 || d >= a.rot_dims ? i : (d < half ? i + half : i - half);
    for (int k = 0; k < a.q_S; k++) {
      v += src[(size_t)k * a.q_stride + i];
      if (j != i) pair += src[(size_t)k * a.q_stride + j];
    }
    if (j != i) v = d < half ? v * cs[d] - pair * sn[d] : v * cs[d - half] + pair * sn[d - half];
    out[i] = from_f32<QT>(v);
  }
  TRACE_EXIT(tr);
}

cudaError_t launch_latent_q(cudaStream_t st, int qdt, const LatentArgs& a) {
  if (a.T <= 0) return cudaSuccess;
  if (qdt == DT_F32) (void)launch_k(latent_q_kernel<float>, dim3(a.T), dim3(256), 0, st, a, next_trace(21));
  else (void)launch_k(latent_q_kernel<bf16>, dim3(a.T), dim3(256), 0, st, a, next_trace(21));
  return cudaGetLastError();
}

// ---------------------------------------------------------------- weight folding (once, at finalize)
// wq[h * Dk + r, k]     = sum_d W_uk[h * dim + d, r] * W_uq[h * (dim + rot) + d, k]     r < R
// wq[h * Dk + R + j, k] = W_uq[h * (dim + rot) + dim + j, k]
// wo[n, h * R + r]      = sum_e W_o[n, h * vdim + e] * W_uv[h * vdim + e, r]
// fp32 accumulation, one rounding to the weight dtype; the padding columns stay zero.
template <typename WT>
__global__ void latent_fold_q_kernel(const WT* __restrict__ w_uq, const WT* __restrict__ w_uk, WT* __restrict__ wq,
                                     int H, int dim, int rot, int R, int q_rank, int ld) {
  const int Dk = R + rot;
  const size_t n = (size_t)H * Dk * q_rank;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int k = (int)(i % q_rank), row = (int)(i / q_rank), h = row / Dk, r = row % Dk;
    float acc = 0.f;
    if (r >= R) {
      acc = to_f32(w_uq[((size_t)h * (dim + rot) + dim + (r - R)) * ld + k]);
    } else {
      for (int d = 0; d < dim; d++)
        acc = fmaf(to_f32(w_uk[((size_t)h * dim + d) * R + r]), to_f32(w_uq[((size_t)h * (dim + rot) + d) * ld + k]), acc);
    }
    wq[(size_t)row * ld + k] = from_f32<WT>(acc);
  }
}
template <typename WT>
__global__ void latent_fold_o_kernel(const WT* __restrict__ w_o, const WT* __restrict__ w_uv, WT* __restrict__ wo,
                                     int W, int H, int vdim, int R, int ld_o, int ld) {
  const size_t n = (size_t)W * H * R;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % ((size_t)H * R)), row = (int)(i / ((size_t)H * R)), h = c / R, r = c % R;
    float acc = 0.f;
    for (int e = 0; e < vdim; e++)
      acc = fmaf(to_f32(w_o[(size_t)row * ld_o + h * vdim + e]), to_f32(w_uv[((size_t)h * vdim + e) * R + r]), acc);
    wo[(size_t)row * ld + c] = from_f32<WT>(acc);
  }
}
cudaError_t launch_latent_fold(cudaStream_t st, int wdt, const void* w_uq, const void* w_uk, void* wq, const void* w_o,
                               const void* w_uv, void* wo, int W, int H, int dim, int rot, int vdim, int R,
                               int q_rank, int q_rank_p, int ov_p, int ovr_p) {
  if (wdt == DT_F32) {
    latent_fold_q_kernel<float><<<148 * 8, 256, 0, st>>>((const float*)w_uq, (const float*)w_uk, (float*)wq, H, dim,
                                                         rot, R, q_rank, q_rank_p);
    latent_fold_o_kernel<float><<<148 * 8, 256, 0, st>>>((const float*)w_o, (const float*)w_uv, (float*)wo, W, H,
                                                         vdim, R, ov_p, ovr_p);
  } else {
    latent_fold_q_kernel<bf16><<<148 * 8, 256, 0, st>>>((const bf16*)w_uq, (const bf16*)w_uk, (bf16*)wq, H, dim, rot,
                                                        R, q_rank, q_rank_p);
    latent_fold_o_kernel<bf16><<<148 * 8, 256, 0, st>>>((const bf16*)w_o, (const bf16*)w_uv, (bf16*)wo, W, H, vdim, R,
                                                        ov_p, ovr_p);
  }
  return cudaGetLastError();
}

// ---------------------------------------------------------------- attention
// grid (tiles, item chunks, key splits).  A tile is LAT_QTILE consecutive new tokens of one
// sequence (the host's tile list; without one, tile = sequence and its single new token).  The
// tile's (query, head) items are dealt to warps, LAT_WARPS per CTA; all of them read the same
// key tiles from shared memory.  Lane j scores key j of a tile (the whole Dk-long dot product,
// query broadcast from shared memory), the warp takes max / sum, and for the weighted sum lane i
// owns latent entries i, i + 32, ... in registers.
template <typename QT, typename KT>
__global__ void __launch_bounds__(LAT_WARPS * 32) latent_attn_kernel(LatentArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  extern __shared__ float sm[];
  const int Dk = a.R + a.rot, ldk = Dk + 1;
  float* Ks = sm;                       // [LAT_KT][Dk + 1]
  float* Qs = sm + LAT_KT * ldk;        // [LAT_WARPS][Dk]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_wait();
  const int tile = blockIdx.x;
  const int seq = a.tile_seq ? a.tile_seq[tile] : tile;
  const int q0 = a.tile_q0 ? a.tile_q0[tile] : 0;
  const int row0 = a.cu_q[seq];
  const int n_new = a.cu_q[seq + 1] - row0;
  const int start = a.tile_seq ? a.seq_start[seq] : a.seq_len[seq] - 1;  // decode steps advance seq_len only
  const int nq = min(a.qtile, n_new - q0);
  const int item0 = blockIdx.y * LAT_WARPS;
  if (item0 >= nq * a.H) return;  // nothing traced: an empty CTA
  const int item = item0 + warp;
  const bool valid = item < nq * a.H;
  const int qi = valid ? item / a.H : 0, head = valid ? item % a.H : 0;
  const int row = row0 + q0 + qi;
  const int qpos = start + q0 + qi;  // last visible key position of this item
  // keys this CTA needs: up to its last item's position; a split takes a contiguous share
  const int last_q = min(nq - 1, (item0 + LAT_WARPS - 1) / a.H);
  const int kv_end = start + q0 + last_q + 1;
  const int n_tiles_k = ceil_div(kv_end, LAT_KT);
  const int per = ceil_div(n_tiles_k, (int)gridDim.z);
  const int kt0 = blockIdx.z * per, kt1 = min(n_tiles_k, kt0 + per);
  const int* bt = a.block_tables + (size_t)seq * a.max_blocks;
  const KT* pool = (const KT*)a.pool;

  if (valid) {
    const QT* qp = (const QT*)a.qabs + ((size_t)row * a.H + head) * Dk;
    for (int d = lane; d < Dk; d += 32) Qs[warp * Dk + d] = to_f32(qp[d]) * a.scale;
  }
  float acc[LAT_NACC];
#pragma unroll
  for (int i = 0; i < LAT_NACC; i++) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  const float* qv = Qs + warp * Dk;

  for (int kt = kt0; kt < kt1; kt++) {
    const int k0 = kt * LAT_KT;
    const int nk = min(LAT_KT, kv_end - k0);
    __syncthreads();
    // a tile never straddles a block (LAT_KT divides KV_BLOCK)
    const KT* src = pool + ((size_t)bt[k0 / KV_BLOCK] * KV_BLOCK + (k0 % KV_BLOCK)) * Dk;
    for (int i = threadIdx.x; i < nk * Dk; i += blockDim.x) Ks[(i / Dk) * ldk + (i % Dk)] = to_f32(src[i]);
    __syncthreads();
    if (!valid) continue;
    const int vis = min(nk, qpos - k0 + 1);  // keys of this tile the item sees
    if (vis <= 0) continue;
    float s = -INFINITY;
    if (lane < vis) {
      const float* kr = Ks + lane * ldk;
      float d0 = 0.f, d1 = 0.f;
      int d = 0;
      for (; d + 1 < Dk; d += 2) {
        d0 = fmaf(qv[d], kr[d], d0);
        d1 = fmaf(qv[d + 1], kr[d + 1], d1);
      }
      if (d < Dk) d0 = fmaf(qv[d], kr[d], d0);
      s = d0 + d1;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);  // m = -inf on the first visible tile -> 0
    const float p = lane < vis ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < LAT_NACC; i++) acc[i] *= corr;
    for (int j = 0; j < vis; j++) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const float* vr = Ks + j * ldk;
#pragma unroll
      for (int i = 0; i < LAT_NACC; i++)
        if (i * 32 < a.R) {
          const int r = i * 32 + lane;
          if (r < a.R) acc[i] = fmaf(pj, vr[r], acc[i]);
        }
    }
    m = m_new;
  }
  TRACE_EXIT(tr);
  if (!valid) return;
  if (gridDim.z == 1) {
    const float inv = a.gate[(size_t)row * a.H + head] / l;  // the head's sigmoid gate rides on the normalisation
    QT* op = (QT*)a.olat + (size_t)row * a.o_ld + head * a.R;
#pragma unroll
    for (int i = 0; i < LAT_NACC; i++) {
      const int r = i * 32 + lane;
      if (r < a.R) op[r] = from_f32<QT>(acc[i] * inv);
    }
    if (head == a.H - 1)  // padding columns of the output projection's input
      for (int r = a.H * a.R + lane; r < a.o_ld; r += 32) ((QT*)a.olat)[(size_t)row * a.o_ld + r] = from_f32<QT>(0.f);
  } else {
    // split record: [R] unnormalised sum, then m, l
    float* rec = a.split_ws + (((size_t)row * a.H + head) * gridDim.z + blockIdx.z) * (a.R + 2);
#pragma unroll
    for (int i = 0; i < LAT_NACC; i++) {
      const int r = i * 32 + lane;
      if (r < a.R) rec[r] = acc[i];
    }
    if (lane == 0) {
      rec[a.R] = m;
      rec[a.R + 1] = l;
    }
  }
}

// ---------------------------------------------------------------- attention, tensor cores
// bf16 path (Dk and R multiples of 16, R <= 8 * NR): the same items and key ranges as the kernel
// above, 64 items per CTA (4 warps x 16 rows of mma.sync m16n8k16).  The tile's absorbed queries
// are one contiguous [items, Dk] block; key tiles of 64 cached rows arrive by cp.async into a
// padded tile (row stride Dk + 8: conflict-free ldmatrix), double-buffered when two fit.  Scores
// S = Q K^T over all Dk columns; the weighted sum P V takes the first R columns of the SAME tile
// (ldmatrix.trans), so a cached row is staged once for both.  Online softmax in the accumulator
// layout; the P fragments come straight from the score accumulators.
constexpr int LM_KT = 64;
// KS > 0: the cached row is exactly KS * 16 columns and R exactly NR * 8 (the common sizes): row
// strides, loop counts and fragment addresses are then compile-time constants and the score loop
// is unrolled; KS == 0 reads them from the arguments.
template <int NR, int LM_ROWS, int KS>
__global__ void __launch_bounds__(LM_ROWS < 64 ? 128 : LM_ROWS * 2, (NR <= 16 && LM_ROWS == 128) ? 2 : 1)
latent_attn_mma_kernel(LatentArgs a, int two_stage, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  extern __shared__ __align__(16) uint8_t smem_lm[];
  const int Dk = KS ? KS * 16 : a.R + a.rot, ld = Dk + 8, cpr = Dk / 8;
  const uint32_t sQ = smem_addr(smem_lm);
  const uint32_t sK0 = sQ + LM_ROWS * ld * 2;
  const uint32_t tile_bytes = LM_KT * ld * 2;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const bool active = LM_ROWS >= 64 || warp * 16 < LM_ROWS;  // warps beyond the CTA's rows only stage tiles
  const int g = lane >> 2, t = lane & 3, mi = lane >> 3, lr = lane & 7;
  pdl_wait();
  const int tile = blockIdx.x;
  const int seq = a.tile_seq ? a.tile_seq[tile] : tile;
  const int q0 = a.tile_q0 ? a.tile_q0[tile] : 0;
  const int row0 = a.cu_q[seq];
  const int n_new = a.cu_q[seq + 1] - row0;
  const int start = a.tile_seq ? a.seq_start[seq] : a.seq_len[seq] - 1;  // decode steps advance seq_len only
  const int nq = min(a.qtile, n_new - q0);
  const int n_items = nq * a.H;
  const int item0 = blockIdx.y * LM_ROWS;
  if (item0 >= n_items) return;
  const int last_q = min(nq - 1, (item0 + LM_ROWS - 1) / a.H);
  const int kv_end = start + q0 + last_q + 1;
  const int n_tiles_k = ceil_div(kv_end, LM_KT);
  const int per = ceil_div(n_tiles_k, (int)gridDim.z);
  const int kt0 = blockIdx.z * per, kt1 = min(n_tiles_k, kt0 + per);
  const int* bt = a.block_tables + (size_t)seq * a.max_blocks;
  const bf16* pool = (const bf16*)a.pool;
  const bf16* qsrc = (const bf16*)a.qabs + ((size_t)(row0 + q0) * a.H + item0) * Dk;
  const int q_rows = min(LM_ROWS, n_items - item0);

  auto load_keys = [&](int kt, int buf) {
    const int k0 = kt * LM_KT;
    const int nk = min(LM_KT, kv_end - k0);
    const bf16* src = pool + ((size_t)bt[k0 / KV_BLOCK] * KV_BLOCK + (k0 % KV_BLOCK)) * Dk;
    const uint32_t dst = sK0 + buf * tile_bytes;
    for (int i = threadIdx.x; i < LM_KT * cpr; i += blockDim.x) {
      const int r = i / cpr, c = i % cpr;
      const bool ok = r < nk;
      cp_async16(dst + (r * ld + c * 8) * 2, ok ? (const void*)(src + (size_t)r * Dk + c * 8) : (const void*)src, ok);
    }
    cp_async_commit();
  };
  for (int i = threadIdx.x; i < LM_ROWS * cpr; i += blockDim.x) {
    const int r = i / cpr, c = i % cpr;
    const bool ok = r < q_rows;
    cp_async16(sQ + (r * ld + c * 8) * 2, ok ? (const void*)(qsrc + (size_t)r * Dk + c * 8) : (const void*)qsrc, ok);
  }
  if (kt0 < kt1) load_keys(kt0, 0);
  else cp_async_commit();

  // rows g and g + 8 of this warp's 16: the last key position each may see (-1: no such item)
  int limit[2];
#pragma unroll
  for (int i = 0; i < 2; i++) {
    const int item = item0 + warp * 16 + g + 8 * i;
    limit[i] = item < n_items ? start + q0 + item / a.H : -1;
  }
  float o[NR][4];
#pragma unroll
  for (int dn = 0; dn < NR; dn++)
#pragma unroll
    for (int i = 0; i < 4; i++) o[dn][i] = 0.f;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
  const float scale_log2 = a.scale * 1.4426950408889634f;
  const int nks = KS ? KS : Dk / 16, nrt = KS ? NR : a.R / 8;

  int buf = 0;
  for (int kt = kt0; kt < kt1; kt++) {
    const bool more = kt + 1 < kt1;
    if (two_stage && more) {
      load_keys(kt + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t sK = sK0 + (two_stage ? buf : 0) * tile_bytes;
    const int kpos0 = kt * LM_KT;
    if (active) {
      float s[8][4];
#pragma unroll
      for (int nt = 0; nt < 8; nt++)
#pragma unroll
        for (int i = 0; i < 4; i++) s[nt][i] = 0.f;
      auto score_step = [&](int ks) {
        uint32_t q0r, q1r, q2r, q3r;
        ldsm_x4(sQ + ((warp * 16 + lr + (mi & 1) * 8) * ld + (ks * 2 + (mi >> 1)) * 8) * 2, q0r, q1r, q2r, q3r);
#pragma unroll
        for (int nt = 0; nt < 8; nt += 2) {
          uint32_t b0, b1, b2, b3;
          ldsm_x4(sK + ((nt * 8 + lr + (mi >> 1) * 8) * ld + (ks * 2 + (mi & 1)) * 8) * 2, b0, b1, b2, b3);
          mma16816(s[nt], q0r, q1r, q2r, q3r, b0, b1);
          mma16816(s[nt + 1], q0r, q1r, q2r, q3r, b2, b3);
        }
      };
      if constexpr (KS > 0) {
#pragma unroll
        for (int ks = 0; ks < KS; ks++) score_step(ks);
      } else {
        for (int ks = 0; ks < nks; ks++) score_step(ks);
      }
      // causal mask (keys past the CTA's range are zero-filled and masked the same way)
#pragma unroll
      for (int nt = 0; nt < 8; nt++) {
        const int kp = kpos0 + nt * 8 + 2 * t;
        if (kp > limit[0]) s[nt][0] = -INFINITY;
        if (kp + 1 > limit[0]) s[nt][1] = -INFINITY;
        if (kp > limit[1]) s[nt][2] = -INFINITY;
        if (kp + 1 > limit[1]) s[nt][3] = -INFINITY;
      }
#pragma unroll
      for (int i = 0; i < 2; i++) {
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; nt++) mx = fmaxf(mx, fmaxf(s[nt][2 * i], s[nt][2 * i + 1]));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m[i], mx);
        const float m_use = (m_new == -INFINITY) ? 0.f : m_new;
        const float corr = exp2f((m[i] - m_use) * scale_log2);  // m = -inf => 0
        m[i] = m_new;
        l[i] *= corr;
#pragma unroll
        for (int dn = 0; dn < NR; dn++) {
          o[dn][2 * i] *= corr;
          o[dn][2 * i + 1] *= corr;
        }
        float rs = 0.f;
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
          const float p0 = exp2f((s[nt][2 * i] - m_use) * scale_log2);
          const float p1 = exp2f((s[nt][2 * i + 1] - m_use) * scale_log2);
          s[nt][2 * i] = p0;
          s[nt][2 * i + 1] = p1;
          rs += p0 + p1;
        }
        l[i] += rs;  // per-thread partial; the quad is reduced once at the end
      }
#pragma unroll
      for (int kk = 0; kk < 4; kk++) {
        const uint32_t a0 = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        const uint32_t a1 = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        const uint32_t a2 = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        const uint32_t a3 = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int dn = 0; dn < NR; dn += 2) {
          if (dn < nrt) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(sK + ((kk * 16 + lr + (mi & 1) * 8) * ld + (dn + (mi >> 1)) * 8) * 2, b0, b1, b2, b3);
            mma16816(o[dn], a0, a1, a2, a3, b0, b1);
            mma16816(o[dn + 1], a0, a1, a2, a3, b2, b3);
          }
        }
      }
    }
    __syncthreads();  // the tile may be overwritten from here on
    if (!two_stage && more) load_keys(kt + 1, 0);
    buf ^= 1;
  }
  cp_async_wait<0>();
  TRACE_EXIT(tr);
#pragma unroll
  for (int i = 0; i < 2; i++) {
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
    l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
  }
#pragma unroll
  for (int i = 0; i < 2; i++) {
    const int item = item0 + warp * 16 + g + 8 * i;
    if (!active || item >= n_items) continue;
    const size_t it = (size_t)(row0 + q0) * a.H + item;  // row * H + head
    if (gridDim.z == 1) {
      const int row = row0 + q0 + item / a.H, head = item % a.H;
      const float inv = a.gate[it] / l[i];  // the head's sigmoid gate rides on the normalisation
      bf16* op = (bf16*)a.olat + (size_t)row * a.o_ld + head * a.R;
#pragma unroll
      for (int dn = 0; dn < NR; dn++)
        if (dn < nrt)
          *reinterpret_cast<uint32_t*>(op + dn * 8 + 2 * t) = pack_bf16(o[dn][2 * i] * inv, o[dn][2 * i + 1] * inv);
      if (head == a.H - 1)  // padding columns of the output projection's input
        for (int r = a.H * a.R + t; r < a.o_ld; r += 4) ((bf16*)a.olat)[(size_t)row * a.o_ld + r] = __float2bfloat16_rn(0.f);
    } else {
      float* rec = a.split_ws + (it * gridDim.z + blockIdx.z) * (a.R + 2);
#pragma unroll
      for (int dn = 0; dn < NR; dn++)
        if (dn < nrt) {
          rec[dn * 8 + 2 * t] = o[dn][2 * i];
          rec[dn * 8 + 2 * t + 1] = o[dn][2 * i + 1];
        }
      if (t == 0) {
        rec[a.R] = m[i] * a.scale;  // the combine kernel works on scaled scores
        rec[a.R + 1] = l[i];
      }
    }
  }
}

static bool latent_mma_enabled() {
  static const bool on = !(getenv("NVLLM_LATENT_MMA") && atoi(getenv("NVLLM_LATENT_MMA")) == 0);
  return on;
}
static bool latent_mma_ok(int qdt, int kvdt, const LatentArgs& a) {
  return latent_mma_enabled() && qdt == DT_BF16 && kvdt == DT_BF16 && ((a.R + a.rot) % 16) == 0 && (a.R % 16) == 0 &&
         a.R <= 256 && a.scale > 0.f;
}
template <int NR, int ROWS, int KS>
static cudaError_t launch_latent_mma_ks(cudaStream_t st, const LatentArgs& a, int ns) {
  const int Dk = a.R + a.rot;
  const size_t one = (size_t)LM_KT * (Dk + 8) * 2, qb = (size_t)ROWS * (Dk + 8) * 2;
  const int two = qb + 2 * one <= 200 * 1024 ? 1 : 0;
  const size_t smem = qb + one * (two ? 2 : 1);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(latent_attn_mma_kernel<NR, ROWS, KS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  dim3 grid(a.n_tiles, ceil_div(a.qtile * a.H, ROWS), ns);
  // CTAs of fewer than 64 rows: a few of them per SM are bound by the latency of staging a key
  // tile, so two more warps help with the copies; many per SM are bound by the tensor pipe, and
  // idle warps would only take registers from resident CTAs
  int threads = ROWS * 2;
  if (ROWS < 64 && (long)grid.x * grid.y * grid.z < 3L * a.sm_count) threads = 128;
  (void)launch_k(latent_attn_mma_kernel<NR, ROWS, KS>, grid, dim3(threads), smem, st, a, two, next_trace(22));
  return cudaGetLastError();
}
// rows of kv_rank = NR * 8 with a rotated part of 16, 32 or 64 take the kernel specialised on the row size
template <int NR, int ROWS>
static cudaError_t launch_latent_mma_r(cudaStream_t st, const LatentArgs& a, int ns) {
  if (a.R == NR * 8) {
    if (a.rot == 16) return launch_latent_mma_ks<NR, ROWS, NR / 2 + 1>(st, a, ns);
    if (a.rot == 32) return launch_latent_mma_ks<NR, ROWS, NR / 2 + 2>(st, a, ns);
    if (a.rot == 64) return launch_latent_mma_ks<NR, ROWS, NR / 2 + 4>(st, a, ns);
  }
  return launch_latent_mma_ks<NR, ROWS, 0>(st, a, ns);
}
// 128 items per CTA (8 warps) when a tile has that many: each staged key tile then serves twice the rows
template <int NR>
static cudaError_t launch_latent_mma(cudaStream_t st, const LatentArgs& a, int ns) {
  const int items = a.qtile * a.H;
  if (NR <= 16 && items >= 128) return launch_latent_mma_r<NR, 128>(st, a, ns);
  if (items <= 16) return launch_latent_mma_r<NR, 16>(st, a, ns);
  if (items <= 32) return launch_latent_mma_r<NR, 32>(st, a, ns);
  return launch_latent_mma_r<NR, 64>(st, a, ns);
}

template <typename QT>
__global__ void latent_combine_kernel(LatentArgs a, int n_splits, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  const size_t item = blockIdx.x;  // row * H + head
  const float* rec = a.split_ws + item * n_splits * (a.R + 2);
  float m = -INFINITY;
  for (int s = 0; s < n_splits; s++) m = fmaxf(m, rec[(size_t)s * (a.R + 2) + a.R]);
  float l = 0.f;
  for (int s = 0; s < n_splits; s++) {
    const float ms = rec[(size_t)s * (a.R + 2) + a.R];
    if (ms != -INFINITY) l += rec[(size_t)s * (a.R + 2) + a.R + 1] * expf(ms - m);
  }
  const size_t row = item / a.H;
  const int head = (int)(item % a.H);
  QT* op = (QT*)a.olat + row * a.o_ld + head * a.R;
  const float inv = a.gate[item] / l;
  for (int r = threadIdx.x; r < a.R; r += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < n_splits; s++) {
      const float ms = rec[(size_t)s * (a.R + 2) + a.R];
      if (ms != -INFINITY) o += rec[(size_t)s * (a.R + 2) + r] * expf(ms - m);
    }
    op[r] = from_f32<QT>(o * inv);
  }
  if (head == a.H - 1)
    for (int r = a.H * a.R + threadIdx.x; r < a.o_ld; r += blockDim.x)
      ((QT*)a.olat)[row * a.o_ld + r] = from_f32<QT>(0.f);
  TRACE_EXIT(tr);
}

int latent_attn_qtile() { return LAT_QTILE; }

int latent_attn_splits(int n_seqs, int H, int max_len, int sm_count) {
  static const int forced = getenv("NVLLM_LATENT_SPLITS") ? atoi(getenv("NVLLM_LATENT_SPLITS")) : 0;
  if (forced > 0) return min(forced, 64);
  // decode is latency-bound per key tile (a cached row is a few hundred bytes for all heads):
  // about three 64-key tiles per split, as long as all CTAs of the step stay resident
  const int ctas = n_seqs * ceil_div(H, 64);
  int ns = ceil_div(ceil_div(max_len, 64), 3);
  ns = min(ns, max(1, 4 * sm_count / max(1, ctas)));
  return max(1, min(ns, 32));
}

cudaError_t launch_latent_attn(cudaStream_t st, int qdt, int kvdt, const LatentArgs& a) {
  if (a.n_tiles <= 0) return cudaSuccess;
  if (a.R > 32 * LAT_NACC || (KV_BLOCK % LAT_KT) != 0) return cudaErrorInvalidValue;
  const int Dk = a.R + a.rot;
  const size_t smem = ((size_t)LAT_KT * (Dk + 1) + (size_t)LAT_WARPS * Dk) * sizeof(float);
  const int ns = max(1, a.n_splits);
  dim3 grid(a.n_tiles, ceil_div(a.qtile * a.H, LAT_WARPS), ns);
  if (latent_mma_ok(qdt, kvdt, a)) {
    cudaError_t e = a.R <= 64 ? launch_latent_mma<8>(st, a, ns)
                    : a.R <= 128 ? launch_latent_mma<16>(st, a, ns) : launch_latent_mma<32>(st, a, ns);
    if (e != cudaSuccess) return e;
    if (ns > 1) (void)launch_k(latent_combine_kernel<bf16>, dim3(a.T * a.H), dim3(64), 0, st, a, ns, next_trace(23));
    return cudaGetLastError();
  }
  if (qdt == DT_F32 && kvdt == DT_F32) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(latent_attn_kernel<float, float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    (void)launch_k(latent_attn_kernel<float, float>, grid, dim3(LAT_WARPS * 32), smem, st, a, next_trace(22));
    if (ns > 1) (void)launch_k(latent_combine_kernel<float>, dim3(a.T * a.H), dim3(64), 0, st, a, ns, next_trace(23));
  } else if (qdt == DT_BF16 && kvdt == DT_BF16) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(latent_attn_kernel<bf16, bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    (void)launch_k(latent_attn_kernel<bf16, bf16>, grid, dim3(LAT_WARPS * 32), smem, st, a, next_trace(22));
    if (ns > 1) (void)launch_k(latent_combine_kernel<bf16>, dim3(a.T * a.H), dim3(64), 0, st, a, ns, next_trace(23));
  } else {
    return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

// logits <- cap * tanh(logits / cap), summing S split-K slices on the way
__global__ void softcap_kernel(const float* __restrict__ p, int S, size_t stride, size_t n, float cap,
                               float* __restrict__ out) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < S; k++) s += p[(size_t)k * stride + i];
    out[i] = cap > 0.f ? cap * tanhf(s / cap) : s;
  }
}
cudaError_t launch_softcap(cudaStream_t st, const float* p, int S, size_t stride, size_t n, float cap,
                           float* out) {
  if (n == 0) return cudaSuccess;
  const int blocks = (int)min((size_t)148 * 8, (n + 255) / 256);
  (void)launch_k(softcap_kernel, dim3(blocks), dim3(256), 0, st, p, S, stride, n, cap, out);
  return cudaGetLastError();
}

}  // namespace nvllm
