// linrec.cu — linear recurrences with a diagonal decay, for the layers of a model given as a list
// (nvllm_mixer_kind NVLLM_MIXER_GLA and the time-mixing side of NVLLM_MIXER_ATTN_TMIX).
//
// Per head a dim x vdim state S in fp32, zero at a sequence's start, kept per state slot:
//   gated linear attention   a_t = sigmoid(z_t)^(1 / tau),  S <- diag(a_t) S + k_t v_t^T,  o_t = S^T q_t
//   time mixing              w_t = exp(-exp(z_t)),  o_t = (S + diag(u) k_t v_t^T)^T r_t,  S <- diag(w_t) S + k_t v_t^T
// with z_t = W_2 f(W_1 x_t) + b per (head, key entry): f = identity / tanh.  The decay rows belong to
// key entries.  The read-out of a head is divided by its root mean square, multiplied by a weight
// and by silu(gate) and goes to the output projection.
//
//   linrec_prep_kernel   per tile of tokens: split-K sums of the projections, q scaled, the second step of
//                        the decay's projection (fp32 FMA, the inner size is small) and the decay itself —
//                        logarithms, exponentials and sigmoids in fp32 (log-sigmoid form, no overflow).
//   linrec_scan_kernel   CTA = (sequence, head, 32 CC value columns), NW warps.  A column of the state is
//                        independent of the others; a warp holds a slice of the rows (RPL each, dealt in
//                        groups of four), a lane CC columns of that slice in registers.  Per token one pass
//                        over the rows; the lanes of a warp read the same q / k / decay entries (broadcast
//                        16-byte loads).  Token inputs are staged through shared memory in chunks, the next
//                        chunk's loads in flight (cp.async) while the current one is scanned; the warps'
//                        partial read-outs meet in shared memory once per chunk.  State read from the slot
//                        when the sequence has earlier tokens, written back at the end.
//   linrec_out_kernel    per token, a warp per head: RMS over vdim, weight, silu(gate) -> act dtype.
//   linrec_decode_kernel steps with one row per sequence (decode): the three kernels above as one launch per layer.
//   token_shift_kernel   the inputs of time mixing's projections: h_t + (h_{t-1} - h_t) mu_s.
//   roll_tails_kernel    after a step, the last inputs of a short convolution / token shift become
//                        the slot's tail (one thread per channel reads all it needs, then writes).
#include <stdlib.h>

#include <algorithm>

#include "common.cuh"
#include "kernels.h"
#include "mma.cuh"

namespace nvllm {

namespace {
__device__ __forceinline__ int lr_seq_of_row(const int* __restrict__ cu_q, int n_seqs, int row) {
  int lo = 0, hi = n_seqs - 1;  // last s with cu_q[s] <= row
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_q[mid] <= row) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}
__device__ __forceinline__ float seg_at(const LinSeg& g, int t, int c) {
  const float* p = g.p + (size_t)t * g.ld + c;
  float acc = 0.f;
  for (int s = 0; s < g.S; s++) acc += p[(size_t)s * g.stride];
  return acc;
}
// q, k and v projections that came out as one slice each need no summing: the scan reads them
// where the GEMMs left them and the prep kernel writes only the decay
__host__ __device__ __forceinline__ bool linrec_direct(const LinRecArgs& a) { return a.q.S == 1 && a.k.S == 1 && a.v.S == 1; }
__device__ __forceinline__ void lr_cp_async4(uint32_t dst, const void* src, bool ok) {
  const int n = ok ? 4 : 0;  // src-size 0: the destination is filled with zeros
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(n) : "memory");
}
}  // namespace

// ------------------------------------------------------------------ projections' epilogue
// grid (ceil(T / TT), Y), 256 threads: a CTA takes TT tokens, a thread one of the H * dim key
// entries at a time.  Output: qkw rows [q | k | decay] and vv (q unscaled: the scan scales its read-outs).  The entry's row of the decay's second-step matrix is read once (16 floats
// at a time, in registers) for all TT tokens, whose inner vectors sit in shared memory and are
// read as broadcasts — the matrix crosses L2 once per TT tokens instead of once per token.
constexpr int LP_RC = 16;  // inner entries per register chunk
constexpr int TAIL_MAX_TAPS_C = 8;  // most taps of a short convolution

template <int TT>
__global__ void __launch_bounds__(256) linrec_prep_kernel(LinRecArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  extern __shared__ __align__(16) float lr[];  // [TT][rank_p], rank_p = rank rounded up to LP_RC, zero padded
  pdl_wait();
  const int t0 = blockIdx.x * TT;
  const int nt = min(TT, a.T - t0);
  const int rank_p = (a.rank + LP_RC - 1) / LP_RC * LP_RC;
  const int hd = a.H * a.dim, hv = a.H * a.vdim;
  for (int i = threadIdx.x; i < TT * rank_p; i += blockDim.x) {
    const int tt = i / rank_p, r = i % rank_p;
    float x = 0.f;
    if (tt < nt && r < a.rank) {
      x = seg_at(a.lr, t0 + tt, r);
      if (a.tmix) x = tanhf(x);
    }
    lr[i] = x;
  }
  __syncthreads();
  const float inv_tau = 1.0f / a.tau;
  const bool vec_ok = (a.rank % 4) == 0;
  const bool direct = linrec_direct(a);
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < hd; c += gridDim.y * blockDim.x) {
    const float* w = a.w2 + (size_t)c * a.rank;
    float z[TT];
#pragma unroll
    for (int tt = 0; tt < TT; tt++) z[tt] = 0.f;
    for (int r0 = 0; r0 < a.rank; r0 += LP_RC) {
      float wr[LP_RC];
      if (vec_ok && r0 + LP_RC <= a.rank) {
#pragma unroll
        for (int q = 0; q < LP_RC / 4; q++) {
          const float4 v = *reinterpret_cast<const float4*>(w + r0 + 4 * q);
          wr[4 * q] = v.x; wr[4 * q + 1] = v.y; wr[4 * q + 2] = v.z; wr[4 * q + 3] = v.w;
        }
      } else {
#pragma unroll
        for (int q = 0; q < LP_RC; q++) wr[q] = r0 + q < a.rank ? w[r0 + q] : 0.f;
      }
#pragma unroll
      for (int tt = 0; tt < TT; tt++) {
        const float* l = lr + tt * rank_p + r0;
#pragma unroll
        for (int q = 0; q < LP_RC / 4; q++) {
          const float4 v = *reinterpret_cast<const float4*>(l + 4 * q);
          z[tt] = fmaf(wr[4 * q], v.x, z[tt]);
          z[tt] = fmaf(wr[4 * q + 1], v.y, z[tt]);
          z[tt] = fmaf(wr[4 * q + 2], v.z, z[tt]);
          z[tt] = fmaf(wr[4 * q + 3], v.w, z[tt]);
        }
      }
    }
    const float b = a.w2b[c];
    float qv[TT], kv[TT];
    if (!direct) {  // all the loads first
#pragma unroll
      for (int tt = 0; tt < TT; tt++)
        if (tt < nt) {
          qv[tt] = seg_at(a.q, t0 + tt, c);
          kv[tt] = seg_at(a.k, t0 + tt, c);
        }
    }
#pragma unroll
    for (int tt = 0; tt < TT; tt++) {
      if (tt >= nt) break;
      const float zz = z[tt] + b;
      float decay;
      if (a.tmix) {
        decay = expf(-expf(zz));
      } else {
        // sigmoid(z)^(1 / tau) = exp(log sigmoid(z) / tau), log sigmoid(z) = min(z, 0) - log1p(exp(-|z|))
        const float ls = fminf(zz, 0.f) - log1pf(expf(-fabsf(zz)));
        decay = expf(ls * inv_tau);
      }
      float* qkw = a.qkw + (size_t)(t0 + tt) * 3 * hd;
      if (!direct) {
        qkw[c] = qv[tt];
        qkw[hd + c] = kv[tt];
      }
      qkw[2 * hd + c] = decay;
    }
  }
  if (direct) return;
  for (int tt = 0; tt < nt; tt++) {
    float* vv = a.vv + (size_t)(t0 + tt) * hv;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < hv; c += gridDim.y * blockDim.x) vv[c] = seg_at(a.v, t0 + tt, c);
  }
  TRACE_EXIT(tr);
}

cudaError_t launch_linrec_prep(cudaStream_t st, const LinRecArgs& a) {
  if (a.T <= 0) return cudaSuccess;
  const int big = std::max(a.H * a.dim, a.H * a.vdim);
  const int rank_p = (a.rank + LP_RC - 1) / LP_RC * LP_RC;
  if (a.T >= 2048) {
    const size_t smem = (size_t)16 * rank_p * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(linrec_prep_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    (void)launch_k(linrec_prep_kernel<16>, dim3(ceil_div(a.T, 16), std::min(4, ceil_div(big, 256))), dim3(256), smem, st, a,
                   next_trace(40));
  } else if (a.T >= 512) {
    const size_t smem = (size_t)4 * rank_p * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(linrec_prep_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    (void)launch_k(linrec_prep_kernel<4>, dim3(ceil_div(a.T, 4), std::min(8, ceil_div(big, 256))), dim3(256), smem, st, a,
                   next_trace(40));
  } else {  // decode-sized steps: latency matters, not the matrix's trips through L2 — a CTA per token and 256 entries
    const size_t smem = (size_t)rank_p * sizeof(float);
    if (smem > 48 * 1024) cudaFuncSetAttribute(linrec_prep_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    (void)launch_k(linrec_prep_kernel<1>, dim3(a.T, std::min(16, ceil_div(big, 256))), dim3(256), smem, st, a, next_trace(40));
  }
  return cudaGetLastError();
}

// ------------------------------------------------------------------ scan over tokens
// A warp holds one slice of the state's rows (RPL rows, dealt in groups of four), its lanes the
// value columns (CC each): all lanes of a warp read the SAME q / k / decay entries — one
// broadcast per 16-byte load instead of a pass per quarter warp — and the NW warps' partial
// read-outs of a chunk of tokens meet in shared memory once per chunk.
template <int RPL, int NW, int CC, bool TMIX>
__global__ void __launch_bounds__(32 * NW) linrec_scan_kernel(LinRecArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  constexpr int NT = 32 * NW;
  constexpr int DP = RPL * NW;            // rows of the state, padded
  constexpr int VC = 32 * CC;             // value columns of this CTA
  constexpr int TC = DP >= 256 ? 4 : 8;   // tokens per staged chunk
  constexpr int ROW = 3 * DP + VC;        // floats of one staged token: q | k | decay | v
  __shared__ __align__(16) float stage[2][TC][ROW];
  __shared__ float part[NW][TC][VC];
  const int seq = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * VC;
  const int tid = threadIdx.x;
  const int l = tid >> 5, lane = tid & 31;  // row slice, column group
  const int dim = a.dim, vdim = a.vdim, hd = a.H * dim, hv = a.H * vdim;
  pdl_wait();
  const int r0 = a.cu_q[seq], n_new = a.cu_q[seq + 1] - r0;
  if (n_new <= 0) return;
  const bool has_prev = a.positions[r0] > 0;
  float* state = a.state_pool + (size_t)a.state_slots[seq] * a.slot_floats + a.state_off + (size_t)head * dim * vdim;

  // q | k | decay | v of the step's rows: the projections' own output when it needs no summing
  const bool direct = linrec_direct(a);
  const float* part_p[3] = {direct ? a.q.p : a.qkw, direct ? a.k.p : a.qkw + hd, a.qkw + 2 * hd};
  const size_t part_ld[3] = {direct ? (size_t)a.q.ld : (size_t)3 * hd, direct ? (size_t)a.k.ld : (size_t)3 * hd, (size_t)3 * hd};
  const float* v_p = direct ? a.v.p : a.vv;
  const size_t v_ld = direct ? (size_t)a.v.ld : (size_t)hv;
  const int qk_head = a.qk_div > 1 ? head / a.qk_div : head;
  auto load_chunk = [&](int t0, int buf) {
    const int nt = min(TC, n_new - t0);
    for (int i = tid; i < TC * 3 * DP; i += NT) {
      const int tt = i / (3 * DP), j = i % (3 * DP), pt = j / DP, r = j % DP;
      const bool ok = tt < nt && r < dim;
      const size_t trow = (size_t)(r0 + t0 + (ok ? tt : 0));
      const float* src = (pt == 2 && a.decay_p) ? a.decay_p + trow * a.decay_ld + head
                                                : part_p[pt] + trow * part_ld[pt] + (pt < 2 ? qk_head : head) * dim + (ok ? r : 0);
      lr_cp_async4(smem_addr(&stage[buf][tt][j]), src, ok);
    }
    for (int i = tid; i < TC * VC; i += NT) {
      const int tt = i / VC, c = i % VC;
      const bool ok = tt < nt && col0 + c < vdim;
      const float* src = v_p + (size_t)(r0 + t0 + (ok ? tt : 0)) * v_ld + head * vdim + (ok ? col0 + c : 0);
      lr_cp_async4(smem_addr(&stage[buf][tt][3 * DP + c]), src, ok);
    }
  };
  load_chunk(0, 0);
  cp_async_commit();

  float S[CC][RPL], U[TMIX ? RPL : 1];
#pragma unroll
  for (int g = 0; g < RPL / 4; g++)
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const int r = (g * NW + l) * 4 + e;
#pragma unroll
      for (int cc = 0; cc < CC; cc++) {
        const int col = col0 + cc * 32 + lane;
        S[cc][g * 4 + e] = (r < dim && col < vdim && has_prev) ? state[(size_t)r * vdim + col] : 0.f;
      }
      if (TMIX) U[g * 4 + e] = r < dim ? a.bonus[head * dim + r] : 0.f;
    }

  const int n_chunks = (n_new + TC - 1) / TC;
  for (int ch = 0; ch < n_chunks; ch++) {
    const int buf = ch & 1;
    if (ch + 1 < n_chunks) load_chunk((ch + 1) * TC, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int nt = min(TC, n_new - ch * TC);
#pragma unroll
    for (int tt = 0; tt < TC; tt++) {
      if (tt >= nt) break;
      const float* row = stage[buf][tt];
      float v[CC], acc[CC];
#pragma unroll
      for (int cc = 0; cc < CC; cc++) {
        v[cc] = row[3 * DP + cc * 32 + lane];
        acc[cc] = 0.f;
      }
#pragma unroll
      for (int g = 0; g < RPL / 4; g++) {
        const int rb = (g * NW + l) * 4;
        const float4 q4 = *reinterpret_cast<const float4*>(row + rb);
        const float4 k4 = *reinterpret_cast<const float4*>(row + DP + rb);
        const float4 w4 = *reinterpret_cast<const float4*>(row + 2 * DP + rb);
        const float qq[4] = {q4.x, q4.y, q4.z, q4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w}, ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
        for (int e = 0; e < 4; e++) {
#pragma unroll
          for (int cc = 0; cc < CC; cc++) {
            float& s = S[cc][g * 4 + e];
            if (TMIX) {
              const float kv = kk[e] * v[cc];
              acc[cc] = fmaf(qq[e], fmaf(U[g * 4 + e], kv, s), acc[cc]);
              s = fmaf(ww[e], s, kv);
            } else {
              s = fmaf(ww[e], s, kk[e] * v[cc]);
              acc[cc] = fmaf(qq[e], s, acc[cc]);
            }
          }
        }
      }
#pragma unroll
      for (int cc = 0; cc < CC; cc++) part[l][tt][cc * 32 + lane] = acc[cc];
    }
    __syncthreads();  // the slices' partial read-outs are in; the staged chunk has been consumed
    for (int i = tid; i < nt * VC; i += NT) {
      const int tt = i / VC, c = i % VC;
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < NW; w++) t += part[w][tt][c];
      if (col0 + c < vdim) a.o[(size_t)(r0 + ch * TC + tt) * hv + head * vdim + col0 + c] = t * a.qmul;
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int g = 0; g < RPL / 4; g++)
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const int r = (g * NW + l) * 4 + e;
#pragma unroll
      for (int cc = 0; cc < CC; cc++) {
        const int col = col0 + cc * 32 + lane;
        if (r < dim && col < vdim) state[(size_t)r * vdim + col] = S[cc][g * 4 + e];
      }
    }
  TRACE_EXIT(tr);
}

template <int RPL, int NW, int CC>
static cudaError_t linrec_scan_launch_cc(cudaStream_t st, const LinRecArgs& a) {
  const dim3 grid(a.n_seqs, a.H, ceil_div(a.vdim, 32 * CC));
  if (a.tmix) (void)launch_k(linrec_scan_kernel<RPL, NW, CC, true>, grid, dim3(32 * NW), 0, st, a, next_trace(41));
  else (void)launch_k(linrec_scan_kernel<RPL, NW, CC, false>, grid, dim3(32 * NW), 0, st, a, next_trace(41));
  return cudaGetLastError();
}
template <int RPL, int NW>
static cudaError_t linrec_scan_launch(cudaStream_t st, const LinRecArgs& a) {
  // more columns per lane where a head has that many (a row's q / k / decay is read once for all of
  // them) — as long as the grid still fills the GPU twice over: a sequence's tokens are scanned in
  // order, so few long sequences want many narrow CTAs
  const long units = (long)a.n_seqs * a.H;
  const long want = 2 * 148;
  if (RPL <= 16 && a.vdim >= 128 && units * ceil_div(a.vdim, 128) >= want) return linrec_scan_launch_cc<RPL, NW, 4>(st, a);
  if (a.vdim >= 64 && units * ceil_div(a.vdim, 64) >= want) return linrec_scan_launch_cc<RPL, NW, 2>(st, a);
  return linrec_scan_launch_cc<RPL, NW, 1>(st, a);
}

cudaError_t launch_linrec_scan(cudaStream_t st, const LinRecArgs& a) {
  if (a.T <= 0 || a.n_seqs <= 0) return cudaSuccess;
  if (a.dim > LINREC_MAX_DIM || (a.tmix && !a.bonus)) return cudaErrorInvalidValue;
  if (a.dim <= 16) return linrec_scan_launch<4, 4>(st, a);
  if (a.dim <= 32) return linrec_scan_launch<8, 4>(st, a);
  if (a.dim <= 64) return linrec_scan_launch<16, 4>(st, a);
  if (a.dim <= 128) return linrec_scan_launch<32, 4>(st, a);
  return linrec_scan_launch<32, 8>(st, a);
}

// ------------------------------------------------------------------ one token per sequence: everything in one kernel
// A decode step gives every sequence one row, and a head whose value columns fit one CTA
// (vdim <= 32 CC) needs nothing from other CTAs: the projections' epilogue (split-K sums, the
// decay), the state update with its read-out, the head's RMS norm, weight and gate run as ONE
// launch per layer instead of three.  CTA = (sequence, head); the state slice of a thread is as
// in linrec_scan_kernel and its loads are in flight while the row's inputs are prepared.
template <int RPL, int NW, int CC, bool TMIX>
__global__ void __launch_bounds__(32 * NW) linrec_decode_kernel(LinRecArgs a, int out_bf16, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  constexpr int NT = 32 * NW;
  constexpr int DP = RPL * NW;
  constexpr int VC = 32 * CC;
  extern __shared__ __align__(16) float sm[];
  float* sq = sm;                 // [DP] q | [DP] k | [DP] decay
  float* sv = sm + 3 * DP;        // [VC]
  float* part = sv + VC;          // [NW][VC]
  float* slr = part + NW * VC;    // [rank]
  __shared__ float red[32];
  const int t = blockIdx.x, head = blockIdx.y;
  const int tid = threadIdx.x, l = tid >> 5, lane = tid & 31;
  const int dim = a.dim, vdim = a.vdim;
  pdl_wait();
  const bool has_prev = a.positions[t] > 0;
  float* state = a.state_pool + (size_t)a.state_slots[t] * a.slot_floats + a.state_off + (size_t)head * dim * vdim;
  float S[CC][RPL], U[TMIX ? RPL : 1];
#pragma unroll
  for (int g = 0; g < RPL / 4; g++)
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const int r = (g * NW + l) * 4 + e;
#pragma unroll
      for (int cc = 0; cc < CC; cc++) {
        const int col = cc * 32 + lane;
        S[cc][g * 4 + e] = (r < dim && col < vdim && has_prev) ? state[(size_t)r * vdim + col] : 0.f;
      }
      if (TMIX) U[g * 4 + e] = r < dim ? a.bonus[head * dim + r] : 0.f;
    }
  for (int r = tid; r < a.rank; r += NT) {
    const float x = seg_at(a.lr, t, r);
    slr[r] = a.tmix ? tanhf(x) : x;
  }
  for (int c = tid; c < VC; c += NT) sv[c] = c < vdim ? seg_at(a.v, t, head * vdim + c) : 0.f;
  __syncthreads();
  const float inv_tau = 1.0f / a.tau;
  for (int i = tid; i < DP; i += NT) {
    float q = 0.f, k = 0.f, decay = 0.f;
    if (i < dim) {
      const int c = head * dim + i;
      const float* w = a.w2 + (size_t)c * a.rank;
      float z = 0.f;
      if ((a.rank & 3) == 0) {  // 16-byte loads of the matrix row, four at a time in flight
#pragma unroll 4
        for (int r = 0; r < a.rank; r += 4) {
          const float4 wv = *reinterpret_cast<const float4*>(w + r);
          z = fmaf(wv.x, slr[r], z);
          z = fmaf(wv.y, slr[r + 1], z);
          z = fmaf(wv.z, slr[r + 2], z);
          z = fmaf(wv.w, slr[r + 3], z);
        }
      } else {
        for (int r = 0; r < a.rank; r++) z = fmaf(w[r], slr[r], z);
      }
      z += a.w2b[c];
      if (a.tmix) {
        decay = expf(-expf(z));
      } else {
        const float ls = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));  // log sigmoid(z)
        decay = expf(ls * inv_tau);
      }
      q = seg_at(a.q, t, c);
      k = seg_at(a.k, t, c);
    }
    sq[i] = q;
    sq[DP + i] = k;
    sq[2 * DP + i] = decay;
  }
  __syncthreads();
  float v[CC], acc[CC];
#pragma unroll
  for (int cc = 0; cc < CC; cc++) {
    v[cc] = sv[cc * 32 + lane];
    acc[cc] = 0.f;
  }
#pragma unroll
  for (int g = 0; g < RPL / 4; g++) {
    const int rb = (g * NW + l) * 4;
    const float4 q4 = *reinterpret_cast<const float4*>(sq + rb);
    const float4 k4 = *reinterpret_cast<const float4*>(sq + DP + rb);
    const float4 w4 = *reinterpret_cast<const float4*>(sq + 2 * DP + rb);
    const float qq[4] = {q4.x, q4.y, q4.z, q4.w}, kk[4] = {k4.x, k4.y, k4.z, k4.w}, ww[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
    for (int e = 0; e < 4; e++) {
#pragma unroll
      for (int cc = 0; cc < CC; cc++) {
        float& st = S[cc][g * 4 + e];
        if (TMIX) {
          const float kv = kk[e] * v[cc];
          acc[cc] = fmaf(qq[e], fmaf(U[g * 4 + e], kv, st), acc[cc]);
          st = fmaf(ww[e], st, kv);
        } else {
          st = fmaf(ww[e], st, kk[e] * v[cc]);
          acc[cc] = fmaf(qq[e], st, acc[cc]);
        }
      }
    }
  }
#pragma unroll
  for (int cc = 0; cc < CC; cc++) part[l * VC + cc * 32 + lane] = acc[cc];
#pragma unroll
  for (int g = 0; g < RPL / 4; g++)
#pragma unroll
    for (int e = 0; e < 4; e++) {
      const int r = (g * NW + l) * 4 + e;
#pragma unroll
      for (int cc = 0; cc < CC; cc++) {
        const int col = cc * 32 + lane;
        if (r < dim && col < vdim) state[(size_t)r * vdim + col] = S[cc][g * 4 + e];
      }
    }
  __syncthreads();
  // the head's read-out: a thread per column (NT >= 128 >= VC)
  float o = 0.f, gt = 0.f, wn = 0.f;
  const bool mine = tid < vdim;
  if (mine) {
#pragma unroll
    for (int w = 0; w < NW; w++) o += part[w * VC + tid];
    o *= a.qmul;
    gt = seg_at(a.gate, t, head * vdim + tid);
    wn = a.onorm_w[(size_t)head * a.onorm_ld + tid];
  }
  const float inv = 1.0f / sqrtf(block_sum(o * o, red) / (float)vdim + a.eps);
  const float res = o * inv * wn * silu(gt);
  if (out_bf16) {
    bf16* out = (bf16*)a.out + (size_t)t * a.o_ld;
    if (mine) out[head * vdim + tid] = __float2bfloat16_rn(res);
    if (head == 0)
      for (int c = a.H * vdim + tid; c < a.o_ld; c += NT) out[c] = __float2bfloat16_rn(0.f);
  } else {
    float* out = (float*)a.out + (size_t)t * a.o_ld;
    if (mine) out[head * vdim + tid] = res;
    if (head == 0)
      for (int c = a.H * vdim + tid; c < a.o_ld; c += NT) out[c] = 0.f;
  }
  TRACE_EXIT(tr);
}

template <int RPL, int NW, int CC>
static cudaError_t linrec_decode_launch_cc(cudaStream_t st, int odt, const LinRecArgs& a) {
  const size_t smem = (size_t)(3 * RPL * NW + 32 * CC + NW * 32 * CC + a.rank) * sizeof(float);
  const int bf = odt == DT_BF16;
  if (a.tmix) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(linrec_decode_kernel<RPL, NW, CC, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    (void)launch_k(linrec_decode_kernel<RPL, NW, CC, true>, dim3(a.T, a.H), dim3(32 * NW), smem, st, a, bf, next_trace(45));
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(linrec_decode_kernel<RPL, NW, CC, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    (void)launch_k(linrec_decode_kernel<RPL, NW, CC, false>, dim3(a.T, a.H), dim3(32 * NW), smem, st, a, bf, next_trace(45));
  }
  return cudaGetLastError();
}
template <int RPL, int NW>
static cudaError_t linrec_decode_launch(cudaStream_t st, int odt, const LinRecArgs& a) {
  if (a.vdim <= 32) return linrec_decode_launch_cc<RPL, NW, 1>(st, odt, a);
  if (a.vdim <= 64) return linrec_decode_launch_cc<RPL, NW, 2>(st, odt, a);
  return linrec_decode_launch_cc<RPL, NW, 4>(st, odt, a);
}
bool linrec_decode_fused_ok(const LinRecArgs& a) {
  static const bool on = [] {
    const char* e = getenv("NVLLM_LINREC_FUSED");
    return e ? atoi(e) != 0 : true;
  }();
  return on && a.T == a.n_seqs && a.vdim <= 128 && a.dim <= LINREC_MAX_DIM;
}
cudaError_t launch_linrec_decode(cudaStream_t st, int odt, const LinRecArgs& a) {
  if (a.T <= 0) return cudaSuccess;
  if (!linrec_decode_fused_ok(a) || (a.tmix && !a.bonus)) return cudaErrorInvalidValue;
  if (a.dim <= 16) return linrec_decode_launch<4, 4>(st, odt, a);
  if (a.dim <= 32) return linrec_decode_launch<8, 4>(st, odt, a);
  if (a.dim <= 64) return linrec_decode_launch<16, 4>(st, odt, a);
  if (a.dim <= 128) return linrec_decode_launch<32, 4>(st, odt, a);
  return linrec_decode_launch<32, 8>(st, odt, a);
}

// ------------------------------------------------------------------ gated norm of the read-out
template <typename OT>
__global__ void __launch_bounds__(256) linrec_out_kernel(LinRecArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int vdim = a.vdim;
  OT* out = (OT*)a.out + (size_t)t * a.o_ld;
  // 16-byte loads when every row and head starts on a 16-byte boundary
  const bool vec = (vdim % 4) == 0 && vdim <= 512 && (a.gate.ld % 4) == 0 && (a.gate.stride % 4) == 0 &&
                   (reinterpret_cast<size_t>(a.gate.p) % 16) == 0 && (a.onorm_ld % 4) == 0;
  for (int h = blockIdx.y * nw + warp; h < a.H; h += gridDim.y * nw) {
    const float* o = a.o + (size_t)t * a.H * vdim + (size_t)h * vdim;
    if (vec) {
      // four neighbouring columns per lane, all loads (read-outs, gate slices, weights) before the arithmetic
      constexpr int MJ = 4;  // vdim <= 512
      float4 ov[MJ], gv[MJ];
      float ss = 0.f;
#pragma unroll
      for (int j = 0; j < MJ; j++) {
        const int i = lane * 4 + 128 * j;
        if (i < vdim) {
          ov[j] = *reinterpret_cast<const float4*>(o + i);
          const float* gp = a.gate.p + (size_t)t * a.gate.ld + h * vdim + i;
          gv[j] = *reinterpret_cast<const float4*>(gp);
          for (int sl = 1; sl < a.gate.S; sl++) {
            const float4 x = *reinterpret_cast<const float4*>(gp + (size_t)sl * a.gate.stride);
            gv[j].x += x.x; gv[j].y += x.y; gv[j].z += x.z; gv[j].w += x.w;
          }
          ss += ov[j].x * ov[j].x + ov[j].y * ov[j].y + ov[j].z * ov[j].z + ov[j].w * ov[j].w;
        }
      }
      const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + a.eps);
      const float* w = a.onorm_w + (size_t)h * a.onorm_ld;
#pragma unroll
      for (int j = 0; j < MJ; j++) {
        const int i = lane * 4 + 128 * j;
        if (i < vdim) {
          const float4 w4 = *reinterpret_cast<const float4*>(w + i);
          const float r[4] = {ov[j].x * inv * w4.x * silu(gv[j].x), ov[j].y * inv * w4.y * silu(gv[j].y),
                              ov[j].z * inv * w4.z * silu(gv[j].z), ov[j].w * inv * w4.w * silu(gv[j].w)};
#pragma unroll
          for (int e = 0; e < 4; e++) out[h * vdim + i + e] = from_f32<OT>(r[e]);
        }
      }
      continue;
    }
    float ss = 0.f;
    for (int i = lane; i < vdim; i += 32) ss += o[i] * o[i];
    const float inv = 1.0f / sqrtf(warp_sum(ss) / (float)vdim + a.eps);
    const float* w = a.onorm_w + (size_t)h * a.onorm_ld;
    for (int i = lane; i < vdim; i += 32) {
      const float gt = seg_at(a.gate, t, h * vdim + i);
      out[h * vdim + i] = from_f32<OT>(o[i] * inv * w[i] * silu(gt));
    }
  }
  if (blockIdx.y == 0)
    for (int c = a.H * vdim + threadIdx.x; c < a.o_ld; c += blockDim.x) out[c] = from_f32<OT>(0.f);
  TRACE_EXIT(tr);
}

cudaError_t launch_linrec_out(cudaStream_t st, int odt, const LinRecArgs& a) {
  if (a.T <= 0) return cudaSuccess;
  const dim3 grid(a.T, a.T >= 1024 ? 1 : ceil_div(a.H, 8));
  if (odt == DT_F32) (void)launch_k(linrec_out_kernel<float>, grid, dim3(256), 0, st, a, next_trace(42));
  else (void)launch_k(linrec_out_kernel<bf16>, grid, dim3(256), 0, st, a, next_trace(42));
  return cudaGetLastError();
}

// ------------------------------------------------------------------ token shift
template <typename AT>
__global__ void __launch_bounds__(256) token_shift_kernel(int T, int n_seqs, int W, int n_mix, const AT* __restrict__ h,
                                                          const float* __restrict__ mu, const int* __restrict__ cu_q,
                                                          const int* __restrict__ positions,
                                                          const int* __restrict__ state_slots,
                                                          const float* __restrict__ state_pool, size_t slot_floats,
                                                          size_t tail_off, AT* __restrict__ out, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  // the row's sequence: every thread tests one sequence's range (one round trip, no dependent chain)
  __shared__ int s_seq;
  if (T == n_seqs) {
    if (threadIdx.x == 0) s_seq = t;
  } else {
    for (int i = threadIdx.x; i < n_seqs; i += blockDim.x)
      if (cu_q[i] <= t && t < cu_q[i + 1]) s_seq = i;
  }
  __syncthreads();
  const int s = s_seq;
  const int r0 = cu_q[s];
  const bool in_step = t > r0;
  const bool in_slot = !in_step && positions[t] > 0;
  const float* tail = state_pool + (size_t)state_slots[s] * slot_floats + tail_off;
  for (int i = threadIdx.x * 8; i < W; i += blockDim.x * 8) {  // W is a multiple of 8
    float x[8], xp[8];
    load8(h + (size_t)t * W + i, x);
    if (in_step) load8(h + (size_t)(t - 1) * W + i, xp);
    else if (in_slot) load8(tail + i, xp);
    else
#pragma unroll
      for (int e = 0; e < 8; e++) xp[e] = 0.f;
    for (int m = 0; m < n_mix; m++) {
      float w[8], y[8];
      load8(mu + (size_t)m * W + i, w);
#pragma unroll
      for (int e = 0; e < 8; e++) y[e] = fmaf(xp[e] - x[e], w[e], x[e]);
      store8(out + ((size_t)m * T + t) * W + i, y);
    }
  }
  TRACE_EXIT(tr);
}

cudaError_t launch_token_shift(cudaStream_t st, int adt, int T, int n_seqs, int W, int n_mix, const void* h,
                               const float* mu, const int* cu_q, const int* positions, const int* state_slots,
                               const float* state_pool, size_t slot_floats, size_t tail_off, void* out) {
  if (T <= 0) return cudaSuccess;
  if (adt == DT_F32)
    (void)launch_k(token_shift_kernel<float>, dim3(T), dim3(128), 0, st, T, n_seqs, W, n_mix, (const float*)h, mu, cu_q,
                   positions, state_slots, state_pool, slot_floats, tail_off, (float*)out, next_trace(43));
  else
    (void)launch_k(token_shift_kernel<bf16>, dim3(T), dim3(128), 0, st, T, n_seqs, W, n_mix, (const bf16*)h, mu, cu_q,
                   positions, state_slots, state_pool, slot_floats, tail_off, (bf16*)out, next_trace(43));
  return cudaGetLastError();
}

// ------------------------------------------------------------------ convolution on a mixer's input
// One CTA per token; TAPS > 0: the number of taps at compile time.  Where tap j's input lives is the
// same for every channel of the row: a row of this step, a row of the slot's tail, or nowhere
// (before the sequence's start).
template <typename AT, int TAPS>
__global__ void __launch_bounds__(256) mixer_conv_kernel(int T, int n_seqs, int W, int taps_rt, const float* __restrict__ h,
                                                         const float* __restrict__ w, const int* __restrict__ cu_q,
                                                         const int* __restrict__ positions,
                                                         const int* __restrict__ state_slots,
                                                         const float* __restrict__ state_pool, size_t slot_floats,
                                                         size_t tail_off, AT* __restrict__ out, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  constexpr int MT = TAPS > 0 ? TAPS : TAIL_MAX_TAPS_C;
  const int taps = TAPS > 0 ? TAPS : taps_rt;
  const int t = blockIdx.x;
  __shared__ int s_seq;
  if (T == n_seqs) {
    if (threadIdx.x == 0) s_seq = t;
  } else {
    for (int i = threadIdx.x; i < n_seqs; i += blockDim.x)
      if (cu_q[i] <= t && t < cu_q[i + 1]) s_seq = i;
  }
  __syncthreads();
  const int s = s_seq;
  const int li = t - cu_q[s], pos = positions[t], keep = taps - 1;
  const float* tail = state_pool + (size_t)state_slots[s] * slot_floats + tail_off;
  const float* src[MT];
#pragma unroll
  for (int j = 0; j < MT; j++) {
    src[j] = nullptr;
    if (j < taps) {
      const int back = keep - j;  // input `back` positions before this token
      if (back <= li) src[j] = h + (size_t)(t - back) * W;
      else if (back <= pos) src[j] = tail + (size_t)(keep - (back - li)) * W;
    }
  }
  for (int c = threadIdx.x; c < W; c += blockDim.x) {
    float u[MT], wv[MT];
#pragma unroll
    for (int j = 0; j < MT; j++) {  // all the loads first
      u[j] = (j < taps && src[j]) ? src[j][c] : 0.f;
      wv[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
    }
    float y = h[(size_t)t * W + c];
#pragma unroll
    for (int j = 0; j < MT; j++) y = fmaf(wv[j], u[j], y);
    out[(size_t)t * W + c] = from_f32<AT>(y);
  }
  TRACE_EXIT(tr);
}

cudaError_t launch_mixer_conv(cudaStream_t st, int adt, int T, int n_seqs, int W, int taps, const float* h, const float* w,
                              const int* cu_q, const int* positions, const int* state_slots, const float* state_pool,
                              size_t slot_floats, size_t tail_off, void* out) {
  if (T <= 0) return cudaSuccess;
  if (taps < 1 || taps > TAIL_MAX_TAPS_C) return cudaErrorInvalidValue;
#define MC(AT_, TP_)                                                                                                  \
  (void)launch_k(mixer_conv_kernel<AT_, TP_>, dim3(T), dim3(256), 0, st, T, n_seqs, W, taps, h, w, cu_q, positions,    \
                 state_slots, state_pool, slot_floats, tail_off, (AT_*)out, next_trace(43))
  if (adt == DT_F32) {
    if (taps == 2) MC(float, 2); else if (taps == 3) MC(float, 3); else if (taps == 4) MC(float, 4); else MC(float, 0);
  } else {
    if (taps == 2) MC(bf16, 2); else if (taps == 3) MC(bf16, 3); else if (taps == 4) MC(bf16, 4); else MC(bf16, 0);
  }
#undef MC
  return cudaGetLastError();
}

// ------------------------------------------------------------------ tails of short convolutions
constexpr int TAIL_MAX_JOBS = 2;
constexpr int TAIL_MAX_TAPS = 8;
struct TailArgs {
  TailJob j[TAIL_MAX_JOBS];
  int n_jobs;
  const int *cu_q, *positions, *state_slots;
  float* state_pool;
  size_t slot_floats;
};
// grid (n_seqs, Y).  Entry i of the new tail is the input at position end - (taps - 1) + i: a row of
// this step, an entry of the old tail, or (before the sequence's start) zero.
template <typename AT>
__global__ void __launch_bounds__(256) roll_tails_kernel(TailArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  const int s = blockIdx.x;
  const int r0 = a.cu_q[s], n_new = a.cu_q[s + 1] - r0;
  if (n_new <= 0) return;
  const int pos0 = a.positions[r0], end = pos0 + n_new;
  float* slot = a.state_pool + (size_t)a.state_slots[s] * a.slot_floats;
  for (int jb = 0; jb < a.n_jobs; jb++) {
    const TailJob& J = a.j[jb];
    const int keep = J.taps - 1;
    float* tail = slot + J.tail_off;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < J.channels; c += gridDim.y * blockDim.x) {
      float nv[TAIL_MAX_TAPS];
#pragma unroll
      for (int i = 0; i < TAIL_MAX_TAPS; i++) {
        nv[i] = 0.f;
        if (i < keep) {
          const int p = end - keep + i;
          if (p >= pos0) {
            const int row = r0 + (p - pos0);
            nv[i] = J.seg.p ? seg_at(J.seg, row, c) + (J.bias ? J.bias[c] : 0.f)
                            : to_f32(((const AT*)J.act)[(size_t)row * J.channels + c]);
          } else if (p >= 0) {
            nv[i] = tail[(size_t)(p - pos0 + keep) * J.channels + c];
          }
        }
      }
#pragma unroll
      for (int i = 0; i < TAIL_MAX_TAPS; i++)
        if (i < keep) tail[(size_t)i * J.channels + c] = nv[i];
    }
  }
  TRACE_EXIT(tr);
}

cudaError_t launch_roll_tails(cudaStream_t st, int adt, int n_seqs, const TailJob* jobs, int n_jobs, const int* cu_q,
                              const int* positions, const int* state_slots, float* state_pool, size_t slot_floats) {
  if (n_seqs <= 0 || n_jobs <= 0) return cudaSuccess;
  if (n_jobs > TAIL_MAX_JOBS) return cudaErrorInvalidValue;
  TailArgs a{};
  int big = 0;
  for (int i = 0; i < n_jobs; i++) {
    if (jobs[i].taps > TAIL_MAX_TAPS) return cudaErrorInvalidValue;
    a.j[i] = jobs[i];
    big = std::max(big, jobs[i].channels);
  }
  a.n_jobs = n_jobs; a.cu_q = cu_q; a.positions = positions; a.state_slots = state_slots;
  a.state_pool = state_pool; a.slot_floats = slot_floats;
  const dim3 grid(n_seqs, std::max(1, std::min(16, ceil_div(big, 256))));
  if (adt == DT_F32) (void)launch_k(roll_tails_kernel<float>, grid, dim3(256), 0, st, a, next_trace(44));
  else (void)launch_k(roll_tails_kernel<bf16>, grid, dim3(256), 0, st, a, next_trace(44));
  return cudaGetLastError();
}

}  // namespace nvllm
