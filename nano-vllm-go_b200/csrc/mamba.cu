// mamba.cu — Mamba2 block of the Granite-4 hybrid (SURVEY.md §8f rank 4;
// purego/tensor/mamba2.go:72-351), for a ragged batch of sequences.  The two projections are
// ordinary GEMMs (forward.cu); this file holds what sits between them:
//   mamba_conv_kernel   sum of the in_proj split-K slices, causal conv1d over the xBC columns
//                       (zero-padded at the start of every CALL, like causalConv1d :209-270 — the
//                       reference never reads its ConvCache), SiLU, and dt = softplus(dt + bias)
//   mamba_scan_kernel   the selective scan (:273-351), sequential over a sequence's new tokens,
//                       one CTA per (sequence, head), one thread per head_dim row holding its
//                       state_size states in registers; the SSM state lives per KV BLOCK
//                       (handle.h) and is read / written through the block table
//   mamba_gate_norm_kernel  y * silu(gate), RMS norm over E with eps 1e-5, * Norm (:139-173)
// Correctness-first kernels: HBM traffic is small next to the projections, and the scan's
// token loop is latency-bound by construction (a chunked scan is the obvious next step).
#include "common.cuh"
#include "kernels.h"

namespace nvllm {

namespace {

__device__ __forceinline__ int seq_of_row(const int* __restrict__ cu_q, int n_seqs, int row) {
  int lo = 0, hi = n_seqs - 1;  // last s with cu_q[s] <= row
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (cu_q[mid] <= row) lo = mid;
    else hi = mid - 1;
  }
  return lo;
}

__device__ __forceinline__ float sum_slices(const float* __restrict__ p, int S, size_t stride) {
  float acc = 0.f;
  for (int s = 0; s < S; s++) acc += p[(size_t)s * stride];
  return acc;
}

}  // namespace

// grid (T, ceil(conv / 256)); proj: [S][T][P] split-K slices of x @ in_proj^T, columns
// [gate (E) | xBC (conv) | dt (heads)]
__global__ void __launch_bounds__(256)
mamba_conv_kernel(MambaArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int s = seq_of_row(a.cu_q, a.n_seqs, t);
  const int li = t - a.cu_q[s];  // index of the token inside this call's rows of its sequence
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c < a.conv) {
    float sum = 0.f;
    for (int k = 0; k < a.K; k++) {
      const int back = a.K - 1 - k;  // tap k reads the token `back` rows earlier
      if (li - back >= 0)
        sum += sum_slices(a.proj + (size_t)(t - back) * a.P + a.E + c, a.S, a.stride) * a.conv_w[c * a.K + k];
    }
    if (a.conv_b) sum += a.conv_b[c];
    a.xbc[(size_t)t * a.conv + c] = silu(sum);
  }
  if (blockIdx.y == 0 && threadIdx.x < a.nh) {
    const int h = threadIdx.x;
    float dt = sum_slices(a.proj + (size_t)t * a.P + a.E + a.conv + h, a.S, a.stride);
    if (a.dt_bias) dt += a.dt_bias[h];
    a.dt[(size_t)t * a.nh + h] = (float)log(1.0 + exp((double)dt));  // Softplus, mamba2.go:369-376
  }
  TRACE_EXIT(tr);
}

// grid (n_seqs, heads), block = head_dim threads (thread d owns state[d][0..N))
template <int NMAX>
__global__ void __launch_bounds__(128)
mamba_scan_kernel(MambaArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float sB[NMAX], sC[NMAX];
  const int s = blockIdx.x, h = blockIdx.y, d = threadIdx.x;
  const int r0 = a.cu_q[s], r1 = a.cu_q[s + 1];
  const int start = a.positions[r0];  // position of the first new token
  const int* bt = a.block_tables + (size_t)s * a.max_blocks;
  const size_t per_layer = (size_t)a.nh * a.hd * a.N;
  const size_t per_block = (size_t)a.n_mamba * per_layer;
  float st[NMAX];
#pragma unroll
  for (int i = 0; i < NMAX; i++) st[i] = 0.f;
  if (start > 0 && d < a.hd) {
    // the state after position start - 1 sits in that position's block
    const float* src = a.ssm_pool + (size_t)bt[(start - 1) / KV_BLOCK] * per_block + (size_t)a.layer * per_layer +
                       ((size_t)h * a.hd + d) * a.N;
#pragma unroll
    for (int i = 0; i < NMAX; i++)
      if (i < a.N) st[i] = src[i];
  }
  int grp = h * a.G / a.nh;
  if (grp >= a.G) grp = a.G - 1;
  const float A = a.a_log ? -(float)exp((double)a.a_log[h]) : 0.f;
  const float Dh = a.d_skip ? a.d_skip[h] : 0.f;
  for (int t = r0; t < r1; t++) {
    __syncthreads();  // the previous token's sB / sC have been consumed
    for (int i = threadIdx.x; i < a.N; i += blockDim.x) {
      sB[i] = a.xbc[(size_t)t * a.conv + a.E + (size_t)grp * a.N + i];
      sC[i] = a.xbc[(size_t)t * a.conv + a.E + (size_t)a.G * a.N + (size_t)grp * a.N + i];
    }
    __syncthreads();
    if (d < a.hd) {
      const float dt = a.dt[(size_t)t * a.nh + h];
      const float abar = a.a_log ? (float)exp((double)(A * dt)) : 1.0f;
      const float u = a.xbc[(size_t)t * a.conv + (size_t)h * a.hd + d];
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < NMAX; i++)
        if (i < a.N) {
          st[i] = abar * st[i] + dt * sB[i] * u;  // mamba2.go:325-331
          sum += sC[i] * st[i];                   // :335-340, s ascending
        }
      a.y[(size_t)t * a.E + (size_t)h * a.hd + d] = sum + Dh * u;
      const int pos = start + (t - r0);
      if ((pos + 1) % KV_BLOCK == 0 || t == r1 - 1) {
        // snapshot: the state after the last token written into this block
        float* dst = a.ssm_pool + (size_t)bt[pos / KV_BLOCK] * per_block + (size_t)a.layer * per_layer +
                     ((size_t)h * a.hd + d) * a.N;
#pragma unroll
        for (int i = 0; i < NMAX; i++)
          if (i < a.N) dst[i] = st[i];
      }
    }
  }
  TRACE_EXIT(tr);
}

// one CTA per token row: y[t, :] * silu(gate[t, :]) -> RMS norm (eps 1e-5, mamba2.go:150-166)
// -> * Norm -> act dtype (the out_proj GEMM's input)
template <typename OT>
__global__ void __launch_bounds__(256)
mamba_gate_norm_kernel(MambaArgs a, OT* __restrict__ out, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row[];
  __shared__ float red[32];
  const int t = blockIdx.x;
  float lsq = 0.f;
  for (int i = threadIdx.x; i < a.E; i += blockDim.x) {
    const float g = sum_slices(a.proj + (size_t)t * a.P + i, a.S, a.stride);
    const float v = a.y[(size_t)t * a.E + i] * silu(g);
    row[i] = v;
    lsq += v * v;
  }
  const float tot = block_sum(lsq, red);
  const float rms = 1.0f / sqrtf(tot / (float)a.E + 1e-5f);
  for (int i = threadIdx.x; i < a.E; i += blockDim.x)
    out[(size_t)t * a.E + i] = from_f32<OT>(row[i] * rms * (a.norm_w ? a.norm_w[i] : 1.f));
  TRACE_EXIT(tr);
}

// ------------------------------------------------------------------ Mamba-2 with state slots
// The Mamba-2 mixer of a model given as a list of layers (forward_layered.cu).  Its state
// S (N x vdim per head, fp32) and the last taps - 1 inputs of its convolution live in the
// sequence's state slot; the recurrence itself runs in the linear-recurrence scan of linrec.cu.
//   mamba2_slot_prep_kernel  one CTA per token: split-K sum of the input projection, causal convolution
//                            over x | B | C (inputs before the step's first row from the slot's tail, zeros
//                            before the sequence's start), + bias, SiLU; dt = softplus(dt + bias) (fp32, no
//                            clamp), the head's decay exp(-exp(A_log) dt), and dt x (the scan's values)
//   mamba2_slot_out_kernel   one CTA per token: y = read-out + D x, times silu(z), RMS norm in norm_groups
//                            equal parts (eps of the model), times the weight -> act dtype
// 16-byte accesses of the row kernels below: four neighbouring channels per thread
__device__ __forceinline__ float4 ld4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 sum_slices4(const float* __restrict__ p, int S, size_t stride) {
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int s = 0; s < S; s++) {
    const float4 v = ld4(p + (size_t)s * stride);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  return acc;
}
__device__ __forceinline__ void st4(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void st4(bf16* p, float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 u;
  u.x = *reinterpret_cast<uint32_t*>(&lo);
  u.y = *reinterpret_cast<uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = u;
}
// every row, segment and tail of the two kernels starts on a 16-byte boundary
__device__ __forceinline__ bool m2_rows_aligned(const Mamba2SlotArgs& a) {
  const int inner = a.heads * a.vdim, gn = a.G * a.N;
  return (a.vdim % 4 == 0) && (gn % 4 == 0) && (a.in_ld % 4 == 0) && (a.in_stride % 4 == 0) && (inner % 4 == 0);
}

template <int TAPS>
__global__ void __launch_bounds__(256) mamba2_slot_prep_kernel(Mamba2SlotArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  constexpr int MT = TAPS > 0 ? TAPS : 8;
  const int taps = TAPS > 0 ? TAPS : a.taps;
  const int t = blockIdx.x;
  const int inner = a.heads * a.vdim, ch = inner + 2 * a.G * a.N;
  __shared__ int s_seq;
  __shared__ float s_dt[256];
  if (a.T == a.n_seqs) {
    if (threadIdx.x == 0) s_seq = t;
  } else {
    for (int i = threadIdx.x; i < a.n_seqs; i += blockDim.x)
      if (a.cu_q[i] <= t && t < a.cu_q[i + 1]) s_seq = i;
  }
  // step sizes and decays of the heads (at most 256 heads)
  for (int hh = threadIdx.x; hh < a.heads; hh += blockDim.x) {
    const float z = sum_slices(a.in_p + (size_t)t * a.in_ld + inner + ch + hh, a.in_S, a.in_stride) + a.dt_bias[hh];
    const float dt = z > 20.f ? z : log1pf(expf(z));  // softplus; above 20 the two agree to fp32 rounding
    s_dt[hh] = dt;
    a.decay[(size_t)t * a.heads + hh] = expf(-expf(a.a_log[hh]) * dt);
  }
  __syncthreads();
  const int s = s_seq;
  const int li = t - a.cu_q[s], pos = a.positions[t], keep = taps - 1;
  const float* tail = a.state_pool + (size_t)a.state_slots[s] * a.slot_floats + a.tail_off;
  const float* src[MT];
  bool part[MT];  // the row is one of this step's partials (slices to sum)
#pragma unroll
  for (int j = 0; j < MT; j++) {
    src[j] = nullptr;
    part[j] = false;
    if (j < taps) {
      const int back = keep - j;
      if (back <= li) { src[j] = a.in_p + (size_t)(t - back) * a.in_ld + inner; part[j] = true; }
      else if (back <= pos) src[j] = tail + (size_t)(keep - (back - li)) * ch;
    }
  }
  const bool one = a.in_S == 1;
  if (TAPS == 4 && m2_rows_aligned(a)) {
    // four channels per thread: their 16 taps are 64 contiguous bytes, every tap's inputs one 16-byte load
    for (int c = threadIdx.x * 4; c < ch; c += blockDim.x * 4) {
      float y[4], wv[4][4];
#pragma unroll
      for (int k = 0; k < 4; k++) {
        const float4 w4 = ld4(a.conv_w + (size_t)(c + k) * 4);
        wv[k][0] = w4.x; wv[k][1] = w4.y; wv[k][2] = w4.z; wv[k][3] = w4.w;
        y[k] = a.conv_b ? a.conv_b[c + k] : 0.f;
      }
#pragma unroll
      for (int j = 0; j < 4; j++) {
        if (!src[j]) continue;  // before the sequence's start: zeros
        const float4 u = (one || !part[j]) ? ld4(src[j] + c) : sum_slices4(src[j] + c, a.in_S, a.in_stride);
        y[0] = fmaf(wv[0][j], u.x, y[0]); y[1] = fmaf(wv[1][j], u.y, y[1]);
        y[2] = fmaf(wv[2][j], u.z, y[2]); y[3] = fmaf(wv[3][j], u.w, y[3]);
      }
      float v[4];
#pragma unroll
      for (int k = 0; k < 4; k++) v[k] = a.fast_act ? __fdividef(y[k], 1.0f + __expf(-y[k])) : silu(y[k]);
      st4(a.xbc + (size_t)t * ch + c, v[0], v[1], v[2], v[3]);
      if (c < inner) {
        const float dt = s_dt[c / a.vdim];
        st4(a.dtx + (size_t)t * inner + c, v[0] * dt, v[1] * dt, v[2] * dt, v[3] * dt);
      }
    }
    TRACE_EXIT(tr);
    return;
  }
  for (int c = threadIdx.x; c < ch; c += blockDim.x) {
    float u[MT], wv[MT];
#pragma unroll
    for (int j = 0; j < MT; j++) {
      u[j] = 0.f;
      wv[j] = j < taps ? a.conv_w[(size_t)c * taps + j] : 0.f;
      if (j < taps && src[j]) u[j] = (one || !part[j]) ? src[j][c] : sum_slices(src[j] + c, a.in_S, a.in_stride);
    }
    float y = a.conv_b ? a.conv_b[c] : 0.f;
#pragma unroll
    for (int j = 0; j < MT; j++) y = fmaf(wv[j], u[j], y);
    const float v = a.fast_act ? __fdividef(y, 1.0f + __expf(-y)) : silu(y);
    a.xbc[(size_t)t * ch + c] = v;
    if (c < inner) a.dtx[(size_t)t * inner + c] = v * s_dt[c / a.vdim];
  }
  TRACE_EXIT(tr);
}

template <typename OT>
__global__ void __launch_bounds__(256) mamba2_slot_out_kernel(Mamba2SlotArgs a, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float row[];
  __shared__ float ginv[64];
  const int t = blockIdx.x;
  const int inner = a.heads * a.vdim, ch = inner + 2 * a.G * a.N;
  const int part = inner / a.norm_groups;
  const bool vec = m2_rows_aligned(a);
  if (vec) {
    for (int i = threadIdx.x * 4; i < inner; i += blockDim.x * 4) {
      const float4 z = sum_slices4(a.in_p + (size_t)t * a.in_ld + i, a.in_S, a.in_stride);
      const float4 x = ld4(a.xbc + (size_t)t * ch + i);
      const float4 o = ld4(a.o + (size_t)t * inner + i);
      const float d = a.d_skip[i / a.vdim];
      const float zz[4] = {z.x, z.y, z.z, z.w};
      const float yy[4] = {o.x + d * x.x, o.y + d * x.y, o.z + d * x.z, o.w + d * x.w};
#pragma unroll
      for (int k = 0; k < 4; k++) row[i + k] = yy[k] * (a.fast_act ? __fdividef(zz[k], 1.0f + __expf(-zz[k])) : silu(zz[k]));
    }
  } else {
    for (int i = threadIdx.x; i < inner; i += blockDim.x) {
      const float z = sum_slices(a.in_p + (size_t)t * a.in_ld + i, a.in_S, a.in_stride);
      const float x = a.xbc[(size_t)t * ch + i];
      const float y = a.o[(size_t)t * inner + i] + a.d_skip[i / a.vdim] * x;
      row[i] = y * (a.fast_act ? __fdividef(z, 1.0f + __expf(-z)) : silu(z));
    }
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  for (int g = warp; g < a.norm_groups; g += nw) {
    float sq = 0.f;
    for (int i = lane; i < part; i += 32) {
      const float v = row[g * part + i];
      sq = fmaf(v, v, sq);
    }
    sq = warp_sum(sq);
    if (lane == 0) ginv[g] = 1.0f / sqrtf(sq / (float)part + a.eps);
  }
  __syncthreads();
  OT* op = (OT*)a.out + (size_t)t * a.o_ld;
  if (vec && part % 4 == 0 && a.o_ld % 4 == 0) {
    for (int i = threadIdx.x * 4; i < a.o_ld; i += blockDim.x * 4) {
      if (i < inner) {  // inner and o_ld are multiples of 4: a quad is all inside or all padding
        const float4 r4 = ld4(row + i), w4 = ld4(a.norm_w + i);
        const float gi = ginv[i / part];
        st4(op + i, r4.x * gi * w4.x, r4.y * gi * w4.y, r4.z * gi * w4.z, r4.w * gi * w4.w);
      } else {
        st4(op + i, 0.f, 0.f, 0.f, 0.f);
      }
    }
  } else {
    for (int i = threadIdx.x; i < a.o_ld; i += blockDim.x)
      op[i] = from_f32<OT>(i < inner ? row[i] * ginv[i / part] * a.norm_w[i] : 0.f);
  }
  TRACE_EXIT(tr);
}

// Steps with one row per sequence: convolution, step size, decay and the recurrence of a (sequence, head)
// pair as ONE launch (mamba2_slot_prep_kernel and the scan of linrec.cu in one).  CTA = (sequence, head), 256
// threads.  Phase 1: the head's step size and decay; the convolution (+ bias, SiLU) of the head's vdim
// channels of x and of its group's N channels of B and of C into shared memory (the x channels also to xbc,
// where mamba2_slot_out_kernel reads them for the D skip).  Phase 2: the head's state [N][vdim] goes once
// through the registers, VW columns per thread and 256 / (vdim / VW) rows in flight:
// S <- decay S + B_n (dt x_p), y_p += S C_n, written back in place; the rows' partial read-outs meet in shared
// memory.  A sequence at position 0 starts from zeros whatever the slot holds.
// VW = 4: 16-byte loads and stores (vdim a multiple of 4); VW = 1 otherwise.
constexpr int M2D_THREADS = 256;
template <int TAPS, int VW>
__global__ void __launch_bounds__(M2D_THREADS) mamba2_slot_decode_kernel(Mamba2SlotArgs a, float* __restrict__ o, Trace tr) {
  TRACE_ENTRY(tr);
  pdl_launch_dependents();
  pdl_wait();
  constexpr int MT = TAPS > 0 ? TAPS : 8;
  const int taps = TAPS > 0 ? TAPS : a.taps;
  const int t = blockIdx.x, hh = blockIdx.y;
  const int P = a.vdim, N = a.N;
  const int inner = a.heads * P, gn = a.G * N, ch = inner + 2 * gn;
  const int g = hh / (a.heads / a.G);
  extern __shared__ __align__(16) float m2d_smem[];
  float* xs = m2d_smem;       // [P]  dt * silu(conv x)
  float* Bs = xs + ((P + 3) & ~3);  // [N]
  float* Cs = Bs + N;         // [N]
  float* red = Cs + N;        // [rows in flight][P]
  __shared__ float s_dt, s_decay;
  if (threadIdx.x == 0) {
    const float z = sum_slices(a.in_p + (size_t)t * a.in_ld + inner + ch + hh, a.in_S, a.in_stride) + a.dt_bias[hh];
    const float dt = z > 20.f ? z : log1pf(expf(z));
    s_dt = dt;
    s_decay = expf(-expf(a.a_log[hh]) * dt);
  }
  const int pos = a.positions[t], keep = taps - 1;
  const float* tail = a.state_pool + (size_t)a.state_slots[t] * a.slot_floats + a.tail_off;
  const float* cur = a.in_p + (size_t)t * a.in_ld + inner;
  __syncthreads();
  const float dt = s_dt, decay = s_decay;
  // the head's P + 2 N convolution channels
  for (int i = threadIdx.x; i < P + 2 * N; i += blockDim.x) {
    const int c = i < P ? hh * P + i : (i < P + N ? inner + g * N + (i - P) : inner + gn + g * N + (i - P - N));
    float y = a.conv_b ? a.conv_b[c] : 0.f;
#pragma unroll
    for (int j = 0; j < MT; j++) {
      if (j >= taps) continue;
      const int back = keep - j;  // the input `back` positions before this token
      float u = 0.f;
      if (back == 0) u = a.in_S == 1 ? cur[c] : sum_slices(cur + c, a.in_S, a.in_stride);
      else if (back <= pos) u = tail[(size_t)(keep - back) * ch + c];
      y = fmaf(a.conv_w[(size_t)c * taps + j], u, y);
    }
    const float v = a.fast_act ? __fdividef(y, 1.0f + __expf(-y)) : silu(y);
    if (i < P) {
      xs[i] = v * dt;
      a.xbc[(size_t)t * ch + c] = v;
    } else if (i < P + N) {
      Bs[i - P] = v;
    } else {
      Cs[i - P - N] = v;
    }
  }
  __syncthreads();
  // the recurrence
  const int cols = P / VW;                       // column units of VW
  const int rows_par = M2D_THREADS / cols;       // rows in flight (the launcher keeps cols <= 256)
  const int u = threadIdx.x % cols, rg = threadIdx.x / cols;
  float* state = const_cast<float*>(a.state_pool) + (size_t)a.state_slots[t] * a.slot_floats + a.state_off + (size_t)hh * N * P;
  const bool has_prev = pos > 0;
  float acc[VW], xv[VW];
#pragma unroll
  for (int e = 0; e < VW; e++) { acc[e] = 0.f; xv[e] = xs[u * VW + e]; }
  if (rg < rows_par) {
#pragma unroll 4
    for (int n = rg; n < N; n += rows_par) {
      float* sp = state + (size_t)n * P + u * VW;
      float sv[VW];
      if (VW == 4) {
        const float4 q4 = has_prev ? *reinterpret_cast<const float4*>(sp) : make_float4(0.f, 0.f, 0.f, 0.f);
        sv[0] = q4.x; sv[1 % VW] = q4.y; sv[2 % VW] = q4.z; sv[3 % VW] = q4.w;
      } else {
        sv[0] = has_prev ? sp[0] : 0.f;
      }
      const float bn = Bs[n], cn = Cs[n];
#pragma unroll
      for (int e = 0; e < VW; e++) {
        sv[e] = fmaf(decay, sv[e], bn * xv[e]);
        acc[e] = fmaf(sv[e], cn, acc[e]);
      }
      if (VW == 4) *reinterpret_cast<float4*>(sp) = make_float4(sv[0], sv[1 % VW], sv[2 % VW], sv[3 % VW]);
      else sp[0] = sv[0];
    }
#pragma unroll
    for (int e = 0; e < VW; e++) red[(size_t)rg * P + u * VW + e] = acc[e];
  }
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    float y = 0.f;
    for (int r = 0; r < rows_par; r++) y += red[(size_t)r * P + p];
    o[(size_t)t * inner + hh * P + p] = y;
  }
  TRACE_EXIT(tr);
}

bool mamba2_slot_decode_ok(const Mamba2SlotArgs& a) {
  static const bool on = !(getenv("NVLLM_MAMBA2_DECODE_FUSED") && atoi(getenv("NVLLM_MAMBA2_DECODE_FUSED")) == 0);
  const int cols = a.vdim % 4 == 0 ? a.vdim / 4 : a.vdim;
  return on && a.T == a.n_seqs && cols <= M2D_THREADS && a.taps >= 1 && a.taps <= 8 && a.heads % a.G == 0;
}

// o: [T, inner] read-outs (what the scan would have written); a.state_off: the layer's state inside a slot
cudaError_t launch_mamba2_slot_decode(cudaStream_t st, const Mamba2SlotArgs& a, float* o) {
  if (a.T <= 0) return cudaSuccess;
  if (!mamba2_slot_decode_ok(a)) return cudaErrorInvalidValue;
  const bool v4 = a.vdim % 4 == 0;
  const int cols = v4 ? a.vdim / 4 : a.vdim;
  const size_t smem = ((size_t)((a.vdim + 3) & ~3) + 2 * a.N + (size_t)(M2D_THREADS / cols) * a.vdim) * sizeof(float);
  const dim3 grid(a.T, a.heads);
#define M2D(TP_, VW_)                                                                                               \
  {                                                                                                                  \
    if (smem > 48 * 1024)                                                                                            \
      cudaFuncSetAttribute(mamba2_slot_decode_kernel<TP_, VW_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    (void)launch_k(mamba2_slot_decode_kernel<TP_, VW_>, grid, dim3(M2D_THREADS), smem, st, a, o, next_trace(21));     \
  }
  if (v4) {
    if (a.taps == 4) M2D(4, 4) else if (a.taps == 3) M2D(3, 4) else if (a.taps == 2) M2D(2, 4) else M2D(0, 4)
  } else {
    M2D(0, 1)
  }
#undef M2D
  return cudaGetLastError();
}

cudaError_t launch_mamba2_slot_prep(cudaStream_t st, const Mamba2SlotArgs& a) {
  if (a.T <= 0) return cudaSuccess;
  if (a.taps < 1 || a.taps > 8 || a.heads > 256) return cudaErrorInvalidValue;
  if (a.taps == 2) (void)launch_k(mamba2_slot_prep_kernel<2>, dim3(a.T), dim3(256), 0, st, a, next_trace(20));
  else if (a.taps == 3) (void)launch_k(mamba2_slot_prep_kernel<3>, dim3(a.T), dim3(256), 0, st, a, next_trace(20));
  else if (a.taps == 4) (void)launch_k(mamba2_slot_prep_kernel<4>, dim3(a.T), dim3(256), 0, st, a, next_trace(20));
  else (void)launch_k(mamba2_slot_prep_kernel<0>, dim3(a.T), dim3(256), 0, st, a, next_trace(20));
  return cudaGetLastError();
}

cudaError_t launch_mamba2_slot_out(cudaStream_t st, int odt, const Mamba2SlotArgs& a) {
  if (a.T <= 0) return cudaSuccess;
  const int inner = a.heads * a.vdim;
  if (a.norm_groups < 1 || a.norm_groups > 64 || inner % a.norm_groups) return cudaErrorInvalidValue;
  const size_t smem = (size_t)inner * sizeof(float);
  if (odt == DT_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(mamba2_slot_out_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    (void)launch_k(mamba2_slot_out_kernel<float>, dim3(a.T), dim3(256), smem, st, a, next_trace(22));
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(mamba2_slot_out_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    (void)launch_k(mamba2_slot_out_kernel<bf16>, dim3(a.T), dim3(256), smem, st, a, next_trace(22));
  }
  return cudaGetLastError();
}

cudaError_t launch_mamba_conv(cudaStream_t st, const MambaArgs& a) {
  if (a.T <= 0) return cudaSuccess;
  (void)launch_k(mamba_conv_kernel, dim3(a.T, ceil_div(a.conv, 256)), dim3(256), 0, st, a, next_trace(20));
  return cudaGetLastError();
}

cudaError_t launch_mamba_scan(cudaStream_t st, const MambaArgs& a) {
  if (a.n_seqs <= 0) return cudaSuccess;
  const int threads = max(32, ((a.hd + 31) / 32) * 32);
  if (threads > 128 || a.N > 128) return cudaErrorInvalidValue;
  const dim3 grid(a.n_seqs, a.nh);
  if (a.N <= 16) (void)launch_k(mamba_scan_kernel<16>, grid, dim3(threads), 0, st, a, next_trace(21));
  else if (a.N <= 32) (void)launch_k(mamba_scan_kernel<32>, grid, dim3(threads), 0, st, a, next_trace(21));
  else if (a.N <= 64) (void)launch_k(mamba_scan_kernel<64>, grid, dim3(threads), 0, st, a, next_trace(21));
  else (void)launch_k(mamba_scan_kernel<128>, grid, dim3(threads), 0, st, a, next_trace(21));
  return cudaGetLastError();
}

cudaError_t launch_mamba_gate_norm(cudaStream_t st, const MambaArgs& a, int odt, void* out) {
  if (a.T <= 0) return cudaSuccess;
  const size_t smem = (size_t)a.E * sizeof(float);
  if (odt == DT_F32)
    (void)launch_k(mamba_gate_norm_kernel<float>, dim3(a.T), dim3(256), smem, st, a, (float*)out, next_trace(22));
  else
    (void)launch_k(mamba_gate_norm_kernel<bf16>, dim3(a.T), dim3(256), smem, st, a, (bf16*)out, next_trace(22));
  return cudaGetLastError();
}

}  // namespace nvllm
