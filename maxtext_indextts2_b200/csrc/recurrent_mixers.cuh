// Linear recurrences with a matrix state per head, over a ragged batch and a pool of state slots.
//
// Per head, with q, k of size d, v of size dv and the state S [d, dv] (fp32, one per page group and layer run):
//
//   GLA    S <- diag(a) S + k v^T,  o = S^T q                      a = sigmoid(z)^(1 / tau) per key channel
//   mLSTM  m' = max(f + m, i);  S <- e^(f + m - m') S + e^(i - m') k v^T;  n likewise with k alone;
//          o = S^T q / (max(|n . q|, e^(-m')) + denom_eps)          (m starts at 0; i, f are log gates)
//   delta  S <- diag(w) S' - (a u)(u^T S') + k v^T,  o = S^T q    (S' the old state in both first terms)
//          u = k / sqrt(|k|^2 + key_eps); w = exp(-rate sigmoid(z)), z = up tanh(down x) + bias; a = sigmoid(. + bias), per key channel
//   gated delta  S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q   (the read-out sees the token's own write)
//          q, k, v after a short causal convolution over time and silu; q, k unit vectors (q / k heads may serve several heads);
//          g = exp(-exp(a_log) softplus(z + bias)) per head or per key channel; beta = sigmoid(.)
//
// A run (consecutive rows of one sequence) is walked in order from the group's state; a run that starts at position 0 starts
// from zero instead, so a slot that is handed to another sequence needs no clearing.  Every value column of S is independent of
// the others, so a (run, head) is spread over CTAs by column block: a CTA keeps its columns of S in registers (8 row slices x
// 8 or 16 columns), stages the run's q / k / decays / v in chunks through shared memory (cp.async, two stages) and walks the
// tokens in order.  The result of a token is the same bits however the sequence is cut into steps.
//
//   recurrent_prepare_kernel   per row: the GLA's decays (low-rank up-projection, bias, sigmoid^(1/tau)) or the mLSTM's two log gates
//   delta_prepare_kernel       per row: the delta rule's decays, unit keys and removal vectors a u
//   lowrank_split_kernel       the inputs of the gated delta rule's low-rank decay and gate projections in the matmul dtype
//   gdelta_prepare_kernel      per row: the gated delta rule's convolutions, silu, unit vectors, decays and write strengths
//   recurrent_scan_kernel      the walk
//   recurrent_out_kernel<T>    per row and head: o / rms(o) * weight * gate(g) * out_scale -> the activation of the output projection
#pragma once

#include "common.cuh"
#include "layer_ops.cuh"
#include "linear_any.cuh"

namespace mtx {

enum { REC_GLA = 1, REC_MLSTM = 2, REC_DELTA = 3, REC_GDELTA = 4 };

__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.0f) - log1pf(expf(-fabsf(z))); }

struct RecPrepareArgs {
  const float* proj;  // [rows, ld]
  long long ld;
  int x_col;          // GLA: first of the decay_rank down-projection columns; mLSTM: first input-gate column (forget gates follow)
  int kind, heads, dim, rank;
  float tau, cap;
  const float* up_t;  // GLA [rank, heads * dim]
  const float* bias;  // GLA [heads * dim]; mLSTM [2 * heads]
  float* out;         // GLA [rows, heads * dim] decays; mLSTM [rows, 2 * heads] log gates (input, then forget)
};

__global__ void __launch_bounds__(256) recurrent_prepare_kernel(const RecPrepareArgs a) {
  extern __shared__ float s_low[];
  griddep_wait();
  const int r = blockIdx.x;
  const float* row = a.proj + size_t(r) * a.ld + a.x_col;
  if (a.kind == REC_GLA) {
    const int n = a.heads * a.dim;
    for (int e = threadIdx.x; e < a.rank; e += blockDim.x) s_low[e] = row[e];
    __syncthreads();
    for (int c = threadIdx.x; c < n; c += blockDim.x) {
      float z = a.bias ? a.bias[c] : 0.0f;
      for (int e = 0; e < a.rank; ++e) z = fmaf(a.up_t[size_t(e) * n + c], s_low[e], z);
      a.out[size_t(r) * n + c] = expf(log_sigmoid_f(z) / a.tau);
    }
  } else {
    const int H = a.heads;
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
      const float ig = a.cap * tanhf((row[h] + a.bias[h]) / a.cap);
      const float fg = log_sigmoid_f(a.cap * tanhf((row[H + h] + a.bias[H + h]) / a.cap));
      a.out[size_t(r) * 2 * H + h] = ig;
      a.out[size_t(r) * 2 * H + H + h] = fg;
    }
  }
}

struct DeltaPrepareArgs {
  const float* proj;   // [rows, ld]: keys at k_col, removal pre-activations at a_col (heads * dim each), the decay's down-projection at x_col (rank)
  long long ld;
  int k_col, a_col, x_col;
  int heads, dim, rank;
  float rate, key_eps;
  const float* up_t;   // [rank, heads * dim]
  const float* w_bias; // [heads * dim]
  const float* a_bias; // [heads * dim]
  float* out;          // [rows, 3, heads * dim]: decays w, unit keys u, removal vectors a * u
};

// grid (rows, ceil(heads / 8)): a warp per head
__global__ void __launch_bounds__(256) delta_prepare_kernel(const DeltaPrepareArgs a) {
  extern __shared__ float s_low[];
  griddep_wait();
  const int r = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, d = a.dim, n = a.heads * d;
  const float* row = a.proj + size_t(r) * a.ld;
  for (int e = threadIdx.x; e < a.rank; e += blockDim.x) s_low[e] = tanhf(row[a.x_col + e]);
  __syncthreads();
  float* out = a.out + size_t(r) * 3 * n;
  for (int h = blockIdx.y * 8 + warp; h < a.heads; h += 8 * gridDim.y) {
    const float* k = row + a.k_col + h * d;
    float ss = 0.0f;
    for (int c = lane; c < d; c += 32) ss = fmaf(k[c], k[c], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss + a.key_eps);
    for (int c = lane; c < d; c += 32) {
      const int col = h * d + c;
      float z = a.w_bias ? a.w_bias[col] : 0.0f;
#pragma unroll 8
      for (int e = 0; e < a.rank; ++e) z = fmaf(a.up_t[size_t(e) * n + col], s_low[e], z);
      const float u = k[c] * inv;
      const float rem = 1.0f / (1.0f + expf(-(row[a.a_col + col] + (a.a_bias ? a.a_bias[col] : 0.0f))));
      out[col] = expf(-a.rate / (1.0f + expf(-z)));
      out[n + col] = u;
      out[2 * n + col] = rem * u;
    }
  }
}

// columns of the plane gdelta_prepare_kernel writes, each part starting on a multiple of four floats
struct GDeltaCols {
  int q, k, v, decay, beta, n;
};
__host__ __device__ inline GDeltaCols gdelta_cols(int heads, int kv_heads, int dim, int vdim) {
  GDeltaCols c;
  auto up4 = [](int x) { return (x + 3) / 4 * 4; };
  c.q = 0;
  c.k = up4(kv_heads * dim);
  c.v = c.k + up4(kv_heads * dim);
  c.decay = c.v + up4(heads * vdim);
  c.beta = c.decay + up4(heads * dim);
  c.n = c.beta + up4(heads);
  return c;
}

template <typename T>
struct GDeltaPrepareArgs {
  const float* proj;     // [rows, ld]: q | k | v (C = 2 * kv_heads * dim + heads * vdim columns from column 0), then beta at b_col (heads),
  long long ld;          // and, rank == 0, the decay's input at a_col (heads)
  int b_col, a_col;
  int heads, kv_heads, dim, vdim, taps, rank;
  float key_eps;
  const float* conv_w;   // [taps, C]
  const float* state;    // [slots, taps - 1, C]: the projection row of position p at p % (taps - 1)
  const float* a_log;    // [heads]
  const float* bias;     // rank == 0: [heads]; else [heads * dim]
  const float* z;        // rank > 0: [rows, heads * dim] the decay's low-rank projection (before the bias)
  const int* group;
  const int* pos;
  float* out;            // [rows, gdelta_cols().n]
};

__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.0f) + log1pf(expf(-fabsf(z))); }

// The inputs of the low-rank projections in the matmul dtype: the decay's (proj columns [a_col, a_col + rank)) as TWO parts side by
// side, hi = the value rounded to the matmul dtype and lo = what the rounding left, so that a product with the up-projection
// written twice along k sums to the fp32 value's product; the gate's (proj columns [g_col, g_col + gate_rank)) rounded once.
template <typename T>
__global__ void __launch_bounds__(256) lowrank_split_kernel(const float* proj, long long ld, int a_col, int rank, int g_col, int gate_rank, T* decay_in,
                                                            T* gate_in, long long rows) {
  griddep_wait();
  const long long per = rank + gate_rank, total = rows * per;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / per;
    const int e = int(i % per);
    if (e < rank) {
      const float v = proj[r * ld + a_col + e];
      const T hi = to_act<T>(v);
      decay_in[r * 2 * rank + e] = hi;
      decay_in[r * 2 * rank + rank + e] = to_act<T>(v - act_f32(hi));
    } else {
      gate_in[r * gate_rank + (e - rank)] = to_act<T>(proj[r * ld + g_col + (e - rank)]);
    }
  }
}

// grid (rows, parts): the CTAs of a row share its units, a warp takes a unit at a time: a q or k head (convolution, silu, unit
// vector), a v head (convolution, silu), a head's decays, or the write strengths.  The row `back` steps before row r is row r - back
// of the batch when that is the same sequence's previous position, a row of the state when the run began later, and zero before
// the sequence's start (up to kGdMaxBack earlier rows are located once per CTA).
constexpr int kGdMaxBack = 16, kGdMaxPerLane = 8;  // (dim <= 32 * kGdMaxPerLane)

template <typename T>
__global__ void __launch_bounds__(256) gdelta_prepare_kernel(const GDeltaPrepareArgs<T> a) {
  __shared__ const float* s_src[kGdMaxBack];
  griddep_wait();
  const int r = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, nw = blockDim.x >> 5;
  const int H = a.heads, G = a.kv_heads, d = a.dim, dv = a.vdim, C = 2 * G * d + H * dv, ring = a.taps - 1;
  const int p = a.pos[r], grp = a.group[r];
  const int n_back = ring < p ? ring : p;
  const float* row = a.proj + size_t(r) * a.ld;
  auto source = [&](int back) {
    const int rr = r - back;
    const bool in_batch = rr >= 0 && a.group[rr] == grp && a.pos[rr] == p - back;
    return in_batch ? a.proj + size_t(rr) * a.ld : a.state + (size_t(grp) * ring + (p - back) % ring) * C;
  };
  if (tid < n_back && tid < kGdMaxBack) s_src[tid] = source(tid + 1);
  __syncthreads();
  auto conv_silu = [&](int c) {
    float y = row[c] * a.conv_w[size_t(ring) * C + c];
    for (int back = 1; back <= n_back; ++back) {
      const float* src = back <= kGdMaxBack ? s_src[back - 1] : source(back);
      y = fmaf(src[c], a.conv_w[size_t(ring - back) * C + c], y);
    }
    return y / (1.0f + expf(-y));
  };
  const GDeltaCols cc = gdelta_cols(H, G, d, dv);
  float* out = a.out + size_t(r) * cc.n;
  const int n_units = 2 * G + 2 * H + 1;
  for (int u = blockIdx.y * nw + warp; u < n_units; u += gridDim.y * nw) {
    if (u < 2 * G) {  // a q head, or a k head: unit vectors
      float v[kGdMaxPerLane];
      float ss = 0.0f;
#pragma unroll
      for (int i = 0; i < kGdMaxPerLane; ++i) {
        const int c = lane + 32 * i;
        v[i] = c < d ? conv_silu(u * d + c) : 0.0f;
        ss = fmaf(v[i], v[i], ss);
      }
      ss = warp_sum(ss);
      const float inv = 1.0f / sqrtf(ss + a.key_eps);
      float* dst = out + (u < G ? cc.q + u * d : cc.k + (u - G) * d);
#pragma unroll
      for (int i = 0; i < kGdMaxPerLane; ++i) {
        const int c = lane + 32 * i;
        if (c < d) dst[c] = v[i] * inv;
      }
    } else if (u < 2 * G + H) {  // a v head
      const int h = u - 2 * G;
      for (int c = lane; c < dv; c += 32) out[cc.v + h * dv + c] = conv_silu(2 * G * d + h * dv + c);
    } else if (u < 2 * G + 2 * H) {  // a head's decays
      const int h = u - 2 * G - H;
      const float rate = expf(a.a_log[h]);
      if (a.rank > 0) {
        for (int c = lane; c < d; c += 32) out[cc.decay + h * d + c] = expf(-rate * softplus_f(a.z[size_t(r) * H * d + h * d + c] + a.bias[h * d + c]));
      } else {
        const float g = expf(-rate * softplus_f(row[a.a_col + h] + a.bias[h]));
        for (int c = lane; c < d; c += 32) out[cc.decay + h * d + c] = g;
      }
    } else {  // the write strengths
      for (int h = lane; h < H; h += 32) out[cc.beta + h] = 1.0f / (1.0f + expf(-row[a.b_col + h]));
    }
  }
}

struct RecScanArgs {
  const float* proj;   // [rows, ld]: q at q_col, k at k_col, v at v_col (heads x dim, heads x dim, heads x vdim)
  long long ld;
  int q_col, k_col, v_col;
  const float* aux;    // the prepare kernel's output
  float* o;            // [rows, heads * vdim]
  float* state_s;      // [slots, heads, vdim, dim]: a value column's dim entries are contiguous
  float* state_n;      // mLSTM [slots, heads, dim]
  float* state_m;      // mLSTM [slots, heads]
  const int* run_row0; // [n_runs + 1]
  const int* group;
  const int* pos;
  int heads, dim, vdim, chunk;
  int vec4;            // 1: every staged row starts on a 16-byte boundary and holds whole float4s (set by the host from the sizes)
  float q_scale, denom_eps;
  // REC_GDELTA: q / k head of head h is h / qk_rep (0 or 1: its own); the decays are the columns [dec_col + h * dim, ..) and the write
  // strength the column beta_col + h of the plane `aux` with row pitch aux_ld
  int qk_rep, dec_col, beta_col;
  long long aux_ld;
};

// A CTA owns CB value columns of one (run, head): thread (column jl, slice sl) keeps RPT key channels of its column of S in
// registers, in groups of four: channels g * 4 SL + sl * 4 .. + 3 for g < RPT / 4 (SL = 8 or 16 slices: dim <= SL * RPT), so that the
// slices of a column read 128 (256) contiguous bytes of the state and of the staged q / k / decays at a time.  The run's q / k / decays (or gates)
// / v arrive in chunks of `chunk` tokens (a multiple of 4) through a four-stage cp.async ring; tokens are walked four at a time
// so that the four read-outs' reductions overlap (the state update itself is the only chain from token to token).
constexpr int kRecSlices = 8, kRecUnroll = 4;  // (kRecSlices: the default; short of CTAs, a column is cut into 16 slices: SL)

// floats of one token in a stage: q, k, decays (8 * RPT channels each), then CB values, then 4 scalars (mLSTM: log input gate,
// log forget gate; later keep, put, floor)
// (nvec per-channel vectors: q, k, decays; the delta rule also stages u and a u)
__host__ __device__ inline int rec_token_floats(int rpt, int cb, int sl, int nvec = 3) { return nvec * sl * rpt + cb + 4; }
inline int rec_rpt(int dim, int sl) {
  const int r = (dim + sl - 1) / sl;
  return r <= 4 ? 4 : (r <= 8 ? 8 : (r <= 16 ? 16 : 32));
}
constexpr int kRecStages = 4;  // chunks in the cp.async ring: three are in flight while one is walked
// tokens per chunk: 16 for prompt portions (as many as 96 KB of ring hold, at least 4), 4 when every run is a single token
inline int rec_chunk_tokens(int dim, int cb, int sl, bool single_tokens, int nvec = 3) {
  if (single_tokens) return kRecUnroll;
  int t = (96 * 1024) / int(sizeof(float) * kRecStages * rec_token_floats(rec_rpt(dim, sl), cb, sl, nvec));
  t = t / kRecUnroll * kRecUnroll;
  return t > 16 ? 16 : (t < kRecUnroll ? kRecUnroll : t);
}
inline size_t rec_scan_smem_bytes(int dim, int cb, int sl, int chunk, int nvec = 3) {
  return sizeof(float) * kRecStages * size_t(chunk) * rec_token_floats(rec_rpt(dim, sl), cb, sl, nvec);
}

__device__ __forceinline__ void rec_cp_async_16(float* dst, const float* src) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}

__device__ __forceinline__ void rec_cp_async_4(float* dst, const float* src) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(src) : "memory");
}

template <int KIND, int RPT, int CB, int SL>
__global__ void __launch_bounds__(CB * SL) recurrent_scan_kernel(const RecScanArgs a) {
  extern __shared__ __align__(16) float rec_smem[];
  constexpr int NV = KIND == REC_DELTA ? 5 : 3;                                   // per-channel vectors of a staged token
  constexpr int NT = CB * SL, QP = SL * RPT, TF = NV * QP + CB + 4, GS = 4 * SL;  // GS: channels per group of float4s
  const int d = a.dim, dv = a.vdim, H = a.heads, TC = a.chunk;
  const int tid = threadIdx.x, jl = tid / SL, sl = tid % SL;
  griddep_wait();
  const int r0 = a.run_row0[blockIdx.x], nr = a.run_row0[blockIdx.x + 1] - r0, h = blockIdx.y;
  if (nr <= 0) return;
  const int col0 = blockIdx.z * CB, j = col0 + jl;
  const bool col_ok = j < dv;
  const int slot = a.group[r0];
  const bool fresh = a.pos[r0] == 0;
  const int hq = a.qk_rep > 1 ? h / a.qk_rep : h;  // the head whose q and k this head reads
  auto channel = [&](int i) { return (i >> 2) * GS + sl * 4 + (i & 3); };  // this thread's i-th key channel
  const bool vec = (d & 3) == 0;  // whole float4s of the state
  float S[RPT], N[RPT];
  float* gs = a.state_s + ((size_t(slot) * H + h) * dv + (col_ok ? j : 0)) * d;
  float* gn = a.state_n + (size_t(slot) * H + h) * d;
#pragma unroll
  for (int i = 0; i < RPT; ++i) S[i] = N[i] = 0.0f;
  float m = 0.0f;  // (thread 0 walks the running maximum)
  if (!fresh) {
#pragma unroll
    for (int i4 = 0; i4 < RPT; i4 += 4) {
      const int r = channel(i4);
      if (vec) {
        if (r < d && col_ok) {
          const float4 v4 = *reinterpret_cast<const float4*>(gs + r);
          S[i4] = v4.x, S[i4 + 1] = v4.y, S[i4 + 2] = v4.z, S[i4 + 3] = v4.w;
        }
        if (KIND == REC_MLSTM && r < d) {
          const float4 v4 = *reinterpret_cast<const float4*>(gn + r);
          N[i4] = v4.x, N[i4 + 1] = v4.y, N[i4 + 2] = v4.z, N[i4 + 3] = v4.w;
        }
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (r + e < d && col_ok) S[i4 + e] = gs[r + e];
          if (KIND == REC_MLSTM && r + e < d) N[i4 + e] = gn[r + e];
        }
      }
    }
    if (KIND == REC_MLSTM) m = a.state_m[size_t(slot) * H + h];
  }
  const int n_chunks = (nr + TC - 1) / TC;

  // stage <- chunk c: every element by a 4-byte cp.async (the projection's columns have no alignment to count on); the tail of
  // the last chunk and the key channels beyond dim are filled with values that leave the state alone (k = v = q = 0, decay 1)
  auto load_chunk = [&](int c, int stage) {
    if (c >= n_chunks) {  // (an empty group keeps the count of groups per iteration uniform)
      asm volatile("cp.async.commit_group;" ::: "memory");
      return;
    }
    float* base = rec_smem + size_t(stage) * TC * TF;
    const int t0 = c * TC;
    const int slots_d = SL * RPT;  // padded key channels
    const int left = (nr - t0 + kRecUnroll - 1) / kRecUnroll * kRecUnroll, TL = left < TC ? left : TC;  // tokens the walk will touch
    if (a.vec4) {  // four channels per copy
      constexpr int Q4 = SL * RPT / 4, C4 = CB / 4;
      for (int e = tid; e < TL * Q4; e += NT) {
        const int t = e / Q4, r = (e % Q4) * 4;
        float* dst = base + t * TF + r;
        const float* row = a.proj + size_t(r0 + t0 + t) * a.ld;
        if (t0 + t < nr && r < d) {
          rec_cp_async_16(dst, row + a.q_col + hq * d + r);
          rec_cp_async_16(dst + QP, row + a.k_col + hq * d + r);
          if (KIND == REC_GLA) rec_cp_async_16(dst + 2 * QP, a.aux + size_t(r0 + t0 + t) * H * d + h * d + r);
          if (KIND == REC_GDELTA) rec_cp_async_16(dst + 2 * QP, a.aux + size_t(r0 + t0 + t) * a.aux_ld + a.dec_col + h * d + r);
          if (KIND == REC_DELTA) {
            const float* ax = a.aux + size_t(r0 + t0 + t) * 3 * H * d + h * d + r;
            rec_cp_async_16(dst + 2 * QP, ax);
            rec_cp_async_16(dst + 3 * QP, ax + H * d);
            rec_cp_async_16(dst + 4 * QP, ax + 2 * H * d);
          }
        } else {
          *reinterpret_cast<float4*>(dst) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          *reinterpret_cast<float4*>(dst + QP) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          if (KIND == REC_GLA || KIND == REC_DELTA || KIND == REC_GDELTA) *reinterpret_cast<float4*>(dst + 2 * QP) = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
          if (KIND == REC_DELTA) {
            *reinterpret_cast<float4*>(dst + 3 * QP) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            *reinterpret_cast<float4*>(dst + 4 * QP) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
          }
        }
      }
      for (int e = tid; e < TL * C4; e += NT) {
        const int t = e / C4, c2 = (e % C4) * 4;
        float* dst = base + t * TF + NV * QP + c2;
        if (t0 + t < nr && col0 + c2 < dv) rec_cp_async_16(dst, a.proj + size_t(r0 + t0 + t) * a.ld + a.v_col + h * dv + col0 + c2);
        else *reinterpret_cast<float4*>(dst) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
      }
    } else {
    for (int e = tid; e < TL * slots_d; e += NT) {
      const int t = e / slots_d, r = e % slots_d;
      float* dst = base + t * TF + r;
      const bool ok = t0 + t < nr && r < d;
      const float* row = a.proj + size_t(r0 + t0 + t) * a.ld;
      if (ok) {
        rec_cp_async_4(dst, row + a.q_col + hq * d + r);
        rec_cp_async_4(dst + QP, row + a.k_col + hq * d + r);
        if (KIND == REC_GLA) rec_cp_async_4(dst + 2 * QP, a.aux + size_t(r0 + t0 + t) * H * d + h * d + r);
        if (KIND == REC_GDELTA) rec_cp_async_4(dst + 2 * QP, a.aux + size_t(r0 + t0 + t) * a.aux_ld + a.dec_col + h * d + r);
        if (KIND == REC_DELTA) {
          const float* ax = a.aux + size_t(r0 + t0 + t) * 3 * H * d + h * d + r;
          rec_cp_async_4(dst + 2 * QP, ax);
          rec_cp_async_4(dst + 3 * QP, ax + H * d);
          rec_cp_async_4(dst + 4 * QP, ax + 2 * H * d);
        }
      } else {
        dst[0] = 0.0f;
        dst[QP] = 0.0f;
        if (KIND == REC_GLA || KIND == REC_DELTA || KIND == REC_GDELTA) dst[2 * QP] = 1.0f;
        if (KIND == REC_DELTA) dst[3 * QP] = dst[4 * QP] = 0.0f;
      }
    }
    for (int e = tid; e < TL * CB; e += NT) {
      const int t = e / CB, c2 = e % CB;
      float* dst = base + t * TF + NV * QP + c2;
      if (t0 + t < nr && col0 + c2 < dv) rec_cp_async_4(dst, a.proj + size_t(r0 + t0 + t) * a.ld + a.v_col + h * dv + col0 + c2);
      else dst[0] = 0.0f;
    }
    }
    if (KIND == REC_MLSTM) {
      for (int e = tid; e < TL * 2; e += NT) {
        const int t = e >> 1, w = e & 1;
        float* dst = base + t * TF + 3 * QP + CB + w;
        if (t0 + t < nr) rec_cp_async_4(dst, a.aux + size_t(r0 + t0 + t) * 2 * H + w * H + h);
        else dst[0] = w ? 0.0f : -INFINITY;  // (forget gate 0, input gate -inf: keep = 1, put = 0)
      }
    }
    if (KIND == REC_GDELTA) {  // the write strength beta (0 beyond the run: nothing is written)
      for (int t = tid; t < TL; t += NT) {
        float* dst = base + t * TF + 3 * QP + CB;
        if (t0 + t < nr) rec_cp_async_4(dst, a.aux + size_t(r0 + t0 + t) * a.aux_ld + a.beta_col + h);
        else dst[0] = 0.0f;
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };

  for (int c = 0; c < kRecStages - 1; ++c) load_chunk(c, c);
  for (int c = 0; c < n_chunks; ++c) {
    load_chunk(c + kRecStages - 1, (c + kRecStages - 1) % kRecStages);  // (its stage was walked in iteration c - 1)
    asm volatile("cp.async.wait_group %0;" ::"n"(kRecStages - 1) : "memory");
    __syncthreads();
    float* base = rec_smem + size_t(c % kRecStages) * TC * TF;
    const int t0 = c * TC;
    const int left = (nr - t0 + kRecUnroll - 1) / kRecUnroll * kRecUnroll, TL = left < TC ? left : TC;
    if (KIND == REC_MLSTM) {
      // the running maximum is a chain over the tokens: one thread walks it, then the factors of all tokens at once
      float* sc = base + 3 * QP + CB;  // [t * TF + 0..3]: i, f -> keep, put, floor; [3] = m before the token
      if (tid == 0) {
        for (int t = 0; t < TL; ++t) {
          sc[t * TF + 3] = m;
          m = fmaxf(sc[t * TF + 1] + m, sc[t * TF]);
          sc[t * TF + 2] = m;
        }
      }
      __syncthreads();
      if (tid < TL) {
        float* q = sc + tid * TF;
        const float ig = q[0], fg = q[1], m_new = q[2], m_old = q[3];
        q[0] = expf(fg + m_old - m_new);
        q[1] = expf(ig - m_new);
        q[2] = expf(-m_new);
      }
      __syncthreads();
    }
    for (int t = 0; t < TL; t += kRecUnroll) {
      float part[kRecUnroll], npart[kRecUnroll], floor_m[kRecUnroll];
#pragma unroll
      for (int u = 0; u < kRecUnroll; ++u) {
        const float* tok = base + (t + u) * TF;
        const float* q = tok + sl * 4;
        const float* k = q + QP;
        const float v = tok[NV * QP + jl];
        part[u] = 0.0f;
        npart[u] = 0.0f;
        floor_m[u] = 0.0f;
        if (KIND == REC_GLA) {
          const float* al = k + QP;
#pragma unroll
          for (int i4 = 0; i4 < RPT; i4 += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(k + i4 * SL), q4 = *reinterpret_cast<const float4*>(q + i4 * SL),
                         a4 = *reinterpret_cast<const float4*>(al + i4 * SL);
            S[i4] = fmaf(a4.x, S[i4], k4.x * v);
            S[i4 + 1] = fmaf(a4.y, S[i4 + 1], k4.y * v);
            S[i4 + 2] = fmaf(a4.z, S[i4 + 2], k4.z * v);
            S[i4 + 3] = fmaf(a4.w, S[i4 + 3], k4.w * v);
            part[u] = fmaf(S[i4], q4.x, part[u]);
            part[u] = fmaf(S[i4 + 1], q4.y, part[u]);
            part[u] = fmaf(S[i4 + 2], q4.z, part[u]);
            part[u] = fmaf(S[i4 + 3], q4.w, part[u]);
          }
        } else if (KIND == REC_GDELTA) {
          // the column decays; what it then holds along k, added over the column's slices, is taken off the written value
          const float* al = k + QP;
          const float beta = tok[3 * QP + CB];
          float along = 0.0f;
#pragma unroll
          for (int i4 = 0; i4 < RPT; i4 += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(k + i4 * SL), a4 = *reinterpret_cast<const float4*>(al + i4 * SL);
            S[i4] *= a4.x;
            S[i4 + 1] *= a4.y;
            S[i4 + 2] *= a4.z;
            S[i4 + 3] *= a4.w;
            along = fmaf(S[i4], k4.x, along);
            along = fmaf(S[i4 + 1], k4.y, along);
            along = fmaf(S[i4 + 2], k4.z, along);
            along = fmaf(S[i4 + 3], k4.w, along);
          }
#pragma unroll
          for (int o = 1; o < SL; o <<= 1) along += __shfl_xor_sync(0xffffffffu, along, o);
          const float w = beta * (v - along);
#pragma unroll
          for (int i4 = 0; i4 < RPT; i4 += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(k + i4 * SL), q4 = *reinterpret_cast<const float4*>(q + i4 * SL);
            S[i4] = fmaf(k4.x, w, S[i4]);
            S[i4 + 1] = fmaf(k4.y, w, S[i4 + 1]);
            S[i4 + 2] = fmaf(k4.z, w, S[i4 + 2]);
            S[i4 + 3] = fmaf(k4.w, w, S[i4 + 3]);
            part[u] = fmaf(S[i4], q4.x, part[u]);
            part[u] = fmaf(S[i4 + 1], q4.y, part[u]);
            part[u] = fmaf(S[i4 + 2], q4.z, part[u]);
            part[u] = fmaf(S[i4 + 3], q4.w, part[u]);
          }
        } else if (KIND == REC_DELTA) {
          // what the old column holds along u, added over the column's slices, comes off along a u
          const float* al = k + QP;
          const float* un = k + 2 * QP;
          const float* rm = k + 3 * QP;
          float along = 0.0f;
#pragma unroll
          for (int i4 = 0; i4 < RPT; i4 += 4) {
            const float4 u4 = *reinterpret_cast<const float4*>(un + i4 * SL);
            along = fmaf(S[i4], u4.x, along);
            along = fmaf(S[i4 + 1], u4.y, along);
            along = fmaf(S[i4 + 2], u4.z, along);
            along = fmaf(S[i4 + 3], u4.w, along);
          }
#pragma unroll
          for (int o = 1; o < SL; o <<= 1) along += __shfl_xor_sync(0xffffffffu, along, o);
#pragma unroll
          for (int i4 = 0; i4 < RPT; i4 += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(k + i4 * SL), q4 = *reinterpret_cast<const float4*>(q + i4 * SL),
                         a4 = *reinterpret_cast<const float4*>(al + i4 * SL), r4 = *reinterpret_cast<const float4*>(rm + i4 * SL);
            S[i4] = fmaf(a4.x, S[i4], fmaf(-r4.x, along, k4.x * v));
            S[i4 + 1] = fmaf(a4.y, S[i4 + 1], fmaf(-r4.y, along, k4.y * v));
            S[i4 + 2] = fmaf(a4.z, S[i4 + 2], fmaf(-r4.z, along, k4.z * v));
            S[i4 + 3] = fmaf(a4.w, S[i4 + 3], fmaf(-r4.w, along, k4.w * v));
            part[u] = fmaf(S[i4], q4.x, part[u]);
            part[u] = fmaf(S[i4 + 1], q4.y, part[u]);
            part[u] = fmaf(S[i4 + 2], q4.z, part[u]);
            part[u] = fmaf(S[i4 + 3], q4.w, part[u]);
          }
        } else {
          const float keep = tok[3 * QP + CB], put = tok[3 * QP + CB + 1];
          floor_m[u] = tok[3 * QP + CB + 2];
#pragma unroll
          for (int i4 = 0; i4 < RPT; i4 += 4) {
            const float4 k4 = *reinterpret_cast<const float4*>(k + i4 * SL), q4 = *reinterpret_cast<const float4*>(q + i4 * SL);
            const float pk[4] = {put * k4.x, put * k4.y, put * k4.z, put * k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              S[i4 + e] = fmaf(keep, S[i4 + e], pk[e] * v);
              N[i4 + e] = fmaf(keep, N[i4 + e], pk[e]);
              part[u] = fmaf(S[i4 + e], qq[e], part[u]);
              npart[u] = fmaf(N[i4 + e], qq[e], npart[u]);
            }
          }
        }
      }
#pragma unroll
      for (int o = 1; o < SL; o <<= 1) {
#pragma unroll
        for (int u = 0; u < kRecUnroll; ++u) {
          part[u] += __shfl_xor_sync(0xffffffffu, part[u], o);
          if (KIND == REC_MLSTM) npart[u] += __shfl_xor_sync(0xffffffffu, npart[u], o);
        }
      }
      if (sl < kRecUnroll && col_ok && t0 + t + sl < nr) {  // slice u writes token t + u
        float out = 0.0f, nq = 0.0f, fl = 0.0f;
#pragma unroll
        for (int u = 0; u < kRecUnroll; ++u)
          if (sl == u) {
            out = part[u];
            nq = npart[u];
            fl = floor_m[u];
          }
        out *= a.q_scale;
        if (KIND == REC_MLSTM) out = out / (fmaxf(fabsf(nq * a.q_scale), fl) + a.denom_eps);
        a.o[size_t(r0 + t0 + t + sl) * H * dv + h * dv + j] = out;
      }
    }
    __syncthreads();  // the stage is free for the next iteration's load
  }
  const bool write_n = KIND == REC_MLSTM && blockIdx.z == 0 && jl == 0;
#pragma unroll
  for (int i4 = 0; i4 < RPT; i4 += 4) {
    const int r = channel(i4);
    if (vec) {
      if (r < d && col_ok) *reinterpret_cast<float4*>(gs + r) = make_float4(S[i4], S[i4 + 1], S[i4 + 2], S[i4 + 3]);
      if (write_n && r < d) *reinterpret_cast<float4*>(gn + r) = make_float4(N[i4], N[i4 + 1], N[i4 + 2], N[i4 + 3]);
    } else {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        if (r + e < d && col_ok) gs[r + e] = S[i4 + e];
        if (write_n && r + e < d) gn[r + e] = N[i4 + e];
      }
    }
  }
  if (write_n && tid == 0) a.state_m[size_t(slot) * H + h] = m;
}

template <typename T>
struct RecOutArgs {
  const float* o;       // [rows, heads * vdim]
  const float* proj;    // [rows, ld]: the output gate's pre-activation at g_col
  long long ld;
  int g_col;
  const float* weight;  // [heads * vdim]
  T* out;               // [rows, ld_out], written from column out_col
  long long ld_out;
  int out_col;
  int heads, vdim, gate_silu;
  float eps, out_scale;
};

// one CTA per row, a warp per head
template <typename T>
__global__ void __launch_bounds__(256) recurrent_out_kernel(const RecOutArgs<T> a) {
  griddep_wait();
  const int r = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5, dv = a.vdim;
  for (int h = warp; h < a.heads; h += nw) {
    const float* o = a.o + size_t(r) * a.heads * dv + h * dv;
    float ss = 0.0f;
    for (int c = lane; c < dv; c += 32) ss = fmaf(o[c], o[c], ss);
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / float(dv) + a.eps);
    for (int c = lane; c < dv; c += 32) {
      const float g = a.proj[size_t(r) * a.ld + a.g_col + h * dv + c];
      const float sig = 1.0f / (1.0f + expf(-g));
      const float gate = a.gate_silu ? g * sig : sig;
      a.out[size_t(r) * a.ld_out + a.out_col + h * dv + c] = to_act<T>(o[c] * inv * a.weight[h * dv + c] * gate * a.out_scale);
    }
  }
}

}  // namespace mtx
