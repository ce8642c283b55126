// The layered engine of include/mtx_b200.h (mtx_layered_*): a decoder given as a list of layer descriptors, stepped over ragged
// batches whose keys and values live in page pools.  Host code only: the kernels are in linear_any.cuh (any-shape projections, also
// grouped by expert), gemm_rows.cuh (the tcgen05 projections, for shapes made of whole 128 x 64 tiles), layer_ops.cuh (norms,
// residual, cache append), grouped_gemm.cuh (the experts' products of steps with many rows), window_attention*.cuh (the sigmoid window mixer), softmax_attention.cuh (causal softmax attention with
// rotary positions), recurrent_mixers.cuh (GLA, mLSTM and the delta rule over state slots), latent_attention.cuh (attention through
// cached latents) and moe.cuh (routing).
#include <cmath>
#include <cstdio>
#include <cstring>
#include <vector>

#include "../../include/mtx_b200.h"
#include "layer_ops.cuh"
#include "linear_any.cuh"
#include "grouped_gemm.cuh"
#include "window_attention.cuh"
#include "window_attention_mma.cuh"
#include "window_attention_decode.cuh"
#include "softmax_attention.cuh"
#include "recurrent_mixers.cuh"
#include "latent_attention.cuh"
#include "moe.cuh"
#include "host_util.cuh"

using namespace mtx;

struct mtx_layered {
  mtx_layered_config cfg;
  std::vector<mtx_layer_desc> layers;
  int num_sms = 148;
  int max_nqkv = 0, max_qdim = 0, max_odim = 0, max_ff = 0, vshared_dim = 0;
  size_t ws_bytes = 0;
  bool bound = false;
  // workspace carve-up
  float *x = nullptr, *y = nullptr, *qkv = nullptr, *v_shared = nullptr;
  void *xa = nullptr, *q = nullptr, *attn = nullptr, *act = nullptr, *wanted = nullptr, *obf = nullptr;
  // mtx_layered_step_graph: one instantiated graph per distinct batch descriptor (a decode loop passes the same one every step)
  struct GraphEntry {
    mtx_ragged_batch key;
    cudaGraphExec_t exec;
  };
  std::vector<GraphEntry> graphs;
  cudaStream_t cap_stream = nullptr;
  float* attn_part = nullptr;  // fp32 partial outputs of the attention's key splits: room for 4 * max_rows rows
  size_t attn_part_rows = 0;
  float* smax_ml = nullptr;    // the softmax attention's key splits: running maximum and sum per (split, row, head)
  int max_attn_heads = 0;
  // composite mixers, sandwich norms, routed feed-forwards
  bool sandwich = false;
  int max_rec_o = 0, max_rec_aux = 0, max_moe_top = 0, max_moe_experts = 0, max_moe_ff = 0;
  float *x0 = nullptr, *rec_o = nullptr, *rec_aux = nullptr, *moe_logits = nullptr, *moe_weight = nullptr, *moe_y = nullptr;
  int *moe_chosen = nullptr, *moe_slot = nullptr, *moe_row = nullptr, *moe_off = nullptr;
  void* moe_act = nullptr;
  // MTX_NORM_PARALLEL layers: the normed rows (fp32), the feed-forward's input, the latent attention's query and result planes
  bool parallel = false;
  int max_lat_q = 0, max_lat_o = 0;
  float *h = nullptr, *lat_q = nullptr;
  void *xb = nullptr, *lat_o = nullptr;
  // MTX_NORM_PRE layers (they share h and xb with the parallel ones): the output gate of a recurrence whose gate is low-rank
  bool prenorm = false;
  int max_rec_gate = 0, max_rec_z = 0;
  float *rec_gate = nullptr, *rec_z = nullptr;
};

namespace {

size_t elem(const mtx_layered* e) { return e->cfg.float32 ? 4 : 2; }

struct LWs {
  size_t x, y, qkv, v_shared, xa, q, attn, act, wanted, obf, attn_part, total;
  size_t smax_ml, x0, rec_o, rec_aux, moe_logits, moe_weight, moe_y, moe_chosen, moe_slot, moe_row, moe_off, moe_act;
  size_t h, xb, lat_q, lat_o, rec_gate, rec_z;
};

LWs layered_layout(const mtx_layered* e) {
  const mtx_layered_config& c = e->cfg;
  // (rows padded to a multiple of 256: the tcgen05 projections read whole row blocks)
  const size_t R = align_up(size_t(c.max_rows), 256), W = align_up(size_t(c.max_want > 0 ? c.max_want : 1), 256), es = elem(e);
  LWs L;
  size_t off = 0;
  auto take = [&](size_t bytes) {
    size_t at = off;
    off = align_up(off + bytes, 1024);
    return at;
  };
  L.x = take(R * c.width * 4);
  L.y = take(R * c.width * 4);
  L.qkv = take(R * e->max_nqkv * 4);
  L.v_shared = take(R * (e->vshared_dim > 0 ? e->vshared_dim : 1) * 4);
  L.xa = take(R * c.width * es);
  L.q = take(R * e->max_qdim * es);
  L.attn = take(R * e->max_odim * es);
  L.act = take(R * (e->max_ff > 0 ? e->max_ff : 1) * es);
  L.wanted = take(W * c.width * es);
  L.obf = take(R * size_t(e->max_nqkv > c.width ? e->max_nqkv : c.width) * 2);  // bf16 output of a tcgen05 projection
  L.attn_part = take(c.float32 ? 1024 : 4 * R * size_t(e->max_odim) * 4);
  L.smax_ml = take(c.float32 ? 4 : 4 * R * size_t(e->max_attn_heads > 0 ? e->max_attn_heads : 1) * 2 * 4);
  L.x0 = take(e->sandwich ? R * c.width * 4 : 4);
  L.rec_o = take(R * size_t(e->max_rec_o > 0 ? e->max_rec_o : 1) * 4);
  L.rec_aux = take(R * size_t(e->max_rec_aux > 0 ? e->max_rec_aux : 1) * 4);
  const size_t RT = R * size_t(e->max_moe_top > 0 ? e->max_moe_top : 0);  // (row, choice) entries
  L.moe_logits = take(R * size_t(e->max_moe_experts > 0 ? e->max_moe_experts : 1) * 4);
  L.moe_weight = take((RT + 1) * 4);
  L.moe_y = take((RT * c.width + 1) * 4);
  L.moe_chosen = take((RT + 1) * 4);
  L.moe_slot = take((RT + 1) * 4);
  L.moe_row = take((RT + 1) * 4);
  L.moe_off = take(size_t(e->max_moe_experts + 2) * 4);
  L.moe_act = take((RT * size_t(e->max_moe_ff) + 1) * es);
  L.h = take(e->parallel || e->prenorm ? R * c.width * 4 : 4);
  L.xb = take(e->parallel || e->prenorm ? R * c.width * es : 4);
  L.rec_gate = take(R * size_t(e->max_rec_gate > 0 ? e->max_rec_gate : 1) * 4);
  L.rec_z = take(R * size_t(e->max_rec_z > 0 ? e->max_rec_z : 1) * 4);
  L.lat_q = take(R * size_t(e->max_lat_q > 0 ? e->max_lat_q : 1) * 4);
  L.lat_o = take(R * size_t(e->max_lat_o > 0 ? e->max_lat_o : 1) * es);
  L.total = off;
  return L;
}

// does the projection [rows, k] x [n, k] fit the tcgen05 GEMM of gemm_rows.cuh?  (whole 128-column weight tiles, 64-element k blocks,
// 16-byte aligned rows for TMA)
bool fits_umma(const mtx_layered* e, int n, int k) {
  static int on = env_int("MTX_LAYERED_UMMA", 1);
  return on != 0 && !e->cfg.float32 && n % 128 == 0 && k % 64 == 0;
}

__global__ void bf16_rows_to_f32_kernel(const bf16* src, const float* bias, float* dst, int n, long long total) {
  griddep_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
    dst[i] = __bfloat162float(src[i]) + (bias ? bias[i % n] : 0.0f);
}

// (mode 0: gelu_tanh(g) u; 1: the clamped form g sigmoid(1.702 g) (u + 1); 2: silu(g) u)
__global__ void gate_up_bf16_kernel(const bf16* src, bf16* act, int ff, long long total, float limit, int mode) {
  griddep_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / ff, f = i % ff;
    const float g = __bfloat162float(src[r * 2 * ff + 2 * f]), u = __bfloat162float(src[r * 2 * ff + 2 * f + 1]);
    act[i] = __float2bfloat16_rn(mode == 1 ? clamped_gate_f(g, u, limit) : (mode == 2 ? silu_gate_f(g, u) : gelu_tanh_f(g) * u));
  }
}

// out (fp32, or the gated activation) = EPI(a[rows, k] . w[n, k]^T)
template <typename T, int EPI>
int run_linear(mtx_layered* e, const void* a, const void* w, const float* bias, float* out, void* act, int rows, int n, int k, cudaStream_t st,
               float limit = 0.0f, long long ldo = 0) {
  if (rows <= 0) return MTX_OK;
  LinArgs<T> p;
  memset(&p, 0, sizeof(p));
  p.limit = limit;
  p.a = static_cast<const T*>(a);
  p.w = static_cast<const T*>(w);
  p.bias = bias;
  p.out = out;
  p.act = static_cast<T*>(act);
  p.lda = k;
  p.ldo = ldo > 0 ? ldo : ((EPI == LIN_GATED || EPI == LIN_GATED_CLAMP) ? n / 2 : n);
  p.rows = rows;
  p.n = n;
  p.k = k;
  const dim3 grid((n + 63) / 64, (rows + 63) / 64);
  if constexpr (sizeof(T) == 4) return launch(linear_f32_kernel<EPI>, grid, dim3(kLinF32Threads), 0, st, p);
  else return launch(linear_mma_kernel<EPI>, grid, dim3(kLinThreads), 0, st, p);
}

// (relu2: max(., 0)^2; act has the row pitch ldo)
__global__ void act_bf16_kernel(const bf16* src, bf16* act, int n, long long ldo, long long total, int relu2) {
  griddep_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    float v = __bfloat162float(src[i]);
    if (relu2) {
      v = fmaxf(v, 0.0f);
      v *= v;
    }
    act[(i / n) * ldo + i % n] = __float2bfloat16_rn(v);
  }
}

// the same product on the tcgen05 GEMM: the bf16 result stays in e->obf (256-row blocks)
int run_umma_raw(mtx_layered* e, const void* a, const void* w, int rows, int n, int k, cudaStream_t st) {
  bf16* tmp = static_cast<bf16*>(e->obf);
  for (int r0 = 0; r0 < rows; r0 += 256) {
    const int nr = rows - r0 < 256 ? rows - r0 : 256;
    EpiArgs ea;
    memset(&ea, 0, sizeof(ea));
    ea.out = tmp + size_t(r0) * n;
    ea.ld_out = n;
    MTX_TRY(single_gemm<EPI_STORE_BF16>(static_cast<const bf16*>(a) + size_t(r0) * k, w, nr, n, k, ea, st));
  }
  return MTX_OK;
}

// ... then the epilogue as a row kernel
template <int EPI>
int run_linear_umma(mtx_layered* e, const void* a, const void* w, const float* bias, float* out, void* act, int rows, int n, int k, cudaStream_t st,
                    float limit = 0.0f, long long ldo = 0) {
  MTX_TRY(run_umma_raw(e, a, w, rows, n, k, st));
  const bf16* tmp = static_cast<const bf16*>(e->obf);
  constexpr bool gated = EPI == LIN_GATED || EPI == LIN_GATED_CLAMP;
  const long long total = (long long)rows * (gated ? n / 2 : n);
  const int blocks = int((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  if (EPI == LIN_ACT || EPI == LIN_RELU2)
    return launch(act_bf16_kernel, dim3(blocks), dim3(256), 0, st, tmp, static_cast<bf16*>(act), n, ldo > 0 ? ldo : (long long)n, total, EPI == LIN_RELU2 ? 1 : 0);
  if (gated)
    return launch(gate_up_bf16_kernel, dim3(blocks), dim3(256), 0, st, tmp, static_cast<bf16*>(act), n / 2, total, limit,
                  EPI == LIN_GATED_CLAMP ? (limit > 0.0f ? 1 : 2) : 0);
  return launch(bf16_rows_to_f32_kernel, dim3(blocks), dim3(256), 0, st, tmp, bias, out, n, total);
}

bool takes_umma(const mtx_layered* e, int rows, int n, int k) { return fits_umma(e, n, k) && rows >= 16; }

template <typename T, int EPI>
int linear(mtx_layered* e, const void* a, const void* w, const float* bias, float* out, void* act, int rows, int n, int k, cudaStream_t st,
           float limit = 0.0f, long long ldo = 0) {
  if constexpr (sizeof(T) == 2) {
    if (takes_umma(e, rows, n, k)) return run_linear_umma<EPI>(e, a, w, bias, out, act, rows, n, k, st, limit, ldo);
  }
  return run_linear<T, EPI>(e, a, w, bias, out, act, rows, n, k, st, limit, ldo);
}

// `batches` products over the same rows whose operands lie side by side (linear_any.cuh, batched mode): batch z reads the columns
// [z * batch_a, z * batch_a + k) of `a`, the weight w + z * w_stride [n, k], and writes the columns [z * batch_o, z * batch_o + n) of
// `act` in the matmul dtype
template <typename T>
int linear_batched(const void* a, long long lda, long long batch_a, const void* w, long long w_stride, void* act, long long ldo, long long batch_o,
                   int rows, int n, int k, int batches, cudaStream_t st) {
  if (rows <= 0) return MTX_OK;
  LinArgs<T> p;
  memset(&p, 0, sizeof(p));
  p.a = static_cast<const T*>(a);
  p.w = static_cast<const T*>(w);
  p.act = static_cast<T*>(act);
  p.lda = lda;
  p.ldo = ldo;
  p.rows = rows;
  p.n = n;
  p.k = k;
  p.w_group_stride = w_stride;
  p.batch_a = batch_a;
  p.batch_o = batch_o;
  const dim3 grid((n + 63) / 64, (rows + 63) / 64, batches);
  if constexpr (sizeof(T) == 4) return launch(linear_f32_kernel<LIN_ACT>, grid, dim3(kLinF32Threads), 0, st, p);
  else return launch(linear_mma_kernel<LIN_ACT>, grid, dim3(kLinThreads), 0, st, p);
}

// one matrix product per group of slots (linear_any.cuh, grouped mode): slot ranges group_off [groups + 1] on the device, at most
// `slots` slots in all; slot s reads row a_row[s] of `a` (a_row null: row s)
template <typename T, int EPI>
int linear_grouped(const void* a, const int* a_row, const void* w, long long w_stride, const int* group_off, int groups, float* out, void* act,
                   int slots, int n, int k, float limit, cudaStream_t st) {
  if (slots <= 0) return MTX_OK;
  LinArgs<T> p;
  memset(&p, 0, sizeof(p));
  p.a = static_cast<const T*>(a);
  p.w = static_cast<const T*>(w);
  p.out = out;
  p.act = static_cast<T*>(act);
  p.lda = k;
  p.ldo = (EPI == LIN_GATED || EPI == LIN_GATED_CLAMP) ? n / 2 : n;
  p.rows = slots;
  p.n = n;
  p.k = k;
  p.limit = limit;
  p.group_off = group_off;
  p.a_row = a_row;
  p.w_group_stride = w_stride;
  // up to 64 groups: their row tiles side by side along y (a CTA finds its group by walking the slot ranges); more: a worst-case
  // range of y per group
  const bool packed = groups <= 64;
  p.groups = packed ? groups : 0;
  if constexpr (sizeof(T) == 2) {
    // many rows per group (a prompt portion): 128-row tiles behind a three-stage cp.async ring (grouped_gemm.cuh); 2 forces it
    // whenever the shape allows, 0 switches it off
    static const int pipe = env_int("MTX_GROUPED_PIPE", 1);
    const bool shape_ok = packed && k % kGgBK == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (w_stride % 8) == 0;
    if (shape_ok && (pipe == 2 || (pipe == 1 && slots >= kGgBM * groups))) {
      static bool attr_set = false;  // per instantiation
      if (!attr_set) {
        MTX_CUDA(cudaFuncSetAttribute(grouped_mma_pipe_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kGgSmemBytes)));
        attr_set = true;
      }
      const dim3 pgrid((n + kGgBN - 1) / kGgBN, (slots + kGgBM - 1) / kGgBM + groups, 1);
      return launch(grouped_mma_pipe_kernel<EPI>, pgrid, dim3(kGgThreads), kGgSmemBytes, st, p);
    }
  }
  const dim3 grid((n + 63) / 64, packed ? (slots + 63) / 64 + groups : (slots + 63) / 64, packed ? 1 : groups);
  if constexpr (sizeof(T) == 4) return launch(linear_f32_kernel<EPI>, grid, dim3(kLinF32Threads), 0, st, p);
  else return launch(linear_mma_kernel<EPI>, grid, dim3(kLinThreads), 0, st, p);
}

int pick_key_tile(const mtx_layer_desc& l) {
  int kt = 32;
  while (kt > 4 && window_attn_smem_bytes(l.heads, l.kv_heads, l.dim, l.vdim, kt) > 200 * 1024) kt /= 2;
  return kt;
}

// x += gain * unit(a . w^T), and the copy of x in the matmul dtype
template <typename T>
int project_norm_residual(mtx_layered* e, const void* a, const void* w, int rows, int n, int k, float gain, cudaStream_t st) {
  const float* y = e->y;
  const bf16* yb = nullptr;
  if (sizeof(T) == 2 && takes_umma(e, rows, n, k)) {
    MTX_TRY(run_umma_raw(e, a, w, rows, n, k, st));
    y = nullptr;
    yb = static_cast<const bf16*>(e->obf);
  } else {
    MTX_TRY((linear<T, LIN_PLAIN>(e, a, w, nullptr, e->y, nullptr, rows, n, k, st)));
  }
  return launch(norm_residual_kernel<T>, dim3(rows), dim3(256), 0, st, y, yb, gain, e->cfg.eps, e->x, static_cast<T*>(e->xa), e->cfg.width);
}

bool use_window_mma() {
  static int on = env_int("MTX_WINDOW_MMA", 1);
  return on != 0;
}

template <int HPW, int DVT>
int launch_window_mma_t(const WindowAttnArgs<bf16>& wa, const WindowMmaExtra& x, size_t smem, cudaStream_t st) {
  static size_t have = 0;  // per instantiation
  if (smem > have) {
    MTX_CUDA(cudaFuncSetAttribute(window_attention_mma_kernel<HPW, DVT>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    have = smem;
  }
  return launch(window_attention_mma_kernel<HPW, DVT>, dim3(x.n_tiles, x.splits), dim3(kWmmaThreads), smem, st, wa, x);
}

// the tensor-core mixer: (query tile, key split) work items, then the sum over the splits
int launch_window_mma(mtx_layered* e, const WindowAttnArgs<bf16>& wa, const WindowMmaPlan& plan, const mtx_ragged_batch& b, cudaStream_t st) {
  WindowMmaExtra x;
  x.tile_row0 = b.tile_row0;
  x.partial = e->attn_part;
  x.n_tiles = b.n_tiles;
  x.bn = plan.bn;
  x.hg = plan.hg;
  const int key_tiles = (wa.window + kWmmaRows - 1 + plan.bn - 1) / plan.bn;  // most key tiles a query tile can have
  // key splits: enough work items to fill the SMs (one CTA each), at least two key tiles per split, and among the next few counts
  // the one whose last wave is fullest (256 tiles x 2 splits on 148 SMs leave the fourth wave half empty; x 4 fill seven waves)
  int cap = key_tiles / 2;
  if (size_t(cap) * wa.rows > e->attn_part_rows) cap = int(e->attn_part_rows / wa.rows);
  if (cap < 1) cap = 1;
  int lo = (e->num_sms + b.n_tiles - 1) / b.n_tiles;
  if (lo > cap) lo = cap;
  int splits = lo;
  double best = 0.0;
  for (int sp = lo; sp <= cap && sp < lo + 8; ++sp) {
    const double waves = double(b.n_tiles) * sp / e->num_sms, eff = waves / std::ceil(waves);
    if (eff > best + 0.02) {
      best = eff;
      splits = sp;
    }
  }
  x.splits = splits;
  int rc = MTX_ERR_UNSUPPORTED;
  if (plan.hpw == 1 && plan.dvt == 8) rc = launch_window_mma_t<1, 8>(wa, x, plan.smem, st);
  else if (plan.hpw == 1 && plan.dvt == 16) rc = launch_window_mma_t<1, 16>(wa, x, plan.smem, st);
  else if (plan.hpw == 1 && plan.dvt == 32) rc = launch_window_mma_t<1, 32>(wa, x, plan.smem, st);
  else if (plan.hpw == 2 && plan.dvt == 8) rc = launch_window_mma_t<2, 8>(wa, x, plan.smem, st);
  else if (plan.hpw == 2 && plan.dvt == 16) rc = launch_window_mma_t<2, 16>(wa, x, plan.smem, st);
  MTX_TRY(rc);
  const long long per_split = (long long)wa.rows * wa.heads * wa.vdim;
  long long blocks = (per_split / 2 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return launch(window_partial_sum_kernel, dim3(unsigned(blocks)), dim3(256), 0, st, (const float*)e->attn_part, wa.out, splits, per_split);
}

template <int CPW, int DT>
int launch_window_decode_t(const WindowAttnArgs<bf16>& wa, const WindowDecodeExtra& x, size_t smem, cudaStream_t st) {
  static size_t have = 0;  // per instantiation
  if (smem > have) {
    MTX_CUDA(cudaFuncSetAttribute(window_attention_decode_kernel<CPW, DT>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    have = smem;
  }
  return launch(window_attention_decode_kernel<CPW, DT>, dim3(wa.rows, x.splits), dim3(kWdecThreads), smem, st, wa, x);
}

// the decode mixer (every row a token of its own sequence): (row, key split) work items, then the sum over the splits
int launch_window_decode(mtx_layered* e, const WindowAttnArgs<bf16>& wa, const WindowDecodePlan& plan, cudaStream_t st) {
  WindowDecodeExtra x;
  x.partial = e->attn_part;
  x.stages = plan.stages;
  const int key_tiles = (wa.window + kWdecKeys - 1) / kWdecKeys;
  // one wave: as many work items as CTAs fit on the GPU at once (a split's start-up -- its first tile's latency, the staging of
  // the queries -- is worth several tiles, so more and shorter splits lose), at least four key tiles per split
  size_t per_sm = (226 * 1024) / (plan.smem + 1024);
  if (per_sm > 8) per_sm = 8;
  int splits = int(per_sm) * e->num_sms / wa.rows;
  if (splits > key_tiles / 4) splits = key_tiles / 4;
  if (size_t(splits) * wa.rows > e->attn_part_rows) splits = int(e->attn_part_rows / wa.rows);
  if (splits < 1) splits = 1;
  x.splits = splits;
  int rc = MTX_ERR_UNSUPPORTED;
  if (plan.cpw == 1 && plan.dt == 4) rc = launch_window_decode_t<1, 4>(wa, x, plan.smem, st);
  else if (plan.cpw == 1 && plan.dt == 8) rc = launch_window_decode_t<1, 8>(wa, x, plan.smem, st);
  else if (plan.cpw == 1 && plan.dt == 16) rc = launch_window_decode_t<1, 16>(wa, x, plan.smem, st);
  else if (plan.cpw == 2 && plan.dt == 4) rc = launch_window_decode_t<2, 4>(wa, x, plan.smem, st);
  else if (plan.cpw == 2 && plan.dt == 8) rc = launch_window_decode_t<2, 8>(wa, x, plan.smem, st);
  MTX_TRY(rc);
  const long long per_split = (long long)wa.rows * wa.heads * wa.vdim;
  long long blocks = (per_split / 2 + 255) / 256;
  if (blocks > 148 * 8) blocks = 148 * 8;
  return launch(window_partial_sum_kernel, dim3(unsigned(blocks)), dim3(256), 0, st, (const float*)e->attn_part, wa.out, splits, per_split);
}

bool use_window_decode() {
  static int on = env_int("MTX_WINDOW_DECODE", 1);
  return on != 0;
}

// a MTX_MIXER_WINDOW_SIGMOID layer with MTX_NORM_OUT_GAIN norms: both sublayers read x itself (xa = x in the matmul dtype)
template <typename T>
int window_layer(mtx_layered* e, int li, const mtx_ragged_batch& b, cudaStream_t st) {
  const mtx_layered_config& c = e->cfg;
  const int rows = b.rows, E = c.width;
  T* xa = static_cast<T*>(e->xa);
  const mtx_layer_desc& l = e->layers[li];
  const int H = l.heads, G = l.kv_heads, nq = H * l.dim, nqkv = nq + G * l.dim + G * l.vdim, no = H * l.vdim;
  // q, k, v = W x + b
  QkvPostArgs<T> qa;
  memset(&qa, 0, sizeof(qa));
  if (sizeof(T) == 2 && takes_umma(e, rows, nqkv, E)) {  // the tcgen05 GEMM's bf16 result; the bias is added where it is read
    MTX_TRY(run_umma_raw(e, xa, l.wqkv, rows, nqkv, E, st));
    qa.qkv_bf16 = static_cast<const bf16*>(e->obf);
    qa.bias = l.bqkv;
  } else {
    if (l.bqkv) MTX_TRY((linear<T, LIN_BIAS>(e, xa, l.wqkv, l.bqkv, e->qkv, nullptr, rows, nqkv, E, st)));
    else MTX_TRY((linear<T, LIN_PLAIN>(e, xa, l.wqkv, nullptr, e->qkv, nullptr, rows, nqkv, E, st)));
    qa.qkv = e->qkv;
  }
  qa.q_norm = l.q_norm;
  qa.k_norm = l.k_norm;
  qa.q_out = static_cast<T*>(e->q);
  qa.k_pages = static_cast<T*>(l.k_pages);
  qa.v_pages = static_cast<T*>(l.v_pages);
  qa.v_shared = e->v_shared;
  qa.group = b.group;
  qa.pos = b.pos;
  qa.page_map = b.page_map;
  qa.heads = H;
  qa.kv_heads = G;
  qa.dim = l.dim;
  qa.vdim = l.vdim;
  qa.num_pages = c.num_pages;
  qa.tokens_per_page = c.tokens_per_page;
  qa.max_pages = c.max_pages_per_group;
  qa.value_mix = l.value_mix;
  qa.value_lambda = l.value_lambda;
  qa.eps = c.eps;
  MTX_TRY(launch(qkv_post_kernel<T>, dim3(rows), dim3(256), 0, st, qa));
  // the mixer
  WindowAttnArgs<T> wa;
  memset(&wa, 0, sizeof(wa));
  wa.q = static_cast<const T*>(e->q);
  wa.out = static_cast<T*>(e->attn);
  wa.k_pages = static_cast<const T*>(l.k_pages);
  wa.v_pages = static_cast<const T*>(l.v_pages);
  wa.group = b.group;
  wa.pos = b.pos;
  wa.page_map = b.page_map;
  wa.dist_bias = l.dist_bias;
  wa.head_bias = l.head_bias;
  wa.talk = l.talk;
  wa.rows = rows;
  wa.heads = H;
  wa.kv_heads = G;
  wa.dim = l.dim;
  wa.vdim = l.vdim;
  wa.window = l.window;
  wa.num_pages = c.num_pages;
  wa.tokens_per_page = c.tokens_per_page;
  wa.max_pages = c.max_pages_per_group;
  wa.scale = l.scale;
  wa.softcap = l.softcap;
  bool done = false;
  if constexpr (sizeof(T) == 2) {
    static const int force_stages = env_int("MTX_WINDOW_DECODE_STAGES", 0);
    const WindowDecodePlan dplan = window_decode_plan(H, G, l.dim, l.vdim, force_stages);
    const WindowMmaPlan plan = window_mma_plan(H, G, l.dim, l.vdim);
    if (dplan.ok && b.n_tiles == rows && b.tile_row0 != nullptr && use_window_mma() && use_window_decode()) {  // all single-row tiles
      MTX_TRY(launch_window_decode(e, wa, dplan, st));
      done = true;
    } else if (plan.ok && b.n_tiles > 0 && b.tile_row0 != nullptr && use_window_mma()) {
      MTX_TRY(launch_window_mma(e, wa, plan, b, st));
      done = true;
    }
  }
  if (!done) {
    wa.kt = pick_key_tile(l);
    const size_t smem = window_attn_smem_bytes(H, G, l.dim, l.vdim, wa.kt);
    static size_t attr_bytes[2] = {0, 0};  // per instantiation (bf16, float)
    size_t& have = attr_bytes[sizeof(T) == 4 ? 1 : 0];
    if (smem > 48 * 1024 && smem > have) {
      MTX_CUDA(cudaFuncSetAttribute(window_attention_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
      have = smem;
    }
    MTX_TRY(launch(window_attention_rows_kernel<T>, dim3(rows), dim3(kWinThreads), smem, st, wa));
  }
  // x += gain1 * unit(Wo attn)
  MTX_TRY(project_norm_residual<T>(e, e->attn, l.wo, rows, E, no, l.gain1, st));
  if (l.ff > 0) {
    // x += gain2 * unit(Wdown (gelu(Wgate x) * Wup x))
    MTX_TRY((linear<T, LIN_GATED>(e, xa, l.w_gate_up, nullptr, nullptr, e->act, rows, 2 * l.ff, E, st)));
    MTX_TRY(project_norm_residual<T>(e, e->act, l.w_down, rows, E, l.ff, l.gain2, st));
  }
  return MTX_OK;
}

// Column layout of a composite mixer's input projection and of the activation its output projection reads.
struct CompositeCols {
  int aq = 0, ak = 0, av = -1, rq = 0, rk = 0, rv = 0, rg = 0, rx = 0, n = 0;
  int out_rec = 0, k_out = 0;
};

CompositeCols composite_cols(const mtx_layer_desc& l) {
  CompositeCols cc;
  int at = 0;
  const mtx_softmax_attn_desc& a = l.attn;
  const mtx_recurrent_desc& r = l.rec;
  if (a.heads > 0) {
    cc.aq = at;
    at += a.heads * a.dim;
    cc.ak = at;
    at += a.kv_heads * a.dim;
    if (!a.values_are_keys) {
      cc.av = at;
      at += a.kv_heads * a.vdim;
    }
    cc.out_rec = a.heads * a.vdim;
  }
  if (r.kind != 0) {
    cc.rq = at;
    at += r.heads * r.dim;
    cc.rk = at;
    at += r.heads * r.dim;
    cc.rv = at;
    at += r.heads * r.vdim;
    cc.rg = at;
    at += r.heads * r.vdim;
    cc.rx = at;
    at += r.kind == MTX_REC_GLA ? r.decay_rank : 2 * r.heads;
  }
  cc.n = at;
  cc.k_out = cc.out_rec + (r.kind != 0 ? r.heads * r.vdim : 0);
  return cc;
}

template <int KIND, int RPT, int CB, int SL>
int launch_rec_scan_t(const RecScanArgs& ra, dim3 grid, dim3 block, size_t smem, cudaStream_t st) {
  static size_t have = 0;  // per instantiation
  if (smem > 48 * 1024 && smem > have) {
    MTX_CUDA(cudaFuncSetAttribute(recurrent_scan_kernel<KIND, RPT, CB, SL>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    have = smem;
  }
  return launch(recurrent_scan_kernel<KIND, RPT, CB, SL>, grid, block, smem, st, ra);
}

template <int KIND, int CB, int SL>
int launch_rec_scan_cb(const RecScanArgs& ra, int n_runs, cudaStream_t st) {
  const dim3 grid(n_runs, ra.heads, (ra.vdim + CB - 1) / CB), block(CB * SL);
  const size_t smem = rec_scan_smem_bytes(ra.dim, CB, SL, ra.chunk, KIND == REC_DELTA ? 5 : 3);  // (the gated delta rule stages q, k, decays)
  const int rpt = rec_rpt(ra.dim, SL);
  if (rpt == 4) return launch_rec_scan_t<KIND, 4, CB, SL>(ra, grid, block, smem, st);
  if (rpt == 8) return launch_rec_scan_t<KIND, 8, CB, SL>(ra, grid, block, smem, st);
  if (rpt == 16) return launch_rec_scan_t<KIND, 16, CB, SL>(ra, grid, block, smem, st);
  if constexpr (SL == 8) return launch_rec_scan_t<KIND, 32, CB, SL>(ra, grid, block, smem, st);
  return fail(MTX_ERR_UNSUPPORTED, "recurrence: dim %d", ra.dim);
}

// A walk is bound by latency, so what counts is how many warps share an SM.  16 value columns per CTA when that still gives every
// SM two CTAs, else 8; and when even 8-column CTAs with 8 slices per column leave the thread slots of the GPU mostly empty (one
// prompt: heads x vdim columns in all), a column is cut into 16 slices.
template <int KIND>
int launch_rec_scan(mtx_layered* e, RecScanArgs& ra, int n_runs, int rows, cudaStream_t st) {
  const long long columns = (long long)n_runs * ra.heads * ra.vdim;
  const bool wide = (long long)n_runs * ra.heads * ((ra.vdim + 15) / 16) >= 2LL * e->num_sms;
  static const int force_sl = env_int("MTX_REC_SLICES", 0);
  const bool fine = force_sl ? force_sl == 16 : (!wide && ra.dim >= 64 && columns * 8 < 512LL * e->num_sms);
  ra.chunk = rec_chunk_tokens(ra.dim, wide ? 16 : 8, fine ? 16 : 8, rows == n_runs, KIND == REC_DELTA ? 5 : 3);
  if (fine && ra.dim >= 16) return launch_rec_scan_cb<KIND, 8, 16>(ra, n_runs, st);
  return wide ? launch_rec_scan_cb<KIND, 16, 8>(ra, n_runs, st) : launch_rec_scan_cb<KIND, 8, 8>(ra, n_runs, st);
}

// MTX_NORM_SANDWICH: x += wnorm(y + bias, post), then what comes before the next sublayer: the pre-adds of the next layer run
// (when this was a layer's last sublayer) and xa = wnorm(x, the next sublayer's weight).  `next_layer` < 0: the next sublayer is
// this layer's feed-forward, whose weight is `pre`.
template <typename T>
int sandwich_step(mtx_layered* e, const float* y, const float* bias, const float* post, const float* pre, int next_layer, int rows, cudaStream_t st) {
  SandwichArgs sa;
  memset(&sa, 0, sizeof(sa));
  sa.y = y;
  sa.y_bias = bias;
  sa.post = post;
  sa.pre = pre;
  sa.x = e->x;
  sa.eps = e->cfg.eps;
  sa.width = e->cfg.width;
  if (next_layer >= 0 && next_layer < e->cfg.num_layers) {
    const mtx_layer_desc& nl = e->layers[next_layer];
    sa.x0 = nl.add_embedding ? e->x0 : nullptr;
    sa.add_vec = nl.add_vector;
    sa.pre = nl.norm1;
  }
  if (!sa.y && !sa.x0 && !sa.add_vec && !sa.pre) return MTX_OK;
  if (sa.width % 4 == 0 && sa.width <= 256 * 4 * kSandwichVec) return launch(sandwich_step_kernel<T, 4>, dim3(rows), dim3(256), 0, st, sa, static_cast<T*>(e->xa));
  return launch(sandwich_step_kernel<T, 1>, dim3(rows), dim3(256), 0, st, sa, static_cast<T*>(e->xa));
}

bool use_softmax_mma() {
  static int on = env_int("MTX_SOFTMAX_MMA", 1);
  return on != 0;
}

template <int D16, int PARTS, int KT>
int launch_softmax_mma_t(const SoftmaxAttnArgs<bf16>& sa, const SoftmaxMmaPlan& plan, int n_tiles, cudaStream_t st) {
  static size_t have = 0;  // per instantiation
  if (plan.smem > 48 * 1024 && plan.smem > have) {
    MTX_CUDA(cudaFuncSetAttribute(softmax_attention_mma_kernel<D16, PARTS, KT>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(plan.smem)));
    have = plan.smem;
  }
  return launch(softmax_attention_mma_kernel<D16, PARTS, KT>, dim3(n_tiles, sa.kv_heads * plan.chunks, sa.splits), dim3(plan.warps * 32), plan.smem, st, sa,
                plan.chunks);
}

int launch_softmax_mma_any(const SoftmaxAttnArgs<bf16>& sa, const SoftmaxMmaPlan& plan, int n_tiles, cudaStream_t st);

template <int D16>
int launch_softmax_decode_t(const SoftmaxAttnArgs<bf16>& sa, cudaStream_t st) {
  const size_t smem = softmax_decode_smem_bytes(sa.dim, sa.k_pages == sa.v_pages);
  static size_t have = 0;  // per instantiation
  if (smem > 48 * 1024 && smem > have) {
    MTX_CUDA(cudaFuncSetAttribute(softmax_attention_decode_kernel<D16>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    have = smem;
  }
  const int chunks = (sa.heads / sa.kv_heads + 7) / 8;
  return launch(softmax_attention_decode_kernel<D16>, dim3(sa.rows, sa.kv_heads * chunks, sa.splits), dim3(kSdecWarps * 32), smem, st, sa);
}

// a step of single tokens (every row its own tile and sequence): the transposed kernel.  Its keys are cut into one to four splits,
// the count that makes the waves of CTAs (as many CTAs at once as the kernel's shared memory lets the GPU hold) times a split's
// length shortest; a split's start-up counts like two key tiles, and a sequence without a window like one of 2048 keys
int launch_softmax_decode(mtx_layered* e, SoftmaxAttnArgs<bf16> sa, int d16, cudaStream_t st) {
  const long long ctas = (long long)sa.rows * sa.kv_heads * ((sa.heads / sa.kv_heads + 7) / 8);
  const size_t smem = softmax_decode_smem_bytes(sa.dim, sa.k_pages == sa.v_pages);
  long long per_sm = (long long)((227 * 1024) / (smem + 1024));
  per_sm = per_sm > 16 ? 16 : (per_sm < 1 ? 1 : per_sm);
  const long long slots = per_sm * e->num_sms;
  const double tiles = sa.window > 0 ? double((sa.window + kSdecKeys - 1) / kSdecKeys) : 32.0;
  static const int force = env_int("MTX_SOFTMAX_DECODE_SPLITS", 0);
  double best = 0.0;
  sa.splits = 1;
  for (int sp = 1; sp <= 4; ++sp) {
    if (size_t(sp) * sa.rows > e->attn_part_rows) break;
    const double cost = double((ctas * sp + slots - 1) / slots) * (tiles / sp + 2.0);
    if (sp == 1 || cost < best - 1e-9) {
      best = cost;
      sa.splits = sp;
    }
  }
  if (force >= 1 && force <= 4 && size_t(force) * sa.rows <= e->attn_part_rows) sa.splits = force;
  sa.part_o = e->attn_part;
  sa.part_ml = e->smax_ml;
  int rc = MTX_ERR_UNSUPPORTED;
  switch (d16) {
    case 1: rc = launch_softmax_decode_t<1>(sa, st); break;
    case 2: rc = launch_softmax_decode_t<2>(sa, st); break;
    case 3: rc = launch_softmax_decode_t<3>(sa, st); break;
    case 4: rc = launch_softmax_decode_t<4>(sa, st); break;
    case 6: rc = launch_softmax_decode_t<6>(sa, st); break;
    case 8: rc = launch_softmax_decode_t<8>(sa, st); break;
    case 16: rc = launch_softmax_decode_t<16>(sa, st); break;
  }
  MTX_TRY(rc);
  if (sa.splits > 1) return launch(softmax_attention_merge_kernel, dim3((sa.rows * sa.heads + 3) / 4), dim3(128), 0, st, sa);
  return MTX_OK;
}

// a step of single tokens has few work items, each a long walk over its sequence's keys: the keys are cut into up to four splits
// (the partial results' room) until every SM has about six CTAs, and a second kernel adds the parts
int launch_softmax_mma(mtx_layered* e, SoftmaxAttnArgs<bf16> sa, const SoftmaxMmaPlan& plan, int n_tiles, bool single_rows, cudaStream_t st) {
  sa.splits = 1;
  const long long ctas = (long long)n_tiles * sa.kv_heads * plan.chunks;
  if (single_rows && ctas < 3LL * e->num_sms) {
    long long sp = (6LL * e->num_sms + ctas - 1) / ctas;
    sa.splits = int(sp > 4 ? 4 : sp);
    if (size_t(sa.splits) * sa.rows > e->attn_part_rows) sa.splits = 1;
  }
  if (sa.splits > 1) {
    sa.part_o = e->attn_part;
    sa.part_ml = e->smax_ml;
  }
  MTX_TRY(launch_softmax_mma_any(sa, plan, n_tiles, st));
  if (sa.splits > 1) return launch(softmax_attention_merge_kernel, dim3((sa.rows * sa.heads + 3) / 4), dim3(128), 0, st, sa);
  return MTX_OK;
}

int launch_softmax_mma_any(const SoftmaxAttnArgs<bf16>& sa, const SoftmaxMmaPlan& plan, int n_tiles, cudaStream_t st) {
  switch (plan.d16) {
    case 1: return launch_softmax_mma_t<1, 1, 64>(sa, plan, n_tiles, st);
    case 2: return launch_softmax_mma_t<2, 1, 64>(sa, plan, n_tiles, st);
    case 3: return launch_softmax_mma_t<3, 1, 64>(sa, plan, n_tiles, st);
    case 4: return launch_softmax_mma_t<4, 1, 64>(sa, plan, n_tiles, st);
    case 6: return launch_softmax_mma_t<6, 1, 64>(sa, plan, n_tiles, st);
    case 8: return launch_softmax_mma_t<8, 1, 64>(sa, plan, n_tiles, st);
    case 16: return launch_softmax_mma_t<16, 2, 32>(sa, plan, n_tiles, st);
  }
  return fail(MTX_ERR_UNSUPPORTED, "no tensor-core attention for dim %d", sa.dim);
}

// causal softmax attention of the step's rows over the paged cache: the tensor-core kernels for bf16 engines whose head sizes they
// are built for (single-token steps: the transposed kernel), else the fp32 row kernel
template <typename T>
int run_softmax_attention(mtx_layered* e, SoftmaxAttnArgs<T>& sa, const mtx_ragged_batch& b, cudaStream_t st) {
  bool done = false;
  if constexpr (sizeof(T) == 2) {
    const SoftmaxMmaPlan plan = softmax_mma_plan(sa.heads, sa.kv_heads, sa.dim, sa.vdim);
    static const int decode_arm = env_int("MTX_SOFTMAX_DECODE", 1);
    if (plan.ok && use_softmax_mma() && sa.ld_out % 2 == 0) {
      if (b.n_tiles == sa.rows && decode_arm) MTX_TRY(launch_softmax_decode(e, sa, plan.d16, st));
      else MTX_TRY(launch_softmax_mma(e, sa, plan, b.n_tiles, b.n_tiles == sa.rows, st));
      done = true;
    }
  }
  const size_t smem = softmax_attn_smem_bytes(sa.dim, sa.vdim);
  static size_t attr_bytes[2] = {0, 0};  // per instantiation (bf16, float)
  size_t& have = attr_bytes[sizeof(T) == 4 ? 1 : 0];
  if (smem > 48 * 1024 && smem > have) {
    MTX_CUDA(cudaFuncSetAttribute(softmax_attention_rows_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)));
    have = smem;
  }
  if (!done) MTX_TRY(launch(softmax_attention_rows_kernel<T>, dim3(b.n_tiles, sa.heads), dim3(kSmaxThreads), smem, st, sa));
  return MTX_OK;
}

// a MTX_MIXER_COMPOSITE layer with MTX_NORM_SANDWICH norms; xa holds wnorm(x, norm1) on entry
template <typename T>
int composite_layer(mtx_layered* e, int li, const mtx_ragged_batch& b, cudaStream_t st) {
  const mtx_layered_config& c = e->cfg;
  const mtx_layer_desc& l = e->layers[li];
  const int rows = b.rows, E = c.width;
  T* xa = static_cast<T*>(e->xa);
  const CompositeCols cc = composite_cols(l);
  const int n_in = l.n_in;
  if (l.b_in) MTX_TRY((linear<T, LIN_BIAS>(e, xa, l.w_in, l.b_in, e->qkv, nullptr, rows, n_in, E, st)));
  else MTX_TRY((linear<T, LIN_PLAIN>(e, xa, l.w_in, nullptr, e->qkv, nullptr, rows, n_in, E, st)));
  T* mix = static_cast<T*>(e->attn);  // [rows, k_out]: the attention's heads, then the recurrence's
  if (l.attn.heads > 0) {
    const mtx_softmax_attn_desc& a = l.attn;
    RopeAppendArgs<T> ra;
    memset(&ra, 0, sizeof(ra));
    ra.proj = e->qkv;
    ra.ld = n_in;
    ra.q_col = cc.aq;
    ra.k_col = cc.ak;
    ra.v_col = cc.av;
    ra.rot_freq = a.rot_freq;
    ra.q_out = static_cast<T*>(e->q);
    ra.k_pages = static_cast<T*>(a.k_pages);
    ra.v_pages = static_cast<T*>(a.v_pages);
    ra.group = b.group;
    ra.pos = b.pos;
    ra.page_map = b.page_map;
    ra.heads = a.heads;
    ra.kv_heads = a.kv_heads;
    ra.dim = a.dim;
    ra.vdim = a.vdim;
    ra.rot_dims = a.rot_dims;
    ra.num_pages = c.num_pages;
    ra.tokens_per_page = c.tokens_per_page;
    ra.max_pages = c.max_pages_per_group;
    MTX_TRY(launch(rope_append_kernel<T>, dim3(rows), dim3(256), 0, st, ra));
    SoftmaxAttnArgs<T> sa;
    memset(&sa, 0, sizeof(sa));
    sa.q = static_cast<const T*>(e->q);
    sa.out = mix;
    sa.ld_out = cc.k_out;
    sa.k_pages = static_cast<const T*>(a.k_pages);
    sa.v_pages = static_cast<const T*>(a.v_pages);
    sa.group = b.group;
    sa.pos = b.pos;
    sa.page_map = b.page_map;
    sa.tile_row0 = b.tile_row0;
    sa.heads = a.heads;
    sa.kv_heads = a.kv_heads;
    sa.dim = a.dim;
    sa.vdim = a.vdim;
    sa.window = a.window;
    sa.num_pages = c.num_pages;
    sa.tokens_per_page = c.tokens_per_page;
    sa.max_pages = c.max_pages_per_group;
    sa.scale = a.scale;
    sa.out_scale = a.out_scale;
    sa.splits = 1;
    sa.rows = rows;
    MTX_TRY(run_softmax_attention<T>(e, sa, b, st));
  }
  if (l.rec.kind != 0) {
    const mtx_recurrent_desc& r = l.rec;
    RecPrepareArgs pa;
    memset(&pa, 0, sizeof(pa));
    pa.proj = e->qkv;
    pa.ld = n_in;
    pa.x_col = cc.rx;
    pa.kind = r.kind;
    pa.heads = r.heads;
    pa.dim = r.dim;
    pa.rank = r.decay_rank;
    pa.tau = r.tau;
    pa.cap = r.gate_cap;
    pa.up_t = r.decay_up_t;
    pa.bias = r.kind == MTX_REC_GLA ? r.decay_bias : r.gate_bias;
    pa.out = e->rec_aux;
    MTX_TRY(launch(recurrent_prepare_kernel, dim3(rows), dim3(256), r.kind == MTX_REC_GLA ? sizeof(float) * r.decay_rank : 0, st, pa));
    RecScanArgs ra;
    memset(&ra, 0, sizeof(ra));
    ra.proj = e->qkv;
    ra.ld = n_in;
    ra.q_col = cc.rq;
    ra.k_col = cc.rk;
    ra.v_col = cc.rv;
    ra.aux = e->rec_aux;
    ra.o = e->rec_o;
    ra.state_s = r.state_s;
    ra.state_n = r.state_n;
    ra.state_m = r.state_m;
    ra.run_row0 = b.run_row0;
    ra.group = b.group;
    ra.pos = b.pos;
    ra.heads = r.heads;
    ra.dim = r.dim;
    ra.vdim = r.vdim;
    ra.q_scale = r.q_scale;
    ra.denom_eps = r.denom_eps;
    ra.vec4 = (n_in % 4 == 0 && cc.rq % 4 == 0 && cc.rk % 4 == 0 && cc.rv % 4 == 0 && r.dim % 4 == 0 && r.vdim % 4 == 0) ? 1 : 0;
    if (r.kind == MTX_REC_GLA) MTX_TRY(launch_rec_scan<REC_GLA>(e, ra, b.n_runs, rows, st));
    else MTX_TRY(launch_rec_scan<REC_MLSTM>(e, ra, b.n_runs, rows, st));
    RecOutArgs<T> oa;
    memset(&oa, 0, sizeof(oa));
    oa.o = e->rec_o;
    oa.proj = e->qkv;
    oa.ld = n_in;
    oa.g_col = cc.rg;
    oa.weight = r.out_norm;
    oa.out = mix;
    oa.ld_out = cc.k_out;
    oa.out_col = cc.out_rec;
    oa.heads = r.heads;
    oa.vdim = r.vdim;
    oa.gate_silu = r.gate_silu;
    oa.eps = c.eps;
    oa.out_scale = r.out_scale;
    MTX_TRY(launch(recurrent_out_kernel<T>, dim3(rows), dim3(256), 0, st, oa));
  }
  MTX_TRY((linear<T, LIN_PLAIN>(e, mix, l.wo, nullptr, e->y, nullptr, rows, E, cc.k_out, st)));
  const bool has_ff = l.ff_kind == MTX_FF_MOE ? l.moe.experts > 0 : l.ff > 0;
  MTX_TRY(sandwich_step<T>(e, e->y, l.bo, l.norm1b, has_ff ? l.norm2 : nullptr, has_ff ? -1 : li + 1, rows, st));
  if (!has_ff) return MTX_OK;
  if (l.ff_kind == MTX_FF_MOE) {
    const mtx_moe_desc& m = l.moe;
    const int entries = rows * m.top;
    if (m.experts <= 64) MTX_TRY(launch(moe_router_kernel<T>, dim3(rows), dim3(256), 0, st, (const T*)xa, static_cast<const T*>(m.w_router), e->moe_logits, m.experts, E));
    else MTX_TRY((linear<T, LIN_PLAIN>(e, xa, m.w_router, nullptr, e->moe_logits, nullptr, rows, m.experts, E, st)));
    MoeRouteArgs ra;
    memset(&ra, 0, sizeof(ra));
    ra.logits = e->moe_logits;
    ra.correction = m.correction;
    ra.chosen = e->moe_chosen;
    ra.weight = e->moe_weight;
    ra.experts = m.experts;
    ra.top = m.top;
    ra.groups = m.groups;
    ra.keep = m.keep_groups;
    MTX_TRY(launch(moe_route_kernel, dim3(rows), dim3(32), sizeof(float) * (2 * m.experts + m.groups), st, ra));
    MTX_TRY(launch(moe_sort_kernel, dim3(1), dim3(1024), sizeof(int) * (2 * m.experts + 1), st, (const int*)e->moe_chosen, entries, m.top, m.experts,
                   e->moe_off, e->moe_slot, e->moe_row));
    MTX_TRY((linear_grouped<T, LIN_GATED_CLAMP>(xa, e->moe_row, m.w_gate_up, (long long)2 * m.ff * E, e->moe_off, m.experts, nullptr, e->moe_act, entries,
                                                2 * m.ff, E, m.limit, st)));
    MTX_TRY((linear_grouped<T, LIN_PLAIN>(e->moe_act, nullptr, m.w_down, (long long)E * m.ff, e->moe_off, m.experts, e->moe_y, nullptr, entries, E, m.ff,
                                          0.0f, st)));
    if (m.shared_ff > 0) {
      MTX_TRY((linear<T, LIN_GATED_CLAMP>(e, xa, m.shared_gate_up, nullptr, nullptr, e->act, rows, 2 * m.shared_ff, E, st, m.shared_limit)));
      MTX_TRY((linear<T, LIN_PLAIN>(e, e->act, m.shared_down, nullptr, e->y, nullptr, rows, E, m.shared_ff, st)));
    }
    MTX_TRY(launch(moe_combine_kernel, dim3(rows), dim3(256), 0, st, (const float*)e->moe_y, (const int*)e->moe_slot, (const float*)e->moe_weight, m.top, E,
                   m.shared_ff > 0 ? 1 : 0, e->y));
  } else {
    if (l.ff_kind == MTX_FF_CLAMPED_GATED)
      MTX_TRY((linear<T, LIN_GATED_CLAMP>(e, xa, l.w_gate_up, nullptr, nullptr, e->act, rows, 2 * l.ff, E, st, l.ff_limit)));
    else MTX_TRY((linear<T, LIN_GATED>(e, xa, l.w_gate_up, nullptr, nullptr, e->act, rows, 2 * l.ff, E, st)));
    MTX_TRY((linear<T, LIN_PLAIN>(e, e->act, l.w_down, nullptr, e->y, nullptr, rows, E, l.ff, st)));
  }
  return sandwich_step<T>(e, e->y, nullptr, l.norm2b, nullptr, li + 1, rows, st);
}

// Column layout of a MTX_NORM_PARALLEL layer's input projection, and the columns its mixer fills of the activation that the
// shared output projection reads (the feed-forward's hidden units follow them).
struct ParallelCols {
  int aq = 0, ak = 0, av = 0, ag = 0;         // softmax attention: q, k, v, head gates
  int lq = 0, lkv = 0, lg = 0;                // latent attention: query latent, key / value latent + rotated part, head gates
  int rq = 0, rk = 0, rv = 0, rg = 0, ra = 0, rx = 0;  // delta rule: q, k, v, output gate, removal, decay down-projection
  int n = 0, k_mix = 0;
};

ParallelCols parallel_cols(const mtx_layer_desc& l) {
  ParallelCols pc;
  int at = 0;
  const mtx_softmax_attn_desc& a = l.attn;
  const mtx_latent_attn_desc& m = l.latent;
  const mtx_recurrent_desc& r = l.rec;
  if (a.heads > 0) {
    pc.aq = at;
    at += a.heads * a.dim;
    if (!a.shared_kv) {
      pc.ak = at;
      at += a.kv_heads * a.dim;
      pc.av = at;
      at += a.kv_heads * a.vdim;
    }
    pc.ag = at;
    if (a.head_gate) at += a.heads;
    pc.k_mix = a.heads * a.vdim;
  } else if (m.heads > 0) {
    pc.lq = at;
    at += m.q_rank;
    pc.lkv = at;
    at += m.kv_rank + m.rot_dim;
    pc.lg = at;
    at += m.heads;
    pc.k_mix = m.heads * m.vdim;
  } else if (r.kind != 0) {
    pc.rq = at;
    at += r.heads * r.dim;
    pc.rk = at;
    at += r.heads * r.dim;
    pc.rv = at;
    at += r.heads * r.vdim;
    pc.rg = at;
    at += r.heads * r.vdim;
    pc.ra = at;
    at += r.heads * r.dim;
    pc.rx = at;
    at += r.decay_rank;
    pc.k_mix = r.heads * r.vdim;
  }
  pc.n = at;
  return pc;
}

// every row of the step is a single token of its own sequence: the norm, the input convolutions and the ring update are one kernel
bool single_token_rows(const mtx_ragged_batch& b) {
  static int on = env_int("MTX_FUSED_NORM_CONV", 1);
  return on != 0 && b.n_runs == b.rows;
}

template <typename T>
InputConvArgs<T> input_conv_args(mtx_layered* e, const mtx_layer_desc& l, const mtx_ragged_batch& b) {
  InputConvArgs<T> ca;
  memset(&ca, 0, sizeof(ca));
  ca.h = e->h;
  ca.w1 = l.conv1;
  ca.w2 = l.ff > 0 ? l.conv2 : nullptr;
  ca.state = l.conv_state;
  ca.out1 = static_cast<T*>(e->xa);  // the mixer's input
  ca.out2 = static_cast<T*>(e->xb);  // the feed-forward's input
  ca.group = b.group;
  ca.pos = b.pos;
  ca.rows = b.rows;
  ca.width = e->cfg.width;
  ca.taps = l.conv_taps;
  return ca;
}

// x += mult * y (y null: no update), then h = gnorm(x) with the weight of layer `next` (none after the last layer); in steps of
// single tokens also that layer's input convolutions
template <typename T>
int group_norm_step(mtx_layered* e, const float* y, float mult, int next, const mtx_ragged_batch& b, cudaStream_t st) {
  const bool last = next >= e->cfg.num_layers;
  const float* w = last ? nullptr : e->layers[next].norm1;
  if (!y && !w) return MTX_OK;
  const mtx_layered_config& c = e->cfg;
  const dim3 grid(b.rows, c.norm_groups < 8 ? c.norm_groups : 1);
  if (!last && single_token_rows(b))
    return launch(group_norm_step_kernel<T, true>, grid, dim3(256), 0, st, y, mult, e->x, w, c.eps, e->h, c.width, c.norm_groups,
                  input_conv_args<T>(e, e->layers[next], b));
  InputConvArgs<T> none;
  memset(&none, 0, sizeof(none));
  return launch(group_norm_step_kernel<T, false>, grid, dim3(256), 0, st, y, mult, e->x, w, c.eps, e->h, c.width, c.norm_groups, none);
}

// a MTX_NORM_PARALLEL layer; h holds gnorm(x, norm1) on entry
template <typename T>
int parallel_layer(mtx_layered* e, int li, const mtx_ragged_batch& b, cudaStream_t st) {
  const mtx_layered_config& c = e->cfg;
  const mtx_layer_desc& l = e->layers[li];
  const int rows = b.rows, E = c.width;
  T* xa = static_cast<T*>(e->xa);  // the mixer's input
  T* xb = static_cast<T*>(e->xb);  // the feed-forward's input
  const ParallelCols pc = parallel_cols(l);
  const int n_in = l.n_in, k_cat = pc.k_mix + l.ff;
  T* cat = static_cast<T*>(e->attn);  // [rows, k_cat]: the mixer's heads, then the feed-forward's hidden units
  if (!single_token_rows(b)) {  // (else the kernel that normed the rows has done this too)
    MTX_TRY(launch(input_conv_kernel<T>, dim3(rows), dim3(256), 0, st, input_conv_args<T>(e, l, b)));
    if (l.conv_taps > 1)
      MTX_TRY(launch(conv_state_update_kernel, dim3(b.n_runs, l.conv_taps - 1), dim3(256), 0, st, (const float*)e->h, l.conv_state, b.run_row0, b.group, b.pos, E,
                     l.conv_taps, (long long)E));
  }
  MTX_TRY((linear<T, LIN_PLAIN>(e, xa, l.w_in, nullptr, e->qkv, nullptr, rows, n_in, E, st)));
  SoftmaxAttnArgs<T> sa;
  memset(&sa, 0, sizeof(sa));
  sa.group = b.group;
  sa.pos = b.pos;
  sa.page_map = b.page_map;
  sa.tile_row0 = b.tile_row0;
  sa.num_pages = c.num_pages;
  sa.tokens_per_page = c.tokens_per_page;
  sa.max_pages = c.max_pages_per_group;
  sa.out_scale = 1.0f;
  sa.splits = 1;
  sa.rows = rows;
  sa.ld_gate = n_in;
  if (l.attn.heads > 0) {
    const mtx_softmax_attn_desc& a = l.attn;
    QkPrepareArgs<T> qa;
    memset(&qa, 0, sizeof(qa));
    qa.proj = e->qkv;
    qa.ld = n_in;
    qa.q_col = pc.aq;
    qa.k_col = pc.ak;
    qa.v_col = pc.av;
    qa.q_norm = a.q_norm;
    qa.k_norm = a.k_norm;
    qa.rot_freq = a.rot_freq;
    qa.q_out = static_cast<T*>(e->q);
    qa.k_pages = static_cast<T*>(a.k_pages);
    qa.v_pages = static_cast<T*>(a.v_pages);
    qa.group = b.group;
    qa.pos = b.pos;
    qa.page_map = b.page_map;
    qa.heads = a.heads;
    qa.kv_heads = a.kv_heads;
    qa.dim = a.dim;
    qa.vdim = a.vdim;
    qa.rot_dims = a.rot_dims;
    qa.rot_half = a.rot_half;
    qa.shared_kv = a.shared_kv;
    qa.num_pages = c.num_pages;
    qa.tokens_per_page = c.tokens_per_page;
    qa.max_pages = c.max_pages_per_group;
    qa.eps = c.eps;
    MTX_TRY(launch(qk_prepare_append_kernel<T>, dim3(rows), dim3(256), 0, st, qa));
    sa.q = static_cast<const T*>(e->q);
    sa.out = cat;
    sa.ld_out = k_cat;
    sa.k_pages = static_cast<const T*>(a.k_pages);
    sa.v_pages = static_cast<const T*>(a.v_pages);
    sa.heads = a.heads;
    sa.kv_heads = a.kv_heads;
    sa.dim = a.dim;
    sa.vdim = a.vdim;
    sa.window = a.window;
    sa.scale = a.scale;
    sa.slopes = a.slopes;
    sa.sink = a.sink;
    sa.gate = a.head_gate ? e->qkv + pc.ag : nullptr;
    MTX_TRY(run_softmax_attention<T>(e, sa, b, st));
  } else if (l.latent.heads > 0) {
    const mtx_latent_attn_desc& m = l.latent;
    const int H = m.heads, dl = m.kv_rank + m.rot_dim, dq = m.dim + m.rot_dim;
    T* cq = static_cast<T*>(e->act);        // [rows, q_rank]
    T* q_plain = static_cast<T*>(e->lat_o);  // [rows, H * dim], consumed before the attention writes its result to the same plane
    T* q_full = static_cast<T*>(e->q);       // [rows, H * dl]
    T* o_lat = static_cast<T*>(e->lat_o);    // [rows, H * dl]
    LatentPrepareArgs<T> la;
    memset(&la, 0, sizeof(la));
    la.proj = e->qkv;
    la.ld = n_in;
    la.q_col = pc.lq;
    la.kv_col = pc.lkv;
    la.q_rank = m.q_rank;
    la.kv_rank = m.kv_rank;
    la.rot_dim = m.rot_dim;
    la.rot_half = m.rot_half;
    la.q_norm = m.q_norm;
    la.kv_norm = m.kv_norm;
    la.rot_freq = m.rot_freq;
    la.cq_out = cq;
    la.pages = static_cast<T*>(m.pages);
    la.group = b.group;
    la.pos = b.pos;
    la.page_map = b.page_map;
    la.tokens_per_page = c.tokens_per_page;
    la.max_pages = c.max_pages_per_group;
    la.eps = c.eps;
    MTX_TRY(launch(latent_prepare_kernel<T>, dim3(rows), dim3(256), 0, st, la));
    MTX_TRY((linear<T, LIN_PLAIN>(e, cq, m.w_uq, nullptr, e->lat_q, nullptr, rows, H * dq, m.q_rank, st)));
    LatentQueryArgs<T> lq;
    memset(&lq, 0, sizeof(lq));
    lq.q = e->lat_q;
    lq.q_plain = q_plain;
    lq.q_full = q_full;
    lq.rot_freq = m.rot_freq;
    lq.pos = b.pos;
    lq.heads = H;
    lq.dim = m.dim;
    lq.rot_dim = m.rot_dim;
    lq.kv_rank = m.kv_rank;
    lq.rot_half = m.rot_half;
    MTX_TRY(launch(latent_query_kernel<T>, dim3(rows), dim3(256), 0, st, lq));
    // the plain query parts into the latent space, head by head
    MTX_TRY(linear_batched<T>(q_plain, (long long)H * m.dim, m.dim, m.w_uk_t, (long long)m.kv_rank * m.dim, q_full, (long long)H * dl, dl, rows, m.kv_rank,
                              m.dim, H, st));
    sa.q = q_full;
    sa.out = o_lat;
    sa.ld_out = (long long)H * dl;
    sa.k_pages = static_cast<const T*>(m.pages);
    sa.v_pages = static_cast<const T*>(m.pages);  // the values are the cached rows themselves
    sa.heads = H;
    sa.kv_heads = 1;
    sa.dim = dl;
    sa.vdim = dl;
    sa.window = 0;
    sa.scale = m.scale;
    sa.sink = m.sink;
    sa.gate = e->qkv + pc.lg;
    MTX_TRY(run_softmax_attention<T>(e, sa, b, st));
    // ... and the weighted latents out of it
    MTX_TRY(linear_batched<T>(o_lat, (long long)H * dl, dl, m.w_uv, (long long)m.vdim * m.kv_rank, cat, k_cat, m.vdim, rows, m.vdim, m.kv_rank, H, st));
  } else {
    const mtx_recurrent_desc& r = l.rec;
    DeltaPrepareArgs pa;
    memset(&pa, 0, sizeof(pa));
    pa.proj = e->qkv;
    pa.ld = n_in;
    pa.k_col = pc.rk;
    pa.a_col = pc.ra;
    pa.x_col = pc.rx;
    pa.heads = r.heads;
    pa.dim = r.dim;
    pa.rank = r.decay_rank;
    pa.rate = r.decay_rate;
    pa.key_eps = r.key_eps;
    pa.up_t = r.decay_up_t;
    pa.w_bias = r.decay_bias;
    pa.a_bias = r.gate_bias;
    pa.out = e->rec_aux;
    MTX_TRY(launch(delta_prepare_kernel, dim3(rows, (r.heads + 7) / 8), dim3(256), sizeof(float) * r.decay_rank, st, pa));
    RecScanArgs ra;
    memset(&ra, 0, sizeof(ra));
    ra.proj = e->qkv;
    ra.ld = n_in;
    ra.q_col = pc.rq;
    ra.k_col = pc.rk;
    ra.v_col = pc.rv;
    ra.aux = e->rec_aux;
    ra.o = e->rec_o;
    ra.state_s = r.state_s;
    ra.run_row0 = b.run_row0;
    ra.group = b.group;
    ra.pos = b.pos;
    ra.heads = r.heads;
    ra.dim = r.dim;
    ra.vdim = r.vdim;
    ra.q_scale = r.q_scale;
    ra.vec4 = (n_in % 4 == 0 && pc.rq % 4 == 0 && pc.rk % 4 == 0 && pc.rv % 4 == 0 && r.dim % 4 == 0 && r.vdim % 4 == 0) ? 1 : 0;
    MTX_TRY(launch_rec_scan<REC_DELTA>(e, ra, b.n_runs, rows, st));
    RecOutArgs<T> oa;
    memset(&oa, 0, sizeof(oa));
    oa.o = e->rec_o;
    oa.proj = e->qkv;
    oa.ld = n_in;
    oa.g_col = pc.rg;
    oa.weight = r.out_norm;
    oa.out = cat;
    oa.ld_out = k_cat;
    oa.out_col = 0;
    oa.heads = r.heads;
    oa.vdim = r.vdim;
    oa.gate_silu = r.gate_silu;
    oa.eps = c.eps;
    oa.out_scale = r.out_scale;
    MTX_TRY(launch(recurrent_out_kernel<T>, dim3(rows), dim3(256), 0, st, oa));
  }
  if (l.ff > 0) MTX_TRY((linear<T, LIN_RELU2>(e, xb, l.w_gate_up, nullptr, nullptr, cat + pc.k_mix, rows, l.ff, E, st, 0.0f, k_cat)));
  MTX_TRY((linear<T, LIN_PLAIN>(e, cat, l.wo, nullptr, e->y, nullptr, rows, E, k_cat, st)));
  return group_norm_step<T>(e, e->y, l.residual_mult, li + 1, b, st);
}

// Column layout of a MTX_NORM_PRE layer's input projection.
struct PreCols {
  int aq = 0, ak = 0, av = 0;                           // softmax attention: q, k, v
  int rq = 0, rb = 0, ra = 0, rg = 0;                   // gated delta rule: q | k | v from rq, write strengths, the decay's input, the gate's input
  int n = 0, k_mix = 0;
};

PreCols pre_cols(const mtx_layer_desc& l) {
  PreCols pc;
  const mtx_softmax_attn_desc& a = l.attn;
  const mtx_recurrent_desc& r = l.rec;
  int at = 0;
  if (a.heads > 0) {
    pc.aq = at;
    at += a.heads * a.dim;
    if (!a.shared_kv) {
      pc.ak = at;
      at += a.kv_heads * a.dim;
      pc.av = at;
      at += a.kv_heads * a.vdim;
    }
    pc.k_mix = a.heads * a.vdim;
  } else {
    const int G = r.kv_heads > 0 ? r.kv_heads : r.heads;
    pc.rq = at;
    at += 2 * G * r.dim + r.heads * r.vdim;
    pc.rb = at;
    at += r.heads;
    pc.ra = at;
    at += r.decay_rank > 0 ? r.decay_rank : r.heads;
    pc.rg = at;
    at += r.gate_rank > 0 ? r.gate_rank : r.heads * r.vdim;
    pc.k_mix = r.heads * r.vdim;
  }
  pc.n = at;
  return pc;
}

// MTX_NORM_PRE: x += y (or unit(y) * y_w; y null: no update), optionally a copy of x in the matmul dtype to xb, then unit(x) * w:
// `next` >= 0: the norm before layer `next`'s mixer (none after the last layer), to the plane h, or -- in steps of single tokens --
// straight through that layer's input convolution into xa; `next` < 0: the norm `w` before a feed-forward, to xa
template <typename T>
int pre_norm_step(mtx_layered* e, const float* y, const float* y_w, const float* self_w, bool copy_x, int next, const float* w, const mtx_ragged_batch& b,
                  cudaStream_t st) {
  PreNormArgs pa;
  memset(&pa, 0, sizeof(pa));
  pa.y = y;
  pa.y_w = y_w;
  pa.self_w = self_w;
  pa.x = e->x;
  pa.eps = e->cfg.eps;
  pa.width = e->cfg.width;
  T* xc = copy_x ? static_cast<T*>(e->xb) : nullptr;
  InputConvArgs<T> cv;
  memset(&cv, 0, sizeof(cv));
  if (next >= 0) {
    if (next >= e->cfg.num_layers) {
      if (!y && !self_w && !copy_x) return MTX_OK;
      return launch(pre_norm_step_kernel<T, false>, dim3(b.rows), dim3(256), 0, st, pa, xc, (T*)nullptr, cv);
    }
    const mtx_layer_desc& nl = e->layers[next];
    pa.w = nl.norm1;
    if (single_token_rows(b)) {
      cv = input_conv_args<T>(e, nl, b);
      cv.w2 = nullptr;
      cv.out2 = nullptr;
      return launch(pre_norm_step_kernel<T, true>, dim3(b.rows), dim3(256), 0, st, pa, xc, (T*)nullptr, cv);
    }
    pa.h = e->h;
    return launch(pre_norm_step_kernel<T, false>, dim3(b.rows), dim3(256), 0, st, pa, xc, (T*)nullptr, cv);
  }
  pa.w = w;
  return launch(pre_norm_step_kernel<T, false>, dim3(b.rows), dim3(256), 0, st, pa, xc, static_cast<T*>(e->xa), cv);
}

// a MTX_NORM_PRE layer; h holds unit(x) * norm1 on entry (steps of single tokens: xa already holds the mixer's input)
template <typename T>
int prenorm_layer(mtx_layered* e, int li, const mtx_ragged_batch& b, cudaStream_t st) {
  const mtx_layered_config& c = e->cfg;
  const mtx_layer_desc& l = e->layers[li];
  const int rows = b.rows, E = c.width;
  T* xa = static_cast<T*>(e->xa);
  const PreCols pc = pre_cols(l);
  const int n_in = l.n_in;
  T* mix = static_cast<T*>(e->attn);  // [rows, k_mix]
  if (!single_token_rows(b)) {  // (else the kernel that normed the rows has done this too)
    InputConvArgs<T> ca = input_conv_args<T>(e, l, b);
    ca.w2 = nullptr;
    ca.out2 = nullptr;
    MTX_TRY(launch(input_conv_kernel<T>, dim3(rows), dim3(256), 0, st, ca));
    if (l.conv_taps > 1)
      MTX_TRY(launch(conv_state_update_kernel, dim3(b.n_runs, l.conv_taps - 1), dim3(256), 0, st, (const float*)e->h, l.conv_state, b.run_row0, b.group, b.pos, E,
                     l.conv_taps, (long long)E));
  }
  MTX_TRY((linear<T, LIN_PLAIN>(e, xa, l.w_in, nullptr, e->qkv, nullptr, rows, n_in, E, st)));
  if (l.attn.heads > 0) {
    const mtx_softmax_attn_desc& a = l.attn;
    QkPrepareArgs<T> qa;
    memset(&qa, 0, sizeof(qa));
    qa.proj = e->qkv;
    qa.ld = n_in;
    qa.q_col = pc.aq;
    qa.k_col = pc.ak;
    qa.v_col = pc.av;
    qa.q_norm = a.q_norm;
    qa.k_norm = a.k_norm;
    qa.norm_whole = a.norm_whole;
    qa.rot_freq = a.rot_freq;
    qa.q_out = static_cast<T*>(e->q);
    qa.k_pages = static_cast<T*>(a.k_pages);
    qa.v_pages = static_cast<T*>(a.v_pages);
    qa.group = b.group;
    qa.pos = b.pos;
    qa.page_map = b.page_map;
    qa.heads = a.heads;
    qa.kv_heads = a.kv_heads;
    qa.dim = a.dim;
    qa.vdim = a.vdim;
    qa.rot_dims = a.rot_dims;
    qa.rot_half = a.rot_half;
    qa.shared_kv = a.shared_kv;
    qa.num_pages = c.num_pages;
    qa.tokens_per_page = c.tokens_per_page;
    qa.max_pages = c.max_pages_per_group;
    qa.eps = c.eps;
    MTX_TRY(launch(qk_prepare_append_kernel<T>, dim3(rows), dim3(256), 0, st, qa));
    if (a.pool > 0 && !a.pool_shared) {  // the blocks that this step's rows complete
      PoolAppendArgs<T> pa;
      memset(&pa, 0, sizeof(pa));
      pa.k_pages = static_cast<const T*>(a.k_pages);
      pa.v_pages = static_cast<const T*>(a.v_pages);
      pa.kp_pages = static_cast<T*>(a.kp_pages);
      pa.vp_pages = static_cast<T*>(a.vp_pages);
      pa.group = b.group;
      pa.pos = b.pos;
      pa.page_map = b.page_map;
      pa.kv_heads = a.kv_heads;
      pa.dim = a.dim;
      pa.vdim = a.vdim;
      pa.pool = a.pool;
      pa.pool_slots = a.pool_slots;
      pa.num_pages = c.num_pages;
      pa.tokens_per_page = c.tokens_per_page;
      pa.max_pages = c.max_pages_per_group;
      MTX_TRY(launch(pool_append_kernel<T>, dim3(rows), dim3(256), 0, st, pa));
    }
    SoftmaxAttnArgs<T> sa;
    memset(&sa, 0, sizeof(sa));
    sa.group = b.group;
    sa.pos = b.pos;
    sa.page_map = b.page_map;
    sa.tile_row0 = b.tile_row0;
    sa.num_pages = c.num_pages;
    sa.tokens_per_page = c.tokens_per_page;
    sa.max_pages = c.max_pages_per_group;
    sa.out_scale = a.out_scale != 0.0f ? a.out_scale : 1.0f;
    sa.splits = 1;
    sa.rows = rows;
    sa.q = static_cast<const T*>(e->q);
    sa.out = mix;
    sa.ld_out = pc.k_mix;
    sa.k_pages = static_cast<const T*>(a.k_pages);
    sa.v_pages = static_cast<const T*>(a.v_pages);
    sa.heads = a.heads;
    sa.kv_heads = a.kv_heads;
    sa.dim = a.dim;
    sa.vdim = a.vdim;
    sa.window = a.window;
    sa.scale = a.scale;
    sa.slopes = a.slopes;
    sa.sink = a.sink;
    sa.softcap = a.softcap;
    sa.pool = a.pool;
    sa.pool_slots = a.pool_slots;
    sa.kp_pages = static_cast<const T*>(a.kp_pages);
    sa.vp_pages = static_cast<const T*>(a.vp_pages);
    MTX_TRY(run_softmax_attention<T>(e, sa, b, st));
  } else {
    const mtx_recurrent_desc& r = l.rec;
    const int G = r.kv_heads > 0 ? r.kv_heads : r.heads, C = 2 * G * r.dim + r.heads * r.vdim;
    const GDeltaCols gc = gdelta_cols(r.heads, G, r.dim, r.vdim);
    // the low-rank projections: the gate's input rounded to the matmul dtype, the decay's split into two such parts so that its
    // up-projection (the matrix written twice along k) keeps fp32 accuracy on the tensor cores
    T* gate_in = static_cast<T*>(e->act);                                                     // [rows, gate_rank]
    T* decay_in = gate_in + align_up(size_t(c.max_rows), 256) * size_t(r.gate_rank);          // [rows, 2 * decay_rank]
    if (r.decay_rank > 0 || r.gate_rank > 0) {
      const long long total = (long long)rows * (r.decay_rank + r.gate_rank);
      const int blocks = int((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
      MTX_TRY(launch(lowrank_split_kernel<T>, dim3(blocks), dim3(256), 0, st, (const float*)e->qkv, (long long)n_in, pc.ra, r.decay_rank, pc.rg, r.gate_rank, decay_in,
                     gate_in, (long long)rows));
    }
    if (r.decay_rank > 0)  // (the any-shape kernel: its result is fp32; the tcgen05 projection would round it)
      MTX_TRY((run_linear<T, LIN_PLAIN>(e, decay_in, r.decay_up_t, nullptr, e->rec_z, nullptr, rows, r.heads * r.dim, 2 * r.decay_rank, st)));
    if (r.gate_rank > 0)
      MTX_TRY((linear<T, LIN_PLAIN>(e, gate_in, r.w_gate_up, nullptr, e->rec_gate, nullptr, rows, r.heads * r.vdim, r.gate_rank, st)));
    GDeltaPrepareArgs<T> ga;
    memset(&ga, 0, sizeof(ga));
    ga.proj = e->qkv + pc.rq;
    ga.ld = n_in;
    ga.b_col = pc.rb - pc.rq;
    ga.a_col = pc.ra - pc.rq;
    ga.heads = r.heads;
    ga.kv_heads = G;
    ga.dim = r.dim;
    ga.vdim = r.vdim;
    ga.taps = r.conv_taps;
    ga.rank = r.decay_rank;
    ga.key_eps = r.key_eps;
    ga.conv_w = r.conv_w;
    ga.state = r.conv_state;
    ga.a_log = r.a_log;
    ga.bias = r.decay_bias;
    ga.z = e->rec_z;
    ga.group = b.group;
    ga.pos = b.pos;
    ga.out = e->rec_aux;
    {
      // a warp per unit (q / k / v heads, decays per head, write strengths); few rows: the units of a row over several CTAs
      const int units = 2 * G + 2 * r.heads + 1;
      int parts = (4 * e->num_sms + rows - 1) / rows;
      if (parts > (units + 7) / 8) parts = (units + 7) / 8;
      if (parts < 1) parts = 1;
      MTX_TRY(launch(gdelta_prepare_kernel<T>, dim3(rows, parts), dim3(256), 0, st, ga));
    }
    if (r.conv_taps > 1)
      MTX_TRY(launch(conv_state_update_kernel, dim3(b.n_runs, r.conv_taps - 1), dim3(256), 0, st, (const float*)(e->qkv + pc.rq), r.conv_state, b.run_row0, b.group,
                     b.pos, C, r.conv_taps, (long long)n_in));
    RecScanArgs ra;
    memset(&ra, 0, sizeof(ra));
    ra.proj = e->rec_aux;
    ra.ld = gc.n;
    ra.q_col = gc.q;
    ra.k_col = gc.k;
    ra.v_col = gc.v;
    ra.aux = e->rec_aux;
    ra.aux_ld = gc.n;
    ra.dec_col = gc.decay;
    ra.beta_col = gc.beta;
    ra.qk_rep = r.heads / G;
    ra.o = e->rec_o;
    ra.state_s = r.state_s;
    ra.run_row0 = b.run_row0;
    ra.group = b.group;
    ra.pos = b.pos;
    ra.heads = r.heads;
    ra.dim = r.dim;
    ra.vdim = r.vdim;
    ra.q_scale = r.q_scale;
    ra.vec4 = (r.dim % 4 == 0 && r.vdim % 4 == 0) ? 1 : 0;  // (the plane's parts start on multiples of four floats)
    MTX_TRY(launch_rec_scan<REC_GDELTA>(e, ra, b.n_runs, rows, st));
    RecOutArgs<T> oa;
    memset(&oa, 0, sizeof(oa));
    oa.o = e->rec_o;
    oa.proj = r.gate_rank > 0 ? e->rec_gate : e->qkv;
    oa.ld = r.gate_rank > 0 ? r.heads * r.vdim : n_in;
    oa.g_col = r.gate_rank > 0 ? 0 : pc.rg;
    oa.weight = r.out_norm;
    oa.out = mix;
    oa.ld_out = pc.k_mix;
    oa.out_col = 0;
    oa.heads = r.heads;
    oa.vdim = r.vdim;
    oa.gate_silu = r.gate_silu;
    oa.eps = c.eps;
    oa.out_scale = r.out_scale != 0.0f ? r.out_scale : 1.0f;
    MTX_TRY(launch(recurrent_out_kernel<T>, dim3(rows), dim3(256), 0, st, oa));
  }
  MTX_TRY((linear<T, LIN_PLAIN>(e, mix, l.wo, nullptr, e->y, nullptr, rows, E, pc.k_mix, st)));
  const mtx_moe_desc& m = l.moe;
  const bool has_ff = m.experts > 0, has_side = l.side_dim > 0;
  if (has_ff) {
    MTX_TRY(pre_norm_step<T>(e, e->y, nullptr, nullptr, false, -1, l.norm2, b, st));  // x += mixer; xa = unit(x) * norm2
    const int entries = rows * m.top;
    const float limit = m.act_silu ? 0.0f : m.limit, shared_limit = m.act_silu ? 0.0f : m.shared_limit;
    if (m.experts <= 64) MTX_TRY(launch(moe_router_kernel<T>, dim3(rows), dim3(256), 0, st, (const T*)xa, static_cast<const T*>(m.w_router), e->moe_logits, m.experts, E));
    else MTX_TRY((linear<T, LIN_PLAIN>(e, xa, m.w_router, nullptr, e->moe_logits, nullptr, rows, m.experts, E, st)));
    MoeRouteArgs ra;
    memset(&ra, 0, sizeof(ra));
    ra.logits = e->moe_logits;
    ra.correction = m.correction;
    ra.chosen = e->moe_chosen;
    ra.weight = e->moe_weight;
    ra.experts = m.experts;
    ra.top = m.top;
    ra.groups = m.groups > 0 ? m.groups : 1;
    ra.keep = m.keep_groups > 0 ? m.keep_groups : 1;
    ra.softmax = m.score_softmax;
    ra.plain = m.plain_weights;
    MTX_TRY(launch(moe_route_kernel, dim3(rows), dim3(32), sizeof(float) * (2 * m.experts + ra.groups), st, ra));
    MTX_TRY(launch(moe_sort_kernel, dim3(1), dim3(1024), sizeof(int) * (2 * m.experts + 1), st, (const int*)e->moe_chosen, entries, m.top, m.experts,
                   e->moe_off, e->moe_slot, e->moe_row));
    MTX_TRY((linear_grouped<T, LIN_GATED_CLAMP>(xa, e->moe_row, m.w_gate_up, (long long)2 * m.ff * E, e->moe_off, m.experts, nullptr, e->moe_act, entries,
                                                2 * m.ff, E, limit, st)));
    MTX_TRY((linear_grouped<T, LIN_PLAIN>(e->moe_act, nullptr, m.w_down, (long long)E * m.ff, e->moe_off, m.experts, e->moe_y, nullptr, entries, E, m.ff,
                                          0.0f, st)));
    if (m.shared_ff > 0) {
      MTX_TRY((linear<T, LIN_GATED_CLAMP>(e, xa, m.shared_gate_up, nullptr, nullptr, e->act, rows, 2 * m.shared_ff, E, st, shared_limit)));
      MTX_TRY((linear<T, LIN_PLAIN>(e, e->act, m.shared_down, nullptr, e->y, nullptr, rows, E, m.shared_ff, st)));
    }
    MTX_TRY(launch(moe_combine_kernel, dim3(rows), dim3(256), 0, st, (const float*)e->moe_y, (const int*)e->moe_slot, (const float*)e->moe_weight, m.top, E,
                   m.shared_ff > 0 ? 1 : 0, e->y));
  }
  if (!has_side) return pre_norm_step<T>(e, e->y, nullptr, nullptr, false, li + 1, nullptr, b, st);  // x += the last sublayer; the next layer's norm
  // x += the last sublayer, and x in the matmul dtype for the side input's gate
  MTX_TRY(pre_norm_step<T>(e, e->y, nullptr, nullptr, true, c.num_layers, nullptr, b, st));
  const int gate_rows = l.side_gate_rows > l.side_dim ? l.side_gate_rows : l.side_dim;
  MTX_TRY((linear<T, LIN_PLAIN>(e, e->xb, l.side_gate, nullptr, e->qkv, nullptr, rows, gate_rows, E, st)));
  const long long total = (long long)rows * l.side_dim;
  const int blocks = int((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  MTX_TRY(launch(side_act_kernel<T>, dim3(blocks), dim3(256), 0, st, (const float*)e->qkv, (long long)gate_rows, b.token, static_cast<const T*>(c.side_embed),
                 (long long)c.side_width, l.side_col, c.vocab, static_cast<T*>(e->act), l.side_dim, total));
  MTX_TRY((linear<T, LIN_PLAIN>(e, e->act, l.side_proj, nullptr, e->y, nullptr, rows, E, l.side_dim, st)));
  return pre_norm_step<T>(e, e->y, l.side_norm, nullptr, false, li + 1, nullptr, b, st);  // x += unit(y) * side_norm; the next layer's norm
}

template <typename T>
int step_typed(mtx_layered* e, const mtx_ragged_batch& b, cudaStream_t st) {
  const mtx_layered_config& c = e->cfg;
  const int rows = b.rows, E = c.width;
  T* xa = static_cast<T*>(e->xa);
  MTX_TRY(launch(embed_rows_kernel<T>, dim3(rows), dim3(128), 0, st, b.token, static_cast<const T*>(c.embedding), c.vocab, c.embed_scale, e->x, xa, E,
                 e->sandwich ? e->x0 : (float*)nullptr));
  if (e->sandwich) MTX_TRY(sandwich_step<T>(e, nullptr, nullptr, nullptr, nullptr, 0, rows, st));  // layer 0's pre-adds and pre-norm
  if (e->parallel) MTX_TRY(group_norm_step<T>(e, nullptr, 0.0f, 0, b, st));                         // layer 0's norm
  if (e->prenorm) MTX_TRY(pre_norm_step<T>(e, nullptr, nullptr, c.embed_norm, false, 0, nullptr, b, st));  // the embedding's norm, layer 0's norm
  for (int li = 0; li < c.num_layers; ++li) {
    if (e->layers[li].norm_style == MTX_NORM_PRE) MTX_TRY(prenorm_layer<T>(e, li, b, st));
    else if (e->layers[li].norm_style == MTX_NORM_PARALLEL) MTX_TRY(parallel_layer<T>(e, li, b, st));
    else if (e->layers[li].mixer == MTX_MIXER_COMPOSITE) MTX_TRY(composite_layer<T>(e, li, b, st));
    else MTX_TRY(window_layer<T>(e, li, b, st));
  }
  if (b.n_want > 0) {
    T* wn = static_cast<T*>(e->wanted);
    if (e->parallel || e->prenorm)
      MTX_TRY(launch(group_norm_rows_kernel<T>, dim3(b.n_want), dim3(256), 0, st, (const float*)e->x, b.want_rows, c.final_norm, c.eps, wn, E,
                     e->prenorm ? 1 : c.norm_groups));
    else if (c.final_norm) MTX_TRY(launch(weighted_norm_rows_kernel<T>, dim3(b.n_want), dim3(256), 0, st, (const float*)e->x, b.want_rows, c.final_norm, c.eps, wn, E));
    else MTX_TRY(launch(scalar_norm_rows_kernel<T>, dim3(b.n_want), dim3(256), 0, st, (const float*)e->x, b.want_rows, c.final_gain, c.eps, wn, E));
    MTX_TRY((linear<T, LIN_PLAIN>(e, wn, c.head, nullptr, b.logits, nullptr, b.n_want, c.vocab, E, st)));
    const float logit_scale = c.logit_scale != 0.0f ? c.logit_scale : 1.0f;
    if (c.logit_softcap > 0.0f || logit_scale != 1.0f) {
      const long long total = (long long)b.n_want * c.vocab;
      const int blocks = int((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
      if (logit_scale != 1.0f) MTX_TRY(launch(logit_post_kernel, dim3(blocks), dim3(256), 0, st, b.logits, logit_scale, c.logit_softcap, total));
      else MTX_TRY(launch(softcap_kernel, dim3(blocks), dim3(256), 0, st, b.logits, c.logit_softcap, total));
    }
  }
  return MTX_OK;
}

// validation and workspace sizes of a MTX_MIXER_COMPOSITE layer
int check_composite(mtx_layered* e, int i) {
  const mtx_layer_desc& l = e->layers[i];
  const mtx_softmax_attn_desc& a = l.attn;
  const mtx_recurrent_desc& r = l.rec;
  if (l.norm_style != MTX_NORM_SANDWICH) return fail(MTX_ERR_UNSUPPORTED, "layer %d: a composite mixer layer has sandwich norms", i);
  if (!l.norm1 || !l.norm1b || !l.w_in || !l.wo) return fail(MTX_ERR_ARG, "layer %d: a norm weight or a projection is missing", i);
  if (a.heads <= 0 && r.kind == 0) return fail(MTX_ERR_ARG, "layer %d: a composite mixer needs an attention or a recurrence", i);
  if (a.heads > 0) {
    if (a.kv_heads < 1 || a.heads % a.kv_heads != 0 || a.dim < 1 || a.vdim < 1 || a.window < 0) return fail(MTX_ERR_ARG, "layer %d: bad attention geometry", i);
    if (a.values_are_keys && a.vdim != a.dim) return fail(MTX_ERR_ARG, "layer %d: values that are the keys need vdim == dim", i);
    if (a.rot_dims < 0 || a.rot_dims > a.dim || (a.rot_dims & 1) || (a.rot_dims > 0 && !a.rot_freq)) return fail(MTX_ERR_ARG, "layer %d: bad rot_dims / rot_freq", i);
    if (!a.k_pages || !a.v_pages) return fail(MTX_ERR_ARG, "layer %d: a page pool is missing", i);
    if (kSmaxRows * a.vdim > kSmaxThreads * kSmaxMaxAcc) return fail(MTX_ERR_UNSUPPORTED, "layer %d: vdim %d exceeds %d", i, a.vdim, kSmaxThreads * kSmaxMaxAcc / kSmaxRows);
    if (softmax_attn_smem_bytes(a.dim, a.vdim) > 200 * 1024) return fail(MTX_ERR_UNSUPPORTED, "layer %d: the attention's heads do not fit shared memory", i);
    if (a.heads * a.dim > e->max_qdim) e->max_qdim = a.heads * a.dim;
    if (a.heads > e->max_attn_heads) e->max_attn_heads = a.heads;
  }
  if (r.kind != 0) {
    if (r.kind != MTX_REC_GLA && r.kind != MTX_REC_MLSTM) return fail(MTX_ERR_UNSUPPORTED, "layer %d: unknown recurrence %d", i, r.kind);
    if (r.heads < 1 || r.dim < 1 || r.vdim < 1 || r.dim > kRecSlices * 32) return fail(MTX_ERR_UNSUPPORTED, "layer %d: recurrence heads / dim (<= %d) / vdim", i, kRecSlices * 32);
    if (!r.state_s || !r.out_norm) return fail(MTX_ERR_ARG, "layer %d: the recurrence's state or output norm is missing", i);
    if (r.kind == MTX_REC_GLA && (r.decay_rank < 1 || !r.decay_up_t || !(r.tau > 0.0f))) return fail(MTX_ERR_ARG, "layer %d: the decay's projection / tau is missing", i);
    if (r.kind == MTX_REC_MLSTM && (!r.state_n || !r.state_m || !r.gate_bias || !(r.gate_cap > 0.0f))) return fail(MTX_ERR_ARG, "layer %d: mLSTM state / gate bias / cap missing", i);
    if (r.heads * r.vdim > e->max_rec_o) e->max_rec_o = r.heads * r.vdim;
    const int aux = r.kind == MTX_REC_GLA ? r.heads * r.dim : 2 * r.heads;
    if (aux > e->max_rec_aux) e->max_rec_aux = aux;
  }
  const CompositeCols cc = composite_cols(l);
  if (l.n_in < cc.n) return fail(MTX_ERR_ARG, "layer %d: n_in = %d, the sub-mixers need %d projection rows", i, l.n_in, cc.n);
  if (l.n_in > e->max_nqkv) e->max_nqkv = l.n_in;
  if (cc.k_out > e->max_odim) e->max_odim = cc.k_out;
  if (l.ff_kind == MTX_FF_MOE) {
    const mtx_moe_desc& m = l.moe;
    if (m.experts > 0) {
      if (!l.norm2 || !l.norm2b) return fail(MTX_ERR_ARG, "layer %d: a feed-forward norm weight is missing", i);
      if (m.top < 1 || m.top > m.experts || m.groups < 1 || m.experts % m.groups != 0 || m.keep_groups < 1 || m.keep_groups > m.groups || m.ff < 1)
        return fail(MTX_ERR_ARG, "layer %d: bad expert / top / groups / ff", i);
      if (m.keep_groups * (m.experts / m.groups) < m.top) return fail(MTX_ERR_ARG, "layer %d: the kept groups hold fewer than `top` experts", i);
      if (m.experts > 4096) return fail(MTX_ERR_UNSUPPORTED, "layer %d: more than 4096 experts", i);
      if (!m.w_router || !m.w_gate_up || !m.w_down || (m.shared_ff > 0 && (!m.shared_gate_up || !m.shared_down))) return fail(MTX_ERR_ARG, "layer %d: an expert weight is missing", i);
      if (m.top > e->max_moe_top) e->max_moe_top = m.top;
      if (m.experts > e->max_moe_experts) e->max_moe_experts = m.experts;
      if (m.ff > e->max_moe_ff) e->max_moe_ff = m.ff;
      if (m.shared_ff > e->max_ff) e->max_ff = m.shared_ff;
      if (2 * m.shared_ff > e->max_nqkv) e->max_nqkv = 2 * m.shared_ff;
    }
  } else if (l.ff > 0) {
    if (!l.norm2 || !l.norm2b || !l.w_gate_up || !l.w_down) return fail(MTX_ERR_ARG, "layer %d: a feed-forward weight is missing", i);
    if (l.ff_kind != MTX_FF_GELU_GATED && l.ff_kind != MTX_FF_CLAMPED_GATED) return fail(MTX_ERR_UNSUPPORTED, "layer %d: unknown feed-forward kind %d", i, l.ff_kind);
    if (2 * l.ff > e->max_nqkv) e->max_nqkv = 2 * l.ff;
    if (l.ff > e->max_ff) e->max_ff = l.ff;
  }
  e->sandwich = true;
  return MTX_OK;
}

// validation and workspace sizes of a MTX_NORM_PARALLEL layer
int check_parallel(mtx_layered* e, int i) {
  const mtx_layered_config& c = e->cfg;
  const mtx_layer_desc& l = e->layers[i];
  const mtx_softmax_attn_desc& a = l.attn;
  const mtx_latent_attn_desc& m = l.latent;
  const mtx_recurrent_desc& r = l.rec;
  if (l.mixer != MTX_MIXER_COMPOSITE) return fail(MTX_ERR_UNSUPPORTED, "layer %d: a parallel layer has a composite mixer", i);
  if (c.norm_groups < 1 || c.width % c.norm_groups != 0) return fail(MTX_ERR_ARG, "norm_groups = %d does not divide the width %d", c.norm_groups, c.width);
  if (!l.norm1 || !l.w_in || !l.wo) return fail(MTX_ERR_ARG, "layer %d: the norm weight or a projection is missing", i);
  if (l.conv_taps < 1 || !l.conv1 || (l.conv_taps > 1 && !l.conv_state)) return fail(MTX_ERR_ARG, "layer %d: the input convolution's taps / weights / state", i);
  const int kinds = (a.heads > 0) + (m.heads > 0) + (r.kind != 0);
  if (kinds != 1) return fail(MTX_ERR_ARG, "layer %d: a parallel layer has exactly one mixer", i);
  if (a.heads > 0) {
    if (a.kv_heads < 1 || a.heads % a.kv_heads != 0 || a.dim < 1 || a.vdim < 1 || a.window < 0) return fail(MTX_ERR_ARG, "layer %d: bad attention geometry", i);
    if (a.rot_dims < 0 || a.rot_dims > a.dim || (a.rot_dims & 1) || (a.rot_dims > 0 && !a.rot_freq)) return fail(MTX_ERR_ARG, "layer %d: bad rot_dims / rot_freq", i);
    if (a.values_are_keys) return fail(MTX_ERR_UNSUPPORTED, "layer %d: values_are_keys belongs to sandwich layers", i);
    if (!a.k_pages || !a.v_pages) return fail(MTX_ERR_ARG, "layer %d: a page pool is missing", i);
    if (kSmaxRows * a.vdim > kSmaxThreads * kSmaxMaxAcc) return fail(MTX_ERR_UNSUPPORTED, "layer %d: vdim %d exceeds %d", i, a.vdim, kSmaxThreads * kSmaxMaxAcc / kSmaxRows);
    if (softmax_attn_smem_bytes(a.dim, a.vdim) > 200 * 1024) return fail(MTX_ERR_UNSUPPORTED, "layer %d: the attention's heads do not fit shared memory", i);
    if (a.heads * a.dim > e->max_qdim) e->max_qdim = a.heads * a.dim;
    if (a.heads > e->max_attn_heads) e->max_attn_heads = a.heads;
  }
  if (m.heads > 0) {
    if (m.dim < 1 || m.rot_dim < 0 || m.vdim < 1 || m.q_rank < 1 || m.kv_rank < 1) return fail(MTX_ERR_ARG, "layer %d: bad latent attention geometry", i);
    if (m.rot_dim > 0 && !m.rot_freq) return fail(MTX_ERR_ARG, "layer %d: rot_freq is missing", i);
    if (!m.q_norm || !m.kv_norm || !m.w_uq || !m.w_uk_t || !m.w_uv || !m.pages) return fail(MTX_ERR_ARG, "layer %d: a latent attention weight or its pool is missing", i);
    const int dl = m.kv_rank + m.rot_dim;
    if (kSmaxRows * dl > kSmaxThreads * kSmaxMaxAcc) return fail(MTX_ERR_UNSUPPORTED, "layer %d: kv_rank + rot_dim = %d exceeds %d", i, dl, kSmaxThreads * kSmaxMaxAcc / kSmaxRows);
    if (softmax_attn_smem_bytes(dl, dl) > 200 * 1024) return fail(MTX_ERR_UNSUPPORTED, "layer %d: the latent rows do not fit shared memory", i);
    if (m.heads * dl > e->max_qdim) e->max_qdim = m.heads * dl;
    if (m.heads * dl > e->max_lat_o) e->max_lat_o = m.heads * dl;
    if (m.heads * dl > e->max_odim) e->max_odim = m.heads * dl;  // (the key splits' partial results are sized by max_odim)
    if (m.heads * m.dim > e->max_lat_o) e->max_lat_o = m.heads * m.dim;
    if (m.heads * (m.dim + m.rot_dim) > e->max_lat_q) e->max_lat_q = m.heads * (m.dim + m.rot_dim);
    if (m.q_rank > e->max_ff) e->max_ff = m.q_rank;  // (the query latent waits in the plane of the feed-forward's activation)
    if (m.heads > e->max_attn_heads) e->max_attn_heads = m.heads;
  }
  if (r.kind != 0) {
    if (r.kind != MTX_REC_DELTA) return fail(MTX_ERR_UNSUPPORTED, "layer %d: a parallel layer's recurrence is the delta rule", i);
    if (r.heads < 1 || r.dim < 1 || r.vdim < 1 || r.dim > kRecSlices * 32) return fail(MTX_ERR_UNSUPPORTED, "layer %d: recurrence heads / dim (<= %d) / vdim", i, kRecSlices * 32);
    if (!r.state_s || !r.out_norm || r.decay_rank < 1 || !r.decay_up_t) return fail(MTX_ERR_ARG, "layer %d: the recurrence's state, output norm or decay projection is missing", i);
    if (r.heads * r.vdim > e->max_rec_o) e->max_rec_o = r.heads * r.vdim;
    if (3 * r.heads * r.dim > e->max_rec_aux) e->max_rec_aux = 3 * r.heads * r.dim;
  }
  const ParallelCols pc = parallel_cols(l);
  if (l.n_in < pc.n) return fail(MTX_ERR_ARG, "layer %d: n_in = %d, the mixer needs %d projection rows", i, l.n_in, pc.n);
  if (l.n_in > e->max_nqkv) e->max_nqkv = l.n_in;
  if (l.ff < 0 || (l.ff > 0 && (l.ff_kind != MTX_FF_RELU2 || !l.w_gate_up))) return fail(MTX_ERR_ARG, "layer %d: a parallel layer's feed-forward is down(relu(up x)^2)", i);
  if (pc.k_mix + l.ff > e->max_odim) e->max_odim = pc.k_mix + l.ff;
  if (l.ff > e->max_nqkv) e->max_nqkv = l.ff;  // (a tcgen05 projection parks its bf16 result in a plane of max_nqkv columns)
  if (m.heads > 0 && m.heads * (m.dim + m.rot_dim) > e->max_nqkv) e->max_nqkv = m.heads * (m.dim + m.rot_dim);
  e->parallel = true;
  return MTX_OK;
}

// validation and workspace sizes of a MTX_NORM_PRE layer
int check_prenorm(mtx_layered* e, int i) {
  const mtx_layered_config& c = e->cfg;
  const mtx_layer_desc& l = e->layers[i];
  const mtx_softmax_attn_desc& a = l.attn;
  const mtx_recurrent_desc& r = l.rec;
  const mtx_moe_desc& m = l.moe;
  if (l.mixer != MTX_MIXER_COMPOSITE) return fail(MTX_ERR_UNSUPPORTED, "layer %d: a pre-norm layer has a composite mixer", i);
  if (!l.norm1 || !l.w_in || !l.wo) return fail(MTX_ERR_ARG, "layer %d: the norm weight or a projection is missing", i);
  if (l.conv_taps < 1 || !l.conv1 || (l.conv_taps > 1 && !l.conv_state)) return fail(MTX_ERR_ARG, "layer %d: the input convolution's taps / weights / state", i);
  if ((a.heads > 0) + (r.kind != 0) != 1 || l.latent.heads > 0) return fail(MTX_ERR_ARG, "layer %d: a pre-norm layer has one mixer, an attention or a recurrence", i);
  if (a.heads > 0) {
    if (a.kv_heads < 1 || a.heads % a.kv_heads != 0 || a.dim < 1 || a.vdim < 1 || a.window < 0) return fail(MTX_ERR_ARG, "layer %d: bad attention geometry", i);
    if (a.rot_dims < 0 || a.rot_dims > a.dim || (a.rot_dims & 1) || (a.rot_dims > 0 && !a.rot_freq)) return fail(MTX_ERR_ARG, "layer %d: bad rot_dims / rot_freq", i);
    if (a.values_are_keys || a.head_gate) return fail(MTX_ERR_UNSUPPORTED, "layer %d: values_are_keys / head gates belong to other layer styles", i);
    if (!a.k_pages || !a.v_pages) return fail(MTX_ERR_ARG, "layer %d: a page pool is missing", i);
    if (a.pool < 0 || (a.pool > 0 && (a.window < 1 || a.pool_slots < 1 || !a.kp_pages || !a.vp_pages || a.k_pages == a.v_pages || a.slopes)))
      return fail(MTX_ERR_ARG, "layer %d: pooled blocks need a window, their pools, and no distance slopes", i);
    if (a.pool > 0 && !(c.tokens_per_page % a.pool == 0 ? a.pool_slots == c.tokens_per_page / a.pool : a.pool_slots == c.tokens_per_page))
      return fail(MTX_ERR_ARG, "layer %d: pool_slots = %d does not fit pages of %d tokens and blocks of %d", i, a.pool_slots, c.tokens_per_page, a.pool);
    if (kSmaxRows * a.vdim > kSmaxThreads * kSmaxMaxAcc) return fail(MTX_ERR_UNSUPPORTED, "layer %d: vdim %d exceeds %d", i, a.vdim, kSmaxThreads * kSmaxMaxAcc / kSmaxRows);
    if (softmax_attn_smem_bytes(a.dim, a.vdim) > 200 * 1024) return fail(MTX_ERR_UNSUPPORTED, "layer %d: the attention's heads do not fit shared memory", i);
    if (a.heads * a.dim > e->max_qdim) e->max_qdim = a.heads * a.dim;
    if (a.heads > e->max_attn_heads) e->max_attn_heads = a.heads;
  } else {
    if (r.kind != MTX_REC_GDELTA) return fail(MTX_ERR_UNSUPPORTED, "layer %d: a pre-norm layer's recurrence is the gated delta rule", i);
    const int G = r.kv_heads > 0 ? r.kv_heads : r.heads;
    if (r.heads < 1 || r.heads % G != 0 || r.dim < 1 || r.vdim < 1 || r.dim > kRecSlices * 32)
      return fail(MTX_ERR_UNSUPPORTED, "layer %d: recurrence heads / kv_heads / dim (<= %d) / vdim", i, kRecSlices * 32);
    if (!r.state_s || !r.out_norm || !r.a_log || !r.decay_bias || !r.conv_w || r.conv_taps < 1 || (r.conv_taps > 1 && !r.conv_state))
      return fail(MTX_ERR_ARG, "layer %d: the recurrence's state, output norm, decay constants or convolution is missing", i);
    if (r.decay_rank < 0 || r.gate_rank < 0 || (r.decay_rank > 0 && !r.decay_up_t) || (r.gate_rank > 0 && !r.w_gate_up))
      return fail(MTX_ERR_ARG, "layer %d: a low-rank decay / gate needs its up-projection", i);
    if (r.heads * r.vdim > e->max_rec_o) e->max_rec_o = r.heads * r.vdim;
    const int aux = gdelta_cols(r.heads, G, r.dim, r.vdim).n;
    if (aux > e->max_rec_aux) e->max_rec_aux = aux;
    if (r.gate_rank > 0 && r.heads * r.vdim > e->max_rec_gate) e->max_rec_gate = r.heads * r.vdim;
    if (r.decay_rank > 0 && r.heads * r.dim > e->max_rec_z) e->max_rec_z = r.heads * r.dim;
    // (the low-rank projections' inputs wait in the plane of the feed-forward's activation)
    if (r.gate_rank + 2 * r.decay_rank > e->max_ff) e->max_ff = r.gate_rank + 2 * r.decay_rank;
  }
  const PreCols pc = pre_cols(l);
  if (l.n_in < pc.n) return fail(MTX_ERR_ARG, "layer %d: n_in = %d, the mixer needs %d projection rows", i, l.n_in, pc.n);
  if (l.n_in > e->max_nqkv) e->max_nqkv = l.n_in;
  if (pc.k_mix > e->max_odim) e->max_odim = pc.k_mix;
  if (m.experts > 0) {
    if (l.ff_kind != MTX_FF_MOE || !l.norm2) return fail(MTX_ERR_ARG, "layer %d: a pre-norm layer's feed-forward is a routed one with a norm weight", i);
    const int groups = m.groups > 0 ? m.groups : 1, keep = m.keep_groups > 0 ? m.keep_groups : 1;
    if (m.top < 1 || m.top > m.experts || m.experts % groups != 0 || keep > groups || m.ff < 1 || keep * (m.experts / groups) < m.top)
      return fail(MTX_ERR_ARG, "layer %d: bad expert / top / groups / ff", i);
    if (m.experts > 4096) return fail(MTX_ERR_UNSUPPORTED, "layer %d: more than 4096 experts", i);
    if (!m.w_router || !m.w_gate_up || !m.w_down || (m.shared_ff > 0 && (!m.shared_gate_up || !m.shared_down))) return fail(MTX_ERR_ARG, "layer %d: an expert weight is missing", i);
    if (m.top > e->max_moe_top) e->max_moe_top = m.top;
    if (m.experts > e->max_moe_experts) e->max_moe_experts = m.experts;
    if (m.ff > e->max_moe_ff) e->max_moe_ff = m.ff;
    if (m.shared_ff > e->max_ff) e->max_ff = m.shared_ff;
    if (2 * m.shared_ff > e->max_nqkv) e->max_nqkv = 2 * m.shared_ff;
  }
  if (l.side_dim < 0) return fail(MTX_ERR_ARG, "layer %d: side_dim", i);
  if (l.side_dim > 0) {
    if (!l.side_gate || !l.side_proj || !l.side_norm || !c.side_embed || l.side_col < 0 || l.side_col + l.side_dim > c.side_width)
      return fail(MTX_ERR_ARG, "layer %d: the side input's weights, table or columns are missing", i);
    if (l.side_dim > e->max_ff) e->max_ff = l.side_dim;
    if (l.side_dim > e->max_nqkv) e->max_nqkv = l.side_dim;
    if (l.side_gate_rows > e->max_nqkv) e->max_nqkv = l.side_gate_rows;
  }
  e->prenorm = true;
  return MTX_OK;
}

}  // namespace

extern "C" {

int mtx_layered_create(const mtx_layered_config* cfg, const mtx_layer_desc* layers, mtx_layered** out) {
  if (!cfg || !layers || !out) return fail(MTX_ERR_ARG, "null argument");
  const mtx_layered_config& c = *cfg;
  if (c.num_layers < 1 || c.width < 1 || c.vocab < 1 || c.max_rows < 1 || c.max_want < 0) return fail(MTX_ERR_ARG, "bad layer count / width / vocab / rows");
  if (c.num_groups < 1 || c.num_pages < 2 || c.tokens_per_page < 1 || c.max_pages_per_group < 1) return fail(MTX_ERR_ARG, "bad page geometry");
  if (!c.embedding || !c.head) return fail(MTX_ERR_ARG, "embedding / head missing");
  mtx_layered* e = new mtx_layered();
  e->cfg = c;
  e->layers.assign(layers, layers + c.num_layers);
  int first_mix = -1;
  for (int i = 0; i < c.num_layers; ++i) {
    const mtx_layer_desc& l = e->layers[i];
    int rc = MTX_OK;
    if (l.norm_style == MTX_NORM_PARALLEL || l.norm_style == MTX_NORM_PRE || l.mixer == MTX_MIXER_COMPOSITE) {
      rc = l.norm_style == MTX_NORM_PRE ? check_prenorm(e, i) : (l.norm_style == MTX_NORM_PARALLEL ? check_parallel(e, i) : check_composite(e, i));
      if (rc != MTX_OK) {
        delete e;
        return rc;
      }
      continue;
    }
    if (l.mixer != MTX_MIXER_WINDOW_SIGMOID) rc = fail(MTX_ERR_UNSUPPORTED, "layer %d: unknown mixer %d", i, l.mixer);
    else if (l.norm_style != MTX_NORM_OUT_GAIN || l.ff_kind != MTX_FF_GELU_GATED)
      rc = fail(MTX_ERR_UNSUPPORTED, "layer %d: a window mixer layer has output-gain norms and a gelu-gated feed-forward", i);
    else if (l.heads < 1 || l.kv_heads < 1 || l.heads % l.kv_heads != 0 || l.dim < 1 || l.vdim < 1 || l.window < 1 || l.ff < 0)
      rc = fail(MTX_ERR_ARG, "layer %d: bad head geometry / window / ff", i);
    else if (l.heads * l.vdim > kWinThreads * kWinMaxAcc)
      rc = fail(MTX_ERR_UNSUPPORTED, "layer %d: heads * vdim = %d exceeds %d", i, l.heads * l.vdim, kWinThreads * kWinMaxAcc);
    else if (window_attn_smem_bytes(l.heads, l.kv_heads, l.dim, l.vdim, 4) > 200 * 1024)
      rc = fail(MTX_ERR_UNSUPPORTED, "layer %d: the heads do not fit the attention kernel's shared memory", i);
    else if (!l.wqkv || !l.wo || !l.dist_bias || !l.k_pages || !l.v_pages || (l.ff > 0 && (!l.w_gate_up || !l.w_down)))
      rc = fail(MTX_ERR_ARG, "layer %d: a weight or a page pool is missing", i);
    else if (l.value_mix < 0 || l.value_mix > 2) rc = fail(MTX_ERR_ARG, "layer %d: value_mix must be 0, 1 or 2", i);
    if (rc == MTX_OK && l.value_mix == 1) {
      if (first_mix >= 0) rc = fail(MTX_ERR_ARG, "layer %d: only one layer keeps its values for the others", i);
      first_mix = i;
      e->vshared_dim = l.kv_heads * l.vdim;
    }
    if (rc == MTX_OK && l.value_mix == 2 && (first_mix < 0 || l.kv_heads * l.vdim != e->vshared_dim))
      rc = fail(MTX_ERR_ARG, "layer %d mixes in the values of an earlier layer: none kept them, or their size differs", i);
    if (rc != MTX_OK) {
      delete e;
      return rc;
    }
    const int nqkv = l.heads * l.dim + l.kv_heads * (l.dim + l.vdim);
    if (nqkv > e->max_nqkv) e->max_nqkv = nqkv;
    if (l.heads * l.dim > e->max_qdim) e->max_qdim = l.heads * l.dim;
    if (l.heads * l.vdim > e->max_odim) e->max_odim = l.heads * l.vdim;
    if (2 * l.ff > e->max_nqkv) e->max_nqkv = 2 * l.ff;  // (the tcgen05 path parks the gate / up product in the same scratch)
    if (l.ff > e->max_ff) e->max_ff = l.ff;
  }
  for (int i = 0; i < c.num_layers; ++i)
    if ((e->layers[i].norm_style == MTX_NORM_SANDWICH) != e->sandwich) {
      delete e;
      return fail(MTX_ERR_UNSUPPORTED, "layer %d: all layers of a model share one norm style", i);
    }
  for (int i = 0; i < c.num_layers; ++i)
    if ((e->layers[i].norm_style == MTX_NORM_PARALLEL) != e->parallel) {
      delete e;
      return fail(MTX_ERR_UNSUPPORTED, "layer %d: all layers of a model share one norm style", i);
    }
  for (int i = 0; i < c.num_layers; ++i)
    if ((e->layers[i].norm_style == MTX_NORM_PRE) != e->prenorm) {
      delete e;
      return fail(MTX_ERR_UNSUPPORTED, "layer %d: all layers of a model share one norm style", i);
    }
  if ((e->parallel || e->prenorm) && !c.final_norm) {
    delete e;
    return fail(MTX_ERR_ARG, "a model of parallel or pre-norm layers has a final norm weight");
  }
  if (e->sandwich && c.width > 256 * kSandwichMax) {
    delete e;
    return fail(MTX_ERR_UNSUPPORTED, "width %d exceeds %d", c.width, 256 * kSandwichMax);
  }
  if (c.vocab > e->max_nqkv) e->max_nqkv = c.vocab;
  int dev = 0, sms = 0;
  if (cudaGetDevice(&dev) == cudaSuccess && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) e->num_sms = sms;
  cudaGetLastError();
  e->ws_bytes = layered_layout(e).total;
  *out = e;
  return MTX_OK;
}

int mtx_layered_destroy(mtx_layered* e) {
  if (e == nullptr) return MTX_OK;
  for (auto& g : e->graphs) cudaGraphExecDestroy(g.exec);
  if (e->cap_stream) cudaStreamDestroy(e->cap_stream);
  delete e;
  return MTX_OK;
}

size_t mtx_layered_workspace_bytes(const mtx_layered* e) { return e ? e->ws_bytes : 0; }

int mtx_layered_bind(mtx_layered* e, void* workspace, size_t workspace_bytes) {
  if (!e || !workspace) return fail(MTX_ERR_ARG, "null argument");
  if (workspace_bytes < e->ws_bytes) return fail(MTX_ERR_ARG, "workspace of %zu bytes, %zu needed", workspace_bytes, e->ws_bytes);
  if ((reinterpret_cast<uintptr_t>(workspace) & 1023) != 0) return fail(MTX_ERR_ARG, "the workspace must be 1024-byte aligned");
  const LWs L = layered_layout(e);
  char* base = static_cast<char*>(workspace);
  e->x = reinterpret_cast<float*>(base + L.x);
  e->y = reinterpret_cast<float*>(base + L.y);
  e->qkv = reinterpret_cast<float*>(base + L.qkv);
  e->v_shared = reinterpret_cast<float*>(base + L.v_shared);
  e->xa = base + L.xa;
  e->q = base + L.q;
  e->attn = base + L.attn;
  e->act = base + L.act;
  e->wanted = base + L.wanted;
  e->obf = base + L.obf;
  e->attn_part = reinterpret_cast<float*>(base + L.attn_part);
  e->attn_part_rows = 4 * align_up(size_t(e->cfg.max_rows), 256);
  e->smax_ml = reinterpret_cast<float*>(base + L.smax_ml);
  e->x0 = reinterpret_cast<float*>(base + L.x0);
  e->rec_o = reinterpret_cast<float*>(base + L.rec_o);
  e->rec_aux = reinterpret_cast<float*>(base + L.rec_aux);
  e->moe_logits = reinterpret_cast<float*>(base + L.moe_logits);
  e->moe_weight = reinterpret_cast<float*>(base + L.moe_weight);
  e->moe_y = reinterpret_cast<float*>(base + L.moe_y);
  e->moe_chosen = reinterpret_cast<int*>(base + L.moe_chosen);
  e->moe_slot = reinterpret_cast<int*>(base + L.moe_slot);
  e->moe_row = reinterpret_cast<int*>(base + L.moe_row);
  e->moe_off = reinterpret_cast<int*>(base + L.moe_off);
  e->moe_act = base + L.moe_act;
  e->h = reinterpret_cast<float*>(base + L.h);
  e->xb = base + L.xb;
  e->lat_q = reinterpret_cast<float*>(base + L.lat_q);
  e->lat_o = base + L.lat_o;
  e->rec_gate = reinterpret_cast<float*>(base + L.rec_gate);
  e->rec_z = reinterpret_cast<float*>(base + L.rec_z);
  e->bound = true;
  return MTX_OK;
}

int mtx_layered_step(mtx_layered* e, const mtx_ragged_batch* b, mtx_stream stream) {
  if (!e || !e->bound || !b) return fail(MTX_ERR_ARG, "engine is not bound / null argument");
  if (b->rows < 1 || b->rows > e->cfg.max_rows) return fail(MTX_ERR_ARG, "rows = %d outside [1, %d]", b->rows, e->cfg.max_rows);
  if (b->n_want < 0 || b->n_want > e->cfg.max_want) return fail(MTX_ERR_ARG, "n_want = %d outside [0, %d]", b->n_want, e->cfg.max_want);
  if (!b->token || !b->group || !b->pos || !b->page_map || (b->n_want > 0 && (!b->want_rows || !b->logits))) return fail(MTX_ERR_ARG, "null batch array");
  if (b->n_tiles < 0 || b->n_tiles > b->rows) return fail(MTX_ERR_ARG, "n_tiles = %d for %d rows", b->n_tiles, b->rows);
  if ((e->sandwich || e->parallel || e->prenorm) && (b->n_tiles < 1 || !b->tile_row0 || b->n_runs < 1 || b->n_runs > b->rows || !b->run_row0))
    return fail(MTX_ERR_ARG, "this model needs the batch's query tiles and runs");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return e->cfg.float32 ? step_typed<float>(e, *b, st) : step_typed<bf16>(e, *b, st);
}

int mtx_layered_step_graph(mtx_layered* e, const mtx_ragged_batch* b, mtx_stream stream) {
  if (!e || !e->bound || !b) return fail(MTX_ERR_ARG, "engine is not bound / null argument");
  for (auto& g : e->graphs) {
    if (memcmp(&g.key, b, sizeof(*b)) == 0) {
      MTX_CUDA(cudaGraphLaunch(g.exec, static_cast<cudaStream_t>(stream)));
      return MTX_OK;
    }
  }
  if (e->graphs.size() >= 64) return mtx_layered_step(e, b, stream);  // (a caller that never repeats a descriptor)
  if (!e->cap_stream) MTX_CUDA(cudaStreamCreateWithFlags(&e->cap_stream, cudaStreamNonBlocking));
  cudaGraph_t graph = nullptr;
  MTX_CUDA(cudaStreamBeginCapture(e->cap_stream, cudaStreamCaptureModeThreadLocal));
  const int rc = mtx_layered_step(e, b, e->cap_stream);
  const cudaError_t end = cudaStreamEndCapture(e->cap_stream, &graph);
  if (rc != MTX_OK) {
    if (graph) cudaGraphDestroy(graph);
    return rc;
  }
  if (end != cudaSuccess) return fail(MTX_ERR_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(end));
  cudaGraphExec_t exec = nullptr;
  const cudaError_t inst = cudaGraphInstantiate(&exec, graph, 0);
  cudaGraphDestroy(graph);
  if (inst != cudaSuccess) return fail(MTX_ERR_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(inst));
  mtx_layered::GraphEntry ge;
  memcpy(&ge.key, b, sizeof(*b));
  ge.exec = exec;
  e->graphs.push_back(ge);
  MTX_CUDA(cudaGraphLaunch(exec, static_cast<cudaStream_t>(stream)));
  return MTX_OK;
}

}  // extern "C"
