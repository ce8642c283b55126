// Grouped matrix products for a mixture of experts with MANY rows per expert (prompt portions): the grouped mode of linear_any.cuh
// (same argument block, same epilogues, slot ranges read on the device, the experts' row tiles packed along the grid's y) on
// larger tiles behind a deeper pipeline.
//
//   grouped_mma_pipe_kernel<EPI>   bf16; CTA tile 128 rows x 64 columns x 64 k, eight warps of 32 x 32 on mma.sync m16n8k16 with fp32
//                                  accumulators; the operands arrive by 16-byte cp.async (rows gathered through a_row, rows beyond
//                                  the group's last and columns beyond n zero-filled) into a ring of three stages, so that two k
//                                  steps are in flight while one is multiplied.  Needs k a multiple of 64, 16-byte aligned rows and
//                                  `groups` set (packed tiles); the host falls back to linear_mma_kernel otherwise, and for steps
//                                  with few rows per expert, whose 128-row tiles would be mostly padding.
#pragma once

#include "common.cuh"
#include "linear_any.cuh"

namespace mtx {

constexpr int kGgThreads = 256, kGgBM = 128, kGgBN = 64, kGgBK = 64, kGgPitch = kGgBK + 8, kGgStages = 3;
constexpr size_t kGgSmemBytes = size_t(kGgStages) * (kGgBM + kGgBN) * kGgPitch * sizeof(bf16);

__device__ __forceinline__ void gg_cp_async_16(void* dst_smem, const void* src, bool valid) {
  const unsigned d = static_cast<unsigned>(__cvta_generic_to_shared(dst_smem));
  const int n = valid ? 16 : 0;  // (0: the 16 bytes are zero-filled, nothing is read)
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}

template <int EPI>
__global__ void __launch_bounds__(kGgThreads) grouped_mma_pipe_kernel(const LinArgs<bf16> p_in) {
  extern __shared__ __align__(16) unsigned char gg_raw[];
  bf16* const ring = reinterpret_cast<bf16*>(gg_raw);  // stage s: A [128][pitch], then B [64][pitch]
  constexpr int STAGE = (kGgBM + kGgBN) * kGgPitch;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  griddep_wait();
  LinArgs<bf16> p = p_in;
  int row_tile;
  if (!lin_enter_group(p, kGgBM, row_tile)) return;
  const int row0 = row_tile * kGgBM, col0 = blockIdx.x * kGgBN;
  const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;
  // this thread's chunks of a stage: four of A (128 rows x 8 chunks), two of B (64 rows x 8 chunks); where they come from does not
  // change with k
  const bf16* a_src[4];
  bool a_ok[4];
#pragma unroll
  for (int it = 0; it < 4; ++it) {
    const int chunk = tid + it * kGgThreads, r = chunk >> 3, gr = row0 + r;
    a_ok[it] = gr < p.rows;
    a_src[it] = p.a + size_t(a_ok[it] ? (p.a_row ? p.a_row[gr] : gr) : 0) * p.lda + (chunk & 7) * 8;
  }
  const bf16* b_src[2];
  bool b_ok[2];
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int chunk = tid + it * kGgThreads, r = chunk >> 3, gc = col0 + r;
    b_ok[it] = gc < p.n;
    b_src[it] = p.w + size_t(b_ok[it] ? gc : 0) * p.k + (chunk & 7) * 8;
  }
  auto load_stage = [&](int kt, int stage) {
    bf16* sa = ring + size_t(stage) * STAGE;
    bf16* sb = sa + kGgBM * kGgPitch;
    const int k0 = kt * kGgBK;
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const int chunk = tid + it * kGgThreads;
      gg_cp_async_16(sa + (chunk >> 3) * kGgPitch + (chunk & 7) * 8, a_src[it] + k0, a_ok[it]);
    }
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int chunk = tid + it * kGgThreads;
      gg_cp_async_16(sb + (chunk >> 3) * kGgPitch + (chunk & 7) * 8, b_src[it] + k0, b_ok[it]);
    }
  };
  float acc[2][4][4];
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.0f;
  const int k_tiles = p.k / kGgBK;
#pragma unroll
  for (int s = 0; s < kGgStages - 1; ++s) {
    if (s < k_tiles) load_stage(s, s);
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  for (int kt = 0; kt < k_tiles; ++kt) {
    asm volatile("cp.async.wait_group %0;" ::"n"(kGgStages - 2) : "memory");  // k step kt has landed (this thread's part)
    __syncthreads();  // ... everybody's; and everybody is done with the stage of step kt - 1, which the next load overwrites
    if (kt + kGgStages - 1 < k_tiles) load_stage(kt + kGgStages - 1, (kt + kGgStages - 1) % kGgStages);
    asm volatile("cp.async.commit_group;" ::: "memory");  // (an empty group keeps the count of groups per iteration uniform)
    const bf16* sa = ring + size_t(kt % kGgStages) * STAGE;
    const bf16* sb = sa + kGgBM * kGgPitch;
#pragma unroll
    for (int kk = 0; kk < kGgBK; kk += 16) {
      uint32_t af[2][4], bfr[4][2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const bf16* base = sa + (wm + i * 16 + g) * kGgPitch + kk + 2 * t;
        af[i][0] = *reinterpret_cast<const uint32_t*>(base);
        af[i][1] = *reinterpret_cast<const uint32_t*>(base + 8 * kGgPitch);
        af[i][2] = *reinterpret_cast<const uint32_t*>(base + 8);
        af[i][3] = *reinterpret_cast<const uint32_t*>(base + 8 * kGgPitch + 8);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const bf16* base = sb + (wn + j * 8 + g) * kGgPitch + kk + 2 * t;
        bfr[j][0] = *reinterpret_cast<const uint32_t*>(base);
        bfr[j][1] = *reinterpret_cast<const uint32_t*>(base + 8);
      }
#pragma unroll
      for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
          asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                       : "+f"(acc[i][j][0]), "+f"(acc[i][j][1]), "+f"(acc[i][j][2]), "+f"(acc[i][j][3])
                       : "r"(af[i][0]), "r"(af[i][1]), "r"(af[i][2]), "r"(af[i][3]), "r"(bfr[j][0]), "r"(bfr[j][1]));
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int r = row0 + wm + i * 16 + g, c = col0 + wn + j * 8 + 2 * t;
      lin_store_pair<bf16, EPI>(p, r, c, acc[i][j][0], acc[i][j][1]);
      lin_store_pair<bf16, EPI>(p, r + 8, c, acc[i][j][2], acc[i][j][3]);
    }
}

}  // namespace mtx
