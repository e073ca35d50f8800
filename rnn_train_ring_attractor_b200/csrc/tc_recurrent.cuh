// Shared definitions of the bf16 tensor-core recurrent kernels (forward and reverse-time).
//
// Decomposition.  The padded neuron count NP (128, 256 or 512) is split over a thread-block cluster of
// C = NP/128 CTAs; a cluster owns one tile of 128 samples at a time and runs all its timesteps.  CTA q of the
// cluster produces neurons [128q, 128q+128) in two sub-slices of 64.  Per step every CTA needs the whole
// previous state as the A operand [128 samples x NP] (bf16, K-major, 128-byte swizzle, one 16 KB chunk per
// 64 neurons); the weights for its own output neurons are the B operand, streamed by TMA through a ring of
// shared-memory stages (or loaded once when they fit).  After the epilogue each CTA pushes its two new
// 64-neuron chunks into every peer's A buffer with one-destination bulk copies over distributed shared
// memory; mbarriers carry the byte counts.
//
// Weight blocks.  For CTA q, sub-slice s the B operand is a block of RB = 208 rows x NP columns:
//   rows   0.. 63  matrix 0 (Wo)   rows 64..127  matrix 1 (Wl)   rows 128..191  matrix 2 (Wr)
//   row  192       ones (for columns < N): its accumulator column is the row sum of the A operand,
//                  which the J0 (global inhibition) term needs;  rows 193..207 zero.
// One tcgen05.mma with N = 208 therefore yields, per sample, the three 64-wide products and the row sum.
#pragma once

#include <cuda_bf16.h>

#include "ringrnn_common.cuh"
#include "tc_ptx.cuh"

namespace ringrnn {
namespace tcr {

constexpr int RB = 208;              // rows of one weight block
constexpr int WT_BYTES = RB * 128;   // one [RB x 64] bf16 tile
constexpr int CHUNK_BYTES = 128 * 128;  // one [128 samples x 64 neurons] bf16 chunk
constexpr int THREADS = 384;         // warps 0-3: TMA / MMA / relay / idle; warps 4-11: epilogue
constexpr int SMEM_LIMIT = 232448;   // 227 KB
constexpr int TMEM_COLS = 512;
constexpr int SUM_COL = 192;

template <int NP>
struct Cfg {
  static constexpr int C = NP / 128;   // CTAs per cluster
  static constexpr int KC = NP / 64;   // K chunks
  static constexpr int A_BYTES = KC * CHUNK_BYTES;
  static constexpr int TILES = 2 * KC;  // weight tiles per step
  static constexpr int AUX = 2048;      // barriers, flags, decode vectors
  static constexpr int NS_FIT = (SMEM_LIMIT - 1024 - AUX - A_BYTES) / WT_BYTES;
  static constexpr bool RESIDENT = NS_FIT >= TILES;
  static constexpr int NS = RESIDENT ? TILES : NS_FIT;
  static constexpr int SMEM = 1024 + A_BYTES + NS * WT_BYTES + AUX;
  static_assert(NS >= 2, "weight ring too small");
  static_assert(NS <= 16, "barrier block sized for 16 stages");
};

// barrier block: byte offsets from its base
constexpr uint32_t OFF_W_FULL = 0;     // [16]
constexpr uint32_t OFF_W_EMPTY = 128;  // [16]
constexpr uint32_t OFF_A_FULL = 256;   // [8]
constexpr uint32_t OFF_D_FULL = 320;   // [2]
constexpr uint32_t OFF_D_EMPTY = 336;  // [2]
constexpr uint32_t OFF_MMA_DONE = 352;
constexpr uint32_t OFF_ALL_FREE = 360;
constexpr uint32_t OFF_TMEM_SLOT = 368;
constexpr uint32_t OFF_DEAD = 372;
constexpr uint32_t OFF_UV = 512;       // float u[128], v[128]

template <int REGS>
__device__ __forceinline__ void reg_dec() {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(REGS));
}
template <int REGS>
__device__ __forceinline__ void reg_inc() {
  asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(REGS));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// F(x) and F'(x) for a group of G independent elements, written stage by stage over the group so that the
// G dependency chains interleave (the epilogue runs with two warps per scheduler: without instruction-level
// parallelism inside the thread it is latency-bound).  Evaluation error is far below bf16 resolution.
template <int ACT, int G>
__device__ __forceinline__ void act_group(const float* x, float* f, float* d) {
  if constexpr (ACT == RINGRNN_ACT_RELU) {
#pragma unroll
    for (int i = 0; i < G; ++i) {
      f[i] = fmaxf(x[i], 0.f);
      d[i] = x[i] > 0.f ? 1.f : 0.f;
    }
  } else if constexpr (ACT == RINGRNN_ACT_TANH) {
#pragma unroll
    for (int i = 0; i < G; ++i) asm("tanh.approx.f32 %0, %1;" : "=f"(f[i]) : "f"(x[i]));
#pragma unroll
    for (int i = 0; i < G; ++i) d[i] = fmaf(-f[i], f[i], 1.f);
  } else if constexpr (ACT == RINGRNN_ACT_SILU) {
    float s[G];
#pragma unroll
    for (int i = 0; i < G; ++i) s[i] = __fdividef(1.f, 1.f + __expf(-x[i]));
#pragma unroll
    for (int i = 0; i < G; ++i) {
      f[i] = x[i] * s[i];
      d[i] = s[i] * fmaf(x[i], 1.f - s[i], 1.f);
    }
  } else {
    // exact-erf GELU: Phi(x) = (1 + erf(x/sqrt2))/2 with erf from Abramowitz-Stegun 7.1.26 (|err| < 1.5e-7);
    // exp(-x^2/2) is shared with the density term of the derivative Phi(x) + x*phi(x).
    float z[G], t[G], e[G], poly[G];
#pragma unroll
    for (int i = 0; i < G; ++i) z[i] = fabsf(x[i]) * 0.70710678118654752f;
#pragma unroll
    for (int i = 0; i < G; ++i) t[i] = __fdividef(1.f, fmaf(0.3275911f, z[i], 1.f));
#pragma unroll
    for (int i = 0; i < G; ++i) e[i] = exp2f(-1.4426950408889634f * z[i] * z[i]);
#pragma unroll
    for (int i = 0; i < G; ++i) poly[i] = fmaf(t[i], 1.061405429f, -1.453152027f);
#pragma unroll
    for (int i = 0; i < G; ++i) poly[i] = fmaf(t[i], poly[i], 1.421413741f);
#pragma unroll
    for (int i = 0; i < G; ++i) poly[i] = fmaf(t[i], poly[i], -0.284496736f);
#pragma unroll
    for (int i = 0; i < G; ++i) poly[i] = fmaf(t[i], poly[i], 0.254829592f);
#pragma unroll
    for (int i = 0; i < G; ++i) poly[i] *= t[i];
#pragma unroll
    for (int i = 0; i < G; ++i) {
      const float erf_abs = fmaf(-poly[i], e[i], 1.f);
      const float cdf = 0.5f + 0.5f * copysignf(erf_abs, x[i]);
      f[i] = x[i] * cdf;
      d[i] = fmaf(x[i] * 0.3989422804014327f, e[i], cdf);
    }
  }
}

}  // namespace tcr
}  // namespace ringrnn
