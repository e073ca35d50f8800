// Shared definitions of the bf16 tensor-core recurrent kernels (forward and reverse-time).
//
// Decomposition.  The padded neuron count NP (128, 256, 512 or 1024) is split into C = NP/128 slices of 128 neurons.
// A thread-block cluster owns one tile of samples at a time and runs all its timesteps; the CTA that owns
// slice q produces neurons [128q, 128q+128) in two sub-slices of 64.  Per step a CTA needs the whole previous
// state of its 128 samples as the A operand [128 x NP] (bf16, K-major, 128-byte swizzle, one 16 KB chunk per
// 64 neurons); the weights of its output neurons are the B operand, streamed by TMA through a ring of
// shared-memory stages (or loaded once when they fit).  After the epilogue each CTA pushes its two new
// 64-neuron chunks into the A buffers of the CTAs that hold the same samples, with one-destination bulk copies
// over distributed shared memory; mbarriers carry the byte counts.
//
// K rounds.  The A buffer has at most 8 chunk slots (128 KB).  For NP = 1024 (16 chunks) a step therefore runs in
// two rounds: round 0 multiplies chunks 0-7 (published by slices 0-3) into the accumulators, then, once every CTA of
// the cluster is done with them, slices 4-7 publish chunks 8-15 into the same slots and round 1 accumulates on top.
// Chunk kc lives in slot kc % 8 and is used in round kc / 8; NP <= 512 has a single round.
//
// Two cluster shapes:
//   single (PAIR = false): C CTAs, 128 samples, each CTA issues its own tcgen05.mma (M = 128, N = 208).
//   pair   (PAIR = true) : 2C CTAs, 256 samples.  Ranks (2q, 2q+1) hold slice q for the two halves of the samples
//          and act as one cta_group::2 MMA unit (M = 256, N = 224): each loads only half of every weight tile,
//          which halves both the L2 -> shared-memory stream and the shared-memory traffic per MMA, the two
//          things that bound the single shape.  The even CTA issues the MMAs; completions are signalled to both.
//
// Weight blocks.  For slice q, sub-slice s the B operand is a block of RB rows x NP columns:
//   rows   0.. 63  matrix 0 (Wo)   rows 64..127  matrix 1 (Wl)   rows 128..191  matrix 2 (Wr)
//   row  192       ones (for columns < N): its accumulator column is the row sum of the A operand,
//                  which the J0 (global inhibition) term needs;  remaining rows zero (RB = 208, or 224 for pairs,
//                  whose MMA wants N to be a multiple of 32).
// One MMA therefore yields, per sample, the three 64-wide products and the row sum.
#pragma once

#include <cuda_bf16.h>
#include <stdio.h>
#include <stdlib.h>

#include "ringrnn_common.cuh"
#include "tc_ptx.cuh"

namespace ringrnn {

// Optional in-kernel timeline (compile with -DRINGRNN_TIMELINE): cycle stamps of CTA `RINGRNN_TIMELINE_CTA` for the
// first 64 steps, 16 slots per step, read back with ringrnn_debug_timeline_read().  Compiled out by default.
#ifdef RINGRNN_TIMELINE
static __device__ long long g_timeline[64 * 16];  // one copy per translation unit
#ifndef RINGRNN_TIMELINE_CTA
#define RINGRNN_TIMELINE_CTA 8
#endif
#define RINGRNN_STAMP(step, slot)                                                                   \
  do {                                                                                              \
    if (blockIdx.x == RINGRNN_TIMELINE_CTA && (step) < 64) g_timeline[(step) * 16 + (slot)] = clock64(); \
  } while (0)
#define RINGRNN_STAMP_VAL(step, slot, v)                                                            \
  do {                                                                                              \
    if (blockIdx.x == RINGRNN_TIMELINE_CTA && (step) < 64) g_timeline[(step) * 16 + (slot)] = (v);  \
  } while (0)
#else
#define RINGRNN_STAMP(step, slot) do {} while (0)
#define RINGRNN_STAMP_VAL(step, slot, v) do {} while (0)
#endif

// Kernel parameters of the two recurrent kernels (filled by ringrnn_bf16.cu).
struct TcFwdParams {
  int B, T, N, BP, a_dim, colL, colR, n_tiles;  // n_tiles = BP / (128 or, for CTA pairs, 256)
  float J0, J1, alpha;
  const float* A;        // [B,T,a_dim]
  const float* r_init;   // [B,N]
  __nv_bfloat16* Rh;     // [T+1][BP][NP] (slot 0 = bf16(r_init), prepared before launch) or nullptr
  __nv_bfloat16* Dh;     // F'(re_t), blocked layout (tc_recurrent.cuh), T*BP*NP elements, or nullptr
  uint32_t* Sg;          // [T][NP/32][2][BP] bit masks "r_t == 0" and "sign bit of r_t" (bit j = neuron 32*block + j), or nullptr
  float* hist;           // [T,B,N] or nullptr
  float* dec_part;       // [2C][3][T][BP] or nullptr
  const float* dec_u;    // [N]
  const float* dec_v;
  float* final_state;    // [B,N] or nullptr
  int* status;
  // generic action columns (more than two active): the weight blocks come in `ng` groups of three matrices,
  // group 0 = {Wo, Wa[cols[0]], Wa[cols[1]]} + ones row, group m = {Wa[cols[3m-1]], Wa[cols[3m]], Wa[cols[3m+1]]}
  int ng, n_act;
  int cols[RINGRNN_MAX_ACTIVE];
  // A launch may cover steps [t0, t0 + T) of a longer sequence of T_total steps (recompute of one stretch between
  // checkpoints): A is indexed with the global step; everything this launch writes with the local one.
  int t0, T_total;
  float* ckpt;           // [ceil(T/ckpt_every)][B][N] fp32: slot c receives the state after step c*ckpt_every - 1
  int ckpt_every;        //   (slot 0, the initial state, is the caller's); nullptr = none
  // Two K rounds (N > 512): the CTAs of a cluster exchange the state through global memory.  X = Rh when the state is
  // saved (step t reads row block t, writes t+1); otherwise X = the initial-state buffer extended to three row blocks,
  // blocks 1 and 2 used in turn (x_ring = 1: step t reads block 1 + (t & 1), writes 1 + ((t+1) & 1)).  The tensor map
  // of the initial state covers X.
  __nv_bfloat16* X;
  int x_ring;
};

struct TcBwdParams {
  int B, T, N, BP, a_dim, colL, colR, n_tiles;
  float J0, J1, alpha;
  const float* A;               // [B,T,a_dim]
  const __nv_bfloat16* Dh;      // F'(re_t), blocked layout (tc_recurrent.cuh)
  const uint32_t* Sg;           // [T][NP/32][2][BP] zero / sign-bit masks of r_t
  const float* grad_output;     // [T,B,N] or nullptr
  const float* coef_x;          // [B,T] or nullptr
  const float* coef_y;
  const float* coef_s;
  const float* dec_u;           // [N]
  const float* dec_v;
  __nv_bfloat16* DL;            // [T*BP][3*NP]
  float* grad_r_init;           // [B,N] or nullptr
  const __nv_bfloat16* Rh;      // [T+1][BP][NP] saved state (read only when dA_part is set)
  float* dA_part;               // [2C][2][T][BP] partial sums of dL/dL_t and dL/dR_t (generic columns:
                                // [4C][n_act][T][BP]), or nullptr
  int* status;
  int ng, n_act;                // as in TcFwdParams; DL then has 1 + n_act column blocks [delta | A_k * delta ...]
  int cols[RINGRNN_MAX_ACTIVE];
  // steps [t0, t0 + T) of a sequence of T_total: A, grad_output and the loss coefficients are indexed with the global
  // step, the saved tensors, DL and the dL/dA partial sums with the local one
  int t0, T_total;
  const float* carry_in;        // [B,N] gradient flowing into the last state of this stretch from later steps, or nullptr
};

// `generic`: more than two active action columns (p.ng > 1 weight groups); NP <= 512, no CTA pairs
int tc_forward_launch(int act, int NP, bool pair, const CUtensorMap& tmW, const CUtensorMap& tmR0, const TcFwdParams& p,
                      cudaStream_t s);
// tmDL: DL with a [128 rows x 64 columns] box (128-byte swizzle: the delta chunks); tmDL32: the same tensor with a
// [32 x 32] box (64-byte swizzle: the scaled copies, one store per epilogue warp)
int tc_backward_launch(int NP, bool pair, const CUtensorMap& tmW, const CUtensorMap& tmDL, const CUtensorMap& tmDL32,
                       const TcBwdParams& p, cudaStream_t s);

namespace tcr {

constexpr int CHUNK_BYTES = 128 * 128;  // one [128 samples x 64 neurons] bf16 chunk
constexpr int THREADS = 384;         // warps 0-3: TMA / MMA / relay / idle; warps 4-11: epilogue
// Register re-distribution (setmaxnreg): the CTA is launched with 168 registers per thread (65536 / 384, rounded down
// to a multiple of 8); warps 0-3 give theirs back down to LOW_REGS, the epilogue warps grow to HIGH_REGS.  The sum
// must fit in what the CTA was launched with -- a request beyond that waits for ever, it is not an error.
constexpr int LOW_REGS = 40, HIGH_REGS = 232;
static_assert((4 * LOW_REGS + 8 * HIGH_REGS) * 32 <= (65536 / THREADS / 8 * 8) * THREADS,
              "setmaxnreg budget exceeds the registers the CTA is launched with");
constexpr int SMEM_LIMIT = 232448;   // 227 KB
constexpr int TMEM_COLS = 512;
constexpr int SUM_COL = 192;

constexpr int block_rows(bool pair) { return pair ? 224 : 208; }

template <int NP, bool PAIR>
struct Cfg {
  static constexpr int C = NP / 128;             // neuron slices
  static constexpr int CL = PAIR ? 2 * C : C;    // CTAs per cluster
  static constexpr int TILE_ROWS = PAIR ? 256 : 128;
  static constexpr int KC = NP / 64;             // K chunks
  static constexpr int SLOTS = KC < 8 ? KC : 8;  // chunk slots of the A buffer
  static constexpr int ROUNDS = KC / SLOTS;      // K rounds per step
  static constexpr int RB = block_rows(PAIR);    // rows of one weight block = accumulator columns used
  static constexpr int WROWS = PAIR ? RB / 2 : RB;  // rows of a weight tile this CTA loads
  // Weight stages: [WROWS x 64] tiles of 26 KB, filled by tiled TMA loads.  Two variations were built, passed the parity
  // suite and were taken out again because they measured slower: stages of 32 k-columns in the 64-byte swizzle (six of
  // 13 KB instead of three of 26 KB at N = 512: forward 6.14 against 5.16 ms) and weights stored tile by tile in the
  // shared-memory layout so that one untiled bulk copy fills a stage (N = 512 unchanged, N = 1024 13 % slower).  The
  // stream is bound by the rate at which data enters an SM (about 50 B/clk, whatever the ring depth), not by latency.
  static constexpr int WT_BYTES = WROWS * 128;   // one [WROWS x 64] bf16 tile
  static constexpr int A_BYTES = SLOTS * CHUNK_BYTES;
  static constexpr int TILES = 2 * KC;           // weight tiles per step
  static constexpr int AUX = 2048;               // barriers, flags, decode vectors
  static constexpr int STAGE_BYTES = 8 * 2048;   // one 32-row x 64-byte transposition buffer per epilogue warp
  static constexpr int NS_FIT = (SMEM_LIMIT - 1024 - AUX - STAGE_BYTES - A_BYTES) / WT_BYTES;
  static constexpr bool RESIDENT = NS_FIT >= TILES;
  static constexpr int NS = RESIDENT ? TILES : (NS_FIT > 16 ? 16 : NS_FIT);
  static constexpr int SMEM = 1024 + A_BYTES + NS * WT_BYTES + AUX + STAGE_BYTES;
  // Early publication (forward, single CTAs, one K round, more than one slice): a CTA sends the new chunk of its
  // sub-slice 0 to its peers while it still works on sub-slice 1, so that half of the state exchange is hidden behind
  // the second half of the epilogue instead of standing between two steps.
  static constexpr bool EARLY = !PAIR && ROUNDS == 1 && C > 1;
  // Exchange through global memory (two K rounds = clusters of 8), used whenever the published tensor is kept in
  // global memory anyway (the saved state in training, delta for the weight gradients).  A chunk that goes to seven
  // peers as seven distributed-shared-memory copies leaves its SM at about 10 B/clk (224 KB per step and CTA: 19-21 K
  // cycles for an all-gather, measured), and the copies may only start once every peer has freed the slots.  Instead
  // the epilogue threads write their part of the chunks straight from registers into that tensor (it replaces the TMA
  // store), fence, and one of them raises a flag in every CTA of the cluster, its own included; a thread per slice in
  // each CTA (puller_loop) loads the chunks into the A buffer with TMA as soon as ITS OWN MMAs have left the slots.
  // Data enters an SM at the 50 B/clk of any TMA load, nothing waits for a cluster-wide "free", and the chunks of the
  // second round -- known since the previous step's epilogue -- are in flight the moment the first round ends.
#ifdef RINGRNN_NO_PULL
  static constexpr bool PULL = false;
#else
  static constexpr bool PULL = ROUNDS > 1;
#endif
  static_assert(NS >= 2, "weight ring too small");
  static_assert(NS <= 16, "barrier block sized for 16 stages");
  static_assert(WT_BYTES % 1024 == 0, "stages must keep the 1024-byte swizzle alignment");
  static_assert(!PAIR || ROUNDS == 1, "CTA pairs are written for a single K round");
  static_assert(!RESIDENT || ROUNDS == 1, "resident weights are written for a single K round");
  static_assert(ROUNDS <= 2, "barrier block sized for two K rounds");
};

// barrier block: byte offsets from its base
constexpr uint32_t OFF_W_FULL = 0;     // [16]
constexpr uint32_t OFF_W_EMPTY = 128;  // [16]
constexpr uint32_t OFF_A_FULL = 256;   // [8]  slot i of this CTA's A buffer holds its chunk of the current round
constexpr uint32_t OFF_D_FULL = 320;   // [2]
constexpr uint32_t OFF_D_EMPTY = 336;  // [2]
constexpr uint32_t OFF_MMA_DONE = 352; // one phase per (step, round): this CTA's MMAs of the round are complete
constexpr uint32_t OFF_ALL_FREE = 360; // [2]  per round, one phase per step: every CTA's MMAs of the round are complete
constexpr uint32_t OFF_TMEM_SLOT = 376;
constexpr uint32_t OFF_DEAD = 380;
constexpr uint32_t OFF_A_PAIR = 384;   // [8]  (even CTA of a pair) chunk kc is complete in the odd CTA too
constexpr uint32_t OFF_STORE_DONE = 448;  // (two rounds) the TMA store of this CTA's own chunks has read them
constexpr uint32_t OFF_OWN0_FREE = 456;   // (early publication) this CTA's MMAs no longer read the slot of its own chunk 0
constexpr uint32_t OFF_SENT_DONE = 464;   // (early publication) the peers have received the copies of own chunk 0
constexpr uint32_t OFF_STORE0_DONE = 472; // (early publication) the TMA store of own chunk 0 has finished reading its slot
constexpr uint32_t OFF_UV = 512;       // float u[128], v[128]
// Exchange through global memory.  Both kinds of barrier come in pairs used alternately (publication n, step g: member
// n & 1, g & 1): a waiter can tell the current phase from the one before by parity, no further, and here a signaller may
// be one publication (one step) ahead of a waiter, never two.
constexpr uint32_t OFF_READY = 1536;   // [8][2] slice i's chunks are complete in global memory
constexpr uint32_t OFF_PAIR_FREE = 1664;  // [2 rounds][4 slot pairs][2] THIS CTA's MMAs of the round no longer read slots 2i, 2i+1

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
// element-wise product of two packed bf16 pairs (each product rounded to bf16)
__device__ __forceinline__ uint32_t mul_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }

// ---- packed fp32 pairs (fma.rn.f32x2 and friends: one instruction for two elements, same rounding as the scalar
// forms).  The epilogues are bound by their instruction count, not by the fp32 pipe.
using f32x2 = unsigned long long;
__device__ __forceinline__ f32x2 pk2(float a, float b) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ f32x2 pk2u(uint32_t a, uint32_t b) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ void upk2(f32x2 v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// 2^x and 1/x as single special-function instructions (no range fix-ups: results that would be denormal are flushed
// to zero, which is what erf and the Gaussian density want in their tails; relative error 2^-22 resp. 1 ulp)
__device__ __forceinline__ float ex2_ftz(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_ftz(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// F(x) and F'(x) for G/2 packed pairs (G even); same formulas as act_group below, the polynomial and the products in
// packed form, the special-function evaluations per element.
template <int ACT, int G>
__device__ __forceinline__ void act_group2(const f32x2* x2, f32x2* f2, f32x2* d2);

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


template <int ACT, int G>
__device__ __forceinline__ void act_group2(const f32x2* x2, f32x2* f2, f32x2* d2) {
  constexpr int P = G / 2;
  if constexpr (ACT == RINGRNN_ACT_GELU) {
    float xs[G], t[G], e[G];
#pragma unroll
    for (int i = 0; i < P; ++i) upk2(x2[i], xs[2 * i], xs[2 * i + 1]);
#pragma unroll
    for (int i = 0; i < G; ++i) t[i] = rcp_ftz(fmaf(0.3275911f * 0.70710678118654752f, fabsf(xs[i]), 1.f));
    const f32x2 kexp = pk2(-0.5f * 1.4426950408889634f, -0.5f * 1.4426950408889634f);
#pragma unroll
    for (int i = 0; i < P; ++i) {
      float a, b;
      upk2(mul2(mul2(x2[i], x2[i]), kexp), a, b);
      e[2 * i] = ex2_ftz(a);
      e[2 * i + 1] = ex2_ftz(b);
    }
    // -poly(t) * t, Abramowitz-Stegun 7.1.26 with negated coefficients so that erf = 1 + (that) * e
    const f32x2 c1 = pk2(-1.061405429f, -1.061405429f), c2 = pk2(1.453152027f, 1.453152027f),
                c3 = pk2(-1.421413741f, -1.421413741f), c4 = pk2(0.284496736f, 0.284496736f),
                c5 = pk2(-0.254829592f, -0.254829592f), one = pk2(1.f, 1.f), half = pk2(0.5f, 0.5f),
                kphi = pk2(0.3989422804014327f, 0.3989422804014327f);
#pragma unroll
    for (int i = 0; i < P; ++i) {
      const f32x2 t2 = pk2(t[2 * i], t[2 * i + 1]), e2 = pk2(e[2 * i], e[2 * i + 1]);
      f32x2 poly = fma2(t2, c1, c2);
      poly = fma2(t2, poly, c3);
      poly = fma2(t2, poly, c4);
      poly = fma2(t2, poly, c5);
      poly = mul2(poly, t2);
      float ea, eb;
      upk2(fma2(poly, e2, one), ea, eb);  // erf(|x| / sqrt 2)
      const f32x2 cdf = fma2(half, pk2(copysignf(ea, xs[2 * i]), copysignf(eb, xs[2 * i + 1])), half);
      f2[i] = mul2(x2[i], cdf);
      d2[i] = fma2(mul2(x2[i], kphi), e2, cdf);
    }
  } else {
    float x[G], f[G], d[G];
#pragma unroll
    for (int i = 0; i < P; ++i) upk2(x2[i], x[2 * i], x[2 * i + 1]);
    act_group<ACT, G>(x, f, d);
#pragma unroll
    for (int i = 0; i < P; ++i) {
      f2[i] = pk2(f[2 * i], f[2 * i + 1]);
      d2[i] = pk2(d[2 * i], d[2 * i + 1]);
    }
  }
}

// ---- per-CTA context and the roles both directions share -------------------------------------------------------
template <int NP, bool PAIR>
struct Ctx {
  uint32_t a_base, w_base, bars, tmem_base, stage_base;
  int q;            // neuron slice of this CTA
  int half;         // which 128 of the tile's samples (always 0 in the single shape)
  bool leader;      // issues the MMAs (every CTA in the single shape, the even CTA of a pair otherwise)
  uint32_t rank, leader_rank;
  uint16_t pair_mask;  // cluster ranks of this CTA's MMA unit
  float* uv;
  tc::WaitCtx wctx;
  __device__ __forceinline__ uint32_t peer_rank(int q2) const { return PAIR ? (uint32_t)(2 * q2 + half) : (uint32_t)q2; }
};

// Barrier init, TMEM allocation, decode vectors, cluster-wide start line.
template <int NP, bool PAIR>
__device__ __forceinline__ Ctx<NP, PAIR> setup_cta(uint8_t* smem_raw, const float* dec_u, const float* dec_v, int N,
                                                    int* status) {
  using C_ = Cfg<NP, PAIR>;
  using namespace tc;
  Ctx<NP, PAIR> c;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  c.a_base = base;
  c.w_base = base + C_::A_BYTES;
  c.bars = c.w_base + C_::NS * C_::WT_BYTES;
  c.stage_base = c.bars + C_::AUX;
  uint8_t* bars_gen = gen + C_::A_BYTES + C_::NS * C_::WT_BYTES;
  volatile uint32_t* tmem_slot_p = reinterpret_cast<volatile uint32_t*>(bars_gen + OFF_TMEM_SLOT);
  volatile int* dead = reinterpret_cast<volatile int*>(bars_gen + OFF_DEAD);
  c.uv = reinterpret_cast<float*>(bars_gen + OFF_UV);
  c.wctx = WaitCtx{dead, status};
  c.rank = (C_::CL > 1) ? cluster_ctarank() : 0u;
  c.q = PAIR ? (int)(c.rank >> 1) : (int)c.rank;
  c.half = PAIR ? (int)(c.rank & 1u) : 0;
  c.leader = c.half == 0;
  c.leader_rank = PAIR ? (c.rank & ~1u) : c.rank;
  c.pair_mask = (uint16_t)(3u << (2 * c.q));
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    *dead = 0;
    for (int i = 0; i < 16; ++i) {
      mbar_init(c.bars + OFF_W_FULL + 8 * i, 1);
      mbar_init(c.bars + OFF_W_EMPTY + 8 * i, 1);
    }
    for (int i = 0; i < 8; ++i) {
      mbar_init(c.bars + OFF_A_FULL + 8 * i, 1);
      mbar_init(c.bars + OFF_A_PAIR + 8 * i, 1);
    }
    mbar_init(c.bars + OFF_D_FULL, 1);
    mbar_init(c.bars + OFF_D_FULL + 8, 1);
    mbar_init(c.bars + OFF_D_EMPTY, PAIR ? 16 : 8);  // every epilogue warp of the MMA unit drains each accumulator
    mbar_init(c.bars + OFF_D_EMPTY + 8, PAIR ? 16 : 8);
    mbar_init(c.bars + OFF_MMA_DONE, 1);
    mbar_init(c.bars + OFF_ALL_FREE, C_::C);
    mbar_init(c.bars + OFF_ALL_FREE + 8, C_::C);
    mbar_init(c.bars + OFF_STORE_DONE, 1);
    mbar_init(c.bars + OFF_OWN0_FREE, 1);
    mbar_init(c.bars + OFF_SENT_DONE, C_::C > 1 ? C_::C - 1 : 1);
    mbar_init(c.bars + OFF_STORE0_DONE, 1);
    for (int i = 0; i < 16; ++i) mbar_init(c.bars + OFF_READY + 8 * i, 1);
    for (int i = 0; i < 16; ++i) mbar_init(c.bars + OFF_PAIR_FREE + 8 * i, 1);
    fence_mbar_init();
  }
  if (threadIdx.x < 256) {
    const int i = threadIdx.x & 127, n = c.q * 128 + i;
    const float* src = (threadIdx.x < 128) ? dec_u : dec_v;
    c.uv[threadIdx.x] = (src != nullptr && n < N) ? src[n] : 0.f;
  }
  if (warp == 1) {
    if (PAIR) tmem_alloc_pair(c.bars + OFF_TMEM_SLOT, TMEM_COLS);
    else tmem_alloc(c.bars + OFF_TMEM_SLOT, TMEM_COLS);
  }
  tcgen05_fence_before();
  __syncthreads();
  if (C_::CL > 1) {  // every CTA's barriers exist before any peer signals them
    cluster_arrive();
    cluster_wait();
  }
  tcgen05_fence_after();
  c.tmem_base = *tmem_slot_p;
  return c;
}

template <int NP, bool PAIR>
__device__ __forceinline__ void teardown_cta(const Ctx<NP, PAIR>& c) {
  using namespace tc;
  // abandoned run: the roles stopped wherever they were, so tensor-core work and copies may still be in flight with
  // nobody left to wait for their barriers; give them time to land before the accumulator memory is handed back
  if (*c.wctx.dead) __nanosleep(200000);
  // nobody leaves while a peer may still signal or copy into this CTA
  tcgen05_fence_before();
  __syncthreads();
  if (Cfg<NP, PAIR>::CL > 1) {
    cluster_arrive();
    cluster_wait();
  }
  if ((threadIdx.x >> 5) == 1) {
    if (PAIR) tmem_dealloc_pair(c.tmem_base, TMEM_COLS);
    else tmem_dealloc(c.tmem_base, TMEM_COLS);
  }
}

// Weight stream (one thread per CTA).  Tile order per step: round by round, sub-slice 0 then 1, within a sub-slice
// the `ng` weight groups one after the other, the slots starting at this slice's own.
// SPLIT (early publication): the tiles of the even slots come first, for both sub-slices, then those of the odd
// slots -- the order in which mma_loop consumes them.
template <int NP, bool PAIR, bool GEN = false, bool SPLIT = false>
__device__ __forceinline__ void producer_loop(const Ctx<NP, PAIR>& c, const CUtensorMap* tmW, uint32_t total_steps,
                                              int code, int ng_arg = 1) {
  using C_ = Cfg<NP, PAIR>;
  const int ng = GEN ? ng_arg : 1;  // a compile-time 1 for the two-column kernels
  using namespace tc;
  constexpr int KC = C_::KC, NS = C_::NS, SL = C_::SLOTS, R = C_::ROUNDS;
  tma_prefetch_desc(tmW);
  if (total_steps == 0) return;
  const uint64_t keep = l2_policy_evict_last();
  const int rot = (2 * c.q) % SL;
  auto issue = [&](int st, int s, int grp, int kc) {
    const uint32_t bar = c.bars + OFF_W_FULL + 8 * st;
    const int y = ((c.q * 2 + s) * ng + grp) * C_::RB + c.half * C_::WROWS;
    if (c.leader) mbar_arrive_expect_tx(bar, (PAIR ? 2 : 1) * C_::WT_BYTES);  // a pair's two halves land on one barrier
    if (PAIR) tma_load_2d_pair(c.w_base + st * C_::WT_BYTES, tmW, bar, kc * 64, y);
    else tma_load_2d_hint(c.w_base + st * C_::WT_BYTES, tmW, bar, kc * 64, y, keep);
  };
  if (C_::RESIDENT && ng == 1) {
    for (int s = 0; s < 2; ++s)
      for (int i = 0; i < KC; ++i) issue(s * KC + i, s, 0, (rot + i) % SL);
  } else if constexpr (SPLIT) {
    int st = 0;
    uint32_t lap = 0;
    for (uint32_t g = 0; g < total_steps; ++g)
      for (int half = 0; half < 2; ++half)
        for (int s = 0; s < 2; ++s)
#pragma unroll 1
          for (int i = half; i < SL; i += 2) {
            if (lap > 0 && !mbar_wait(c.bars + OFF_W_EMPTY + 8 * st, (lap - 1) & 1u, c.wctx, code)) return;
            issue(st, s, 0, (rot + i) % SL);
            if (++st == NS) {
              st = 0;
              ++lap;
            }
          }
  } else {
    int st = 0;              // ring stage of the next tile
    uint32_t lap = 0;        // how many times the ring has been filled
    for (uint32_t g = 0; g < total_steps; ++g)
      for (int round = 0; round < R; ++round)
        for (int s = 0; s < 2; ++s)
          for (int grp = 0; grp < ng; ++grp)
#pragma unroll 1
            for (int i = 0; i < SL; ++i) {
              if (lap > 0 && !mbar_wait(c.bars + OFF_W_EMPTY + 8 * st, (lap - 1) & 1u, c.wctx, code))
                return;  // abandoned: issue nothing more
              issue(st, s, grp, round * SL + (rot + i) % SL);
              if (++st == NS) {
                st = 0;
                ++lap;
              }
            }
  }
}

// Every role leaves its loop at the first abandoned wait (a wait that ran out sets the CTA's `dead` flag and the
// global status word): nothing more is issued, and the CTA drains through teardown_cta.
//
// MMA issuer (one thread of the leader CTA).  `stores`: the epilogue publishes this CTA's chunks with a TMA store
// (only looked at with two K rounds, where a peer overwrites the slots of this CTA's own chunks in the other round).
template <int NP, bool PAIR, bool FWD, bool GEN = false>
__device__ __forceinline__ void mma_loop(const Ctx<NP, PAIR>& c, uint32_t total_steps, int T, int code, bool stores,
                                         int ng_arg = 1) {
  using C_ = Cfg<NP, PAIR>;
  const int ng = GEN ? ng_arg : 1;  // a compile-time 1 for the two-column kernels
  using namespace tc;
  constexpr int KC = C_::KC, NS = C_::NS, SL = C_::SLOTS, R = C_::ROUNDS;
  constexpr uint32_t idesc = make_idesc_bf16(PAIR ? 256 : 128, C_::RB, 0, 0);
  constexpr bool EARLY_ANY = !GEN && C_::EARLY && (FWD || NP >= 512);  // as the kernels' own EARLY flags
#ifdef RINGRNN_NO_SPLIT
  constexpr bool SPLIT = false;
#else
  constexpr bool SPLIT = EARLY_ANY;
#endif
  const int rot = (2 * c.q) % SL, rq = (2 * c.q) / SL;
  uint32_t ph = 0, npub = 0;
  int wst = 0;          // ring stage of the next weight tile
  uint32_t wpar = 0;    // parity of that stage's current fill
  int t = 0;            // step within the tile
  const bool pull = C_::PULL && stores;  // every chunk, this CTA's own included, arrives as a TMA load (puller_loop)
  if (!FWD && total_steps > 0)  // reverse: nothing loads the first A operand by TMA, peers push it
    for (int slot = 0; slot < SL; ++slot)
      if (pull || (slot >> 1) != c.q) mbar_arrive_expect_tx(c.bars + OFF_A_FULL + 8 * slot, CHUNK_BYTES);
  auto commit = [&](uint32_t bar) {
    if (PAIR) umma_commit_pair(bar, c.pair_mask);
    else umma_commit(bar);
  };
  for (uint32_t g = 0; g < total_steps; ++g) {
#ifdef RINGRNN_TIMELINE
    long long acc_w = 0, acc_a = 0, acc_p = 0, t0;
#endif
    if constexpr (SPLIT) {
      // Split schedule (with early publication, both directions).  The chunks in the even slots -- chunk 0 of every
      // slice -- are published while the epilogue of sub-slice 1 is still running, so their share of the next step's
      // MMAs, for both accumulators, is issued first and overlaps that epilogue; the odd slots follow once chunk 1 has
      // arrived.  Accumulator s is complete after the odd half of sub-slice s.  (In the reverse kernel this pays only
      // since the scaled copies of delta leave the epilogue as TMA stores: -3 % at N = 512; before, the epilogue of
      // sub-slice 0, no longer hidden behind a whole pass, cost as much as the overlap gained.)
      const int next_t = (t + 1 == T) ? 0 : t + 1;
      const bool next_by_copy = FWD ? next_t != 0 : g + 1 < total_steps;
      for (int half = 0; half < 2; ++half) {
        for (int s = 0; s < 2; ++s) {
          if (half == 0) {
            if (g >= 1 && !mbar_wait(c.bars + OFF_D_EMPTY + 8 * s, (g - 1) & 1u, c.wctx, code + 0)) return;
            if (s == 0) RINGRNN_STAMP(g, 0);
          } else if (s == 0) {
            RINGRNN_STAMP(g, 2);
          }
          tcgen05_fence_after();
#pragma unroll 1
          for (int i = half; i < SL; i += 2) {
            const int slot = (rot + i) % SL;
            if (s == 0) {
#ifdef RINGRNN_TIMELINE
              t0 = clock64();
#endif
              if (!mbar_wait(c.bars + OFF_A_FULL + 8 * slot, ph & 1u, c.wctx, code + 1)) return;
#ifdef RINGRNN_TIMELINE
              acc_a += clock64() - t0;
              if (i == 0) RINGRNN_STAMP(g, 1);
#endif
              if (next_by_copy && (slot >> 1) != c.q) mbar_arrive_expect_tx(c.bars + OFF_A_FULL + 8 * slot, CHUNK_BYTES);
            }
            const int st = wst;
#ifdef RINGRNN_TIMELINE
            t0 = clock64();
#endif
            if (!mbar_wait(c.bars + OFF_W_FULL + 8 * st, wpar, c.wctx, code + 3)) return;
#ifdef RINGRNN_TIMELINE
            acc_w += clock64() - t0;
#endif
            tcgen05_fence_after();
            const uint32_t a_lo = desc_lo(c.a_base + slot * CHUNK_BYTES, 16), b_lo = desc_lo(c.w_base + st * C_::WT_BYTES, 16);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              umma_ss_lo(c.tmem_base + s * 256, a_lo + 2 * ks, b_lo + 2 * ks, idesc, (half > 0 || i > 0 || ks > 0) ? 1u : 0u);
            commit(c.bars + OFF_W_EMPTY + 8 * st);
            if (++wst == NS) {
              wst = 0;
              wpar ^= 1u;
            }
            // nothing issued later reads the slot of this CTA's own chunk 0
            if (half == 0 && s == 1 && i == 0) commit(c.bars + OFF_OWN0_FREE);
          }
          if (half == 1) {
            commit(c.bars + OFF_D_FULL + 8 * s);
            RINGRNN_STAMP(g, s == 0 ? 3 : 4);
          }
        }
      }
      commit(c.bars + OFF_MMA_DONE);
      umma_commit_fanout(c.bars + OFF_ALL_FREE, (uint16_t)((1u << C_::CL) - 1u));
      ++ph;
    } else
#pragma unroll
    for (int round = 0; round < R; ++round, ++ph) {
      // Will the chunks of the next phase arrive as bulk copies from peers (then their byte counts are armed here,
      // right after this phase's wait)?  Forward: the first step of every tile is loaded by TMA instead (armed
      // there); reverse: every phase but the last.
      const int next_round = (round + 1) % R;
      const int next_t = (round + 1 < R) ? t : (t + 1 == T ? 0 : t + 1);
      const bool next_by_copy = FWD ? (next_t != 0) : (ph + 1 < total_steps * (uint32_t)R);
      // A pass = all K chunks of this round into one accumulator: (sub-slice s, weight group grp).  Passes take
      // the two accumulators in turn: pass number n uses accumulator n & 1 for the (n >> 1)-th time.  (With two K
      // rounds there is one group, and both rounds of a sub-slice go into the same accumulator.)
      const bool resident = C_::RESIDENT && ng == 1;
      for (int s = 0; s < 2; ++s) {
        for (int grp = 0; grp < ng; ++grp) {
          const uint32_t pass = (g * 2u + (uint32_t)s) * (uint32_t)ng + (uint32_t)grp;
          const uint32_t acc = pass & 1u;
          if (round == 0) {
            if (pass >= 2 && !mbar_wait<PAIR>(c.bars + OFF_D_EMPTY + 8 * acc, ((pass >> 1) - 1) & 1u, c.wctx, code + 0))
              return;
            if (grp == 0) RINGRNN_STAMP(g, s == 0 ? 0 : 2);
          }
          tcgen05_fence_after();
          // kept rolled: a small loop body keeps this thread within its 40 registers and its instruction footprint
          // small (the unrolled loop measured slower)
#pragma unroll 1
          for (int i = 0; i < SL; ++i) {
            const int slot = (rot + i) % SL;
            if (s == 0 && grp == 0) {
#ifdef RINGRNN_TIMELINE
              t0 = clock64();
#endif
              if (!mbar_wait(c.bars + OFF_A_FULL + 8 * slot, ph & 1u, c.wctx, code + 1)) return;
#ifdef RINGRNN_TIMELINE
              acc_a += clock64() - t0;
              t0 = clock64();
#endif
              if (next_by_copy && (pull || ((next_round * SL + slot) >> 1) != c.q))
                mbar_arrive_expect_tx(c.bars + OFF_A_FULL + 8 * slot, CHUNK_BYTES);
              if (PAIR && !mbar_wait<true>(c.bars + OFF_A_PAIR + 8 * slot, g & 1u, c.wctx, code + 2)) return;
#ifdef RINGRNN_TIMELINE
              acc_p += clock64() - t0;
              if (i == 1 && round == 0) RINGRNN_STAMP(g, 1);
#endif
            }
            int st;
            if (resident) {
              st = s * KC + i;
              if (g == 0 && !mbar_wait(c.bars + OFF_W_FULL + 8 * st, 0, c.wctx, code + 3)) return;
            } else {
              st = wst;
#ifdef RINGRNN_TIMELINE
              t0 = clock64();
#endif
              if (!mbar_wait(c.bars + OFF_W_FULL + 8 * st, wpar, c.wctx, code + 3)) return;
#ifdef RINGRNN_TIMELINE
              acc_w += clock64() - t0;
#endif
            }
            tcgen05_fence_after();
            const uint32_t a_lo = desc_lo(c.a_base + slot * CHUNK_BYTES, 16), b_lo = desc_lo(c.w_base + st * C_::WT_BYTES, 16);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
              const uint32_t accum = (round > 0 || i > 0 || ks > 0) ? 1u : 0u;
              if (PAIR) umma_ss_pair_lo(c.tmem_base + acc * 256, a_lo + 2 * ks, b_lo + 2 * ks, idesc, accum);
              else umma_ss_lo(c.tmem_base + acc * 256, a_lo + 2 * ks, b_lo + 2 * ks, idesc, accum);
            }
            if (!resident) {
              commit(c.bars + OFF_W_EMPTY + 8 * st);
              if (++wst == NS) {
                wst = 0;
                wpar ^= 1u;
              }
            }
            // exchange through global memory: the second pass is the last reader of a slot; a pair of slots (one
            // slice's two chunks) is handed to its puller as soon as the pass is past it
            if (C_::PULL && s == 1 && (slot & 1))
              commit(c.bars + OFF_PAIR_FREE + 64 * round + 16 * (slot >> 1) + 8 * (g & 1u));
            // early publication: the passes start at this CTA's own chunks, so after the first tile of the last pass
            // nothing issued later reads the slot of own chunk 0: the epilogue may overwrite it once these complete
            if (EARLY_ANY && s == 1 && grp == ng - 1 && i == 0) commit(c.bars + OFF_OWN0_FREE);
          }
          if (round == R - 1) {
            commit(c.bars + OFF_D_FULL + 8 * acc);
            if (grp == ng - 1) RINGRNN_STAMP(g, s == 0 ? 3 : 4);
          }
        }
      }
      if (R > 1 && round == rq && stores && !pull && (!FWD || t != 0)) {
        // this CTA's own chunks sit in slots a peer fills in the next phase: the TMA store that also reads them
        // must be through before "free" goes out
        if (!mbar_wait(c.bars + OFF_STORE_DONE, npub & 1u, c.wctx, code + 4)) return;
        ++npub;
      }
      commit(c.bars + OFF_MMA_DONE);
      // "this MMA unit no longer reads the A buffer of this round", straight to every CTA of the cluster
      const uint32_t free_bar = c.bars + OFF_ALL_FREE + 8 * round;
      if (PAIR) umma_commit_pair(free_bar, (uint16_t)((1u << C_::CL) - 1u));
      else if (C_::CL > 1) umma_commit_fanout(free_bar, (uint16_t)((1u << C_::CL) - 1u));
      else umma_commit(free_bar);
    }
    t = (t + 1 == T) ? 0 : t + 1;
#ifdef RINGRNN_TIMELINE
    RINGRNN_STAMP_VAL(g, 13, acc_w);
    RINGRNN_STAMP_VAL(g, 14, acc_a);
    RINGRNN_STAMP_VAL(g, 15, acc_p);
#endif
  }
}

// Relay (one thread per CTA): follows every phase of mma_done, so it knows when the A buffer may take new contents:
// `tile_start(tile_index, round)` runs before each round of the first step of each tile (forward: TMA load of that
// round's chunks of the initial state into this CTA's A buffer).  The odd CTA of a pair also forwards "chunk kc is
// complete here" to its leader and arms its own incoming copies.
template <int NP, bool PAIR, bool FWD, bool ACKS = false, class TileStart>
__device__ __forceinline__ void relay_loop(const Ctx<NP, PAIR>& c, uint32_t total_steps, int T, int code,
                                           TileStart tile_start) {
  using C_ = Cfg<NP, PAIR>;
  using namespace tc;
  constexpr int KC = C_::KC, R = C_::ROUNDS;
  if (PAIR && !c.leader && !FWD && total_steps > 0)
    for (int kc = 0; kc < KC; ++kc)
      if ((kc >> 1) != c.q) mbar_arrive_expect_tx(c.bars + OFF_A_FULL + 8 * kc, CHUNK_BYTES);
  uint32_t ph = 0;
  int t = 0, it = 0;
  for (uint32_t g = 0; g < total_steps; ++g) {
    for (int round = 0; round < R; ++round, ++ph) {
      if (t == 0) tile_start(it, round);
      if (ACKS && (!FWD || t != 0)) {  // (ACKS: the kernel's own early-publication flag)  // (early_acks: the kernel's own EARLY flag)
        // early publication: chunk 0 of every peer reached this CTA as a copy out of the peer's own A slot; tell the
        // peer once it has landed, so that the peer knows when it may overwrite that slot again
        for (int q2 = 0; q2 < C_::C; ++q2)
          if (q2 != c.q) {
            if (!mbar_wait(c.bars + OFF_A_FULL + 8 * (2 * q2), ph & 1u, c.wctx, code + 2)) return;
            mbar_arrive_cluster(c.bars + OFF_SENT_DONE, (uint32_t)q2);
          }
      }
      if (PAIR && !c.leader) {
        const bool next_by_copy = FWD ? (t + 1 < T) : (g + 1 < total_steps);
        for (int i = 0; i < KC; ++i) {
          const int kc = (2 * c.q + i) % KC;
          if (!mbar_wait(c.bars + OFF_A_FULL + 8 * kc, g & 1u, c.wctx, code + 0)) return;
          if ((kc >> 1) != c.q && next_by_copy) mbar_arrive_expect_tx(c.bars + OFF_A_FULL + 8 * kc, CHUNK_BYTES);
          mbar_arrive_cluster(c.bars + OFF_A_PAIR + 8 * kc, c.leader_rank);
        }
      }
      if (!mbar_wait(c.bars + OFF_MMA_DONE, ph & 1u, c.wctx, code + 1)) return;
    }
    if (++t == T) {
      t = 0;
      ++it;
    }
  }
}

// Which phases of the per-round "free" barriers an epilogue thread has consumed.  Every thread consumes every phase
// of every round's barrier, in order and never twice (a parity wait on a barrier that has moved on by two phases
// would never return).
template <int NP, bool PAIR>
struct FreePhases {
  static constexpr int R = Cfg<NP, PAIR>::ROUNDS;
  uint32_t cnt[R];
  __device__ __forceinline__ FreePhases() {
#pragma unroll
    for (int r = 0; r < R; ++r) cnt[r] = 0;
  }
  __device__ __forceinline__ void upto(const Ctx<NP, PAIR>& c, int r, uint32_t n, int code) {
    while (cnt[r] < n) {
      tc::mbar_wait<true>(c.bars + OFF_ALL_FREE + 8 * r, cnt[r] & 1u, c.wctx, code);
      ++cnt[r];
    }
  }
  // Once an accumulator of step g is complete, every round of step g but the last is over in the whole cluster
  // (the chunks of a round are only published after the previous round's "free").
  __device__ __forceinline__ void early(const Ctx<NP, PAIR>& c, uint32_t g, int code) {
#pragma unroll
    for (int r = 0; r + 1 < R; ++r) upto(c, r, g + 1, code);
  }
  // all rounds of steps <= g
  __device__ __forceinline__ void end_of_step(const Ctx<NP, PAIR>& c, uint32_t g, int code) {
#pragma unroll
    for (int r = 0; r < R; ++r) upto(c, r, g + 1, code);
  }
  // everything that precedes round rq of step gt: the slots of this CTA's own chunks may be rewritten
  __device__ __forceinline__ void before_publish(const Ctx<NP, PAIR>& c, uint32_t gt, int rq, int code) {
#pragma unroll
    for (int r = 0; r < R; ++r) upto(c, r, gt + (r < rq ? 1u : 0u), code);
  }
};

// Epilogue helpers ------------------------------------------------------------------------------------------------
// "this warp has read accumulator s of step g": to the leader's barrier (remote for the odd CTA of a pair)
template <int NP, bool PAIR>
__device__ __forceinline__ void release_accumulator(const Ctx<NP, PAIR>& c, int s, int lane) {
  using namespace tc;
  tcgen05_fence_before();
  __syncwarp();
  if (lane == 0) {
    if (PAIR && !c.leader) mbar_arrive_cluster(c.bars + OFF_D_EMPTY + 8 * s, c.leader_rank);
    else mbar_arrive(c.bars + OFF_D_EMPTY + 8 * s);
  }
}

// Writes this thread's 2 x 32 bf16 values (packed[s*16 + ..], columns [32h, 32h+32) of sub-slice s) into the CTA's own
// two chunks of the A buffer, then (one thread) marks them complete locally, copies them to the CTAs that hold the
// same samples for the other slices and, if `tm_store` is given, stores them with TMA to rows [y, y+128),
// columns [x0, x0+128) of a row-major bf16 tensor (the saved state, or delta for the weight-gradient GEMM): the
// chunks are already in the layout a 128-byte-swizzled TMA box expects, so this costs no load/store instructions.
// All 256 epilogue threads must call it.  Returns true, to all of them alike, if a wait of this CTA was abandoned
// (nothing is copied then): the one place where the epilogue threads may leave their loops together.
template <int NP, bool PAIR>
__device__ __forceinline__ bool publish_chunks(const Ctx<NP, PAIR>& c, const uint32_t* packed, int row, int h, int warp,
                                               int lane, const CUtensorMap* tm_store, int x0, int y) {
  using C_ = Cfg<NP, PAIR>;
  using namespace tc;
  // the TMA stores of the previous call have finished reading the chunks (the issuing thread waits before arriving)
  if (tm_store != nullptr) {
    if (warp == 4 && lane == 0) bulk_wait_read<0>();
    named_bar_sync(2, 256);
  }
#pragma unroll
  for (int s = 0; s < 2; ++s) {
    const uint32_t tile_addr = c.a_base + ((2 * c.q + s) % C_::SLOTS) * CHUNK_BYTES;
#pragma unroll
    for (int v = 0; v < 4; ++v) {
      const uint32_t unit = (uint32_t)(4 * h + v);
      const uint32_t addr = tile_addr + row * 128 + ((unit ^ ((uint32_t)row & 7u)) << 4);
      asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(packed[s * 16 + 4 * v]),
                   "r"(packed[s * 16 + 4 * v + 1]), "r"(packed[s * 16 + 4 * v + 2]), "r"(packed[s * 16 + 4 * v + 3])
                   : "memory");
    }
  }
  fence_proxy_async_smem();
  const bool stop = named_bar_or(1, 256, *c.wctx.dead != 0);
  if (warp == 4 && lane == 0 && !stop) {
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const int slot = (2 * c.q + s) % C_::SLOTS;
      const uint32_t tile_addr = c.a_base + slot * CHUNK_BYTES;
      mbar_arrive(c.bars + OFF_A_FULL + 8 * slot);
      for (int q2 = 0; q2 < C_::C; ++q2)
        if (q2 != c.q) dsmem_bulk_copy(tile_addr, tile_addr, CHUNK_BYTES, c.bars + OFF_A_FULL + 8 * slot, c.peer_rank(q2));
    }
    if (tm_store != nullptr) {
#pragma unroll
      for (int s = 0; s < 2; ++s)
        tma_store_2d(tm_store, c.a_base + ((2 * c.q + s) % C_::SLOTS) * CHUNK_BYTES, x0 + 64 * s, y);
      bulk_commit();
      if (C_::ROUNDS > 1) {  // a peer refills these slots in the next phase: tell the MMA thread when the store has read them
        bulk_wait_read<0>();
        mbar_arrive(c.bars + OFF_STORE_DONE);
      }
    }
  }
  return stop;
}

// Early publication, forward kernel (Cfg::EARLY).  The two chunks of a step are published separately:
//   write_chunk   : every epilogue thread stores its 16 packed words of sub-slice s into the CTA's own A slot
//   send_chunk    : (chunk 1) after a barrier over the 256 epilogue threads, one of them marks the slot complete locally,
//                   copies it to the peers and (training) stores it to the saved state with TMA.  Returns `stop` as
//                   publish_chunks does.
//   sender_loop   : (chunk 0) the same hand-over done by a thread of its own (warp 3), so that no epilogue thread waits
//                   for it: the epilogue threads arrive at named barrier 3 once their part of chunk 0 is in the slot
//                   and go on with sub-slice 1; the sender waits there, then for "every CTA of the cluster has finished
//                   this step's MMAs" (the peers' slots are free), and sends.
template <int NP, bool PAIR>
__device__ __forceinline__ void write_chunk(const Ctx<NP, PAIR>& c, const uint32_t* packed16, int s, int row, int h) {
  using C_ = Cfg<NP, PAIR>;
  const uint32_t tile_addr = c.a_base + ((2 * c.q + s) % C_::SLOTS) * CHUNK_BYTES;
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const uint32_t unit = (uint32_t)(4 * h + v);
    const uint32_t addr = tile_addr + row * 128 + ((unit ^ ((uint32_t)row & 7u)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(packed16[4 * v]), "r"(packed16[4 * v + 1]),
                 "r"(packed16[4 * v + 2]), "r"(packed16[4 * v + 3])
                 : "memory");
  }
  tc::fence_proxy_async_smem();
}
template <int NP, bool PAIR>
__device__ __forceinline__ bool send_chunk(const Ctx<NP, PAIR>& c, int s, int warp, int lane, uint32_t bar_id,
                                           const CUtensorMap* tm_store, int x0, int y) {
  using C_ = Cfg<NP, PAIR>;
  using namespace tc;
  const bool stop = named_bar_or(bar_id, 256, *c.wctx.dead != 0);
  if (warp == 4 && lane == 0 && !stop) {
    const int slot = (2 * c.q + s) % C_::SLOTS;
    const uint32_t tile_addr = c.a_base + slot * CHUNK_BYTES;
    mbar_arrive(c.bars + OFF_A_FULL + 8 * slot);
    for (int q2 = 0; q2 < C_::C; ++q2)
      if (q2 != c.q) dsmem_bulk_copy(tile_addr, tile_addr, CHUNK_BYTES, c.bars + OFF_A_FULL + 8 * slot, c.peer_rank(q2));
    if (tm_store != nullptr) {
      tma_store_2d(tm_store, tile_addr, x0 + 64 * s, y);
      bulk_commit();
    }
  }
  return stop;
}

constexpr uint32_t SENDER_BAR = 3, SENDER_BAR_THREADS = 288;  // 8 epilogue warps arrive, warp 3 waits

// All 32 threads of warp 3 run this (named barriers are warp-wide); lane 0 does the work.
// Forward: step t of a tile publishes r_t, row block t+1 of the saved state, unless it is the tile's last step.
// Reverse: a tile first publishes delta_{T-1} (before its first step), then step t publishes delta_{t-1}, row block t-1
// of DL, unless t = 0.  Either way the thread consumes the "every CTA has finished this step's MMAs" phase of every
// step, so a send that follows it finds the peers' slots free.
template <int NP, bool PAIR, bool FWD = true>
__device__ __forceinline__ void sender_loop(const Ctx<NP, PAIR>& c, uint32_t total_steps, int T, int code,
                                            const CUtensorMap* tm_store, int BP, int cluster_id, int n_clusters) {
  using C_ = Cfg<NP, PAIR>;
  using namespace tc;
  const int lane = threadIdx.x & 31;
  const int slot = (2 * c.q) % C_::SLOTS;
  const uint32_t tile_addr = c.a_base + slot * CHUNK_BYTES;
  if (tm_store != nullptr && lane == 0) tma_prefetch_desc(tm_store);
  auto send = [&](int row_block, int tile) {
    mbar_arrive(c.bars + OFF_A_FULL + 8 * slot);
    for (int q2 = 0; q2 < C_::C; ++q2)
      if (q2 != c.q) dsmem_bulk_copy(tile_addr, tile_addr, CHUNK_BYTES, c.bars + OFF_A_FULL + 8 * slot, c.peer_rank(q2));
    if (tm_store != nullptr) {
      tma_store_2d(tm_store, tile_addr, c.q * 128, row_block * BP + tile * C_::TILE_ROWS + c.half * 128);
      bulk_commit();
      bulk_wait_read<0>();
    }
    mbar_arrive(c.bars + OFF_STORE0_DONE);
  };
  int t = 0, it = 0;  // step within the tile (counted upwards in both directions), tile of this cluster
  for (uint32_t g = 0; g < total_steps; ++g) {
    const int tile = cluster_id + it * n_clusters;
    if (!FWD && t == 0) {  // reverse: the first delta of the tile, before its first step
      named_bar_sync(SENDER_BAR, SENDER_BAR_THREADS);
      bool ok0 = *c.wctx.dead == 0;
      if (lane == 0 && ok0) send(T - 1, tile);
      if (!ok0) return;
    }
    const bool sends = t + 1 < T;
    if (sends) named_bar_sync(SENDER_BAR, SENDER_BAR_THREADS);  // chunk 0 of this step is complete in the slot
    bool ok = *c.wctx.dead == 0;
    if (lane == 0 && ok) {
      // one phase per step, consumed every step: every CTA of the cluster has finished this step's MMAs
      ok = mbar_wait<true>(c.bars + OFF_ALL_FREE, g & 1u, c.wctx, code);
      if (ok && sends) send(FWD ? t + 1 : T - 2 - t, tile);
    }
    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
    if (!ok) return;  // abandoned: the epilogue threads leave at their next publication and release this barrier
    if (++t == T) {
      t = 0;
      ++it;
    }
  }
  if (tm_store != nullptr && lane == 0) bulk_wait_all<0>();
}

// Exchange through global memory (Cfg::PULL).
// Publisher: all 256 epilogue threads call publish_global with their 2 x 16 packed words; `row_ptr` points at the
// thread's sample row, first column of the CTA's 128-column block, in the tensor that keeps the published values
// (saved state, or the delta block of DL), whose rows are `row_stride` elements apart; `n_pub` counts this CTA's
// publications.  Returns `stop` as publish_chunks does.
template <bool STREAM = true>
__device__ __forceinline__ void store_rows_via_smem(uint32_t stage, int lane, const uint32_t* w16, uint8_t* dst_row0,
                                                    size_t row_stride_bytes);

template <int NP, bool PAIR>
__device__ __forceinline__ bool publish_global(const Ctx<NP, PAIR>& c, const uint32_t* packed, int h, int warp, int lane,
                                               __nv_bfloat16* row_ptr, size_t row_stride, uint32_t n_pub) {
  using C_ = Cfg<NP, PAIR>;
  using namespace tc;
  // through the warp's transposition buffer: a store instruction then covers 8 rows x 64 bytes instead of 32 rows x
  // 16 bytes (the direct form kept the load/store unit busy for 1.3-2.8 K cycles per publication)
  const uint32_t stage = c.stage_base + (uint32_t)(warp - 4) * 2048u;
  if (lane == 0) bulk_wait_read<0>();  // (reverse kernel) a TMA store of the scaled copies may still be reading the buffer
  __syncwarp();
#pragma unroll
  for (int s = 0; s < 2; ++s)
    store_rows_via_smem<false>(stage, lane, packed + 16 * s,
                               reinterpret_cast<uint8_t*>(row_ptr - (size_t)lane * row_stride + 64 * s + 32 * h), row_stride * 2);
  // The barrier orders the 256 threads' stores before the one fence below, whose release is cumulative over them (the
  // pattern of a grid-wide barrier: sync the block, then one thread fences and signals).
  const bool stop = named_bar_or(1, 256, *c.wctx.dead != 0);
  if (warp == 4 && !stop) {
    if (lane == 0) {
      __threadfence();          // the release for all the signals below
      fence_proxy_async_all();  // the readers are TMA loads
    }
    __syncwarp();  // the fence precedes the other lanes' signals
    if (lane < C_::C)  // one signal per lane: in turn they took 1 K cycles
      mbar_arrive_cluster_relaxed(c.bars + OFF_READY + 16 * c.q + 8 * (n_pub & 1u), c.peer_rank(lane));
  }
  return stop;
}

// Consumer: all 32 threads of warp 3 run this; lane i < C fetches what slice i publishes (this CTA's own slice too).
// It waits for this CTA's MMAs of the phase before the one the chunks belong to (they read what the slots hold
// now), then for that slice's flag, then loads the two chunks with TMA; the loads complete the barriers the MMA thread
// has armed.  `tmX` maps the tensor the publishers write; a step's operand is row block t (forward: the state
// before step t; the first one of a tile is loaded by the relay thread; `ring`: block 1 + (t & 1) of a three-block
// buffer when no state is saved) resp. T-1-t (reverse: delta of that step).
// How far a flag can run ahead of its reader: slice i's publication n+2 follows MMAs that needed this CTA's publication
// n+1, which follows this CTA's MMAs on the chunks of publication n -- so at most one ahead, which the paired barriers
// tell apart.  Likewise the MMA thread is at most one step ahead of a lane (a forward tile's first step needs no lane).
// Forward with T = 1 publishes nothing: the caller does not start this loop then.
template <int NP, bool PAIR, bool FWD>
__device__ __forceinline__ void puller_loop(const Ctx<NP, PAIR>& c, uint32_t total_steps, int T, int code,
                                            const CUtensorMap* tmX, int BP, int cluster_id, int n_clusters,
                                            bool ring = false) {
  using C_ = Cfg<NP, PAIR>;
  using namespace tc;
  constexpr int R = C_::ROUNDS;
  const int q2 = threadIdx.x & 31;
  if (q2 >= C_::C) return;
  const int round = (2 * q2) / C_::SLOTS;  // the K round slice q2's chunks belong to
  static_assert(R == 2, "the slot hand-over below is written for two K rounds");
  uint32_t n = 0;  // publications of slice q2 fetched so far
  int t = 0, it = 0;
  for (uint32_t g = 0; g < total_steps; ++g) {
    // The two slots hold chunks of the phase before: round 0 of this step (for a slice of round 1) or round 1 of the
    // previous step (for a slice of round 0).  One phase of that barrier per step, consumed every step, whether a
    // load follows or not, so that the parity never slips.
    const uint32_t pair_free = c.bars + OFF_PAIR_FREE + 16 * (q2 % (C_::SLOTS / 2));
    if (round == 1) {
      if (!mbar_wait(pair_free + 8 * (g & 1u), (g >> 1) & 1u, c.wctx, code + 1)) return;
    } else if (g > 0) {
      if (!mbar_wait(pair_free + 64 + 8 * ((g - 1) & 1u), ((g - 1) >> 1) & 1u, c.wctx, code + 1)) return;
    }
    if (!FWD || t != 0) {
      if (!mbar_wait<true>(c.bars + OFF_READY + 16 * q2 + 8 * (n & 1u), (n >> 1) & 1u, c.wctx, code)) return;
      ++n;
      fence_proxy_async_all();
      const int tile = cluster_id + it * n_clusters;
      const int rb = FWD ? (ring ? 1 + (t & 1) : t) : T - 1 - t;
      const int y = rb * BP + tile * C_::TILE_ROWS + c.half * 128;
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        const int slot = (2 * q2 + s) % C_::SLOTS;
        tma_load_2d(c.a_base + slot * CHUNK_BYTES, tmX, c.bars + OFF_A_FULL + 8 * slot, q2 * 128 + 64 * s, y);
      }
    }
    if (++t == T) {
      t = 0;
      ++it;
    }
  }
}

// ---- epilogue global-memory traffic ---------------------------------------------------------------------------
// A thread owns one sample (row) and 32 consecutive neurons: 64 bytes of a bf16 row.  Writing or reading that
// directly makes every warp instruction touch 32 different cache lines.  Two remedies:
//  * tensors only these kernels read (the activation-derivative history) live in a BLOCKED layout: one 2 KB block per
//    (32 samples, 32 neurons), 16-byte piece v of sample r at byte v*512 + r*16, so a warp instruction is one
//    contiguous 512 bytes;
//  * row-major tensors the GEMM reads by TMA go through a per-warp 2 KB transposition buffer in shared memory, after
//    which each warp instruction covers 8 rows x 64 bytes.
__device__ __forceinline__ size_t blocked_offset(int t, int b, int n32, int BP, int NP) {
  // element offset of the block that holds sample b, neurons [32*n32, 32*n32+32) at step t
  return (((size_t)t * (BP >> 5) + (b >> 5)) * (NP >> 5) + n32) * 1024;
}
__device__ __forceinline__ void store_blocked(__nv_bfloat16* base, int lane, const uint32_t* w16) {
#pragma unroll
  for (int v = 0; v < 4; ++v)
    tc::st_cs_v4(reinterpret_cast<uint8_t*>(base) + v * 512 + lane * 16, w16[4 * v], w16[4 * v + 1], w16[4 * v + 2],
                 w16[4 * v + 3]);
}
__device__ __forceinline__ void load_blocked(const __nv_bfloat16* base, int lane, uint4* out4) {
#pragma unroll
  for (int v = 0; v < 4; ++v) out4[v] = tc::ld_cs_v4(reinterpret_cast<const uint8_t*>(base) + v * 512 + lane * 16);
}
// The warp's 32 rows x 64 bytes (lane = row, w16 = its 16 words) to row-major global memory: `dst_row0` points at
// row 0 of the warp's block, consecutive rows are `row_stride_bytes` apart; `stage` is the warp's 2 KB buffer.
template <bool STREAM>
__device__ __forceinline__ void store_rows_via_smem(uint32_t stage, int lane, const uint32_t* w16, uint8_t* dst_row0,
                                                    size_t row_stride_bytes) {
  const uint32_t sw = ((uint32_t)lane >> 1) & 3u;
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const uint32_t addr = stage + lane * 64 + (((uint32_t)v ^ sw) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w16[4 * v]), "r"(w16[4 * v + 1]),
                 "r"(w16[4 * v + 2]), "r"(w16[4 * v + 3])
                 : "memory");
  }
  __syncwarp();
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int r = 8 * k + (lane >> 2);
    const uint32_t piece = (uint32_t)lane & 3u;
    const uint32_t addr = stage + r * 64 + ((piece ^ (((uint32_t)r >> 1) & 3u)) << 4);
    uint32_t a, b, c2, d;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c2), "=r"(d) : "r"(addr));
    uint8_t* dst = dst_row0 + (size_t)r * row_stride_bytes + piece * 16;
    if (STREAM) tc::st_cs_v4(dst, a, b, c2, d);
    else *reinterpret_cast<uint4*>(dst) = make_uint4(a, b, c2, d);
  }
  __syncwarp();
}

// The same 32 rows x 64 bytes as ONE TMA store out of the warp's buffer (a [32 rows x 32 columns] box in the 64-byte
// swizzle, which is the arrangement the buffer is written in): no shared-memory loads and no global store instructions
// in the epilogue threads.  `tm` maps the row-major destination with that box; (x, y) = first column, first row.
// Lane 0 issues the store and, before the buffer is written again, waits until the previous one has read it; at the
// end of the kernel it must wait for its stores to complete (bulk_wait_all).
__device__ __forceinline__ void store_rows_via_tma(uint32_t stage, int lane, const uint32_t* w16, const CUtensorMap* tm,
                                                   int x, int y) {
  if (lane == 0) tc::bulk_wait_read<0>();
  __syncwarp();
  const uint32_t sw = ((uint32_t)lane >> 1) & 3u;
#pragma unroll
  for (int v = 0; v < 4; ++v) {
    const uint32_t addr = stage + lane * 64 + (((uint32_t)v ^ sw) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w16[4 * v]), "r"(w16[4 * v + 1]),
                 "r"(w16[4 * v + 2]), "r"(w16[4 * v + 3])
                 : "memory");
  }
  tc::fence_proxy_async_smem();
  __syncwarp();
  if (lane == 0) {
    tc::tma_store_2d(tm, stage, x, y);
    tc::bulk_commit();
  }
}

}  // namespace tcr

// How many clusters to launch: one per tile, but never more than can be resident at once (a second wave would
// double the time of these persistent kernels; with fewer clusters the tiles are taken round-robin instead).
inline int clusters_to_launch(const void* kernel, cudaLaunchConfig_t* cfg, int cluster_size, int n_tiles) {
  int max_active = 0;
  cfg->gridDim = dim3((unsigned)(cluster_size * n_tiles), 1, 1);
  if (cudaOccupancyMaxActiveClusters(&max_active, kernel, cfg) != cudaSuccess || max_active < 1) {
    (void)cudaGetLastError();
    max_active = 148 / cluster_size;
  }
  if (getenv("RINGRNN_DEBUG") != nullptr)
    fprintf(stderr, "[ringrnn] cluster size %d: %d tiles, at most %d clusters resident\n", cluster_size, n_tiles, max_active);
  return n_tiles < max_active ? n_tiles : max_active;
}

}  // namespace ringrnn
