// fp32 mode of the ring-attractor operator: persistent CUDA-core kernels.
//
// One CTA owns BT samples for the whole sequence and keeps their state in shared memory, so the
// T timesteps run inside one launch (the reference launches one kernel per step,
// cpp/kernels/fwd_fp32.cuh:252-262, and five per step in backward,
// cpp/kernels/bwd_mixed_precision_aggressive.cuh:563-672).  The per-sample effective weight matrix
// of the reference is never formed:  re = J0*sum_j r + J1*(r Wo^T) + sum_k A_k*(r Wa_k^T).
// Weight gradients are not accumulated inside the sequential loop: the reverse-time kernel writes
// delta_t = alpha*F'(re_t)*g_t, and a batched-over-(t,b) product kernel forms
// dW_m = sum_{t,b} s_m[t,b] * delta_t[b,:]^T r_{t-1}[b,:] with a fixed split of the (t,b) range and a
// fixed-order reduction of the partial sums, so results are bit-reproducible (no atomics).
#include "ringrnn_common.cuh"

namespace ringrnn {

namespace {

constexpr int FT = 256;      // threads per CTA in the recurrent kernels

// WT[m][j][i] = W_m[i][j], m = 0 -> Wo, m >= 1 -> Wa[cols[m-1]]
__global__ void transpose_weights_kernel(DevProblem p, float* __restrict__ WT) {
  __shared__ float tile[32][33];
  const int m = blockIdx.z;
  const float* W = (m == 0) ? p.Wo : p.Wa + (size_t)active_col(p, m - 1) * p.N * p.N;
  float* O = WT + (size_t)m * p.N * p.N;
  const int j0 = blockIdx.x * 32, i0 = blockIdx.y * 32;
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int i = i0 + r, j = j0 + threadIdx.x;
    tile[r][threadIdx.x] = (i < p.N && j < p.N) ? W[(size_t)i * p.N + j] : 0.f;
  }
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += blockDim.y) {
    const int j = j0 + r, i = i0 + threadIdx.x;
    if (i < p.N && j < p.N) O[(size_t)j * p.N + i] = tile[threadIdx.x][r];
  }
}

// Sums over neurons of the state held as s[n][BT]: up to four weighted sums per sample.
// out[b*4 + {0,1,2,3}] = { sum s, sum s*u, sum s*v, sum |s| }.  Fixed summation order.
template <int BT>
__device__ __forceinline__ void state_stats(const float* __restrict__ s, int N, const float* __restrict__ u,
                                            const float* __restrict__ v, float* red, float* out) {
  constexpr int G = FT / BT;
  const int b = threadIdx.x % BT, g = threadIdx.x / BT;
  float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
  for (int n = g; n < N; n += G) {
    const float x = s[n * BT + b];
    a0 += x;
    a3 += fabsf(x);
    if (u != nullptr) {
      a1 += x * __ldg(u + n);
      a2 += x * __ldg(v + n);
    }
  }
  float* slot = red + (g * BT + b) * 4;
  slot[0] = a0; slot[1] = a1; slot[2] = a2; slot[3] = a3;
  __syncthreads();
  if (threadIdx.x < BT * 4) {
    const int bb = threadIdx.x / 4, c = threadIdx.x % 4;
    float acc = 0.f;
    for (int gg = 0; gg < G; ++gg) acc += red[(gg * BT + bb) * 4 + c];
    out[bb * 4 + c] = acc;
  }
  __syncthreads();
}

template <int BT>
__device__ __forceinline__ void load_scales(const DevProblem& p, int b0, int t, float* sc) {
  for (int idx = threadIdx.x; idx < p.n_mat * BT; idx += FT) {
    const int m = idx / BT, b = idx % BT;
    float v = p.J1;
    if (m > 0) v = (b0 + b < p.B) ? __ldg(p.A + ((size_t)(b0 + b) * p.T + t) * p.a_dim + active_col(p, m - 1)) : 0.f;
    sc[idx] = v;
  }
}

// re[b] for one neuron i:  J0*S[b] + sum_m sc[m][b] * sum_j r[j][b] * WT[m][j][i]
template <int BT>
__device__ __forceinline__ void contract_row(const DevProblem& p, const float* __restrict__ W, size_t mat_stride,
                                             size_t k_stride, const float* __restrict__ st, const float* sc,
                                             float* re) {
  for (int m = 0; m < p.n_mat; ++m) {
    float tmp[BT];
#pragma unroll
    for (int b = 0; b < BT; ++b) tmp[b] = 0.f;
    const float* w = W + (size_t)m * mat_stride;
#pragma unroll 4
    for (int k = 0; k < p.N; ++k) {
      const float wv = __ldg(w + (size_t)k * k_stride);
      const float4* s4 = reinterpret_cast<const float4*>(st + k * BT);
#pragma unroll
      for (int b4 = 0; b4 < BT / 4; ++b4) {
        const float4 s = s4[b4];
        tmp[b4 * 4 + 0] = fmaf(s.x, wv, tmp[b4 * 4 + 0]);
        tmp[b4 * 4 + 1] = fmaf(s.y, wv, tmp[b4 * 4 + 1]);
        tmp[b4 * 4 + 2] = fmaf(s.z, wv, tmp[b4 * 4 + 2]);
        tmp[b4 * 4 + 3] = fmaf(s.w, wv, tmp[b4 * 4 + 3]);
      }
    }
#pragma unroll
    for (int b = 0; b < BT; ++b) re[b] = fmaf(sc[m * BT + b], tmp[b], re[b]);
  }
}

struct Fp32FwdOut {
  float* hist;         // [T,B,N] or nullptr
  float* dec_x;        // [B,T] or nullptr
  float* dec_y;
  float* dec_ta;
  const float* dec_u;  // [N]
  const float* dec_v;
  float* final_state;  // [B,N] or nullptr
};

template <int ACT, int BT>
__global__ void __launch_bounds__(FT) fwd_fp32_kernel(DevProblem p, const float* __restrict__ WT, Fp32FwdOut o) {
  extern __shared__ __align__(16) float smem[];
  const int N = p.N;
  float* cur = smem;                         // [N][BT] state r_{t-1}
  float* nxt = cur + (size_t)N * BT;         // [N][BT] state r_t
  float* sc = nxt + (size_t)N * BT;          // [n_mat][BT]
  float* red = sc + p.n_mat * BT;            // [FT/BT][BT][4]
  float* stats = red + (FT / BT) * BT * 4;   // [BT][4]
  const int b0 = blockIdx.x * BT;
  const bool want_dec = (o.dec_x != nullptr) || (o.dec_y != nullptr) || (o.dec_ta != nullptr);

  for (int idx = threadIdx.x; idx < N * BT; idx += FT) {
    const int b = idx / N, j = idx % N;
    cur[j * BT + b] = (b0 + b < p.B) ? p.r_init[(size_t)(b0 + b) * N + j] : 0.f;
  }
  __syncthreads();

  for (int t = 0; t <= p.T; ++t) {
    // statistics of r_{t-1} (the row sum feeds step t; the decode belongs to time t-1)
    state_stats<BT>(cur, N, want_dec ? o.dec_u : nullptr, o.dec_v, red, stats);
    if (t > 0 && want_dec && threadIdx.x < BT && b0 + threadIdx.x < p.B) {
      const size_t at = (size_t)(b0 + threadIdx.x) * p.T + (t - 1);
      if (o.dec_x) o.dec_x[at] = stats[threadIdx.x * 4 + 1];
      if (o.dec_y) o.dec_y[at] = stats[threadIdx.x * 4 + 2];
      if (o.dec_ta) o.dec_ta[at] = stats[threadIdx.x * 4 + 3];
    }
    if (t == p.T) break;
    load_scales<BT>(p, b0, t, sc);
    __syncthreads();
    for (int i = threadIdx.x; i < N; i += FT) {
      float re[BT];
#pragma unroll
      for (int b = 0; b < BT; ++b) re[b] = p.J0 * stats[b * 4];
      contract_row<BT>(p, WT + i, (size_t)N * N, (size_t)N, cur, sc, re);
#pragma unroll
      for (int b = 0; b < BT; ++b) {
        const float r = fmaf(p.alpha, act_fn<ACT>(re[b]), (1.f - p.alpha) * cur[i * BT + b]);
        nxt[i * BT + b] = r;
        if (o.hist != nullptr && b0 + b < p.B) o.hist[((size_t)t * p.B + b0 + b) * N + i] = r;
      }
    }
    __syncthreads();
    float* tmp = cur; cur = nxt; nxt = tmp;
  }
  if (o.final_state != nullptr) {
    for (int idx = threadIdx.x; idx < N * BT; idx += FT) {
      const int b = idx / N, j = idx % N;
      if (b0 + b < p.B) o.final_state[(size_t)(b0 + b) * N + j] = cur[j * BT + b];
    }
  }
}

struct Fp32BwdIn {
  const float* hist;         // [T,B,N]
  const float* grad_output;  // [T,B,N] or nullptr
  const float* coef_x;       // [B,T] or nullptr
  const float* coef_y;
  const float* coef_s;
  const float* dec_u;        // [N]
  const float* dec_v;
  float* delta;              // [T,B,N] out
  float* grad_r_init;        // [B,N] or nullptr
  float* grad_A;             // [B,T,a_dim] or nullptr (columns of inactive matrices are zeroed by the host)
};

template <int ACT, int BT>
__global__ void __launch_bounds__(FT) bwd_fp32_kernel(DevProblem p, const float* __restrict__ WT, Fp32BwdIn in) {
  extern __shared__ __align__(16) float smem[];
  const int N = p.N;
  float* rp = smem;                         // [N][BT] r_{t-1}
  float* gs = rp + (size_t)N * BT;          // [N][BT] carry, then g_t
  float* ds = gs + (size_t)N * BT;          // [N][BT] delta_t
  float* sc = ds + (size_t)N * BT;          // [n_mat][BT]
  float* cf = sc + p.n_mat * BT;            // [3][BT] loss coefficients of this step
  float* red = cf + 3 * BT;                 // [FT/BT][BT][4]
  float* stats = red + (FT / BT) * BT * 4;  // [BT][4]
  float* dacc = stats + BT * 4;             // [n_mat][BT][FT/32] per-warp sums for dL/dA
  const int b0 = blockIdx.x * BT;
  const bool has_coef = in.coef_x != nullptr;
  const bool want_dA = in.grad_A != nullptr;
  const int warp_id = threadIdx.x >> 5, lane_id = threadIdx.x & 31;

  for (int idx = threadIdx.x; idx < N * BT; idx += FT) gs[idx] = 0.f;

  for (int t = p.T - 1; t >= 0; --t) {
    const float* prev = (t == 0) ? p.r_init : in.hist + (size_t)(t - 1) * p.B * N;
    for (int idx = threadIdx.x; idx < N * BT; idx += FT) {
      const int b = idx / N, j = idx % N;
      rp[j * BT + b] = (b0 + b < p.B) ? prev[(size_t)(b0 + b) * N + j] : 0.f;
    }
    load_scales<BT>(p, b0, t, sc);
    if (threadIdx.x < 3 * BT) {
      const int c = threadIdx.x / BT, b = threadIdx.x % BT;
      float v = 0.f;
      if (has_coef && b0 + b < p.B) {
        const float* src = (c == 0) ? in.coef_x : (c == 1) ? in.coef_y : in.coef_s;
        v = src[(size_t)(b0 + b) * p.T + t];
      }
      cf[threadIdx.x] = v;
    }
    if (want_dA)
      for (int idx = threadIdx.x; idx < p.n_mat * BT * (FT / 32); idx += FT) dacc[idx] = 0.f;
    __syncthreads();
    state_stats<BT>(rp, N, nullptr, nullptr, red, stats);
    // phase 1: recompute re_t, form g_t and delta_t for the neurons this thread owns
    for (int i = threadIdx.x; i < N; i += FT) {
      float re[BT];
#pragma unroll
      for (int b = 0; b < BT; ++b) re[b] = p.J0 * stats[b * 4];
      contract_row<BT>(p, WT + i, (size_t)N * N, (size_t)N, rp, sc, re);
      const float ui = has_coef ? __ldg(in.dec_u + i) : 0.f;
      const float vi = has_coef ? __ldg(in.dec_v + i) : 0.f;
#pragma unroll
      for (int b = 0; b < BT; ++b) {
        float g = gs[i * BT + b];
        float d = 0.f;
        if (b0 + b < p.B) {
          const size_t at = ((size_t)t * p.B + b0 + b) * N + i;
          if (in.grad_output != nullptr) g += in.grad_output[at];
          if (has_coef) {
            const float rt = in.hist[at];
            const float sg = (rt > 0.f) ? 1.f : ((rt < 0.f) ? -1.f : 0.f);
            g += cf[b] * ui + cf[BT + b] * vi + cf[2 * BT + b] * sg;
          }
          d = p.alpha * act_grad<ACT>(re[b]) * g;
          in.delta[at] = d;
        }
        gs[i * BT + b] = g;
        ds[i * BT + b] = d;
      }
    }
    __syncthreads();
    state_stats<BT>(ds, N, nullptr, nullptr, red, stats);
    // phase 2: carry_{t-1}[b,j] = (1-alpha) g + J0*sum_i delta + sum_m sc_m * sum_i delta[b,i] W_m[i,j]
    // (uniform trip count: the dL/dA sums below use warp shuffles)
    for (int j0 = 0; j0 < N; j0 += FT) {
      const int j = j0 + threadIdx.x;
      const bool live = j < N;
      float acc[BT];
#pragma unroll
      for (int b = 0; b < BT; ++b) acc[b] = live ? fmaf(p.J0, stats[b * 4], (1.f - p.alpha) * gs[j * BT + b]) : 0.f;
      // m = 0 is Wo, m >= 1 are the active Wa matrices, all in their original [i][j] layout
      for (int m = 0; m < p.n_mat; ++m) {
        const float* W = (m == 0) ? p.Wo : p.Wa + (size_t)active_col(p, m - 1) * N * N;
        float tmp[BT];
#pragma unroll
        for (int b = 0; b < BT; ++b) tmp[b] = 0.f;
        if (live) {
#pragma unroll 4
          for (int i = 0; i < N; ++i) {
            const float wv = __ldg(W + (size_t)i * N + j);
            const float4* s4 = reinterpret_cast<const float4*>(ds + i * BT);
#pragma unroll
            for (int b4 = 0; b4 < BT / 4; ++b4) {
              const float4 s = s4[b4];
              tmp[b4 * 4 + 0] = fmaf(s.x, wv, tmp[b4 * 4 + 0]);
              tmp[b4 * 4 + 1] = fmaf(s.y, wv, tmp[b4 * 4 + 1]);
              tmp[b4 * 4 + 2] = fmaf(s.z, wv, tmp[b4 * 4 + 2]);
              tmp[b4 * 4 + 3] = fmaf(s.w, wv, tmp[b4 * 4 + 3]);
            }
          }
        }
#pragma unroll
        for (int b = 0; b < BT; ++b) acc[b] = fmaf(sc[m * BT + b], tmp[b], acc[b]);
        if (want_dA && m > 0) {
          // dL/dA[b,t,k] = sum_j r_{t-1}[b,j] * (delta_t W_k)[b,j]: per-warp sums in fixed order, one writer per slot
#pragma unroll
          for (int b = 0; b < BT; ++b) {
            float v = live ? rp[j * BT + b] * tmp[b] : 0.f;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
            if (lane_id == 0) dacc[(m * BT + b) * (FT / 32) + warp_id] += v;
          }
        }
      }
      if (live) {
#pragma unroll
        for (int b = 0; b < BT; ++b) gs[j * BT + b] = acc[b];
      }
    }
    __syncthreads();
    if (want_dA) {
      for (int idx = threadIdx.x; idx < (p.n_mat - 1) * BT; idx += FT) {
        const int m = 1 + idx / BT, b = idx % BT;
        float v = 0.f;
        for (int w = 0; w < FT / 32; ++w) v += dacc[(m * BT + b) * (FT / 32) + w];
        if (b0 + b < p.B) in.grad_A[((size_t)(b0 + b) * p.T + t) * p.a_dim + active_col(p, m - 1)] = v;
      }
      __syncthreads();  // dacc is zeroed at the top of the next step
    }
  }
  if (in.grad_r_init != nullptr) {
    for (int idx = threadIdx.x; idx < N * BT; idx += FT) {
      const int b = idx / N, j = idx % N;
      if (b0 + b < p.B) in.grad_r_init[(size_t)(b0 + b) * N + j] = gs[j * BT + b];
    }
  }
}

// ---- weight gradients: partial[s][m][i][j] = sum_{k in split s} scale_m[k] delta[k][i] rprev[k][j]
constexpr int DW_TILE = 64;
constexpr int DW_KC = 16;

__global__ void __launch_bounds__(256) dw_fp32_kernel(DevProblem p, const float* __restrict__ delta,
                                                      const float* __restrict__ hist, float* __restrict__ partial,
                                                      int ksplit, long long k_per_split) {
  __shared__ __align__(16) float dsm[DW_KC][DW_TILE];
  __shared__ __align__(16) float rsm[DW_KC][DW_TILE];
  const int N = p.N;
  const int m = blockIdx.z / ksplit, s = blockIdx.z % ksplit;
  const int i0 = blockIdx.y * DW_TILE, j0 = blockIdx.x * DW_TILE;
  const long long K = (long long)p.T * p.B;
  const long long k_begin = (long long)s * k_per_split;
  const long long k_end = (k_begin + k_per_split < K) ? k_begin + k_per_split : K;
  const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
  const int lr = threadIdx.x / 16;        // k row this thread loads
  const int lc = (threadIdx.x % 16) * 4;  // first of 4 columns it loads
  float acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;

  for (long long kk = k_begin; kk < k_end; kk += DW_KC) {
    const long long k = kk + lr;
    float dv[4] = {0.f, 0.f, 0.f, 0.f}, rv[4] = {0.f, 0.f, 0.f, 0.f};
    if (k < k_end) {
      const int t = (int)(k / p.B), b = (int)(k % p.B);
      const float sc = (m == 0) ? 1.f : __ldg(p.A + ((size_t)b * p.T + t) * p.a_dim + active_col(p, m - 1));
      const float* drow = delta + (size_t)k * N;
      const float* rrow = (t == 0) ? p.r_init + (size_t)b * N : hist + ((size_t)(t - 1) * p.B + b) * N;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        if (i0 + lc + c < N) dv[c] = sc * __ldg(drow + i0 + lc + c);
        if (j0 + lc + c < N) rv[c] = __ldg(rrow + j0 + lc + c);
      }
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      dsm[lr][lc + c] = dv[c];
      rsm[lr][lc + c] = rv[c];
    }
    __syncthreads();
#pragma unroll
    for (int q = 0; q < DW_KC; ++q) {
      const float4 a4 = *reinterpret_cast<const float4*>(&dsm[q][ty * 4]);
      const float4 b4 = *reinterpret_cast<const float4*>(&rsm[q][tx * 4]);
      const float av[4] = {a4.x, a4.y, a4.z, a4.w};
      const float bv[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = fmaf(av[a], bv[b], acc[a][b]);
    }
  }
  float* out = partial + ((size_t)s * p.n_mat + m) * N * N;
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int i = i0 + ty * 4 + a;
    if (i >= N) continue;
#pragma unroll
    for (int b = 0; b < 4; ++b) {
      const int j = j0 + tx * 4 + b;
      if (j < N) out[(size_t)i * N + j] = acc[a][b];
    }
  }
}

// grad_Wo = J1 * sum_s partial[s][0], grad_Wa[cols[m-1]] = sum_s partial[s][m]; raw[] keeps the
// unscaled m = 0 sum for the J0/J1 gradients.
__global__ void dw_reduce_kernel(DevProblem p, const float* __restrict__ partial, int ksplit, float* grad_Wa,
                                 float* grad_Wo, float* raw) {
  const size_t NN = (size_t)p.N * p.N;
  const size_t total = NN * p.n_mat;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int m = (int)(idx / NN);
    const size_t e = idx % NN;
    float acc = 0.f;
    for (int s = 0; s < ksplit; ++s) acc += partial[((size_t)s * p.n_mat + m) * NN + e];
    if (m == 0) {
      grad_Wo[e] = p.J1 * acc;
      if (raw != nullptr) raw[e] = acc;
    } else {
      grad_Wa[(size_t)active_col(p, m - 1) * NN + e] = acc;
    }
  }
}

}  // namespace

// dJ0 = sum_ij G_ij, dJ1 = sum_ij G_ij Wo_ij with G = sum_{t,b} delta^T r_prev.  Two passes, fixed order: `partial`
// holds 2 doubles per block of the first pass (grid GRAD_J_BLOCKS), the second pass (one block) adds them up.
__global__ void grad_j_partial_kernel(const float* __restrict__ raw, const float* __restrict__ Wo, size_t NN,
                                      double* __restrict__ partial) {
  __shared__ double s0[256], s1[256];
  double a0 = 0.0, a1 = 0.0;
  for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < NN; e += (size_t)gridDim.x * blockDim.x) {
    const double g = raw[e];
    a0 += g;
    a1 += g * Wo[e];
  }
  s0[threadIdx.x] = a0;
  s1[threadIdx.x] = a1;
  __syncthreads();
  for (int w = blockDim.x / 2; w > 0; w >>= 1) {
    if ((int)threadIdx.x < w) {
      s0[threadIdx.x] += s0[threadIdx.x + w];
      s1[threadIdx.x] += s1[threadIdx.x + w];
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    partial[2 * blockIdx.x] = s0[0];
    partial[2 * blockIdx.x + 1] = s1[0];
  }
}
__global__ void grad_j_finish_kernel(const double* __restrict__ partial, int nblocks, float* grad_J) {
  if (threadIdx.x == 0) {
    double a0 = 0.0, a1 = 0.0;
    for (int b = 0; b < nblocks; ++b) {
      a0 += partial[2 * b];
      a1 += partial[2 * b + 1];
    }
    grad_J[0] = (float)a0;
    grad_J[1] = (float)a1;
  }
}
// `scratch` needs GRAD_J_BLOCKS * 2 doubles
int launch_grad_j(const float* raw, const float* Wo, size_t NN, float* grad_J, double* scratch, cudaStream_t s) {
  {
    LaunchScope ls(K_REDUCE, s);
    grad_j_partial_kernel<<<GRAD_J_BLOCKS, 256, 0, s>>>(raw, Wo, NN, scratch);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  {
    LaunchScope ls(K_REDUCE, s);
    grad_j_finish_kernel<<<1, 32, 0, s>>>(scratch, GRAD_J_BLOCKS, grad_J);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  return RINGRNN_OK;
}

namespace {

int pick_ksplit(const RingRnnProblem& p, int n_mat) {
  const int tiles = ((p.N + DW_TILE - 1) / DW_TILE) * ((p.N + DW_TILE - 1) / DW_TILE) * n_mat;
  long long K = (long long)p.T * p.B;
  int ks = (4 * 148 + tiles - 1) / tiles;
  if (ks < 1) ks = 1;
  if (ks > 64) ks = 64;
  while (ks > 1 && K / ks < 64) --ks;
  return ks;
}

int n_mat_of(const RingRnnProblem& p) { return 1 + (p.n_active < 0 ? p.a_dim : p.n_active); }

size_t fwd_smem(int N, int n_mat, int BT) {
  return sizeof(float) * ((size_t)2 * N * BT + (size_t)n_mat * BT + (FT / BT) * BT * 4 + BT * 4);
}
size_t bwd_smem(int N, int n_mat, int BT) {
  return sizeof(float) * ((size_t)3 * N * BT + (size_t)n_mat * BT + 3 * BT + (FT / BT) * BT * 4 + BT * 4 +
                          (size_t)n_mat * BT * (FT / 32));
}
constexpr size_t SMEM_MAX = 227 * 1024;

template <int BT>
int launch_fwd(const DevProblem& dp, int act, const float* WT, const Fp32FwdOut& o, cudaStream_t s) {
  const size_t smem = fwd_smem(dp.N, dp.n_mat, BT);
  const int grid = (dp.B + BT - 1) / BT;
#define RINGRNN_FWD_CASE(ACT)                                                                                  \
  case ACT:                                                                                                    \
    RINGRNN_CUDA_TRY(cudaFuncSetAttribute(fwd_fp32_kernel<ACT, BT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                          (int)smem));                                                         \
    { LaunchScope ls(K_FWD, s); fwd_fp32_kernel<ACT, BT><<<grid, FT, smem, s>>>(dp, WT, o); }                  \
    break;
  switch (act) {
    RINGRNN_FWD_CASE(RINGRNN_ACT_RELU)
    RINGRNN_FWD_CASE(RINGRNN_ACT_GELU)
    RINGRNN_FWD_CASE(RINGRNN_ACT_TANH)
    RINGRNN_FWD_CASE(RINGRNN_ACT_SILU)
    default:
      return RINGRNN_ERR_ARG;
  }
#undef RINGRNN_FWD_CASE
  RINGRNN_CUDA_TRY(cudaGetLastError());
  return RINGRNN_OK;
}

template <int BT>
int launch_bwd(const DevProblem& dp, int act, const float* WT, const Fp32BwdIn& in, cudaStream_t s) {
  const size_t smem = bwd_smem(dp.N, dp.n_mat, BT);
  const int grid = (dp.B + BT - 1) / BT;
#define RINGRNN_BWD_CASE(ACT)                                                                                  \
  case ACT:                                                                                                    \
    RINGRNN_CUDA_TRY(cudaFuncSetAttribute(bwd_fp32_kernel<ACT, BT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                          (int)smem));                                                         \
    { LaunchScope ls(K_BWD, s); bwd_fp32_kernel<ACT, BT><<<grid, FT, smem, s>>>(dp, WT, in); }                 \
    break;
  switch (act) {
    RINGRNN_BWD_CASE(RINGRNN_ACT_RELU)
    RINGRNN_BWD_CASE(RINGRNN_ACT_GELU)
    RINGRNN_BWD_CASE(RINGRNN_ACT_TANH)
    RINGRNN_BWD_CASE(RINGRNN_ACT_SILU)
    default:
      return RINGRNN_ERR_ARG;
  }
#undef RINGRNN_BWD_CASE
  RINGRNN_CUDA_TRY(cudaGetLastError());
  return RINGRNN_OK;
}

int launch_transpose(const DevProblem& dp, float* WT, cudaStream_t s) {
  dim3 grid((dp.N + 31) / 32, (dp.N + 31) / 32, dp.n_mat), block(32, 8);
  { LaunchScope ls(K_PREP, s); transpose_weights_kernel<<<grid, block, 0, s>>>(dp, WT); }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  return RINGRNN_OK;
}

}  // namespace

// workspace layouts ----------------------------------------------------------------------------
//   FWD : WT[n_mat][N][N]
//   SAVED (only when the caller does not keep bump_history): hist[T][B][N]
//   BWD : WT[n_mat][N][N] | delta[T][B][N] | partial[ksplit][n_mat][N][N] | raw[N][N]
size_t fp32_fwd_workspace_bytes(const RingRnnProblem& p) {
  return align_up(sizeof(float) * (size_t)n_mat_of(p) * p.N * p.N, 256);
}
size_t fp32_saved_bytes(const RingRnnProblem& p, int history_given) {
  return history_given ? 0 : align_up(sizeof(float) * (size_t)p.T * p.B * p.N, 256);
}
// bytes of the split-(t,b) partial sums; never less than the scratch the dJ reduction borrows from the same region
static size_t partial_bytes(const RingRnnProblem& p, int n_mat) {
  const size_t b = sizeof(float) * (size_t)pick_ksplit(p, n_mat) * n_mat * p.N * p.N;
  const size_t min_b = sizeof(double) * 2 * GRAD_J_BLOCKS;
  return align_up(b > min_b ? b : min_b, 256);
}
size_t fp32_bwd_workspace_bytes(const RingRnnProblem& p) {
  const int n_mat = n_mat_of(p);
  const size_t NN = (size_t)p.N * p.N;
  return align_up(sizeof(float) * n_mat * NN, 256) + align_up(sizeof(float) * (size_t)p.T * p.B * p.N, 256) +
         partial_bytes(p, n_mat) + align_up(sizeof(float) * NN, 256);
}

int fp32_forward(const RingRnnFwdArgs& a, const DevProblem& dp, cudaStream_t s) {
  const RingRnnProblem& p = a.p;
  if (a.workspace == nullptr || a.workspace_bytes < fp32_fwd_workspace_bytes(p)) return RINGRNN_ERR_WORKSPACE;
  float* hist = a.bump_history;
  if (hist == nullptr && a.saved != nullptr) {
    if (a.saved_bytes < fp32_saved_bytes(p, 0)) return RINGRNN_ERR_WORKSPACE;
    hist = static_cast<float*>(a.saved);
  }
  float* WT = static_cast<float*>(a.workspace);
  int rc = launch_transpose(dp, WT, s);
  if (rc != RINGRNN_OK) return rc;
  Fp32FwdOut o{hist, a.dec_x, a.dec_y, a.dec_ta, a.dec_u, a.dec_v, a.final_state};
  if (fwd_smem(p.N, dp.n_mat, 16) <= SMEM_MAX) return launch_fwd<16>(dp, p.activation, WT, o, s);
  if (fwd_smem(p.N, dp.n_mat, 8) <= SMEM_MAX) return launch_fwd<8>(dp, p.activation, WT, o, s);
  if (fwd_smem(p.N, dp.n_mat, 4) <= SMEM_MAX) return launch_fwd<4>(dp, p.activation, WT, o, s);
  return RINGRNN_ERR_SHAPE;
}

int fp32_backward(const RingRnnBwdArgs& a, const DevProblem& dp, cudaStream_t s) {
  const RingRnnProblem& p = a.p;
  if (a.workspace == nullptr || a.workspace_bytes < fp32_bwd_workspace_bytes(p)) return RINGRNN_ERR_WORKSPACE;
  const float* hist = a.bump_history;
  if (hist == nullptr) {
    if (a.saved == nullptr || a.saved_bytes < fp32_saved_bytes(p, 0)) return RINGRNN_ERR_WORKSPACE;
    hist = static_cast<const float*>(a.saved);
  }
  const int n_mat = dp.n_mat;
  const size_t NN = (size_t)p.N * p.N;
  const int ksplit = pick_ksplit(p, n_mat);
  char* w = static_cast<char*>(a.workspace);
  float* WT = reinterpret_cast<float*>(w);
  w += align_up(sizeof(float) * n_mat * NN, 256);
  float* delta = reinterpret_cast<float*>(w);
  w += align_up(sizeof(float) * (size_t)p.T * p.B * p.N, 256);
  float* partial = reinterpret_cast<float*>(w);
  w += partial_bytes(p, n_mat);
  float* raw = reinterpret_cast<float*>(w);

  int rc = launch_transpose(dp, WT, s);
  if (rc != RINGRNN_OK) return rc;
  if (a.grad_A != nullptr)
    RINGRNN_CUDA_TRY(cudaMemsetAsync(a.grad_A, 0, sizeof(float) * (size_t)p.B * p.T * p.a_dim, s));
  Fp32BwdIn in{hist, a.grad_output, a.coef_x, a.coef_y, a.coef_s, a.dec_u, a.dec_v, delta, a.grad_r_init, a.grad_A};
  if (bwd_smem(p.N, n_mat, 16) <= SMEM_MAX) rc = launch_bwd<16>(dp, p.activation, WT, in, s);
  else if (bwd_smem(p.N, n_mat, 8) <= SMEM_MAX) rc = launch_bwd<8>(dp, p.activation, WT, in, s);
  else if (bwd_smem(p.N, n_mat, 4) <= SMEM_MAX) rc = launch_bwd<4>(dp, p.activation, WT, in, s);
  else rc = RINGRNN_ERR_SHAPE;
  if (rc != RINGRNN_OK) return rc;

  const long long K = (long long)p.T * p.B;
  long long kps = (K + ksplit - 1) / ksplit;
  kps = (kps + DW_KC - 1) / DW_KC * DW_KC;
  dim3 grid((p.N + DW_TILE - 1) / DW_TILE, (p.N + DW_TILE - 1) / DW_TILE, n_mat * ksplit);
  { LaunchScope ls(K_DW, s); dw_fp32_kernel<<<grid, 256, 0, s>>>(dp, delta, hist, partial, ksplit, kps); }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  RINGRNN_CUDA_TRY(cudaMemsetAsync(a.grad_Wa, 0, sizeof(float) * (size_t)p.a_dim * NN, s));
  { LaunchScope ls(K_REDUCE, s); dw_reduce_kernel<<<296, 256, 0, s>>>(dp, partial, ksplit, a.grad_Wa, a.grad_Wo, raw); }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  if (a.grad_J != nullptr) {
    // the split-(t,b) partials are dead after the reduction above: their storage serves as scratch
    rc = launch_grad_j(raw, p.Wo, NN, a.grad_J, reinterpret_cast<double*>(partial), s);
    if (rc != RINGRNN_OK) return rc;
  }
  return RINGRNN_OK;
}

}  // namespace ringrnn
