// bf16 mode, stepwise variant: one tensor-core GEMM per timestep instead of a persistent kernel.
//
// Used for shapes the persistent tcgen05 kernels do not take (N > 1024, or N > 512 with more than two active action
// columns), i.e. the large-N, wide-action-signal rows of the reference's published latency table, where the batch
// is small (256) and one step is already a full-machine GEMM.  Replaces, for those shapes, the same reference
// kernels as the persistent path (cpp/kernels/fwd_1loop_tc_idx.cuh:265-277 and the five per-step launches of
// cpp/kernels/bwd_mixed_precision_aggressive.cuh:564-671), without materialising W_eff[B,N,N].
//
// With m = 0 for Wo and m = 1..n for the active action matrices (coefficient c_0 = 1 -- J1 is folded into the
// stacked weights -- and c_m = A[b,t,cols[m-1]]):
//   forward   X_t[b, m*NP + j] = c_m r_{t-1}[b,j]  (bf16)      re_t = X_t . Wst^T + J0 sum_j r_{t-1}[b,j]
//             Wst[i, m*NP + j] = W_m[i,j]                       (one GEMM [BP,(1+n)NP] x [(1+n)NP,NP] per step)
//   backward  Z_t = delta_t . WstT^T,  WstT[m*NP + j, i] = W_m[i,j]   ([BP,NP] x [NP,(1+n)NP] per step)
//             carry[b,j] = (1-alpha) g_t[b,j] + J0 sum_i delta_t[b,i] + sum_m c_m Z_t[b, m*NP + j]
//             dL/dA[b,t,cols[k]] = sum_j r_{t-1}[b,j] Z_t[b,(1+k)*NP + j]
//   weights   dWst = sum_t delta_t^T X_t: one split-K GEMM over all (t, b) at the end.
// Between the GEMMs a row kernel (one block per sample) applies the epilogue of one step and prepares the operand
// of the next, so a step costs two launches.  Split-K partial sums are reduced in fixed order: bit-reproducible.
#include <string.h>

#include "ringrnn_common.cuh"

namespace ringrnn {

namespace {

constexpr int ROW_THREADS = 256;

struct SwCols {
  int n;
  int c[RINGRNN_MAX_ACTIVE];
};

struct SwLayout {
  int NP, BP, n_act, blocks;  // blocks = 1 + n_act column blocks of NP
  long long KX;               // (1 + n_act) * NP
  int ns_fwd, ns_bwd, ns_dw;  // split-K factors of the three GEMMs
};

int sw_active(const RingRnnProblem& p) { return p.n_active < 0 ? p.a_dim : p.n_active; }

int splits_for(long long tiles, long long K) {
  long long ns = 148 / (tiles > 0 ? tiles : 1);
  while (ns > 1 && K / ns < 512) --ns;
  return (int)(ns < 1 ? 1 : ns);
}

SwLayout sw_layout(const RingRnnProblem& p) {
  SwLayout l;
  l.NP = (p.N + 127) / 128 * 128;
  l.BP = (p.B + 127) / 128 * 128;
  l.n_act = sw_active(p);
  l.blocks = 1 + l.n_act;
  l.KX = (long long)l.blocks * l.NP;
  const int nt_fwd = (l.NP % 512 == 0) ? 512 : (l.NP % 256 == 0) ? 256 : 128;
  l.ns_fwd = splits_for((long long)(l.BP / 128) * (l.NP / nt_fwd), l.KX);
  const int nt_bwd = (l.KX % 512 == 0) ? 512 : (l.KX % 256 == 0) ? 256 : 128;
  l.ns_bwd = splits_for((long long)(l.BP / 128) * (l.KX / nt_bwd), l.NP);
  l.ns_dw = splits_for((long long)(l.NP / 128) * (l.KX / nt_bwd), (long long)p.T * l.BP);
  return l;
}

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16(x)); }

// block-wide sum (blockDim.x == ROW_THREADS); every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();  // red may still be read from the previous call
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < ROW_THREADS / 32; ++w) tot += red[w];
  return tot;
}

// Wst [NP][KX] and WstT [KX][NP] (bf16, zero padded); block 0 carries J1.  grid (NP, blocks), block 256
__global__ void sw_prep_weights_kernel(const float* __restrict__ Wo, const float* __restrict__ Wa, SwCols cols, float J1,
                                       int N, int NP, long long KX, __nv_bfloat16* __restrict__ Wst,
                                       __nv_bfloat16* __restrict__ WstT) {
  const int i = blockIdx.x, m = blockIdx.y;
  const float* W = (m == 0) ? Wo : Wa + (size_t)cols.c[m - 1] * N * N;
  const float scale = (m == 0) ? J1 : 1.f;
  for (int j = threadIdx.x; j < NP; j += blockDim.x) {
    const float v = (i < N && j < N) ? scale * W[(size_t)i * N + j] : 0.f;
    if (Wst != nullptr) Wst[(size_t)i * KX + (size_t)m * NP + j] = __float2bfloat16(v);
    // WstT row (m, j) holds W_m[:, j]: written from the same thread's transposed element for coalescing
    if (WstT != nullptr) {
      const float vt = (i < N && j < N) ? scale * W[(size_t)j * N + i] : 0.f;  // W_m[j, i] -> WstT[(m, i), j]
      WstT[((size_t)m * NP + i) * NP + j] = __float2bfloat16(vt);
    }
  }
}

struct SwFwd {
  int B, T, N, NP, BP, a_dim, nsplit;
  long long KX;
  float J0, alpha;
  const float* A;
  const float* r_init;
  const float* partial;    // [nsplit][BP][NP]
  float* state;            // [BP][NP] fp32 master state
  float* rowsum;           // [BP]
  __nv_bfloat16* X;        // [BP][KX]
  __nv_bfloat16* Rh;       // [T+1][BP][NP] or nullptr
  __nv_bfloat16* Dh;       // [T][BP][NP] or nullptr
  float* hist;             // [T,B,N] or nullptr
  float* final_state;      // [B,N] or nullptr
  float* dec_x;            // [B,T] or nullptr
  float* dec_y;
  float* dec_ta;
  const float* dec_u;
  const float* dec_v;
  SwCols cols;
};

// One block per padded sample row.  t >= 0: finishes step t (r_t from the GEMM of step t), then builds the operand
// of step t+1.  t = -1: loads r_init and builds the operand of step 0.
template <int ACT>
__global__ void sw_forward_row_kernel(SwFwd q, int t) {
  __shared__ float red[ROW_THREADS / 32];
  const int b = blockIdx.x;
  const bool valid = b < q.B;
  float* st = q.state + (size_t)b * q.NP;
  float px = 0.f, py = 0.f, pa = 0.f, rs = 0.f;
  const float s_prev = (t >= 0) ? q.rowsum[b] : 0.f;
  const bool build = t + 1 < q.T;
  const float* a_next = q.A + ((size_t)b * q.T + (t + 1)) * q.a_dim;  // read only when valid && build
  __nv_bfloat16* xrow = q.X + (size_t)b * q.KX;
  for (int i = threadIdx.x; i < q.NP; i += ROW_THREADS) {
    float r = 0.f;
    if (valid && i < q.N) {
      if (t < 0) {
        r = q.r_init[(size_t)b * q.N + i];
      } else {
        float re = q.J0 * s_prev;
        for (int s = 0; s < q.nsplit; ++s) re += q.partial[((size_t)s * q.BP + b) * q.NP + i];
        r = fmaf(q.alpha, act_fn<ACT>(re), (1.f - q.alpha) * st[i]);
        if (q.Dh != nullptr) q.Dh[((size_t)t * q.BP + b) * q.NP + i] = __float2bfloat16(act_grad<ACT>(re));
        if (q.hist != nullptr) q.hist[((size_t)t * q.B + b) * q.N + i] = r;
        if (q.final_state != nullptr && t + 1 == q.T) q.final_state[(size_t)b * q.N + i] = r;
        if (q.dec_x != nullptr || q.dec_y != nullptr) {
          px = fmaf(r, q.dec_u[i], px);
          py = fmaf(r, q.dec_v[i], py);
        }
        pa += fabsf(r);
      }
    } else if (t >= 0 && q.Dh != nullptr) {
      q.Dh[((size_t)t * q.BP + b) * q.NP + i] = __float2bfloat16(0.f);
    }
    st[i] = r;
    const __nv_bfloat16 rb = __float2bfloat16(r);
    if (q.Rh != nullptr) q.Rh[((size_t)(t + 1) * q.BP + b) * q.NP + i] = rb;
    if (build) {
      const float rf = __bfloat162float(rb);
      rs += rf;
      xrow[i] = rb;
      for (int k = 0; k < q.cols.n; ++k) {
        const float ck = valid ? __ldg(a_next + q.cols.c[k]) : 0.f;
        xrow[(size_t)(1 + k) * q.NP + i] = __float2bfloat16(ck * rf);
      }
    }
  }
  if (build) {
    const float tot = block_sum(rs, red);
    if (threadIdx.x == 0) q.rowsum[b] = tot;
  }
  if (t >= 0 && valid && (q.dec_x != nullptr || q.dec_y != nullptr || q.dec_ta != nullptr)) {
    const float sx = block_sum(px, red), sy = block_sum(py, red), sa = block_sum(pa, red);
    if (threadIdx.x == 0) {
      const size_t o = (size_t)b * q.T + t;
      if (q.dec_x != nullptr) q.dec_x[o] = sx;
      if (q.dec_y != nullptr) q.dec_y[o] = sy;
      if (q.dec_ta != nullptr) q.dec_ta[o] = sa;
    }
  }
}

struct SwBwd {
  int B, T, N, NP, BP, a_dim, nsplit;
  long long KX;
  float J0, alpha;
  const float* A;
  const float* grad_output;  // [T,B,N] or nullptr
  const float* coef_x;       // [B,T] or nullptr
  const float* coef_y;
  const float* coef_s;
  const float* dec_u;
  const float* dec_v;
  const __nv_bfloat16* Rh;   // [T+1][BP][NP]
  const __nv_bfloat16* Dh;   // [T][BP][NP]
  const float* partial;      // [nsplit][BP][KX]: Z of the step whose carry is formed
  float* g;                  // [BP][NP] fp32: g_t of the step in flight
  float* sum_delta;          // [BP]
  __nv_bfloat16* Delta;      // [T][BP][NP]
  float* grad_r_init;        // [B,N] or nullptr
  float* grad_A;             // [B,T,a_dim] or nullptr (pre-zeroed)
  SwCols cols;
};

// One block per padded sample row.  t_carry >= 0: forms the carry out of step t_carry from Z (and dL/dA of that
// step); t_delta >= 0: g and delta of step t_delta from the carry (zero when t_carry < 0).
__global__ void sw_backward_row_kernel(SwBwd q, int t_carry, int t_delta) {
  __shared__ float red[ROW_THREADS / 32];
  const int b = blockIdx.x;
  const bool valid = b < q.B;
  float* g = q.g + (size_t)b * q.NP;
  const float beta = 1.f - q.alpha;
  const float sd = (t_carry >= 0) ? q.sum_delta[b] : 0.f;
  const float* a_c = q.A + ((size_t)b * q.T + (t_carry >= 0 ? t_carry : 0)) * q.a_dim;
  float cx = 0.f, cy = 0.f, cs = 0.f;
  if (valid && t_delta >= 0 && q.coef_x != nullptr) {
    cx = q.coef_x[(size_t)b * q.T + t_delta];
    cy = q.coef_y[(size_t)b * q.T + t_delta];
    cs = q.coef_s[(size_t)b * q.T + t_delta];
  }
  float ds = 0.f;
  for (int j = threadIdx.x; j < q.NP; j += ROW_THREADS) {
    float carry = 0.f;
    const bool live = valid && j < q.N;
    if (t_carry >= 0 && live) {
      carry = fmaf(beta, g[j], q.J0 * sd);
      for (int m = 0; m <= q.cols.n; ++m) {
        float z = 0.f;
        for (int s = 0; s < q.nsplit; ++s) z += q.partial[((size_t)s * q.BP + b) * q.KX + (size_t)m * q.NP + j];
        const float cm = (m == 0) ? 1.f : __ldg(a_c + q.cols.c[m - 1]);
        carry = fmaf(cm, z, carry);
      }
    }
    if (t_delta >= 0) {
      float gg = carry;
      if (live) {
        if (q.grad_output != nullptr) gg += q.grad_output[((size_t)t_delta * q.B + b) * q.N + j];
        if (q.coef_x != nullptr) {
          const float r = __bfloat162float(q.Rh[((size_t)(t_delta + 1) * q.BP + b) * q.NP + j]);
          gg = fmaf(cx, q.dec_u[j], gg);
          gg = fmaf(cy, q.dec_v[j], gg);
          gg = fmaf(cs, (r > 0.f) ? 1.f : ((r < 0.f) ? -1.f : 0.f), gg);
        }
      } else {
        gg = 0.f;
      }
      g[j] = gg;
      const float dact = __bfloat162float(q.Dh[((size_t)t_delta * q.BP + b) * q.NP + j]);
      const __nv_bfloat16 db = __float2bfloat16(q.alpha * dact * gg);
      q.Delta[((size_t)t_delta * q.BP + b) * q.NP + j] = db;
      ds += __bfloat162float(db);
    } else if (live && q.grad_r_init != nullptr) {
      q.grad_r_init[(size_t)b * q.N + j] = carry;
    }
  }
  if (t_delta >= 0) {
    const float tot = block_sum(ds, red);
    if (threadIdx.x == 0) q.sum_delta[b] = tot;
  }
  if (t_carry >= 0 && valid && q.grad_A != nullptr) {
    // dL/dA[b,t,cols[k]] = sum_j r_{t-1}[b,j] Z[b,(1+k)NP + j]
    const __nv_bfloat16* rprev = q.Rh + ((size_t)t_carry * q.BP + b) * q.NP;
    for (int k = 0; k < q.cols.n; ++k) {
      float acc = 0.f;
      for (int j = threadIdx.x; j < q.N; j += ROW_THREADS) {
        float z = 0.f;
        for (int s = 0; s < q.nsplit; ++s) z += q.partial[((size_t)s * q.BP + b) * q.KX + (size_t)(1 + k) * q.NP + j];
        acc = fmaf(__bfloat162float(rprev[j]), z, acc);
      }
      const float tot = block_sum(acc, red);
      if (threadIdx.x == 0) q.grad_A[((size_t)b * q.T + t_carry) * q.a_dim + q.cols.c[k]] = tot;
    }
  }
}

// Xall[t][b][m*NP + j] = c_m(b,t) * r_{t-1}[b,j] for all t: the B operand of the weight-gradient GEMM.
// grid (BP, T), block 256
__global__ void sw_build_xall_kernel(const __nv_bfloat16* __restrict__ Rh, const float* __restrict__ A, SwCols cols,
                                     int B, int T, int a_dim, int NP, int BP, long long KX,
                                     __nv_bfloat16* __restrict__ Xall) {
  const int b = blockIdx.x, t = blockIdx.y;
  const bool valid = b < B;
  const __nv_bfloat16* r = Rh + ((size_t)t * BP + b) * NP;
  __nv_bfloat16* x = Xall + ((size_t)t * BP + b) * KX;
  const float* at = A + ((size_t)b * T + t) * a_dim;
  for (int j = threadIdx.x; j < NP; j += blockDim.x) {
    const __nv_bfloat16 rb = r[j];
    const float rf = __bfloat162float(rb);
    x[j] = rb;
    for (int k = 0; k < cols.n; ++k) {
      const float ck = valid ? __ldg(at + cols.c[k]) : 0.f;
      x[(size_t)(1 + k) * NP + j] = __float2bfloat16(ck * rf);
    }
  }
}

// dWst [NP][KX] -> grad_Wo = J1 * block 0 (the operand block 0 is the unscaled state), raw = block 0,
// grad_Wa[cols[k]] = block 1 + k
__global__ void sw_unpack_dw_kernel(const float* __restrict__ dWst, int N, int NP, long long KX, float J1, SwCols cols,
                                    float* grad_Wo, float* grad_Wa, float* raw) {
  const size_t NN = (size_t)N * N;
  for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < NN; e += (size_t)gridDim.x * blockDim.x) {
    const int i = (int)(e / N), j = (int)(e % N);
    const float g0 = dWst[(size_t)i * KX + j];
    grad_Wo[e] = J1 * g0;
    raw[e] = g0;
    for (int k = 0; k < cols.n; ++k) grad_Wa[(size_t)cols.c[k] * NN + e] = dWst[(size_t)i * KX + (size_t)(1 + k) * NP + j];
  }
}

SwCols cols_of(const DevProblem& dp) {
  SwCols c;
  c.n = dp.n_mat - 1;
  for (int k = 0; k < c.n; ++k) c.c[k] = dp.cols[k];
  return c;
}

template <int ACT>
void launch_forward_row(const SwFwd& q, int t, cudaStream_t s) {
  LaunchScope ls(K_FWD, s);
  sw_forward_row_kernel<ACT><<<q.BP, ROW_THREADS, 0, s>>>(q, t);
}

void forward_row(int act, const SwFwd& q, int t, cudaStream_t s) {
  switch (act) {
    case RINGRNN_ACT_RELU: launch_forward_row<RINGRNN_ACT_RELU>(q, t, s); break;
    case RINGRNN_ACT_GELU: launch_forward_row<RINGRNN_ACT_GELU>(q, t, s); break;
    case RINGRNN_ACT_SILU: launch_forward_row<RINGRNN_ACT_SILU>(q, t, s); break;
    default: launch_forward_row<RINGRNN_ACT_TANH>(q, t, s); break;
  }
}

}  // namespace

// Any N (padded to a multiple of 128) and up to RINGRNN_MAX_ACTIVE active columns; the stacked operand of one step
// must stay below 2^31 elements per row block for the GEMM's 32-bit extents.
bool stepwise_supported(const RingRnnProblem& p) {
  const int n_act = sw_active(p);
  if (p.B < 1 || p.T < 1 || p.N < 1 || n_act > RINGRNN_MAX_ACTIVE) return false;
  const long long NP = (p.N + 127) / 128 * 128;
  return NP <= 16384 && (1 + n_act) * NP <= (1ll << 30);
}

// FWD workspace: status(1024) | Wst | X | state | rowsum | split-K partials
size_t stepwise_fwd_workspace_bytes(const RingRnnProblem& p) {
  const SwLayout l = sw_layout(p);
  return 1024 + align_up((size_t)l.NP * l.KX * 2, 1024) + align_up((size_t)l.BP * l.KX * 2, 1024) +
         align_up((size_t)l.BP * l.NP * 4, 1024) + align_up((size_t)l.BP * 4, 1024) +
         align_up((size_t)l.ns_fwd * l.BP * l.NP * 4, 1024);
}
// SAVED: Rh [T+1][BP][NP] | Dh [T][BP][NP] (bf16)
size_t stepwise_saved_bytes(const RingRnnProblem& p) {
  const SwLayout l = sw_layout(p);
  return align_up((size_t)(p.T + 1) * l.BP * l.NP * 2, 1024) + align_up((size_t)p.T * l.BP * l.NP * 2, 1024);
}
// BWD workspace: status(1024) | WstT | Delta [T][BP][NP] | g | sum_delta | Z partials | Xall [T][BP][KX] |
//                dW partials | dWst | raw
size_t stepwise_bwd_workspace_bytes(const RingRnnProblem& p) {
  const SwLayout l = sw_layout(p);
  return 1024 + align_up((size_t)l.KX * l.NP * 2, 1024) + align_up((size_t)p.T * l.BP * l.NP * 2, 1024) +
         align_up((size_t)l.BP * l.NP * 4, 1024) + align_up((size_t)l.BP * 4, 1024) +
         align_up((size_t)l.ns_bwd * l.BP * l.KX * 4, 1024) + align_up((size_t)p.T * l.BP * l.KX * 2, 1024) +
         align_up((size_t)l.ns_dw * l.NP * l.KX * 4, 1024) + align_up((size_t)l.NP * l.KX * 4, 1024) +
         align_up((size_t)p.N * p.N * 4, 1024);
}

int stepwise_forward(const RingRnnFwdArgs& a, const DevProblem& dp, cudaStream_t s) {
  const RingRnnProblem& p = a.p;
  const SwLayout l = sw_layout(p);
  if (a.workspace == nullptr || a.workspace_bytes < stepwise_fwd_workspace_bytes(p)) return RINGRNN_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(a.workspace) & 255) != 0) return RINGRNN_ERR_WORKSPACE;
  const bool train = a.saved != nullptr;
  if (train && (a.saved_bytes < stepwise_saved_bytes(p) || (reinterpret_cast<uintptr_t>(a.saved) & 255) != 0))
    return RINGRNN_ERR_WORKSPACE;
  char* w = static_cast<char*>(a.workspace);
  int* status = a.status != nullptr ? a.status : reinterpret_cast<int*>(w);
  w += 1024;
  __nv_bfloat16* Wst = reinterpret_cast<__nv_bfloat16*>(w);
  w += align_up((size_t)l.NP * l.KX * 2, 1024);
  __nv_bfloat16* X = reinterpret_cast<__nv_bfloat16*>(w);
  w += align_up((size_t)l.BP * l.KX * 2, 1024);
  float* state = reinterpret_cast<float*>(w);
  w += align_up((size_t)l.BP * l.NP * 4, 1024);
  float* rowsum = reinterpret_cast<float*>(w);
  w += align_up((size_t)l.BP * 4, 1024);
  float* partial = reinterpret_cast<float*>(w);
  if (a.status == nullptr) RINGRNN_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(int), s));

  const SwCols cols = cols_of(dp);
  {
    LaunchScope ls(K_PREP, s);
    sw_prep_weights_kernel<<<dim3(l.NP, l.blocks), 256, 0, s>>>(p.Wo, dp.Wa, cols, p.J1, p.N, l.NP, l.KX, Wst, nullptr);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());

  SwFwd q;
  memset(&q, 0, sizeof(q));
  q.B = p.B; q.T = p.T; q.N = p.N; q.NP = l.NP; q.BP = l.BP; q.a_dim = p.a_dim; q.nsplit = l.ns_fwd;
  q.KX = l.KX; q.J0 = p.J0; q.alpha = p.alpha;
  q.A = p.A; q.r_init = p.r_init; q.partial = partial; q.state = state; q.rowsum = rowsum; q.X = X;
  q.Rh = train ? static_cast<__nv_bfloat16*>(a.saved) : nullptr;
  q.Dh = train ? reinterpret_cast<__nv_bfloat16*>(static_cast<char*>(a.saved) +
                                                   align_up((size_t)(p.T + 1) * l.BP * l.NP * 2, 1024))
               : nullptr;
  q.hist = a.bump_history; q.final_state = a.final_state;
  q.dec_x = a.dec_x; q.dec_y = a.dec_y; q.dec_ta = a.dec_ta; q.dec_u = a.dec_u; q.dec_v = a.dec_v;
  q.cols = cols;

  forward_row(p.activation, q, -1, s);
  RINGRNN_CUDA_TRY(cudaGetLastError());
  for (int t = 0; t < p.T; ++t) {
    // partial[s] = X_t[BP, KX] x Wst[NP, KX]^T over the s-th slice of KX (summed by the row kernel)
    int rc = tc_gemm(0, X, Wst, partial, nullptr, l.BP, l.NP, l.KX, l.ns_fwd, status, s);
    if (rc != RINGRNN_OK) return rc;
    forward_row(p.activation, q, t, s);
    RINGRNN_CUDA_TRY(cudaGetLastError());
  }
  return RINGRNN_OK;
}

int stepwise_backward(const RingRnnBwdArgs& a, const DevProblem& dp, cudaStream_t s) {
  const RingRnnProblem& p = a.p;
  const SwLayout l = sw_layout(p);
  if (a.workspace == nullptr || a.workspace_bytes < stepwise_bwd_workspace_bytes(p)) return RINGRNN_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(a.workspace) & 255) != 0) return RINGRNN_ERR_WORKSPACE;
  if (a.saved == nullptr || a.saved_bytes < stepwise_saved_bytes(p) || (reinterpret_cast<uintptr_t>(a.saved) & 255) != 0)
    return RINGRNN_ERR_WORKSPACE;
  char* w = static_cast<char*>(a.workspace);
  int* status = a.status != nullptr ? a.status : reinterpret_cast<int*>(w);
  w += 1024;
  __nv_bfloat16* WstT = reinterpret_cast<__nv_bfloat16*>(w);
  w += align_up((size_t)l.KX * l.NP * 2, 1024);
  __nv_bfloat16* Delta = reinterpret_cast<__nv_bfloat16*>(w);
  w += align_up((size_t)p.T * l.BP * l.NP * 2, 1024);
  float* g = reinterpret_cast<float*>(w);
  w += align_up((size_t)l.BP * l.NP * 4, 1024);
  float* sum_delta = reinterpret_cast<float*>(w);
  w += align_up((size_t)l.BP * 4, 1024);
  float* zpart = reinterpret_cast<float*>(w);
  w += align_up((size_t)l.ns_bwd * l.BP * l.KX * 4, 1024);
  __nv_bfloat16* Xall = reinterpret_cast<__nv_bfloat16*>(w);
  w += align_up((size_t)p.T * l.BP * l.KX * 2, 1024);
  float* dwpart = reinterpret_cast<float*>(w);
  w += align_up((size_t)l.ns_dw * l.NP * l.KX * 4, 1024);
  float* dWst = reinterpret_cast<float*>(w);
  w += align_up((size_t)l.NP * l.KX * 4, 1024);
  float* raw = reinterpret_cast<float*>(w);
  const __nv_bfloat16* Rh = static_cast<const __nv_bfloat16*>(a.saved);
  const __nv_bfloat16* Dh = reinterpret_cast<const __nv_bfloat16*>(static_cast<const char*>(a.saved) +
                                                                    align_up((size_t)(p.T + 1) * l.BP * l.NP * 2, 1024));
  if (a.status == nullptr) RINGRNN_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(int), s));

  const SwCols cols = cols_of(dp);
  {
    LaunchScope ls(K_PREP, s);
    sw_prep_weights_kernel<<<dim3(l.NP, l.blocks), 256, 0, s>>>(p.Wo, dp.Wa, cols, p.J1, p.N, l.NP, l.KX, nullptr, WstT);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  if (a.grad_A != nullptr)
    RINGRNN_CUDA_TRY(cudaMemsetAsync(a.grad_A, 0, sizeof(float) * (size_t)p.B * p.T * p.a_dim, s));

  SwBwd q;
  memset(&q, 0, sizeof(q));
  q.B = p.B; q.T = p.T; q.N = p.N; q.NP = l.NP; q.BP = l.BP; q.a_dim = p.a_dim; q.nsplit = l.ns_bwd;
  q.KX = l.KX; q.J0 = p.J0; q.alpha = p.alpha;
  q.A = p.A; q.grad_output = a.grad_output;
  q.coef_x = a.coef_x; q.coef_y = a.coef_y; q.coef_s = a.coef_s; q.dec_u = a.dec_u; q.dec_v = a.dec_v;
  q.Rh = Rh; q.Dh = Dh; q.partial = zpart; q.g = g; q.sum_delta = sum_delta; q.Delta = Delta;
  q.grad_r_init = a.grad_r_init; q.grad_A = a.grad_A; q.cols = cols;

  {
    LaunchScope ls(K_BWD, s);
    sw_backward_row_kernel<<<l.BP, ROW_THREADS, 0, s>>>(q, -1, p.T - 1);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  for (int t = p.T - 1; t >= 0; --t) {
    // Z_t[BP, KX] = delta_t[BP, NP] x WstT[KX, NP]^T
    int rc = tc_gemm(0, Delta + (size_t)t * l.BP * l.NP, WstT, zpart, nullptr, l.BP, (int)l.KX, l.NP, l.ns_bwd, status, s);
    if (rc != RINGRNN_OK) return rc;
    {
      LaunchScope ls(K_BWD, s);
      sw_backward_row_kernel<<<l.BP, ROW_THREADS, 0, s>>>(q, t, t - 1);
    }
    RINGRNN_CUDA_TRY(cudaGetLastError());
  }
  {
    LaunchScope ls(K_PREP, s);
    sw_build_xall_kernel<<<dim3(l.BP, p.T), 256, 0, s>>>(Rh, p.A, cols, p.B, p.T, p.a_dim, l.NP, l.BP, l.KX, Xall);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  // dWst[NP, KX] = Delta^T [NP, T*BP] x Xall [T*BP, KX]
  int rc = tc_gemm(1, Delta, Xall, dwpart, dWst, l.NP, (int)l.KX, (long long)p.T * l.BP, l.ns_dw, status, s);
  if (rc != RINGRNN_OK) return rc;
  const size_t NN = (size_t)p.N * p.N;
  RINGRNN_CUDA_TRY(cudaMemsetAsync(a.grad_Wa, 0, sizeof(float) * (size_t)p.a_dim * NN, s));
  {
    LaunchScope ls(K_REDUCE, s);
    sw_unpack_dw_kernel<<<296, 256, 0, s>>>(dWst, p.N, l.NP, l.KX, p.J1, cols, a.grad_Wo, a.grad_Wa, raw);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  if (a.grad_J != nullptr) {
    // the dW split-K partials are dead after the reduction inside tc_gemm: their storage serves as scratch
    rc = launch_grad_j(raw, p.Wo, NN, a.grad_J, reinterpret_cast<double*>(dwpart), s);
    if (rc != RINGRNN_OK) return rc;
  }
  return RINGRNN_OK;
}

}  // namespace ringrnn
