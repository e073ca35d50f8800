// bf16 mode of the ring-attractor operator: host orchestration of the tensor-core kernels
// (tc_fwd.cu, tc_bwd.cu, tc_gemm.cu), operand preparation and buffer layouts.
//
// Layouts (NP = N rounded up to 128/256/512/1024, BP = B rounded up to the tile height 128 (256 for CTA pairs), C = NP/128):
//   weights, forward  Wf [C*2*NG*RB, NP] bf16 (NG = 1 weight group for up to two active action columns; with more, the
//                     1 + n_act matrices come in NG = ceil((1+n_act)/3) groups of three and block (q,s,grp) follows
//                     block (q,s,grp-1); described here for NG = 1) (RB = 208, or 224 when CTA pairs are used, i.e. B > 128): block (q,s) rows = {Wo[i,:], Wl[i,:], Wr[i,:] for the 64 neurons i of
//                     sub-slice s of CTA q, a row of ones, zero rows}; columns j >= N zero
//   weights, backward Wb, same shape: rows = {Wo[:,j], Wl[:,j], Wr[:,j] for the 64 neurons j, ones, zeros}
//   saved             Rh [T+1][BP][NP] bf16 row-major (Rh[0] = r_init, Rh[t+1] = r_t; the last slot stays unwritten:
//                     nothing reads r_T) | Dh = F'(re_t) bf16, T*BP*NP elements in 32x32 blocks | sign masks of r_t
//   backward scratch  DL [T*BP][3*NP] bf16 = [delta | L*delta | R*delta] (A operand of the weight-gradient
//                     GEMM) | split-K partials | dWcat [3*NP][NP] fp32
#include <string.h>

#include "tc_recurrent.cuh"

namespace ringrnn {

using namespace tcr;


namespace {

int padded_n(int N) { return N <= 128 ? 128 : (N <= 256 ? 256 : (N <= 512 ? 512 : (N <= 1024 ? 1024 : 0))); }
// CTA pairs (tiles of 256 samples, cta_group::2 MMAs sharing every weight tile) halve the weight stream, but a B200
// keeps at most 15 clusters of 8 CTAs resident against 33 clusters of 4, so for N = 512 the single shape finishes a
// 4096-sample batch in one wave and pairs need two.  Pairs are therefore opt-in (RINGRNN_PAIRS=1), for experiments.
bool use_pairs(int B, int N) {
  static const bool on = getenv("RINGRNN_PAIRS") != nullptr && getenv("RINGRNN_PAIRS")[0] == '1';
  return on && B > 128 && N <= 512;
}
int padded_b(int B, int N, int n_act) {
  return (use_pairs(B, N) && n_act <= 2) ? (B + 255) / 256 * 256 : (B + 127) / 128 * 128;
}
int n_active_of(const RingRnnProblem& p) { return p.n_active < 0 ? p.a_dim : p.n_active; }

struct ActiveCols {
  int n;
  int c[RINGRNN_MAX_ACTIVE];
};

// Wf / Wb blocks, see the header comment.  grid (NP/64 column chunks, C*2*NG blocks), block 256.  Matrix 3*grp + m of
// the list {Wo, Wa[cols[0]], Wa[cols[1]], ...} fills rows [64m, 64m+64) of block (q, s, grp); missing ones are zero.
__global__ void prep_weights_kernel(const float* __restrict__ Wo, const float* __restrict__ Wa, ActiveCols cols, int ng,
                                    int N, int NP, int RB, __nv_bfloat16* __restrict__ Wf,
                                    __nv_bfloat16* __restrict__ Wb) {
  const int blk = blockIdx.y;  // (q*2 + s)*ng + grp
  const int grp = blk % ng;
  const int n_first = (blk / ng) * 64;
  for (int idx = threadIdx.x; idx < RB * 64; idx += blockDim.x) {
    const int rr = idx / 64, k = blockIdx.x * 64 + idx % 64;
    float vf = 0.f, vb = 0.f;
    if (rr < 192) {
      const int mi = 3 * grp + rr / 64, n = n_first + rr % 64;
      const float* W = (mi == 0) ? Wo : (mi - 1 < cols.n ? Wa + (size_t)cols.c[mi - 1] * N * N : nullptr);
      if (W != nullptr && n < N && k < N) {
        vf = W[(size_t)n * N + k];
        vb = W[(size_t)k * N + n];
      }
    } else if (rr == SUM_COL && grp == 0) {
      vf = vb = (k < N) ? 1.f : 0.f;
    }
    const size_t at = ((size_t)blk * RB + rr) * NP + k;
    if (Wf != nullptr) Wf[at] = __float2bfloat16(vf);
    if (Wb != nullptr) Wb[at] = __float2bfloat16(vb);
  }
}

// R0[b][n] = bf16(r_init[b][n]) with zero padding
__global__ void prep_r0_kernel(const float* __restrict__ r_init, int B, int N, int BP, int NP,
                               __nv_bfloat16* __restrict__ R0) {
  const size_t total = (size_t)BP * NP;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int b = (int)(idx / NP), n = (int)(idx % NP);
    R0[idx] = __float2bfloat16((b < B && n < N) ? r_init[(size_t)b * N + n] : 0.f);
  }
}

// dec_{x,y,ta}[b*T + t] = sum over slots of part[slot][k][t][b]
__global__ void dec_reduce_kernel(const float* __restrict__ part, int slots, int B, int T, int BP, float* dec_x,
                                  float* dec_y, float* dec_ta) {
  const size_t total = (size_t)B * T;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(idx / B), b = (int)(idx % B);
    float acc[3] = {0.f, 0.f, 0.f};
    for (int sl = 0; sl < slots; ++sl)
#pragma unroll
      for (int k = 0; k < 3; ++k) acc[k] += part[(((size_t)sl * 3 + k) * T + t) * BP + b];
    const size_t o = (size_t)b * T + t;
    if (dec_x) dec_x[o] = acc[0];
    if (dec_y) dec_y[o] = acc[1];
    if (dec_ta) dec_ta[o] = acc[2];
  }
}

struct Layout {
  int NP, BP, C, RB, tile_rows;
  int n_act, ng;   // active action columns; weight groups of three matrices (1 for up to two columns)
  bool pair;
  size_t w_bytes, r0_bytes, dec_bytes, state_bytes;
};

Layout layout_of(const RingRnnProblem& p) {
  Layout l;
  l.NP = padded_n(p.N);
  l.BP = padded_b(p.B, p.N, n_active_of(p));
  l.C = l.NP / 128;
  l.n_act = n_active_of(p);
  l.ng = l.n_act <= 2 ? 1 : (1 + l.n_act + 2) / 3;
  l.pair = use_pairs(p.B, p.N) && l.ng == 1;
  l.RB = block_rows(l.pair);
  l.tile_rows = l.pair ? 256 : 128;
  l.w_bytes = align_up((size_t)l.C * 2 * l.ng * l.RB * l.NP * 2, 1024);
  // initial state in bf16; with two K rounds (N > 512) two more row blocks through which the CTAs of a cluster
  // exchange the state when none is saved (TcFwdParams::X)
  l.r0_bytes = align_up((size_t)l.BP * l.NP * 2 * (l.NP > 512 ? 3 : 1), 1024);
  l.dec_bytes = align_up((size_t)2 * l.C * 3 * p.T * l.BP * 4, 1024);
  l.state_bytes = align_up((size_t)l.BP * l.NP * 2, 1024);  // one time slot of Rh / Dh
  return l;
}

}  // namespace

// Which bf16 requests the persistent kernels take: N <= 1024 with up to two active action columns; N <= 512 with up to
// RINGRNN_MAX_ACTIVE of them when the batch is large.  A persistent kernel keeps one cluster busy per 128 samples and
// its step time grows with the number of weight groups, so with more than two columns and at most 1024 samples the
// stepwise path (one full-machine GEMM per step, ringrnn_stepwise.cu) is faster (measured on the shapes of the
// reference's published table, B = 256: 0.53 / 0.57 / 0.79 ms against 0.81 / 0.99 / 0.98 ms at N = 256 / 384 / 512),
// while at B = 4096 the persistent kernels win several times over.
// RINGRNN_STEPWISE=1 sends every bf16 request to the stepwise path (for comparisons).
bool bf16_supported(const RingRnnProblem& p) {
  static const bool force_stepwise = getenv("RINGRNN_STEPWISE") != nullptr && getenv("RINGRNN_STEPWISE")[0] == '1';
  if (force_stepwise) return false;
  const int NP = padded_n(p.N), n_act = n_active_of(p);
  if (NP == 0 || p.B < 1 || p.T < 1) return false;
  if (n_act <= 2) return true;
  return NP <= 512 && n_act <= RINGRNN_MAX_ACTIVE && p.B > 1024;
}

// FWD workspace: status(1024) | Wf | R0 | dec partials
size_t bf16_fwd_workspace_bytes(const RingRnnProblem& p) {
  const Layout l = layout_of(p);
  return 1024 + l.w_bytes + l.r0_bytes + l.dec_bytes;
}
// SAVED: Rh[T+1] row-major | Dh[T] blocked | sign masks [T][NP/32][2][BP] uint32
size_t sign_mask_bytes(const RingRnnProblem& p, const Layout& l) {
  return align_up((size_t)p.T * (l.NP / 32) * 2 * l.BP * 4, 1024);
}
// checkpoint interval in force (0 = every step is kept)
int ckpt_interval(const RingRnnProblem& p) { return (p.ckpt_every > 0 && p.ckpt_every < p.T) ? p.ckpt_every : 0; }
size_t ckpt_slot_bytes(const RingRnnProblem& p) { return (size_t)p.B * p.N * sizeof(float); }
size_t saved_every_step_bytes(const RingRnnProblem& p) {
  const Layout l = layout_of(p);
  return (size_t)(2 * p.T + 1) * l.state_bytes + sign_mask_bytes(p, l);
}
// with checkpoints: [ceil(T/K)][B][N] fp32 states (slot 0 = r_init)
size_t bf16_saved_bytes(const RingRnnProblem& p) {
  const int K = ckpt_interval(p);
  if (K == 0) return saved_every_step_bytes(p);
  return align_up((size_t)((p.T + K - 1) / K) * ckpt_slot_bytes(p), 1024);
}


int bf16_forward(const RingRnnFwdArgs& a, const DevProblem& dp, cudaStream_t s) {
  const RingRnnProblem& p = a.p;
  const Layout l = layout_of(p);
  if (a.workspace == nullptr || a.workspace_bytes < bf16_fwd_workspace_bytes(p)) return RINGRNN_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(a.workspace) & 255) != 0) return RINGRNN_ERR_WORKSPACE;
  const bool train = a.saved != nullptr;
  if (train && (a.saved_bytes < bf16_saved_bytes(p) || (reinterpret_cast<uintptr_t>(a.saved) & 255) != 0))
    return RINGRNN_ERR_WORKSPACE;
  char* w = static_cast<char*>(a.workspace);
  int* status = a.status != nullptr ? a.status : reinterpret_cast<int*>(w);
  __nv_bfloat16* Wf = reinterpret_cast<__nv_bfloat16*>(w + 1024);
  __nv_bfloat16* R0 = reinterpret_cast<__nv_bfloat16*>(w + 1024 + l.w_bytes);
  float* dec_part = reinterpret_cast<float*>(w + 1024 + l.w_bytes + l.r0_bytes);
  const int K = train ? ckpt_interval(p) : 0;
  const bool keep_all = train && K == 0;
  __nv_bfloat16* Rh = keep_all ? static_cast<__nv_bfloat16*>(a.saved) : nullptr;
  __nv_bfloat16* Dh = keep_all ? Rh + (size_t)(p.T + 1) * l.BP * l.NP : nullptr;
  uint32_t* Sg = keep_all ? reinterpret_cast<uint32_t*>(static_cast<char*>(a.saved) + (size_t)(2 * p.T + 1) * l.state_bytes)
                          : nullptr;
  if (keep_all) R0 = Rh;  // slot 0 of the saved state doubles as the initial A operand
  if (K > 0)              // checkpoint 0 is the initial state
    RINGRNN_CUDA_TRY(cudaMemcpyAsync(a.saved, p.r_init, ckpt_slot_bytes(p), cudaMemcpyDeviceToDevice, s));

  if (a.status == nullptr) RINGRNN_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(int), s));
  ActiveCols ac;
  ac.n = dp.n_mat - 1;
  for (int k = 0; k < ac.n; ++k) ac.c[k] = dp.cols[k];
  {
    LaunchScope ls(K_PREP, s);
    prep_weights_kernel<<<dim3(l.NP / 64, l.C * 2 * l.ng), 256, 0, s>>>(p.Wo, dp.Wa, ac, l.ng, p.N, l.NP, l.RB, Wf, nullptr);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  {
    LaunchScope ls(K_PREP, s);
    prep_r0_kernel<<<296, 256, 0, s>>>(p.r_init, p.B, p.N, l.BP, l.NP, R0);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());

  CUtensorMap tmW, tmR0;
  if (!make_tmap_bf16_2d(&tmW, Wf, (uint64_t)l.C * 2 * l.ng * l.RB, (uint64_t)l.NP, l.pair ? l.RB / 2 : l.RB, 64))
    return RINGRNN_ERR_CUDA;
  // one map serves the initial-state loads (rows [0, BP)) and, in training, the saved-state stores (rows up to T*BP)
  const bool two_rounds = l.NP > 512;
  if (!make_tmap_bf16_2d(&tmR0, R0, (uint64_t)(keep_all ? p.T + 1 : (two_rounds ? 3 : 1)) * l.BP, (uint64_t)l.NP, 128, 64))
    return RINGRNN_ERR_CUDA;

  const bool want_dec = a.dec_x || a.dec_y || a.dec_ta;
  TcFwdParams fp;
  memset(&fp, 0, sizeof(fp));
  fp.B = p.B; fp.T = p.T; fp.N = p.N; fp.BP = l.BP; fp.a_dim = p.a_dim;
  fp.colL = dp.n_mat > 1 ? dp.cols[0] : -1;
  fp.colR = dp.n_mat > 2 ? dp.cols[1] : -1;
  fp.ng = l.ng; fp.n_act = ac.n;
  for (int k = 0; k < ac.n; ++k) fp.cols[k] = ac.c[k];
  fp.n_tiles = l.BP / l.tile_rows;
  fp.J0 = p.J0; fp.J1 = p.J1; fp.alpha = p.alpha;
  fp.A = p.A; fp.r_init = p.r_init;
  fp.Rh = Rh; fp.Dh = Dh; fp.Sg = Sg;
  fp.X = two_rounds ? R0 : nullptr;  // (= Rh when every step is kept)
  fp.x_ring = keep_all ? 0 : 1;
  fp.hist = a.bump_history;
  fp.dec_part = want_dec ? dec_part : nullptr;
  fp.dec_u = a.dec_u; fp.dec_v = a.dec_v;
  fp.final_state = a.final_state;
  fp.status = status;
  fp.t0 = 0; fp.T_total = p.T;
  fp.ckpt = K > 0 ? static_cast<float*>(a.saved) : nullptr;
  fp.ckpt_every = K;
  int rc = tc_forward_launch(p.activation, l.NP, l.pair, tmW, tmR0, fp, s);
  if (rc != RINGRNN_OK) return rc;
  if (want_dec) {
    LaunchScope ls(K_LOSS, s);
    dec_reduce_kernel<<<296, 256, 0, s>>>(dec_part, 2 * l.C, p.B, p.T, l.BP, a.dec_x, a.dec_y, a.dec_ta);
    RINGRNN_CUDA_TRY(cudaGetLastError());
  }
  return RINGRNN_OK;
}

// ---- backward ------------------------------------------------------------------------------------------

namespace {

// dWcat [(1+n)*NP][NP] -> grad_Wo = J1 * block 0, grad_Wa[cols[k]] = block 1 + k (unpadded);
// raw = block 0 unscaled and unpadded (for the J0 / J1 gradients)
__global__ void unpack_dw_kernel(const float* __restrict__ dWcat, int N, int NP, float J1, ActiveCols cols,
                                 float* grad_Wo, float* grad_Wa, float* raw) {
  const size_t NN = (size_t)N * N;
  for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < NN; e += (size_t)gridDim.x * blockDim.x) {
    const int i = (int)(e / N), j = (int)(e % N);
    const float g0 = dWcat[(size_t)i * NP + j];
    grad_Wo[e] = J1 * g0;
    raw[e] = g0;
    for (int k = 0; k < cols.n; ++k) grad_Wa[(size_t)cols.c[k] * NN + e] = dWcat[((size_t)(1 + k) * NP + i) * NP + j];
  }
}

int gemm_splits(const Layout& l, int T) {
  const int blocks = l.ng == 1 ? 3 : 1 + l.n_act;  // column blocks of DL = row blocks of dWcat
  const int tiles = (blocks * l.NP / 128) * (l.NP > 512 ? l.NP / 512 : 1);
  int ns = 148 / tiles;
  const long long K = (long long)T * l.BP;
  while (ns > 1 && K / ns < 256) --ns;
  return ns < 1 ? 1 : ns;
}

struct BwdLayout {
  size_t w_bytes, dl_bytes, partial_bytes, dw_bytes, raw_bytes, da_bytes;
  int nsplit, blocks, da_slots, da_per_slot;
};

// grad_A[b,t,cols[k]] = sum over slots of part[slot][k][t][b]   (`per_slot` entries k per slot, of which the first
// cols.n are used)
// (`part` covers the T steps that start at step t0 of a sequence of T_total)
__global__ void da_reduce_kernel(const float* __restrict__ part, int slots, int per_slot, int B, int T, int BP, int a_dim,
                                 ActiveCols cols, float* grad_A, int t0, int T_total) {
  const size_t total = (size_t)B * T;
  for (size_t idx = blockIdx.x * (size_t)blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const int t = (int)(idx / B), b = (int)(idx % B);
    float* o = grad_A + ((size_t)b * T_total + t0 + t) * a_dim;
    for (int k = 0; k < cols.n; ++k) {
      float acc = 0.f;
      for (int sl = 0; sl < slots; ++sl) acc += part[(((size_t)sl * per_slot + k) * T + t) * BP + b];
      o[cols.c[k]] = acc;
    }
  }
}

BwdLayout bwd_layout_of(const RingRnnProblem& p, const Layout& l) {
  BwdLayout b;
  b.nsplit = gemm_splits(l, p.T);
  b.w_bytes = l.w_bytes;
  b.blocks = l.ng == 1 ? 3 : 1 + l.n_act;
  b.dl_bytes = align_up((size_t)p.T * l.BP * b.blocks * l.NP * 2, 1024);
  b.partial_bytes = align_up((size_t)b.nsplit * b.blocks * l.NP * l.NP * 4, 1024);
  b.dw_bytes = align_up((size_t)b.blocks * l.NP * l.NP * 4, 1024);
  b.raw_bytes = align_up((size_t)p.N * p.N * 4, 1024);
  // dL/dA partial sums: [2C][2] (up to two columns) or [4C][n_act] entries of T*BP floats
  b.da_slots = l.ng == 1 ? 2 * l.C : 4 * l.C;
  b.da_per_slot = l.ng == 1 ? 2 : l.n_act;
  b.da_bytes = align_up((size_t)b.da_slots * b.da_per_slot * p.T * l.BP * 4, 1024);
  return b;
}

}  // namespace

// BWD workspace: status(1024) | Wb | DL | split-K partials | dWcat | raw | dL/dA partials
size_t bf16_bwd_workspace_bytes(const RingRnnProblem& p) {
  const Layout l = layout_of(p);
  const int K = ckpt_interval(p);
  if (K > 0) {
    // with checkpoints: status | Wb | Wf | saved tensors of one stretch | DL, split-K partials, dW of one stretch |
    //                   dWcat | raw | dL/dA partials of one stretch | two carry buffers
    RingRnnProblem pc = p;
    pc.T = K;
    pc.ckpt_every = 0;
    const BwdLayout b = bwd_layout_of(pc, l);
    return 1024 + 2 * b.w_bytes + align_up(saved_every_step_bytes(pc), 1024) + b.dl_bytes + b.partial_bytes +
           2 * b.dw_bytes + b.raw_bytes + b.da_bytes + 2 * align_up(ckpt_slot_bytes(p), 1024);
  }
  const BwdLayout b = bwd_layout_of(p, l);
  return 1024 + b.w_bytes + b.dl_bytes + b.partial_bytes + b.dw_bytes + b.raw_bytes + b.da_bytes;
}

namespace {

// out[e] = first ? in[e] : out[e] + in[e]
__global__ void accumulate_kernel(float* __restrict__ out, const float* __restrict__ in, size_t n, int first) {
  for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x)
    out[e] = first ? in[e] : out[e] + in[e];
}

// Backward with checkpoints: the stretches of K steps are taken last to first; each is recomputed from its fp32
// checkpoint by the forward kernel (which saves state, derivative history and sign masks of the stretch exactly as
// the keep-everything forward would have), then the reverse-time kernel runs through it, starting from the gradient
// the later stretch handed back, and the stretch's weight-gradient GEMM is added to the total.
int bf16_backward_ckpt(const RingRnnBwdArgs& a, const DevProblem& dp, cudaStream_t s, int K) {
  const RingRnnProblem& p = a.p;
  const Layout l = layout_of(p);
  RingRnnProblem pc = p;
  pc.T = K;
  pc.ckpt_every = 0;
  const BwdLayout bl = bwd_layout_of(pc, l);
  char* w = static_cast<char*>(a.workspace);
  int* status = a.status != nullptr ? a.status : reinterpret_cast<int*>(w);
  w += 1024;
  __nv_bfloat16* Wb = reinterpret_cast<__nv_bfloat16*>(w);
  w += bl.w_bytes;
  __nv_bfloat16* Wf = reinterpret_cast<__nv_bfloat16*>(w);
  w += bl.w_bytes;
  char* savedc = w;
  w += align_up(saved_every_step_bytes(pc), 1024);
  __nv_bfloat16* DL = reinterpret_cast<__nv_bfloat16*>(w);
  w += bl.dl_bytes;
  float* partial = reinterpret_cast<float*>(w);
  w += bl.partial_bytes;
  float* dWchunk = reinterpret_cast<float*>(w);
  w += bl.dw_bytes;
  float* dWcat = reinterpret_cast<float*>(w);
  w += bl.dw_bytes;
  float* raw = reinterpret_cast<float*>(w);
  w += bl.raw_bytes;
  float* dA_part = reinterpret_cast<float*>(w);
  w += bl.da_bytes;
  float* carry[2];
  carry[0] = reinterpret_cast<float*>(w);
  carry[1] = reinterpret_cast<float*>(w + align_up(ckpt_slot_bytes(p), 1024));
  const float* ckpt = static_cast<const float*>(a.saved);

  if (a.status == nullptr) RINGRNN_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(int), s));
  ActiveCols ac;
  ac.n = dp.n_mat - 1;
  for (int k = 0; k < ac.n; ++k) ac.c[k] = dp.cols[k];
  {
    LaunchScope ls(K_PREP, s);
    prep_weights_kernel<<<dim3(l.NP / 64, l.C * 2 * l.ng), 256, 0, s>>>(p.Wo, dp.Wa, ac, l.ng, p.N, l.NP, l.RB, Wf, Wb);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  CUtensorMap tmWf, tmWb;
  if (!make_tmap_bf16_2d(&tmWf, Wf, (uint64_t)l.C * 2 * l.ng * l.RB, (uint64_t)l.NP, l.pair ? l.RB / 2 : l.RB, 64) ||
      !make_tmap_bf16_2d(&tmWb, Wb, (uint64_t)l.C * 2 * l.ng * l.RB, (uint64_t)l.NP, l.pair ? l.RB / 2 : l.RB, 64))
    return RINGRNN_ERR_CUDA;
  if (a.grad_A != nullptr)
    RINGRNN_CUDA_TRY(cudaMemsetAsync(a.grad_A, 0, sizeof(float) * (size_t)p.B * p.T * p.a_dim, s));

  const int n_ck = (p.T + K - 1) / K;
  for (int c = n_ck - 1; c >= 0; --c) {
    const int t0 = c * K, Tc = (p.T - t0 < K) ? p.T - t0 : K;
    const float* state0 = ckpt + (size_t)c * p.B * p.N;
    // saved tensors of the stretch, laid out as for a sequence of Tc steps
    __nv_bfloat16* Rh = reinterpret_cast<__nv_bfloat16*>(savedc);
    __nv_bfloat16* Dh = Rh + (size_t)(Tc + 1) * l.BP * l.NP;
    uint32_t* Sg = reinterpret_cast<uint32_t*>(savedc + (size_t)(2 * Tc + 1) * l.state_bytes);
    {
      LaunchScope ls(K_PREP, s);
      prep_r0_kernel<<<296, 256, 0, s>>>(state0, p.B, p.N, l.BP, l.NP, Rh);
    }
    RINGRNN_CUDA_TRY(cudaGetLastError());
    CUtensorMap tmR0, tmDL, tmDL32;
    if (!make_tmap_bf16_2d(&tmR0, Rh, (uint64_t)(Tc + 1) * l.BP, (uint64_t)l.NP, 128, 64) ||
        !make_tmap_bf16_2d(&tmDL, DL, (uint64_t)Tc * l.BP, (uint64_t)bl.blocks * l.NP, 128, 64) ||
        !make_tmap_bf16_2d(&tmDL32, DL, (uint64_t)Tc * l.BP, (uint64_t)bl.blocks * l.NP, 32, 32, 64))
      return RINGRNN_ERR_CUDA;

    TcFwdParams fp;
    memset(&fp, 0, sizeof(fp));
    fp.B = p.B; fp.T = Tc; fp.N = p.N; fp.BP = l.BP; fp.a_dim = p.a_dim;
    fp.colL = dp.n_mat > 1 ? dp.cols[0] : -1;
    fp.colR = dp.n_mat > 2 ? dp.cols[1] : -1;
    fp.ng = l.ng; fp.n_act = ac.n;
    for (int k = 0; k < ac.n; ++k) fp.cols[k] = ac.c[k];
    fp.n_tiles = l.BP / l.tile_rows;
    fp.J0 = p.J0; fp.J1 = p.J1; fp.alpha = p.alpha;
    fp.A = p.A; fp.r_init = state0;
    fp.Rh = Rh; fp.Dh = Dh; fp.Sg = Sg;
    fp.X = l.NP > 512 ? Rh : nullptr;
    fp.x_ring = 0;
    fp.status = status;
    fp.t0 = t0; fp.T_total = p.T;
    int rc = tc_forward_launch(p.activation, l.NP, l.pair, tmWf, tmR0, fp, s);
    if (rc != RINGRNN_OK) return rc;

    TcBwdParams bp;
    memset(&bp, 0, sizeof(bp));
    bp.B = p.B; bp.T = Tc; bp.N = p.N; bp.BP = l.BP; bp.a_dim = p.a_dim;
    bp.colL = fp.colL; bp.colR = fp.colR;
    bp.ng = l.ng; bp.n_act = ac.n;
    for (int k = 0; k < ac.n; ++k) bp.cols[k] = ac.c[k];
    bp.n_tiles = fp.n_tiles;
    bp.J0 = p.J0; bp.J1 = p.J1; bp.alpha = p.alpha;
    bp.A = p.A; bp.Dh = Dh; bp.Sg = Sg;
    bp.grad_output = a.grad_output;
    bp.coef_x = a.coef_x; bp.coef_y = a.coef_y; bp.coef_s = a.coef_s;
    bp.dec_u = a.dec_u; bp.dec_v = a.dec_v;
    bp.DL = DL;
    bp.grad_r_init = (c == 0) ? a.grad_r_init : carry[c & 1];
    bp.Rh = Rh;
    bp.dA_part = a.grad_A != nullptr ? dA_part : nullptr;
    bp.status = status;
    bp.t0 = t0; bp.T_total = p.T;
    bp.carry_in = (c == n_ck - 1) ? nullptr : carry[(c + 1) & 1];
    rc = tc_backward_launch(l.NP, l.pair, tmWb, tmDL, tmDL32, bp, s);
    if (rc != RINGRNN_OK) return rc;

    if (a.grad_A != nullptr) {
      LaunchScope ls(K_REDUCE, s);
      da_reduce_kernel<<<296, 256, 0, s>>>(dA_part, bl.da_slots, bl.da_per_slot, p.B, Tc, l.BP, p.a_dim, ac, a.grad_A, t0,
                                           p.T);
      RINGRNN_CUDA_TRY(cudaGetLastError());
    }
    rc = tc_gemm(1, DL, Rh, partial, dWchunk, bl.blocks * l.NP, l.NP, (long long)Tc * l.BP, gemm_splits(l, Tc), status, s);
    if (rc != RINGRNN_OK) return rc;
    {
      LaunchScope ls(K_REDUCE, s);
      accumulate_kernel<<<296, 256, 0, s>>>(dWcat, dWchunk, (size_t)bl.blocks * l.NP * l.NP, c == n_ck - 1 ? 1 : 0);
    }
    RINGRNN_CUDA_TRY(cudaGetLastError());
  }
  const size_t NN = (size_t)p.N * p.N;
  RINGRNN_CUDA_TRY(cudaMemsetAsync(a.grad_Wa, 0, sizeof(float) * (size_t)p.a_dim * NN, s));
  {
    LaunchScope ls(K_REDUCE, s);
    unpack_dw_kernel<<<296, 256, 0, s>>>(dWcat, p.N, l.NP, p.J1, ac, a.grad_Wo, a.grad_Wa, raw);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  if (a.grad_J != nullptr) {
    int rc = launch_grad_j(raw, p.Wo, NN, a.grad_J, reinterpret_cast<double*>(partial), s);
    if (rc != RINGRNN_OK) return rc;
  }
  return RINGRNN_OK;
}

}  // namespace


int bf16_backward(const RingRnnBwdArgs& a, const DevProblem& dp, cudaStream_t s) {
  const RingRnnProblem& p = a.p;
  const Layout l = layout_of(p);
  const BwdLayout bl = bwd_layout_of(p, l);
  if (a.workspace == nullptr || a.workspace_bytes < bf16_bwd_workspace_bytes(p)) return RINGRNN_ERR_WORKSPACE;
  if ((reinterpret_cast<uintptr_t>(a.workspace) & 255) != 0) return RINGRNN_ERR_WORKSPACE;
  if (a.saved == nullptr || a.saved_bytes < bf16_saved_bytes(p) || (reinterpret_cast<uintptr_t>(a.saved) & 255) != 0)
    return RINGRNN_ERR_WORKSPACE;
  if (ckpt_interval(p) > 0) return bf16_backward_ckpt(a, dp, s, ckpt_interval(p));
  char* w = static_cast<char*>(a.workspace);
  int* status = a.status != nullptr ? a.status : reinterpret_cast<int*>(w);
  w += 1024;
  __nv_bfloat16* Wb = reinterpret_cast<__nv_bfloat16*>(w);
  w += bl.w_bytes;
  __nv_bfloat16* DL = reinterpret_cast<__nv_bfloat16*>(w);
  w += bl.dl_bytes;
  float* partial = reinterpret_cast<float*>(w);
  w += bl.partial_bytes;
  float* dWcat = reinterpret_cast<float*>(w);
  w += bl.dw_bytes;
  float* raw = reinterpret_cast<float*>(w);
  w += bl.raw_bytes;
  float* dA_part = reinterpret_cast<float*>(w);
  const __nv_bfloat16* Rh = static_cast<const __nv_bfloat16*>(a.saved);
  const __nv_bfloat16* Dh = Rh + (size_t)(p.T + 1) * l.BP * l.NP;

  if (a.status == nullptr) RINGRNN_CUDA_TRY(cudaMemsetAsync(status, 0, sizeof(int), s));
  const int colL = dp.n_mat > 1 ? dp.cols[0] : -1, colR = dp.n_mat > 2 ? dp.cols[1] : -1;
  ActiveCols ac;
  ac.n = dp.n_mat - 1;
  for (int k = 0; k < ac.n; ++k) ac.c[k] = dp.cols[k];
  {
    LaunchScope ls(K_PREP, s);
    prep_weights_kernel<<<dim3(l.NP / 64, l.C * 2 * l.ng), 256, 0, s>>>(p.Wo, dp.Wa, ac, l.ng, p.N, l.NP, l.RB, nullptr, Wb);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  CUtensorMap tmW;
  if (!make_tmap_bf16_2d(&tmW, Wb, (uint64_t)l.C * 2 * l.ng * l.RB, (uint64_t)l.NP, l.pair ? l.RB / 2 : l.RB, 64))
    return RINGRNN_ERR_CUDA;

  TcBwdParams bp;
  memset(&bp, 0, sizeof(bp));
  bp.B = p.B; bp.T = p.T; bp.N = p.N; bp.BP = l.BP; bp.a_dim = p.a_dim;
  bp.colL = colL; bp.colR = colR;
  bp.ng = l.ng; bp.n_act = ac.n;
  for (int k = 0; k < ac.n; ++k) bp.cols[k] = ac.c[k];
  bp.n_tiles = l.BP / l.tile_rows;
  bp.J0 = p.J0; bp.J1 = p.J1; bp.alpha = p.alpha;
  bp.A = p.A; bp.Dh = Dh;
  bp.Sg = reinterpret_cast<const uint32_t*>(static_cast<const char*>(a.saved) + (size_t)(2 * p.T + 1) * l.state_bytes);
  bp.grad_output = a.grad_output;
  bp.coef_x = a.coef_x; bp.coef_y = a.coef_y; bp.coef_s = a.coef_s;
  bp.dec_u = a.dec_u; bp.dec_v = a.dec_v;
  bp.DL = DL;
  bp.grad_r_init = a.grad_r_init;
  bp.Rh = Rh;
  bp.dA_part = a.grad_A != nullptr ? dA_part : nullptr;
  bp.status = status;
  bp.t0 = 0; bp.T_total = p.T;
  CUtensorMap tmDL, tmDL32;
  if (!make_tmap_bf16_2d(&tmDL, DL, (uint64_t)p.T * l.BP, (uint64_t)bl.blocks * l.NP, 128, 64) ||
      !make_tmap_bf16_2d(&tmDL32, DL, (uint64_t)p.T * l.BP, (uint64_t)bl.blocks * l.NP, 32, 32, 64))
    return RINGRNN_ERR_CUDA;
  int rc = tc_backward_launch(l.NP, l.pair, tmW, tmDL, tmDL32, bp, s);
  if (rc != RINGRNN_OK) return rc;

  if (a.grad_A != nullptr) {
    RINGRNN_CUDA_TRY(cudaMemsetAsync(a.grad_A, 0, sizeof(float) * (size_t)p.B * p.T * p.a_dim, s));
    LaunchScope ls(K_REDUCE, s);
    da_reduce_kernel<<<296, 256, 0, s>>>(dA_part, bl.da_slots, bl.da_per_slot, p.B, p.T, l.BP, p.a_dim, ac, a.grad_A, 0,
                                         p.T);
    RINGRNN_CUDA_TRY(cudaGetLastError());
  }
  // dWcat[blocks*NP, NP] = DL^T [blocks*NP, T*BP] x Rh[0..T) [T*BP, NP]
  rc = tc_gemm(1, DL, Rh, partial, dWcat, bl.blocks * l.NP, l.NP, (long long)p.T * l.BP, bl.nsplit, status, s);
  if (rc != RINGRNN_OK) return rc;
  const size_t NN = (size_t)p.N * p.N;
  RINGRNN_CUDA_TRY(cudaMemsetAsync(a.grad_Wa, 0, sizeof(float) * (size_t)p.a_dim * NN, s));
  {
    LaunchScope ls(K_REDUCE, s);
    unpack_dw_kernel<<<296, 256, 0, s>>>(dWcat, p.N, l.NP, p.J1, ac, a.grad_Wo, a.grad_Wa, raw);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  if (a.grad_J != nullptr) {
    // the split-K partials are dead after the reduction inside tc_gemm: their storage serves as scratch
    rc = launch_grad_j(raw, p.Wo, NN, a.grad_J, reinterpret_cast<double*>(partial), s);
    if (rc != RINGRNN_OK) return rc;
  }
  return RINGRNN_OK;
}

}  // namespace ringrnn
