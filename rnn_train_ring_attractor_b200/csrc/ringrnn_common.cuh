// Shared device/host helpers of libringrnn: status plumbing, activations, small utilities.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stddef.h>

#include "ringrnn.h"

namespace ringrnn {

// ---- host-side error plumbing -------------------------------------------------------------
// The reference prints and calls std::exit on any CUDA error (cpp/cuda_common.cuh:30-39); here the
// error is remembered per host thread and turned into a status code.
void set_last_cuda_error(cudaError_t e);

#define RINGRNN_CUDA_TRY(expr)                         \
  do {                                                 \
    cudaError_t _e = (expr);                           \
    if (_e != cudaSuccess) {                           \
      ::ringrnn::set_last_cuda_error(_e);              \
      return RINGRNN_ERR_CUDA;                         \
    }                                                  \
  } while (0)

// ---- launch accounting / optional per-kernel event timing ---------------------------------
enum KernelSlot { K_PREP = 0, K_FWD = 1, K_BWD = 2, K_DW = 3, K_REDUCE = 4, K_LOSS = 5, K_SLOTS = 6 };
// Construct right before a kernel launch and let it go out of scope right after: counts the launch and,
// when timing is enabled, records an event pair around it on `s`.
struct LaunchScope {
  LaunchScope(int slot, cudaStream_t s);
  ~LaunchScope();
  int slot_;
  cudaStream_t s_;
  cudaEvent_t start_;
  bool timed_;
};

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// ---- activations (numerical contract: cpp/cuda_common.cuh:56-89) ------------------------
// F and F' are evaluated with the accurate libdevice functions; the tensor-core kernels have their
// own cheaper evaluations with error well inside bf16 resolution.
template <int ACT>
__device__ __forceinline__ float act_fn(float x) {
  if constexpr (ACT == RINGRNN_ACT_RELU) {
    return fmaxf(x, 0.f);
  } else if constexpr (ACT == RINGRNN_ACT_GELU) {
    return x * normcdff(x);
  } else if constexpr (ACT == RINGRNN_ACT_SILU) {
    return x / (1.f + expf(-x));
  } else {
    return tanhf(x);
  }
}

template <int ACT>
__device__ __forceinline__ float act_grad(float x) {
  if constexpr (ACT == RINGRNN_ACT_RELU) {
    return x > 0.f ? 1.f : 0.f;
  } else if constexpr (ACT == RINGRNN_ACT_GELU) {
    // d/dx [x Phi(x)] = Phi(x) + x phi(x)
    return normcdff(x) + x * 0.3989422804014327f * expf(-0.5f * x * x);
  } else if constexpr (ACT == RINGRNN_ACT_SILU) {
    const float s = 1.f / (1.f + expf(-x));
    return s * (1.f + x * (1.f - s));
  } else {
    const float y = tanhf(x);
    return 1.f - y * y;
  }
}

// Problem description as the kernels see it (plain data, passed by value).
struct DevProblem {
  int B, T, N, a_dim;
  float J0, J1, alpha;
  const float* A;       // [B,T,a_dim]
  const float* Wa;      // [a_dim,N,N]
  const float* Wo;      // [N,N]
  const float* r_init;  // [B,N]
  int n_mat;            // 1 + number of active action columns
  int all_cols;         // non-zero: every column of A is active, column k is k (cols[] unused; a_dim may exceed its size)
  int cols[RINGRNN_MAX_ACTIVE];  // active action columns
};
// the k-th active action column
__host__ __device__ __forceinline__ int active_col(const DevProblem& p, int k) { return p.all_cols ? k : p.cols[k]; }

// Deferred report of a bounded device-side wait that ran out: queues a copy of the kernels' status word into pinned
// host memory behind them on `s` (no synchronisation); the next ringrnn_fwd / ringrnn_bwd / ringrnn_device_status call
// on this process looks at the words that have arrived.
int queue_status_report(const int* dev_status, cudaStream_t s);

// dJ0 / dJ1 from the unscaled Wo gradient (ringrnn_fp32.cu); scratch: GRAD_J_BLOCKS * 2 doubles
constexpr int GRAD_J_BLOCKS = 128;
int launch_grad_j(const float* raw, const float* Wo, size_t NN, float* grad_J, double* scratch, cudaStream_t s);

// fp32 (CUDA-core) path ----------------------------------------------------------------------
size_t fp32_fwd_workspace_bytes(const RingRnnProblem& p);
size_t fp32_saved_bytes(const RingRnnProblem& p, int history_given);
size_t fp32_bwd_workspace_bytes(const RingRnnProblem& p);
int fp32_forward(const RingRnnFwdArgs& a, const DevProblem& dp, cudaStream_t s);
int fp32_backward(const RingRnnBwdArgs& a, const DevProblem& dp, cudaStream_t s);

// split-K bf16 tensor-core GEMM (tc_gemm.cu); see there for the argument contract
int tc_gemm(int mn_major, const void* A, const void* B, float* partial, float* out, int M, int N, long long K,
            int nsplit, int* status, cudaStream_t s);

int tc_gemm_pair(const void* A, const void* B, float* out, int M, int N, long long K, int* status, cudaStream_t s);

// bf16 tensor-core path ----------------------------------------------------------------------
bool bf16_supported(const RingRnnProblem& p);
size_t bf16_fwd_workspace_bytes(const RingRnnProblem& p);
size_t bf16_saved_bytes(const RingRnnProblem& p);
size_t bf16_bwd_workspace_bytes(const RingRnnProblem& p);
int bf16_forward(const RingRnnFwdArgs& a, const DevProblem& dp, cudaStream_t s);
int bf16_backward(const RingRnnBwdArgs& a, const DevProblem& dp, cudaStream_t s);

// bf16 stepwise path: one tensor-core GEMM per timestep (ringrnn_stepwise.cu), for the shapes the persistent
// kernels do not take
bool stepwise_supported(const RingRnnProblem& p);
size_t stepwise_fwd_workspace_bytes(const RingRnnProblem& p);
size_t stepwise_saved_bytes(const RingRnnProblem& p);
size_t stepwise_bwd_workspace_bytes(const RingRnnProblem& p);
int stepwise_forward(const RingRnnFwdArgs& a, const DevProblem& dp, cudaStream_t s);
int stepwise_backward(const RingRnnBwdArgs& a, const DevProblem& dp, cudaStream_t s);

}  // namespace ringrnn
