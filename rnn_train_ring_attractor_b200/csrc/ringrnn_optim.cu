// Optimizer step on the flat parameter / gradient buffers: clip-by-global-norm followed by Adam, on the device, with
// no host synchronisation.  The reference does this with torch.nn.utils.clip_grad_norm_(params, 1.0) and
// torch.optim.Adam (train_general_ring_no_gain.py:335-336), which read the norm back to the host every step.
// Same arithmetic as those two calls (L2 norm over all gradients, coefficient max_norm / (norm + 1e-6) clamped to 1;
// Adam without weight decay or amsgrad, bias-corrected).  The norm is summed in double precision in a fixed order:
// bit-reproducible.
#include <math.h>

#include "ringrnn_common.cuh"

namespace ringrnn {

namespace {

constexpr int NORM_BLOCKS = 128;

// scratch[b] = sum of g^2 over block b's grid-stride share
__global__ void grad_sq_partial_kernel(const float* __restrict__ g, size_t n, double* __restrict__ scratch) {
  __shared__ double red[256];
  double acc = 0.0;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const double v = g[i];
    acc += v * v;
  }
  red[threadIdx.x] = acc;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if ((int)threadIdx.x < o) red[threadIdx.x] += red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) scratch[blockIdx.x] = red[0];
}

__global__ void clip_adam_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                 float* __restrict__ v, size_t n, float lr, float beta1, float beta2, float eps,
                                 float step_size, float bias2_sqrt, float max_norm, double* __restrict__ scratch) {
  __shared__ float coef_s;
  if (threadIdx.x == 0) {
    double tot = 0.0;
    for (int b = 0; b < NORM_BLOCKS; ++b) tot += scratch[b];
    const double norm = sqrt(tot);
    float coef = 1.f;
    if (max_norm > 0.f) {
      coef = (float)((double)max_norm / (norm + 1e-6));
      coef = coef < 1.f ? coef : 1.f;
    }
    coef_s = coef;
    if (blockIdx.x == 0) scratch[NORM_BLOCKS] = norm;  // for the caller's log
  }
  __syncthreads();
  const float coef = coef_s;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float gi = g[i] * coef;
    const float mi = beta1 * m[i] + (1.f - beta1) * gi;
    const float vi = beta2 * v[i] + (1.f - beta2) * gi * gi;
    m[i] = mi;
    v[i] = vi;
    const float denom = sqrtf(vi) / bias2_sqrt + eps;
    p[i] -= step_size * (mi / denom);
  }
}

}  // namespace
}  // namespace ringrnn

extern "C" int ringrnn_clip_adam(float* params, const float* grads, float* exp_avg, float* exp_avg_sq, size_t n,
                                 float lr, float beta1, float beta2, float eps, int step, float max_norm,
                                 double* scratch, void* stream) {
  using namespace ringrnn;
  if (!params || !grads || !exp_avg || !exp_avg_sq || !scratch || step < 1) return RINGRNN_ERR_ARG;
  if (n == 0) return RINGRNN_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  {
    LaunchScope ls(K_REDUCE, s);
    grad_sq_partial_kernel<<<NORM_BLOCKS, 256, 0, s>>>(grads, n, scratch);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  // bias corrections in double on the host and rounded once, as torch.optim.Adam computes them (Python floats)
  const double bias1 = 1.0 - pow((double)beta1, (double)step);
  const float step_size = (float)((double)lr / bias1);
  const float bias2_sqrt = (float)sqrt(1.0 - pow((double)beta2, (double)step));
  {
    LaunchScope ls(K_REDUCE, s);
    clip_adam_kernel<<<296, 256, 0, s>>>(params, grads, exp_avg, exp_avg_sq, n, lr, beta1, beta2, eps, step_size, bias2_sqrt,
                                        max_norm, scratch);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  return RINGRNN_OK;
}
