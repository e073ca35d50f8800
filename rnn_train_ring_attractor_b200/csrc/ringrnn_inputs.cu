// Synthetic angular-velocity trials generated on the device, so that a training or roll-out step needs no host->device
// copy of its inputs (C5-sized roll-outs would otherwise copy 2.1 GB per call).
//
// What the reference generates on the host (utils/generate_av_integration_data.py:11-58) and turns into the operator's
// inputs (train_general_ring_no_gain.py:176-188, :200-223; train/train_ring_attractor.py:21-52), per trial:
//   theta0 ~ U(0, 2pi);  a zero-ratio drawn uniformly from `ratios`;  the first n0 = int(T * start_ratio) steps are zero;
//   of the remaining `rest` steps an EXACT count keep = rest - floor(rest * ratio) stays non-zero, at positions drawn
//   uniformly without replacement, each with a value U(-max_av, max_av);
//   target[0] = theta0, target[t] = (theta0 + sum_{u<t} av[u]) mod 2pi  (the target lags the velocity by one step);
//   A[t] = [relu(-av)/scale, relu(av)/scale, 0, ...];  r_init = a bump centred at theta0.
// The reference picks the non-zero positions by ranking a second array of uniforms (argsort); here they are picked by
// sequential selection sampling (position i is kept with probability (keep - kept so far)/(rest - i)), which yields
// the same distribution -- every subset of size keep equally likely -- in one pass without sorting.  Random numbers:
// Philox4x32-10 (counter-based: trial b uses subsequence b of `seed`, so a trial's values do not depend on the batch
// it is generated in).  The stream therefore differs from torch's host generator; the distribution does not.
#include <curand_kernel.h>

#include "ringrnn_common.cuh"

namespace ringrnn {
namespace {

constexpr int MAX_RATIOS = 8;
struct Ratios {
  int n;
  float v[MAX_RATIOS];
};

// one thread per trial
__global__ void __launch_bounds__(128) generate_trials_kernel(int B, int T, int a_dim, unsigned long long seed,
                                                              long long first_trial, float max_av, float scale,
                                                              float start_ratio, Ratios ratios,
                                                              float* __restrict__ A, float* __restrict__ target,
                                                              float* __restrict__ theta0_out) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  curandStatePhilox4_32_10_t st;
  curand_init(seed, (unsigned long long)(first_trial + b), 0ULL, &st);
  const float two_pi = 6.283185307179586f;
  const float4 head = curand_uniform4(&st);  // (0, 1]
  const float theta0 = (1.f - head.x) * two_pi;  // [0, 2pi)
  int ri = (int)((1.f - head.y) * ratios.n);
  ri = ri < ratios.n ? ri : ratios.n - 1;
  const int n0 = (int)(T * start_ratio);
  const int rest = T - n0;
  const int keep = rest - (int)(rest * ratios.v[ri]);
  float* a_row = A + (size_t)b * T * a_dim;
  float* t_row = target + (size_t)b * T;
  if (theta0_out != nullptr) theta0_out[b] = theta0;
  float csum = 0.f;  // running sum of av, fp32 like torch.cumsum
  int kept = 0;
  for (int t0 = 0; t0 < T; t0 += 2) {
    const float4 u = curand_uniform4(&st);  // two steps per draw: (selection, value) each
    const float sel[2] = {1.f - u.x, 1.f - u.z}, val[2] = {1.f - u.y, 1.f - u.w};
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int t = t0 + e;
      if (t >= T) break;
      // target lags by one step: the angle BEFORE this step's velocity is applied
      float ang = fmodf(theta0 + csum, two_pi);
      if (ang < 0.f) ang += two_pi;
      t_row[t] = ang;
      float av = 0.f;
      if (t >= n0) {
        const int i = t - n0;
        // keep this position with probability (keep - kept) / (rest - i): exactly `keep` positions survive
        if (sel[e] * (float)(rest - i) < (float)(keep - kept)) {
          av = (val[e] - 0.5f) * 2.f * max_av;
          ++kept;
        }
      }
      csum += av;
      float* o = a_row + (size_t)t * a_dim;
      o[0] = fmaxf(-av, 0.f) / scale;
      if (a_dim > 1) o[1] = fmaxf(av, 0.f) / scale;
      for (int k = 2; k < a_dim; ++k) o[k] = 0.f;
    }
  }
}

// r_init[b, i]: kind 0 = exp(kappa * (cos(2 pi i / N - theta0) - 1))   (benchmark configurations, kappa = 4)
//               kind 1 = unit-norm Gaussian of width N / width on the ring (train/train_ring_attractor.py:21-52)
__global__ void __launch_bounds__(128) initial_bump_kernel(int B, int N, const float* __restrict__ theta0, int kind,
                                                           float param, float* __restrict__ r_init) {
  const int b = blockIdx.x;
  const float th = theta0[b];
  const float two_pi = 6.283185307179586f;
  __shared__ float red[4];
  float ss = 0.f;
  for (int i = threadIdx.x; i < N; i += blockDim.x) {
    float v;
    if (kind == 0) {
      v = expf(param * (cosf(two_pi * (float)i / (float)N - th) - 1.f));
    } else {
      const float c = th * (float)N / two_pi;
      float d = fabsf((float)i - c);
      d = fminf(d, (float)N - d);
      const float w = (float)N / param;
      v = expf(-(d * d) / (2.f * w * w));
    }
    r_init[(size_t)b * N + i] = v;
    ss += v * v;
  }
  if (kind == 1) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_down_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    const float inv = rsqrtf(red[0] + red[1] + red[2] + red[3]);
    for (int i = threadIdx.x; i < N; i += blockDim.x) r_init[(size_t)b * N + i] *= inv;
  }
}

}  // namespace
}  // namespace ringrnn

extern "C" int ringrnn_generate_trials(int B, int T, int N, int a_dim, unsigned long long seed, long long first_trial,
                                       float max_av, float scale, float start_ratio, const float* zero_ratios,
                                       int n_ratios, int bump_kind, float bump_param, float* A, float* target,
                                       float* r_init, float* theta0_scratch, void* stream) {
  using namespace ringrnn;
  if (B <= 0 || T <= 0 || a_dim <= 0 || (r_init != nullptr && N <= 0)) return RINGRNN_ERR_SHAPE;
  if (!A || !target || !zero_ratios || n_ratios < 1 || n_ratios > MAX_RATIOS) return RINGRNN_ERR_ARG;
  if (r_init != nullptr && theta0_scratch == nullptr) return RINGRNN_ERR_ARG;
  if (!(max_av > 0.f) || !(scale > 0.f) || start_ratio < 0.f || start_ratio > 1.f) return RINGRNN_ERR_ARG;
  if (bump_kind != 0 && bump_kind != 1) return RINGRNN_ERR_ARG;
  Ratios r;
  r.n = n_ratios;
  for (int i = 0; i < n_ratios; ++i) {
    if (zero_ratios[i] < 0.f || zero_ratios[i] > 1.f) return RINGRNN_ERR_ARG;
    r.v[i] = zero_ratios[i];
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  {
    LaunchScope ls(K_PREP, s);
    generate_trials_kernel<<<(B + 127) / 128, 128, 0, s>>>(B, T, a_dim, seed, first_trial, max_av, scale, start_ratio, r, A,
                                                          target, theta0_scratch);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  if (r_init != nullptr) {
    LaunchScope ls(K_PREP, s);
    initial_bump_kernel<<<B, 128, 0, s>>>(B, N, theta0_scratch, bump_kind, bump_param, r_init);
    RINGRNN_CUDA_TRY(cudaGetLastError());
  }
  return RINGRNN_OK;
}
