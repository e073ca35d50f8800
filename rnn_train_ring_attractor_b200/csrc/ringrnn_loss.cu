// Decode + loss on the per-(sample, step) scalars x = r.u, y = r.v, ta = sum|r| that the forward emits.
//
// The reference forms r @ W_delta7, divides by the row maximum, takes the first Fourier component and
// an atan2 (train_general_ring_no_gain.py:113-116, train/train_ring_attractor.py:196-206).  atan2 ignores the
// positive 1/max scale, so the decoded angle is atan2(r.v, r.u) with u = W_delta7 cos(phi),
// v = W_delta7 sin(phi).  Loss per (b,t): (cos th - cos th*)^2 + (sin th - sin th*)^2 = 2 - 2 cos(th - th*);
// amplitude loss: (ta_t - ta_0)^2 (train/train_ring_attractor.py:289-296).  The kernel also emits the
// coefficients of the closed-form gradient with respect to r_t:
//   dL/dr_t = coef_x*u + coef_y*v + coef_s*sign(r_t).
#include <mutex>

#include "ringrnn_common.cuh"

namespace ringrnn {
namespace {

constexpr int LT = 256;

__device__ __forceinline__ float block_sum(float v, float* red) {
  // fixed-order block reduction (warp shuffles, then the warp leaders in order)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < LT / 32; ++w) tot += red[w];
  return tot;
}

__global__ void __launch_bounds__(LT) angle_loss_kernel(int B, int T, const float* __restrict__ dec_x,
                                                        const float* __restrict__ dec_y,
                                                        const float* __restrict__ dec_ta,
                                                        const float* __restrict__ target, float bump_weight,
                                                        float inv_count, float* coef_x, float* coef_y, float* coef_s,
                                                        float* decoded, float* scratch) {
  __shared__ float red[LT / 32];
  const int b = blockIdx.x;
  const size_t row = (size_t)b * T;
  const float ta0 = dec_ta[row];
  const float two_pi = 6.283185307179586f;
  float l_cos = 0.f, l_amp = 0.f, c_sum = 0.f;
  for (int t = threadIdx.x; t < T; t += LT) {
    const float x = dec_x[row + t], y = dec_y[row + t];
    const float th = atan2f(y, x);
    float sd, cd;
    sincosf(th - target[row + t], &sd, &cd);
    l_cos += 2.f - 2.f * cd;
    const float n2 = x * x + y * y;
    const float k = (n2 > 1e-30f) ? 2.f * sd / n2 * inv_count : 0.f;
    coef_x[row + t] = -k * y;
    coef_y[row + t] = k * x;
    const float dev = dec_ta[row + t] - ta0;
    l_amp += dev * dev;
    const float c = 2.f * bump_weight * dev * inv_count;
    if (t > 0) {
      coef_s[row + t] = c;
      c_sum += c;
    }
    if (decoded != nullptr) {
      float a = fmodf(th + two_pi, two_pi);
      decoded[row + t] = a;
    }
  }
  l_cos = block_sum(l_cos, red);
  l_amp = block_sum(l_amp, red);
  c_sum = block_sum(c_sum, red);
  if (threadIdx.x == 0) {
    coef_s[row] = -c_sum;
    scratch[b] = l_cos;
    scratch[B + b] = l_amp;
  }
}

__global__ void __launch_bounds__(LT) loss_finish_kernel(int B, const float* __restrict__ scratch, float inv_count,
                                                         float* loss_out) {
  __shared__ float red[LT / 32];
  float a = 0.f, c = 0.f;
  for (int b = threadIdx.x; b < B; b += LT) {
    a += scratch[b];
    c += scratch[B + b];
  }
  a = block_sum(a, red);
  c = block_sum(c, red);
  if (threadIdx.x == 0) {
    loss_out[0] = a * inv_count;
    loss_out[1] = c * inv_count;
  }
}

}  // namespace
}  // namespace ringrnn

extern "C" int ringrnn_angle_loss(int B, int T, const float* dec_x, const float* dec_y, const float* dec_ta,
                                  const float* target, float bump_weight, float inv_count, float* coef_x,
                                  float* coef_y, float* coef_s, float* decoded, float* loss_out, float* scratch,
                                  void* stream) {
  using namespace ringrnn;
  if (B <= 0 || T <= 0) return RINGRNN_ERR_SHAPE;
  if (!dec_x || !dec_y || !dec_ta || !target || !coef_x || !coef_y || !coef_s || !loss_out || !scratch)
    return RINGRNN_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  {
    LaunchScope ls(K_LOSS, s);
    angle_loss_kernel<<<B, LT, 0, s>>>(B, T, dec_x, dec_y, dec_ta, target, bump_weight, inv_count, coef_x, coef_y,
                                       coef_s, decoded, scratch);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  { LaunchScope ls(K_LOSS, s); loss_finish_kernel<<<1, LT, 0, s>>>(B, scratch, inv_count, loss_out); }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  return RINGRNN_OK;
}

// ---- the same loss with library-owned scratch -------------------------------------------------------------
// For callers that cannot allocate device memory where they need the loss (a process whose framework pool owns
// all of it, or a loop that cannot take the device-wide synchronisation of an allocation).  The per-sample
// partial sums live in this file-scope array; every GPU that loads the library carries its 512 KB.
static __device__ __align__(256) float g_static_loss_scratch[2 * RINGRNN_STATIC_LOSS_MAX_B];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
float* g_static_addr[kMaxDevices];  // device address of g_static_loss_scratch on each device, looked up once

// In host code the array's name is only a handle for the runtime, not a device pointer: the address a kernel
// may use has to be asked for, on the device that will run the kernel.
int static_scratch_address(float** out) {
  int dev = -1;
  RINGRNN_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return RINGRNN_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lk(g_static_mu);
  if (g_static_addr[dev] == nullptr) {
    float* ptr = nullptr;
    RINGRNN_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_static_loss_scratch));
    if (ptr == nullptr) return RINGRNN_ERR_CUDA;
    g_static_addr[dev] = ptr;
  }
  *out = g_static_addr[dev];
  return RINGRNN_OK;
}
}  // namespace

extern "C" int ringrnn_angle_loss_static(int B, int T, const float* dec_x, const float* dec_y, const float* dec_ta,
                                         const float* target, float bump_weight, float inv_count, float* coef_x,
                                         float* coef_y, float* coef_s, float* decoded, float* loss_out,
                                         void* stream) {
  using namespace ringrnn;
  if (B <= 0 || T <= 0) return RINGRNN_ERR_SHAPE;
  if (B > RINGRNN_STATIC_LOSS_MAX_B) return RINGRNN_ERR_TOO_LARGE;
  if (!dec_x || !dec_y || !dec_ta || !target || !coef_x || !coef_y || !coef_s || !loss_out) return RINGRNN_ERR_ARG;
  float* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);  // first call per device: the lookup; later calls: a table read
  if (rc != RINGRNN_OK) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // entries [0,B) and [B,2B) are written by the first kernel before the second reads them: nothing to clear
  {
    LaunchScope ls(K_LOSS, s);
    angle_loss_kernel<<<B, LT, 0, s>>>(B, T, dec_x, dec_y, dec_ta, target, bump_weight, inv_count, coef_x, coef_y,
                                       coef_s, decoded, scratch);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  {
    LaunchScope ls(K_LOSS, s);
    loss_finish_kernel<<<1, LT, 0, s>>>(B, scratch, inv_count, loss_out);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  return RINGRNN_OK;
}
