// extern "C" surface of libringrnn.so: argument checking, precision dispatch, error reporting.
#include <string.h>

#include <atomic>
#include <mutex>
#include <vector>

#include "ringrnn_common.cuh"
#include "tc_ptx.cuh"

namespace ringrnn {

// Self-test of the bounded wait every tensor-core kernel is built on: one thread waits, through the same mbar_wait(),
// for a barrier phase that nothing will ever complete.  After `limit` cycles the wait gives up, records `code` in the
// status word and the kernel ends normally.
__global__ void wait_selftest_kernel(int* status, long long limit, int code) {
  __shared__ alignas(8) unsigned long long bar;
  __shared__ int dead;
  if (threadIdx.x == 0) {
    dead = 0;
    tc::mbar_init(tc::smem_u32(&bar), 1);
    tc::fence_mbar_init();
    tc::WaitCtx w{&dead, status, limit};
    (void)tc::mbar_wait(tc::smem_u32(&bar), 0, w, code);
  }
}

static thread_local cudaError_t g_last_cuda_error = cudaSuccess;
void set_last_cuda_error(cudaError_t e) { g_last_cuda_error = e; }

// ---- launch accounting ---------------------------------------------------------------------
static std::atomic<long long> g_launches{0};
static std::atomic<int> g_timing_on{0};
static std::mutex g_timing_mu;
struct TimedLaunch { int slot; cudaEvent_t start, stop; };
static std::vector<TimedLaunch> g_timed;
static float g_slot_ms[K_SLOTS];
static int g_slot_n[K_SLOTS];

LaunchScope::LaunchScope(int slot, cudaStream_t s) : slot_(slot), s_(s), start_(nullptr), timed_(false) {
  g_launches.fetch_add(1, std::memory_order_relaxed);
  if (g_timing_on.load(std::memory_order_relaxed)) {
    if (cudaEventCreate(&start_) == cudaSuccess) {
      cudaEventRecord(start_, s_);
      timed_ = true;
    }
  }
}
LaunchScope::~LaunchScope() {
  if (!timed_) return;
  cudaEvent_t stop;
  if (cudaEventCreate(&stop) != cudaSuccess) { cudaEventDestroy(start_); return; }
  cudaEventRecord(stop, s_);
  std::lock_guard<std::mutex> lk(g_timing_mu);
  g_timed.push_back({slot_, start_, stop});
}

static void drain_timed_locked() {
  for (auto& t : g_timed) {
    float ms = 0.f;
    if (cudaEventSynchronize(t.stop) == cudaSuccess && cudaEventElapsedTime(&ms, t.start, t.stop) == cudaSuccess) {
      g_slot_ms[t.slot] += ms;
      g_slot_n[t.slot] += 1;
    }
    cudaEventDestroy(t.start);
    cudaEventDestroy(t.stop);
  }
  g_timed.clear();
}

// ---- deferred device status --------------------------------------------------------------------
// The reference learns of a failed kernel at once, because it synchronises and exits (cpp/cuda_common.cuh:30-39).
// Here a launch returns before its kernels run, so the status word they may set is copied, behind them on the same
// stream, into a ring of pinned host words; every later entry into the library looks at the ring and reports a
// non-zero word as RINGRNN_ERR_DEVICE.  No synchronisation anywhere.
constexpr int STATUS_SLOTS = 64;
static std::mutex g_status_mu;
static volatile int* g_status_ring = nullptr;  // pinned host memory, STATUS_SLOTS words
static int g_status_next = 0;
static int g_status_sticky = 0;                // first unreported code

int queue_status_report(const int* dev_status, cudaStream_t s) {
  if (dev_status == nullptr) return RINGRNN_OK;
  std::lock_guard<std::mutex> lk(g_status_mu);
  if (g_status_ring == nullptr) {
    void* h = nullptr;
    RINGRNN_CUDA_TRY(cudaHostAlloc(&h, sizeof(int) * STATUS_SLOTS, cudaHostAllocPortable));
    memset(h, 0, sizeof(int) * STATUS_SLOTS);
    g_status_ring = static_cast<volatile int*>(h);
  }
  const int slot = g_status_next;
  g_status_next = (g_status_next + 1) % STATUS_SLOTS;
  if (g_status_ring[slot] != 0 && g_status_sticky == 0) g_status_sticky = g_status_ring[slot];
  g_status_ring[slot] = 0;
  RINGRNN_CUDA_TRY(cudaMemcpyAsync(const_cast<int*>(g_status_ring) + slot, dev_status, sizeof(int), cudaMemcpyDeviceToHost, s));
  return RINGRNN_OK;
}

// first unreported non-zero status word that has arrived on the host (0 if none); clears what it returns
static int take_device_status() {
  std::lock_guard<std::mutex> lk(g_status_mu);
  int code = g_status_sticky;
  g_status_sticky = 0;
  if (g_status_ring != nullptr)
    for (int i = 0; i < STATUS_SLOTS; ++i)
      if (g_status_ring[i] != 0) {
        if (code == 0) code = g_status_ring[i];
        g_status_ring[i] = 0;
      }
  return code;
}
static thread_local int g_last_device_code = 0;

namespace {

int check_problem(const RingRnnProblem& p) {
  if (p.B <= 0 || p.T <= 0 || p.N <= 0 || p.a_dim <= 0) return RINGRNN_ERR_SHAPE;
  if (p.activation < RINGRNN_ACT_RELU || p.activation > RINGRNN_ACT_SILU) return RINGRNN_ERR_ARG;
  if (p.precision != RINGRNN_PREC_FP32 && p.precision != RINGRNN_PREC_BF16) return RINGRNN_ERR_ARG;
  if (p.n_active > p.a_dim || p.n_active > RINGRNN_MAX_ACTIVE) return RINGRNN_ERR_ARG;
  if (p.ckpt_every < 0) return RINGRNN_ERR_ARG;
  // more than RINGRNN_MAX_ACTIVE columns ("all columns", a_dim beyond the list's size): the fp32 mode takes them, as the
  // reference's kernels take any a_dim (cpp/fwd.cu:21-50); the tensor-core modes do not
  if (p.n_active < 0 && p.a_dim > RINGRNN_MAX_ACTIVE && p.precision != RINGRNN_PREC_FP32) return RINGRNN_ERR_UNSUPPORTED;
  for (int k = 0; k < p.n_active; ++k)
    if (p.active_cols[k] < 0 || p.active_cols[k] >= p.a_dim) return RINGRNN_ERR_ARG;
  return RINGRNN_OK;
}

int check_pointers(const RingRnnProblem& p) {
  if (!p.A || !p.Wa || !p.Wo || !p.r_init) return RINGRNN_ERR_ARG;
  return RINGRNN_OK;
}

DevProblem to_dev(const RingRnnProblem& p) {
  DevProblem d;
  memset(&d, 0, sizeof(d));
  d.B = p.B; d.T = p.T; d.N = p.N; d.a_dim = p.a_dim;
  d.J0 = p.J0; d.J1 = p.J1; d.alpha = p.alpha;
  d.A = p.A; d.Wa = p.Wa; d.Wo = p.Wo; d.r_init = p.r_init;
  const int n = (p.n_active < 0) ? p.a_dim : p.n_active;
  d.n_mat = 1 + n;
  d.all_cols = p.n_active < 0 ? 1 : 0;
  for (int k = 0; k < n && k < RINGRNN_MAX_ACTIVE; ++k) d.cols[k] = (p.n_active < 0) ? k : p.active_cols[k];
  return d;
}

}  // namespace
}  // namespace ringrnn

using namespace ringrnn;

extern "C" int ringrnn_version(void) { return 100; }

extern "C" const char* ringrnn_strerror(int status) {
  switch (status) {
    case RINGRNN_OK: return "ok";
    case RINGRNN_ERR_ARG: return "invalid argument (null pointer or bad enum value)";
    case RINGRNN_ERR_SHAPE: return "invalid or unsupported shape";
    case RINGRNN_ERR_WORKSPACE: return "workspace or saved buffer missing or too small";
    case RINGRNN_ERR_CUDA: return "CUDA runtime error";
    case RINGRNN_ERR_UNSUPPORTED: return "request not supported by this precision mode";
    case RINGRNN_ERR_DEVICE: return "a bounded device-side wait ran out";
    case RINGRNN_ERR_TOO_LARGE: return "size exceeds the capacity of the library's built-in scratch array";
    default: return "unknown status";
  }
}

extern "C" int ringrnn_last_cuda_error(void) { return (int)g_last_cuda_error; }
extern "C" const char* ringrnn_last_cuda_error_string(void) { return cudaGetErrorString(g_last_cuda_error); }

extern "C" size_t ringrnn_workspace_bytes(const RingRnnProblem* p, int which, int history_given) {
  if (p == nullptr || check_problem(*p) != RINGRNN_OK) return (size_t)-1;
  const bool bf16 = p->precision == RINGRNN_PREC_BF16;
  if (bf16 && !bf16_supported(*p)) {
    // bf16 arithmetic, one GEMM per timestep: the shapes the persistent kernels do not take
    if (!stepwise_supported(*p)) return (size_t)-1;
    switch (which) {
      case RINGRNN_WS_FWD: return stepwise_fwd_workspace_bytes(*p);
      case RINGRNN_WS_SAVED: return stepwise_saved_bytes(*p);
      case RINGRNN_WS_BWD: return stepwise_bwd_workspace_bytes(*p);
      default: return (size_t)-1;
    }
  }
  switch (which) {
    case RINGRNN_WS_FWD: return bf16 ? bf16_fwd_workspace_bytes(*p) : fp32_fwd_workspace_bytes(*p);
    case RINGRNN_WS_SAVED: return bf16 ? bf16_saved_bytes(*p) : fp32_saved_bytes(*p, history_given);
    case RINGRNN_WS_BWD: return bf16 ? bf16_bwd_workspace_bytes(*p) : fp32_bwd_workspace_bytes(*p);
    default: return (size_t)-1;
  }
}

extern "C" int ringrnn_fwd(const RingRnnFwdArgs* a, void* stream) {
  if (a == nullptr) return RINGRNN_ERR_ARG;
  int rc = check_problem(a->p);
  if (rc != RINGRNN_OK) return rc;
  rc = check_pointers(a->p);
  if (rc != RINGRNN_OK) return rc;
  const bool want_dec = a->dec_x || a->dec_y || a->dec_ta;
  if (want_dec && (!a->dec_u || !a->dec_v)) return RINGRNN_ERR_ARG;
  if (!a->bump_history && !a->saved && !want_dec && !a->final_state) return RINGRNN_ERR_ARG;  // nothing to produce
  if (const int code = take_device_status()) {  // an EARLIER launch abandoned a bounded wait: its results are invalid
    g_last_device_code = code;
    return RINGRNN_ERR_DEVICE;
  }
  const DevProblem dp = to_dev(a->p);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a->p.precision == RINGRNN_PREC_BF16) {
    if (!bf16_supported(a->p) && !stepwise_supported(a->p)) return RINGRNN_ERR_UNSUPPORTED;
    rc = bf16_supported(a->p) ? bf16_forward(*a, dp, s) : stepwise_forward(*a, dp, s);
    if (rc != RINGRNN_OK) return rc;
    return queue_status_report(a->status != nullptr ? a->status : static_cast<const int*>(a->workspace), s);
  }
  return fp32_forward(*a, dp, s);
}

extern "C" int ringrnn_bwd(const RingRnnBwdArgs* a, void* stream) {
  if (a == nullptr) return RINGRNN_ERR_ARG;
  int rc = check_problem(a->p);
  if (rc != RINGRNN_OK) return rc;
  rc = check_pointers(a->p);
  if (rc != RINGRNN_OK) return rc;
  if (!a->grad_Wa || !a->grad_Wo) return RINGRNN_ERR_ARG;
  if (!a->grad_output && !a->coef_x) return RINGRNN_ERR_ARG;
  if (a->coef_x && (!a->coef_y || !a->coef_s || !a->dec_u || !a->dec_v)) return RINGRNN_ERR_ARG;
  if (const int code = take_device_status()) {
    g_last_device_code = code;
    return RINGRNN_ERR_DEVICE;
  }
  const DevProblem dp = to_dev(a->p);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a->p.precision == RINGRNN_PREC_BF16) {
    if (!bf16_supported(a->p) && !stepwise_supported(a->p)) return RINGRNN_ERR_UNSUPPORTED;
    rc = bf16_supported(a->p) ? bf16_backward(*a, dp, s) : stepwise_backward(*a, dp, s);
    if (rc != RINGRNN_OK) return rc;
    return queue_status_report(a->status != nullptr ? a->status : static_cast<const int*>(a->workspace), s);
  }
  return fp32_backward(*a, dp, s);
}

extern "C" int ringrnn_fwd_cuda(const void* A, const void* Wa, float J0, float J1, const void* Wo,
                                const void* r_init, void* bump_history, float alpha, int N, int a_dim, int seq_len,
                                int batch_size, int activation_type, int precision, void* saved, size_t saved_bytes,
                                void* workspace, size_t workspace_bytes, void* stream) {
  RingRnnFwdArgs a;
  memset(&a, 0, sizeof(a));
  a.p.B = batch_size; a.p.T = seq_len; a.p.N = N; a.p.a_dim = a_dim;
  a.p.activation = activation_type; a.p.precision = precision;
  a.p.J0 = J0; a.p.J1 = J1; a.p.alpha = alpha;
  a.p.A = static_cast<const float*>(A); a.p.Wa = static_cast<const float*>(Wa);
  a.p.Wo = static_cast<const float*>(Wo); a.p.r_init = static_cast<const float*>(r_init);
  a.p.n_active = -1;
  a.bump_history = static_cast<float*>(bump_history);
  a.saved = saved; a.saved_bytes = saved_bytes;
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  return ringrnn_fwd(&a, stream);
}

extern "C" int ringrnn_bwd_cuda(const void* grad_output, const void* A, const void* Wa, float J0, float J1,
                                const void* Wo, const void* bump_history, const void* r_init, void* grad_Wa,
                                void* grad_Wo, float alpha, int N, int a_dim, int seq_len, int batch_size,
                                int activation_type, int precision, const void* saved, size_t saved_bytes,
                                void* workspace, size_t workspace_bytes, void* stream) {
  RingRnnBwdArgs a;
  memset(&a, 0, sizeof(a));
  a.p.B = batch_size; a.p.T = seq_len; a.p.N = N; a.p.a_dim = a_dim;
  a.p.activation = activation_type; a.p.precision = precision;
  a.p.J0 = J0; a.p.J1 = J1; a.p.alpha = alpha;
  a.p.A = static_cast<const float*>(A); a.p.Wa = static_cast<const float*>(Wa);
  a.p.Wo = static_cast<const float*>(Wo); a.p.r_init = static_cast<const float*>(r_init);
  a.p.n_active = -1;
  a.grad_output = static_cast<const float*>(grad_output);
  a.bump_history = static_cast<const float*>(bump_history);
  a.saved = saved; a.saved_bytes = saved_bytes;
  a.grad_Wa = static_cast<float*>(grad_Wa); a.grad_Wo = static_cast<float*>(grad_Wo);
  a.workspace = workspace; a.workspace_bytes = workspace_bytes;
  return ringrnn_bwd(&a, stream);
}

extern "C" int ringrnn_selftest_wait(long long limit_cycles, int code, int* status, void* stream) {
  if (status == nullptr || limit_cycles < 0 || limit_cycles > 4000000000LL || code == 0) return RINGRNN_ERR_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  {
    LaunchScope ls(K_PREP, s);
    wait_selftest_kernel<<<1, 32, 0, s>>>(status, limit_cycles, code);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  return queue_status_report(status, s);
}

extern "C" int ringrnn_device_status(int* code) {
  const int c = take_device_status();
  if (c != 0) g_last_device_code = c;
  if (code != nullptr) *code = c != 0 ? c : 0;
  return c != 0 ? RINGRNN_ERR_DEVICE : RINGRNN_OK;
}
extern "C" int ringrnn_last_device_code(void) { return g_last_device_code; }

extern "C" long long ringrnn_launch_count(void) { return g_launches.load(); }
extern "C" int ringrnn_timing_slots(void) { return K_SLOTS; }
extern "C" const char* ringrnn_timing_name(int slot) {
  static const char* names[K_SLOTS] = {"prep", "fwd_recurrent", "bwd_recurrent", "dw_product", "dw_reduce", "loss"};
  return (slot >= 0 && slot < K_SLOTS) ? names[slot] : "";
}
extern "C" int ringrnn_timing_enable(int on) {
  g_timing_on.store(on ? 1 : 0);
  return RINGRNN_OK;
}
extern "C" int ringrnn_timing_read(int slot, float* total_ms, int* launches) {
  if (slot < 0 || slot >= K_SLOTS || !total_ms || !launches) return RINGRNN_ERR_ARG;
  std::lock_guard<std::mutex> lk(g_timing_mu);
  drain_timed_locked();
  *total_ms = g_slot_ms[slot];
  *launches = g_slot_n[slot];
  return RINGRNN_OK;
}
extern "C" int ringrnn_timing_reset(void) {
  std::lock_guard<std::mutex> lk(g_timing_mu);
  drain_timed_locked();
  for (int i = 0; i < K_SLOTS; ++i) { g_slot_ms[i] = 0.f; g_slot_n[i] = 0; }
  g_launches.store(0);
  return RINGRNN_OK;
}
