/* ringrnn.h -- C ABI of libringrnn.so: the ring-attractor recurrent forward and
 * backward-through-time operator for NVIDIA B200 (sm_100a).
 *
 * Plain pointers and sizes only; every pointer named "device" is CUDA device memory owned by
 * the caller, including all scratch ("workspace") and saved-for-backward storage, whose sizes
 * ringrnn_workspace_bytes() reports.  No entry point allocates device memory, exits the process
 * or throws: each returns a RINGRNN_* status.  (Host side, the library keeps one 256-byte block of pinned
 * host memory for the deferred status reports described at RingRnnFwdArgs, allocated once on first use.)  Calls are asynchronous on `stream` (a cudaStream_t
 * passed as void*; NULL = the legacy default stream) and may come from any host thread.
 *
 * Each declaration cites the interface of the reference project (chongxi/rnn_train_ring_attractor,
 * paths relative to its root) that it replaces.
 */
#ifndef RINGRNN_H
#define RINGRNN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes */
enum {
  RINGRNN_OK = 0,
  RINGRNN_ERR_ARG = 1,         /* NULL where a pointer is required, bad enum value            */
  RINGRNN_ERR_SHAPE = 2,       /* non-positive or unsupported dimension                        */
  RINGRNN_ERR_WORKSPACE = 3,   /* workspace / saved buffer missing, misaligned or too small    */
  RINGRNN_ERR_CUDA = 4,        /* a CUDA runtime call failed (see ringrnn_last_cuda_error)     */
  RINGRNN_ERR_UNSUPPORTED = 5, /* valid request that this precision mode cannot serve          */
  RINGRNN_ERR_DEVICE = 6,      /* a kernel of an EARLIER call reported a bounded wait that ran out */
  RINGRNN_ERR_TOO_LARGE = 7    /* size exceeds the capacity of the library's built-in scratch  */
};

/* activation codes: the enum order of cpp/cuda_common.cuh:56 and the activation_map of
 * cpp/ring_rnn_cuda.py:63 */
enum { RINGRNN_ACT_RELU = 0, RINGRNN_ACT_GELU = 1, RINGRNN_ACT_TANH = 2, RINGRNN_ACT_SILU = 3 };

/* arithmetic mode.  FP32: CUDA-core FFMA throughout (the reference's fwd_fp32 path,
 * cpp/kernels/fwd_fp32.cuh).  BF16: bf16 tensor-core operands with fp32 accumulation and an fp32
 * master state (the reference's WMMA path, cpp/kernels/fwd_1loop_tc_idx.cuh). */
enum { RINGRNN_PREC_FP32 = 0, RINGRNN_PREC_BF16 = 1 };

/* which buffer ringrnn_workspace_bytes() sizes */
enum { RINGRNN_WS_FWD = 0, RINGRNN_WS_SAVED = 1, RINGRNN_WS_BWD = 2 };

#define RINGRNN_MAX_ACTIVE 64

/* The problem both directions share.  Tensor arguments follow cpp/fwd.cu:5-19:
 *   A[B,T,a_dim], Wa[a_dim,N,N], Wo[N,N], r_init[B,N], all fp32, contiguous, device memory.
 * n_active / active_cols name the columns of A that are not identically zero (the root training
 * script pads the L/R signal to 16 columns with zeros, train_general_ring_no_gain.py:200-223);
 * n_active < 0 means "all a_dim columns" (the fp32 mode then takes any a_dim; the bf16 mode at most
 * RINGRNN_MAX_ACTIVE active columns).  Gradients of skipped columns are exactly zero.
 * ckpt_every = K > 0 (bf16 mode, persistent kernels): the forward keeps only the fp32 state every K steps and the
 * backward recomputes each stretch of K steps from its checkpoint before it propagates through it -- the saved
 * storage shrinks from two bf16 tensors of T*B*N to T/K fp32 states of B*N, for one extra forward pass.  0 = keep every
 * step (the default; faster whenever the saved tensors fit).  The fp32 mode and the stepwise path ignore it. */
typedef struct RingRnnProblem {
  int B, T, N, a_dim;
  int activation; /* RINGRNN_ACT_*  */
  int precision;  /* RINGRNN_PREC_* */
  float J0, J1, alpha;
  const float* A;
  const float* Wa;
  const float* Wo;
  const float* r_init;
  int n_active;
  int active_cols[RINGRNN_MAX_ACTIVE];
  int ckpt_every;
} RingRnnProblem;

/* Forward.  Replaces fwd_cuda() (cpp/fwd.cu:21-50) and its launchers
 * (cpp/kernels/fwd_1loop_tc_idx.cuh:280-311, cpp/kernels/fwd_fp32.cuh:277-298).
 *   bump_history  [T,B,N] fp32 out, layout of cpp/ring_rnn_cuda.py:62; NULL = do not write the history
 *   saved         storage the backward call needs (RINGRNN_WS_SAVED bytes); NULL = inference
 *   dec_x, dec_y  [B,T] fp32 out: population-vector components r_t.u and r_t.v (NULL = skip)
 *   dec_ta        [B,T] fp32 out: sum_i |r_t[b,i]|                              (NULL = skip)
 *   dec_u, dec_v  [N] fp32 in, required when any dec_* output is requested
 *   final_state   [B,N] fp32 out, r_T (NULL = skip)
 *   workspace     RINGRNN_WS_FWD bytes of scratch
 *   status        optional device int that the CALLER has set to zero: the bf16-mode kernels set it non-zero if a
 *                 bounded device-side wait ran out, and once it is non-zero every later wait of kernels that share the
 *                 word gives up at once (NULL = the library uses, and zeroes, the first word of `workspace`).
 * Error reporting is deferred, because the call returns before its kernels have run (the reference synchronises and
 * exits instead, cpp/cuda_common.cuh:30-39): the status word is copied to the host behind the kernels, and the NEXT
 * ringrnn_fwd / ringrnn_bwd call of the process returns RINGRNN_ERR_DEVICE if a word that has arrived is non-zero --
 * the results of the launches since the last successful report are then invalid.  ringrnn_device_status() does the same
 * check on demand, e.g. right after the caller's own synchronisation. */
typedef struct RingRnnFwdArgs {
  RingRnnProblem p;
  float* bump_history;
  void* saved;
  size_t saved_bytes;
  float* dec_x;
  float* dec_y;
  float* dec_ta;
  const float* dec_u;
  const float* dec_v;
  float* final_state;
  void* workspace;
  size_t workspace_bytes;
  int* status;
} RingRnnFwdArgs;

/* Backward through time.  Replaces bwd_cuda() (cpp/bwd.cu:4-52) and
 * bwd_wmma_launcher (cpp/kernels/bwd_mixed_precision_aggressive.cuh:676-707).
 * The cotangent of the history is the sum of two optional sources:
 *   grad_output [T,B,N] fp32 (cpp/ring_rnn_cuda.py:88), and
 *   coef_x, coef_y, coef_s [B,T] fp32 with dec_u, dec_v [N]:
 *     g_t[b,i] += coef_x[b,t]*u[i] + coef_y[b,t]*v[i] + coef_s[b,t]*sign(r_t[b,i])
 *   (the closed-form gradient of the decode + cosine + bump-amplitude loss).
 *   bump_history  the forward output when it was written; NULL = use `saved`
 *   grad_Wa [a_dim,N,N], grad_Wo [N,N]  fp32 out, overwritten (cpp/ring_rnn_cuda.py:98-99, :144)
 *   grad_J        float[2] out = {dL/dJ0, dL/dJ1}, NULL = skip (the reference returns None)
 *   grad_r_init   [B,N] out, NULL = skip (the reference returns None)
 *   grad_A        [B,T,a_dim] out = dL/dA, NULL = skip (the reference returns None; needed by models whose action
 *                 signal comes from trainable gain networks, train/train_ring_attractor.py:131-146).  Columns that
 *                 n_active / active_cols leave out receive zero: pass n_active < 0 to get every column. */
typedef struct RingRnnBwdArgs {
  RingRnnProblem p;
  const float* grad_output;
  const float* coef_x;
  const float* coef_y;
  const float* coef_s;
  const float* dec_u;
  const float* dec_v;
  const float* bump_history;
  const void* saved;
  size_t saved_bytes;
  float* grad_Wa;
  float* grad_Wo;
  float* grad_J;
  float* grad_r_init;
  float* grad_A;
  void* workspace;
  size_t workspace_bytes;
  int* status;
} RingRnnBwdArgs;

/* library version (major*10000 + minor*100 + patch) */
int ringrnn_version(void);

/* text for a RINGRNN_* status.  Replaces the print-and-exit of CHECK_CUDA_ERROR
 * (cpp/cuda_common.cuh:30-39): errors are returned, never fatal. */
const char* ringrnn_strerror(int status);

/* cudaError_t of the most recent failing CUDA call on this host thread (0 if none) and its text */
int ringrnn_last_cuda_error(void);
const char* ringrnn_last_cuda_error_string(void);

/* Bytes of RINGRNN_WS_FWD / _SAVED / _BWD storage for a problem.  `history_given` says whether the
 * caller keeps bump_history itself (then the fp32 mode saves nothing).  Replaces the per-call
 * torch allocations of cpp/ring_rnn_cuda.py:105-114 and the cudaMalloc/cudaFree inside
 * cpp/kernels/fwd_fp32.cuh:246-274.  Returns (size_t)-1 for an invalid problem. */
size_t ringrnn_workspace_bytes(const RingRnnProblem* p, int which, int history_given);

int ringrnn_fwd(const RingRnnFwdArgs* args, void* stream);
int ringrnn_bwd(const RingRnnBwdArgs* args, void* stream);

/* The reference's own native signatures with a status return, an explicit precision, caller
 * scratch and a stream appended.  Argument meaning as cpp/fwd.cu:5-19 and cpp/bwd.cu:4-30; the
 * reference's bwd scratch tensors (grad_r, W_eff_temp, ...) and cuBLAS handle are not needed. */
int ringrnn_fwd_cuda(const void* A, const void* Wa, float J0, float J1, const void* Wo, const void* r_init,
                     void* bump_history, float alpha, int N, int a_dim, int seq_len, int batch_size,
                     int activation_type, int precision, void* saved, size_t saved_bytes, void* workspace,
                     size_t workspace_bytes, void* stream);
int ringrnn_bwd_cuda(const void* grad_output, const void* A, const void* Wa, float J0, float J1, const void* Wo,
                     const void* bump_history, const void* r_init, void* grad_Wa, void* grad_Wo, float alpha,
                     int N, int a_dim, int seq_len, int batch_size, int activation_type, int precision,
                     const void* saved, size_t saved_bytes, void* workspace, size_t workspace_bytes, void* stream);

/* Deferred device-side failures (see RingRnnFwdArgs).  Returns RINGRNN_ERR_DEVICE and stores the kernel's code in *code
 * (may be NULL) if a bf16-mode launch whose status word has reached the host abandoned a bounded wait; RINGRNN_OK and 0
 * otherwise.  Reading clears the report.  Never synchronises: call it after a stream or device synchronisation of your
 * own to learn about everything launched before it.  ringrnn_last_device_code(): the code of the most recent report
 * delivered to this host thread.  Replaces CHECK_CUDA_ERROR after each kernel (cpp/cuda_common.cuh:30-39,
 * cpp/fwd.cu:49). */
int ringrnn_device_status(int* code);
int ringrnn_last_device_code(void);

/* Self-test of the bounded wait (no counterpart in the reference): launches one thread that waits for an event that
 * never happens, with a limit of `limit_cycles` SM cycles (<= 4e9) instead of the kernels' ~1 s.  The kernel ends
 * normally, `*status` (device int, zeroed by the caller) receives `code` (non-zero), and the report is queued like any
 * other, so the next ringrnn_fwd / ringrnn_bwd / ringrnn_device_status sees RINGRNN_ERR_DEVICE. */
int ringrnn_selftest_wait(long long limit_cycles, int code, int* status, void* stream);

/* Decode + loss on the [B,T] scalars the forward emits.  Replaces the [B,T,N]-sized chain
 * `bump @ W_delta7`, max-normalise (train_general_ring_no_gain.py:113-116), cosine_similarity_loss
 * (train/train_ring_attractor.py:190-220) and bump_amplitude_loss (:275-298).
 *   target  [B,T] true angle;  inv_count = 1/(B_global*T);  bump_weight = 0.2 in the reference
 *   coef_x/y/s [B,T] out (inputs of ringrnn_bwd);  decoded [B,T] out in [0,2pi), NULL = skip
 *   loss_out  float[2] out = {sum of (2-2cos(err)) * inv_count, sum of amplitude deviations^2 * inv_count}
 *   scratch   B floats * 2 */
int ringrnn_angle_loss(int B, int T, const float* dec_x, const float* dec_y, const float* dec_ta,
                       const float* target, float bump_weight, float inv_count, float* coef_x, float* coef_y,
                       float* coef_s, float* decoded, float* loss_out, float* scratch, void* stream);

/* ringrnn_angle_loss without the caller-supplied scratch.  No counterpart in the reference.
 *
 * Same computation, arguments and outputs as ringrnn_angle_loss, minus `scratch`: the per-sample partial
 * losses go to an array that lives inside the library (2 * RINGRNN_STATIC_LOSS_MAX_B floats = 512 KB of
 * device memory, held by every GPU that loads the library until the process exits).  It is meant for hosts
 * that may not allocate device memory at the point where they need the loss: a serving process whose
 * memory is owned entirely by its framework's pool, so that a raw allocation would fail or fragment it, or a
 * latency-critical loop that cannot afford the device-wide synchronisation an allocation implies.  The call
 * itself performs no cudaMalloc / cudaFree and calls no allocating library routine -- with one exception you
 * control: while ringrnn_timing_enable(1) is in force every launch of this library, this one included, creates a
 * pair of CUDA events (cudaEventCreate); leave timing off where that matters.
 *   - B > RINGRNN_STATIC_LOSS_MAX_B is rejected with RINGRNN_ERR_TOO_LARGE before anything is launched.
 *   - The first call on each device looks up the array's device address (once per device, with that device
 *     current); make that first call outside any stream capture.
 *   - All calls on a device share the one array, and it keeps the previous call's contents.  Nothing in it has
 *     to start at zero: each call overwrites entries [0,B) and [B,2B) before it reads them and reads no
 *     others.  Two calls that overlap in time on the same GPU (different streams or threads) race on it;
 *     order them on one stream or with events. */
#define RINGRNN_STATIC_LOSS_MAX_B 65536
int ringrnn_angle_loss_static(int B, int T, const float* dec_x, const float* dec_y, const float* dec_ta,
                              const float* target, float bump_weight, float inv_count, float* coef_x,
                              float* coef_y, float* coef_s, float* decoded, float* loss_out, void* stream);

/* Synthetic trials of the angular-velocity integration task, generated on the device (no host->device copy of inputs).
 * Replaces, in distribution, generate_av_integration_data_ultra_fast (utils/generate_av_integration_data.py:11-58),
 * av_to_action_signal_ND with zero padding (train_general_ring_no_gain.py:200-223) and create_initial_bump
 * (train/train_ring_attractor.py:21-52) / the benchmark configurations' von-Mises bump:
 *   per trial: theta0 ~ U(0,2pi); one of `zero_ratios` drawn uniformly; the first int(T*start_ratio) steps zero; of the
 *   `rest` others exactly rest - floor(rest*ratio) stay non-zero, at uniformly drawn positions, each U(-max_av, max_av);
 *   target[b,0] = theta0, target[b,t] = (theta0 + sum_{u<t} av[b,u]) mod 2pi;
 *   A[b,t,:] = [relu(-av)/scale, relu(av)/scale, 0, ...]  (a_dim columns);
 *   r_init[b,:] = bump_kind 0: exp(bump_param*(cos(2pi i/N - theta0) - 1));  1: unit-norm Gaussian of width N/bump_param.
 * Random numbers are Philox4x32-10 with trial `first_trial + b` as the subsequence of `seed`: the same trial index gives
 * the same trial whatever batch it is generated in (the stream is not torch's; the distribution is the reference's).
 *   A [B,T,a_dim], target [B,T] out;  r_init [B,N] out or NULL;  theta0_scratch [B] floats (required with r_init). */
int ringrnn_generate_trials(int B, int T, int N, int a_dim, unsigned long long seed, long long first_trial,
                            float max_av, float scale, float start_ratio, const float* zero_ratios, int n_ratios,
                            int bump_kind, float bump_param, float* A, float* target, float* r_init,
                            float* theta0_scratch, void* stream);

/* Optimizer step on flat buffers, entirely on the device: clip the gradient to a global L2 norm of `max_norm`
 * (max_norm <= 0: no clipping), then one Adam update (no weight decay, no amsgrad).  Replaces the pair
 * torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0); optimizer.step() of
 * train_general_ring_no_gain.py:335-336 for parameters kept in one contiguous fp32 buffer laid out like the
 * gradient buffer of the data-parallel step ([Wo | Wa | J0 J1]); same arithmetic, no read-back of the norm.
 *   params, grads, exp_avg, exp_avg_sq   n floats each (grads is not modified)
 *   step                                 1 for the first update (bias correction)
 *   scratch                              129 doubles; scratch[128] receives the unclipped gradient norm */
int ringrnn_clip_adam(float* params, const float* grads, float* exp_avg, float* exp_avg_sq, size_t n, float lr,
                      float beta1, float beta2, float eps, int step, float max_norm, double* scratch, void* stream);

/* Launch accounting and per-kernel timing (the reference's counterpart is the NVTX / cudaProfiler
 * bracketing in legacy/bwd_fp32.py:705-740 and utils/benchmark.py:58-79).
 *   ringrnn_launch_count   kernels launched by this library since the last reset
 *   ringrnn_timing_enable  when on, every kernel launch is bracketed by a CUDA event pair on its stream
 *   ringrnn_timing_read    synchronises the recorded events and returns, for kernel class `slot`
 *                          (0 <= slot < ringrnn_timing_slots()), the summed milliseconds and launch count
 *   ringrnn_timing_reset   drops recorded events and zeroes the counters */
long long ringrnn_launch_count(void);
int ringrnn_timing_slots(void);
const char* ringrnn_timing_name(int slot);
int ringrnn_timing_enable(int on);
int ringrnn_timing_read(int slot, float* total_ms, int* launches);
int ringrnn_timing_reset(void);

/* Library self-test: one split-K bf16 GEMM on the tcgen05 tensor-core path the bf16 mode is built from
 * (TMA-fed shared-memory ring, TMEM accumulator).  No counterpart in the reference; it exists so that the
 * operand layouts can be checked in isolation.  out[M,N] fp32 = A * B over K:
 *   mn_major = 1: A is [K,M] and B is [K,N] bf16 row-major;  mn_major = 0: A is [M,K] and B is [N,K];
 *   mn_major = 2: as 0, computed by CTA pairs (cta_group::2 MMAs, M % 256 == 0, N % 128 == 0 or N % 224 == 0,
 *   nsplit ignored).
 * M % 128 == 0, N % 128 == 0, partial holds nsplit*M*N floats, status is a zero-initialised device int. */
int ringrnn_selftest_gemm(int mn_major, const void* A, const void* B, float* partial, float* out, int M, int N,
                          long long K, int nsplit, int* status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* RINGRNN_H */
