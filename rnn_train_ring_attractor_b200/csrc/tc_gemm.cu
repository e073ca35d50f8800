// Split-K bf16 GEMM on tcgen05 tensor cores with fp32 accumulation in tensor memory.
//
// Used for the weight-gradient products of the bf16 mode,
//   dWcat[3*NP, NP] = [delta | L*delta | R*delta]^T [3*NP, T*B]  x  r_prev [T*B, NP],
// whose reduction dimension is the whole (time, batch) range (the reference accumulates these with one
// cuBLAS sgemm plus one WMMA kernel per timestep, cpp/kernels/bwd_mixed_precision_aggressive.cuh:607-671).
// Both operands are consumed in the layout the recurrent kernels write them, [row = (t,b)] x [neuron], i.e.
// "MN-major" for the MMA; a K-major variant of the same kernel exists for the library self-test.
//
// One CTA owns a 128 x NT output tile for one slice of the reduction range: warp 0 streams operand tiles with
// TMA into a ring of shared-memory stages, warp 1 issues tcgen05.mma into one TMEM accumulator, warps 2-5
// move the finished accumulator to global memory as an fp32 partial; a second kernel sums the partials in a
// fixed order (no atomics, bit-reproducible).
#include <string.h>

#include "ringrnn_common.cuh"
#include "tc_ptx.cuh"

namespace ringrnn {

// ---- host: tensor map creation through the driver entry point (no link-time libcuda dependency) ----------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

bool make_tmap_bf16_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
                       uint32_t box_cols, int swizzle_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

namespace {

using namespace tc;

constexpr int GEMM_THREADS = 192;

template <bool MN_MAJOR, int NT>
struct GemmCfg {
  static constexpr int KC = MN_MAJOR ? 32 : 64;                       // reduction rows per stage
  static constexpr int A_BYTES = MN_MAJOR ? 2 * KC * 128 : 128 * 128;  // 128 output rows
  static constexpr int B_BYTES = MN_MAJOR ? (NT / 64) * KC * 128 : NT * 128;
  static constexpr int STAGE = A_BYTES + B_BYTES;
  static constexpr int NSTAGE = (200 * 1024) / STAGE < 8 ? (200 * 1024) / STAGE : 8;
  static constexpr int SMEM = NSTAGE * STAGE + 1024 /*align*/ + 256 /*barriers*/;
  static constexpr int TMEM_COLS = NT < 32 ? 32 : NT;
  static constexpr int NI = NT > 256 ? NT / 256 : 1;  // MMA instructions along N per k-step
  static constexpr int NMMA = NT > 256 ? 256 : NT;
};

// out[split][M_total][N_total] fp32;  the CTA's output tile starts at (m0 = blockIdx.x*128, n0 = blockIdx.y*NT)
// K-major:  tmA over A[M_total, K] box [128 x 64], tmB over B[N_total, K] box [min(NT,256) x 64]
// MN-major: tmA over A[K, M_total] box [KC x 64],  tmB over B[K, N_total] box [KC x 64]
template <bool MN_MAJOR, int NT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               float* __restrict__ out, int M_total, int N_total, long long K_total, long long k_per_split,
               int* status) {
  using Cfg = GemmCfg<MN_MAJOR, NT>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + Cfg::NSTAGE * Cfg::STAGE;  // full[NSTAGE], empty[NSTAGE], done, tmem slot, dead
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (Cfg::NSTAGE + s); };
  const uint32_t done_bar = bars + 8u * (2 * Cfg::NSTAGE);
  const uint32_t tmem_slot = done_bar + 8;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_p = reinterpret_cast<volatile uint32_t*>(gen + Cfg::NSTAGE * Cfg::STAGE + 8 * (2 * Cfg::NSTAGE + 1));
  volatile int* dead = reinterpret_cast<volatile int*>(gen + Cfg::NSTAGE * Cfg::STAGE + 8 * (2 * Cfg::NSTAGE + 1) + 4);
  const WaitCtx wctx{dead, status};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int m0 = blockIdx.x * 128, n0 = blockIdx.y * NT;
  const long long k_begin = (long long)blockIdx.z * k_per_split;
  long long k_end = k_begin + k_per_split;
  if (k_end > K_total) k_end = K_total;
  const int iters = k_end > k_begin ? (int)((k_end - k_begin + Cfg::KC - 1) / Cfg::KC) : 0;

  if (threadIdx.x == 0) {
    *dead = 0;
    for (int s = 0; s < Cfg::NSTAGE; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(done_bar, 1);
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_p;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      for (int it = 0; it < iters; ++it) {
        const int s = it % Cfg::NSTAGE;
        const uint32_t round = it / Cfg::NSTAGE;
        if (it >= Cfg::NSTAGE && !mbar_wait(empty_bar(s), (round - 1) & 1, wctx, 101)) break;
        const uint32_t a_dst = base + s * Cfg::STAGE, b_dst = a_dst + Cfg::A_BYTES;
        mbar_arrive_expect_tx(full_bar(s), Cfg::STAGE);
        const int k = (int)(k_begin + (long long)it * Cfg::KC);
        if (MN_MAJOR) {
          for (int blk = 0; blk < 2; ++blk) tma_load_2d(a_dst + blk * Cfg::KC * 128, &tmA, full_bar(s), m0 + blk * 64, k);
          for (int blk = 0; blk < NT / 64; ++blk)
            tma_load_2d(b_dst + blk * Cfg::KC * 128, &tmB, full_bar(s), n0 + blk * 64, k);
        } else {
          tma_load_2d(a_dst, &tmA, full_bar(s), k, m0);
          for (int nh = 0; nh < Cfg::NI; ++nh) tma_load_2d(b_dst + nh * 256 * 128, &tmB, full_bar(s), k, n0 + nh * 256);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(128, Cfg::NMMA, MN_MAJOR ? 1 : 0, MN_MAJOR ? 1 : 0);
      bool ok = true;
      for (int it = 0; it < iters && ok; ++it) {
        const int s = it % Cfg::NSTAGE;
        const uint32_t round = it / Cfg::NSTAGE;
        ok = mbar_wait(full_bar(s), round & 1, wctx, 102);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t a_src = base + s * Cfg::STAGE, b_src = a_src + Cfg::A_BYTES;
        constexpr int KSTEPS = Cfg::KC / 16;
        const uint32_t a_lo = desc_lo(a_src, MN_MAJOR ? Cfg::KC * 128 : 16);
        const uint32_t b_lo = desc_lo(b_src, MN_MAJOR ? Cfg::KC * 128 : 16);
        constexpr uint32_t KSTEP_LO = MN_MAJOR ? (2048u >> 4) : (32u >> 4);
        constexpr uint32_t NH_LO = MN_MAJOR ? ((4u * Cfg::KC * 128u) >> 4) : ((256u * 128u) >> 4);
#pragma unroll
        for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
          for (int nh = 0; nh < Cfg::NI; ++nh)
            umma_ss_lo(tmem_base + nh * 256, a_lo + ks * KSTEP_LO, b_lo + nh * NH_LO + ks * KSTEP_LO, idesc,
                       (it > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(empty_bar(s));  // frees the stage when these MMAs have read it
      }
      umma_commit(done_bar);
    }
  } else {
    // epilogue: warp w owns TMEM lanes 32*(w%4)..+31 = output rows m0 + that
    const int q = warp & 3;
    const bool ok = mbar_wait(done_bar, 0, wctx, 103);
    tcgen05_fence_after();
    const int row = m0 + q * 32 + lane;
    float* orow = out + ((size_t)blockIdx.z * M_total + row) * N_total + n0;
    for (int c0 = 0; c0 < NT; c0 += 32) {
      uint32_t v[32];
      if (iters > 0 && ok) {
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + c0, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0u;
      }
      if (row < M_total) {
#pragma unroll
        for (int j = 0; j < 32; j += 4) {
          if (n0 + c0 + j < N_total)
            *reinterpret_cast<float4*>(orow + c0 + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                     __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
}


// ---- CTA-pair variant (K-major operands): a cluster of two CTAs owns a 256 x NT output tile; each CTA loads its
// own 128 rows of A and half of the B rows, the even CTA issues cta_group::2 MMAs for both.  Used by the
// library self-test to validate the pair building blocks the recurrent kernels rely on.
template <int NT>
struct PairCfg {
  static constexpr int KC = 64;
  static constexpr int A_BYTES = 128 * 128;
  static constexpr int B_BYTES = (NT / 2) * 128;  // this CTA's half of the B rows
  static constexpr int STAGE = A_BYTES + B_BYTES;
  static constexpr int NSTAGE = (200 * 1024) / STAGE < 8 ? (200 * 1024) / STAGE : 8;
  static constexpr int SMEM = NSTAGE * STAGE + 1024 + 256;
  static constexpr int TMEM_COLS = NT <= 32 ? 32 : NT <= 64 ? 64 : NT <= 128 ? 128 : NT <= 256 ? 256 : 512;  // power of two
};

template <int NT>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 float* __restrict__ out, int M_total, int N_total, long long K_total, int* status) {
  using Cfg = PairCfg<NT>;
  static_assert(NT <= 256, "one MMA instruction along N");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bars = base + Cfg::NSTAGE * Cfg::STAGE;
  auto full_bar = [&](int s) { return bars + 8u * s; };
  auto empty_bar = [&](int s) { return bars + 8u * (Cfg::NSTAGE + s); };
  const uint32_t done_bar = bars + 8u * (2 * Cfg::NSTAGE);
  const uint32_t tmem_slot = done_bar + 8;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  volatile uint32_t* tmem_slot_p = reinterpret_cast<volatile uint32_t*>(gen + Cfg::NSTAGE * Cfg::STAGE + 8 * (2 * Cfg::NSTAGE + 1));
  volatile int* dead = reinterpret_cast<volatile int*>(gen + Cfg::NSTAGE * Cfg::STAGE + 8 * (2 * Cfg::NSTAGE + 1) + 4);
  const WaitCtx wctx{dead, status};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t h = cluster_ctarank();  // 0 = even CTA (issues the MMAs), 1 = odd CTA
  const int pair = blockIdx.x >> 1;
  const int m0 = pair * 256 + (int)h * 128, n0 = blockIdx.y * NT;
  const int iters = (int)((K_total + Cfg::KC - 1) / Cfg::KC);

  if (threadIdx.x == 0) {
    *dead = 0;
    for (int s = 0; s < Cfg::NSTAGE; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    mbar_init(done_bar, 1);
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS);
  tcgen05_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_p;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tmA);
      tma_prefetch_desc(&tmB);
      for (int it = 0; it < iters; ++it) {
        const int s = it % Cfg::NSTAGE;
        const uint32_t round = it / Cfg::NSTAGE;
        if (it >= Cfg::NSTAGE && !mbar_wait(empty_bar(s), (round - 1) & 1u, wctx, 111)) break;
        const uint32_t a_dst = base + s * Cfg::STAGE, b_dst = a_dst + Cfg::A_BYTES;
        if (h == 0) mbar_arrive_expect_tx(full_bar(s), 2 * Cfg::STAGE);  // both CTAs' bytes land on this barrier
        const int k = it * Cfg::KC;
        tma_load_2d_pair(a_dst, &tmA, full_bar(s), k, m0);
        tma_load_2d_pair(b_dst, &tmB, full_bar(s), k, n0 + (int)h * (NT / 2));
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && h == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(256, NT, 0, 0);
      bool ok = true;
      for (int it = 0; it < iters && ok; ++it) {
        const int s = it % Cfg::NSTAGE;
        const uint32_t round = it / Cfg::NSTAGE;
        ok = mbar_wait(full_bar(s), round & 1u, wctx, 112);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t a_src = base + s * Cfg::STAGE, b_src = a_src + Cfg::A_BYTES;
        const uint32_t a_lo = desc_lo(a_src, 16), b_lo = desc_lo(b_src, 16);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) umma_ss_pair_lo(tmem_base, a_lo + 2 * ks, b_lo + 2 * ks, idesc, (it > 0 || ks > 0) ? 1u : 0u);
        umma_commit_pair(empty_bar(s), 3);
      }
      umma_commit_pair(done_bar, 3);
    }
  } else {
    const int q = warp & 3;
    const bool ok = mbar_wait(done_bar, 0, wctx, 113);
    tcgen05_fence_after();
    const int row = m0 + q * 32 + lane;
    float* orow = out + (size_t)row * N_total + n0;
    for (int c0 = 0; c0 < NT; c0 += 32) {
      uint32_t v[32];
      if (iters > 0 && ok) {
        tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + c0, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0u;
      }
      if (row < M_total) {
#pragma unroll
        for (int j = 0; j < 32; j += 4)
          *reinterpret_cast<float4*>(orow + c0 + j) = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]),
                                                                   __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_arrive();
  cluster_wait();
  if (warp == 1) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
}

template <int NT>
int launch_gemm_pair(const void* A, const void* B, float* out, int M_total, int N_total, long long K_total, int* status,
                     cudaStream_t s) {
  using Cfg = PairCfg<NT>;
  CUtensorMap tmA, tmB;
  if (!make_tmap_bf16_2d(&tmA, A, (uint64_t)M_total, (uint64_t)K_total, 128, 64) ||
      !make_tmap_bf16_2d(&tmB, B, (uint64_t)N_total, (uint64_t)K_total, NT / 2, 64))
    return RINGRNN_ERR_CUDA;
  RINGRNN_CUDA_TRY(cudaFuncSetAttribute(gemm_pair_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * (M_total / 256), N_total / NT, 1);
  cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  {
    LaunchScope ls(K_DW, s);
    RINGRNN_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_pair_kernel<NT>, tmA, tmB, out, M_total, N_total, K_total, status));
  }
  return RINGRNN_OK;
}

// out[e] = scale * sum_s partial[s][e]   (fixed order)
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, int nsplit, size_t elems, float* out) {
  for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < elems; e += (size_t)gridDim.x * blockDim.x) {
    float acc = 0.f;
    for (int s = 0; s < nsplit; ++s) acc += partial[(size_t)s * elems + e];
    out[e] = acc;
  }
}

template <bool MN_MAJOR, int NT>
int launch_gemm(const void* A, const void* B, float* partial, int M_total, int N_total, long long K_total, int nsplit,
                int* status, cudaStream_t s) {
  using Cfg = GemmCfg<MN_MAJOR, NT>;
  CUtensorMap tmA, tmB;
  bool ok;
  if (MN_MAJOR) {
    ok = make_tmap_bf16_2d(&tmA, A, (uint64_t)K_total, (uint64_t)M_total, Cfg::KC, 64) &&
         make_tmap_bf16_2d(&tmB, B, (uint64_t)K_total, (uint64_t)N_total, Cfg::KC, 64);
  } else {
    ok = make_tmap_bf16_2d(&tmA, A, (uint64_t)M_total, (uint64_t)K_total, 128, 64) &&
         make_tmap_bf16_2d(&tmB, B, (uint64_t)N_total, (uint64_t)K_total, Cfg::NMMA, 64);
  }
  if (!ok) return RINGRNN_ERR_CUDA;
  long long kps = (K_total + nsplit - 1) / nsplit;
  kps = (kps + Cfg::KC - 1) / Cfg::KC * Cfg::KC;
  RINGRNN_CUDA_TRY(cudaFuncSetAttribute(gemm_tc_kernel<MN_MAJOR, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        Cfg::SMEM));
  dim3 grid((M_total + 127) / 128, (N_total + NT - 1) / NT, nsplit);
  {
    LaunchScope ls(K_DW, s);
    gemm_tc_kernel<MN_MAJOR, NT><<<grid, GEMM_THREADS, Cfg::SMEM, s>>>(tmA, tmB, partial, M_total, N_total, K_total,
                                                                        kps, status);
  }
  RINGRNN_CUDA_TRY(cudaGetLastError());
  return RINGRNN_OK;
}

}  // namespace

// C[M,N] (fp32, partial sums over nsplit slices then reduced into `out`) = A * B with bf16 operands.
//   mn_major = 1: A is [K, M], B is [K, N] (row-major);  mn_major = 0: A is [M, K], B is [N, K].
// M multiple of 128; N in {128, 256, 512} or a multiple of 512 (N % NT == 0).  partial: nsplit*M*N floats.
int tc_gemm(int mn_major, const void* A, const void* B, float* partial, float* out, int M, int N, long long K,
            int nsplit, int* status, cudaStream_t s) {
  if (M % 128 != 0 || nsplit < 1) return RINGRNN_ERR_SHAPE;
  int rc;
  const int NT = (N % 512 == 0) ? 512 : (N % 256 == 0) ? 256 : (N % 128 == 0) ? 128 : 0;
  if (NT == 0) return RINGRNN_ERR_SHAPE;
#define RINGRNN_GEMM_CASE(MN, NTV)                                                            \
  if (mn_major == MN && NT == NTV) rc = launch_gemm<MN != 0, NTV>(A, B, partial, M, N, K, nsplit, status, s); else
  RINGRNN_GEMM_CASE(1, 512)
  RINGRNN_GEMM_CASE(1, 256)
  RINGRNN_GEMM_CASE(1, 128)
  RINGRNN_GEMM_CASE(0, 512)
  RINGRNN_GEMM_CASE(0, 256)
  RINGRNN_GEMM_CASE(0, 128)
  rc = RINGRNN_ERR_SHAPE;
#undef RINGRNN_GEMM_CASE
  if (rc != RINGRNN_OK) return rc;
  if (out != nullptr) {
    LaunchScope ls(K_REDUCE, s);
    splitk_reduce_kernel<<<296, 256, 0, s>>>(partial, nsplit, (size_t)M * N, out);
    RINGRNN_CUDA_TRY(cudaGetLastError());
  }
  return RINGRNN_OK;
}

// CTA-pair K-major GEMM: out[M,N] = A[M,K] * B[N,K]^T, M % 256 == 0, N a multiple of 256, 224 or 128 (the pair MMA wants N % 32 == 0) (N % NT == 0)
int tc_gemm_pair(const void* A, const void* B, float* out, int M, int N, long long K, int* status, cudaStream_t s) {
  if (M % 256 != 0) return RINGRNN_ERR_SHAPE;
  if (N % 256 == 0) return launch_gemm_pair<256>(A, B, out, M, N, K, status, s);
  if (N % 224 == 0) return launch_gemm_pair<224>(A, B, out, M, N, K, status, s);
  if (N % 128 == 0) return launch_gemm_pair<128>(A, B, out, M, N, K, status, s);
  return RINGRNN_ERR_SHAPE;
}

}  // namespace ringrnn

// Library self-test hook: one bf16 tensor-core GEMM with caller-provided device buffers.
extern "C" int ringrnn_selftest_gemm(int mn_major, const void* A, const void* B, float* partial, float* out, int M,
                                     int N, long long K, int nsplit, int* status, void* stream) {
  if (!A || !B || !partial || !out) return RINGRNN_ERR_ARG;
  if (mn_major == 2) return ringrnn::tc_gemm_pair(A, B, out, M, N, K, status, static_cast<cudaStream_t>(stream));
  return ringrnn::tc_gemm(mn_major, A, B, partial, out, M, N, K, nsplit, status, static_cast<cudaStream_t>(stream));
}
