// bf16 mode, forward: one persistent tcgen05 kernel runs all T timesteps of a 128-sample tile on a
// thread-block cluster (see tc_recurrent.cuh for the decomposition).  Replaces the T launches of
// fwd_wmma_kernel (cpp/kernels/fwd_1loop_tc_idx.cuh:265-277), which rebuild the per-sample effective
// weight matrix on tensor cores and do the actual recurrence on CUDA cores.
//
// Per step and CTA:   D_s[128, 208] = r_{t-1}[128, NP] x Wblock_s^T      (s = 0, 1; fp32 in TMEM)
// epilogue (thread = sample):   re = J0*S + J1*Yo + L*Yl + R*Yr,  r_t = (1-alpha) r_{t-1} + alpha F(re)
// with the fp32 master copy of r in registers; bf16(r_t) goes to the A buffers of all CTAs of the cluster
// for the next step, to the saved state, and F'(re) (bf16) to the saved derivative history; optional fp32
// history and per-step decode sums (r.u, r.v, sum|r|).
#include <string.h>

#include "tc_recurrent.cuh"

namespace ringrnn {

using namespace tc;
using namespace tcr;

struct TcFwdParams {
  int B, T, N, BP, a_dim, colL, colR, n_tiles;
  float J0, J1, alpha;
  const float* A;        // [B,T,a_dim]
  const float* r_init;   // [B,N]
  __nv_bfloat16* Rh;     // [T+1][BP][NP] (slot 0 = bf16(r_init), prepared before launch) or nullptr
  __nv_bfloat16* Dh;     // [T][BP][NP] or nullptr
  float* hist;           // [T,B,N] or nullptr
  float* dec_part;       // [2C][3][T][BP] or nullptr
  const float* dec_u;    // [N]
  const float* dec_v;
  float* final_state;    // [B,N] or nullptr
  int* status;
};

template <int ACT, int NP>
__global__ void __launch_bounds__(THREADS, 1)
fwd_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmR0, const TcFwdParams p) {
  using C_ = Cfg<NP>;
  constexpr int C = C_::C, KC = C_::KC, NS = C_::NS;
  constexpr bool RESIDENT = C_::RESIDENT;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gen = smem_raw + (base - smem_u32(smem_raw));
  const uint32_t a_base = base;
  const uint32_t w_base = base + C_::A_BYTES;
  const uint32_t bars = w_base + NS * WT_BYTES;
  uint8_t* bars_gen = gen + C_::A_BYTES + NS * WT_BYTES;
  volatile uint32_t* tmem_slot_p = reinterpret_cast<volatile uint32_t*>(bars_gen + OFF_TMEM_SLOT);
  volatile int* dead = reinterpret_cast<volatile int*>(bars_gen + OFF_DEAD);
  float* uv = reinterpret_cast<float*>(bars_gen + OFF_UV);
  const WaitCtx wctx{dead, p.status};

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t q = (C > 1) ? cluster_ctarank() : 0u;
  const int cluster_id = blockIdx.x / C, n_clusters = gridDim.x / C;
  const int T = p.T;

  if (threadIdx.x == 0) {
    *dead = 0;
    for (int i = 0; i < 16; ++i) {
      mbar_init(bars + OFF_W_FULL + 8 * i, 1);
      mbar_init(bars + OFF_W_EMPTY + 8 * i, 1);
    }
    for (int i = 0; i < 8; ++i) mbar_init(bars + OFF_A_FULL + 8 * i, 1);
    mbar_init(bars + OFF_D_FULL, 1);
    mbar_init(bars + OFF_D_FULL + 8, 1);
    mbar_init(bars + OFF_D_EMPTY, 8);      // all eight epilogue warps drain each accumulator
    mbar_init(bars + OFF_D_EMPTY + 8, 8);
    mbar_init(bars + OFF_MMA_DONE, 1);
    mbar_init(bars + OFF_ALL_FREE, C);
    fence_mbar_init();
  }
  if (threadIdx.x < 256) {
    const int i = threadIdx.x & 127, n = (int)q * 128 + i;
    const float* src = (threadIdx.x < 128) ? p.dec_u : p.dec_v;
    uv[threadIdx.x] = (src != nullptr && n < p.N) ? src[n] : 0.f;
  }
  if (warp == 1) tmem_alloc(bars + OFF_TMEM_SLOT, TMEM_COLS);
  tcgen05_fence_before();
  __syncthreads();
  if (C > 1) {  // every CTA's barriers exist before any peer signals them
    cluster_arrive();
    cluster_wait();
  }
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_p;

  if (warp < 4) {
    reg_dec<40>();
    if (warp == 0 && lane == 0) {
      // ---------------- TMA producer: the weight stream ----------------
      tma_prefetch_desc(&tmW);
      uint32_t wcount = 0;
      int it = 0;
      for (int tile = cluster_id; tile < p.n_tiles; tile += n_clusters, ++it) {
        if (RESIDENT) {
          if (it == 0) {
            for (int s = 0; s < 2; ++s)
              for (int i = 0; i < KC; ++i) {
                const int kc = (2 * (int)q + i) % KC, st = s * KC + i;
                mbar_arrive_expect_tx(bars + OFF_W_FULL + 8 * st, WT_BYTES);
                tma_load_2d(w_base + st * WT_BYTES, &tmW, bars + OFF_W_FULL + 8 * st, kc * 64, ((int)q * 2 + s) * RB);
              }
          }
        } else {
          for (int t = 0; t < T; ++t)
            for (int s = 0; s < 2; ++s)
              for (int i = 0; i < KC; ++i, ++wcount) {
                const int kc = (2 * (int)q + i) % KC, st = wcount % NS;
                if (wcount >= (uint32_t)NS) mbar_wait(bars + OFF_W_EMPTY + 8 * st, (wcount / NS - 1) & 1u, wctx, 202);
                mbar_arrive_expect_tx(bars + OFF_W_FULL + 8 * st, WT_BYTES);
                tma_load_2d(w_base + st * WT_BYTES, &tmW, bars + OFF_W_FULL + 8 * st, kc * 64, ((int)q * 2 + s) * RB);
              }
        }
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t idesc = make_idesc_bf16(128, RB, 0, 0);
      uint32_t wcount = 0, g = 0;
      for (int tile = cluster_id; tile < p.n_tiles; tile += n_clusters) {
        for (int t = 0; t < T; ++t, ++g) {
          for (int s = 0; s < 2; ++s) {
            if (g > 0) mbar_wait(bars + OFF_D_EMPTY + 8 * s, (g - 1) & 1u, wctx, 203);
            tcgen05_fence_after();
            for (int i = 0; i < KC; ++i) {
              const int kc = (2 * (int)q + i) % KC;
              if (s == 0) {
                mbar_wait(bars + OFF_A_FULL + 8 * kc, g & 1u, wctx, 204);
                // chunks owned by peers arrive as bulk copies: arm the byte count of the next step's copy
                if ((kc >> 1) != (int)q && t + 1 < T) mbar_arrive_expect_tx(bars + OFF_A_FULL + 8 * kc, CHUNK_BYTES);
              }
              int st;
              if (RESIDENT) {
                st = s * KC + i;
                if (g == 0) mbar_wait(bars + OFF_W_FULL + 8 * st, 0, wctx, 205);
              } else {
                st = wcount % NS;
                mbar_wait(bars + OFF_W_FULL + 8 * st, (wcount / NS) & 1u, wctx, 205);
              }
              tcgen05_fence_after();
              const uint32_t a_src = a_base + kc * CHUNK_BYTES, b_src = w_base + st * WT_BYTES;
#pragma unroll
              for (int ks = 0; ks < 4; ++ks)
                umma_ss(tmem_base + s * 256, make_smem_desc(a_src + ks * 32, 16, 1024),
                        make_smem_desc(b_src + ks * 32, 16, 1024), idesc, (i > 0 || ks > 0) ? 1u : 0u);
              if (!RESIDENT) {
                umma_commit(bars + OFF_W_EMPTY + 8 * st);
                ++wcount;
              }
            }
            umma_commit(bars + OFF_D_FULL + 8 * s);
          }
          umma_commit(bars + OFF_MMA_DONE);
        }
      }
    } else if (warp == 2 && lane == 0) {
      // ---------------- relay: loads the initial state of each tile; after every step tells every CTA of the
      // cluster that this CTA no longer reads its A buffer (it follows every phase of mma_done, so it is
      // also the one that knows when the buffer may take the next tile) ----------------
      tma_prefetch_desc(&tmR0);
      uint32_t g = 0;
      for (int tile = cluster_id; tile < p.n_tiles; tile += n_clusters) {
        for (int kc = 0; kc < KC; ++kc) {
          mbar_arrive_expect_tx(bars + OFF_A_FULL + 8 * kc, CHUNK_BYTES);
          tma_load_2d(a_base + kc * CHUNK_BYTES, &tmR0, bars + OFF_A_FULL + 8 * kc, kc * 64, tile * 128);
        }
        for (int t = 0; t < T; ++t, ++g) {
          mbar_wait(bars + OFF_MMA_DONE, g & 1u, wctx, 206);
          for (uint32_t r = 0; r < (uint32_t)C; ++r) mbar_arrive_cluster(bars + OFF_ALL_FREE, r);
        }
      }
    }
  } else {
    reg_inc<232>();
    // ---------------- epilogue: thread = sample.  Warps 4-7 (h = 0) own columns [0,32) and warps 8-11 (h = 1)
    // columns [32,64) of BOTH 64-neuron sub-slices, so every accumulator is drained by all eight warps at once
    // (two warps per scheduler) and the part of the step that nothing overlaps -- the epilogue of the last
    // sub-slice -- is 32 elements per thread.  master[s*32 + j] is neuron 128q + 64s + 32h + j. ----------------
    const int h = (warp - 4) >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int nq = (int)q * 128 + 32 * h;  // neuron of master[0]; sub-slice s adds 64*s
    const int slot = 2 * (int)q + h;
    const float J0 = p.J0, J1 = p.J1, alpha = p.alpha, beta = 1.f - p.alpha;
    const bool want_dec = p.dec_part != nullptr;
    uint32_t g = 0;
    for (int tile = cluster_id; tile < p.n_tiles; tile += n_clusters) {
      const int b = tile * 128 + row;
      const bool valid = b < p.B;
      float master[64];
#pragma unroll
      for (int s = 0; s < 2; ++s)
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int n = nq + 64 * s + j;
          master[s * 32 + j] = (valid && n < p.N) ? __ldg(p.r_init + (size_t)b * p.N + n) : 0.f;
        }
      for (int t = 0; t < T; ++t, ++g) {
        float L = 0.f, R = 0.f;
        if (valid) {
          const float* at = p.A + ((size_t)b * T + t) * p.a_dim;
          if (p.colL >= 0) L = __ldg(at + p.colL);
          if (p.colR >= 0) R = __ldg(at + p.colR);
        }
        uint32_t packed[32];
        float px = 0.f, py = 0.f, pa = 0.f, c0 = 0.f;
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          mbar_wait(bars + OFF_D_FULL + 8 * s, g & 1u, wctx, 207);
          tcgen05_fence_after();
          uint32_t yo[32], yl[32], yr[32];
          const uint32_t col = tmem_base + lane_base + s * 256 + 32 * h;
          if (s == 0) {
            uint32_t sraw;
            tmem_ld1(tmem_base + lane_base + SUM_COL, &sraw);  // row sum of r_{t-1}
            tmem_ld32(col, yo);
            tmem_ld32(col + 64, yl);
            tmem_ld32(col + 128, yr);
            tmem_ld_wait();
            c0 = J0 * __uint_as_float(sraw);
          } else {
            tmem_ld32(col, yo);
            tmem_ld32(col + 64, yl);
            tmem_ld32(col + 128, yr);
            tmem_ld_wait();
          }
          // the accumulator is in registers: hand it back to the MMA warp
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bars + OFF_D_EMPTY + 8 * s);
          uint32_t dpk[16];
#pragma unroll
          for (int j0 = 0; j0 < 32; j0 += 8) {
            float re[8], f[8], d[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              float v = fmaf(J1, __uint_as_float(yo[j0 + e]), c0);
              v = fmaf(L, __uint_as_float(yl[j0 + e]), v);
              re[e] = fmaf(R, __uint_as_float(yr[j0 + e]), v);
            }
            act_group<ACT, 8>(re, f, d);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const int idx = s * 32 + j0 + e;
              float r = fmaf(alpha, f[e], beta * master[idx]);
              if (nq + 64 * s + j0 + e >= p.N) { r = 0.f; d[e] = 0.f; }
              master[idx] = r;
              f[e] = r;
              if (want_dec) {
                px = fmaf(r, uv[64 * s + 32 * h + j0 + e], px);
                py = fmaf(r, uv[128 + 64 * s + 32 * h + j0 + e], py);
                pa += fabsf(r);
              }
            }
#pragma unroll
            for (int e = 0; e < 8; e += 2) {
              packed[s * 16 + ((j0 + e) >> 1)] = pack_bf16x2(f[e], f[e + 1]);
              dpk[(j0 + e) >> 1] = pack_bf16x2(d[e], d[e + 1]);
            }
          }
          if (p.Dh != nullptr) {
            uint4* dst = reinterpret_cast<uint4*>(p.Dh + ((size_t)t * p.BP + b) * NP + nq + 64 * s);
#pragma unroll
            for (int v = 0; v < 4; ++v) dst[v] = make_uint4(dpk[4 * v], dpk[4 * v + 1], dpk[4 * v + 2], dpk[4 * v + 3]);
          }
        }
        // every CTA of the cluster has finished reading r_{t-1} (waited for in every step so that no phase of
        // the barrier is skipped); then publish r_t
        mbar_wait<true>(bars + OFF_ALL_FREE, g & 1u, wctx, 208);
        if (t + 1 < T) {
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const uint32_t tile_addr = a_base + (2 * (int)q + s) * CHUNK_BYTES;
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const uint32_t unit = (uint32_t)(4 * h + v);
              const uint32_t addr = tile_addr + row * 128 + ((unit ^ ((uint32_t)row & 7u)) << 4);
              asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(packed[s * 16 + 4 * v]),
                           "r"(packed[s * 16 + 4 * v + 1]), "r"(packed[s * 16 + 4 * v + 2]),
                           "r"(packed[s * 16 + 4 * v + 3])
                           : "memory");
            }
          }
          fence_proxy_async_smem();
          named_bar_sync(1, 256);
          if (warp == 4 && lane == 0) {
#pragma unroll
            for (int s = 0; s < 2; ++s) {
              const int kc = 2 * (int)q + s;
              const uint32_t tile_addr = a_base + kc * CHUNK_BYTES;
              mbar_arrive(bars + OFF_A_FULL + 8 * kc);
              for (uint32_t r = 0; r < (uint32_t)C; ++r)
                if (r != q) dsmem_bulk_copy(tile_addr, tile_addr, CHUNK_BYTES, bars + OFF_A_FULL + 8 * kc, r);
            }
          }
        }
        // off the critical path: saved state, fp32 history, decode sums
        if (p.Rh != nullptr) {
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            uint4* dst = reinterpret_cast<uint4*>(p.Rh + ((size_t)(t + 1) * p.BP + b) * NP + nq + 64 * s);
#pragma unroll
            for (int v = 0; v < 4; ++v)
              dst[v] = make_uint4(packed[s * 16 + 4 * v], packed[s * 16 + 4 * v + 1], packed[s * 16 + 4 * v + 2],
                                  packed[s * 16 + 4 * v + 3]);
          }
        }
        if (p.hist != nullptr && valid) {
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            float* dst = p.hist + ((size_t)t * p.B + b) * p.N + nq + 64 * s;
            if ((p.N & 3) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                if (nq + 64 * s + j < p.N)
                  *reinterpret_cast<float4*>(dst + j) = make_float4(master[s * 32 + j], master[s * 32 + j + 1],
                                                                    master[s * 32 + j + 2], master[s * 32 + j + 3]);
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (nq + 64 * s + j < p.N) dst[j] = master[s * 32 + j];
            }
          }
        }
        if (want_dec) {
          float* dp = p.dec_part + ((size_t)slot * 3 * T + t) * p.BP + b;
          dp[0] = px;
          dp[(size_t)T * p.BP] = py;
          dp[(size_t)2 * T * p.BP] = pa;
        }
      }
      if (p.final_state != nullptr && valid) {
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (nq + 64 * s + j < p.N) p.final_state[(size_t)b * p.N + nq + 64 * s + j] = master[s * 32 + j];
      }
    }
  }
  // ---------------- teardown: nobody leaves while a peer may still signal or copy into this CTA ----------------
  tcgen05_fence_before();
  __syncthreads();
  if (C > 1) {
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int ACT, int NP>
static int launch_fwd_tc(const CUtensorMap& tmW, const CUtensorMap& tmR0, const TcFwdParams& p, cudaStream_t s) {
  using C_ = Cfg<NP>;
  RINGRNN_CUDA_TRY(cudaFuncSetAttribute(fwd_tc_kernel<ACT, NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, C_::SMEM));
  int max_clusters = 148 / C_::C;
  int n_clusters = p.n_tiles < max_clusters ? p.n_tiles : max_clusters;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(n_clusters * C_::C, 1, 1);
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = C_::SMEM;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = C_::C;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  {
    LaunchScope ls(K_FWD, s);
    RINGRNN_CUDA_TRY(cudaLaunchKernelEx(&cfg, fwd_tc_kernel<ACT, NP>, tmW, tmR0, p));
  }
  return RINGRNN_OK;
}

int tc_forward_launch(int act, int NP, const CUtensorMap& tmW, const CUtensorMap& tmR0, const void* params,
                      cudaStream_t s) {
  const TcFwdParams& p = *static_cast<const TcFwdParams*>(params);  // same field order as the host-side mirror
#define RINGRNN_TCF(ACT, NPV) \
  if (act == ACT && NP == NPV) return launch_fwd_tc<ACT, NPV>(tmW, tmR0, p, s);
  RINGRNN_TCF(RINGRNN_ACT_RELU, 128) RINGRNN_TCF(RINGRNN_ACT_RELU, 256) RINGRNN_TCF(RINGRNN_ACT_RELU, 512)
  RINGRNN_TCF(RINGRNN_ACT_GELU, 128) RINGRNN_TCF(RINGRNN_ACT_GELU, 256) RINGRNN_TCF(RINGRNN_ACT_GELU, 512)
  RINGRNN_TCF(RINGRNN_ACT_TANH, 128) RINGRNN_TCF(RINGRNN_ACT_TANH, 256) RINGRNN_TCF(RINGRNN_ACT_TANH, 512)
  RINGRNN_TCF(RINGRNN_ACT_SILU, 128) RINGRNN_TCF(RINGRNN_ACT_SILU, 256) RINGRNN_TCF(RINGRNN_ACT_SILU, 512)
#undef RINGRNN_TCF
  return RINGRNN_ERR_UNSUPPORTED;
}

}  // namespace ringrnn
