// bf16 mode, reverse-time: one persistent tcgen05 kernel propagates delta_t = alpha*F'(re_t)*g_t through the
// transposed weights for all T steps of a 128-sample tile (same cluster decomposition as the forward kernel,
// see tc_recurrent.cuh).  Replaces the per-step launches recompute_Weff_re_grad_re_kernel +
// compute_grad_r_kernel_vec (cpp/kernels/bwd_mixed_precision_aggressive.cuh:53-318), which write and re-read
// a [B,N,N] fp32 effective-weight tensor every step.
//
// Per step and CTA:   Z_s[128, 208] = delta_t[128, NP] x WblockT_s^T        (fp32 in TMEM)
// epilogue (thread = sample):   carry = (1-alpha) g_t + J0*sum_i delta_t + J1*Zo + L_t*Zl + R_t*Zr
//                               g_{t-1} = carry + dL/dr_{t-1},   delta_{t-1} = alpha * F'(re_{t-1}) * g_{t-1}
// F'(re) comes from the derivative history the forward saved (no recompute); dL/dr is the caller's
// grad_output and/or the closed-form loss gradient coef_x*u + coef_y*v + coef_s*sign(r).  delta_t, L_t*delta_t
// and R_t*delta_t are written in bf16 as the A operand of the weight-gradient GEMM (tc_gemm.cu).
#include <string.h>

#include "tc_recurrent.cuh"

namespace ringrnn {

using namespace tc;
using namespace tcr;

struct TcBwdParams {
  int B, T, N, BP, a_dim, colL, colR, n_tiles;
  float J0, J1, alpha;
  const float* A;               // [B,T,a_dim]
  const __nv_bfloat16* Rh;      // [T+1][BP][NP]
  const __nv_bfloat16* Dh;      // [T][BP][NP]
  const float* grad_output;     // [T,B,N] or nullptr
  const float* coef_x;          // [B,T] or nullptr
  const float* coef_y;
  const float* coef_s;
  const float* dec_u;           // [N]
  const float* dec_v;
  __nv_bfloat16* DL;            // [T*BP][3*NP]
  float* grad_r_init;           // [B,N] or nullptr
  int* status;
};

template <int NP>
__global__ void __launch_bounds__(THREADS, 1)
bwd_tc_kernel(const __grid_constant__ CUtensorMap tmW, const TcBwdParams p) {
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
  const int my_tiles = (p.n_tiles - cluster_id + n_clusters - 1) / n_clusters;
  const uint32_t total_steps = (uint32_t)my_tiles * (uint32_t)T;

  if (threadIdx.x == 0) {
    *dead = 0;
    for (int i = 0; i < 16; ++i) {
      mbar_init(bars + OFF_W_FULL + 8 * i, 1);
      mbar_init(bars + OFF_W_EMPTY + 8 * i, 1);
    }
    for (int i = 0; i < 8; ++i) mbar_init(bars + OFF_A_FULL + 8 * i, 1);
    mbar_init(bars + OFF_D_FULL, 1);
    mbar_init(bars + OFF_D_FULL + 8, 1);
    mbar_init(bars + OFF_D_EMPTY, 8);  // all eight epilogue warps drain each accumulator
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
  if (C > 1) {
    cluster_arrive();
    cluster_wait();
  }
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_p;

  if (warp < 4) {
    reg_dec<40>();
    if (warp == 0 && lane == 0) {
      // ---------------- TMA producer: the (transposed) weight stream ----------------
      tma_prefetch_desc(&tmW);
      if (RESIDENT) {
        if (total_steps > 0)
          for (int s = 0; s < 2; ++s)
            for (int i = 0; i < KC; ++i) {
              const int kc = (2 * (int)q + i) % KC, st = s * KC + i;
              mbar_arrive_expect_tx(bars + OFF_W_FULL + 8 * st, WT_BYTES);
              tma_load_2d(w_base + st * WT_BYTES, &tmW, bars + OFF_W_FULL + 8 * st, kc * 64, ((int)q * 2 + s) * RB);
            }
      } else {
        uint32_t wcount = 0;
        for (uint32_t g = 0; g < total_steps; ++g)
          for (int s = 0; s < 2; ++s)
            for (int i = 0; i < KC; ++i, ++wcount) {
              const int kc = (2 * (int)q + i) % KC, st = wcount % NS;
              if (wcount >= (uint32_t)NS) mbar_wait(bars + OFF_W_EMPTY + 8 * st, (wcount / NS - 1) & 1u, wctx, 302);
              mbar_arrive_expect_tx(bars + OFF_W_FULL + 8 * st, WT_BYTES);
              tma_load_2d(w_base + st * WT_BYTES, &tmW, bars + OFF_W_FULL + 8 * st, kc * 64, ((int)q * 2 + s) * RB);
            }
      }
    } else if (warp == 1 && lane == 0) {
      // ---------------- MMA issuer ----------------
      constexpr uint32_t idesc = make_idesc_bf16(128, RB, 0, 0);
      uint32_t wcount = 0;
      // chunks owned by peers arrive as bulk copies; arm the byte count of the first step
      if (total_steps > 0)
        for (int kc = 0; kc < KC; ++kc)
          if ((kc >> 1) != (int)q) mbar_arrive_expect_tx(bars + OFF_A_FULL + 8 * kc, CHUNK_BYTES);
      for (uint32_t g = 0; g < total_steps; ++g) {
        for (int s = 0; s < 2; ++s) {
          if (g > 0) mbar_wait(bars + OFF_D_EMPTY + 8 * s, (g - 1) & 1u, wctx, 303);
          tcgen05_fence_after();
          for (int i = 0; i < KC; ++i) {
            const int kc = (2 * (int)q + i) % KC;
            if (s == 0) {
              mbar_wait(bars + OFF_A_FULL + 8 * kc, g & 1u, wctx, 304);
              if ((kc >> 1) != (int)q && g + 1 < total_steps) mbar_arrive_expect_tx(bars + OFF_A_FULL + 8 * kc, CHUNK_BYTES);
            }
            int st;
            if (RESIDENT) {
              st = s * KC + i;
              if (g == 0) mbar_wait(bars + OFF_W_FULL + 8 * st, 0, wctx, 305);
            } else {
              st = wcount % NS;
              mbar_wait(bars + OFF_W_FULL + 8 * st, (wcount / NS) & 1u, wctx, 305);
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
    } else if (warp == 2 && lane == 0) {
      // ---------------- relay: "this CTA no longer reads its A buffer for step g" to every CTA ----------------
      for (uint32_t g = 0; g < total_steps; ++g) {
        mbar_wait(bars + OFF_MMA_DONE, g & 1u, wctx, 306);
        for (uint32_t r = 0; r < (uint32_t)C; ++r) mbar_arrive_cluster(bars + OFF_ALL_FREE, r);
      }
    }
  } else {
    reg_inc<232>();
    // ---------------- epilogue: thread = sample.  Warps 4-7 (h = 0) own columns [0,32) and warps 8-11 (h = 1)
    // columns [32,64) of both 64-neuron sub-slices; master[s*32 + j] is neuron 128q + 64s + 32h + j. ----------------
    const int h = (warp - 4) >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int nq = (int)q * 128 + 32 * h;
    const float J0 = p.J0, J1 = p.J1, alpha = p.alpha, beta = 1.f - p.alpha;
    const bool has_coef = p.coef_x != nullptr;
    uint32_t g = 0;
    for (int tile = cluster_id; tile < p.n_tiles; tile += n_clusters) {
      const int b = tile * 128 + row;
      const bool valid = b < p.B;
      float master[64];  // carry on entry of `produce`, g_t afterwards
#pragma unroll
      for (int j = 0; j < 64; ++j) master[j] = 0.f;
      float L = 0.f, R = 0.f;        // action scalars of the step whose delta is in flight
      float Ln = 0.f, Rn = 0.f, cx = 0.f, cy = 0.f, cs = 0.f;  // prefetched for the next `produce`
      uint4 dv[8], rv[8];            // prefetched rows of F'(re_t) and r_t (bf16): [s*4 + v]

      // loads for produce(t); issued before the wait on the accumulators so that their latency is hidden
      auto prefetch = [&](int t) {
        Ln = 0.f; Rn = 0.f; cx = 0.f; cy = 0.f; cs = 0.f;
        if (valid) {
          const float* at = p.A + ((size_t)b * T + t) * p.a_dim;
          if (p.colL >= 0) Ln = __ldg(at + p.colL);
          if (p.colR >= 0) Rn = __ldg(at + p.colR);
          if (has_coef) {
            cx = __ldg(p.coef_x + (size_t)b * T + t);
            cy = __ldg(p.coef_y + (size_t)b * T + t);
            cs = __ldg(p.coef_s + (size_t)b * T + t);
          }
        }
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const uint4* dsrc = reinterpret_cast<const uint4*>(p.Dh + ((size_t)t * p.BP + b) * NP + nq + 64 * s);
          const uint4* rsrc = reinterpret_cast<const uint4*>(p.Rh + ((size_t)(t + 1) * p.BP + b) * NP + nq + 64 * s);
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            dv[s * 4 + v] = __ldg(dsrc + v);
            rv[s * 4 + v] = has_coef ? __ldg(rsrc + v) : make_uint4(0u, 0u, 0u, 0u);
          }
        }
      };

      // delta_t from the carry: adds dL/dr_t, applies alpha*F'(re_t), publishes the bf16 chunks, writes DL
      auto produce = [&](int t) {
        L = Ln;
        R = Rn;
        if (p.grad_output != nullptr && valid) {
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const float* gsrc = p.grad_output + ((size_t)t * p.B + b) * p.N + nq + 64 * s;
            if ((p.N & 3) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4)
                if (nq + 64 * s + j < p.N) {
                  const float4 gv = __ldg(reinterpret_cast<const float4*>(gsrc + j));
                  master[s * 32 + j] += gv.x; master[s * 32 + j + 1] += gv.y;
                  master[s * 32 + j + 2] += gv.z; master[s * 32 + j + 3] += gv.w;
                }
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j)
                if (nq + 64 * s + j < p.N) master[s * 32 + j] += __ldg(gsrc + j);
            }
          }
        }
        uint32_t packed[32];
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          __nv_bfloat16* drow = p.DL + ((size_t)t * p.BP + b) * (3 * NP) + nq + 64 * s;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const uint32_t dw[4] = {dv[s * 4 + v].x, dv[s * 4 + v].y, dv[s * 4 + v].z, dv[s * 4 + v].w};
            const uint32_t rw[4] = {rv[s * 4 + v].x, rv[s * 4 + v].y, rv[s * 4 + v].z, rv[s * 4 + v].w};
            uint32_t o0[4], o1[4], o2[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
              float dl[2];
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int j = v * 8 + w * 2 + e;
                const int idx = s * 32 + j;
                float gg = master[idx];
                if (has_coef) {
                  const float rr = e ? bf16_hi(rw[w]) : bf16_lo(rw[w]);
                  const float sg = (rr > 0.f) ? 1.f : ((rr < 0.f) ? -1.f : 0.f);
                  gg = fmaf(cx, uv[64 * s + 32 * h + j], gg);
                  gg = fmaf(cy, uv[128 + 64 * s + 32 * h + j], gg);
                  gg = fmaf(cs, sg, gg);
                }
                master[idx] = gg;
                const float dact = e ? bf16_hi(dw[w]) : bf16_lo(dw[w]);
                dl[e] = alpha * dact * gg;
              }
              o0[w] = pack_bf16x2(dl[0], dl[1]);
              o1[w] = pack_bf16x2(L * dl[0], L * dl[1]);
              o2[w] = pack_bf16x2(R * dl[0], R * dl[1]);
              packed[s * 16 + v * 4 + w] = o0[w];
            }
            *reinterpret_cast<uint4*>(drow + v * 8) = make_uint4(o0[0], o0[1], o0[2], o0[3]);
            *reinterpret_cast<uint4*>(drow + NP + v * 8) = make_uint4(o1[0], o1[1], o1[2], o1[3]);
            *reinterpret_cast<uint4*>(drow + 2 * NP + v * 8) = make_uint4(o2[0], o2[1], o2[2], o2[3]);
          }
        }
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
      };

      prefetch(T - 1);
      produce(T - 1);
      for (int t = T - 1; t >= 0; --t, ++g) {
        if (t > 0) prefetch(t - 1);
        float c0 = 0.f;
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          mbar_wait(bars + OFF_D_FULL + 8 * s, g & 1u, wctx, 307);
          tcgen05_fence_after();
          if (s == 0) {
            uint32_t sraw;
            tmem_ld1(tmem_base + lane_base + SUM_COL, &sraw);  // sum_i delta_t[b,i]
            tmem_ld_wait();
            c0 = J0 * __uint_as_float(sraw);
          }
#pragma unroll
          for (int c16 = 0; c16 < 2; ++c16) {
            uint32_t zo[16], zl[16], zr[16];
            const uint32_t col = tmem_base + lane_base + s * 256 + 32 * h + 16 * c16;
            tmem_ld16(col, zo);
            tmem_ld16(col + 64, zl);
            tmem_ld16(col + 128, zr);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int idx = s * 32 + c16 * 16 + j;
              float c = fmaf(beta, master[idx], c0);
              c = fmaf(J1, __uint_as_float(zo[j]), c);
              c = fmaf(L, __uint_as_float(zl[j]), c);
              c = fmaf(R, __uint_as_float(zr[j]), c);
              master[idx] = (nq + 64 * s + c16 * 16 + j < p.N) ? c : 0.f;
            }
          }
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(bars + OFF_D_EMPTY + 8 * s);
        }
        mbar_wait<true>(bars + OFF_ALL_FREE, g & 1u, wctx, 308);
        if (t > 0) {
          produce(t - 1);
        } else if (p.grad_r_init != nullptr && valid) {
#pragma unroll
          for (int s = 0; s < 2; ++s)
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nq + 64 * s + j < p.N) p.grad_r_init[(size_t)b * p.N + nq + 64 * s + j] = master[s * 32 + j];
        }
      }
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (C > 1) {
    cluster_arrive();
    cluster_wait();
  }
  if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int NP>
static int launch_bwd_tc(const CUtensorMap& tmW, const TcBwdParams& p, cudaStream_t s) {
  using C_ = Cfg<NP>;
  RINGRNN_CUDA_TRY(cudaFuncSetAttribute(bwd_tc_kernel<NP>, cudaFuncAttributeMaxDynamicSharedMemorySize, C_::SMEM));
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
    LaunchScope ls(K_BWD, s);
    RINGRNN_CUDA_TRY(cudaLaunchKernelEx(&cfg, bwd_tc_kernel<NP>, tmW, p));
  }
  return RINGRNN_OK;
}

int tc_backward_launch(int NP, const CUtensorMap& tmW, const void* params, cudaStream_t s) {
  const TcBwdParams& p = *static_cast<const TcBwdParams*>(params);  // same field order as the host-side mirror
  if (NP == 128) return launch_bwd_tc<128>(tmW, p, s);
  if (NP == 256) return launch_bwd_tc<256>(tmW, p, s);
  if (NP == 512) return launch_bwd_tc<512>(tmW, p, s);
  return RINGRNN_ERR_UNSUPPORTED;
}

}  // namespace ringrnn
