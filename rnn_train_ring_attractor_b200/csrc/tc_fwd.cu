// bf16 mode, forward: one persistent tcgen05 kernel runs all T timesteps of a 128-sample tile on a
// thread-block cluster (see tc_recurrent.cuh for the decomposition).  Replaces the T launches of
// fwd_wmma_kernel (cpp/kernels/fwd_1loop_tc_idx.cuh:265-277), which rebuild the per-sample effective
// weight matrix on tensor cores and do the actual recurrence on CUDA cores.
//
// Per step and MMA unit:   D_s[128 or 256, RB] = r_{t-1}[.., NP] x Wblock_s^T      (s = 0, 1; fp32 in TMEM)
// epilogue (thread = sample):   re = J0*S + J1*Yo + L*Yl + R*Yr,  r_t = (1-alpha) r_{t-1} + alpha F(re)
// with the fp32 master copy of r in registers; bf16(r_t) goes to the A buffers of all CTAs of the cluster
// for the next step, to the saved state, and F'(re) (bf16) to the saved derivative history; optional fp32
// history and per-step decode sums (r.u, r.v, sum|r|).
#include <string.h>

#include "tc_recurrent.cuh"

namespace ringrnn {

using namespace tc;
using namespace tcr;


// GEN: more than two active action columns -- the weights come in p.ng groups of three matrices, and the epilogue
// gathers the pre-activation over the groups before it applies F (one K round, no CTA pairs).
template <int ACT, int NP, bool PAIR, bool GEN>
__global__ void __launch_bounds__(THREADS, 1)
fwd_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmR0, const TcFwdParams p) {
  using C_ = Cfg<NP, PAIR>;
  static_assert(!GEN || (C_::ROUNDS == 1 && !PAIR), "weight groups: one K round, single CTAs");
  constexpr bool EARLY = C_::EARLY && !GEN;  // chunk 0 of a step is published while sub-slice 1 is still being worked on
  extern __shared__ uint8_t smem_raw[];
  const Ctx<NP, PAIR> c = setup_cta<NP, PAIR>(smem_raw, p.dec_u, p.dec_v, p.N, p.status);
  const int ng = GEN ? p.ng : 1;
  const uint32_t a_base = c.a_base, bars = c.bars, tmem_base = c.tmem_base;
  const WaitCtx& wctx = c.wctx;
  float* uv = c.uv;
  const int q = c.q;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int cluster_id = blockIdx.x / C_::CL, n_clusters = gridDim.x / C_::CL;
  const int T = p.T;
  const int my_tiles = (p.n_tiles - cluster_id + n_clusters - 1) / n_clusters;
  const uint32_t total_steps = (uint32_t)my_tiles * (uint32_t)T;

  if (warp < 4) {
    reg_dec<LOW_REGS>();
    if (warp == 0 && lane == 0) {
#ifdef RINGRNN_NO_SPLIT
      producer_loop<NP, PAIR, GEN>(c, &tmW, total_steps, 202, ng);
#else
      producer_loop<NP, PAIR, GEN, EARLY>(c, &tmW, total_steps, 202, ng);
#endif
    } else if (warp == 1 && lane == 0) {
      if (c.leader) mma_loop<NP, PAIR, true, GEN>(c, total_steps, T, 210, p.Rh != nullptr || (C_::PULL && p.X != nullptr), ng);
    } else if (warp == 2 && lane == 0) {
      tma_prefetch_desc(&tmR0);
      relay_loop<NP, PAIR, true, EARLY>(c, total_steps, T, 220, [&](int it, int round) {
        // initial state of the tile: this CTA's 128 samples, the K chunks of this round (the MMAs that read the
        // slots before are done: the relay has seen every phase of mma_done)
        const int tile = cluster_id + it * n_clusters;
        for (int slot = 0; slot < C_::SLOTS; ++slot) {
          mbar_arrive_expect_tx(bars + OFF_A_FULL + 8 * slot, CHUNK_BYTES);
          tma_load_2d(a_base + slot * CHUNK_BYTES, &tmR0, bars + OFF_A_FULL + 8 * slot, (round * C_::SLOTS + slot) * 64,
                      tile * C_::TILE_ROWS + c.half * 128);
        }
      });
    } else if (warp == 3) {
      if constexpr (EARLY)
        sender_loop<NP, PAIR>(c, total_steps, T, 230, p.Rh != nullptr ? &tmR0 : nullptr, p.BP, cluster_id, n_clusters);
      else if constexpr (C_::PULL) {
        if (p.X != nullptr && T > 1)
          puller_loop<NP, PAIR, true>(c, total_steps, T, 230, &tmR0, p.BP, cluster_id, n_clusters, p.x_ring != 0);
      }
    }
  } else {
    reg_inc<HIGH_REGS>();
    // ---------------- epilogue: thread = sample.  Warps 4-7 (h = 0) own columns [0,32) and warps 8-11 (h = 1)
    // columns [32,64) of BOTH 64-neuron sub-slices, so every accumulator is drained by all eight warps at once
    // (two warps per scheduler) and the part of the step that nothing overlaps -- the epilogue of the last
    // sub-slice -- is 32 elements per thread.  master[s*32 + j] is neuron 128q + 64s + 32h + j. ----------------
    const int h = (warp - 4) >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int nq = q * 128 + 32 * h;  // neuron of master[0]; sub-slice s adds 64*s
    const int slot = 2 * q + h;
    const float J0 = p.J0, J1 = p.J1, alpha = p.alpha, beta = 1.f - p.alpha;
    const bool want_dec = p.dec_part != nullptr;
    const bool padded = p.N != NP;  // some of the NP columns are padding
    const int rq = (2 * q) / C_::SLOTS;  // the K round this CTA's own chunks belong to
    FreePhases<NP, PAIR> freed;
    // exchange through global memory (Cfg::PULL): the state is written from registers and flagged; nothing here waits
    // for the peers' slots
    const bool pull = C_::PULL && p.X != nullptr;
    uint32_t n_pub = 0;
    uint32_t g = 0;
    uint32_t n_sent = 0, sent_waited = 0;  // early publication: copies of own chunk 0 sent / known to have arrived
    bool stop = false;  // a wait of this CTA was abandoned (the status word says which): same value in all 256 threads
    for (int tile = cluster_id; tile < p.n_tiles && !stop; tile += n_clusters) {
      const int b = tile * C_::TILE_ROWS + c.half * 128 + row;
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
        // this sample's action scalars (read only if valid)
        const float* at = p.A + ((size_t)b * p.T_total + p.t0 + t) * p.a_dim;
        float L = 0.f, R = 0.f;
        if (!GEN && valid) {
          if (p.colL >= 0) L = __ldg(at + p.colL);
          if (p.colR >= 0) R = __ldg(at + p.colR);
        }
        uint32_t packed[32];
        f32x2 px2 = pk2(0.f, 0.f), py2 = pk2(0.f, 0.f);  // decode sums, even / odd columns apart
        float pa = 0.f, c0 = 0.f;
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          // The pre-activation of this thread's 32 neurons of sub-slice s.  Two active columns: one accumulator holds
          // the three products, mixed inside the activation loop below (yo, yl, yr).  Weight groups: one accumulator
          // per group, summed here into re_all.
          uint32_t yo[GEN ? 1 : 32], yl[GEN ? 1 : 32], yr[GEN ? 1 : 32];
          float re_all[GEN ? 32 : 1];
          if constexpr (!GEN) {
            mbar_wait(bars + OFF_D_FULL + 8 * s, g & 1u, wctx, 207);
            if (warp == 4 && lane == 0) RINGRNN_STAMP(g, s == 0 ? 5 : 7);
            tcgen05_fence_after();
            if (s == 0 && !pull) freed.early(c, g, 208);
            // Last step of a tile: nothing is published, and the next tile's first operand comes by TMA, so its MMAs
            // wait for nothing but this accumulator.  The step's "free" phases must be consumed BEFORE the accumulator
            // is handed back, or the barrier could complete another phase first and the parity wait below would
            // never return.  (They complete together with this accumulator, give or take the skew between the CTAs.)
            if (s == 1 && t + 1 == T && !pull) freed.end_of_step(c, g, 208);
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
            release_accumulator<NP, PAIR>(c, s, lane);  // the accumulator is in registers: hand it back
          } else {
            for (int grp = 0; grp < ng; ++grp) {
              // coefficients of the group's three matrices: J1 for Wo, the action scalar for an action matrix
              float k0, k1 = 0.f, k2 = 0.f;
              {
                const int i0 = 3 * grp - 1;  // index into cols[] of the group's first matrix (-1: Wo)
                k0 = (grp == 0) ? J1 : ((valid && i0 < p.n_act) ? __ldg(at + p.cols[i0]) : 0.f);
                if (valid && i0 + 1 < p.n_act) k1 = __ldg(at + p.cols[i0 + 1]);
                if (valid && i0 + 2 < p.n_act) k2 = __ldg(at + p.cols[i0 + 2]);
              }
              const uint32_t pass = (g * 2u + (uint32_t)s) * (uint32_t)ng + (uint32_t)grp, acc = pass & 1u;
              mbar_wait(bars + OFF_D_FULL + 8 * acc, (pass >> 1) & 1u, wctx, 207);
              tcgen05_fence_after();
              // last pass of the last step of a tile: see the comment in the two-column branch
              if (s == 1 && grp == ng - 1 && t + 1 == T) freed.end_of_step(c, g, 208);
              const uint32_t col = tmem_base + lane_base + acc * 256 + 32 * h;
              if (s == 0 && grp == 0) {
                uint32_t sraw;
                tmem_ld1(tmem_base + lane_base + acc * 256 + SUM_COL, &sraw);  // row sum of r_{t-1}
                tmem_ld_wait();
                c0 = J0 * __uint_as_float(sraw);
              }
#pragma unroll
              for (int c16 = 0; c16 < 2; ++c16) {
                uint32_t z0[16], z1[16], z2[16];
                tmem_ld16(col + 16 * c16, z0);
                tmem_ld16(col + 64 + 16 * c16, z1);
                tmem_ld16(col + 128 + 16 * c16, z2);
                tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  float v = (grp == 0) ? c0 : re_all[16 * c16 + j];
                  v = fmaf(k0, __uint_as_float(z0[j]), v);
                  v = fmaf(k1, __uint_as_float(z1[j]), v);
                  re_all[16 * c16 + j] = fmaf(k2, __uint_as_float(z2[j]), v);
                }
              }
              release_accumulator<NP, PAIR>(c, (int)acc, lane);
            }
          }
          if (warp == 4 && lane == 0) RINGRNN_STAMP(g, s == 0 ? 6 : 8);
          // Sign masks of r_t for the backward's d|r|/dr (bit j = this thread's j-th neuron of the sub-slice): the sign
          // bits, shifted in with one instruction per element (first element ends up in bit 31, undone by one bit
          // reversal), and a mask of exact zeros (sign(0) = 0), which is only worked out when min_mag -- the smallest
          // magnitude seen -- says there is one.
          uint32_t dpk[16], negr = 0u;
          float min_mag = 3.0e38f;
          const f32x2 J1p = pk2(J1, J1), Lp = pk2(L, L), Rp = pk2(R, R), c0p = pk2(c0, c0), alphap = pk2(alpha, alpha),
                      betap = pk2(beta, beta);
#pragma unroll
          for (int j0 = 0; j0 < 32; j0 += 8) {
            // eight neurons as four packed pairs
            f32x2 re2[4], f2[4], d2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int e = j0 + 2 * i;
              if constexpr (GEN) {
                re2[i] = pk2(re_all[e], re_all[e + 1]);
              } else {
                f32x2 v = fma2(J1p, pk2u(yo[e], yo[e + 1]), c0p);
                v = fma2(Lp, pk2u(yl[e], yl[e + 1]), v);
                re2[i] = fma2(Rp, pk2u(yr[e], yr[e + 1]), v);
              }
            }
            act_group2<ACT, 8>(re2, f2, d2);
            float f[8], d[8];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              upk2(f2[i], f[2 * i], f[2 * i + 1]);
              upk2(d2[i], d[2 * i], d[2 * i + 1]);
            }
            if (padded) {  // neurons beyond N stay at zero (their master state is zero): one uniform branch per group
#pragma unroll
              for (int e = 0; e < 8; ++e)
                if (nq + 64 * s + j0 + e >= p.N) { f[e] = 0.f; d[e] = 0.f; }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int idx = s * 32 + j0 + 2 * i;
              const f32x2 r2 = fma2(alphap, pk2(f[2 * i], f[2 * i + 1]), mul2(betap, pk2(master[idx], master[idx + 1])));
              upk2(r2, master[idx], master[idx + 1]);
              f[2 * i] = master[idx];
              f[2 * i + 1] = master[idx + 1];
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              negr = __funnelshift_l(__float_as_uint(f[e]), negr, 1);  // (negr << 1) | sign bit of r
              min_mag = fminf(min_mag, fabsf(f[e]));
            }
            if (want_dec) {
              // the group's eight decode weights in four 16-byte shared-memory loads (same address in every lane)
              const float4* up = reinterpret_cast<const float4*>(uv + 64 * s + 32 * h + j0);
              const float4* vp = reinterpret_cast<const float4*>(uv + 128 + 64 * s + 32 * h + j0);
              const float4 u0 = up[0], u1 = up[1], v0 = vp[0], v1 = vp[1];
              const f32x2 uu[4] = {pk2(u0.x, u0.y), pk2(u0.z, u0.w), pk2(u1.x, u1.y), pk2(u1.z, u1.w)};
              const f32x2 vv[4] = {pk2(v0.x, v0.y), pk2(v0.z, v0.w), pk2(v1.x, v1.y), pk2(v1.z, v1.w)};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const f32x2 r2 = pk2(f[2 * i], f[2 * i + 1]);
                px2 = fma2(r2, uu[i], px2);
                py2 = fma2(r2, vv[i], py2);
                pa += fabsf(f[2 * i]) + fabsf(f[2 * i + 1]);
              }
            }
#pragma unroll
            for (int e = 0; e < 8; e += 2) {
              packed[s * 16 + ((j0 + e) >> 1)] = pack_bf16x2(f[e], f[e + 1]);
              dpk[(j0 + e) >> 1] = pack_bf16x2(d[e], d[e + 1]);
            }
          }
          if (p.Dh != nullptr) {
            const int n32 = (nq + 64 * s) >> 5;
            store_blocked(p.Dh + blocked_offset(t, b, n32, p.BP, NP), lane, dpk);
            uint32_t zero = 0u;
            if (min_mag == 0.f) {  // an exact zero among the 32 (always so for padding columns): mark them
#pragma unroll
              for (int j = 0; j < 32; ++j) zero |= (master[s * 32 + j] == 0.f ? 1u : 0u) << j;
            }
            uint32_t* sg = p.Sg + (((size_t)t * (NP >> 5) + n32) * 2) * p.BP + b;
            sg[0] = zero;
            sg[p.BP] = __brev(negr);
          }
          if constexpr (EARLY) {
            if (s == 0) {
              // this CTA's MMAs no longer read the slot of its own chunk 0 (one phase per step, consumed every step)
              mbar_wait(bars + OFF_OWN0_FREE, g & 1u, wctx, 209);
              if (t + 1 < T) {
                // ... every copy sent out of that slot so far has arrived at its peer, and the TMA store has read it
                while (sent_waited < n_sent) {
                  mbar_wait<true>(bars + OFF_SENT_DONE, sent_waited & 1u, wctx, 209);
                  mbar_wait(bars + OFF_STORE0_DONE, sent_waited & 1u, wctx, 209);
                  ++sent_waited;
                }
                write_chunk<NP, PAIR>(c, packed, 0, row, h);
                named_bar_arrive(SENDER_BAR, SENDER_BAR_THREADS);  // hand it to the sender thread and carry on
                ++n_sent;
              }
            }
          }
        }
        if (stop) break;
        // every CTA of the cluster has finished reading what the slots of this CTA's chunks held (every phase of
        // the barriers is waited for, published or not, so that none is skipped); then publish r_t:
        // it becomes the A operand of step t+1 everywhere and, in training, row block t+1 of the saved state
        if (warp == 4 && lane == 0) RINGRNN_STAMP(g, 9);
        if (C_::PULL && pull) {
          if (t + 1 < T) {
            const int rb = p.x_ring ? 1 + ((t + 1) & 1) : t + 1;
            stop = publish_global<NP, PAIR>(c, packed, h, warp, lane, p.X + ((size_t)rb * p.BP + b) * NP + q * 128, (size_t)NP,
                                            n_pub++);
            if (stop) break;
          }
        } else if (t + 1 < T) {
          freed.before_publish(c, g + 1, rq, 208);
          if (warp == 4 && lane == 0) RINGRNN_STAMP(g, 10);
          if constexpr (EARLY) {
            // chunk 1: the TMA stores issued so far have finished reading the slots (the issuing thread waits before
            // it arrives), then write, then send
            if (p.Rh != nullptr) {
              if (warp == 4 && lane == 0) bulk_wait_read<0>();
              named_bar_sync(2, 256);
            }
            write_chunk<NP, PAIR>(c, packed + 16, 1, row, h);
            stop = send_chunk<NP, PAIR>(c, 1, warp, lane, 1, p.Rh != nullptr ? &tmR0 : nullptr, q * 128,
                                        (t + 1) * p.BP + tile * C_::TILE_ROWS + c.half * 128);
          } else {
            stop = publish_chunks<NP, PAIR>(c, packed, row, h, warp, lane, p.Rh != nullptr ? &tmR0 : nullptr, q * 128,
                                            (t + 1) * p.BP + tile * C_::TILE_ROWS + c.half * 128);
          }
          if (stop) break;
        } else {
          freed.end_of_step(c, g, 208);
        }
        if (warp == 4 && lane == 0) RINGRNN_STAMP(g, 11);
        // off the critical path: checkpoint of the fp32 state, fp32 history, decode sums
        if (p.ckpt != nullptr && valid && t + 1 < T && (t + 1) % p.ckpt_every == 0) {
          float* dst = p.ckpt + ((size_t)((t + 1) / p.ckpt_every) * p.B + b) * p.N + nq;
#pragma unroll
          for (int s = 0; s < 2; ++s)
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nq + 64 * s + j < p.N) dst[64 * s + j] = master[s * 32 + j];
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
          float pxa, pxb, pya, pyb;
          upk2(px2, pxa, pxb);
          upk2(py2, pya, pyb);
          dp[0] = pxa + pxb;
          dp[(size_t)T * p.BP] = pya + pyb;
          dp[(size_t)2 * T * p.BP] = pa;
        }
      }
      if (stop) break;
      if (p.final_state != nullptr && valid) {
#pragma unroll
        for (int s = 0; s < 2; ++s)
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (nq + 64 * s + j < p.N) p.final_state[(size_t)b * p.N + nq + 64 * s + j] = master[s * 32 + j];
      }
    }
    if (EARLY && stop) named_bar_arrive(SENDER_BAR, SENDER_BAR_THREADS);  // a sender waiting for the next chunk 0 is let go
    if (warp == 4 && lane == 0) bulk_wait_all<0>();  // the saved-state stores have left shared memory and landed
  }
  teardown_cta<NP, PAIR>(c);
}

template <int ACT, int NP, bool PAIR, bool GEN = false>
static int launch_fwd_tc(const CUtensorMap& tmW, const CUtensorMap& tmR0, const TcFwdParams& p, cudaStream_t s) {
  using C_ = Cfg<NP, PAIR>;
  auto kernel = fwd_tc_kernel<ACT, NP, PAIR, GEN>;
  RINGRNN_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C_::SMEM));
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.blockDim = dim3(THREADS, 1, 1);
  cfg.dynamicSmemBytes = C_::SMEM;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = C_::CL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const int n_clusters = clusters_to_launch(reinterpret_cast<const void*>(kernel), &cfg, C_::CL, p.n_tiles);
  cfg.gridDim = dim3(n_clusters * C_::CL, 1, 1);
  {
    LaunchScope ls(K_FWD, s);
    RINGRNN_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, tmW, tmR0, p));
  }
  return RINGRNN_OK;
}

int tc_forward_launch(int act, int NP, bool pair, const CUtensorMap& tmW, const CUtensorMap& tmR0, const TcFwdParams& p,
                      cudaStream_t s) {
  if (p.ng > 1) {  // more than two active action columns
    if (pair) return RINGRNN_ERR_UNSUPPORTED;
#define RINGRNN_TCG(ACT, NPV) \
  if (act == ACT && NP == NPV) return launch_fwd_tc<ACT, NPV, false, true>(tmW, tmR0, p, s);
    RINGRNN_TCG(RINGRNN_ACT_RELU, 128) RINGRNN_TCG(RINGRNN_ACT_RELU, 256) RINGRNN_TCG(RINGRNN_ACT_RELU, 512)
    RINGRNN_TCG(RINGRNN_ACT_GELU, 128) RINGRNN_TCG(RINGRNN_ACT_GELU, 256) RINGRNN_TCG(RINGRNN_ACT_GELU, 512)
    RINGRNN_TCG(RINGRNN_ACT_TANH, 128) RINGRNN_TCG(RINGRNN_ACT_TANH, 256) RINGRNN_TCG(RINGRNN_ACT_TANH, 512)
    RINGRNN_TCG(RINGRNN_ACT_SILU, 128) RINGRNN_TCG(RINGRNN_ACT_SILU, 256) RINGRNN_TCG(RINGRNN_ACT_SILU, 512)
#undef RINGRNN_TCG
    return RINGRNN_ERR_UNSUPPORTED;
  }
#define RINGRNN_TCF(ACT, NPV)                                                              \
  if (act == ACT && NP == NPV)                                                             \
    return pair ? launch_fwd_tc<ACT, NPV, true>(tmW, tmR0, p, s) : launch_fwd_tc<ACT, NPV, false>(tmW, tmR0, p, s);
  RINGRNN_TCF(RINGRNN_ACT_RELU, 128) RINGRNN_TCF(RINGRNN_ACT_RELU, 256) RINGRNN_TCF(RINGRNN_ACT_RELU, 512)
  RINGRNN_TCF(RINGRNN_ACT_GELU, 128) RINGRNN_TCF(RINGRNN_ACT_GELU, 256) RINGRNN_TCF(RINGRNN_ACT_GELU, 512)
  RINGRNN_TCF(RINGRNN_ACT_TANH, 128) RINGRNN_TCF(RINGRNN_ACT_TANH, 256) RINGRNN_TCF(RINGRNN_ACT_TANH, 512)
  RINGRNN_TCF(RINGRNN_ACT_SILU, 128) RINGRNN_TCF(RINGRNN_ACT_SILU, 256) RINGRNN_TCF(RINGRNN_ACT_SILU, 512)
#undef RINGRNN_TCF
  if (NP == 1024 && !pair) {  // two K rounds per step, clusters of 8
    if (act == RINGRNN_ACT_RELU) return launch_fwd_tc<RINGRNN_ACT_RELU, 1024, false>(tmW, tmR0, p, s);
    if (act == RINGRNN_ACT_GELU) return launch_fwd_tc<RINGRNN_ACT_GELU, 1024, false>(tmW, tmR0, p, s);
    if (act == RINGRNN_ACT_TANH) return launch_fwd_tc<RINGRNN_ACT_TANH, 1024, false>(tmW, tmR0, p, s);
    if (act == RINGRNN_ACT_SILU) return launch_fwd_tc<RINGRNN_ACT_SILU, 1024, false>(tmW, tmR0, p, s);
  }
  return RINGRNN_ERR_UNSUPPORTED;
}

}  // namespace ringrnn

#ifdef RINGRNN_TIMELINE
extern "C" int ringrnn_debug_timeline_read(long long* out) {
  return (int)cudaMemcpyFromSymbol(out, ringrnn::g_timeline, sizeof(long long) * 64 * 16);
}
#endif
