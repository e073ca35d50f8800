// bf16 mode, reverse-time: one persistent tcgen05 kernel propagates delta_t = alpha*F'(re_t)*g_t through the
// transposed weights for all T steps of a 128-sample tile (same cluster decomposition as the forward kernel,
// see tc_recurrent.cuh).  Replaces the per-step launches recompute_Weff_re_grad_re_kernel +
// compute_grad_r_kernel_vec (cpp/kernels/bwd_mixed_precision_aggressive.cuh:53-318), which write and re-read
// a [B,N,N] fp32 effective-weight tensor every step.
//
// Per step and MMA unit:   Z_s[128 or 256, RB] = delta_t[.., NP] x WblockT_s^T        (fp32 in TMEM)
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


// GEN: more than two active action columns -- the transposed weights come in p.ng groups of three matrices, the
// carry is gathered over the groups, and DL gets one scaled copy of delta per active column.
template <int NP, bool PAIR, bool GEN>
__global__ void __launch_bounds__(THREADS, 1)
bwd_tc_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmDL,
              const __grid_constant__ CUtensorMap tmDL32, const TcBwdParams p) {
  using C_ = Cfg<NP, PAIR>;
  static_assert(!GEN || (C_::ROUNDS == 1 && !PAIR), "weight groups: one K round, single CTAs");
  // Carry and delta arithmetic on packed fp32 pairs: fewer instructions, a few more registers (measured: -9 % at
  // N = 256, -8 % at N = 128; at N = 512 it cost 1.5 % while the scaled copies still went through shared-memory loads
  // and global stores, and gains 1.7 % now that they leave as TMA stores).
  constexpr bool PACKED = true;
  // delta of sub-slice 0 is published while accumulator 1 is still being filled (see Cfg::EARLY and sender_loop).
  // Measured at N = 512 (cluster of 4): -4.5 % on this kernel; at N = 256 (cluster of 2, half the exchange, a step a
  // third as long) the extra hand-over costs more than the overlap gains (+6 %), so it stays off there.
  constexpr bool EARLY = C_::EARLY && !GEN && NP >= 512;
  extern __shared__ uint8_t smem_raw[];
  const Ctx<NP, PAIR> c = setup_cta<NP, PAIR>(smem_raw, p.dec_u, p.dec_v, p.N, p.status);
  const int ng = GEN ? p.ng : 1;
  const int dl_blocks = GEN ? 1 + p.n_act : 3;  // column blocks of NP in a row of DL
  // The scaled copies of delta leave each epilogue warp's transposition buffer as one TMA store (store_rows_via_tma)
  // or through shared-memory loads and global stores (store_rows_via_smem).  Measured, reverse kernel: TMA -3 % at
  // N = 512, -8 % at N = 128, -2 % at N = 1024, but +5 % at N = 256, where the wait for the previous store's read of
  // the one buffer is not hidden.
  constexpr bool DL_BY_TMA = NP != 256;
  const uint32_t bars = c.bars, tmem_base = c.tmem_base;
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
      producer_loop<NP, PAIR, GEN>(c, &tmW, total_steps, 302, ng);
#else
      producer_loop<NP, PAIR, GEN, EARLY>(c, &tmW, total_steps, 302, ng);
#endif
    } else if (warp == 1 && lane == 0) {
      if (c.leader) mma_loop<NP, PAIR, false, GEN>(c, total_steps, T, 310, true, ng);
    } else if (warp == 2 && lane == 0) {
      relay_loop<NP, PAIR, false, EARLY>(c, total_steps, T, 320, [](int, int) {});
    } else if (warp == 3) {
      if constexpr (EARLY) sender_loop<NP, PAIR, false>(c, total_steps, T, 330, &tmDL, p.BP, cluster_id, n_clusters);
      else if constexpr (C_::PULL) puller_loop<NP, PAIR, false>(c, total_steps, T, 330, &tmDL, p.BP, cluster_id, n_clusters);
    }
  } else {
    reg_inc<HIGH_REGS>();
    // ---------------- epilogue: thread = sample.  Warps 4-7 (h = 0) own columns [0,32) and warps 8-11 (h = 1)
    // columns [32,64) of both 64-neuron sub-slices; master[s*32 + j] is neuron 128q + 64s + 32h + j. ----------------
    const int h = (warp - 4) >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const int nq = q * 128 + 32 * h;
    const float J0 = p.J0, J1 = p.J1, alpha = p.alpha, beta = 1.f - p.alpha;
    const bool has_coef = p.coef_x != nullptr;
    const bool want_dA = p.dA_part != nullptr;
    const int rq = (2 * q) / C_::SLOTS;  // the K round this CTA's own chunks belong to
    FreePhases<NP, PAIR> freed;
    // the warp's 32 rows x 32 columns `o` to DL at (first column x, first row y)
    auto store_copy = [&](const uint32_t* o, int x, int y) {
      const uint32_t stage = c.stage_base + (uint32_t)(warp - 4) * 2048u;
      if constexpr (DL_BY_TMA)
        store_rows_via_tma(stage, lane, o, &tmDL32, x, y);
      else
        store_rows_via_smem(stage, lane, o, reinterpret_cast<uint8_t*>(p.DL + (size_t)y * ((size_t)dl_blocks * NP) + x),
                            (size_t)dl_blocks * NP * 2);
    };
    uint32_t g = 0;
    uint32_t n_sent = 0, sent_waited = 0;  // early publication: sends of own chunk 0 handed over / known complete
    uint32_t n_pub = 0;                    // exchange through global memory: publications of this CTA
    bool stop = false;  // a wait of this CTA was abandoned (the status word says which): same value in all 256 threads
    for (int tile = cluster_id; tile < p.n_tiles && !stop; tile += n_clusters) {
      const int b = tile * C_::TILE_ROWS + c.half * 128 + row;
      const bool valid = b < p.B;
      float master[64];  // carry on entry of `produce`, g_t afterwards
#pragma unroll
      for (int s = 0; s < 2; ++s)
#pragma unroll
        for (int j = 0; j < 32; ++j) {
          const int n = nq + 64 * s + j;
          master[s * 32 + j] = (p.carry_in != nullptr && valid && n < p.N) ? __ldg(p.carry_in + (size_t)b * p.N + n) : 0.f;
        }
      float L = 0.f, R = 0.f;        // action scalars of the step whose delta is in flight
      float Ln = 0.f, Rn = 0.f, cx = 0.f, cy = 0.f, cs = 0.f;  // prefetched for the next `produce`
      uint4 dv[8];                   // prefetched F'(re_t) (bf16): [s*4 + v]
      uint32_t mzero[2], mneg[2];    // prefetched masks of r_t per sub-slice: exact zeros, sign bits

      // loads for produce(t); issued before the wait on the accumulators so that their latency is hidden
      auto prefetch = [&](int t) {
        Ln = 0.f; Rn = 0.f; cx = 0.f; cy = 0.f; cs = 0.f;
        if (valid) {
          const size_t bt = (size_t)b * p.T_total + p.t0 + t;
          const float* at = p.A + bt * p.a_dim;
          if (!GEN && p.colL >= 0) Ln = __ldg(at + p.colL);
          if (!GEN && p.colR >= 0) Rn = __ldg(at + p.colR);
          if (has_coef) {
            cx = __ldg(p.coef_x + bt);
            cy = __ldg(p.coef_y + bt);
            cs = __ldg(p.coef_s + bt);
          }
        }
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          const int n32 = (nq + 64 * s) >> 5;
          load_blocked(p.Dh + blocked_offset(t, b, n32, p.BP, NP), lane, dv + 4 * s);
          mzero[s] = 0u;
          mneg[s] = 0u;
          if (has_coef) {
            const uint32_t* sg = p.Sg + (((size_t)t * (NP >> 5) + n32) * 2) * p.BP + b;
            mzero[s] = __ldg(sg);
            mneg[s] = __ldg(sg + p.BP);
          }
        }
      };

      // delta_t of sub-slice s from the carry: adds dL/dr_t and applies alpha*F'(re_t) (uses the prefetched values).
      // packed[s*16 + w] receives the bf16 delta of neurons 2w, 2w+1 of sub-slice s.
      auto produce_half = [&](int t, int s, uint32_t* packed) {
        if (p.grad_output != nullptr && valid) {
          const float* gsrc = p.grad_output + ((size_t)(p.t0 + t) * p.B + b) * p.N + nq + 64 * s;
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
        const f32x2 cxp = pk2(cx, cx), cyp = pk2(cy, cy), onep = pk2(1.f, 1.f), alphap = pk2(alpha, alpha);
        // d|r|/dr = sign(r_t) is applied below as +cs or -cs by the sign bit alone (two instructions per element);
        // where r_t is an exact zero (rare; always so for padding columns) the term must vanish: take it out of
        // the carry beforehand
        if (has_coef && mzero[s] != 0u) {
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (mzero[s] & (1u << j)) master[s * 32 + j] -= (mneg[s] & (1u << j)) ? -cs : cs;
        }
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint32_t dw[4] = {dv[s * 4 + v].x, dv[s * 4 + v].y, dv[s * 4 + v].z, dv[s * 4 + v].w};
          // the eight decode weights of this group in four 16-byte shared-memory loads (same address in every lane)
          float uu[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, vv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          if (has_coef) {
            const float4* up = reinterpret_cast<const float4*>(uv + 64 * s + 32 * h + 8 * v);
            const float4* vp = reinterpret_cast<const float4*>(uv + 128 + 64 * s + 32 * h + 8 * v);
            const float4 u0 = up[0], u1 = up[1], v0 = vp[0], v1 = vp[1];
            uu[0] = u0.x; uu[1] = u0.y; uu[2] = u0.z; uu[3] = u0.w; uu[4] = u1.x; uu[5] = u1.y; uu[6] = u1.z; uu[7] = u1.w;
            vv[0] = v0.x; vv[1] = v0.y; vv[2] = v0.z; vv[3] = v0.w; vv[4] = v1.x; vv[5] = v1.y; vv[6] = v1.z; vv[7] = v1.w;
          }
#pragma unroll
          for (int w = 0; w < 4; ++w) {  // two neurons at a time
            const int j = v * 8 + w * 2;
            const int idx = s * 32 + j;
            if constexpr (PACKED) {
              f32x2 gg = pk2(master[idx], master[idx + 1]);
              if (has_coef) {
                gg = fma2(cxp, pk2(uu[w * 2], uu[w * 2 + 1]), gg);
                gg = fma2(cyp, pk2(vv[w * 2], vv[w * 2 + 1]), gg);
                // + cs * sign(r_t) by the sign bit; exact zeros were pre-compensated
                gg = fma2(onep, pk2((mneg[s] & (1u << j)) ? -cs : cs, (mneg[s] & (2u << j)) ? -cs : cs), gg);
              }
              upk2(gg, master[idx], master[idx + 1]);
              float d0, d1;
              upk2(mul2(mul2(alphap, pk2(bf16_lo(dw[w]), bf16_hi(dw[w]))), gg), d0, d1);
              packed[s * 16 + v * 4 + w] = pack_bf16x2(d0, d1);
            } else {
              float dl[2];
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                float gg = master[idx + e];
                if (has_coef) {
                  gg = fmaf(cx, uu[w * 2 + e], gg);
                  gg = fmaf(cy, vv[w * 2 + e], gg);
                  gg += (mneg[s] & (1u << (j + e))) ? -cs : cs;  // + cs * sign(r_t); exact zeros were pre-compensated
                }
                master[idx + e] = gg;
                dl[e] = alpha * (e ? bf16_hi(dw[w]) : bf16_lo(dw[w])) * gg;
              }
              packed[s * 16 + v * 4 + w] = pack_bf16x2(dl[0], dl[1]);
            }
          }
        }
      };

      // [L*delta | R*delta] of sub-slice s for the weight-gradient GEMM (two active columns; off the critical path).  The
      // scaled copies are formed from the bf16 delta the MMA sees, so the three blocks are consistent with one another;
      // packed bf16 multiplies (one instruction per two elements): the action scalar is rounded to bf16 first.
      auto dl_copies = [&](int t, int s, float Ls, float Rs, const uint32_t* packed) {
        // row 0 of this warp's 32-row block, first of this thread's 32 columns within a column block
        const int y0 = t * p.BP + (b - lane), x0 = nq + 64 * s;
        const uint32_t L2 = pack_bf16x2(Ls, Ls), R2 = pack_bf16x2(Rs, Rs);
        uint32_t o[16];
#pragma unroll
        for (int w = 0; w < 16; ++w) o[w] = mul_bf16x2(packed[s * 16 + w], L2);
        store_copy(o, NP + x0, y0);
#pragma unroll
        for (int w = 0; w < 16; ++w) o[w] = mul_bf16x2(packed[s * 16 + w], R2);
        store_copy(o, 2 * NP + x0, y0);
      };
      // one scaled copy per active column (weight groups): block 1 + k = A[b,t,cols[k]] * delta_t
      auto dl_copies_generic = [&](int t, const uint32_t* packed) {
        const float* at = p.A + ((size_t)b * p.T_total + p.t0 + t) * p.a_dim;
        for (int k = 0; k < p.n_act; ++k) {
          const float ak = valid ? __ldg(at + p.cols[k]) : 0.f;
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            uint32_t o[16];
#pragma unroll
            for (int w = 0; w < 16; ++w) {
              const uint32_t d2 = packed[s * 16 + w];
              o[w] = pack_bf16x2(ak * bf16_lo(d2), ak * bf16_hi(d2));
            }
            store_copy(o, (1 + k) * NP + nq + 64 * s, t * p.BP + (b - lane));
          }
        }
      };

      // early publication of chunk 0 of delta_t: into this CTA's own slot, then over to the sender thread
      auto hand_over_chunk0 = [&](const uint32_t* packed) {
        while (sent_waited < n_sent) {  // the previous copies out of that slot have arrived, the TMA store has read it
          mbar_wait<true>(bars + OFF_SENT_DONE, sent_waited & 1u, wctx, 309);
          mbar_wait(bars + OFF_STORE0_DONE, sent_waited & 1u, wctx, 309);
          ++sent_waited;
        }
        write_chunk<NP, PAIR>(c, packed, 0, row, h);
        named_bar_arrive(SENDER_BAR, SENDER_BAR_THREADS);
        ++n_sent;
      };
      // chunk 1 of delta_t: write, then one epilogue thread sends it (delta_t is also column block 0 of DL row block t)
      auto publish_chunk1 = [&](int t, const uint32_t* packed) {
        if (warp == 4 && lane == 0) bulk_wait_read<0>();  // the TMA stores issued so far have read the slot
        named_bar_sync(2, 256);
        write_chunk<NP, PAIR>(c, packed + 16, 1, row, h);
        stop = send_chunk<NP, PAIR>(c, 1, warp, lane, 1, &tmDL, q * 128, t * p.BP + tile * C_::TILE_ROWS + c.half * 128);
      };

      // Both sub-slices at once, published together (CTA pairs, two K rounds, weight groups, a single slice, N = 256):
      // delta_t from the carry: adds dL/dr_t, applies alpha*F'(re_t), publishes the bf16 chunks, writes DL
      auto produce = [&](int t) {
        L = Ln;
        R = Rn;
        if (p.grad_output != nullptr && valid) {
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            const float* gsrc = p.grad_output + ((size_t)(p.t0 + t) * p.B + b) * p.N + nq + 64 * s;
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
        const f32x2 cxp = pk2(cx, cx), cyp = pk2(cy, cy), onep = pk2(1.f, 1.f), alphap = pk2(alpha, alpha);
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          // d|r|/dr = sign(r_t) is applied below as +cs or -cs by the sign bit alone (two instructions per element);
          // where r_t is an exact zero (rare; always so for padding columns) the term must vanish: take it out of
          // the carry beforehand
          if (has_coef && mzero[s] != 0u) {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (mzero[s] & (1u << j)) master[s * 32 + j] -= (mneg[s] & (1u << j)) ? -cs : cs;
          }
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const uint32_t dw[4] = {dv[s * 4 + v].x, dv[s * 4 + v].y, dv[s * 4 + v].z, dv[s * 4 + v].w};
            // the eight decode weights of this group in four 16-byte shared-memory loads (same address in every lane)
            float uu[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, vv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (has_coef) {
              const float4* up = reinterpret_cast<const float4*>(uv + 64 * s + 32 * h + 8 * v);
              const float4* vp = reinterpret_cast<const float4*>(uv + 128 + 64 * s + 32 * h + 8 * v);
              const float4 u0 = up[0], u1 = up[1], v0 = vp[0], v1 = vp[1];
              uu[0] = u0.x; uu[1] = u0.y; uu[2] = u0.z; uu[3] = u0.w; uu[4] = u1.x; uu[5] = u1.y; uu[6] = u1.z; uu[7] = u1.w;
              vv[0] = v0.x; vv[1] = v0.y; vv[2] = v0.z; vv[3] = v0.w; vv[4] = v1.x; vv[5] = v1.y; vv[6] = v1.z; vv[7] = v1.w;
            }
#pragma unroll
            for (int w = 0; w < 4; ++w) {  // two neurons at a time
              const int j = v * 8 + w * 2;
              const int idx = s * 32 + j;
              if constexpr (PACKED) {
                f32x2 gg = pk2(master[idx], master[idx + 1]);
                if (has_coef) {
                  gg = fma2(cxp, pk2(uu[w * 2], uu[w * 2 + 1]), gg);
                  gg = fma2(cyp, pk2(vv[w * 2], vv[w * 2 + 1]), gg);
                  // + cs * sign(r_t) by the sign bit; exact zeros were pre-compensated
                  gg = fma2(onep, pk2((mneg[s] & (1u << j)) ? -cs : cs, (mneg[s] & (2u << j)) ? -cs : cs), gg);
                }
                upk2(gg, master[idx], master[idx + 1]);
                float d0, d1;
                upk2(mul2(mul2(alphap, pk2(bf16_lo(dw[w]), bf16_hi(dw[w]))), gg), d0, d1);
                packed[s * 16 + v * 4 + w] = pack_bf16x2(d0, d1);
              } else {
                float dl[2];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                  float gg = master[idx + e];
                  if (has_coef) {
                    gg = fmaf(cx, uu[w * 2 + e], gg);
                    gg = fmaf(cy, vv[w * 2 + e], gg);
                    gg += (mneg[s] & (1u << (j + e))) ? -cs : cs;  // + cs * sign(r_t); exact zeros were pre-compensated
                  }
                  master[idx + e] = gg;
                  dl[e] = alpha * (e ? bf16_hi(dw[w]) : bf16_lo(dw[w])) * gg;
                }
                packed[s * 16 + v * 4 + w] = pack_bf16x2(dl[0], dl[1]);
              }
            }
          }
        }
        // delta_t: A operand of this step everywhere, and column block 0 of DL row block t (TMA store from the chunks)
        if constexpr (C_::PULL)  // straight from registers into DL; the CTAs of the cluster, this one too, fetch it from there
          stop = publish_global<NP, PAIR>(c, packed, h, warp, lane,
                                          p.DL + ((size_t)t * p.BP + b) * ((size_t)dl_blocks * NP) + q * 128,
                                          (size_t)dl_blocks * NP, n_pub++);
        else
          stop = publish_chunks<NP, PAIR>(c, packed, row, h, warp, lane, &tmDL, q * 128,
                                          t * p.BP + tile * C_::TILE_ROWS + c.half * 128);
        if (stop) return;
        if (warp == 4 && lane == 0) RINGRNN_STAMP(g, 12);
        // off the critical path: [delta | L*delta | R*delta] for the weight-gradient GEMM.  The scaled copies are
        // formed from the bf16 delta the MMA sees, so the three blocks are consistent with one another.
        if constexpr (!GEN) {
          // packed bf16 multiplies (one instruction per two elements): the action scalar is rounded to bf16 first
#pragma unroll
          for (int s = 0; s < 2; ++s) {
            // row 0 of this warp's 32-row block, first of this thread's 32 columns within a column block
            const int y0 = t * p.BP + (b - lane), x0 = nq + 64 * s;
            const uint32_t L2 = pack_bf16x2(L, L), R2 = pack_bf16x2(R, R);
            uint32_t o[16];
#pragma unroll
            for (int w = 0; w < 16; ++w) {
              o[w] = mul_bf16x2(packed[s * 16 + w], L2);
            }
            store_copy(o, NP + x0, y0);
#pragma unroll
            for (int w = 0; w < 16; ++w) {
              o[w] = mul_bf16x2(packed[s * 16 + w], R2);
            }
            store_copy(o, 2 * NP + x0, y0);
          }
        } else {
          // one scaled copy per active column: block 1 + k = A[b,t,cols[k]] * delta_t
          const float* at = p.A + ((size_t)b * p.T_total + p.t0 + t) * p.a_dim;
          for (int k = 0; k < p.n_act; ++k) {
            const float ak = valid ? __ldg(at + p.cols[k]) : 0.f;
#pragma unroll
            for (int s = 0; s < 2; ++s) {
              uint32_t o[16];
#pragma unroll
              for (int w = 0; w < 16; ++w) {
                const uint32_t d2 = packed[s * 16 + w];
                o[w] = pack_bf16x2(ak * bf16_lo(d2), ak * bf16_hi(d2));
              }
              store_copy(o, (1 + k) * NP + nq + 64 * s, t * p.BP + (b - lane));
            }
          }
        }
      };

      prefetch(T - 1);
      if (!C_::PULL) freed.before_publish(c, g, rq, 308);
      if constexpr (EARLY) {
        uint32_t packed[32];
        produce_half(T - 1, 0, packed);
        hand_over_chunk0(packed);
        produce_half(T - 1, 1, packed);
        publish_chunk1(T - 1, packed);
        if (stop) break;
        L = Ln;
        R = Rn;
        dl_copies(T - 1, 0, L, R, packed);
        dl_copies(T - 1, 1, L, R, packed);
      } else {
        produce(T - 1);
        if (stop) break;
      }
      for (int t = T - 1; t >= 0; --t, ++g) {
        if (t > 0) prefetch(t - 1);
        float c0 = 0.f, dAl = 0.f, dAr = 0.f;
        uint32_t packed[EARLY ? 32 : 1];  // (early publication) bf16 delta_{t-1}, produced sub-slice by sub-slice
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          if constexpr (GEN) {
            // carry of sub-slice s gathered over the weight groups; one accumulator per (s, group)
            const float* at = p.A + ((size_t)b * p.T_total + p.t0 + t) * p.a_dim;
            for (int grp = 0; grp < ng; ++grp) {
              const int i0 = 3 * grp - 1;  // index into cols[] of the group's first matrix (-1: Wo)
              float k0, k1 = 0.f, k2 = 0.f;
              k0 = (grp == 0) ? J1 : ((valid && i0 < p.n_act) ? __ldg(at + p.cols[i0]) : 0.f);
              if (valid && i0 + 1 < p.n_act) k1 = __ldg(at + p.cols[i0 + 1]);
              if (valid && i0 + 2 < p.n_act) k2 = __ldg(at + p.cols[i0 + 2]);
              const uint32_t pass = (g * 2u + (uint32_t)s) * (uint32_t)ng + (uint32_t)grp, acc = pass & 1u;
              mbar_wait(bars + OFF_D_FULL + 8 * acc, (pass >> 1) & 1u, wctx, 307);
              tcgen05_fence_after();
              if (s == 0 && grp == 0) {
                uint32_t sraw;
                tmem_ld1(tmem_base + lane_base + acc * 256 + SUM_COL, &sraw);  // sum_i delta_t[b,i]
                tmem_ld_wait();
                c0 = J0 * __uint_as_float(sraw);
              }
              float da0 = 0.f, da1 = 0.f, da2 = 0.f;
#pragma unroll
              for (int c16 = 0; c16 < 2; ++c16) {
                uint32_t z0[16], z1[16], z2[16];
                const uint32_t col = tmem_base + lane_base + acc * 256 + 32 * h + 16 * c16;
                tmem_ld16(col, z0);
                tmem_ld16(col + 64, z1);
                tmem_ld16(col + 128, z2);
                tmem_ld_wait();
                if (want_dA) {
                  // dL/dA[b,t,col] = sum_j r_{t-1}[j] (delta_t W_col)[j]: this thread's 16 columns
                  const uint4* rsrc = reinterpret_cast<const uint4*>(p.Rh + ((size_t)t * p.BP + b) * NP + nq + 64 * s + 16 * c16);
                  const uint4 r0 = __ldg(rsrc), r1 = __ldg(rsrc + 1);
                  const uint32_t rw[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
                  for (int j = 0; j < 16; ++j) {
                    const float rp = (j & 1) ? bf16_hi(rw[j >> 1]) : bf16_lo(rw[j >> 1]);
                    da0 = fmaf(rp, __uint_as_float(z0[j]), da0);
                    da1 = fmaf(rp, __uint_as_float(z1[j]), da1);
                    da2 = fmaf(rp, __uint_as_float(z2[j]), da2);
                  }
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  const int idx = s * 32 + c16 * 16 + j;
                  float cv = (grp == 0) ? fmaf(beta, master[idx], c0) : master[idx];
                  cv = fmaf(k0, __uint_as_float(z0[j]), cv);
                  cv = fmaf(k1, __uint_as_float(z1[j]), cv);
                  cv = fmaf(k2, __uint_as_float(z2[j]), cv);
                  master[idx] = cv;  // padding columns need no masking: their F' is zero, so their delta is
                }
              }
              release_accumulator<NP, PAIR>(c, (int)acc, lane);
              if (want_dA) {
                // partial sums [slot = ((2q+h)*2+s)][k][t][b] of the group's action matrices
                const size_t slot4 = (size_t)((2 * q + h) * 2 + s);
                const float dav[3] = {da0, da1, da2};
#pragma unroll
                for (int m = 0; m < 3; ++m) {
                  const int k = i0 + m;
                  if (k >= 0 && k < p.n_act) p.dA_part[((slot4 * p.n_act + k) * T + t) * p.BP + b] = dav[m];
                }
              }
            }
            continue;
          }
          mbar_wait(bars + OFF_D_FULL + 8 * s, g & 1u, wctx, 307);
          if (warp == 4 && lane == 0) RINGRNN_STAMP(g, s == 0 ? 5 : 7);
          tcgen05_fence_after();
          if (s == 0) {
            if (!C_::PULL) freed.early(c, g, 308);
            uint32_t sraw;
            tmem_ld1(tmem_base + lane_base + SUM_COL, &sraw);  // sum_i delta_t[b,i]
            tmem_ld_wait();
            c0 = J0 * __uint_as_float(sraw);
          }
          const f32x2 betap = pk2(beta, beta), c0p = pk2(c0, c0), J1p = pk2(J1, J1), Lp = pk2(L, L), Rp = pk2(R, R);
#pragma unroll
          for (int c16 = 0; c16 < 2; ++c16) {
            uint32_t zo[16], zl[16], zr[16];
            const uint32_t col = tmem_base + lane_base + s * 256 + 32 * h + 16 * c16;
            tmem_ld16(col, zo);
            tmem_ld16(col + 64, zl);
            tmem_ld16(col + 128, zr);
            tmem_ld_wait();
            if (want_dA) {
              // dL/dL_t = sum_j r_{t-1}[j] (delta_t Wl)[j], likewise for R: this thread's 16 columns
              const uint4* rsrc = reinterpret_cast<const uint4*>(p.Rh + ((size_t)t * p.BP + b) * NP + nq + 64 * s + 16 * c16);
              const uint4 r0 = __ldg(rsrc), r1 = __ldg(rsrc + 1);
              const uint32_t rw[8] = {r0.x, r0.y, r0.z, r0.w, r1.x, r1.y, r1.z, r1.w};
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float rp = (j & 1) ? bf16_hi(rw[j >> 1]) : bf16_lo(rw[j >> 1]);
                dAl = fmaf(rp, __uint_as_float(zl[j]), dAl);
                dAr = fmaf(rp, __uint_as_float(zr[j]), dAr);
              }
            }
            // padding columns need no masking: their F' is zero, so their delta is
            if constexpr (PACKED) {
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const int idx = s * 32 + c16 * 16 + 2 * i;
                f32x2 cv = fma2(betap, pk2(master[idx], master[idx + 1]), c0p);
                cv = fma2(J1p, pk2u(zo[2 * i], zo[2 * i + 1]), cv);
                cv = fma2(Lp, pk2u(zl[2 * i], zl[2 * i + 1]), cv);
                cv = fma2(Rp, pk2u(zr[2 * i], zr[2 * i + 1]), cv);
                upk2(cv, master[idx], master[idx + 1]);
              }
            } else {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const int idx = s * 32 + c16 * 16 + j;
                float cv = fmaf(beta, master[idx], c0);
                cv = fmaf(J1, __uint_as_float(zo[j]), cv);
                cv = fmaf(L, __uint_as_float(zl[j]), cv);
                cv = fmaf(R, __uint_as_float(zr[j]), cv);
                master[idx] = cv;
              }
            }
          }
          release_accumulator<NP, PAIR>(c, s, lane);
          if (warp == 4 && lane == 0) RINGRNN_STAMP(g, s == 0 ? 6 : 8);
          if constexpr (EARLY) {
            if (s == 0) {
              // this CTA's MMAs no longer read the slot of its own chunk 0 (one phase per step, consumed every step)
              mbar_wait(bars + OFF_OWN0_FREE, g & 1u, wctx, 309);
              if (t > 0) {
                // the carry of sub-slice 0 is complete: its delta goes out while accumulator 1 is still being filled,
                // and its scaled copies are written in the wait for that accumulator
                produce_half(t - 1, 0, packed);
                hand_over_chunk0(packed);
                dl_copies(t - 1, 0, Ln, Rn, packed);
              }
            }
          }
        }
        if (!GEN && want_dA) {
          float* dp = p.dA_part + (((size_t)(2 * q + h) * 2) * T + t) * p.BP + b;
          dp[0] = dAl;
          dp[(size_t)T * p.BP] = dAr;
        }
        if (warp == 4 && lane == 0) RINGRNN_STAMP(g, 9);
        if (!C_::PULL) {  // (with the exchange through global memory nothing here waits for the peers' slots)
          if (t > 0) freed.before_publish(c, g + 1, rq, 308);
          else freed.end_of_step(c, g, 308);
        }
        if (warp == 4 && lane == 0) RINGRNN_STAMP(g, 10);
        if (t > 0) {
          if constexpr (EARLY) {
            produce_half(t - 1, 1, packed);
            publish_chunk1(t - 1, packed);
            if (stop) break;
            if (warp == 4 && lane == 0) RINGRNN_STAMP(g, 12);
            L = Ln;
            R = Rn;
            dl_copies(t - 1, 1, L, R, packed);
          } else {
            produce(t - 1);
            if (stop) break;
          }
          if (warp == 4 && lane == 0) RINGRNN_STAMP(g, 11);
        } else if (p.grad_r_init != nullptr && valid) {
#pragma unroll
          for (int s = 0; s < 2; ++s)
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (nq + 64 * s + j < p.N) p.grad_r_init[(size_t)b * p.N + nq + 64 * s + j] = master[s * 32 + j];
        }
      }
    }
    if (EARLY && stop) named_bar_arrive(SENDER_BAR, SENDER_BAR_THREADS);  // a sender waiting for the next chunk 0 is let go
    if (lane == 0) bulk_wait_all<0>();  // this warp's stores (delta chunks, scaled copies) have left shared memory and landed
  }
  teardown_cta<NP, PAIR>(c);
}

template <int NP, bool PAIR, bool GEN = false>
static int launch_bwd_tc(const CUtensorMap& tmW, const CUtensorMap& tmDL, const CUtensorMap& tmDL32, const TcBwdParams& p,
                         cudaStream_t s) {
  using C_ = Cfg<NP, PAIR>;
  auto kernel = bwd_tc_kernel<NP, PAIR, GEN>;
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
    LaunchScope ls(K_BWD, s);
    RINGRNN_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, tmW, tmDL, tmDL32, p));
  }
  return RINGRNN_OK;
}

int tc_backward_launch(int NP, bool pair, const CUtensorMap& tmW, const CUtensorMap& tmDL, const CUtensorMap& tmDL32,
                       const TcBwdParams& p,
                       cudaStream_t s) {
  if (p.ng > 1) {  // more than two active action columns
    if (pair) return RINGRNN_ERR_UNSUPPORTED;
    if (NP == 128) return launch_bwd_tc<128, false, true>(tmW, tmDL, tmDL32, p, s);
    if (NP == 256) return launch_bwd_tc<256, false, true>(tmW, tmDL, tmDL32, p, s);
    if (NP == 512) return launch_bwd_tc<512, false, true>(tmW, tmDL, tmDL32, p, s);
    return RINGRNN_ERR_UNSUPPORTED;
  }
  if (NP == 128) return pair ? launch_bwd_tc<128, true>(tmW, tmDL, tmDL32, p, s) : launch_bwd_tc<128, false>(tmW, tmDL, tmDL32, p, s);
  if (NP == 256) return pair ? launch_bwd_tc<256, true>(tmW, tmDL, tmDL32, p, s) : launch_bwd_tc<256, false>(tmW, tmDL, tmDL32, p, s);
  if (NP == 512) return pair ? launch_bwd_tc<512, true>(tmW, tmDL, tmDL32, p, s) : launch_bwd_tc<512, false>(tmW, tmDL, tmDL32, p, s);
  if (NP == 1024 && !pair) return launch_bwd_tc<1024, false>(tmW, tmDL, tmDL32, p, s);  // two K rounds per step, clusters of 8
  return RINGRNN_ERR_UNSUPPORTED;
}

}  // namespace ringrnn

#ifdef RINGRNN_TIMELINE
extern "C" int ringrnn_debug_timeline_read_bwd(long long* out) {
  return (int)cudaMemcpyFromSymbol(out, ringrnn::g_timeline, sizeof(long long) * 64 * 16);
}
#endif
