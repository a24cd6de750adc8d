// dQ kernels for sm_100a.
//
// (1) dq_recompute_kernel -- general path (no bias, bool mask, float bias).
// Persistent, one CTA per SM, scheduled like the forward kernel: a tile is 128 query
// rows of one (batch, head); a CTA walks its tiles and, inside a tile, the key blocks;
// rings, tensor-memory buffers and barrier phases carry on from tile to tile.
// Roles (608 threads): warps 0-15 row threads (lanes 32*(w&3).., key quarter w>>2),
// warp 16 TMA producer, warp 17 MMA issuer for S and dP (tensor-memory owner),
// warp 18 MMA issuer for dQ.  Per key block:
//   S  = Q K_j^T, dP = dO V_j^T   (tensor memory)
//   row threads: P = exp2(S*scale*log2e + bias*log2e - LSE2); dS = P*(dP - delta)
//                -> 16-bit tile sDS in shared memory
//   dQ += dS K_j                  (sDS K-major, K_j MN-major)
// The S and dP columns are handed back to the MMA issuer as soon as they sit in
// registers, so the next block's products run while the row threads compute.
//
// (2) dq_from_ds_kernel -- used when the dK/dV kernel has just written dS as
// dbias in the same 16-bit dtype as q: dQ = sm_scale * dS . K is then a plain
// streamed GEMM whose A operand is loaded by TMA from the dbias tensor
// (64-key stages, two CTAs per SM).  The reference itself rounds dS to the
// 16-bit dtype before this product (flash_attention.py line 517), so the
// result is the same.
//
// Both replace _attn_bwd_dq / _attn_bwd_dq_inner (flash_attention.py 458-646).
#include "fa_common.cuh"
#include "fa_host.cuh"

namespace fa {
namespace {

struct DqParams {
  CUtensorMap map_q;
  CUtensorMap map_k;
  CUtensorMap map_v;
  CUtensorMap map_do;
  CUtensorMap map_ds;  // dbias viewed as the A operand of variant (2)
  const void* bias;
  void* dq;
  const float* lse;
  const float* delta;
  int* status;
  int64_t bias_sB, bias_sH, bias_sM;
  int64_t dq_sB, dq_sM, dq_sH;
  int H, M, N, D;
  int n_mblk, n_tiles;  // query blocks per (batch, head); tiles = n_mblk * B * H
  int causal, bias_vec32;
  float scale_log2;
  float sm_scale;
};

enum DqSite { kSiteQdo = 1, kSiteKFull, kSiteKEmpty, kSiteVFull, kSiteVEmpty, kSiteSFull,
              kSiteDpFull, kSiteSFree, kSiteDpFree, kSiteDsReady, kSiteDqDone, kSiteEpilogue,
              kSiteStageFull, kSiteStageEmpty, kSiteQdoEmpty };

template <int DP>
struct DqSmem {
  static constexpr int kTile = 128 * DP * 2;
  static constexpr int kQ = 0;
  static constexpr int kDo = kQ + kTile;
  static constexpr int kK = kDo + kTile;
  static constexpr int kV = kK + 2 * kTile;
  static constexpr int kDs = kV + 2 * kTile;
  static constexpr int kTotal = kDs + 2 * kBlk;
  static constexpr int kDynamic = kTotal + 1024;
};

template <int DP, typename T, int BIAS>
__global__ void __launch_bounds__(608, 1) dq_recompute_kernel(const __grid_constant__ DqParams p) {
  using L = DqSmem<DP>;
  using P2 = Pack2<T>;
  constexpr int KB = DP / 64;
  constexpr int KS_D = DP / 16;
  constexpr uint32_t kColS = 0, kColDp = 128, kColDq = 256;
  constexpr uint32_t kTmemCols = 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t qdo_full, qdo_empty, k_full[2], k_empty[2], v_full[2], v_empty[2];
  __shared__ uint64_t s_full, dp_full, s_free, dp_free, ds_ready, dq_done;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x;
  // the warp index as a value the compiler knows to be the same in all lanes: the issuer
  // warps then run converged and only elect a lane for the issue itself
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int lane = tid & 31;

  // Persistent CTA with the schedule of the forward kernel: tiles (128 query rows of one
  // (batch, head)) are numbered (batch*head)-major, CTA c takes units c, c+G, ...; a unit is
  // one tile or - causal - a heavy and a light tile of the same (batch, head).  All roles keep
  // running counters, so rings, tensor-memory buffers and barrier phases carry on from tile to
  // tile and the next tile's loads and first products overlap the current tile's epilogue.
  const int nblk_all = (p.N + 127) >> 7;
  const int sched_sh = p.causal ? 1 : 0;
  auto tile_at = [&](int it, int& bh, int& m_block, int& nblk) -> bool {
    const int u = static_cast<int>(blockIdx.x) + (it >> sched_sh) * static_cast<int>(gridDim.x);
    const int k = (u << sched_sh) + (it & sched_sh);
    if (k >= p.n_tiles) return false;
    bh = k / p.n_mblk;
    const int pos = k - bh * p.n_mblk;
    m_block = p.causal ? ((pos & 1) ? (pos >> 1) : p.n_mblk - 1 - (pos >> 1)) : pos;
    nblk = p.causal ? min(nblk_all, m_block + 1) : nblk_all;
    return true;
  };

  WaitCtx ctx{&abort_flag, p.status, 3};

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&qdo_full, 1);
    mbar_init(&qdo_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 2);  // S_j and dQ_j both read K_j
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    mbar_init(&s_full, 1);
    mbar_init(&dp_full, 1);
    mbar_init(&s_free, 16);
    mbar_init(&dp_free, 16);
    mbar_init(&ds_ready, 16);
    mbar_init(&dq_done, 1);
    mbar_fence_init();
  }
  if (warp == 17) {
    tmem_alloc(&tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  grid_dep_launch_next();
  grid_dep_wait();  // the previous kernel's results (and its status word) are visible from here
  const bool live = *reinterpret_cast<volatile int*>(p.status) == 0;

  if (warp == 16) {
    // ------------------------------------------------------------------ producer
    // (whole warp converged, one elected lane issues)
    if (live) {
      if (lane == 0) {
        tma_prefetch_desc(&p.map_q);
        tma_prefetch_desc(&p.map_k);
        tma_prefetch_desc(&p.map_v);
        tma_prefetch_desc(&p.map_do);
      }
      bool ok = true;
      uint32_t gj = 0;  // key blocks issued so far, over all tiles
      int bh, m_block, nblk;
      for (int it = 0; ok && tile_at(it, bh, m_block, nblk); ++it) {
        const int b = bh / p.H, h = bh - b * p.H, m0 = m_block * 128;
        // Q and dO are single tiles: free once the previous tile's last S and dP are through
        if (it >= 1) ok = wait_warp(&qdo_empty, (it - 1) & 1, ctx, kSiteQdoEmpty, it);
        if (!ok) break;
        if (elect_one()) {
          mbar_expect_tx(&qdo_full, 2 * L::kTile);
          for (int kb = 0; kb < KB; ++kb) {
            tma_load_4d(smem + L::kQ + kb * kBlk, &p.map_q, &qdo_full, kb * 64, h, m0, b);
            tma_load_4d(smem + L::kDo + kb * kBlk, &p.map_do, &qdo_full, kb * 64, h, m0, b);
          }
        }
        __syncwarp();
        for (int j = 0; j < nblk && ok; ++j) {
          const uint32_t g = gj + j;
          const int st = g & 1;
          const int n0 = j * 128;
          if (g >= 2) ok = wait_warp(&k_empty[st], ((g >> 1) - 1) & 1, ctx, kSiteKEmpty, j);
          if (!ok) break;
          if (elect_one()) {
            mbar_expect_tx(&k_full[st], L::kTile);
            for (int kb = 0; kb < KB; ++kb)
              tma_load_4d(smem + L::kK + st * L::kTile + kb * kBlk, &p.map_k, &k_full[st], kb * 64, h,
                          n0, b);
          }
          __syncwarp();
          if (g >= 2) ok = wait_warp(&v_empty[st], ((g >> 1) - 1) & 1, ctx, kSiteVEmpty, j);
          if (!ok) break;
          if (elect_one()) {
            mbar_expect_tx(&v_full[st], L::kTile);
            for (int kb = 0; kb < KB; ++kb)
              tma_load_4d(smem + L::kV + st * L::kTile + kb * kBlk, &p.map_v, &v_full[st], kb * 64, h,
                          n0, b);
          }
          __syncwarp();
        }
        gj += nblk;
      }
    }
  } else if (warp == 17) {
    // ------------------------------------------------------- MMA issuer: S and dP
    // (whole warp converged, one elected lane issues: the descriptors stay warp-uniform)
    if (live) {
      constexpr bool bf = P2::kIsBf16;
      constexpr uint32_t idesc_s = make_idesc(bf, false, false, 128, 128);
      const uint32_t q_addr = smem_u32(smem + L::kQ), do_addr = smem_u32(smem + L::kDo);
      const uint32_t k_addr = smem_u32(smem + L::kK), v_addr = smem_u32(smem + L::kV);
      const uint64_t q_km = make_sdesc(q_addr, 0, 1024), do_km = make_sdesc(do_addr, 0, 1024);
      const uint64_t k_km_0 = make_sdesc(k_addr, 0, 1024), k_km_1 = make_sdesc(k_addr + L::kTile, 0, 1024);
      const uint64_t v_km_0 = make_sdesc(v_addr, 0, 1024), v_km_1 = make_sdesc(v_addr + L::kTile, 0, 1024);
      bool ok = true;
      uint32_t gj = 0;
      int bh, m_block, nblk;
      for (int it = 0; ok && tile_at(it, bh, m_block, nblk); ++it) {
        for (int j = 0; j < nblk && ok; ++j) {
          const uint32_t g = gj + j;
          const int st = g & 1;
          const uint32_t ph = (g >> 1) & 1;
          // S_g: its columns are free once the row threads hold S_{g-1} in registers
          if (g >= 1) ok = wait_warp_hot(&s_free, (g - 1) & 1, ctx, kSiteSFree, j);
          if (ok && j == 0) ok = wait_warp(&qdo_full, it & 1, ctx, kSiteQdo, it);
          if (ok) ok = wait_warp(&k_full[st], ph, ctx, kSiteKFull, j);
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            issue_gemm_ss<KS_D, false, false>(tmem + kColS, q_km, st ? k_km_1 : k_km_0, kBlk, kBlk,
                                              idesc_s, false);
            mma_commit(&s_full);
            mma_commit(&k_empty[st]);
          }
          __syncwarp();
          if (g >= 1) ok = wait_warp_hot(&dp_free, (g - 1) & 1, ctx, kSiteDpFree, j);
          if (ok) ok = wait_warp(&v_full[st], ph, ctx, kSiteVFull, j);
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            issue_gemm_ss<KS_D, false, false>(tmem + kColDp, do_km, st ? v_km_1 : v_km_0, kBlk, kBlk,
                                              idesc_s, false);
            mma_commit(&dp_full);
            mma_commit(&v_empty[st]);
            if (j == nblk - 1) mma_commit(&qdo_empty);  // Q and dO may be replaced
          }
          __syncwarp();
        }
        gj += nblk;
      }
    }
    __syncwarp();
  } else if (warp == 18) {
    // ------------------------------------------------------- MMA issuer: dQ += dS K
    if (live) {
      constexpr uint32_t idesc_dq = make_idesc(P2::kIsBf16, false, true, 128, DP);
      const uint32_t k_addr = smem_u32(smem + L::kK);
      const uint64_t k_mn_0 = make_sdesc(k_addr, kBlk, 1024), k_mn_1 = make_sdesc(k_addr + L::kTile, kBlk, 1024);
      const uint64_t ds_km = make_sdesc(smem_u32(smem + L::kDs), 0, 1024);
      bool ok = true;
      uint32_t gj = 0;
      int bh, m_block, nblk;
      for (int it = 0; ok && tile_at(it, bh, m_block, nblk); ++it) {
        for (int j = 0; j < nblk && ok; ++j) {
          const uint32_t g = gj + j;
          const int st = g & 1;
          // dS of a new tile is only announced by all sixteen row warps after they have read
          // the previous tile's dQ, so the first product of a tile may overwrite it
          ok = wait_warp_hot(&ds_ready, g & 1, ctx, kSiteDsReady, j);
          if (ok) ok = wait_warp(&k_full[st], (g >> 1) & 1, ctx, kSiteKFull, j);
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            issue_gemm_ss<8, false, true>(tmem + kColDq, ds_km, st ? k_mn_1 : k_mn_0, kBlk, kBlk, idesc_dq,
                                          j > 0);
            mma_commit(&k_empty[st]);
            mma_commit(&dq_done);
          }
          __syncwarp();
        }
        gj += nblk;
      }
    }
    __syncwarp();
  } else {
    // --------------------------------------------------------------- row threads
    const int r = (warp & 3) * 32 + lane;
    const int qt = warp >> 2;  // key quarter of every block
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32u;
    bool ok = live;
    uint8_t* sDS = smem + L::kDs + (qt >> 1) * kBlk;
    const int chunk0 = (qt & 1) * 4;
    uint32_t gj = 0;
    int bh, m_block, nblk;
    for (int it = 0; ok && tile_at(it, bh, m_block, nblk); ++it) {
      const int b = bh / p.H, h = bh - b * p.H, m0 = m_block * 128;
      const int m = m0 + r;
      const bool row_ok = m < p.M;
      const int64_t bias_row = b * p.bias_sB + h * p.bias_sH + (int64_t)m * p.bias_sM;
      const float neg_lse = row_ok ? -__ldcg(p.lse + (int64_t)bh * p.M + m) : -INFINITY;
      const float delta_r = row_ok ? __ldcg(p.delta + (int64_t)bh * p.M + m) : 0.f;
      BiasRegs<BIAS> bnext;
      if (BIAS != 0)
        load_bias_row<BIAS>(bnext, p.bias, bias_row, row_ok, qt * 32, p.N, p.bias_vec32 != 0);

      for (int j = 0; j < nblk && ok; ++j) {
        const uint32_t g = gj + j;
        const int col0 = j * 128 + qt * 32;
        BiasRegs<BIAS> bcur = bnext;
        if (BIAS != 0 && j + 1 < nblk)
          load_bias_row<BIAS>(bnext, p.bias, bias_row, row_ok, col0 + 128, p.N, p.bias_vec32 != 0);

        ok = wait_warp(&s_full, g & 1, ctx, kSiteSFull, j);
        if (!ok) break;
        tc_fence_after();
        float pr[32];
        tmem_ld32(tmem_addr(tmem, lane_base, kColS + qt * 32), reinterpret_cast<uint32_t*>(pr));
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free);

#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          f32x2 a;
          if (BIAS == 1) {
            const float2 f = P2::unpack(bcur.w[i >> 1]);
            a = ffma2(f2(pr[i], pr[i + 1]), f2(p.scale_log2, p.scale_log2),
                      ffma2(f2(f.x, f.y), f2(kLog2e, kLog2e), f2(neg_lse, neg_lse)));
          } else {
            a = ffma2(f2(pr[i], pr[i + 1]), f2(p.scale_log2, p.scale_log2), f2(neg_lse, neg_lse));
          }
          const f32x2 pe = f2(ex2(f2_lo(a)), ex2(f2_hi(a)));
          if (BIAS == 2) {
            const uint32_t m2 = bcur.w[i >> 2] >> (8 * (i & 3));
            pr[i] = (m2 & 0xFFu) != 0 ? f2_lo(pe) : 0.f;
            pr[i + 1] = (m2 & 0xFF00u) != 0 ? f2_hi(pe) : 0.f;
          } else {
            pr[i] = f2_lo(pe);
            pr[i + 1] = f2_hi(pe);
          }
        }
        if ((col0 + 32 > p.N) || (p.causal && col0 + 31 > m0)) {
          int limit = p.N - col0;
          if (p.causal) limit = min(limit, m - col0 + 1);
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i >= limit) pr[i] = 0.f;
        }

        uint32_t pdp = 0, pdq = 1;
        if (j >= 1)
          mbar_poll2(&dp_full, g & 1, &dq_done, (g - 1) & 1, pdp, pdq);
        else
          pdp = mbar_poll(&dp_full, g & 1);
        ok = wait_warp_polled(pdp, &dp_full, g & 1, ctx, kSiteDpFull, j);
        if (!ok) break;
        tc_fence_after();
        uint32_t dsu[16];
        {
          uint32_t dp[32];
          tmem_ld32(tmem_addr(tmem, lane_base, kColDp + qt * 32), dp);
          tmem_ld_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&dp_free);
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const f32x2 d = fmul2(f2(pr[2 * i], pr[2 * i + 1]),
                                  fadd2(f2(__uint_as_float(dp[2 * i]), __uint_as_float(dp[2 * i + 1])),
                                        f2(-delta_r, -delta_r)));
            dsu[i] = P2::pack(f2_lo(d), f2_hi(d));
          }
        }
        // the previous dQ product has read sDS (for the first block of a tile its barrier was
        // seen in the previous tile's epilogue)
        if (j >= 1) {
          ok = wait_warp_polled(pdq, &dq_done, (g - 1) & 1, ctx, kSiteDqDone, j);
          if (!ok) break;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const uint4 v = make_uint4(dsu[c * 4 + 0], dsu[c * 4 + 1], dsu[c * 4 + 2], dsu[c * 4 + 3]);
          *reinterpret_cast<uint4*>(sDS + swz_off(r, chunk0 + c)) = v;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ds_ready);
      }
      if (!ok) break;
      gj += nblk;

      // ---- epilogue: dQ * sm_scale -> global
      ok = wait_warp(&dq_done, (gj - 1) & 1, ctx, kSiteEpilogue, nblk);
      if (!ok) break;
      tc_fence_after();
      constexpr int kQD = DP / 4;
      const int d0 = qt * kQD;
      T* row = reinterpret_cast<T*>(p.dq) + b * p.dq_sB + (int64_t)m * p.dq_sM + h * p.dq_sH;
      uint32_t a[kQD];
      tmem_ld_cols<kQD>(tmem_addr(tmem, lane_base, kColDq + d0), a);
      tmem_ld_wait();
      // dQ is in registers: the next tile's first product may overwrite it
      tc_fence_before();
      if (row_ok) {
#pragma unroll
        for (int c = 0; c < kQD / 8; ++c) {
          const int d = d0 + c * 8;
          if (d < p.D) *reinterpret_cast<uint4*>(row + d) = pack8<P2>(a + c * 8, p.sm_scale);
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 17) tmem_dealloc(tmem, kTmemCols);
}

// ----------------------------------------------------------------------------
// variant (2): dQ = sm_scale * dS . K with dS streamed from the dbias tensor
// ----------------------------------------------------------------------------
template <int DP>
struct DqDsSmem {
  static constexpr int kStages = 3;
  static constexpr int kDsBytes = 128 * 64 * 2;  // [128 m][64 n]
  static constexpr int kKBytes = 64 * DP * 2;    // [64 n][DP]
  static constexpr int kStage = kDsBytes + kKBytes;
  static constexpr int kTotal = kStages * kStage;
  static constexpr int kDynamic = kTotal + 1024;
};

template <int DP, typename T>
__global__ void __launch_bounds__(192, 2) dq_from_ds_kernel(const __grid_constant__ DqParams p) {
  using L = DqDsSmem<DP>;
  using P2 = Pack2<T>;
  constexpr int KB = DP / 64;
  constexpr uint32_t kTmemCols = DP;  // 64 or 128 accumulator columns

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t full[L::kStages], empty[L::kStages], acc_done;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x;
  // the warp index as a value the compiler knows to be the same in all lanes: the issuer
  // warps then run converged and only elect a lane for the issue itself
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int lane = tid & 31;
  const int m_block = gridDim.x - 1 - blockIdx.x;
  // the (batch, head) problems in reverse: the dS tiles written last by the dK/dV kernel are
  // still in L2 when this kernel starts
  const int bh = gridDim.y - 1 - blockIdx.y;
  const int b = bh / p.H;
  const int h = bh - b * p.H;
  const int m0 = m_block * 128;
  // 64-key steps; causal rows of this block see keys < m0 + 128
  int n_end = p.N;
  if (p.causal) n_end = min(n_end, m0 + 128);
  const int nsteps = (n_end + 63) >> 6;

  WaitCtx ctx{&abort_flag, p.status, 4};
  if (tid == 0) {
    abort_flag = 0;
    for (int i = 0; i < L::kStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(&acc_done, 1);
    mbar_fence_init();
  }
  if (warp == 5) {
    tmem_alloc(&tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  grid_dep_launch_next();
  grid_dep_wait();  // the previous kernel's results (and its status word) are visible from here
  const bool live = *reinterpret_cast<volatile int*>(p.status) == 0;

  if (warp == 4) {
    if (lane == 0 && live) {
      tma_prefetch_desc(&p.map_ds);
      tma_prefetch_desc(&p.map_k);
      const uint64_t pol_stream = policy_evict_first();
      bool ok = true;
      for (int s = 0; s < nsteps && ok; ++s) {
        const int st = s % L::kStages;
        const int use = s / L::kStages;
        if (use >= 1) ok = mbar_wait(&empty[st], (use - 1) & 1, ctx, kSiteStageEmpty, s);
        if (!ok) break;
        uint8_t* base = smem + st * L::kStage;
        mbar_expect_tx(&full[st], L::kStage);
        tma_load_4d_hint(base, &p.map_ds, &full[st], s * 64, m0, h, b, pol_stream);
        for (int kb = 0; kb < KB; ++kb)
          tma_load_4d(base + L::kDsBytes + kb * (64 * 128), &p.map_k, &full[st], kb * 64, h, s * 64,
                      b);
      }
    }
  } else if (warp == 5) {
    // (whole warp converged, one elected lane issues)
    if (live) {
      constexpr uint32_t idesc = make_idesc(P2::kIsBf16, false, true, 128, DP);
      bool ok = true;
      for (int s = 0; s < nsteps && ok; ++s) {
        const int st = s % L::kStages;
        ok = wait_warp(&full[st], (s / L::kStages) & 1, ctx, kSiteStageFull, s);
        if (!ok) break;
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + st * L::kStage);
        const uint32_t b_addr = a_addr + L::kDsBytes;
        if (elect_one()) {
          issue_gemm_ss<4, false, true>(tmem, make_sdesc(a_addr, 0, 1024),
                                        make_sdesc(b_addr, 64 * 128, 1024), 0, 0, idesc, s > 0);
          mma_commit(&empty[st]);
        }
        __syncwarp();
      }
      if (ok && elect_one()) mma_commit(&acc_done);
    }
    __syncwarp();
  } else {
    const int r = tid;
    const uint32_t lane_base = static_cast<uint32_t>(warp) * 32u;
    const int m = m0 + r;
    bool ok = live;
    if (ok) ok = wait_warp(&acc_done, 0, ctx, kSiteEpilogue, 0);
    if (ok) {
      tc_fence_after();
      T* row = reinterpret_cast<T*>(p.dq) + b * p.dq_sB + (int64_t)m * p.dq_sM + h * p.dq_sH;
#pragma unroll
      for (int g = 0; g < DP / 32; ++g) {
        uint32_t a[32];
        tmem_ld32(tmem_addr(tmem, lane_base, g * 32), a);
        tmem_ld_wait();
        if (m < p.M) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const int d = g * 32 + c * 8;
            if (d < p.D) *reinterpret_cast<uint4*>(row + d) = pack8<P2>(a + c * 8, p.sm_scale);
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem, kTmemCols);
}

template <typename K>
int configure(K kern, int smem_bytes, bool* configured) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) !=
        cudaSuccess)
      return FA_ERR_CUDA;
    configured[dev] = true;
  }
  return FA_OK;
}

template <int DP, typename T, int BIAS>
int launch_recompute(const DqParams& kp, dim3 /*tile_grid*/, cudaStream_t stream) {
  const dim3 grid(persistent_grid(kp.causal ? (kp.n_tiles + 1) / 2 : kp.n_tiles));
  using L = DqSmem<DP>;
  static bool configured[64] = {};
  auto kern = dq_recompute_kernel<DP, T, BIAS>;
  if (int r = configure(kern, L::kDynamic, configured)) return r;
  return launch_overlapped(kern, grid, 608, L::kDynamic, stream, kp);
}

template <int DP, typename T>
int launch_from_ds(const DqParams& kp, dim3 grid, cudaStream_t stream) {
  using L = DqDsSmem<DP>;
  static bool configured[64] = {};
  auto kern = dq_from_ds_kernel<DP, T>;
  if (int r = configure(kern, L::kDynamic, configured)) return r;
  return launch_overlapped(kern, grid, 192, L::kDynamic, stream, kp);
}

template <int DP, typename T>
int launch_bias(const DqParams& kp, int bias_kind, bool from_ds, dim3 grid, cudaStream_t stream) {
  if (from_ds) return launch_from_ds<DP, T>(kp, grid, stream);
  switch (bias_kind) {
    case FA_BIAS_NONE: return launch_recompute<DP, T, 0>(kp, grid, stream);
    case FA_BIAS_SAME: return launch_recompute<DP, T, 1>(kp, grid, stream);
    case FA_BIAS_BOOL: return launch_recompute<DP, T, 2>(kp, grid, stream);
    default: return FA_ERR_UNSUPPORTED;
  }
}

}  // namespace

int launch_bwd_dq(const fa_params& p, cudaStream_t stream, int* status) {
  DqParams kp;
  // When the dK/dV stage has just left dS in a 16-bit tensor (the bias gradient itself, or the
  // scratch an fp32 bias comes with) the streamed GEMM variant is used, otherwise the general
  // kernel.
  // At head dimension 256 only the streamed variant exists: its dK/dV kernel always leaves dS.
  const bool f32 = p.bias_kind == FA_BIAS_F32;
  const bool d256 = p.D == 256;
  if (f32 && !p.ds16) return FA_ERR_NULL;
  const bool from_ds = d256 || f32 || (p.write_dbias && p.bias_kind == FA_BIAS_SAME);
  const int64_t* ds_stride = f32 ? p.ds16_stride : p.dbias_stride;
  const void* ds = f32 ? p.ds16 : p.dbias;
  if (d256) ds = d256_ds_tensor(p, &ds_stride);
  if (from_ds && !ds) return FA_ERR_NULL;
  int r = make_tmap_bshd(&kp.map_q, p.q, p.B, p.M, p.H, p.D, p.q_stride, 128);
  if (r) return r;
  r = make_tmap_bshd(&kp.map_k, p.k, p.B, p.N, p.H, p.D, p.k_stride, from_ds ? 64 : 128);
  if (r) return r;
  r = make_tmap_bshd(&kp.map_v, p.v, p.B, p.N, p.H, p.D, p.v_stride, 128);
  if (r) return r;
  r = make_tmap_bshd(&kp.map_do, p.d_o, p.B, p.M, p.H, p.D, p.do_stride, 128);
  if (r) return r;
  if (from_ds) {
    int bm, hm;
    r = make_tmap_bhmn(&kp.map_ds, ds, 2, p.B, p.H, p.M, p.N, ds_stride, 64, 128, &bm, &hm);
    if (r) return r;
    if (!bm || !hm) return FA_ERR_ALIGN;
  } else {
    kp.map_ds = kp.map_q;
  }
  if (reinterpret_cast<uintptr_t>(p.dq) % 16 != 0 || p.dq_stride[0] % 8 || p.dq_stride[1] % 8 ||
      p.dq_stride[2] % 8)
    return FA_ERR_ALIGN;
  if (p.bias_kind != FA_BIAS_NONE && !from_ds) {
    const int eb = p.bias_kind == FA_BIAS_BOOL ? 1 : 2;
    if (reinterpret_cast<uintptr_t>(p.bias) % 16 != 0 || (p.bias_stride[0] * eb) % 16 ||
        (p.bias_stride[1] * eb) % 16 || (p.bias_stride[2] * eb) % 16)
      return FA_ERR_ALIGN;
  }
  kp.bias = p.bias;
  kp.dq = p.dq;
  kp.lse = p.lse;
  kp.delta = p.delta;
  kp.status = status;
  kp.bias_sB = p.bias_stride[0];
  kp.bias_sH = p.bias_stride[1];
  kp.bias_sM = p.bias_stride[2];
  kp.dq_sB = p.dq_stride[0];
  kp.dq_sM = p.dq_stride[1];
  kp.dq_sH = p.dq_stride[2];
  kp.H = p.H;
  kp.M = p.M;
  kp.N = p.N;
  kp.D = p.D;
  kp.causal = p.causal ? 1 : 0;
  {
    const int eb = p.bias_kind == FA_BIAS_BOOL ? 1 : 2;
    kp.bias_vec32 = p.bias_kind != FA_BIAS_NONE && reinterpret_cast<uintptr_t>(p.bias) % 32 == 0 &&
                    (p.bias_stride[0] * eb) % 32 == 0 && (p.bias_stride[1] * eb) % 32 == 0 &&
                    (p.bias_stride[2] * eb) % 32 == 0;
  }
  kp.scale_log2 = p.sm_scale * kLog2e;
  kp.sm_scale = p.sm_scale;
  kp.n_mblk = (p.M + 127) / 128;
  kp.n_tiles = kp.n_mblk * p.B * p.H;
  const dim3 grid((p.M + 127) / 128, p.B * p.H);  // streamed-dS variant: one CTA per tile
  const int dp = padded_head_dim(p.D);
  if (dp == 256)
    return p.dtype == FA_BF16 ? launch_from_ds<256, __nv_bfloat16>(kp, grid, stream)
                              : launch_from_ds<256, __half>(kp, grid, stream);
  if (p.dtype == FA_BF16) {
    return dp == 64 ? launch_bias<64, __nv_bfloat16>(kp, p.bias_kind, from_ds, grid, stream)
                    : launch_bias<128, __nv_bfloat16>(kp, p.bias_kind, from_ds, grid, stream);
  }
  return dp == 64 ? launch_bias<64, __half>(kp, p.bias_kind, from_ds, grid, stream)
                  : launch_bias<128, __half>(kp, p.bias_kind, from_ds, grid, stream);
}

}  // namespace fa
