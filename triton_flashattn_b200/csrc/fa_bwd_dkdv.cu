// dK / dV (and dbias) kernel for sm_100a.
//
// One CTA owns 128 keys of one (batch, head) and walks the query blocks of 128
// rows (only those at or below the diagonal when causal).  Roles (640 threads):
//   warps 0-15 "row" threads: warp w works on tensor-memory lanes 32*(w&3)..+31
//              (query rows of the block) and on the 32-key column quarter (w>>2)
//   warp 16    TMA producer (one lane): K, V once; Q ring (2), dO ring
//   warp 17    MMA issuer for S and dP (one lane), tensor-memory owner
//   warp 18    MMA issuer for dV and dK (one lane)
//   warp 19    bulk tensor stores of the dS tile into dbias (one lane)
// A barrier operation answers after ~200 cycles on this GPU, so two issuers keep
// the tensor pipe fed while the other one waits, and every role polls the
// barriers it will need before it starts a stretch of independent work.
// Per query block t:
//   S  = Q_t K^T            (tensor memory, 128 columns)
//   dP = dO_t V^T           (tensor memory, 128 columns)
//   row threads: P = exp2(S*scale*log2e + bias*log2e - LSE2) -> 16-bit tile sP
//                dS = P * (dP - delta)                        -> 16-bit tile sDS
//   dV += P^T dO_t          (sP and dO_t consumed MN-major)
//   dK += dS^T Q_t          (sDS and Q_t consumed MN-major)
//   dbias[b,h,m-block,n-block] <- sDS  (one bulk tensor store of the same tile)
// The bias never touches shared memory: every row thread fetches its own 64
// contiguous bytes (32 keys) with 256-bit loads one query block ahead.
// Causally skipped tiles of dbias are written as zeros by this kernel, so dbias
// needs no prior fill.
//
// Replaces _attn_bwd_dkdv / _attn_bwd_dkdv_inner of the reference
// (flash_attention.py 237-454): same P, dS, dbias = dS, dK scaled by sm_scale.
#include "fa_common.cuh"
#include "fa_host.cuh"

namespace fa {
#ifdef FA_TRACE
__device__ long long g_fa_trace_dkdv[8192];
#define TR(role, step, slot) do { if (blockIdx.x == 0 && blockIdx.y == 0 && (step) < 16) g_fa_trace_dkdv[(role) * 2048 + (step) * 16 + (slot)] = clock64(); } while (0)
#else
#define TR(role, step, slot) do {} while (0)
#endif
namespace {

struct DkdvParams {
  CUtensorMap map_q;
  CUtensorMap map_k;
  CUtensorMap map_v;
  CUtensorMap map_do;
  CUtensorMap map_dbias;
  CUtensorMap map_bias;  // only used to prefetch bias tiles into L2
  const void* bias;
  void* dk;
  void* dv;
  const float* lse;
  const float* delta;
  int* status;
  int64_t bias_sB, bias_sH, bias_sM;
  int64_t dk_sB, dk_sN, dk_sH, dv_sB, dv_sN, dv_sH;
  int H, M, N, D;
  int causal, write_dbias, bias_vec32, bias_b_mul, bias_h_mul;
  float scale_log2;  // sm_scale * log2(e)
  float sm_scale;
};

enum DkdvSite { kSiteKV = 1, kSiteQFull, kSiteQEmpty, kSiteDoFull, kSiteDoEmpty, kSiteSFull,
                kSiteDpFull, kSitePReady, kSiteDsReady, kSiteDvDone, kSiteDkDone, kSiteStDone,
                kSiteZeroReady, kSiteEpilogue, kSiteSFree, kSiteDpFree };

template <int DP>
struct DkdvSmem {
  static constexpr int kTile = 128 * DP * 2;
  static constexpr int kDoStages = DP == 128 ? 1 : 2;
  static constexpr int kK = 0;
  static constexpr int kV = kK + kTile;
  static constexpr int kQ = kV + kTile;
  static constexpr int kDo = kQ + 2 * kTile;
  static constexpr int kP = kDo + kDoStages * kTile;
  static constexpr int kDs = kP + 2 * kBlk;
  static constexpr int kTotal = kDs + 2 * kBlk;
  static constexpr int kDynamic = kTotal + 1024;
};

template <int DP, typename T, int BIAS>
__global__ void __launch_bounds__(640, 1) dkdv_kernel(const __grid_constant__ DkdvParams p) {
  using L = DkdvSmem<DP>;
  using P2 = Pack2<T>;
  constexpr int KB = DP / 64;
  constexpr int KS_D = DP / 16;  // K slices of the two "score" products
  constexpr int kDoStages = L::kDoStages;
  constexpr uint32_t kColS = 0, kColDp = 128, kColDv = 256, kColDk = 384;
  constexpr uint32_t kTmemCols = 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t kv_full, q_full[2], q_empty[2], do_full[2], do_empty[2];
  __shared__ uint64_t s_full, dp_full, p_ready, ds_ready, dv_done, dk_done, st_done, zero_ready;
  __shared__ uint64_t s_free, dp_free;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  const int nb = blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.H;
  const int h = bh - b * p.H;
  const int n0 = nb * 128;
  const int n_mblk = (p.M + 127) >> 7;
  const int i_start = p.causal ? min(nb, n_mblk) : 0;
  const int T_steps = n_mblk - i_start;

  WaitCtx ctx{&abort_flag, p.status, 2};

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&kv_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 2);
      mbar_init(&do_full[i], 1);
      mbar_init(&do_empty[i], 2);
    }
    mbar_init(&s_full, 1);
    mbar_init(&dp_full, 1);
    mbar_init(&p_ready, 16);
    mbar_init(&ds_ready, 16);
    mbar_init(&dv_done, 1);
    mbar_init(&dk_done, 1);
    mbar_init(&st_done, 1);
    mbar_init(&zero_ready, 16);
    mbar_init(&s_free, 16);
    mbar_init(&dp_free, 16);
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
  const bool live = *reinterpret_cast<volatile int*>(p.status) == 0;

  if (warp == 16) {
    // ------------------------------------------------------------------ producer
    if (lane == 0 && live && T_steps > 0) {
      tma_prefetch_desc(&p.map_q);
      tma_prefetch_desc(&p.map_k);
      tma_prefetch_desc(&p.map_v);
      tma_prefetch_desc(&p.map_do);
      mbar_expect_tx(&kv_full, 2 * L::kTile);
      for (int kb = 0; kb < KB; ++kb) {
        tma_load_4d(smem + L::kK + kb * kBlk, &p.map_k, &kv_full, kb * 64, h, n0, b);
        tma_load_4d(smem + L::kV + kb * kBlk, &p.map_v, &kv_full, kb * 64, h, n0, b);
      }
      bool ok = true;
      constexpr int kBiasAhead = 2;  // bias tiles are pulled into L2 this many steps early
      if (BIAS != 0) {
        for (int t = 0; t < kBiasAhead && t < T_steps; ++t) {
          const int mp = (i_start + t) * 128;
          tma_prefetch_l2_4d(&p.map_bias, n0, mp, h * p.bias_h_mul, b * p.bias_b_mul);
          if (BIAS == 1 && n0 + 64 < p.N)
            tma_prefetch_l2_4d(&p.map_bias, n0 + 64, mp, h * p.bias_h_mul, b * p.bias_b_mul);
        }
      }
      for (int t = 0; t < T_steps && ok; ++t) {
        const int m0 = (i_start + t) * 128;
        const int qs = t & 1;
        if (BIAS != 0 && t + kBiasAhead < T_steps) {
          const int mp = (i_start + t + kBiasAhead) * 128;
          tma_prefetch_l2_4d(&p.map_bias, n0, mp, h * p.bias_h_mul, b * p.bias_b_mul);
          if (BIAS == 1 && n0 + 64 < p.N)
            tma_prefetch_l2_4d(&p.map_bias, n0 + 64, mp, h * p.bias_h_mul, b * p.bias_b_mul);
        }
        if (t >= 2) ok = mbar_wait(&q_empty[qs], ((t >> 1) - 1) & 1, ctx, kSiteQEmpty, t);
        if (!ok) break;
        mbar_expect_tx(&q_full[qs], L::kTile);
        for (int kb = 0; kb < KB; ++kb)
          tma_load_4d(smem + L::kQ + qs * L::kTile + kb * kBlk, &p.map_q, &q_full[qs], kb * 64, h,
                      m0, b);
        const int ds = t % kDoStages;
        const int du = t / kDoStages;
        if (du >= 1) ok = mbar_wait(&do_empty[ds], (du - 1) & 1, ctx, kSiteDoEmpty, t);
        if (!ok) break;
        mbar_expect_tx(&do_full[ds], L::kTile);
        for (int kb = 0; kb < KB; ++kb)
          tma_load_4d(smem + L::kDo + ds * L::kTile + kb * kBlk, &p.map_do, &do_full[ds], kb * 64,
                      h, m0, b);
      }
    }
  } else if (warp == 17) {
    // ------------------------------------------------------- MMA issuer: S and dP
    if (lane == 0 && live && T_steps > 0) {
      constexpr bool bf = P2::kIsBf16;
      constexpr uint32_t idesc_s = make_idesc(bf, false, false, 128, 128);
      const uint32_t k_addr = smem_u32(smem + L::kK), v_addr = smem_u32(smem + L::kV);
      const uint32_t q_addr = smem_u32(smem + L::kQ), do_addr = smem_u32(smem + L::kDo);
      const uint64_t k_km = make_sdesc(k_addr, 0, 1024), v_km = make_sdesc(v_addr, 0, 1024);
      const uint64_t q_km_0 = make_sdesc(q_addr, 0, 1024), q_km_1 = make_sdesc(q_addr + L::kTile, 0, 1024);
      const uint64_t do_km_0 = make_sdesc(do_addr, 0, 1024),
                     do_km_1 = make_sdesc(do_addr + (kDoStages - 1) * L::kTile, 0, 1024);
      auto issue_s = [&](int t) {
        issue_gemm_ss<KS_D, false, false>(tmem + kColS, (t & 1) ? q_km_1 : q_km_0, k_km, kBlk, kBlk,
                                          idesc_s, false);
        mma_commit(&s_full);
        mma_commit(&q_empty[t & 1]);
      };
      auto issue_dp = [&](int t) {
        issue_gemm_ss<KS_D, false, false>(tmem + kColDp, (t % kDoStages) ? do_km_1 : do_km_0, v_km,
                                          kBlk, kBlk, idesc_s, false);
        mma_commit(&dp_full);
        mma_commit(&do_empty[t % kDoStages]);
      };
      bool ok = mbar_wait(&kv_full, 0, ctx, kSiteKV, 0);
      if (ok) ok = mbar_wait(&q_full[0], 0, ctx, kSiteQFull, 0);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        ok = mbar_wait(&do_full[0], 0, ctx, kSiteDoFull, 0);
      }
      if (ok) {
        tc_fence_after();
        issue_dp(0);
      }
      for (int t = 0; t + 1 < T_steps && ok; ++t) {
        const int ds1 = (t + 1) % kDoStages;
        const uint32_t q_par = ((t + 1) >> 1) & 1, do_par = ((t + 1) / kDoStages) & 1;
        // S_{t+1}: its columns are free once the row threads hold S_t in registers
        const uint32_t pq = mbar_poll(&q_full[(t + 1) & 1], q_par);
        ok = mbar_wait(&s_free, t & 1, ctx, kSiteSFree, t);
        if (ok) ok = wait_polled(pq, &q_full[(t + 1) & 1], q_par, ctx, kSiteQFull, t + 1);
        if (!ok) break;
        TR(1, t, 1);
        tc_fence_after();
        const uint32_t pdo = mbar_poll(&do_full[ds1], do_par);
        issue_s(t + 1);
        TR(1, t, 2);
        // dP_{t+1}: same for the dP columns; dO_{t+1} replaces dO_t after dV_t when single-staged
        ok = mbar_wait(&dp_free, t & 1, ctx, kSiteDpFree, t);
        if (ok) ok = wait_polled(pdo, &do_full[ds1], do_par, ctx, kSiteDoFull, t + 1);
        if (!ok) break;
        TR(1, t, 3);
        tc_fence_after();
        issue_dp(t + 1);
        TR(1, t, 4);
      }
    }
    __syncwarp();
  } else if (warp == 18) {
    // ------------------------------------------------------ MMA issuer: dV and dK
    if (lane == 0 && live) {
      constexpr bool bf = P2::kIsBf16;
      constexpr uint32_t idesc_g = make_idesc(bf, true, true, 128, DP);
      const uint32_t q_addr = smem_u32(smem + L::kQ), do_addr = smem_u32(smem + L::kDo);
      const uint32_t p_addr = smem_u32(smem + L::kP), ds_addr = smem_u32(smem + L::kDs);
      const uint64_t q_mn_0 = make_sdesc(q_addr, kBlk, 1024), q_mn_1 = make_sdesc(q_addr + L::kTile, kBlk, 1024);
      const uint64_t do_mn_0 = make_sdesc(do_addr, kBlk, 1024),
                     do_mn_1 = make_sdesc(do_addr + (kDoStages - 1) * L::kTile, kBlk, 1024);
      const uint64_t p_mn = make_sdesc(p_addr, kBlk, 1024), ds_mn = make_sdesc(ds_addr, kBlk, 1024);
      bool ok = true;
      for (int t = 0; t < T_steps && ok; ++t) {
        const int qs = t & 1;
        const int ds = t % kDoStages;
        // dV += P^T dO  (dO_t must have landed: P_t only depends on S_t)
        const uint32_t pdo = mbar_poll(&do_full[ds], (t / kDoStages) & 1);
        const uint32_t pq = mbar_poll(&q_full[qs], (t >> 1) & 1);
        ok = mbar_wait(&p_ready, t & 1, ctx, kSitePReady, t);
        if (ok) ok = wait_polled(pdo, &do_full[ds], (t / kDoStages) & 1, ctx, kSiteDoFull, t);
        if (!ok) break;
        TR(2, t, 1);
        tc_fence_after();
        issue_gemm_ss<8, true, true>(tmem + kColDv, p_mn, ds ? do_mn_1 : do_mn_0, kBlk, kBlk, idesc_g,
                                     t > 0);
        mma_commit(&do_empty[ds]);
        mma_commit(&dv_done);
        TR(2, t, 2);
        // dK += dS^T Q
        ok = mbar_wait(&ds_ready, t & 1, ctx, kSiteDsReady, t);
        if (ok) ok = wait_polled(pq, &q_full[qs], (t >> 1) & 1, ctx, kSiteQFull, t);
        if (!ok) break;
        TR(2, t, 3);
        tc_fence_after();
        issue_gemm_ss<8, true, true>(tmem + kColDk, ds_mn, qs ? q_mn_1 : q_mn_0, kBlk, kBlk, idesc_g,
                                     t > 0);
        mma_commit(&q_empty[qs]);
        mma_commit(&dk_done);
        TR(2, t, 4);
      }
    }
    __syncwarp();
  } else if (warp == 19) {
    // ------------------------------------------------------------- dbias stores
    // phase 0 of st_done: zero tiles above the diagonal are out (or nothing to do);
    // phase t+1: the store of dS_t has finished reading sDS.
    if (lane == 0 && live && p.write_dbias) {
      bool ok = true;
      if (p.causal) {
        ok = mbar_wait(&zero_ready, 0, ctx, kSiteZeroReady, 0);
        if (ok) {
          const int nz = min(nb, n_mblk);
          for (int i = 0; i < nz; ++i) {
            tma_store_4d(&p.map_dbias, smem + L::kDs, n0, i * 128, h, b);
            if (n0 + 64 < p.N)
              tma_store_4d(&p.map_dbias, smem + L::kDs + kBlk, n0 + 64, i * 128, h, b);
          }
          tma_store_commit();
          tma_store_wait_read<0>();
        }
      }
      mbar_arrive(&st_done);
      for (int t = 0; t < T_steps && ok; ++t) {
        ok = mbar_wait(&ds_ready, t & 1, ctx, kSiteDsReady, t);
        if (!ok) break;
        const int m0 = (i_start + t) * 128;
        tma_store_4d(&p.map_dbias, smem + L::kDs, n0, m0, h, b);
        if (n0 + 64 < p.N) tma_store_4d(&p.map_dbias, smem + L::kDs + kBlk, n0 + 64, m0, h, b);
        tma_store_commit();
        tma_store_wait_read<0>();
        mbar_arrive(&st_done);
      }
      tma_store_wait_all<0>();
    }
    __syncwarp();
  } else {
    // --------------------------------------------------------------- row threads
    const int r = (warp & 3) * 32 + lane;  // query row inside the block = tensor-memory lane
    const int qt = warp >> 2;              // column quarter: keys n0 + 32*qt .. +31
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32u;
    bool ok = live;
    // this thread's four 16-byte chunks inside the [128][128] 16-bit tiles
    uint8_t* sP = smem + L::kP + (qt >> 1) * kBlk;
    uint8_t* sDS = smem + L::kDs + (qt >> 1) * kBlk;
    const int chunk0 = (qt & 1) * 4;

    if (p.write_dbias && p.causal && ok) {
      // zero tile for the causally skipped part of dbias
      uint4* z = reinterpret_cast<uint4*>(smem + L::kDs);
      for (int i = tid; i < 2 * kBlk / 16; i += 512) z[i] = make_uint4(0, 0, 0, 0);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&zero_ready);
    }

    const int col0 = n0 + qt * 32;
    const int64_t bias_bh = b * p.bias_sB + h * p.bias_sH;
    BiasRegs<BIAS> bnext;
    float lse_next = INFINITY, delta_next = 0.f;
    auto prefetch = [&](int t) {
      const int m = (i_start + t) * 128 + r;
      const bool row_ok = m < p.M;
      if (BIAS == 1 && p.bias_vec32 && col0 + 32 <= p.N) {
        // warp-wide: one request per line, then a shuffle pass (see load_bias_rows_paired)
        const int mrow0 = (i_start + t) * 128 + (warp & 3) * 32;
        if constexpr (BIAS == 1)
          load_bias_rows_paired(bnext, p.bias, bias_bh + (int64_t)mrow0 * p.bias_sM, p.bias_sM,
                                p.M - mrow0, col0, lane);
      } else if (BIAS != 0) {
        load_bias_row<BIAS>(bnext, p.bias, bias_bh + (int64_t)m * p.bias_sM, row_ok, col0, p.N,
                            p.bias_vec32 != 0);
      }
      // clamped address: the value of a row beyond M is replaced when it is used
      const int mc = row_ok ? m : p.M - 1;
      lse_next = __ldg(p.lse + (int64_t)bh * p.M + mc);
      delta_next = __ldg(p.delta + (int64_t)bh * p.M + mc);
    };
    if (ok && T_steps > 0) prefetch(0);

    for (int t = 0; t < T_steps && ok; ++t) {
      const int m0 = (i_start + t) * 128;
      BiasRegs<BIAS> bcur = bnext;
      if constexpr (BIAS == 1) {
        if (p.bias_vec32 && col0 + 32 <= p.N) redistribute_bias_rows(bcur, lane);
      }
      const bool row_in = m0 + r < p.M;
      const float lse_raw = lse_next, delta_raw = delta_next;
      if (t + 1 < T_steps) prefetch(t + 1);
      // S_t and "dV_{t-1} has read P_{t-1}" are usually true by now: one combined look
      uint32_t ps = 0, pdv = 1;
      if (t >= 1)
        mbar_poll2(&s_full, t & 1, &dv_done, (t - 1) & 1, ps, pdv);
      else
        ps = mbar_poll(&s_full, t & 1);

      // ---- P
      if (tid == 0) TR(0, t, 0);
      ok = wait_warp_polled(ps, &s_full, t & 1, ctx, kSiteSFull, t);
      if (!ok) break;
      if (tid == 0) TR(0, t, 1);
      tc_fence_after();
      float pr[32];
      tmem_ld32(tmem_addr(tmem, lane_base, kColS + qt * 32), reinterpret_cast<uint32_t*>(pr));
      tmem_ld_wait();
      // S_t now lives in registers: hand its columns back for S_{t+1}
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_free);
      // P = exp2(S * scale * log2e + bias * log2e - LSE2); rows beyond M have LSE2 = +inf
      const float neg_lse = row_in ? -lse_raw : -INFINITY;
      const float delta_r = row_in ? delta_raw : 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        if (BIAS == 1) {
          const float2 f = P2::unpack(bcur.w[i >> 1]);
          pr[i] = ex2(fmaf(pr[i], p.scale_log2, fmaf((i & 1) ? f.y : f.x, kLog2e, neg_lse)));
        } else if (BIAS == 2) {
          const bool keep = ((bcur.w[i >> 2] >> (8 * (i & 3))) & 0xFFu) != 0;
          pr[i] = keep ? ex2(fmaf(pr[i], p.scale_log2, neg_lse)) : 0.f;
        } else {
          pr[i] = ex2(fmaf(pr[i], p.scale_log2, neg_lse));
        }
      }
      if ((col0 + 32 > p.N) || (p.causal && col0 + 31 > m0)) {
        int limit = p.N - col0;
        if (p.causal) limit = min(limit, m0 + r - col0 + 1);
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i >= limit) pr[i] = 0.f;
      }
      if (tid == 0) TR(0, t, 2);
      if (t >= 1) {
        ok = wait_warp_polled(pdv, &dv_done, (t - 1) & 1, ctx, kSiteDvDone, t);
        if (!ok) break;
      }
      if (tid == 0) TR(0, t, 3);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint4 v;
        v.x = P2::pack(pr[c * 8 + 0], pr[c * 8 + 1]);
        v.y = P2::pack(pr[c * 8 + 2], pr[c * 8 + 3]);
        v.z = P2::pack(pr[c * 8 + 4], pr[c * 8 + 5]);
        v.w = P2::pack(pr[c * 8 + 6], pr[c * 8 + 7]);
        *reinterpret_cast<uint4*>(sP + swz_off(r, chunk0 + c)) = v;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready);
      if (tid == 0) TR(0, t, 4);

      // ---- dS
      // dP_t, "dK_{t-1} has read dS_{t-1}" and "its dbias store has": one combined look
      uint32_t pdp = 0, pdk = 1, pst = 1;
      if (t >= 1 && p.write_dbias)
        mbar_poll3(&dp_full, t & 1, &dk_done, (t - 1) & 1, &st_done, t & 1, pdp, pdk, pst);
      else if (t >= 1)
        mbar_poll2(&dp_full, t & 1, &dk_done, (t - 1) & 1, pdp, pdk);
      else if (p.write_dbias)
        mbar_poll2(&dp_full, t & 1, &st_done, t & 1, pdp, pst);
      else
        pdp = mbar_poll(&dp_full, t & 1);
      ok = wait_warp_polled(pdp, &dp_full, t & 1, ctx, kSiteDpFull, t);
      if (!ok) break;
      if (tid == 0) TR(0, t, 5);
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
          const float d0 = pr[2 * i] * (__uint_as_float(dp[2 * i]) - delta_r);
          const float d1 = pr[2 * i + 1] * (__uint_as_float(dp[2 * i + 1]) - delta_r);
          dsu[i] = P2::pack(d0, d1);
        }
      }
      if (tid == 0) TR(0, t, 6);
      if (t >= 1) {
        ok = wait_warp_polled(pdk, &dk_done, (t - 1) & 1, ctx, kSiteDkDone, t);
        if (!ok) break;
      }
      if (tid == 0) TR(0, t, 7);
      if (p.write_dbias) {
        ok = wait_warp_polled(pst, &st_done, t & 1, ctx, kSiteStDone, t);
        if (!ok) break;
      }
      if (tid == 0) TR(0, t, 8);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 v = make_uint4(dsu[c * 4 + 0], dsu[c * 4 + 1], dsu[c * 4 + 2], dsu[c * 4 + 3]);
        *reinterpret_cast<uint4*>(sDS + swz_off(r, chunk0 + c)) = v;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_ready);
      if (tid == 0) TR(0, t, 9);
    }

    // ---- epilogue: dV, dK (rows = keys) -> global
    if (ok && T_steps > 0) {
      ok = wait_warp(&dv_done, (T_steps - 1) & 1, ctx, kSiteEpilogue, 0);
      if (ok) ok = wait_warp(&dk_done, (T_steps - 1) & 1, ctx, kSiteEpilogue, 1);
    }
    if (ok) {
      tc_fence_after();
      const int n = n0 + r;
      constexpr int kQD = DP / 4;  // columns of the head dim this thread stores (16 or 32)
      const int d0 = qt * kQD;
      T* dkrow = reinterpret_cast<T*>(p.dk) + b * p.dk_sB + (int64_t)n * p.dk_sN + h * p.dk_sH;
      T* dvrow = reinterpret_cast<T*>(p.dv) + b * p.dv_sB + (int64_t)n * p.dv_sN + h * p.dv_sH;
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        T* row = which == 0 ? dvrow : dkrow;
        const uint32_t colbase = which == 0 ? kColDv : kColDk;
        const float mul = which == 0 ? 1.0f : p.sm_scale;
        uint32_t a[kQD];
        if (T_steps > 0) {
          tmem_ld_cols<kQD>(tmem_addr(tmem, lane_base, colbase + d0), a);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < kQD; ++i) a[i] = 0;
        }
        if (n < p.N) {
#pragma unroll
          for (int c = 0; c < kQD / 8; ++c) {
            const int d = d0 + c * 8;
            if (d < p.D) *reinterpret_cast<uint4*>(row + d) = pack8<P2>(a + c * 8, mul);
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 17) tmem_dealloc(tmem, kTmemCols);
}

template <int DP, typename T, int BIAS>
int launch_inst(const DkdvParams& kp, dim3 grid, cudaStream_t stream) {
  using L = DkdvSmem<DP>;
  auto kern = dkdv_kernel<DP, T, BIAS>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic) !=
        cudaSuccess)
      return FA_ERR_CUDA;
    configured[dev] = true;
  }
  kern<<<grid, 640, L::kDynamic, stream>>>(kp);
  return cudaGetLastError() == cudaSuccess ? FA_OK : FA_ERR_CUDA;
}

template <int DP, typename T>
int launch_bias(const DkdvParams& kp, int bias_kind, dim3 grid, cudaStream_t stream) {
  switch (bias_kind) {
    case FA_BIAS_NONE: return launch_inst<DP, T, 0>(kp, grid, stream);
    case FA_BIAS_SAME: return launch_inst<DP, T, 1>(kp, grid, stream);
    case FA_BIAS_BOOL: return launch_inst<DP, T, 2>(kp, grid, stream);
    default: return FA_ERR_UNSUPPORTED;
  }
}

}  // namespace

#ifdef FA_TRACE
extern "C" int fa_debug_read_trace_dkdv(long long* out, int n) {
  cudaDeviceSynchronize();
  return cudaMemcpyFromSymbol(out, g_fa_trace_dkdv, sizeof(long long) * n) == cudaSuccess ? 0 : 1;
}
#endif

int launch_bwd_dkdv(const fa_params& p, cudaStream_t stream, int* status) {
  DkdvParams kp;
  int r = make_tmap_bshd(&kp.map_q, p.q, p.B, p.M, p.H, p.D, p.q_stride, 128);
  if (r) return r;
  r = make_tmap_bshd(&kp.map_k, p.k, p.B, p.N, p.H, p.D, p.k_stride, 128);
  if (r) return r;
  r = make_tmap_bshd(&kp.map_v, p.v, p.B, p.N, p.H, p.D, p.v_stride, 128);
  if (r) return r;
  r = make_tmap_bshd(&kp.map_do, p.d_o, p.B, p.M, p.H, p.D, p.do_stride, 128);
  if (r) return r;
  if (p.write_dbias) {
    int bm, hm;
    r = make_tmap_bhmn(&kp.map_dbias, p.dbias, 2, p.B, p.H, p.M, p.N, p.dbias_stride, 64, 128, &bm,
                       &hm);
    if (r) return r;
    if (!bm || !hm) return FA_ERR_ALIGN;  // dbias must be a real (B,H,M,N) tensor
  } else {
    kp.map_dbias = kp.map_q;
  }
  auto bad = [](const void* ptr, const int64_t s[3]) {
    return reinterpret_cast<uintptr_t>(ptr) % 16 != 0 || s[0] % 8 || s[1] % 8 || s[2] % 8;
  };
  if (bad(p.dk, p.dk_stride) || bad(p.dv, p.dv_stride)) return FA_ERR_ALIGN;
  kp.bias_b_mul = kp.bias_h_mul = 0;
  kp.map_bias = kp.map_q;
  if (p.bias_kind == FA_BIAS_SAME) {
    r = make_tmap_bhmn(&kp.map_bias, p.bias, 2, p.B, p.H, p.M, p.N, p.bias_stride, 64, 128,
                       &kp.bias_b_mul, &kp.bias_h_mul);
    if (r) return r;
  } else if (p.bias_kind == FA_BIAS_BOOL) {
    r = make_tmap_bhmn(&kp.map_bias, p.bias, 1, p.B, p.H, p.M, p.N, p.bias_stride, 128, 128,
                       &kp.bias_b_mul, &kp.bias_h_mul);
    if (r) return r;
  }
  if (p.bias_kind != FA_BIAS_NONE) {
    const int eb = p.bias_kind == FA_BIAS_BOOL ? 1 : 2;
    if (reinterpret_cast<uintptr_t>(p.bias) % 16 != 0 || (p.bias_stride[0] * eb) % 16 ||
        (p.bias_stride[1] * eb) % 16 || (p.bias_stride[2] * eb) % 16)
      return FA_ERR_ALIGN;
  }
  kp.bias = p.bias;
  kp.dk = p.dk;
  kp.dv = p.dv;
  kp.lse = p.lse;
  kp.delta = p.delta;
  kp.status = status;
  kp.bias_sB = p.bias_stride[0];
  kp.bias_sH = p.bias_stride[1];
  kp.bias_sM = p.bias_stride[2];
  kp.dk_sB = p.dk_stride[0];
  kp.dk_sN = p.dk_stride[1];
  kp.dk_sH = p.dk_stride[2];
  kp.dv_sB = p.dv_stride[0];
  kp.dv_sN = p.dv_stride[1];
  kp.dv_sH = p.dv_stride[2];
  kp.H = p.H;
  kp.M = p.M;
  kp.N = p.N;
  kp.D = p.D;
  kp.causal = p.causal ? 1 : 0;
  kp.write_dbias = p.write_dbias ? 1 : 0;
  {
    const int eb = p.bias_kind == FA_BIAS_BOOL ? 1 : 2;
    kp.bias_vec32 = p.bias_kind != FA_BIAS_NONE && reinterpret_cast<uintptr_t>(p.bias) % 32 == 0 &&
                    (p.bias_stride[0] * eb) % 32 == 0 && (p.bias_stride[1] * eb) % 32 == 0 &&
                    (p.bias_stride[2] * eb) % 32 == 0;
  }
  kp.scale_log2 = p.sm_scale * kLog2e;
  kp.sm_scale = p.sm_scale;
  const dim3 grid((p.N + 127) / 128, p.B * p.H);
  const int dp = padded_head_dim(p.D);
  if (p.dtype == FA_BF16) {
    return dp == 64 ? launch_bias<64, __nv_bfloat16>(kp, p.bias_kind, grid, stream)
                    : launch_bias<128, __nv_bfloat16>(kp, p.bias_kind, grid, stream);
  }
  return dp == 64 ? launch_bias<64, __half>(kp, p.bias_kind, grid, stream)
                  : launch_bias<128, __half>(kp, p.bias_kind, grid, stream);
}

}  // namespace fa
