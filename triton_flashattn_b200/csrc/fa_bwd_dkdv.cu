// dK / dV (and dbias) kernel for sm_100a.
//
// Persistent kernel, one CTA per SM.  A tile is 128 keys of one (batch, head); a CTA
// walks its tiles one after the other and, inside a tile, the query blocks of 128 rows
// (only those at or below the diagonal when causal).  Ring stages, tensor-memory buffers
// and barrier phases run on from tile to tile, so the next tile's K / V / Q / dO loads,
// its first S and dP products and its first bias rows overlap the current tile's
// epilogue.  Roles (640 threads):
//   warps 0-15 "row" threads: warp w works on tensor-memory lanes 32*(w&3)..+31
//              (query rows of the block) and on the 32-key column quarter (w>>2)
//   warp 16    TMA producer: K, V per tile; Q ring (2), dO ring; bias tiles are asked
//              into L2 one step ahead
//   warp 17    MMA issuer for S and dP, tensor-memory owner
//   warp 18    MMA issuer for dV and dK, bulk tensor stores of dS into dbias
//   warp 19    TMA loads of the 16-bit bias tiles
// The four control warps walk their loops with all lanes converged and elect a lane only
// for the TMA / MMA / commit instructions, whose operands are then warp-uniform values.
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
// A 16-bit bias tile is brought in by TMA (warp 19) and lands exactly where the row threads
// then write P: each thread reads the four 16-byte chunks it is about to overwrite, so the
// bias needs no shared memory of its own (none is left at head dim 128); warp 18 then also
// issues the dbias stores.  A byte mask is read by the row threads straight from global
// memory, 32 contiguous bytes per thread, one query block ahead.
// Causally skipped tiles of dbias are written as zeros by this kernel, so dbias
// needs no prior fill.
// Rule kept by every barrier here: the next completion of a barrier needs progress of
// every thread that waits on it, so a parity wait can never be two phases behind.
//
// Replaces _attn_bwd_dkdv / _attn_bwd_dkdv_inner of the reference
// (flash_attention.py 237-454): same P, dS, dbias = dS, dK scaled by sm_scale.
#include "fa_common.cuh"
#include "fa_host.cuh"

namespace fa {
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
  int n_nblk, n_tiles;  // key blocks per (batch, head); tiles = n_nblk * B * H
  int causal, bias_vec32, bias_b_mul, bias_h_mul;
  int dkv_vec32;  // dk / dv bases and strides are multiples of 32 bytes
  int store_ds;    // the 16-bit dS tiles go out through map_dbias (as dbias, or as scratch for dQ)
  int zero_tiles;  // ... and zero tiles go to the causally skipped part (16-bit dbias only)
  float* dbias_f32;  // fp32 bias gradient, written from registers (fp32 bias only), or null
  int64_t dbf_sB, dbf_sH, dbf_sM;
  float scale_log2;  // sm_scale * log2(e)
  float sm_scale;
};

enum DkdvSite { kSiteKV = 1, kSiteQFull, kSiteQEmpty, kSiteDoFull, kSiteDoEmpty, kSiteSFull,
                kSiteDpFull, kSitePReady, kSiteDsReady, kSiteDvDone, kSiteDkDone, kSiteStDone,
                kSiteZeroReady, kSiteEpilogue, kSiteSFree, kSiteDpFree, kSiteKVEmpty, kSiteBiasFull };

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
  // BIAS: 0 none; 1 16-bit bias, brought in by TMA (warp 19; the dbias stores then move to
  // warp 18); 2 byte mask and 3 fp32 bias, read by the row threads from global memory (the mask
  // one step ahead, the fp32 row - 32 registers - at the start of its own step)
  constexpr int BK = BIAS;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t kv_full, kv_empty, q_full[2], q_empty[2], do_full[2], do_empty[2];
  __shared__ uint64_t s_full, dp_full, p_ready, ds_ready, dv_done, dk_done, st_done, zero_ready;
  __shared__ uint64_t s_free, dp_free, bias_full;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x;
  // the warp index as a value the compiler knows to be the same in all lanes: the role
  // branches below are then warp-uniform and the issuer warps run converged
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int lane = tid & 31;
  const int n_mblk = (p.M + 127) >> 7;

  // Schedule: tiles are numbered (batch*head)-major; CTA c takes units c, c+G, c+2G, ... so
  // that CTAs running at the same time work on neighbouring tiles and share Q / dO in L2.  A
  // unit is one tile, or - causal - two consecutive entries of the per-(batch, head) order
  // [first, last, first+1, last-1, ...]: a heavy and a light key block.
  const int sched_sh = p.causal ? 1 : 0;
  auto tile_at = [&](int it, int& bh, int& nb, int& i_start, int& T_steps) -> bool {
    const int u = static_cast<int>(blockIdx.x) + (it >> sched_sh) * static_cast<int>(gridDim.x);
    const int k = (u << sched_sh) + (it & sched_sh);
    if (k >= p.n_tiles) return false;
    bh = k / p.n_nblk;
    const int pos = k - bh * p.n_nblk;
    nb = p.causal ? ((pos & 1) ? p.n_nblk - 1 - (pos >> 1) : (pos >> 1)) : pos;
    i_start = p.causal ? min(nb, n_mblk) : 0;
    T_steps = n_mblk - i_start;
    return true;
  };

  WaitCtx ctx{&abort_flag, p.status, 2};

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&kv_full, 1);
    mbar_init(&kv_empty, 1);
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
    mbar_init(&bias_full, 1);
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
      constexpr int kBiasAhead = 1;  // bias tiles are pulled into L2 this many steps early
      uint32_t g = 0;                // steps issued so far, over all tiles
      uint32_t kvi = 0;              // tiles with at least one step so far
      int pf_done = 0;               // bias tiles of the coming tile already requested
      int bh, nb, i_start, T_steps;
      for (int it = 0; ok && tile_at(it, bh, nb, i_start, T_steps); ++it) {
        if (T_steps <= 0) continue;
        const int b = bh / p.H, h = bh - b * p.H, n0 = nb * 128;
        // K and V are single tiles: free once the previous tile's last S and dP are through
        if (kvi >= 1) ok = wait_warp(&kv_empty, (kvi - 1) & 1, ctx, kSiteKVEmpty, it);
        if (!ok) break;
        ++kvi;
        if (elect_one()) {
          mbar_expect_tx(&kv_full, 2 * L::kTile);
          for (int kb = 0; kb < KB; ++kb) {
            tma_load_4d(smem + L::kK + kb * kBlk, &p.map_k, &kv_full, kb * 64, h, n0, b);
            tma_load_4d(smem + L::kV + kb * kBlk, &p.map_v, &kv_full, kb * 64, h, n0, b);
          }
        }
        __syncwarp();
        // Bias tiles are pulled into L2 kBiasAhead steps before the row threads read them,
        // as one stream over tile boundaries: the last steps of a tile request the first
        // tiles of the next one (pf_done of them are out when that tile starts).
        auto bias_l2 = [&](int b_, int h_, int n0_, int mblk) {
          const int mp = mblk * 128;
          constexpr int kBox = BK == 1 ? 64 : (BK == 3 ? 32 : 128);  // keys per box of map_bias
          if (elect_one()) {
#pragma unroll
            for (int c = 0; c < 128; c += kBox)
              if (c == 0 || n0_ + c < p.N)
                tma_prefetch_l2_4d(&p.map_bias, n0_ + c, mp, h_ * p.bias_h_mul, b_ * p.bias_b_mul);
          }
          __syncwarp();
        };
        if (BIAS != 0) {
          for (int t = pf_done; t < kBiasAhead && t < T_steps; ++t) bias_l2(b, h, n0, i_start + t);
          pf_done = 0;
        }
        int bh2 = 0, nb2 = 0, is2 = 0, T2 = 0;
        if (BIAS != 0 && !tile_at(it + 1, bh2, nb2, is2, T2)) T2 = 0;
        for (int t = 0; t < T_steps && ok; ++t) {
          const uint32_t gs = g + t;
          const int m0 = (i_start + t) * 128;
          const int qs = gs & 1;
          if (BIAS != 0) {
            if (t + kBiasAhead < T_steps) {
              bias_l2(b, h, n0, i_start + t + kBiasAhead);
            } else if (t + kBiasAhead - T_steps < T2) {
              const int b2 = bh2 / p.H;
              bias_l2(b2, bh2 - b2 * p.H, nb2 * 128, is2 + t + kBiasAhead - T_steps);
              ++pf_done;
            }
          }
          if (gs >= 2) ok = wait_warp(&q_empty[qs], ((gs >> 1) - 1) & 1, ctx, kSiteQEmpty, t);
          if (!ok) break;
          if (elect_one()) {
            mbar_expect_tx(&q_full[qs], L::kTile);
            for (int kb = 0; kb < KB; ++kb)
              tma_load_4d(smem + L::kQ + qs * L::kTile + kb * kBlk, &p.map_q, &q_full[qs], kb * 64, h,
                          m0, b);
          }
          __syncwarp();
          const int ds = gs % kDoStages;
          const uint32_t du = gs / kDoStages;
          if (du >= 1) ok = wait_warp(&do_empty[ds], (du - 1) & 1, ctx, kSiteDoEmpty, t);
          if (!ok) break;
          if (elect_one()) {
            mbar_expect_tx(&do_full[ds], L::kTile);
            for (int kb = 0; kb < KB; ++kb)
              tma_load_4d(smem + L::kDo + ds * L::kTile + kb * kBlk, &p.map_do, &do_full[ds], kb * 64,
                          h, m0, b);
          }
          __syncwarp();
        }
        g += T_steps;
      }
    }
  } else if (warp == 17) {
    // ------------------------------------------------------- MMA issuer: S and dP
    // The whole warp walks the loop (waits included) and one elected lane issues: the
    // descriptors are then warp-uniform values, which the tensor-core instructions take
    // without a per-operand transfer from a lane's registers.
    if (live) {
      constexpr bool bf = P2::kIsBf16;
      constexpr uint32_t idesc_s = make_idesc(bf, false, false, 128, 128);
      const uint32_t k_addr = smem_u32(smem + L::kK), v_addr = smem_u32(smem + L::kV);
      const uint32_t q_addr = smem_u32(smem + L::kQ), do_addr = smem_u32(smem + L::kDo);
      const uint64_t k_km = make_sdesc(k_addr, 0, 1024), v_km = make_sdesc(v_addr, 0, 1024);
      const uint64_t q_km_0 = make_sdesc(q_addr, 0, 1024), q_km_1 = make_sdesc(q_addr + L::kTile, 0, 1024);
      const uint64_t do_km_0 = make_sdesc(do_addr, 0, 1024),
                     do_km_1 = make_sdesc(do_addr + (kDoStages - 1) * L::kTile, 0, 1024);
      bool ok = true;
      uint32_t g = 0, kvi = 0;
      int bh, nb, i_start, T_steps;
      for (int it = 0; ok && tile_at(it, bh, nb, i_start, T_steps); ++it) {
        if (T_steps <= 0) continue;
        ok = wait_warp(&kv_full, kvi & 1, ctx, kSiteKV, it);
        ++kvi;
        for (int t = 0; t < T_steps && ok; ++t) {
          const uint32_t gs = g + t;
          const int qs = gs & 1, ds = gs % kDoStages;
          const uint32_t q_par = (gs >> 1) & 1, do_par = (gs / kDoStages) & 1;
          // S_gs: its columns are free once the row threads hold S_{gs-1} in registers
          if (gs >= 1) ok = wait_warp_hot(&s_free, (gs - 1) & 1, ctx, kSiteSFree, t);
          if (ok) ok = wait_warp(&q_full[qs], q_par, ctx, kSiteQFull, t);
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            issue_gemm_ss<KS_D, false, false>(tmem + kColS, qs ? q_km_1 : q_km_0, k_km, kBlk, kBlk,
                                              idesc_s, false);
            mma_commit(&s_full);
            mma_commit(&q_empty[qs]);
          }
          __syncwarp();
          // dP_gs: same for the dP columns; dO_gs replaces dO_{gs-1} after dV_{gs-1} when
          // single-staged
          if (gs >= 1) ok = wait_warp_hot(&dp_free, (gs - 1) & 1, ctx, kSiteDpFree, t);
          if (ok) ok = wait_warp(&do_full[ds], do_par, ctx, kSiteDoFull, t);
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            issue_gemm_ss<KS_D, false, false>(tmem + kColDp, ds ? do_km_1 : do_km_0, v_km, kBlk, kBlk,
                                              idesc_s, false);
            mma_commit(&dp_full);
            mma_commit(&do_empty[ds]);
            if (t == T_steps - 1) mma_commit(&kv_empty);  // K and V may be replaced
          }
          __syncwarp();
        }
        g += T_steps;
      }
    }
    __syncwarp();
  } else if (warp == 18) {
    // ------------------------------------------------------ MMA issuer: dV and dK
    // (whole warp converged, one elected lane issues: see the S / dP issuer)
    if (live) {
      constexpr bool bf = P2::kIsBf16;
      constexpr uint32_t idesc_g = make_idesc(bf, true, true, 128, DP);
      const uint32_t q_addr = smem_u32(smem + L::kQ), do_addr = smem_u32(smem + L::kDo);
      const uint32_t p_addr = smem_u32(smem + L::kP), ds_addr = smem_u32(smem + L::kDs);
      const uint64_t q_mn_0 = make_sdesc(q_addr, kBlk, 1024), q_mn_1 = make_sdesc(q_addr + L::kTile, kBlk, 1024);
      const uint64_t do_mn_0 = make_sdesc(do_addr, kBlk, 1024),
                     do_mn_1 = make_sdesc(do_addr + (kDoStages - 1) * L::kTile, kBlk, 1024);
      const uint64_t p_mn = make_sdesc(p_addr, kBlk, 1024), ds_mn = make_sdesc(ds_addr, kBlk, 1024);
      // The elected lane also sends the dS tiles out as dbias (a bias gradient only exists for a
      // 16-bit bias).  st_done completes once per step when the store of dS has finished
      // reading sDS and - causal only - once per tile before that, when the zero tiles above
      // the diagonal are out.  (Without the zero tiles there is no per-tile completion: two
      // completions in a row that no row thread has to wait for in between would let a parity
      // wait fall two phases behind.)  The wait for the store's read sits right after the
      // store: the next thing this warp needs, P of the next step, is further away.
      const bool stores_here = p.store_ds != 0;
      bool zeros_in_flight = false;
      bool ok = true;
      uint32_t g = 0;
      int bh, nb, i_start, T_steps;
      for (int it = 0; ok && tile_at(it, bh, nb, i_start, T_steps); ++it) {
        const int b = bh / p.H, h = bh - b * p.H, n0 = nb * 128;
        if (p.zero_tiles) {
          ok = wait_warp(&zero_ready, it & 1, ctx, kSiteZeroReady, it);
          if (!ok) break;
          if (elect_one()) {
            for (int i = 0; i < i_start; ++i) {
              tma_store_4d(&p.map_dbias, smem + L::kDs, n0, i * 128, h, b);
              if (n0 + 64 < p.N)
                tma_store_4d(&p.map_dbias, smem + L::kDs + kBlk, n0 + 64, i * 128, h, b);
            }
            tma_store_commit();
            if (T_steps <= 0) {
              tma_store_wait_read<0>();
              mbar_arrive(&st_done);
            }
          }
          __syncwarp();
          // the zero tiles are read out of sDS while P of the first step is formed and dV is
          // issued; their completion is announced just before this warp needs dS
          zeros_in_flight = T_steps > 0;
        }
        for (int t = 0; t < T_steps && ok; ++t) {
          const uint32_t gs = g + t;
          const int qs = gs & 1;
          const int ds = gs % kDoStages;
          // dV += P^T dO  (dO must have landed: P only depends on S).  The first product of a
          // tile overwrites dV / dK: P and dS of a new tile are only announced by all sixteen
          // row warps after they have read the previous tile's accumulators.
          ok = wait_warp_hot(&p_ready, gs & 1, ctx, kSitePReady, t);
          if (ok) ok = wait_warp(&do_full[ds], (gs / kDoStages) & 1, ctx, kSiteDoFull, t);
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            issue_gemm_ss<8, true, true>(tmem + kColDv, p_mn, ds ? do_mn_1 : do_mn_0, kBlk, kBlk, idesc_g,
                                         t > 0);
            mma_commit(&do_empty[ds]);
            mma_commit(&dv_done);
            if (zeros_in_flight) {
              tma_store_wait_read<0>();
              mbar_arrive(&st_done);
            }
          }
          __syncwarp();
          zeros_in_flight = false;
          // dK += dS^T Q
          ok = wait_warp_hot(&ds_ready, gs & 1, ctx, kSiteDsReady, t);
          if (ok) ok = wait_warp(&q_full[qs], (gs >> 1) & 1, ctx, kSiteQFull, t);
          if (!ok) break;
          tc_fence_after();
          if (elect_one()) {
            issue_gemm_ss<8, true, true>(tmem + kColDk, ds_mn, qs ? q_mn_1 : q_mn_0, kBlk, kBlk, idesc_g,
                                         t > 0);
            mma_commit(&q_empty[qs]);
            mma_commit(&dk_done);
            if (stores_here) {
              const int m0 = (i_start + t) * 128;
              tma_store_4d(&p.map_dbias, smem + L::kDs, n0, m0, h, b);
              if (n0 + 64 < p.N) tma_store_4d(&p.map_dbias, smem + L::kDs + kBlk, n0 + 64, m0, h, b);
              tma_store_commit();
              tma_store_wait_read<0>();
              mbar_arrive(&st_done);
            }
          }
          __syncwarp();
        }
        g += T_steps;
      }
      if (stores_here && elect_one()) tma_store_wait_all<0>();
    }
    __syncwarp();
  } else if (warp == 19) {
    // ----------------------------------------------------------- bias tile loads
    // The [128 rows][128 keys] 16-bit bias tile of a step lands exactly where the row threads
    // will then write P (same two swizzled blocks, every thread reads the four 16-byte
    // chunks it is about to overwrite): no extra shared memory.  sP is free for it once the
    // dV product of the previous step has read P.
    // (whole warp converged, one elected lane issues: the load follows the barrier sooner)
    if (BIAS == 1 && live) {
      if (lane == 0) tma_prefetch_desc(&p.map_bias);
      bool ok = true;
      uint32_t g = 0;
      int bh, nb, i_start, T_steps;
      for (int it = 0; ok && tile_at(it, bh, nb, i_start, T_steps); ++it) {
        const int b = bh / p.H, h = bh - b * p.H, n0 = nb * 128;
        const bool two = n0 + 64 < p.N;
        for (int t = 0; t < T_steps && ok; ++t) {
          const uint32_t gs = g + t;
          if (gs >= 1) ok = wait_warp_hot(&dv_done, (gs - 1) & 1, ctx, kSiteDvDone, t);
          if (!ok) break;
          const int m0 = (i_start + t) * 128;
          if (elect_one()) {
            mbar_expect_tx(&bias_full, two ? 2 * kBlk : kBlk);
            tma_load_4d(smem + L::kP, &p.map_bias, &bias_full, n0, m0, h * p.bias_h_mul,
                        b * p.bias_b_mul);
            if (two)
              tma_load_4d(smem + L::kP + kBlk, &p.map_bias, &bias_full, n0 + 64, m0, h * p.bias_h_mul,
                          b * p.bias_b_mul);
          }
          __syncwarp();
        }
        g += T_steps;
      }
    }
    __syncwarp();
  } else {
    // --------------------------------------------------------------- row threads
    const int r = (warp & 3) * 32 + lane;  // query row inside the block = tensor-memory lane
    const int qt = warp >> 2;              // column quarter: keys n0 + 32*qt .. +31
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32u;
    bool ok = live;
    // this thread's four 16-byte chunks inside the [128][128] 16-bit tiles: chunk c of the
    // row lands at sp_row + ((chunk0 + c) ^ (r & 7)) * 16; the dS tile sits kDs - kP further
    const uint32_t sp_row = smem_u32(smem + L::kP + (qt >> 1) * kBlk) + static_cast<uint32_t>(r) * 128u;
    const uint32_t chunk0 = (qt & 1) * 4;
    // tensor-memory address of this thread's 32 columns of S (dP: + kColDp)
    const uint32_t tm_sc = tmem_addr(tmem, lane_base, kColS + qt * 32);

    constexpr int BR = BIAS == 1 ? 0 : BK;  // bias staged in registers only for kinds 2 and 3
    BiasRegs<BR> bnext;
    // LSE2 and delta of the coming step's row, as loaded: they are only looked at (negated,
    // replaced for rows beyond M) when that step starts, so the loads travel during this one
    float lse_next = 0.f, delta_next = 0.f;
    bool row_ok_next = false;
    // fetches bias / -LSE2 / delta of query block `mblk` for the tile (bh_, key column c0)
    auto prefetch = [&](int bh_, int c0, int mblk) {
      const int b_ = bh_ / p.H, h_ = bh_ - b_ * p.H;
      const int64_t bias_bh = b_ * p.bias_sB + h_ * p.bias_sH;
      const int m = mblk * 128 + r;
      const bool row_ok = m < p.M;
      if constexpr (BR == 2) {
        load_bias_row<BK>(bnext, p.bias, bias_bh + (int64_t)m * p.bias_sM, row_ok, c0, p.N,
                          p.bias_vec32 != 0);
      }
      const int64_t idx = (int64_t)bh_ * p.M + min(m, p.M - 1);
      lse_next = __ldcg(p.lse + idx);
      delta_next = __ldcg(p.delta + idx);
      row_ok_next = row_ok;
    };
    // Loop state is kept small on purpose (registers): the running step count gs, the tile
    // counter it, and per tile bh, col0 and the current query block mb; the first query block
    // of a tile is recomputed from col0 where needed.
    uint32_t gs = 0;  // steps done so far, over all tiles
    int bh, nb, i_start, T_steps;
    if (ok && tile_at(0, bh, nb, i_start, T_steps) && T_steps > 0) prefetch(bh, nb * 128 + qt * 32, i_start);
#pragma unroll 1
    for (int it = 0; ok && tile_at(it, bh, nb, i_start, T_steps); ++it) {
      const int col0 = nb * 128 + qt * 32;
      if (p.zero_tiles) {
        // sDS becomes the zero tile for the causally skipped part of dbias: the last dbias
        // store of the previous tile must have read it (the last dK product has: its barrier
        // was seen in that tile's epilogue).  Causal completions of st_done: tile `it` owns
        // indices gs+it (zero tiles out) and gs+it+1+t (store of step t).
        if (it >= 1) ok = wait_warp(&st_done, (gs + it - 1) & 1, ctx, kSiteStDone, it);
        if (!ok) break;
        const uint32_t z = sp_row - static_cast<uint32_t>(r) * 128u - (qt >> 1) * kBlk + (L::kDs - L::kP);
        for (int i = tid; i < 2 * kBlk / 16; i += 512) sts128(z + i * 16, 0, 0, 0, 0);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&zero_ready);
      }

#pragma unroll 1
      for (int mb = i_start; mb < n_mblk && ok; ++mb, ++gs) {
        const int i0 = p.causal ? min(col0 >> 7, n_mblk) : 0;  // first query block of the tile
        const int t = mb - i0;
        const int m0 = mb * 128;
        BiasRegs<BR> bcur = bnext;
        if constexpr (BR == 3) {
          // fp32 bias row of this step: asked for now, used once S has arrived
          const int b_ = bh / p.H, h_ = bh - b_ * p.H;
          load_bias_row<3>(bcur, p.bias, b_ * p.bias_sB + h_ * p.bias_sH + (int64_t)(m0 + r) * p.bias_sM,
                           m0 + r < p.M, col0, p.N, p.bias_vec32 != 0);
        }
        // rows beyond M get -inf / 0, which makes their P and dS zero
        const float neg_lse = row_ok_next ? -lse_next : -INFINITY, delta_r = row_ok_next ? delta_next : 0.f;
        if (mb + 1 < n_mblk) prefetch(bh, col0, mb + 1);
        // S and "dV of the previous step has read P" are usually true by now: one combined look
        uint32_t ps = 0, pdv = 1, pb = 1;
        if (BIAS == 1 && t >= 1)
          mbar_poll3(&s_full, gs & 1, &dv_done, (gs - 1) & 1, &bias_full, gs & 1, ps, pdv, pb);
        else if (BIAS == 1)
          mbar_poll2(&s_full, gs & 1, &bias_full, gs & 1, ps, pb);
        else if (t >= 1)
          mbar_poll2(&s_full, gs & 1, &dv_done, (gs - 1) & 1, ps, pdv);
        else
          ps = mbar_poll(&s_full, gs & 1);

        // ---- P
        ok = wait_warp_polled(ps, &s_full, gs & 1, ctx, kSiteSFull, t);
        if (!ok) break;
        tc_fence_after();
        float pr[32];
        tmem_ld32(tm_sc, reinterpret_cast<uint32_t*>(pr));
        tmem_ld_wait();
        // S now lives in registers: hand its columns back for the next S
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free);
        // P = exp2(S * scale * log2e + bias * log2e - LSE2); rows beyond M have LSE2 = +inf
        if constexpr (BIAS == 1) {
          // the bias tile sits where this thread's P chunks go; what does not need it is
          // computed while it travels: x = S * scale * log2e - LSE2
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const f32x2 x = ffma2(f2(pr[i], pr[i + 1]), f2(p.scale_log2, p.scale_log2), f2(neg_lse, neg_lse));
            pr[i] = f2_lo(x);
            pr[i + 1] = f2_hi(x);
          }
          ok = wait_warp_polled(pb, &bias_full, gs & 1, ctx, kSiteBiasFull, t);
          if (!ok) break;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint4 v = lds128(sp_row + (((chunk0 + c) ^ (r & 7)) << 4));
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = P2::unpack(w[e]);
              const int i = c * 8 + e * 2;
              const f32x2 a = ffma2(f2(f.x, f.y), f2(kLog2e, kLog2e), f2(pr[i], pr[i + 1]));
              const f32x2 pe = f2(ex2(f2_lo(a)), ex2(f2_hi(a)));
              pr[i] = f2_lo(pe);
              pr[i + 1] = f2_hi(pe);
            }
          }
        } else {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          f32x2 a = ffma2(f2(pr[i], pr[i + 1]), f2(p.scale_log2, p.scale_log2), f2(neg_lse, neg_lse));
          if (BK == 3)
            a = ffma2(f2(__uint_as_float(bcur.w[i]), __uint_as_float(bcur.w[i + 1])), f2(kLog2e, kLog2e), a);
          const f32x2 pe = f2(ex2(f2_lo(a)), ex2(f2_hi(a)));
          if (BK == 2) {
            const uint32_t m2 = bcur.w[i >> 2] >> (8 * (i & 3));
            pr[i] = (m2 & 0xFFu) != 0 ? f2_lo(pe) : 0.f;
            pr[i + 1] = (m2 & 0xFF00u) != 0 ? f2_hi(pe) : 0.f;
          } else {
            pr[i] = f2_lo(pe);
            pr[i + 1] = f2_hi(pe);
          }
        }
        }
        if ((col0 + 32 > p.N) || (p.causal && col0 + 31 > m0)) {
          int limit = p.N - col0;
          if (p.causal) limit = min(limit, m0 + r - col0 + 1);
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i >= limit) pr[i] = 0.f;
        }
        if (t >= 1) {
          ok = wait_warp_polled(pdv, &dv_done, (gs - 1) & 1, ctx, kSiteDvDone, t);
          if (!ok) break;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c)
          sts128(sp_row + (((chunk0 + c) ^ (r & 7)) << 4), P2::pack(pr[c * 8 + 0], pr[c * 8 + 1]),
                 P2::pack(pr[c * 8 + 2], pr[c * 8 + 3]), P2::pack(pr[c * 8 + 4], pr[c * 8 + 5]),
                 P2::pack(pr[c * 8 + 6], pr[c * 8 + 7]));
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_ready);

        // ---- dS
        // dP, "dK of the previous step has read dS" and "its dbias store has": one combined look
        uint32_t pdp = 0, pdk = 1, pst = 1;
        // sDS may be rewritten once its previous dbias store has read it: causal -> completion
        // gs+it of st_done (see above); otherwise completion gs-1 (the store of step gs-1)
        const uint32_t st_par = (p.zero_tiles ? gs + it : gs - 1) & 1;
        const bool st_wait = p.store_ds && (p.zero_tiles || gs >= 1);
        if (t >= 1 && st_wait)
          mbar_poll3(&dp_full, gs & 1, &dk_done, (gs - 1) & 1, &st_done, st_par, pdp, pdk, pst);
        else if (t >= 1)
          mbar_poll2(&dp_full, gs & 1, &dk_done, (gs - 1) & 1, pdp, pdk);
        else if (st_wait)
          mbar_poll2(&dp_full, gs & 1, &st_done, st_par, pdp, pst);
        else
          pdp = mbar_poll(&dp_full, gs & 1);
        ok = wait_warp_polled(pdp, &dp_full, gs & 1, ctx, kSiteDpFull, t);
        if (!ok) break;
        tc_fence_after();
        uint32_t dsu[16];
        // dP is fetched in two halves: fewer registers are live at once
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          uint32_t dp[16];
          tmem_ld16(tm_sc + (kColDp - kColS) + hf * 16, dp);
          tmem_ld_wait();
          if (hf == 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&dp_free);
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int e = hf * 16 + 2 * i;
            const f32x2 d = fmul2(f2(pr[e], pr[e + 1]),
                                  fadd2(f2(__uint_as_float(dp[2 * i]), __uint_as_float(dp[2 * i + 1])),
                                        f2(-delta_r, -delta_r)));
            dsu[hf * 8 + i] = P2::pack(f2_lo(d), f2_hi(d));
            if (BIAS == 3) {
              dp[2 * i] = __float_as_uint(f2_lo(d));
              dp[2 * i + 1] = __float_as_uint(f2_hi(d));
            }
          }
          if (BIAS == 3 && p.dbias_f32 != nullptr && m0 + r < p.M) {
            // the fp32 bias gradient goes out unrounded, 64 contiguous bytes per thread and half
            const int b_ = bh / p.H, h_ = bh - b_ * p.H;
            const int c0 = col0 + hf * 16;
            float* drow = p.dbias_f32 + b_ * p.dbf_sB + h_ * p.dbf_sH + (int64_t)(m0 + r) * p.dbf_sM + c0;
            if (c0 + 16 <= p.N) {
#pragma unroll
              for (int k = 0; k < 4; ++k)
                *reinterpret_cast<uint4*>(drow + 4 * k) = make_uint4(dp[4 * k], dp[4 * k + 1], dp[4 * k + 2], dp[4 * k + 3]);
            } else {
#pragma unroll
              for (int k = 0; k < 16; ++k)
                if (c0 + k < p.N) drow[k] = __uint_as_float(dp[k]);
            }
          }
        }
        if (t >= 1) {
          ok = wait_warp_polled(pdk, &dk_done, (gs - 1) & 1, ctx, kSiteDkDone, t);
          if (!ok) break;
        }
        if (st_wait) {
          ok = wait_warp_polled(pst, &st_done, st_par, ctx, kSiteStDone, t);
          if (!ok) break;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c)
          sts128(sp_row + (L::kDs - L::kP) + (((chunk0 + c) ^ (r & 7)) << 4), dsu[c * 4 + 0],
                 dsu[c * 4 + 1], dsu[c * 4 + 2], dsu[c * 4 + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ds_ready);
      }
      if (!ok) break;

      // the next tile's first bias / LSE / delta rows travel while this tile's result is stored
      {
        int bh2, nb2, is2, T2;
        if (tile_at(it + 1, bh2, nb2, is2, T2) && T2 > 0) prefetch(bh2, nb2 * 128 + qt * 32, is2);
      }

      // ---- epilogue: dV, dK (rows = keys) -> global
      const int steps_here = n_mblk - (p.causal ? min(col0 >> 7, n_mblk) : 0);
      if (steps_here > 0) {
        ok = wait_warp(&dv_done, (gs - 1) & 1, ctx, kSiteEpilogue, 0);
        if (ok) ok = wait_warp(&dk_done, (gs - 1) & 1, ctx, kSiteEpilogue, 1);
        if (!ok) break;
      }
      {
        tc_fence_after();
        const int b = bh / p.H, h = bh - b * p.H;
        const int n = (col0 & ~127) + r;
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
          if (steps_here > 0) {
            tmem_ld_cols<kQD>(tm_sc - qt * 32 + colbase + d0, a);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < kQD; ++i) a[i] = 0;
          }
          if (n < p.N) {
            if (p.dkv_vec32 && d0 + kQD <= p.D) {
              // whole 32-byte sectors per store: half as many transactions as 16-byte stores for
              // these row-strided writes
#pragma unroll
              for (int c = 0; c < kQD / 16; ++c) {
                const uint4 lo = pack8<P2>(a + c * 16, mul), hi = pack8<P2>(a + c * 16 + 8, mul);
                asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(row + d0 + c * 16),
                             "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
                             : "memory");
              }
            } else {
#pragma unroll
              for (int c = 0; c < kQD / 8; ++c) {
                const int d = d0 + c * 8;
                if (d < p.D) *reinterpret_cast<uint4*>(row + d) = pack8<P2>(a + c * 8, mul);
              }
            }
          }
        }
        // the accumulators are in registers: the next tile's first products may overwrite them
        tc_fence_before();
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
  return launch_overlapped(kern, grid, 640, L::kDynamic, stream, kp);
}

template <int DP, typename T>
int launch_bias(const DkdvParams& kp, int bias_kind, dim3 grid, cudaStream_t stream) {
  switch (bias_kind) {
    case FA_BIAS_NONE: return launch_inst<DP, T, 0>(kp, grid, stream);
    case FA_BIAS_SAME: return launch_inst<DP, T, 1>(kp, grid, stream);
    case FA_BIAS_BOOL: return launch_inst<DP, T, 2>(kp, grid, stream);
    case FA_BIAS_F32: return launch_inst<DP, T, 3>(kp, grid, stream);
    default: return FA_ERR_UNSUPPORTED;
  }
}

}  // namespace


int launch_bwd_dkdv(const fa_params& p, cudaStream_t stream, int* status) {
  if (p.D == 256) return launch_bwd_dkdv_d256(p, stream, status);
  DkdvParams kp;
  int r = make_tmap_bshd(&kp.map_q, p.q, p.B, p.M, p.H, p.D, p.q_stride, 128);
  if (r) return r;
  r = make_tmap_bshd(&kp.map_k, p.k, p.B, p.N, p.H, p.D, p.k_stride, 128);
  if (r) return r;
  r = make_tmap_bshd(&kp.map_v, p.v, p.B, p.N, p.H, p.D, p.v_stride, 128);
  if (r) return r;
  r = make_tmap_bshd(&kp.map_do, p.d_o, p.B, p.M, p.H, p.D, p.do_stride, 128);
  if (r) return r;
  const bool f32 = p.bias_kind == FA_BIAS_F32;
  kp.store_ds = f32 ? 1 : (p.write_dbias ? 1 : 0);
  kp.zero_tiles = !f32 && p.write_dbias && p.causal;
  kp.dbias_f32 = nullptr;
  kp.dbf_sB = kp.dbf_sH = kp.dbf_sM = 0;
  if (kp.store_ds) {
    // the 16-bit dS tiles: the bias gradient itself, or (fp32 bias) the scratch the dQ stage reads
    const void* dst = f32 ? p.ds16 : p.dbias;
    const int64_t* dst_stride = f32 ? p.ds16_stride : p.dbias_stride;
    if (!dst) return FA_ERR_NULL;
    int bm, hm;
    r = make_tmap_bhmn(&kp.map_dbias, dst, 2, p.B, p.H, p.M, p.N, dst_stride, 64, 128, &bm, &hm);
    if (r) return r;
    if (!bm || !hm) return FA_ERR_ALIGN;  // must be a real (B,H,M,N) tensor
  } else {
    kp.map_dbias = kp.map_q;
  }
  if (f32 && p.write_dbias) {
    if (reinterpret_cast<uintptr_t>(p.dbias) % 16 != 0 || p.dbias_stride[0] % 4 || p.dbias_stride[1] % 4 ||
        p.dbias_stride[2] % 4)
      return FA_ERR_ALIGN;
    kp.dbias_f32 = static_cast<float*>(p.dbias);
    kp.dbf_sB = p.dbias_stride[0];
    kp.dbf_sH = p.dbias_stride[1];
    kp.dbf_sM = p.dbias_stride[2];
  }
  auto bad = [](const void* ptr, const int64_t s[3]) {
    return reinterpret_cast<uintptr_t>(ptr) % 16 != 0 || s[0] % 8 || s[1] % 8 || s[2] % 8;
  };
  if (bad(p.dk, p.dk_stride) || bad(p.dv, p.dv_stride)) return FA_ERR_ALIGN;
  auto al32 = [](const void* ptr, const int64_t s[3]) {
    return reinterpret_cast<uintptr_t>(ptr) % 32 == 0 && s[0] % 16 == 0 && s[1] % 16 == 0 && s[2] % 16 == 0;
  };
  kp.dkv_vec32 = al32(p.dk, p.dk_stride) && al32(p.dv, p.dv_stride);
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
  } else if (f32) {
    r = make_tmap_bhmn(&kp.map_bias, p.bias, 4, p.B, p.H, p.M, p.N, p.bias_stride, 32, 128,
                       &kp.bias_b_mul, &kp.bias_h_mul);
    if (r) return r;
  }
  if (p.bias_kind != FA_BIAS_NONE) {
    const int eb = p.bias_kind == FA_BIAS_BOOL ? 1 : (f32 ? 4 : 2);
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
  {
    const int eb = p.bias_kind == FA_BIAS_BOOL ? 1 : (f32 ? 4 : 2);
    kp.bias_vec32 = p.bias_kind != FA_BIAS_NONE && reinterpret_cast<uintptr_t>(p.bias) % 32 == 0 &&
                    (p.bias_stride[0] * eb) % 32 == 0 && (p.bias_stride[1] * eb) % 32 == 0 &&
                    (p.bias_stride[2] * eb) % 32 == 0;
  }
  kp.scale_log2 = p.sm_scale * kLog2e;
  kp.sm_scale = p.sm_scale;
  kp.n_nblk = (p.N + 127) / 128;
  kp.n_tiles = kp.n_nblk * p.B * p.H;
  const int units = p.causal ? (kp.n_tiles + 1) / 2 : kp.n_tiles;
  const dim3 grid(persistent_grid(units));
  const int dp = padded_head_dim(p.D);
  if (p.dtype == FA_BF16) {
    return dp == 64 ? launch_bias<64, __nv_bfloat16>(kp, p.bias_kind, grid, stream)
                    : launch_bias<128, __nv_bfloat16>(kp, p.bias_kind, grid, stream);
  }
  return dp == 64 ? launch_bias<64, __half>(kp, p.bias_kind, grid, stream)
                  : launch_bias<128, __half>(kp, p.bias_kind, grid, stream);
}

}  // namespace fa
