// Forward attention kernel for sm_100a.
//
// Persistent kernel, one CTA per SM.  A CTA works on PAIRS of query tiles: two
// consecutive blocks of 128 query rows of one (batch, head), which share every K / V
// block they visit.  Roles (384 threads):
//   warps 0-3   softmax group of tile 0: thread = one query row (= tensor-memory lane)
//   warps 4-7   softmax group of tile 1
//   warp 8      TMA producer (converged, an elected lane issues): Q pair per unit, K ring (128-key stages), V ring
//               (64-key half stages)
//   warp 9      MMA issuer of tile 0 (converged, an elected lane issues), tensor-memory owner
//   warp 10     TMA producer of the bias / mask ring (converged, an elected lane issues).
//               (Asking TMA to pull the tiles a few units ahead into L2 as well made the
//               kernel 4-5 % slower and was removed.)
//   warp 11     MMA issuer of tile 1 (converged, an elected lane issues)
// Tensor memory: S0 | S1 | O0 | O1, 128 columns each.  The 128 score columns of a tile are
// two halves of 64 that swap roles every key block.  In step c (f = c & 1):
//   columns [64f, 64f+64)       scores of keys 0-63, read first; afterwards they hold the
//                               16-bit P of all 128 keys (two halves of 32 columns)
//   columns [64(1-f), +64)      scores of keys 64-127, read second; once they are in
//                               registers the columns are free, and the scores of keys 0-63
//                               of the NEXT block are computed into them while this step's
//                               second softmax half still runs
// Per key block j and tile t:
//   S_t[half] = Q_t K_j[half]^T    (both operands in shared memory, N = 64)
//   the row thread adds the bias tile (streamed by TMA into a ring of [128 rows][64 keys]
//   units), applies the masks, updates the running maximum (log2 domain), forms
//   P = exp2(s - m) and writes the 16-bit P half
//   O_t += P_t[half] V_j[half]     (P is the tensor-memory operand, V MN-major in shared
//                                   memory), issued per half
//   the scores of keys 64-127 of block j+1 go over the columns P_t(j) was read from: same
//   issuing thread, and products issued by one thread execute in issue order, so no barrier
//   is needed between them
// The control warps (producers, issuers) walk their loops with all 32 lanes converged and
// elect a lane only for the TMA / MMA / commit instructions themselves: the descriptors and
// coordinates are then warp-uniform values.  (Run by a single lane under a divergent branch,
// every operand of every such instruction is first moved from that lane's registers, which
// made a product of eight instructions take ~850 cycles to issue and a bias load reach the
// ring a few hundred cycles later: 5-20 % of the kernel, depending on the workload.)
// So a softmax group only waits for the tensor core at the start of a unit; the two tiles'
// products interleave freely on the tensor core.  A row is owned by one thread: the row
// maximum and the row sum need no exchange between threads.  The running maximum is only
// raised when it grows by more than 8 (log2 units); only then is O rescaled (by the row's
// own thread, after the products into it have finished).  Ring stages, tensor-memory
// buffers and barrier phases run on from unit to unit.  K / V ring stages are handed back
// by both issuers (their "empty" barriers count two arrivals); an issuer whose tile does
// not visit a block still waits for its loads and hands the stages back, so that every
// waiter sees every completion of a barrier it waits on.
//
// Replaces _attn_fwd / _attn_fwd_inner of the reference (flash_attention.py
// lines 12-194): same masks (bounds, top-left causal, bool, additive float
// bias), same base-2 softmax and the same saved log2-domain log-sum-exp.
#include "fa_common.cuh"
#include "fa_host.cuh"

namespace fa {
namespace {

struct FwdParams {
  CUtensorMap map_q;
  CUtensorMap map_k;
  CUtensorMap map_v;  // box of 64 keys
  CUtensorMap map_bias;
  void* o;
  float* lse;
  int* status;
  int64_t o_sB, o_sM, o_sH;
  int H, M, N, D;
  int causal;
  int o_vec32;  // o's base and strides are multiples of 32 bytes
  int bias_b_mul, bias_h_mul;
  int n_mblk, n_pairs, n_units;  // query blocks / block pairs per (batch, head); units = pairs * B * H
  float sm_scale;
};

enum FwdSite { kSiteQFull = 1, kSiteQEmpty, kSiteKFull, kSiteKEmpty, kSiteVFull, kSiteVEmpty,
               kSiteSFull, kSiteSRead, kSitePFull, kSitePvDone, kSiteBiasFull, kSiteBiasEmpty, kSiteEpilogue };

template <int DP, int BIAS>
struct FwdSmem {
  static constexpr int kQTile = 128 * DP * 2;   // one query tile
  static constexpr int kKStage = 128 * DP * 2;  // 128 keys
  static constexpr int kVHalf = 64 * DP * 2;    // 64 keys
  // Head dim 256: one query tile per unit, single K stage, two V half stages, two bias units
  // (64 + 64 + 64 + 32 KB); otherwise two tiles, 2 / 3 / 3 stages (64 + 64 + 48 + 48 KB at 128).
  static constexpr int kTiles = DP == 256 ? 1 : 2;
  static constexpr int kKStages = DP == 256 ? 1 : 2;
  static constexpr int kVStages = DP == 256 ? 2 : 3;
  static constexpr int kBiasStages = BIAS == 0 ? 0 : (DP == 256 ? 2 : 3);  // 16 KB units
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTiles * kQTile;
  static constexpr int kV = kK + kKStages * kKStage;
  static constexpr int kBias = kV + kVStages * kVHalf;
  static constexpr int kTotal = kBias + kBiasStages * kBlk;
  static constexpr int kDynamic = kTotal + 1024;  // slack for 1024-byte alignment
};

// The unit (pair of query tiles) number `it` of this CTA.  Units are numbered
// (batch*head)-major; CTA c takes c, c+G, c+2G, ... so that CTAs running at the same time
// share K / V in L2.  Causal: the entries of one (batch, head) are ordered [last, first,
// last-1, first+1, ...] and a CTA takes two consecutive ones, a heavy and a light pair.
struct Unit {
  int bh, mb0;   // (batch, head) and first query block of the pair
  int nb0, nb1;  // key blocks each tile visits (0: the tile does not exist)
  int nmax;
  __device__ __forceinline__ int nb(int t) const { return t ? nb1 : nb0; }
};
template <int TILES>  // query tiles per unit: 2, or 1 at head dim 256
__device__ __forceinline__ bool unit_at(const FwdParams& p, int it, Unit& u) {
  const int sh = p.causal ? 1 : 0;
  const int c = static_cast<int>(blockIdx.x) + (it >> sh) * static_cast<int>(gridDim.x);
  const int k = (c << sh) + (it & sh);
  if (k >= p.n_units) return false;
  u.bh = k / p.n_pairs;
  const int pos = k - u.bh * p.n_pairs;
  const int pair = p.causal ? ((pos & 1) ? (pos >> 1) : p.n_pairs - 1 - (pos >> 1)) : pos;
  u.mb0 = pair * TILES;
  const int nblk_all = (p.N + 127) >> 7;
  u.nb0 = u.mb0 >= p.n_mblk ? 0 : (p.causal ? min(nblk_all, u.mb0 + 1) : nblk_all);
  u.nb1 = (TILES < 2 || u.mb0 + 1 >= p.n_mblk) ? 0 : (p.causal ? min(nblk_all, u.mb0 + 2) : nblk_all);
  u.nmax = max(u.nb0, u.nb1);
  return true;
}

// Walks the bias units of this CTA in the order the softmax groups consume them:
// per unit, per key block j, per tile t (if it visits j): two 64-key halves (16-bit bias),
// four 32-key quarters (fp32 bias) or one unit (byte mask, [128][128] bytes per block).
template <int BIAS, int TILES>
struct BiasWalk {
  static constexpr int kSub = BIAS == 1 ? 2 : (BIAS == 3 ? 4 : 1);  // units per (tile, block)
  int it = 0, j = 0, t = 0, h = 0;
  Unit u;
  bool valid = false;
  __device__ __forceinline__ void settle(const FwdParams& p) {
    // moves (it, j, t) forward to the next existing (tile, block), h stays 0
    while (valid) {
      if (j >= u.nmax) {
        ++it;
        j = 0;
        t = 0;
        valid = unit_at<TILES>(p, it, u);
        continue;
      }
      if (t >= 2) {
        ++j;
        t = 0;
        continue;
      }
      if (j >= u.nb(t)) {
        ++t;
        continue;
      }
      return;
    }
  }
  __device__ __forceinline__ void start(const FwdParams& p) {
    valid = unit_at<TILES>(p, 0, u);
    settle(p);
  }
  __device__ __forceinline__ void next(const FwdParams& p) {
    if (h + 1 < kSub) {
      ++h;
      return;
    }
    h = 0;
    ++t;
    settle(p);
  }
  // coordinates of the current unit's box: (key, row, head, batch)
  __device__ __forceinline__ void coords(const FwdParams& p, int& n0, int& m0, int& hh, int& bb) const {
    const int b = u.bh / p.H;
    n0 = j * 128 + h * (128 / kSub);
    m0 = (u.mb0 + t) * 128;
    hh = (u.bh - b * p.H) * p.bias_h_mul;
    bb = b * p.bias_b_mul;
  }
};

template <int DP, typename T, int BIAS>
__global__ void __launch_bounds__(384, 1) fwd_kernel(const __grid_constant__ FwdParams p) {
  using L = FwdSmem<DP, BIAS>;
  using P2 = Pack2<T>;
  constexpr int KB = DP / 64;     // 64-column blocks per Q / K / V tile
  constexpr int KS_QK = DP / 16;  // MMA K slices of Q K^T
  constexpr uint32_t NB = L::kBiasStages > 0 ? L::kBiasStages : 1;
  constexpr uint32_t VS = L::kVStages;
  constexpr uint32_t KST = L::kKStages;
  constexpr uint32_t kTmemCols = 512;
  constexpr int kVBlk = 64 * 128;  // bytes of one [64 keys][64] block of a V half stage

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t q_full, q_empty, k_full[2], k_empty[2], v_full[3], v_empty[3];  // rings: up to 2 / 3 stages
  __shared__ uint64_t s_full[2][2], s_read[2], p_full[2][2], pv_done[2][2];
  __shared__ uint64_t bias_full[2][3], bias_empty[3];  // full: one set per consuming group
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x;
  // the warp index as a value the compiler knows to be the same in all lanes
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int lane = tid & 31;

  WaitCtx ctx{&abort_flag, p.status, 1};

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&q_full, 1);
    mbar_init(&q_empty, 2);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 2);
      mbar_init(&s_read[i], 4);
      for (int h = 0; h < 2; ++h) {
        mbar_init(&s_full[i][h], 1);
        mbar_init(&p_full[i][h], 4);
        mbar_init(&pv_done[i][h], 1);
      }
    }
    for (int i = 0; i < 3; ++i) {
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 2);
      mbar_init(&bias_full[0][i], 1);
      mbar_init(&bias_full[1][i], 1);
      mbar_init(&bias_empty[i], 4);
    }
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(&tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;
  grid_dep_launch_next();
  grid_dep_wait();  // the previous kernel's results (and its status word) are visible from here
  // A kernel launched after an earlier one recorded an error does no work.
  const bool live = *reinterpret_cast<volatile int*>(p.status) == 0;

  if (warp == 8) {
    // ------------------------------------------------------------------ producer
    // (whole warp converged, one elected lane issues)
    if (live) {
      if (lane == 0) {
        tma_prefetch_desc(&p.map_q);
        tma_prefetch_desc(&p.map_k);
        tma_prefetch_desc(&p.map_v);
      }
      bool ok = true;
      uint32_t gk = 0, gv = 0;  // key blocks / V halves issued so far, over all units
      Unit u;
      for (int it = 0; ok && unit_at<L::kTiles>(p, it, u); ++it) {
        const int b = u.bh / p.H, h = u.bh - b * p.H;
        // the Q pair is free once every Q K^T product of the previous unit is through
        if (it >= 1) ok = wait_warp(&q_empty, (it - 1) & 1, ctx, kSiteQEmpty, it);
        if (!ok) break;
        if (elect_one()) {
          mbar_expect_tx(&q_full, L::kTiles * L::kQTile);
          for (int t = 0; t < L::kTiles; ++t)
            for (int kb = 0; kb < KB; ++kb)
              tma_load_4d(smem + L::kQ + t * L::kQTile + kb * kBlk, &p.map_q, &q_full, kb * 64, h,
                          (u.mb0 + t) * 128, b);
        }
        __syncwarp();
        for (int j = 0; j < u.nmax && ok; ++j, ++gk) {
          const uint32_t ks = gk % KST;
          const int n0 = j * 128;
          if (gk >= KST) ok = wait_warp(&k_empty[ks], (gk / KST - 1) & 1, ctx, kSiteKEmpty, j);
          if (!ok) break;
          if (elect_one()) {
            mbar_expect_tx(&k_full[ks], L::kKStage);
            for (int kb = 0; kb < KB; ++kb)
              tma_load_4d(smem + L::kK + ks * L::kKStage + kb * kBlk, &p.map_k, &k_full[ks], kb * 64, h,
                          n0, b);
          }
          __syncwarp();
          for (int hf = 0; hf < 2 && ok; ++hf, ++gv) {
            const uint32_t vs = gv % VS, use = gv / VS;
            if (use >= 1) ok = wait_warp(&v_empty[vs], (use - 1) & 1, ctx, kSiteVEmpty, j);
            if (!ok) break;
            if (elect_one()) {
              mbar_expect_tx(&v_full[vs], L::kVHalf);
              for (int kb = 0; kb < KB; ++kb)
                tma_load_4d(smem + L::kV + vs * L::kVHalf + kb * kVBlk, &p.map_v, &v_full[vs], kb * 64, h,
                            n0 + hf * 64, b);
            }
            __syncwarp();
          }
        }
      }
    }
  } else if (warp == 9 || warp == 11) {
    // ------------------------------------------- MMA issuer of tile slot t (converged, an elected lane issues)
    // (the whole warp walks the loop converged, one elected lane issues)
    if (live) {
      const int t = warp == 9 ? 0 : 1;
      constexpr bool bf = P2::kIsBf16;
      constexpr uint32_t idesc_qk = make_idesc(bf, false, false, 128, 64);
      constexpr uint32_t idesc_pv = make_idesc(bf, false, true, 128, DP);
      const uint32_t q_addr = smem_u32(smem + L::kQ) + t * L::kQTile, k_addr = smem_u32(smem + L::kK);
      const uint32_t v_addr = smem_u32(smem + L::kV);
      const uint32_t tm_s = tmem + t * 128, tm_o = tmem + 256 + t * 128;
      bool ok = true;
      uint32_t cs = 0;          // steps done by this tile slot, over all units
      uint32_t gk = 0, gv = 0;  // key blocks / V halves consumed before this unit
      Unit u;
      // scores of one 64-key half of the block in ring stage `kslot` -> column half `ch`
      auto issue_qk = [&](uint32_t kslot, int keys, uint32_t ch) {
        if (elect_one()) {
          issue_gemm_ss<KS_QK, false, false>(tm_s + ch * 64, make_sdesc(q_addr, 0, 1024),
                                             make_sdesc(k_addr + kslot * L::kKStage + keys * (64 * 128), 0, 1024),
                                             kBlk, kBlk, idesc_qk, false);
          mma_commit(&s_full[t][keys]);
        }
        __syncwarp();
      };
      auto commit = [&](uint64_t* bar) {
        if (elect_one()) mma_commit(bar);
        __syncwarp();
      };
      for (int it = 0; ok && unit_at<L::kTiles>(p, it, u); ++it) {
        if (u.nmax == 0) continue;
        const int nblk = u.nb(t);
        ok = wait_warp(&q_full, it & 1, ctx, kSiteQFull, it);
        if (ok) ok = wait_warp(&k_full[gk % KST], (gk / KST) & 1, ctx, kSiteKFull, 0);
        if (!ok) break;
        tc_fence_after();
        if (nblk > 0) {
          issue_qk(gk % KST, 0, cs & 1);
          issue_qk(gk % KST, 1, (cs & 1) ^ 1);
        }
        commit(&k_empty[gk % KST]);
        if (u.nmax == 1) commit(&q_empty);
        for (int j = 0; j < u.nmax && ok; ++j) {
          const uint32_t kn = (gk + j + 1) % KST, kn_par = ((gk + j + 1) / KST) & 1;
          const bool more = j + 1 < u.nmax;  // the unit has a block j+1 (this tile may not visit it)
          const bool mine = j < nblk, mine_next = j + 1 < nblk;
          const uint32_t f = cs & 1;  // column half that holds keys 0-63 of this step, and P
          for (int h = 0; h < 2 && ok; ++h) {
            const uint32_t gh = gv + 2 * j + h;
            const uint32_t vs = gh % VS, v_par = (gh / VS) & 1;
            if (mine) {
              ok = wait_warp_hot(&p_full[t][h], cs & 1, ctx, kSitePFull, j);
              if (ok) ok = wait_warp(&v_full[vs], v_par, ctx, kSiteVFull, j);
              if (!ok) break;
              tc_fence_after();
              if (elect_one()) {
                issue_gemm_ts<4, true>(tm_o, tm_s + f * 64 + h * 32,
                                       make_sdesc(v_addr + vs * L::kVHalf, kVBlk, 1024), kVBlk, idesc_pv,
                                       j > 0 || h > 0);
                mma_commit(&pv_done[t][h]);
              }
              __syncwarp();
            } else {
              // a block only the other tile visits: keep the ring counters in step
              ok = wait_warp(&v_full[vs], v_par, ctx, kSiteVFull, j);
              if (!ok) break;
            }
            commit(&v_empty[vs]);
            if (h == 0) {
              // Keys 0-63 of block j+1 go into the column half whose scores (keys 64-127 of
              // block j) the row threads have just taken into registers: this product runs
              // under the second half of this step's softmax.
              if (mine) ok = wait_warp_hot(&s_read[t], cs & 1, ctx, kSiteSRead, j);
              if (ok && more) ok = wait_warp(&k_full[kn], kn_par, ctx, kSiteKFull, j + 1);
              if (!ok) break;
              if (mine_next) {
                tc_fence_after();
                issue_qk(kn, 0, f ^ 1);
              }
            } else {
              // Keys 64-127 of block j+1 go over the columns P of block j is read from: same
              // issuing thread, so it executes after the products just issued.
              if (mine_next) issue_qk(kn, 1, f);
              if (more) {
                commit(&k_empty[kn]);
                if (j + 2 >= u.nmax) commit(&q_empty);
              }
            }
          }
          if (mine) ++cs;
        }
        gk += u.nmax;
        gv += 2 * u.nmax;
      }
    }
    __syncwarp();
  } else if (warp == 10) {
    // ------------------------------------------------------------ bias producer
    // (whole warp converged, one elected lane issues)
    if (BIAS != 0 && live) {
      if (lane == 0) tma_prefetch_desc(&p.map_bias);
      const uint64_t pol_stream = policy_evict_first();
      BiasWalk<BIAS, L::kTiles> cur;
      cur.start(p);
      bool ok = true;
      for (uint32_t unit = 0; ok && cur.valid; ++unit) {
        const uint32_t bs = unit % NB, use = unit / NB;
        if (use >= 1) ok = wait_warp(&bias_empty[bs], (use - 1) & 1, ctx, kSiteBiasEmpty, cur.j);
        if (!ok) break;
        int n0, m0, hh, bb;
        cur.coords(p, n0, m0, hh, bb);
        // the "full" barrier of the group that will read this unit (see the softmax side)
        uint64_t* full = &bias_full[cur.t][bs];
        if (elect_one()) {
          mbar_expect_tx(full, kBlk);
          tma_load_4d_hint(smem + L::kBias + bs * kBlk, &p.map_bias, full, n0, m0, hh, bb, pol_stream);
        }
        __syncwarp();
        cur.next(p);
      }
    }
  } else {
    // ------------------------------------------------------------------- softmax
    const int t = warp >> 2;                 // tile slot of this group
    const int r = (warp & 3) * 32 + lane;    // query row inside the tile = tensor-memory lane
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32u;
    const uint32_t tm_s = tmem_addr(tmem, lane_base, t * 128);
    const uint32_t tm_o = tmem_addr(tmem, lane_base, 256 + t * 128);
    constexpr int kU = BIAS == 1 ? 2 : (BIAS == 3 ? 4 : 1);  // bias units per (tile, key block)
    constexpr int kUH = kU / 2;  // units per 64-key half (0: one unit serves both halves)
    bool ok = live;
    const bool fold_scale = p.sm_scale > 0.f;  // no-bias path: maximum taken on raw q.k
    const float scale_log2 = p.sm_scale * kLog2e;
    uint32_t cs = 0;  // steps done by this tile slot, over all units
    uint32_t bu = 0;  // bias units before the current key block, over all units and both tiles
    // The ring slots are shared by both groups, the "full" barriers are not: bias_full[t][slot]
    // completes once per unit of tile slot t that lands in that ring slot, so its only waiter
    // (this group) is never more than one completion behind and a parity wait is safe.  (With
    // one barrier per slot a group could ask for completion k+1 before completion k - the other
    // group's unit - had happened, which a parity wait cannot tell from "done".)  Bit s of
    // b_phase is the parity of this group's next unit in slot s.
    uint32_t b_phase = 0;
    Unit u;
    for (int it = 0; ok && unit_at<L::kTiles>(p, it, u); ++it) {
      const int nblk = u.nb(t);
      const int m0 = (u.mb0 + t) * 128;
      float m_used = -INFINITY;  // running maximum, log2 domain
      float l = 0.f;             // row sum
      for (int j = 0; j < u.nmax && ok; ++j) {
        const int both = (j < u.nb0 ? 1 : 0) + (j < u.nb1 ? 1 : 0);
        if (j < nblk) {
          const uint32_t first = bu + ((t == 1 && j < u.nb0) ? kU : 0);
          const uint32_t f = cs & 1;  // column half of keys 0-63 in this step (and of P)
#pragma unroll 1
          for (int h = 0; h < 2 && ok; ++h) {
            ok = wait_warp(&s_full[t][h], cs & 1, ctx, kSiteSFull, j);
            if (!ok) break;
            tc_fence_after();
            const uint32_t tm_sh = tm_s + ((static_cast<uint32_t>(h) ^ f) << 6);
            const uint32_t unit = first + h * kUH;
            uint32_t bs = unit % NB, b_par = (b_phase >> bs) & 1;
            uint32_t pbias = 1;
            if (BIAS != 0 && (BIAS != 2 || h == 0)) pbias = mbar_poll(&bias_full[t][bs], b_par);
            float s[64];
            tmem_ld32(tm_sh, reinterpret_cast<uint32_t*>(s));
            tmem_ld32(tm_sh + 32, reinterpret_cast<uint32_t*>(s) + 32);
            tmem_ld_wait();
            if (h == 1) {
              // these columns are free: the first half of the next block's scores may land there
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&s_read[t]);
            }
            const int n0 = j * 128 + h * 64;  // first key of this half
            // ---- score in the natural domain: q.k * sm_scale (+ bias), -inf where masked.
            // Without a bias (and a positive scale) the raw q.k is kept and the scale is
            // folded into the exponent below.
            float mul = kLog2e;  // exponent = s * mul - m
            if (BIAS == 0) {
              if (fold_scale) {
                mul = scale_log2;
              } else {
#pragma unroll
                for (int i = 0; i < 64; ++i) s[i] *= p.sm_scale;
              }
            } else {
              if (BIAS != 2 || h == 0) {
                ok = wait_warp_polled(pbias, &bias_full[t][bs], b_par, ctx, kSiteBiasFull, j);
                if (!ok) break;
              }
              const uint32_t row = smem_u32(smem + L::kBias + bs * kBlk) + static_cast<uint32_t>(r) * 128u;
              if (BIAS == 3) {
                // fp32 bias: two [128 rows][32 keys] units per half, four floats per 16-byte chunk
                const f32x2 sc2 = f2(p.sm_scale, p.sm_scale);
#pragma unroll
                for (int sub = 0; sub < 2; ++sub) {
                  if (sub == 1) {
                    bs = (unit + 1) % NB;
                    b_par = (b_phase >> bs) & 1;
                    ok = wait_warp(&bias_full[t][bs], b_par, ctx, kSiteBiasFull, j);
                    if (!ok) break;
                  }
                  const uint32_t row3 = smem_u32(smem + L::kBias + bs * kBlk) + static_cast<uint32_t>(r) * 128u;
#pragma unroll
                  for (int c = 0; c < 8; ++c) {
                    const uint4 v = lds128(row3 + (static_cast<uint32_t>(c ^ (r & 7)) << 4));
                    const int i = sub * 32 + c * 4;
                    const f32x2 x0 = ffma2(f2(s[i], s[i + 1]), sc2, f2(__uint_as_float(v.x), __uint_as_float(v.y)));
                    const f32x2 x1 = ffma2(f2(s[i + 2], s[i + 3]), sc2, f2(__uint_as_float(v.z), __uint_as_float(v.w)));
                    s[i] = f2_lo(x0);
                    s[i + 1] = f2_hi(x0);
                    s[i + 2] = f2_lo(x1);
                    s[i + 3] = f2_hi(x1);
                  }
                  b_phase ^= 1u << bs;
                  __syncwarp();
                  if (lane == 0) mbar_arrive(&bias_empty[bs]);
                }
                if (!ok) break;
              } else if (BIAS == 1) {
                const f32x2 sc2 = f2(p.sm_scale, p.sm_scale);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                  const uint4 v = lds128(row + (static_cast<uint32_t>(c ^ (r & 7)) << 4));
                  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    const float2 f = P2::unpack(w[e]);
                    const int i = c * 8 + e * 2;
                    const f32x2 x = ffma2(f2(s[i], s[i + 1]), sc2, f2(f.x, f.y));
                    s[i] = f2_lo(x);
                    s[i + 1] = f2_hi(x);
                  }
                }
              } else {
                // byte mask unit: [128 rows][128 bytes]; this half reads chunks 4h .. 4h+3
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                  const uint4 v = lds128(row + (static_cast<uint32_t>((h * 4 + c) ^ (r & 7)) << 4));
                  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                      const int i = c * 16 + e * 4 + k;
                      const bool keep = ((w[e] >> (8 * k)) & 0xFFu) != 0;
                      s[i] = keep ? s[i] * p.sm_scale : -INFINITY;
                    }
                  }
                }
              }
              if (BIAS == 1 || (BIAS == 2 && h == 1)) {
                b_phase ^= 1u << bs;
                __syncwarp();
                if (lane == 0) mbar_arrive(&bias_empty[bs]);
              }
            }
            // ---- bounds and causal masks (only on halves that need them)
            if ((n0 + 64 > p.N) || (p.causal && n0 + 63 > m0)) {
              int limit = p.N - n0;
              if (p.causal) limit = min(limit, m0 + r - n0 + 1);
#pragma unroll
              for (int i = 0; i < 64; ++i)
                if (i >= limit) s[i] = -INFINITY;
            }
            // ---- row maximum of this half
            float mx0 = max3(s[0], s[1], s[2]), mx1 = max3(s[3], s[4], s[5]);
            float mx2 = max3(s[6], s[7], s[8]), mx3 = max3(s[9], s[10], s[11]);
#pragma unroll
            for (int i = 12; i + 7 < 64; i += 8) {
              mx0 = max3(mx0, s[i], s[i + 1]);
              mx1 = max3(mx1, s[i + 2], s[i + 3]);
              mx2 = max3(mx2, s[i + 4], s[i + 5]);
              mx3 = max3(mx3, s[i + 6], s[i + 7]);
            }
            mx0 = max3(mx0, s[60], s[61]);  // 12 + 6*8 = 60 consumed; 60..63 left
            mx1 = max3(mx1, s[62], s[63]);
            const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * mul;  // log2 domain
            const bool need = mx > m_used + 8.0f;
            if (__any_sync(0xffffffffu, need)) {
              const float m_new = need ? mx : m_used;
              const float alpha = need ? ex2(m_used - m_new) : 1.0f;
              l *= alpha;
              m_used = m_new;
              if (j > 0 || h > 0) {
                // O may only be touched once every product into it has finished: the last one
                // issued is P V of the previous half
                ok = h == 1 ? wait_warp(&pv_done[t][0], cs & 1, ctx, kSitePvDone, j)
                            : wait_warp(&pv_done[t][1], (cs - 1) & 1, ctx, kSitePvDone, j);
                if (!ok) break;
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < DP / 32; ++c) {
                  uint32_t o[32];
                  tmem_ld32(tm_o + c * 32, o);
                  tmem_ld_wait();
#pragma unroll
                  for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                  tmem_st32(tm_o + c * 32, o);
                }
              }
            }
            const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
            f32x2 sum01 = f2(0.f, 0.f), sum23 = f2(0.f, 0.f);
            const f32x2 mul2 = f2(mul, mul), negm2 = f2(neg_m, neg_m);
            uint32_t pk[32];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const f32x2 a01 = ffma2(f2(s[2 * i], s[2 * i + 1]), mul2, negm2);
              const f32x2 a23 = ffma2(f2(s[2 * i + 2], s[2 * i + 3]), mul2, negm2);
              // All exponentials on the special-function unit: a polynomial evaluated on the FMA
              // pipe for part of them only adds instructions, and the row warps' time follows
              // their instruction count (measured 2-4 % slower with an eighth to a quarter moved).
              const float p0 = ex2(f2_lo(a01)), p1 = ex2(f2_hi(a01));
              const float p2 = ex2(f2_lo(a23)), p3 = ex2(f2_hi(a23));
              sum01 = fadd2(sum01, f2(p0, p1));
              sum23 = fadd2(sum23, f2(p2, p3));
              pk[i] = P2::pack(p0, p1);
              pk[i + 1] = P2::pack(p2, p3);
            }
            l += (f2_lo(sum01) + f2_hi(sum01)) + (f2_lo(sum23) + f2_hi(sum23));
            // P (16 bit) over the score columns of keys 0-63, which this thread has read
            tmem_st32(tm_s + f * 64 + h * 32, pk);
            tmem_st_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[t][h]);
          }
          if (!ok) break;
          ++cs;
        }
        bu += both * kU;
      }
      if (!ok) break;
      if (nblk == 0) continue;
      // ---- epilogue: O / l -> global, log-sum-exp
      ok = wait_warp(&pv_done[t][1], (cs - 1) & 1, ctx, kSiteEpilogue, nblk);
      if (!ok) break;
      tc_fence_after();
      const int m = m0 + r;
      const int b = u.bh / p.H, hd = u.bh - b * p.H;
      // a row whose keys are all masked out keeps m_used = -inf and l = 0: output 0, LSE +inf
      const bool any_key = m_used != -INFINITY && l > 0.f;
      const float inv = any_key ? 1.0f / l : 0.f;
      T* orow = reinterpret_cast<T*>(p.o) + b * p.o_sB + static_cast<int64_t>(m) * p.o_sM + hd * p.o_sH;
#pragma unroll
      for (int c = 0; c < DP / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(tm_o + c * 32, o);
        tmem_ld_wait();
        if (m < p.M) {
          if (p.o_vec32 && c * 32 + 32 <= p.D) {
            // whole 32-byte sectors per store: half as many transactions as 16-byte stores for
            // these row-strided writes
#pragma unroll
            for (int q2 = 0; q2 < 2; ++q2) {
              const uint4 lo = pack8<P2>(o + q2 * 16, inv), hi = pack8<P2>(o + q2 * 16 + 8, inv);
              asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(orow + c * 32 + q2 * 16),
                           "r"(lo.x), "r"(lo.y), "r"(lo.z), "r"(lo.w), "r"(hi.x), "r"(hi.y), "r"(hi.z), "r"(hi.w)
                           : "memory");
            }
          } else {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              const int d = c * 32 + q4 * 8;
              if (d < p.D) *reinterpret_cast<uint4*>(orow + d) = pack8<P2>(o + q4 * 8, inv);
            }
          }
        }
      }
      // O is in registers / stored: the next unit's first P V product may overwrite it (it is
      // issued after all four warps have announced that unit's first P)
      tc_fence_before();
      if (m < p.M) p.lse[static_cast<int64_t>(u.bh) * p.M + m] = any_key ? m_used + log2f(l) : INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tmem, kTmemCols);
}

template <int DP, typename T, int BIAS>
int launch_inst(const FwdParams& fp, dim3 grid, cudaStream_t stream) {
  using L = FwdSmem<DP, BIAS>;
  auto kern = fwd_kernel<DP, T, BIAS>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kDynamic) !=
        cudaSuccess)
      return FA_ERR_CUDA;
    configured[dev] = true;
  }
  return launch_overlapped(kern, grid, 384, L::kDynamic, stream, fp);
}

template <int DP, typename T>
int launch_bias(const FwdParams& fp, int bias_kind, dim3 grid, cudaStream_t stream) {
  switch (bias_kind) {
    case FA_BIAS_NONE: return launch_inst<DP, T, 0>(fp, grid, stream);
    case FA_BIAS_SAME: return launch_inst<DP, T, 1>(fp, grid, stream);
    case FA_BIAS_BOOL: return launch_inst<DP, T, 2>(fp, grid, stream);
    case FA_BIAS_F32: return launch_inst<DP, T, 3>(fp, grid, stream);
    default: return FA_ERR_UNSUPPORTED;
  }
}

}  // namespace

int launch_fwd(const fa_params& p, cudaStream_t stream, int* status) {
  FwdParams fp;
  int r = make_tmap_bshd(&fp.map_q, p.q, p.B, p.M, p.H, p.D, p.q_stride, 128);
  if (r) return r;
  r = make_tmap_bshd(&fp.map_k, p.k, p.B, p.N, p.H, p.D, p.k_stride, 128);
  if (r) return r;
  r = make_tmap_bshd(&fp.map_v, p.v, p.B, p.N, p.H, p.D, p.v_stride, 64);
  if (r) return r;
  fp.bias_b_mul = fp.bias_h_mul = 0;
  if (p.bias_kind == FA_BIAS_SAME) {
    r = make_tmap_bhmn(&fp.map_bias, p.bias, 2, p.B, p.H, p.M, p.N, p.bias_stride, 64, 128,
                       &fp.bias_b_mul, &fp.bias_h_mul);
    if (r) return r;
  } else if (p.bias_kind == FA_BIAS_BOOL) {
    r = make_tmap_bhmn(&fp.map_bias, p.bias, 1, p.B, p.H, p.M, p.N, p.bias_stride, 128, 128,
                       &fp.bias_b_mul, &fp.bias_h_mul);
    if (r) return r;
  } else if (p.bias_kind == FA_BIAS_F32) {
    r = make_tmap_bhmn(&fp.map_bias, p.bias, 4, p.B, p.H, p.M, p.N, p.bias_stride, 32, 128,
                       &fp.bias_b_mul, &fp.bias_h_mul);
    if (r) return r;
  } else {
    fp.map_bias = fp.map_q;
  }
  if (reinterpret_cast<uintptr_t>(p.o) % 16 != 0 || p.o_stride[0] % 8 || p.o_stride[1] % 8 ||
      p.o_stride[2] % 8)
    return FA_ERR_ALIGN;
  fp.o = p.o;
  fp.o_vec32 = reinterpret_cast<uintptr_t>(p.o) % 32 == 0 && p.o_stride[0] % 16 == 0 && p.o_stride[1] % 16 == 0 &&
               p.o_stride[2] % 16 == 0;
  fp.lse = p.lse;
  fp.status = status;
  fp.o_sB = p.o_stride[0];
  fp.o_sM = p.o_stride[1];
  fp.o_sH = p.o_stride[2];
  fp.H = p.H;
  fp.M = p.M;
  fp.N = p.N;
  fp.D = p.D;
  fp.causal = p.causal ? 1 : 0;
  fp.sm_scale = p.sm_scale;
  fp.n_mblk = (p.M + 127) / 128;
  const int dp = padded_head_dim(p.D);
  const int tiles = dp == 256 ? 1 : 2;  // query tiles per unit (FwdSmem::kTiles)
  fp.n_pairs = (fp.n_mblk + tiles - 1) / tiles;
  fp.n_units = fp.n_pairs * p.B * p.H;
  const dim3 grid(persistent_grid(p.causal ? (fp.n_units + 1) / 2 : fp.n_units));
  if (p.dtype == FA_BF16) {
    return dp == 64    ? launch_bias<64, __nv_bfloat16>(fp, p.bias_kind, grid, stream)
           : dp == 128 ? launch_bias<128, __nv_bfloat16>(fp, p.bias_kind, grid, stream)
                       : launch_bias<256, __nv_bfloat16>(fp, p.bias_kind, grid, stream);
  }
  return dp == 64    ? launch_bias<64, __half>(fp, p.bias_kind, grid, stream)
         : dp == 128 ? launch_bias<128, __half>(fp, p.bias_kind, grid, stream)
                     : launch_bias<256, __half>(fp, p.bias_kind, grid, stream);
}

}  // namespace fa
