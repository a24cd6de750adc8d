// Forward attention kernel for sm_100a.
//
// Persistent kernel, one CTA per SM.  A tile is 128 query rows of one (batch,
// head); a CTA walks its tiles one after the other and, inside a tile, the key
// blocks of 128 keys.  Ring stages, tensor-memory buffers and barrier phases run on
// from tile to tile, so the next tile's Q / K / V / bias loads and its first
// Q K^T product overlap the current tile's epilogue.  Roles (640 threads):
//   warps 0-15 softmax: warp w owns query rows 32*(w&3)..+31 (= tensor-memory
//              lanes) and the 32-key quarter (w>>2) of every block; the four
//              quarters of a row exchange partial maxima through shared memory
//   warp 16    TMA producer (one elected lane): Q per tile, K / V rings
//   warp 17    MMA issuer for S = Q K^T (one lane), tensor-memory owner
//   warp 18    MMA issuer for O += P V (one lane)
//   warp 19    TMA producer of the bias / mask ring (one lane)
// A barrier operation answers after ~200 cycles on this GPU; two issuers keep the
// tensor pipe fed while one of them waits, and barriers are polled ahead of use.
// Per key block j:  S_j = Q K_j^T (both operands in shared memory, accumulator
// in tensor memory, double buffered) -> softmax threads read S_j, add the bias
// tile (streamed by TMA into a shared-memory ring), apply masks, run the online
// softmax in the log2 domain and write P_j (16 bit) back into tensor memory over
// S_j -> O += P_j V_j with P as the tensor-memory operand and V MN-major in
// shared memory.  S_{j+1} is issued before P_j V_j so the tensor core works
// while the softmax of block j runs.  The running maximum is only raised when
// it grows by more than 8 (log2 units); O in tensor memory is rescaled only
// then.
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
  CUtensorMap map_v;
  CUtensorMap map_bias;
  void* o;
  float* lse;
  int* status;
  int64_t o_sB, o_sM, o_sH;
  int H, M, N, D;
  int causal;
  int bias_b_mul, bias_h_mul;
  int n_mblk, n_tiles;  // query blocks per (batch, head); tiles = n_mblk * B * H
  float sm_scale;
};

enum FwdSite { kSiteQ = 1, kSiteKFull, kSiteKEmpty, kSiteVFull, kSiteVEmpty, kSiteSFull,
               kSitePFull, kSitePvDone, kSiteBiasFull, kSiteBiasEmpty, kSiteEpilogue, kSitePair, kSiteQEmpty, kSitePvDoneQK };

template <int DP, int BIAS>
struct FwdSmem {
  static constexpr int kTile = 128 * DP * 2;
  // 16 KB bias units (one 64-key column half each); 3 at D=128 to stay inside 227 KB
  static constexpr int kBiasStages = BIAS == 0 ? 0 : (DP == 128 ? 3 : 4);
  static constexpr int kQ = 0;
  static constexpr int kK = kQ + kTile;
  static constexpr int kV = kK + 2 * kTile;
  static constexpr int kBias = kV + 2 * kTile;
  static constexpr int kTotal = kBias + kBiasStages * kBlk;
  static constexpr int kDynamic = kTotal + 1024;  // slack for 1024-byte alignment
};

template <int DP, typename T, int BIAS>
__global__ void __launch_bounds__(640, 1) fwd_kernel(const __grid_constant__ FwdParams p) {
  using L = FwdSmem<DP, BIAS>;
  using P2 = Pack2<T>;
  constexpr int KB = DP / 64;    // 64-column blocks per Q/K/V tile
  constexpr int KS_QK = DP / 16; // MMA K slices of Q K^T
  constexpr int kQD = DP / 4;    // output columns handled by one softmax thread (16 or 32)
  constexpr uint32_t NB = L::kBiasStages > 0 ? L::kBiasStages : 1;
  constexpr uint32_t kColS = 0, kColO = 256;
  constexpr uint32_t kTmemCols = 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t q_full, q_empty, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2],
      p_full, pv_done[2];
  __shared__ uint64_t bias_full[4], bias_empty[4], row_bars[4];
  __shared__ float xchg[2][4][128];  // [step parity][key quarter][row]: partial row maxima / sums
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int lane = tid & 31;
  // Persistent CTA: it walks tiles (tile = 128 query rows of one (batch, head)) and all
  // roles keep running counters, so the rings, the tensor-memory buffers and every barrier
  // phase carry on from one tile to the next: the loads and the first products of the next
  // tile overlap the epilogue of the current one.
  // Schedule: tiles are numbered (batch*head)-major; CTA c takes units c, c+G, c+2G, ...
  // so that the CTAs running at the same time work on neighbouring tiles and share K / V in
  // L2.  A unit is one tile, or - causal - two consecutive entries of the per-(batch, head)
  // order [last, first, last-1, first+1, ...]: a heavy and a light block, so every unit
  // carries about the same number of key blocks.
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

  WaitCtx ctx{&abort_flag, p.status, 1};

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&q_full, 1);
    mbar_init(&q_empty, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
    }
    mbar_init(&p_full, 16);
    mbar_init(&pv_done[0], 1);
    mbar_init(&pv_done[1], 1);
    for (int i = 0; i < 4; ++i) {
      mbar_init(&bias_full[i], 1);
      mbar_init(&bias_empty[i], BIAS == 2 ? 16 : 8);
      mbar_init(&row_bars[i], 4);
    }
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
  // A kernel launched after an earlier one recorded an error does no work.
  grid_dep_launch_next();
  grid_dep_wait();  // the previous kernel's results (and its status word) are visible from here
  const bool live = *reinterpret_cast<volatile int*>(p.status) == 0;

  if (warp == 16) {
    // ------------------------------------------------------------------ producer
    if (lane == 0 && live) {
      tma_prefetch_desc(&p.map_q);
      tma_prefetch_desc(&p.map_k);
      tma_prefetch_desc(&p.map_v);
      bool ok = true;
      uint32_t gj = 0;  // key blocks issued so far, over all tiles
      int bh, m_block, nblk;
      for (int it = 0; ok && tile_at(it, bh, m_block, nblk); ++it) {
        const int b = bh / p.H, h = bh - b * p.H, m0 = m_block * 128;
        // the single Q tile is free once every Q K^T product of the previous tile is through
        if (it >= 1) ok = mbar_wait(&q_empty, (it - 1) & 1, ctx, kSiteQEmpty, it);
        if (!ok) break;
        mbar_expect_tx(&q_full, L::kTile);
        for (int kb = 0; kb < KB; ++kb)
          tma_load_4d(smem + L::kQ + kb * kBlk, &p.map_q, &q_full, kb * 64, h, m0, b);
        for (int j = 0; j < nblk && ok; ++j) {
          const uint32_t g = gj + j;
          const int st = g & 1;
          const int n0 = j * 128;
          if (g >= 2) ok = mbar_wait(&k_empty[st], ((g >> 1) - 1) & 1, ctx, kSiteKEmpty, j);
          if (!ok) break;
          mbar_expect_tx(&k_full[st], L::kTile);
          for (int kb = 0; kb < KB; ++kb)
            tma_load_4d(smem + L::kK + st * L::kTile + kb * kBlk, &p.map_k, &k_full[st], kb * 64,
                        h, n0, b);
          if (g >= 2) ok = mbar_wait(&v_empty[st], ((g >> 1) - 1) & 1, ctx, kSiteVEmpty, j);
          if (!ok) break;
          mbar_expect_tx(&v_full[st], L::kTile);
          for (int kb = 0; kb < KB; ++kb)
            tma_load_4d(smem + L::kV + st * L::kTile + kb * kBlk, &p.map_v, &v_full[st], kb * 64,
                        h, n0, b);
        }
        gj += nblk;
      }
    }
  } else if (warp == 17) {
    // ------------------------------------------------------- MMA issuer: S = Q K^T
    if (lane == 0 && live) {
      constexpr bool bf = P2::kIsBf16;
      constexpr uint32_t idesc_qk = make_idesc(bf, false, false, 128, 128);
      const uint32_t q_addr = smem_u32(smem + L::kQ);
      const uint32_t k_addr = smem_u32(smem + L::kK);
      const uint64_t q_desc = make_sdesc(q_addr, 0, 1024);
      const uint64_t k_desc_0 = make_sdesc(k_addr, 0, 1024), k_desc_1 = make_sdesc(k_addr + L::kTile, 0, 1024);
      bool ok = true;
      uint32_t gj = 0;
      int bh, m_block, nblk;
      for (int it = 0; ok && tile_at(it, bh, m_block, nblk); ++it) {
        for (int j = 0; j < nblk && ok; ++j) {
          const uint32_t g = gj + j;
          const int st = g & 1;
          const uint32_t pk = mbar_poll(&k_full[st], (g >> 1) & 1);
          // S_g overwrites the columns that held P_{g-2}: P_{g-2} V_{g-2} must be through.
          // One barrier per S buffer: its next completion (P_g V_g) needs this very S_g, so
          // the barrier can never run two phases ahead of this wait, however long the issuer
          // sat in another wait (a new tile's Q) in between.
          if (g >= 2)
            ok = mbar_wait_hot(&pv_done[st], ((g >> 1) - 1) & 1, ctx, kSitePvDoneQK, j);
          if (ok && j == 0) ok = mbar_wait(&q_full, it & 1, ctx, kSiteQ, it);
          if (ok) ok = wait_polled(pk, &k_full[st], (g >> 1) & 1, ctx, kSiteKFull, j);
          if (!ok) break;
          tc_fence_after();
          issue_gemm_ss<KS_QK, false, false>(tmem + kColS + st * 128, q_desc,
                                             st ? k_desc_1 : k_desc_0, kBlk, kBlk, idesc_qk, false);
          mma_commit(&s_full[st]);
          mma_commit(&k_empty[st]);
          if (j == nblk - 1) mma_commit(&q_empty);
        }
        gj += nblk;
      }
    }
    __syncwarp();
  } else if (warp == 18) {
    // ------------------------------------------------------- MMA issuer: O += P V
    if (lane == 0 && live) {
      constexpr bool bf = P2::kIsBf16;
      constexpr uint32_t idesc_pv = make_idesc(bf, false, true, 128, DP);
      const uint32_t v_addr = smem_u32(smem + L::kV);
      const uint64_t v_desc_0 = make_sdesc(v_addr, kBlk, 1024), v_desc_1 = make_sdesc(v_addr + L::kTile, kBlk, 1024);
      bool ok = true;
      uint32_t gj = 0;
      int bh, m_block, nblk;
      for (int it = 0; ok && tile_at(it, bh, m_block, nblk); ++it) {
        for (int j = 0; j < nblk && ok; ++j) {
          const uint32_t g = gj + j;
          const int st = g & 1;
          const uint32_t pv = mbar_poll(&v_full[st], (g >> 1) & 1);
          // P_g of a new tile is only announced after all sixteen softmax warps have read
          // the previous tile's O, so the first product of a tile may overwrite it
          ok = mbar_wait_hot(&p_full, g & 1, ctx, kSitePFull, j);
          if (ok) ok = wait_polled(pv, &v_full[st], (g >> 1) & 1, ctx, kSiteVFull, j);
          if (!ok) break;
          tc_fence_after();
          issue_gemm_ts<8, true>(tmem + kColO, tmem + kColS + st * 128, st ? v_desc_1 : v_desc_0,
                                 kBlk, idesc_pv, j > 0);
          mma_commit(&v_empty[st]);
          mma_commit(&pv_done[st]);
        }
        gj += nblk;
      }
    }
    __syncwarp();
  } else if (warp == 19) {
    // ------------------------------------------------------------ bias producer
    // Its own thread: the bias ring is the HBM-latency-critical stream and must not
    // queue behind the K / V ring's waits.
    if (BIAS != 0 && lane == 0 && live) {
      tma_prefetch_desc(&p.map_bias);
      const uint64_t pol_stream = policy_evict_first();
      uint32_t unit = 0;
      bool ok = true;
      int bh, m_block, nblk;
      for (int it = 0; ok && tile_at(it, bh, m_block, nblk); ++it) {
        const int b = bh / p.H, h = bh - b * p.H, m0 = m_block * 128;
        for (int j = 0; j < nblk && ok; ++j) {
          const int n0 = j * 128;
          // 16 KB units: 16-bit bias -> one per 64-key column half ([128 rows][64 keys]);
          // byte mask -> one per block ([128 rows][128 keys]) shared by both halves
          constexpr int kUnits = BIAS == 1 ? 2 : 1;
          for (int u = 0; u < kUnits && ok; ++u, ++unit) {
            const int bs = unit % NB;
            const uint32_t use = unit / NB;
            if (use >= 1) ok = mbar_wait(&bias_empty[bs], (use - 1) & 1, ctx, kSiteBiasEmpty, j);
            if (!ok) break;
            mbar_expect_tx(&bias_full[bs], kBlk);
            tma_load_4d_hint(smem + L::kBias + bs * kBlk, &p.map_bias, &bias_full[bs],
                             n0 + u * 64, m0, h * p.bias_h_mul, b * p.bias_b_mul, pol_stream);
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------- softmax
    // thread = (query row r, key quarter qt): 32 of the 128 scores of the row per block
    const int r = (warp & 3) * 32 + lane;
    const int qt = warp >> 2;
    const uint32_t lane_base = static_cast<uint32_t>(warp & 3) * 32u;
    uint64_t* row_bar = &row_bars[warp & 3];  // shared by the four warps that own the same rows
    bool ok = live;
    const bool fold_scale = p.sm_scale > 0.f;  // no-bias path: maximum taken on raw q.k
    const float scale_log2 = p.sm_scale * kLog2e;
    uint32_t gj = 0;  // key blocks done so far, over all tiles (ring stages and barrier phases)
    int bh, m_block, nblk;
    for (int it = 0; ok && tile_at(it, bh, m_block, nblk); ++it) {
    const int m0 = m_block * 128;
    float m_used = -INFINITY;  // running maximum, log2 domain
    float l = 0.f;             // partial row sum over this thread's keys
    for (int j = 0; j < nblk && ok; ++j) {
      const uint32_t g = gj + j;
      const int st = g & 1;
      const uint32_t gx = g + it;  // quarter exchanges so far: one per block, one per tile
      // bias unit of this step: 16-bit bias -> two per block (this quarter's half); mask -> one
      const uint32_t unit = BIAS == 1 ? 2 * g + (qt >> 1) : g;
      const int n0 = j * 128 + qt * 32;  // first key of this thread's quarter
      // the scores and the bias unit of this step are usually there already: one combined
      // look at both barriers (their answers travel together), blocking waits only if not
      uint32_t ps = 1, pbias = 1;
      if (BIAS != 0)
        mbar_poll2(&s_full[st], (g >> 1) & 1, &bias_full[unit % NB], (unit / NB) & 1, ps, pbias);
      else
        ps = mbar_poll(&s_full[st], (g >> 1) & 1);
      ok = wait_warp_polled(ps, &s_full[st], (g >> 1) & 1, ctx, kSiteSFull, j);
      if (!ok) break;
      tc_fence_after();
      float s[32];
      tmem_ld32(tmem_addr(tmem, lane_base, kColS + st * 128 + qt * 32), reinterpret_cast<uint32_t*>(s));
      tmem_ld_wait();
      // ---- score in the natural domain: q.k * sm_scale (+ bias), -inf where masked.
      // Without a bias (and a positive scale) the raw q.k is kept and the scale is
      // folded into the exponent below.
      float mul = kLog2e;  // exponent = s * mul - m
      if (BIAS == 0) {
        if (fold_scale) {
          mul = scale_log2;
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) s[i] *= p.sm_scale;
        }
      } else {
        const int bs = unit % NB;
        ok = wait_warp_polled(pbias, &bias_full[bs], (unit / NB) & 1, ctx, kSiteBiasFull, j);
        if (!ok) break;
        const uint8_t* tile = smem + L::kBias + bs * kBlk;
        if (BIAS == 1) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const uint4 v = *reinterpret_cast<const uint4*>(tile + swz_off(r, (qt & 1) * 4 + c));
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 f = P2::unpack(w[e]);
              const int i = c * 8 + e * 2;
              const f32x2 t = ffma2(f2(s[i], s[i + 1]), f2(p.sm_scale, p.sm_scale), f2(f.x, f.y));
              s[i] = f2_lo(t);
              s[i + 1] = f2_hi(t);
            }
          }
        } else {
          // byte mask tile: [128 rows][128 bytes]; this quarter reads chunks 2*qt, 2*qt+1
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const uint4 v = *reinterpret_cast<const uint4*>(tile + swz_off(r, qt * 2 + c));
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
        __syncwarp();
        if (lane == 0) mbar_arrive(&bias_empty[bs]);
      }
      // ---- bounds and causal masks (only on blocks that need them)
      if ((n0 + 32 > p.N) || (p.causal && n0 + 31 > m0)) {
        int limit = p.N - n0;
        if (p.causal) limit = min(limit, m0 + r - n0 + 1);
#pragma unroll
        for (int i = 0; i < 32; ++i)
          if (i >= limit) s[i] = -INFINITY;
      }
      // ---- row maximum over this quarter, exchanged with the three partner quarters
      float mx0 = max3(s[0], s[1], s[2]), mx1 = max3(s[3], s[4], s[5]);
      float mx2 = max3(s[6], s[7], s[8]), mx3 = max3(s[9], s[10], s[11]);
#pragma unroll
      for (int i = 12; i + 7 < 32; i += 8) {
        mx0 = max3(mx0, s[i], s[i + 1]);
        mx1 = max3(mx1, s[i + 2], s[i + 3]);
        mx2 = max3(mx2, s[i + 4], s[i + 5]);
        mx3 = max3(mx3, s[i + 6], s[i + 7]);
      }
      mx0 = max3(mx0, s[28], s[29]);  // 12 + 2*8 = 28 consumed; 28..31 left
      mx1 = max3(mx1, s[30], s[31]);
      float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      xchg[gx & 1][qt][r] = mx;
      __syncwarp();
      if (lane == 0) mbar_arrive(row_bar);
      // the exchange barrier and "P_{j-1} V_{j-1} is through" are looked at together
      uint32_t prow = 0, ppv = 1;
      if (j > 0)
        mbar_poll2(row_bar, gx & 1, &pv_done[st ^ 1], ((g - 1) >> 1) & 1, prow, ppv);
      else
        prow = mbar_poll(row_bar, gx & 1);
      ok = wait_warp_polled(prow, row_bar, gx & 1, ctx, kSitePair, j);
      if (!ok) break;
      mx = fmaxf(fmaxf(xchg[gx & 1][0][r], xchg[gx & 1][1][r]),
                 fmaxf(xchg[gx & 1][2][r], xchg[gx & 1][3][r])) * mul;  // block maximum, log2 domain
      const bool need = mx > m_used + 8.0f;
      const bool any_need = __any_sync(0xffffffffu, need);
      // O may only be touched once P_{j-1} V_{j-1} has completed.
      if (j > 0) {
        ok = wait_warp_polled(ppv, &pv_done[st ^ 1], ((g - 1) >> 1) & 1, ctx, kSitePvDone, j);
        if (!ok) break;
      }
      if (any_need) {
        const float m_new = need ? mx : m_used;
        const float alpha = need ? ex2(m_used - m_new) : 1.0f;
        l *= alpha;
        m_used = m_new;
        if (j > 0) {
          tc_fence_after();
          uint32_t o[kQD];
          tmem_ld_cols<kQD>(tmem_addr(tmem, lane_base, kColO + qt * kQD), o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < kQD; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_cols<kQD>(tmem_addr(tmem, lane_base, kColO + qt * kQD), o);
        }
      }
      const float neg_m = (m_used == -INFINITY) ? 0.f : -m_used;
      f32x2 sum01 = f2(0.f, 0.f), sum23 = f2(0.f, 0.f);
      const f32x2 mul2 = f2(mul, mul), negm2 = f2(neg_m, neg_m);
      uint32_t pk[16];
#pragma unroll
      for (int i = 0; i < 16; i += 2) {
        const f32x2 a01 = ffma2(f2(s[2 * i], s[2 * i + 1]), mul2, negm2);
        const f32x2 a23 = ffma2(f2(s[2 * i + 2], s[2 * i + 3]), mul2, negm2);
        // a quarter of the exponentials on the FMA pipe, the rest on the special-function unit
        const float p0 = ex2(f2_lo(a01)), p1 = ex2(f2_hi(a01));
        float p2, p3;
        if ((i & 2) != 0) {
          const f32x2 e23 = ex2_poly2(a23);
          p2 = f2_lo(e23);
          p3 = f2_hi(e23);
        } else {
          p2 = ex2(f2_lo(a23));
          p3 = ex2(f2_hi(a23));
        }
        sum01 = fadd2(sum01, f2(p0, p1));
        sum23 = fadd2(sum23, f2(p2, p3));
        pk[i] = P2::pack(p0, p1);
        pk[i + 1] = P2::pack(p2, p3);
      }
      l += (f2_lo(sum01) + f2_hi(sum01)) + (f2_lo(sum23) + f2_hi(sum23));
      // P (16 bit) over the S columns: this quarter's 32 keys -> 16 packed columns
      tmem_st16(tmem_addr(tmem, lane_base, kColS + st * 128 + qt * 16), pk);
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full);
    }
    // ---- epilogue: O / l -> global, log-sum-exp
    if (!ok) break;
    gj += nblk;
    ok = wait_warp(&pv_done[(gj - 1) & 1], ((gj - 1) >> 1) & 1, ctx, kSiteEpilogue, nblk);
    // full row sum = sum of the four quarters
    const uint32_t gx = gj + it;
    if (ok) {
      xchg[gx & 1][qt][r] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(row_bar);
      ok = wait_warp(row_bar, gx & 1, ctx, kSitePair, nblk);
    }
    if (ok) {
      l = (xchg[gx & 1][0][r] + xchg[gx & 1][1][r]) + (xchg[gx & 1][2][r] + xchg[gx & 1][3][r]);
      tc_fence_after();
      const int m = m0 + r;
      const int b = bh / p.H, h = bh - b * p.H;
      // a row whose keys are all masked out keeps m_used = -inf: output 0, LSE +inf (its
      // polynomial exponentials are 1e-38, not 0, so l alone does not tell)
      const bool any_key = m_used != -INFINITY && l > 0.f;
      const float inv = any_key ? 1.0f / l : 0.f;
      T* orow = reinterpret_cast<T*>(p.o) + b * p.o_sB + static_cast<int64_t>(m) * p.o_sM +
                h * p.o_sH;
      uint32_t o[kQD];
      tmem_ld_cols<kQD>(tmem_addr(tmem, lane_base, kColO + qt * kQD), o);
      tmem_ld_wait();
      // O is in registers: the next tile's first P V product may overwrite it (it is issued
      // after all sixteen warps have announced that tile's first P)
      tc_fence_before();
      if (m < p.M) {
#pragma unroll
        for (int c = 0; c < kQD / 8; ++c) {
          const int d = qt * kQD + c * 8;
          if (d < p.D) *reinterpret_cast<uint4*>(orow + d) = pack8<P2>(o + c * 8, inv);
        }
      }
      if (qt == 0 && m < p.M)
        p.lse[(static_cast<int64_t>(bh)) * p.M + m] = any_key ? m_used + log2f(l) : INFINITY;
    }
    }  // tiles
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 17) tmem_dealloc(tmem, kTmemCols);
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
  return launch_overlapped(kern, grid, 640, L::kDynamic, stream, fp);
}

template <int DP, typename T>
int launch_bias(const FwdParams& fp, int bias_kind, dim3 grid, cudaStream_t stream) {
  switch (bias_kind) {
    case FA_BIAS_NONE: return launch_inst<DP, T, 0>(fp, grid, stream);
    case FA_BIAS_SAME: return launch_inst<DP, T, 1>(fp, grid, stream);
    case FA_BIAS_BOOL: return launch_inst<DP, T, 2>(fp, grid, stream);
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
  r = make_tmap_bshd(&fp.map_v, p.v, p.B, p.N, p.H, p.D, p.v_stride, 128);
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
  } else {
    fp.map_bias = fp.map_q;
  }
  if (reinterpret_cast<uintptr_t>(p.o) % 16 != 0 || p.o_stride[0] % 8 || p.o_stride[1] % 8 ||
      p.o_stride[2] % 8)
    return FA_ERR_ALIGN;
  fp.o = p.o;
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
  fp.n_tiles = fp.n_mblk * p.B * p.H;
  const dim3 grid(persistent_grid(p.causal ? (fp.n_tiles + 1) / 2 : fp.n_tiles));
  const int dp = padded_head_dim(p.D);
  if (p.dtype == FA_BF16) {
    return dp == 64 ? launch_bias<64, __nv_bfloat16>(fp, p.bias_kind, grid, stream)
                    : launch_bias<128, __nv_bfloat16>(fp, p.bias_kind, grid, stream);
  }
  return dp == 64 ? launch_bias<64, __half>(fp, p.bias_kind, grid, stream)
                  : launch_bias<128, __half>(fp, p.bias_kind, grid, stream);
}

}  // namespace fa
