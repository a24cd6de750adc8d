// dK / dV (and dS) kernel for head dimension 256 on sm_100a.
//
// At D = 256 the four accumulators S, dP, dV, dK of a [128 x 128] tile would need 768
// tensor-memory columns and K, V, Q, dO alone 256 KB of shared memory, so this kernel
// works on tiles of 128 query rows x 64 keys and keeps the two gradients TRANSPOSED:
//   S    = Q K^T          [128 q x 64 keys]   (64 columns)
//   dP   = dO V^T         [128 q x 64 keys]   (64 columns)
//   dV^T += dO^T P        [256 d x 64 keys]   two products with M = 128 (2 x 64 columns)
//   dK^T += Q^T dS        [256 d x 64 keys]   two products with M = 128 (2 x 64 columns)
// The transposed products take the dO / Q tiles as MN-major A operands and the 16-bit
// P / dS tiles [128 q][64 keys] as MN-major B operands - the same shared-memory tiles,
// read through other descriptors, no data movement.
// One CTA per (batch, head, block of 64 keys); it walks the 128-row query blocks that see
// its keys.  Roles (192 threads): warps 0-3 row threads (thread = query row = tensor-memory
// lane), warp 4 TMA producer, warp 5 MMA issuer and tensor-memory owner (both run converged and elect
// a lane for the issue).  Shared memory:
// K 32 KB, V 32, Q 64, dO 64, P 16, dS 16 = 224 KB, everything single-staged: a step is
//   loads of Q, dO -> S, dP -> row threads (P, dS) -> dV^T, dK^T -> next loads
// without overlap between steps.  This is the correct-first version for a head dimension
// the tile kernels do not reach; it is not tuned.
// Bias / mask rows are read by the row threads straight from global memory.  The 16-bit
// dS always goes out to global memory (the bias gradient itself for a 16-bit bias,
// otherwise a scratch tensor): the dQ stage at this head dimension is the streamed product
// dQ = sm_scale * dS K.  An fp32 bias gets its unrounded fp32 gradient from registers.
// Query blocks above the causal diagonal are not visited: the caller zero-fills dbias.
//
// Replaces _attn_bwd_dkdv / _attn_bwd_dkdv_inner of the reference (flash_attention.py
// 237-454) at BLOCK_HEADDIM = 256: same P, dS, dbias = dS, dK scaled by sm_scale.
#include "fa_common.cuh"
#include "fa_host.cuh"

namespace fa {
namespace {

struct Dkdv256Params {
  CUtensorMap map_q;   // box of 128 rows
  CUtensorMap map_k;   // box of 64 rows
  CUtensorMap map_v;   // box of 64 rows
  CUtensorMap map_do;  // box of 128 rows
  const void* bias;
  void* dk;
  void* dv;
  void* ds16;        // (B, H, M, N) 16-bit dS out; rows 16-byte aligned
  float* dbias_f32;  // fp32 bias gradient or null
  const float* lse;
  const float* delta;
  int* status;
  int64_t bias_sB, bias_sH, bias_sM;
  int64_t ds_sB, ds_sH, ds_sM;
  int64_t dbf_sB, dbf_sH, dbf_sM;
  int64_t dk_sB, dk_sN, dk_sH, dv_sB, dv_sN, dv_sH;
  int H, M, N;
  int causal, bias_vec32;
  float scale_log2;  // sm_scale * log2(e)
  float sm_scale;
};

enum Dkdv256Site { kSiteKV = 1, kSiteQdoFull, kSiteQdoEmpty, kSiteSdpFull, kSitePdsReady, kSiteAccDone };

constexpr int kQTile256 = 128 * 256 * 2;  // 64 KB: four [128][64] blocks
constexpr int kKTile256 = 64 * 256 * 2;   // 32 KB: four [64][64] blocks
constexpr int kKBlk256 = 64 * 128;        // bytes of one [64 rows][64] block
constexpr int kPTile256 = 128 * 128;      // [128 q][64 keys] 16-bit
constexpr int kOffK = 0, kOffV = kOffK + kKTile256, kOffQ = kOffV + kKTile256, kOffDo = kOffQ + kQTile256;
constexpr int kOffP = kOffDo + kQTile256, kOffDs = kOffP + kPTile256;
constexpr int kSmem256 = kOffDs + kPTile256 + 1024;  // + slack for 1024-byte alignment

template <typename T, int BIAS>
__global__ void __launch_bounds__(192, 1) dkdv256_kernel(const __grid_constant__ Dkdv256Params p) {
  using P2 = Pack2<T>;
  constexpr uint32_t kColS = 0, kColDp = 64, kColDv = 128, kColDk = 256;
  constexpr uint32_t kTmemCols = 512;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t kv_full, qdo_full, qdo_empty, sdp_full, pds_ready, acc_done;
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x;
  // the warp index as a value the compiler knows to be the same in all lanes
  const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
  const int lane = tid & 31;
  const int n0 = static_cast<int>(blockIdx.x) * 64;
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh - b * p.H;
  const int n_mblk = (p.M + 127) >> 7;
  // causal (top-left aligned): query block i sees key n0 when 128 i + 127 >= n0
  const int i_start = p.causal ? min(n0 >> 7, n_mblk) : 0;
  const int steps = n_mblk - i_start;

  WaitCtx ctx{&abort_flag, p.status, 5};

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&kv_full, 1);
    mbar_init(&qdo_full, 1);
    mbar_init(&qdo_empty, 1);
    mbar_init(&sdp_full, 1);
    mbar_init(&pds_ready, 4);
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
  grid_dep_wait();  // the previous kernels' results (and the status word) are visible from here
  const bool live = *reinterpret_cast<volatile int*>(p.status) == 0;

  if (warp == 4) {
    // ------------------------------------------------------------------ producer
    // (whole warp converged, one elected lane issues: the operands of the bulk loads and of
    // the tensor-core instructions are then warp-uniform values)
    if (live && steps > 0) {
      if (elect_one()) {
        tma_prefetch_desc(&p.map_q);
        tma_prefetch_desc(&p.map_k);
        tma_prefetch_desc(&p.map_v);
        tma_prefetch_desc(&p.map_do);
        mbar_expect_tx(&kv_full, 2 * kKTile256);
        for (int kb = 0; kb < 4; ++kb) {
          tma_load_4d(smem + kOffK + kb * kKBlk256, &p.map_k, &kv_full, kb * 64, h, n0, b);
          tma_load_4d(smem + kOffV + kb * kKBlk256, &p.map_v, &kv_full, kb * 64, h, n0, b);
        }
      }
      __syncwarp();
      bool ok = true;
      for (int s = 0; s < steps && ok; ++s) {
        // Q / dO (and the P / dS tiles) are free once the previous step's products are through
        if (s >= 1) ok = wait_warp(&qdo_empty, (s - 1) & 1, ctx, kSiteQdoEmpty, s);
        if (!ok) break;
        const int m0 = (i_start + s) * 128;
        if (elect_one()) {
          mbar_expect_tx(&qdo_full, 2 * kQTile256);
          for (int kb = 0; kb < 4; ++kb) {
            tma_load_4d(smem + kOffQ + kb * kBlk, &p.map_q, &qdo_full, kb * 64, h, m0, b);
            tma_load_4d(smem + kOffDo + kb * kBlk, &p.map_do, &qdo_full, kb * 64, h, m0, b);
          }
        }
        __syncwarp();
      }
    }
  } else if (warp == 5) {
    // --------------------------------------------------------------- MMA issuer
    if (live && steps > 0) {
      constexpr bool bf = P2::kIsBf16;
      constexpr uint32_t idesc_s = make_idesc(bf, false, false, 128, 64);
      constexpr uint32_t idesc_t = make_idesc(bf, true, true, 128, 64);
      const uint32_t q_addr = smem_u32(smem + kOffQ), do_addr = smem_u32(smem + kOffDo);
      const uint32_t k_addr = smem_u32(smem + kOffK), v_addr = smem_u32(smem + kOffV);
      const uint64_t p_mn = make_sdesc(smem_u32(smem + kOffP), kBlk, 1024);
      const uint64_t ds_mn = make_sdesc(smem_u32(smem + kOffDs), kBlk, 1024);
      bool ok = wait_warp(&kv_full, 0, ctx, kSiteKV, 0);
      for (int s = 0; s < steps && ok; ++s) {
        ok = wait_warp(&qdo_full, s & 1, ctx, kSiteQdoFull, s);
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          // S = Q K^T, dP = dO V^T: 16 K slices over four 64-column blocks
          issue_gemm_ss<16, false, false>(tmem + kColS, make_sdesc(q_addr, 0, 1024), make_sdesc(k_addr, 0, 1024),
                                          kBlk, kKBlk256, idesc_s, false);
          issue_gemm_ss<16, false, false>(tmem + kColDp, make_sdesc(do_addr, 0, 1024), make_sdesc(v_addr, 0, 1024),
                                          kBlk, kKBlk256, idesc_s, false);
          mma_commit(&sdp_full);
        }
        __syncwarp();
        ok = wait_warp_hot(&pds_ready, s & 1, ctx, kSitePdsReady, s);
        if (!ok) break;
        tc_fence_after();
        if (elect_one()) {
          // dV^T[d half] += dO^T[d half] P,  dK^T[d half] += Q^T[d half] dS  (K = 128 query rows)
          for (int hh = 0; hh < 2; ++hh) {
            issue_gemm_ss<8, true, true>(tmem + kColDv + hh * 64, make_sdesc(do_addr + 2 * hh * kBlk, kBlk, 1024),
                                         p_mn, kBlk, kBlk, idesc_t, s > 0);
            issue_gemm_ss<8, true, true>(tmem + kColDk + hh * 64, make_sdesc(q_addr + 2 * hh * kBlk, kBlk, 1024),
                                         ds_mn, kBlk, kBlk, idesc_t, s > 0);
          }
          mma_commit(&qdo_empty);
        }
        __syncwarp();
      }
      if (ok && elect_one()) mma_commit(&acc_done);
    }
    __syncwarp();
  } else {
    // --------------------------------------------------------------- row threads
    const int r = warp * 32 + lane;  // query row inside the block = tensor-memory lane
    const uint32_t lane_base = static_cast<uint32_t>(warp) * 32u;
    const uint32_t sp_row = smem_u32(smem + kOffP) + static_cast<uint32_t>(r) * 128u;
    const uint32_t sds_row = smem_u32(smem + kOffDs) + static_cast<uint32_t>(r) * 128u;
    const int64_t bias_bh = b * p.bias_sB + h * p.bias_sH;
    bool ok = live;
#pragma unroll 1
    for (int s = 0; s < steps && ok; ++s) {
      const int m0 = (i_start + s) * 128;
      const int m = m0 + r;
      const bool row_ok = m < p.M;
      const int64_t idx = static_cast<int64_t>(bh) * p.M + min(m, p.M - 1);
      // rows beyond M get -inf / 0, which makes their P and dS zero
      const float neg_lse = row_ok ? -__ldcg(p.lse + idx) : -INFINITY;
      const float delta_r = row_ok ? __ldcg(p.delta + idx) : 0.f;
      ok = wait_warp(&sdp_full, s & 1, ctx, kSiteSdpFull, s);
      if (!ok) break;
      tc_fence_after();
#pragma unroll 1
      for (int q = 0; q < 2; ++q) {
        const int col0 = n0 + q * 32;
        BiasRegs<BIAS> br;
        if (BIAS != 0)
          load_bias_row<BIAS>(br, p.bias, bias_bh + static_cast<int64_t>(m) * p.bias_sM, row_ok, col0, p.N,
                              p.bias_vec32 != 0);
        float pr[32];
        tmem_ld32(tmem_addr(tmem, lane_base, kColS + q * 32), reinterpret_cast<uint32_t*>(pr));
        tmem_ld_wait();
        // P = exp2(S * scale * log2e + bias * log2e - LSE2)
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          f32x2 a = ffma2(f2(pr[i], pr[i + 1]), f2(p.scale_log2, p.scale_log2), f2(neg_lse, neg_lse));
          if (BIAS == 1) {
            const float2 f = P2::unpack(br.w[i >> 1]);
            a = ffma2(f2(f.x, f.y), f2(kLog2e, kLog2e), a);
          } else if (BIAS == 3) {
            a = ffma2(f2(__uint_as_float(br.w[i]), __uint_as_float(br.w[i + 1])), f2(kLog2e, kLog2e), a);
          }
          float e0 = ex2(f2_lo(a)), e1 = ex2(f2_hi(a));
          if (BIAS == 2) {
            const uint32_t m2 = br.w[i >> 2] >> (8 * (i & 3));
            e0 = (m2 & 0xFFu) != 0 ? e0 : 0.f;
            e1 = (m2 & 0xFF00u) != 0 ? e1 : 0.f;
          }
          pr[i] = e0;
          pr[i + 1] = e1;
        }
        if ((col0 + 32 > p.N) || (p.causal && col0 + 31 > m0)) {
          int limit = p.N - col0;
          if (p.causal) limit = min(limit, m - col0 + 1);
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i >= limit) pr[i] = 0.f;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c)
          sts128(sp_row + (static_cast<uint32_t>((q * 4 + c) ^ (r & 7)) << 4), P2::pack(pr[c * 8 + 0], pr[c * 8 + 1]),
                 P2::pack(pr[c * 8 + 2], pr[c * 8 + 3]), P2::pack(pr[c * 8 + 4], pr[c * 8 + 5]),
                 P2::pack(pr[c * 8 + 6], pr[c * 8 + 7]));
        // dS = P * (dP - delta)
        uint32_t dp[32];
        tmem_ld32(tmem_addr(tmem, lane_base, kColDp + q * 32), dp);
        tmem_ld_wait();
        uint32_t dsu[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const f32x2 d = fmul2(f2(pr[2 * i], pr[2 * i + 1]),
                                fadd2(f2(__uint_as_float(dp[2 * i]), __uint_as_float(dp[2 * i + 1])),
                                      f2(-delta_r, -delta_r)));
          dsu[i] = P2::pack(f2_lo(d), f2_hi(d));
          dp[2 * i] = __float_as_uint(f2_lo(d));
          dp[2 * i + 1] = __float_as_uint(f2_hi(d));
        }
#pragma unroll
        for (int c = 0; c < 4; ++c)
          sts128(sds_row + (static_cast<uint32_t>((q * 4 + c) ^ (r & 7)) << 4), dsu[c * 4 + 0], dsu[c * 4 + 1],
                 dsu[c * 4 + 2], dsu[c * 4 + 3]);
        if (row_ok && col0 < p.N) {
          // the 16-bit dS row segment: 64 contiguous bytes
          T* drow = reinterpret_cast<T*>(p.ds16) + b * p.ds_sB + h * p.ds_sH + static_cast<int64_t>(m) * p.ds_sM + col0;
          if (col0 + 32 <= p.N) {
#pragma unroll
            for (int c = 0; c < 4; ++c)
              *reinterpret_cast<uint4*>(drow + 8 * c) =
                  make_uint4(dsu[c * 4 + 0], dsu[c * 4 + 1], dsu[c * 4 + 2], dsu[c * 4 + 3]);
          } else {
            const uint16_t* half = reinterpret_cast<const uint16_t*>(dsu);
#pragma unroll
            for (int k = 0; k < 32; ++k)
              if (col0 + k < p.N) reinterpret_cast<uint16_t*>(drow)[k] = half[k];
          }
          if (BIAS == 3 && p.dbias_f32 != nullptr) {
            float* frow = p.dbias_f32 + b * p.dbf_sB + h * p.dbf_sH + static_cast<int64_t>(m) * p.dbf_sM + col0;
            if (col0 + 32 <= p.N) {
#pragma unroll
              for (int k = 0; k < 8; ++k)
                *reinterpret_cast<uint4*>(frow + 4 * k) = make_uint4(dp[4 * k], dp[4 * k + 1], dp[4 * k + 2], dp[4 * k + 3]);
            } else {
#pragma unroll
              for (int k = 0; k < 32; ++k)
                if (col0 + k < p.N) frow[k] = __uint_as_float(dp[k]);
            }
          }
        }
      }
      // P and dS are in shared memory, S and dP in registers: the tensor core may go on
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pds_ready);
    }

    // ---- epilogue: dV^T, dK^T (lane = head-dim column, columns = keys) -> global
    if (ok && steps > 0) ok = wait_warp(&acc_done, 0, ctx, kSiteAccDone, 0);
    if (ok) {
      tc_fence_after();
#pragma unroll 1
      for (int which = 0; which < 2; ++which) {
        T* base = reinterpret_cast<T*>(which == 0 ? p.dv : p.dk) + b * (which == 0 ? p.dv_sB : p.dk_sB) +
                  h * (which == 0 ? p.dv_sH : p.dk_sH);
        const int64_t sN = which == 0 ? p.dv_sN : p.dk_sN;
        const float mul = which == 0 ? 1.0f : p.sm_scale;
#pragma unroll 1
        for (int hh = 0; hh < 2; ++hh) {
#pragma unroll 1
          for (int q = 0; q < 2; ++q) {
            uint32_t a[32];
            if (steps > 0) {
              tmem_ld32(tmem_addr(tmem, lane_base, (which == 0 ? kColDv : kColDk) + hh * 64 + q * 32), a);
              tmem_ld_wait();
            } else {
#pragma unroll
              for (int k = 0; k < 32; ++k) a[k] = 0;  // keys no query row sees
            }
            const int d = hh * 128 + r;
#pragma unroll
            for (int k = 0; k < 32; ++k) {
              const int n = n0 + q * 32 + k;
              // the 32 lanes of a warp write 64 contiguous bytes of one key's row
              if (n < p.N) base[static_cast<int64_t>(n) * sN + d] = static_cast<T>(__uint_as_float(a[k]) * mul);
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 5) tmem_dealloc(tmem, kTmemCols);
}

template <typename T, int BIAS>
int launch_inst(const Dkdv256Params& kp, dim3 grid, cudaStream_t stream) {
  auto kern = dkdv256_kernel<T, BIAS>;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem256) != cudaSuccess)
      return FA_ERR_CUDA;
    configured[dev] = true;
  }
  return launch_overlapped(kern, grid, 192, kSmem256, stream, kp);
}

template <typename T>
int launch_bias(const Dkdv256Params& kp, int bias_kind, dim3 grid, cudaStream_t stream) {
  switch (bias_kind) {
    case FA_BIAS_NONE: return launch_inst<T, 0>(kp, grid, stream);
    case FA_BIAS_SAME: return launch_inst<T, 1>(kp, grid, stream);
    case FA_BIAS_BOOL: return launch_inst<T, 2>(kp, grid, stream);
    case FA_BIAS_F32: return launch_inst<T, 3>(kp, grid, stream);
    default: return FA_ERR_UNSUPPORTED;
  }
}

}  // namespace

// The 16-bit dS tensor of a head-dim-256 backward: the bias gradient itself when one is
// wanted for a 16-bit bias, otherwise the caller's scratch.
const void* d256_ds_tensor(const fa_params& p, const int64_t** stride) {
  if (p.write_dbias && p.bias_kind == FA_BIAS_SAME) {
    *stride = p.dbias_stride;
    return p.dbias;
  }
  *stride = p.ds16_stride;
  return p.ds16;
}

int launch_bwd_dkdv_d256(const fa_params& p, cudaStream_t stream, int* status) {
  Dkdv256Params kp;
  int r = make_tmap_bshd(&kp.map_q, p.q, p.B, p.M, p.H, p.D, p.q_stride, 128);
  if (r) return r;
  r = make_tmap_bshd(&kp.map_k, p.k, p.B, p.N, p.H, p.D, p.k_stride, 64);
  if (r) return r;
  r = make_tmap_bshd(&kp.map_v, p.v, p.B, p.N, p.H, p.D, p.v_stride, 64);
  if (r) return r;
  r = make_tmap_bshd(&kp.map_do, p.d_o, p.B, p.M, p.H, p.D, p.do_stride, 128);
  if (r) return r;
  const int64_t* ds_stride = nullptr;
  const void* ds = d256_ds_tensor(p, &ds_stride);
  if (!ds) return FA_ERR_NULL;
  if (reinterpret_cast<uintptr_t>(ds) % 16 != 0 || ds_stride[0] % 8 || ds_stride[1] % 8 || ds_stride[2] % 8)
    return FA_ERR_ALIGN;
  kp.ds16 = const_cast<void*>(ds);
  kp.ds_sB = ds_stride[0];
  kp.ds_sH = ds_stride[1];
  kp.ds_sM = ds_stride[2];
  const bool f32 = p.bias_kind == FA_BIAS_F32;
  kp.dbias_f32 = nullptr;
  kp.dbf_sB = kp.dbf_sH = kp.dbf_sM = 0;
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
  const int eb = p.bias_kind == FA_BIAS_BOOL ? 1 : (f32 ? 4 : 2);
  if (p.bias_kind != FA_BIAS_NONE) {
    if (reinterpret_cast<uintptr_t>(p.bias) % 16 != 0 || (p.bias_stride[0] * eb) % 16 ||
        (p.bias_stride[1] * eb) % 16 || (p.bias_stride[2] * eb) % 16)
      return FA_ERR_ALIGN;
  }
  kp.bias_vec32 = p.bias_kind != FA_BIAS_NONE && reinterpret_cast<uintptr_t>(p.bias) % 32 == 0 &&
                  (p.bias_stride[0] * eb) % 32 == 0 && (p.bias_stride[1] * eb) % 32 == 0 &&
                  (p.bias_stride[2] * eb) % 32 == 0;
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
  kp.causal = p.causal ? 1 : 0;
  kp.scale_log2 = p.sm_scale * kLog2e;
  kp.sm_scale = p.sm_scale;
  const dim3 grid((p.N + 63) / 64, p.B * p.H);
  return p.dtype == FA_BF16 ? launch_bias<__nv_bfloat16>(kp, p.bias_kind, grid, stream)
                            : launch_bias<__half>(kp, p.bias_kind, grid, stream);
}

}  // namespace fa
