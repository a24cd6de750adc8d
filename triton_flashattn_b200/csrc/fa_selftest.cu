// One-tile self-test of the tcgen05 / TMA building blocks (fa_selftest_umma).
// A single CTA of 128 threads loads two [128][128] 16-bit matrices with TMA,
// multiplies them in one of the operand arrangements the attention kernels use
// and writes the fp32 accumulator (or, in mode 4, a re-written 16-bit tile via a
// bulk tensor store) back to global memory.
#include "fa_common.cuh"
#include "fa_host.cuh"

namespace fa {
namespace {

struct SelftestParams {
  CUtensorMap map_a;
  CUtensorMap map_b;
  CUtensorMap map_c16;
  float* c;
  int* status;
  int mode;
  uint32_t is_bf16;
};

constexpr int kTile = 128 * 128 * 2;  // bytes of one [128][128] 16-bit tile (two blocks)

__global__ void __launch_bounds__(128, 1) selftest_kernel(const __grid_constant__ SelftestParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kTile;
  uint8_t* sC = smem + 2 * kTile;
  __shared__ uint64_t bar_load, bar_mma;
  __shared__ uint32_t tmem_base_slot;
  __shared__ int abort_flag;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  WaitCtx ctx{&abort_flag, p.status, 100};

  if (tid == 0) {
    abort_flag = 0;
    mbar_init(&bar_load, 1);
    mbar_init(&bar_mma, 1);
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(&tmem_base_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_slot;

  if (tid == 0) {
    mbar_expect_tx(&bar_load, 2 * kTile);
    tma_load_4d(sA, &p.map_a, &bar_load, 0, 0, 0, 0);
    tma_load_4d(sA + kTile / 2, &p.map_a, &bar_load, 64, 0, 0, 0);
    tma_load_4d(sB, &p.map_b, &bar_load, 0, 0, 0, 0);
    tma_load_4d(sB + kTile / 2, &p.map_b, &bar_load, 64, 0, 0, 0);
  }
  bool ok = mbar_wait(&bar_load, 0, ctx, 1);

  const uint32_t a_addr = smem_u32(sA), b_addr = smem_u32(sB);
  const bool bf = p.is_bf16 != 0;

  if (ok && p.mode == 3) {
    // stage A through tensor memory: thread = row, 16-bit pairs packed per column
    uint32_t regs[32];
    for (int half = 0; half < 2; ++half) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint4 v = *reinterpret_cast<const uint4*>(sA + half * (kTile / 2) + swz_off(tid, c));
        regs[c * 4 + 0] = v.x;
        regs[c * 4 + 1] = v.y;
        regs[c * 4 + 2] = v.z;
        regs[c * 4 + 3] = v.w;
      }
      tmem_st32(tmem_addr(tmem, warp * 32, 128 + half * 32), regs);
    }
    tmem_st_wait();
  }
  if (ok && p.mode == 4) {
    // rewrite A into sC through the generic proxy, then bulk-store it
    for (int half = 0; half < 2; ++half) {
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint4 v = *reinterpret_cast<const uint4*>(sA + half * (kTile / 2) + swz_off(tid, c));
        *reinterpret_cast<uint4*>(sC + half * (kTile / 2) + swz_off(tid, c)) = v;
      }
    }
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

  if (p.mode == 4) {
    if (tid == 0 && ok) {
      tma_store_4d(&p.map_c16, sC, 0, 0, 0, 0);
      tma_store_4d(&p.map_c16, sC + kTile / 2, 64, 0, 0, 0);
      tma_store_commit();
      tma_store_wait_all<0>();
    }
  } else {
    if (tid == 0 && ok) {
      uint32_t idesc;
      switch (p.mode) {
        case 0: idesc = make_idesc(bf, false, false, 128, 128); break;
        case 1: idesc = make_idesc(bf, false, true, 128, 128); break;
        case 2: idesc = make_idesc(bf, true, true, 128, 128); break;
        default: idesc = make_idesc(bf, false, true, 128, 128); break;
      }
      for (int ks = 0; ks < 8; ++ks) {
        const uint64_t bdesc = p.mode == 0 ? sdesc_kmajor(b_addr, kTile / 2, ks)
                                           : sdesc_mnmajor(b_addr, kTile / 2, ks);
        if (p.mode == 3) {
          mma_ts(tmem, tmem_addr(tmem, 0, 128 + ks * 8), bdesc, idesc, ks > 0);
        } else {
          const uint64_t adesc = p.mode == 2 ? sdesc_mnmajor(a_addr, kTile / 2, ks)
                                             : sdesc_kmajor(a_addr, kTile / 2, ks);
          mma_ss(tmem, adesc, bdesc, idesc, ks > 0);
        }
      }
      mma_commit(&bar_mma);
    }
    ok = ok && mbar_wait(&bar_mma, 0, ctx, 2);
    tc_fence_after();
    if (ok) {
      for (int g = 0; g < 4; ++g) {
        uint32_t r[32];
        tmem_ld32(tmem_addr(tmem, warp * 32, g * 32), r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) p.c[tid * 128 + g * 32 + i] = __uint_as_float(r[i]);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

// One CTA whose threads all wait, with a limit the caller chooses, for a barrier phase that
// nothing ever completes.  The wait gives up, the status word (and its host copy) records
// kernel 101 / site 7, and the kernel returns: the failure path of every kernel of this
// library, exercised without hanging or faulting anything.
__global__ void __launch_bounds__(128, 1) selftest_timeout_kernel(int* status, uint32_t limit_us) {
  __shared__ uint64_t never;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&never, 1);
    mbar_fence_init();
  }
  __syncthreads();
  WaitCtx ctx{&abort_flag, status, 101, static_cast<uint64_t>(limit_us) * 1000ull};
  const bool live = *reinterpret_cast<volatile int*>(status) == 0;
  if (live) (void)mbar_wait(&never, 0, ctx, 7, static_cast<int>(limit_us));
}

}  // namespace

int launch_selftest_timeout(uint32_t limit_us, cudaStream_t stream, int* status) {
  selftest_timeout_kernel<<<1, 128, 0, stream>>>(status, limit_us);
  return cudaGetLastError() == cudaSuccess ? FA_OK : FA_ERR_CUDA;
}

int launch_selftest(int mode, int dtype, const void* a, const void* b, void* c, cudaStream_t stream,
                    int* status) {
  SelftestParams sp;
  const int64_t st[3] = {128 * 128, 128, 128};  // (B=1, S=128, H=1, D=128)
  int r = make_tmap_bshd(&sp.map_a, a, 1, 128, 1, 128, st, 128);
  if (r) return r;
  r = make_tmap_bshd(&sp.map_b, b, 1, 128, 1, 128, st, 128);
  if (r) return r;
  r = make_tmap_bshd(&sp.map_c16, c, 1, 128, 1, 128, st, 128);
  if (r) return r;
  sp.c = static_cast<float*>(c);
  sp.status = status;
  sp.mode = mode;
  sp.is_bf16 = dtype == FA_BF16;
  const int smem = 3 * kTile + 1024;
  if (cudaFuncSetAttribute(selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) !=
      cudaSuccess)
    return FA_ERR_CUDA;
  selftest_kernel<<<1, 128, smem, stream>>>(sp);
  return cudaGetLastError() == cudaSuccess ? FA_OK : FA_ERR_CUDA;
}

}  // namespace fa
