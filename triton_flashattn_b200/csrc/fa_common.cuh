// Device-side building blocks shared by every sm_100a kernel of this library:
// mbarrier waits with an iteration limit, TMA tile loads/stores, tcgen05
// (tensor-memory) allocation, MMA issue, commit and load/store wrappers, and the
// shared-memory / instruction descriptors the tcgen05 MMAs consume.
//
// Conventions used by all kernels:
//  * a "tile block" is [rows][64] 16-bit elements (128 bytes per row) written by
//    TMA with the 128-byte swizzle; 16-byte chunk c of row r sits at chunk
//    position c ^ (r & 7).  Block bases are 1024-byte aligned.
//  * a tile with more than 64 columns is a sequence of such blocks.
//  * every spin on an mbarrier is bounded; on expiry the kernel records an error
//    in a global status word, all roles leave their loops, tensor memory is
//    released and the kernel returns.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fa {

// ----------------------------------------------------------------------------
// status word layout (int[8] in global memory, owned by the host API)
//   [0] error code (0 = ok), [1] kernel id, [2] blockIdx.x, [3] blockIdx.y,
//   [4] wait site id, [5] loop iteration,
//   [6..7] 64-bit device-visible address of a pinned host copy of words 0..5 (0 = none):
//          the kernel that records an error also writes it there, so the host learns of it
//          without synchronising
// ----------------------------------------------------------------------------
enum : int { kStatusOk = 0, kStatusWaitTimeout = 1, kStatusTmemAlloc = 2 };

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "elect.sync _|P, 0xffffffff;\n"
      "selp.b32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ----------------------------------------------------------------------------
// mbarrier
// ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n"
      "selp.b32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Non-blocking look at a phase.  A barrier operation takes ~200 cycles to answer on
// B200, so the result is requested early (before a stretch of independent work) and
// consumed later with wait_polled / wait_warp_polled.
__device__ __forceinline__ uint32_t mbar_poll(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n"
      "selp.b32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok;
}

// Two / three phases looked at in one go: the barrier queries are issued back to back
// and their answers (each ~200 cycles away) come back together, instead of one
// round trip after the other.
__device__ __forceinline__ void mbar_poll2(uint64_t* b0, uint32_t p0, uint64_t* b1, uint32_t p1,
                                           uint32_t& r0, uint32_t& r1) {
  asm volatile(
      "{\n"
      ".reg .pred P0, P1;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 P0, [%2], %3;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 P1, [%4], %5;\n"
      "selp.b32 %0, 1, 0, P0;\n"
      "selp.b32 %1, 1, 0, P1;\n"
      "}\n"
      : "=r"(r0), "=r"(r1)
      : "r"(smem_u32(b0)), "r"(p0), "r"(smem_u32(b1)), "r"(p1)
      : "memory");
}
__device__ __forceinline__ void mbar_poll3(uint64_t* b0, uint32_t p0, uint64_t* b1, uint32_t p1,
                                           uint64_t* b2, uint32_t p2, uint32_t& r0, uint32_t& r1,
                                           uint32_t& r2) {
  asm volatile(
      "{\n"
      ".reg .pred P0, P1, P2;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 P0, [%3], %4;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 P1, [%5], %6;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 P2, [%7], %8;\n"
      "selp.b32 %0, 1, 0, P0;\n"
      "selp.b32 %1, 1, 0, P1;\n"
      "selp.b32 %2, 1, 0, P2;\n"
      "}\n"
      : "=r"(r0), "=r"(r1), "=r"(r2)
      : "r"(smem_u32(b0)), "r"(p0), "r"(smem_u32(b1)), "r"(p1), "r"(smem_u32(b2)), "r"(p2)
      : "memory");
}

__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Per-CTA abort context.  `abort_flag` lives in shared memory and is set by the
// first waiter whose limit expires; every other waiter polls it so that all
// roles leave together.  `status` is the global status word.
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // 2 s per wait

struct WaitCtx {
  volatile int* abort_flag;  // shared
  int* status;               // global
  int kernel_id;
  uint64_t limit_ns = kWaitLimitNs;
};

// Returns true when the phase completed, false when the kernel must bail out.
static __device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, const WaitCtx& ctx,
                                            int site, int iter) {
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*ctx.abort_flag) return false;
    if ((++spins & 63u) == 0) {
      if (*reinterpret_cast<volatile int*>(ctx.status) != 0) {
        *ctx.abort_flag = 1;
        return false;
      }
      if (global_timer_ns() - t0 > ctx.limit_ns) {
        *ctx.abort_flag = 1;
        if (atomicCAS(ctx.status, 0, kStatusWaitTimeout) == 0) {
          const int rec[6] = {kStatusWaitTimeout, ctx.kernel_id, (int)blockIdx.x, (int)blockIdx.y, site, iter};
          for (int i = 1; i < 6; ++i) ctx.status[i] = rec[i];
          __threadfence();
          // host copy, if one is registered (words 6..7 hold its address)
          volatile int* host = reinterpret_cast<volatile int*>(
              *reinterpret_cast<volatile unsigned long long*>(ctx.status + 6));
          if (host != nullptr) {
            for (int i = 5; i >= 0; --i) host[i] = rec[i];
            __threadfence_system();
          }
        }
        return false;
      }
    }
  }
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const WaitCtx& ctx,
                                          int site, int iter = 0) {
  // fast path: a few polls without bookkeeping
#pragma unroll 1
  for (int i = 0; i < 16; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, ctx, site, iter);
}

// Wait of a single-lane control role that sits on the critical path: polls the phase
// without suspending (a suspended try_wait wakes up a few hundred cycles after the phase
// completes), then falls back to the bounded wait.
__device__ __forceinline__ bool mbar_wait_hot(uint64_t* bar, uint32_t parity, const WaitCtx& ctx,
                                              int site, int iter = 0) {
#pragma unroll 1
  for (int i = 0; i < 2048; ++i)
    if (mbar_poll(bar, parity)) return true;
  return mbar_wait(bar, parity, ctx, site, iter);
}

// ----------------------------------------------------------------------------
// proxies and fences
// ----------------------------------------------------------------------------
// Make this thread's generic-proxy shared-memory writes visible to the async
// proxy (TMA stores and tcgen05.mma operand reads).
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ----------------------------------------------------------------------------
// TMA (tiled bulk tensor copies, one CTA, no cluster features)
// ----------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d_hint(void* smem_dst, const CUtensorMap* map,
                                                 uint64_t* bar, int c0, int c1, int c2, int c3,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4, %5, %6}], [%2], %7;" ::"r"(smem_u32(smem_dst)),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3),
      "l"(policy)
      : "memory");
}

// Asks the TMA unit to pull a tile into L2 only (no shared-memory destination).
__device__ __forceinline__ void tma_prefetch_l2_4d(const CUtensorMap* map, int c0, int c1, int c2,
                                                   int c3) {
  asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}

__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, const void* smem_src, int c0,
                                             int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
          reinterpret_cast<uint64_t>(map)),
      "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Wait until at most N of this thread's bulk store groups still READ shared memory.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Wait until at most N bulk store groups are still in flight at all.
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// ----------------------------------------------------------------------------
// tensor memory
// ----------------------------------------------------------------------------
// One warp (all 32 lanes) allocates `ncols` (power of two, >= 32) columns and the
// base address is written to *smem_dst.
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}

// tensor-memory address = (lane << 16) | column
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, uint32_t lane, uint32_t col) {
  return base + (lane << 16) + col;
}

// 32 lanes x 32 bits, 32 consecutive columns: thread t of the warp receives lane
// (lane_base + t), registers r[0..31] = columns col .. col+31.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
// NC (16 or 32) consecutive columns
template <int NC>
__device__ __forceinline__ void tmem_ld_cols(uint32_t taddr, uint32_t* r) {
  if (NC == 32) tmem_ld32(taddr, r); else tmem_ld16(taddr, r);
}
template <int NC>
__device__ __forceinline__ void tmem_st_cols(uint32_t taddr, const uint32_t* r) {
  if (NC == 32) tmem_st32(taddr, r); else tmem_st16(taddr, r);
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ----------------------------------------------------------------------------
// tcgen05.mma descriptors
// ----------------------------------------------------------------------------
// Instruction descriptor for kind::f16 (fp16 or bf16 operands, fp32 accumulate).
//   bits 4-5   accumulator format (1 = f32)
//   bits 7-9   A format (0 = f16, 1 = bf16); bits 10-12 B format
//   bit 15     A major (0 = K-major, 1 = MN-major); bit 16 B major
//   bits 17-22 N >> 3; bits 24-28 M >> 4
__host__ __device__ constexpr uint32_t make_idesc(bool is_bf16, bool a_mn_major, bool b_mn_major,
                                                  int m, int n) {
  return (1u << 4) | ((is_bf16 ? 1u : 0u) << 7) | ((is_bf16 ? 1u : 0u) << 10) |
         ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// Shared-memory matrix descriptor, 128-byte swizzle.
//   bits 0-13  start address >> 4
//   bits 16-29 leading-dimension byte offset >> 4
//   bits 32-45 stride-dimension byte offset >> 4
//   bits 46-47 descriptor version (1 on sm_100)
//   bits 61-63 swizzle mode (2 = 128-byte)
__device__ __forceinline__ uint64_t make_sdesc(uint32_t smem_addr, uint32_t lbo_bytes,
                                               uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= 1ull << 46;
  d |= 2ull << 61;
  return d;
}

// K-major operand stored as tile blocks [rows][64]: the K slice `ks` (16 elements)
// of a tile whose blocks are `block_bytes` apart.
//   8-row groups are 1024 bytes apart (stride-dimension offset); a slice inside a
//   block starts 32 bytes after the previous one.
__device__ __forceinline__ uint64_t sdesc_kmajor(uint32_t tile_addr, uint32_t block_bytes, int ks) {
  const uint32_t a = tile_addr + static_cast<uint32_t>(ks >> 2) * block_bytes +
                     static_cast<uint32_t>(ks & 3) * 32u;
  return make_sdesc(a, 0, 1024);
}

// MN-major operand stored as tile blocks [k rows][64 mn]: the K slice `ks` covers
// rows 16*ks .. 16*ks+15 (2048 bytes further per slice); 64-element MN chunks are
// `block_bytes` apart (leading-dimension offset); 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t sdesc_mnmajor(uint32_t tile_addr, uint32_t block_bytes,
                                                  int ks) {
  const uint32_t a = tile_addr + static_cast<uint32_t>(ks) * 2048u;
  return make_sdesc(a, block_bytes, 1024);
}

// Offsets (in descriptor units of 16 bytes) of K slice `ks` relative to slice 0;
// adding them to a base descriptor only touches the start-address field.
__host__ __device__ constexpr uint64_t kmajor_step(int ks, uint32_t block_bytes) {
  return (static_cast<uint64_t>(ks >> 2) * block_bytes + static_cast<uint64_t>(ks & 3) * 32u) >> 4;
}
__host__ __device__ constexpr uint64_t mnmajor_step(int ks) {
  return (static_cast<uint64_t>(ks) * 2048u) >> 4;
}

// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate))
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc,
                                       uint32_t idesc, bool accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(static_cast<uint32_t>(accumulate))
      : "memory");
}
// Arrive on an mbarrier once every tcgen05 operation issued so far by this thread
// has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// One tile product as KS unrolled tcgen05.mma instructions (K = 16 each).  The
// descriptors of slice 0 are computed once by the caller; per slice only a
// constant is added, so the issuing thread spends a few instructions per MMA.
template <int KS, bool A_MN, bool B_MN>
__device__ __forceinline__ void issue_gemm_ss(uint32_t d_tmem, uint64_t a_base, uint64_t b_base,
                                              uint32_t a_block_bytes, uint32_t b_block_bytes,
                                              uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const uint64_t a = a_base + (A_MN ? mnmajor_step(ks) : kmajor_step(ks, a_block_bytes));
    const uint64_t b = b_base + (B_MN ? mnmajor_step(ks) : kmajor_step(ks, b_block_bytes));
    mma_ss(d_tmem, a, b, idesc, accumulate || ks > 0);
  }
}
// Same with the A operand in tensor memory (16-bit pairs, 8 columns per K slice).
template <int KS, bool B_MN>
__device__ __forceinline__ void issue_gemm_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_base,
                                              uint32_t b_block_bytes, uint32_t idesc,
                                              bool accumulate) {
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const uint64_t b = b_base + (B_MN ? mnmajor_step(ks) : kmajor_step(ks, b_block_bytes));
    mma_ts(d_tmem, a_tmem + ks * 8, b, idesc, accumulate || ks > 0);
  }
}

// ----------------------------------------------------------------------------
// small numeric helpers
// ----------------------------------------------------------------------------
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T>
struct Pack2;
template <>
struct Pack2<__nv_bfloat16> {
  static constexpr bool kIsBf16 = true;
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
  }
  __device__ static __forceinline__ float2 unpack(uint32_t v) {
    float2 f;
    f.x = __uint_as_float(v << 16);
    f.y = __uint_as_float(v & 0xFFFF0000u);
    return f;
  }
};
template <>
struct Pack2<__half> {
  static constexpr bool kIsBf16 = false;
  __device__ static __forceinline__ uint32_t pack(float lo, float hi) {
    uint32_t r;
    asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
  }
  __device__ static __forceinline__ float2 unpack(uint32_t v) {
    __half2 h = *reinterpret_cast<__half2*>(&v);
    return __half22float2(h);
  }
};

// Byte offset of 16-byte chunk `chunk` (0..7) of row `row` inside a swizzled tile block.
__device__ __forceinline__ uint32_t swz_off(int row, int chunk) {
  return static_cast<uint32_t>(row) * 128u + (static_cast<uint32_t>(chunk ^ (row & 7)) << 4);
}

// Packed fp32 pairs: sm_100 executes fma / add / mul on two fp32 lanes per instruction
// (each lane rounds exactly like the scalar instruction), which halves the instruction
// count of the element-wise loops.  A pair lives in one 64-bit register.
typedef uint64_t f32x2;
__device__ __forceinline__ f32x2 f2(float lo, float hi) {
  f32x2 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ float f2_lo(f32x2 v) {
  float a, b;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
  (void)b;
  return a;
}
__device__ __forceinline__ float f2_hi(f32x2 v) {
  float a, b;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
  (void)a;
  return b;
}
__device__ __forceinline__ f32x2 ffma2(f32x2 a, f32x2 b, f32x2 c) {
  f32x2 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ f32x2 fadd2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ f32x2 fmul2(f32x2 a, f32x2 b) {
  f32x2 d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// 16-byte store to shared memory through a 32-bit shared-space address.
__device__ __forceinline__ void sts128(uint32_t addr, uint32_t x, uint32_t y, uint32_t z, uint32_t w) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(x), "r"(y), "r"(z), "r"(w)
               : "memory");
}

// 16-byte load from shared memory through a 32-bit shared-space address.
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr)
               : "memory");
  return v;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Programmatic dependent launch.  Every kernel of this library is launched with the
// "programmatic stream serialization" attribute: its CTAs may be placed on an SM as soon as
// the previous kernel's CTA there has left, and run their prologue (barrier set-up, tensor
// memory allocation).  grid_dep_wait() returns once the previous kernel has completed
// and its memory is visible; nothing before it may touch global memory.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch_next() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Named barrier among `count` threads (count a multiple of 32); id 0 is __syncthreads'.
__device__ __forceinline__ void named_bar_sync(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// 32-byte (one full sector) global load served from L2.  Not the non-coherent (.nc) path:
// every kernel here may start while its predecessor in the stream still runs, and .nc is
// only defined for data that nobody writes during the whole lifetime of the reading kernel.
__device__ __forceinline__ void ldg256(const void* ptr, uint32_t* r) {
  asm volatile("ld.global.cg.v8.u32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
                 "=r"(r[7])
               : "l"(ptr));
}

// ----------------------------------------------------------------------------
// helpers shared by the attention kernels
// ----------------------------------------------------------------------------

constexpr int kBlk = 128 * 128;  // bytes of one [128][64] 16-bit tile block (also [128][128] u8)

// All lanes wait, then agree: a warp leaves its loop as a whole.
__device__ __forceinline__ bool wait_warp(uint64_t* bar, uint32_t parity, const WaitCtx& ctx,
                                          int site, int iter) {
  const bool ok = mbar_wait(bar, parity, ctx, site, iter);
  return __all_sync(0xffffffffu, ok);
}

// The same for a converged control warp on the critical path: every lane polls without
// suspending first.
__device__ __forceinline__ bool wait_warp_hot(uint64_t* bar, uint32_t parity, const WaitCtx& ctx,
                                              int site, int iter) {
  const bool ok = mbar_wait_hot(bar, parity, ctx, site, iter);
  return __all_sync(0xffffffffu, ok);
}

// Finish a wait whose phase was polled earlier: no further barrier traffic when the
// poll had already seen the phase complete.
__device__ __forceinline__ bool wait_polled(uint32_t polled, uint64_t* bar, uint32_t parity,
                                            const WaitCtx& ctx, int site, int iter) {
  if (polled) return true;
  return mbar_wait(bar, parity, ctx, site, iter);
}
__device__ __forceinline__ bool wait_warp_polled(uint32_t polled, uint64_t* bar, uint32_t parity,
                                                 const WaitCtx& ctx, int site, int iter) {
  if (__all_sync(0xffffffffu, polled != 0)) return true;
  return wait_warp(bar, parity, ctx, site, iter);
}

// 32 bias values of one row quarter, as raw 16-bit pairs (BIAS == 1), bytes (BIAS == 2) or
// fp32 words (BIAS == 3).
template <int BIAS>
struct BiasRegs {
  uint32_t w[BIAS == 1 ? 16 : (BIAS == 2 ? 8 : (BIAS == 3 ? 32 : 1))];
};

// Reads bias[row][col0 .. col0+31] straight from global memory; out-of-range elements
// read as zero.  `vec32` (uniform): rows are 32-byte aligned, so whole sectors are
// fetched with 256-bit loads; otherwise 128-bit loads; element-wise at a ragged edge.
template <int BIAS>
__device__ __forceinline__ void load_bias_row(BiasRegs<BIAS>& br, const void* bias_base,
                                              int64_t row_off, bool row_ok, int col0, int N,
                                              bool vec32) {
  constexpr int kElem = BIAS == 1 ? 2 : (BIAS == 3 ? 4 : 1);  // bytes per element
  constexpr int kWords = 8 * kElem;                           // 32-bit words per 32 elements
  constexpr int kPerWord = 4 / kElem;                         // elements per word
  if (BIAS == 0) return;
  const uint8_t* rowp = reinterpret_cast<const uint8_t*>(bias_base) + row_off * kElem;
  if (!row_ok || col0 >= N) {
#pragma unroll
    for (int i = 0; i < kWords; ++i) br.w[i] = 0;
    return;
  }
  if (col0 + 32 <= N) {
    if (vec32) {
#pragma unroll
      for (int c = 0; c < kWords / 8; ++c) ldg256(rowp + (col0 * kElem) + c * 32, br.w + c * 8);
    } else {
#pragma unroll
      for (int c = 0; c < kWords / 4; ++c) {
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(rowp + (col0 * kElem) + c * 16));
        br.w[c * 4 + 0] = v.x;
        br.w[c * 4 + 1] = v.y;
        br.w[c * 4 + 2] = v.z;
        br.w[c * 4 + 3] = v.w;
      }
    }
    return;
  }
  // ragged right edge: element-wise
#pragma unroll
  for (int i = 0; i < kWords; ++i) {
    uint32_t word = 0;
#pragma unroll
    for (int k = 0; k < kPerWord; ++k) {
      const int col = col0 + i * kPerWord + k;
      if (col < N) {
        const uint32_t e = BIAS == 1   ? (uint32_t)__ldcg(reinterpret_cast<const uint16_t*>(rowp) + col)
                           : BIAS == 3 ? __ldcg(reinterpret_cast<const uint32_t*>(rowp) + col)
                                       : (uint32_t)__ldcg(rowp + col);
        word |= e << ((8 * kElem * k) & 31);
      }
    }
    br.w[i] = word;
  }
}

// Packs 8 consecutive fp32 values (scaled) into one 16-byte vector of T.
template <typename P2>
__device__ __forceinline__ uint4 pack8(const uint32_t* a, float mul) {
  uint4 v;
  v.x = P2::pack(__uint_as_float(a[0]) * mul, __uint_as_float(a[1]) * mul);
  v.y = P2::pack(__uint_as_float(a[2]) * mul, __uint_as_float(a[3]) * mul);
  v.z = P2::pack(__uint_as_float(a[4]) * mul, __uint_as_float(a[5]) * mul);
  v.w = P2::pack(__uint_as_float(a[6]) * mul, __uint_as_float(a[7]) * mul);
  return v;
}

}  // namespace fa
