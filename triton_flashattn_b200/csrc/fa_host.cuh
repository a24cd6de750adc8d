// Host-side helpers shared by the translation units of libfa_sm100.so: tensor-map
// encoding without linking libcuda, the per-device status word, and the launcher
// prototypes that fa_api.cu dispatches to.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/fa_sm100.h"

namespace fa {

// ---- tensor maps -----------------------------------------------------------
// 4-D tiled map over 16-bit (or 8-bit) elements with the 128-byte swizzle.
//   dims[0] is the innermost (unit stride) extent; strides_bytes[i] is the byte
//   stride of dims[i+1].  box[] is the tile copied per request.
// Returns FA_OK, FA_ERR_ALIGN (address/stride rule broken) or FA_ERR_CUDA.
int make_tmap_4d(CUtensorMap* out, const void* base, int elem_bytes, const uint64_t dims[4],
                 const uint64_t strides_bytes[3], const uint32_t box[4]);

// ---- status word -----------------------------------------------------------
// Device address of the int[8] status word of the current device (file-scope
// __device__ storage inside the library; nothing is allocated).
int* device_status_ptr(int device);

// ---- launchers (defined next to their kernels) -----------------------------
int launch_fwd(const fa_params& p, cudaStream_t stream, int* status);
int launch_bwd_pre(const fa_params& p, cudaStream_t stream, int* status);
int launch_bwd_dkdv(const fa_params& p, cudaStream_t stream, int* status);
int launch_bwd_dq(const fa_params& p, cudaStream_t stream, int* status);
// Head dimension 256: its own dK/dV kernel, which always leaves the 16-bit dS in global
// memory (in dbias for a 16-bit bias that wants its gradient, else in the ds16 scratch);
// d256_ds_tensor names that tensor, the dQ stage streams it.
int launch_bwd_dkdv_d256(const fa_params& p, cudaStream_t stream, int* status);
const void* d256_ds_tensor(const fa_params& p, const int64_t** stride);
int launch_selftest(int mode, int dtype, const void* a, const void* b, void* c, cudaStream_t stream,
                    int* status);
int launch_selftest_timeout(uint32_t limit_us, cudaStream_t stream, int* status);

// Grid of a persistent kernel: one CTA per SM of the current device, never more than
// there are work units.  The environment variable FA_MAX_CTAS (a positive integer, read at
// every launch) lowers the cap; tests use it to make small problems walk many tiles
// per CTA.
int persistent_grid(int n_tiles);

// Kernels launched by this library since it was loaded (all devices, all threads).
extern std::atomic<uint64_t> g_kernel_launches;

// Launch with the programmatic-stream-serialization attribute (see grid_dep_wait()).
template <typename Kern, typename Params>
inline int launch_overlapped(Kern kern, dim3 grid, int threads, size_t smem, cudaStream_t stream,
                             const Params& params) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (cudaLaunchKernelEx(&cfg, kern, params) != cudaSuccess) return FA_ERR_CUDA;
  g_kernel_launches.fetch_add(1, std::memory_order_relaxed);
  return FA_OK;
}

// Head dims are computed on a padded width: 16/32/64 -> 64, 128 -> 128, 256 -> 256.
inline int padded_head_dim(int d) { return d <= 64 ? 64 : d; }

// Tile map for a (B, S, H, D) tensor: dims {D, H, S, B}, box {64, 1, rows, 1}.
inline int make_tmap_bshd(CUtensorMap* out, const void* base, int B, int S, int H, int D,
                          const int64_t stride[3], int box_rows) {
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  const uint64_t sb[3] = {(uint64_t)stride[2] * 2, (uint64_t)stride[1] * 2, (uint64_t)stride[0] * 2};
  const uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
  return make_tmap_4d(out, base, 2, dims, sb, box);
}

// Tile map for a (B, H, M, N) bias-like tensor: dims {N, M, H, B}; a zero stride
// on B or H collapses that dimension to extent 1 (the kernel then passes
// coordinate 0).  box {box_cols, box_rows, 1, 1}.
inline int make_tmap_bhmn(CUtensorMap* out, const void* base, int elem_bytes, int B, int H, int M,
                          int N, const int64_t stride[3], int box_cols, int box_rows, int* b_mul,
                          int* h_mul) {
  const bool b0 = stride[0] == 0, h0 = stride[1] == 0;
  *b_mul = b0 ? 0 : 1;
  *h_mul = h0 ? 0 : 1;
  const uint64_t row_bytes = (uint64_t)stride[2] * elem_bytes;
  const uint64_t dims[4] = {(uint64_t)N, (uint64_t)M, (uint64_t)(h0 ? 1 : H), (uint64_t)(b0 ? 1 : B)};
  // a collapsed dimension still needs a legal (non-zero, 16-byte multiple) stride
  const uint64_t sb[3] = {row_bytes, h0 ? row_bytes * (uint64_t)M : (uint64_t)stride[1] * elem_bytes,
                          b0 ? row_bytes * (uint64_t)M : (uint64_t)stride[0] * elem_bytes};
  const uint32_t box[4] = {(uint32_t)box_cols, (uint32_t)box_rows, 1, 1};
  return make_tmap_4d(out, base, elem_bytes, dims, sb, box);
}

}  // namespace fa
