// Backward preprocess: delta[b,h,m] = sum_d o[b,m,h,d] * do[b,m,h,d] in fp32.
// A pure bandwidth kernel: D/8 threads share one row, each reads 16 bytes of o
// and of do, and the partial sums are combined with shuffles.
// Replaces _attn_bwd_preprocess of the reference (flash_attention.py 197-233).
#include "fa_common.cuh"
#include "fa_host.cuh"

namespace fa {
namespace {

struct PreParams {
  const void* o;
  const void* d_o;
  float* delta;
  int64_t o_sB, o_sM, o_sH, do_sB, do_sM, do_sH;
  int H, M, D;
};

template <typename T>
__global__ void __launch_bounds__(256) bwd_pre_kernel(const PreParams p) {
  using P2 = Pack2<T>;
  const int tpr = p.D >> 3;  // threads per row: 2, 4, 8 or 16
  const int rows_per_block = 256 / tpr;
  const int sub = threadIdx.x % tpr;
  const int m = blockIdx.x * rows_per_block + threadIdx.x / tpr;
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh - b * p.H;
  float acc = 0.f;
  grid_dep_launch_next();
  grid_dep_wait();  // o and do of the previous kernels are visible from here
  if (m < p.M) {
    const T* orow = reinterpret_cast<const T*>(p.o) + b * p.o_sB + (int64_t)m * p.o_sM + h * p.o_sH;
    const T* drow =
        reinterpret_cast<const T*>(p.d_o) + b * p.do_sB + (int64_t)m * p.do_sM + h * p.do_sH;
    const uint4 a = __ldcg(reinterpret_cast<const uint4*>(orow) + sub);
    const uint4 g = __ldcg(reinterpret_cast<const uint4*>(drow) + sub);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = P2::unpack(aw[i]), y = P2::unpack(gw[i]);
      acc = fmaf(x.x, y.x, acc);
      acc = fmaf(x.y, y.y, acc);
    }
  }
  for (int off = tpr >> 1; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if (sub == 0 && m < p.M) p.delta[(int64_t)bh * p.M + m] = acc;
}

}  // namespace

int launch_bwd_pre(const fa_params& p, cudaStream_t stream, int* /*status*/) {
  auto bad = [](const void* ptr, const int64_t s[3]) {
    return reinterpret_cast<uintptr_t>(ptr) % 16 != 0 || s[0] % 8 || s[1] % 8 || s[2] % 8;
  };
  if (bad(p.o, p.o_stride) || bad(p.d_o, p.do_stride)) return FA_ERR_ALIGN;
  PreParams pp;
  pp.o = p.o;
  pp.d_o = p.d_o;
  pp.delta = p.delta;
  pp.o_sB = p.o_stride[0];
  pp.o_sM = p.o_stride[1];
  pp.o_sH = p.o_stride[2];
  pp.do_sB = p.do_stride[0];
  pp.do_sM = p.do_stride[1];
  pp.do_sH = p.do_stride[2];
  pp.H = p.H;
  pp.M = p.M;
  pp.D = p.D;
  const int rows_per_block = 256 / (p.D / 8);
  const dim3 grid((p.M + rows_per_block - 1) / rows_per_block, p.B * p.H);
  if (p.dtype == FA_BF16)
    return launch_overlapped(bwd_pre_kernel<__nv_bfloat16>, grid, 256, 0, stream, pp);
  else
    return launch_overlapped(bwd_pre_kernel<__half>, grid, 256, 0, stream, pp);
}

}  // namespace fa
