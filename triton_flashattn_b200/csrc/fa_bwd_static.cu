// fa_bwd_static_scratch: the whole backward pass for callers that are not allowed
// to allocate device memory.
//
// The regular fa_bwd needs one scratch tensor from its caller: `delta`, the fp32
// row sums of o * do, (B, H, M) floats, written by the preprocess stage and read
// by the dK/dV and dQ stages.  Some callers have nowhere to get it from: a plugin
// that is handed raw pointers by a host runtime with a frozen, pre-planned memory
// arena; a real-time loop that must not touch the allocator after start-up; a
// binding layer in a language without access to the process's CUDA allocator.
// For them this entry point keeps the scratch inside the library, in the
// file-scope device array below, so the call needs nothing beyond the inputs and
// outputs it is given.
//
// Facts a caller must know:
//  * Limit: B * H * M <= 2,097,152 rows (8 MiB of fp32).  Larger problems are refused
//    with FA_ERR_TOO_LARGE; use fa_bwd with your own `delta` buffer instead.
//  * Every GPU whose context loads this library holds those 8 MiB until the process
//    exits.
//  * The first call on a device looks up the device address of the array (once per
//    device, cached).  Make that first call before you start capturing a stream.
//  * The array is shared by all calls on a device and keeps whatever the last call
//    wrote.  Nothing in it needs to start at zero: the preprocess stage overwrites
//    every row the later stages read.  Two calls that overlap on the GPU (different
//    streams, no ordering between them) race on it; order them yourself.
//  * Nothing here calls cudaMalloc, cudaFree or any allocating routine.
#include <mutex>

#include "fa_host.cuh"

namespace fa {
namespace {

constexpr long long kStaticScratchRows = 2097152;  // B * H * M limit

static __device__ __align__(256) float g_delta_scratch[kStaticScratchRows];

constexpr int kMaxDevicesStatic = 64;
float* g_scratch_ptr[kMaxDevicesStatic];
std::mutex g_scratch_mu;

// Device address of g_delta_scratch on `device`.  In host code the array's name is
// only a handle for the runtime, not an address a kernel can use, so the address is
// asked for with cudaGetSymbolAddress while `device` is current, once per device.
int scratch_address(int device, float** out) {
  if (device < 0 || device >= kMaxDevicesStatic) return FA_ERR_CUDA;
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  if (!g_scratch_ptr[device]) {
    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess) return FA_ERR_CUDA;
    if (prev != device && cudaSetDevice(device) != cudaSuccess) return FA_ERR_CUDA;
    float* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_delta_scratch);
    if (prev != device) cudaSetDevice(prev);
    if (e != cudaSuccess || ptr == nullptr) return FA_ERR_CUDA;
    g_scratch_ptr[device] = ptr;
  }
  *out = g_scratch_ptr[device];
  return FA_OK;
}

}  // namespace
}  // namespace fa

extern "C" int fa_bwd_static_scratch(const fa_params* p, void* stream) {
  using namespace fa;
  if (!p) return FA_ERR_NULL;
  if (p->struct_size != sizeof(fa_params)) return FA_ERR_ABI;
  if (p->B < 1 || p->H < 1 || p->M < 1) return FA_ERR_SHAPE;
  if (static_cast<long long>(p->B) * p->H * p->M > kStaticScratchRows) return FA_ERR_TOO_LARGE;
  float* scratch = nullptr;
  if (int r = scratch_address(p->device, &scratch)) return r;
  fa_params q = *p;   // the caller's struct is left untouched
  q.delta = scratch;  // whatever the caller put in `delta` is ignored
  return fa_bwd(&q, stream);
}
