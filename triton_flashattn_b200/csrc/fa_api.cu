// extern "C" entry points of libfa_sm100.so: argument validation, tensor-map
// encoding, the per-device status word and dispatch to the kernel launchers.
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "fa_host.cuh"

namespace fa {

// One status word per device that loads the library (file-scope device storage).
__device__ int g_fa_status[8];

std::atomic<uint64_t> g_kernel_launches{0};

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

constexpr int kMaxDevices = 64;
int* g_status_ptr[kMaxDevices];
volatile int32_t* g_mirror_host[kMaxDevices];  // pinned host copies of the status words
std::mutex g_status_mu;

struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  cudaError_t err = cudaSuccess;
  explicit DeviceGuard(int dev) {
    err = cudaGetDevice(&prev);
    if (err == cudaSuccess && prev != dev) {
      err = cudaSetDevice(dev);
      switched = (err == cudaSuccess);
    }
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
};

}  // namespace

int make_tmap_4d(CUtensorMap* out, const void* base, int elem_bytes, const uint64_t dims[4],
                 const uint64_t strides_bytes[3], const uint32_t box[4]) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return FA_ERR_CUDA;
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0) return FA_ERR_ALIGN;
  for (int i = 0; i < 3; ++i)
    if (strides_bytes[i] % 16 != 0 || strides_bytes[i] == 0) return FA_ERR_ALIGN;
  // Encoding is a pure function of these arguments, and a training loop presents the same
  // handful of (address, shape, stride) combinations step after step: a small per-thread
  // cache answers them without calling into the driver (about fifteen maps per step).
  struct Key {
    uint64_t v[12];
    bool operator==(const Key& o) const { return memcmp(v, o.v, sizeof(v)) == 0; }
  };
  struct Entry {
    Key key;
    CUtensorMap map;
    bool valid;
  };
  constexpr int kSlots = 256;
  thread_local Entry cache[kSlots] = {};
  Key key = {{reinterpret_cast<uint64_t>(base), (uint64_t)elem_bytes, dims[0], dims[1], dims[2], dims[3],
              strides_bytes[0], strides_bytes[1], strides_bytes[2],
              ((uint64_t)box[0] << 32) | box[1], ((uint64_t)box[2] << 32) | box[3], 0}};
  uint64_t hsh = 0x9E3779B97F4A7C15ull;
  for (int i = 0; i < 11; ++i) hsh = (hsh ^ key.v[i]) * 0xBF58476D1CE4E5B9ull + (hsh >> 29);
  Entry& e = cache[(hsh >> 20) % kSlots];
  if (e.valid && e.key == key) {
    memcpy(out, &e.map, sizeof(CUtensorMap));
    return FA_OK;
  }
  cuuint64_t gdim[4] = {dims[0], dims[1], dims[2], dims[3]};
  cuuint64_t gstr[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
  cuuint32_t bx[4] = {box[0], box[1], box[2], box[3]};
  cuuint32_t es[4] = {1, 1, 1, 1};
  const CUtensorMapDataType dt =
      elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT16
                      : (elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT32);
  CUresult r = fn(out, dt, 4, const_cast<void*>(base), gdim, gstr, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return FA_ERR_CUDA;
  e.key = key;
  memcpy(&e.map, out, sizeof(CUtensorMap));
  e.valid = true;
  return FA_OK;
}

int persistent_grid(int n_tiles) {
  static int sm_count[kMaxDevices] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  int sms = 0;
  if (dev >= 0 && dev < kMaxDevices) sms = sm_count[dev];
  if (sms <= 0) {
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
      sms = 148;
    if (dev >= 0 && dev < kMaxDevices) sm_count[dev] = sms;
  }
  if (const char* cap = getenv("FA_MAX_CTAS")) {
    const int c = atoi(cap);
    if (c > 0 && c < sms) sms = c;
  }
  return n_tiles < sms ? (n_tiles < 1 ? 1 : n_tiles) : sms;
}

int* device_status_ptr(int device) {
  if (device < 0 || device >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_status_mu);
  if (!g_status_ptr[device]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_fa_status) != cudaSuccess) return nullptr;
    g_status_ptr[device] = static_cast<int*>(p);
  }
  return g_status_ptr[device];
}

namespace {

int validate_common(const fa_params* p) {
  if (!p) return FA_ERR_NULL;
  if (p->struct_size != sizeof(fa_params)) return FA_ERR_ABI;
  if (p->B < 1 || p->H < 1 || p->M < 1 || p->N < 1) return FA_ERR_SHAPE;
  if (!(p->D == 16 || p->D == 32 || p->D == 64 || p->D == 128 || p->D == 256)) return FA_ERR_SHAPE;
  if (p->dtype != FA_F16 && p->dtype != FA_BF16) return FA_ERR_DTYPE;
  if (p->bias_kind < FA_BIAS_NONE || p->bias_kind > FA_BIAS_F32) return FA_ERR_DTYPE;
  if (!p->q || !p->k || !p->v || !p->o || !p->lse) return FA_ERR_NULL;
  if (p->bias_kind != FA_BIAS_NONE && !p->bias) return FA_ERR_NULL;
  if ((int64_t)p->B * p->H > 65535) return FA_ERR_TOO_LARGE;
  return FA_OK;
}

int validate_bwd(const fa_params* p) {
  int r = validate_common(p);
  if (r) return r;
  if (!p->d_o || !p->dq || !p->dk || !p->dv || !p->delta) return FA_ERR_NULL;
  if (p->write_dbias) {
    if (p->bias_kind != FA_BIAS_SAME && p->bias_kind != FA_BIAS_F32) return FA_ERR_DTYPE;
    if (!p->dbias) return FA_ERR_NULL;
  }
  if (p->bias_kind == FA_BIAS_F32 && !p->ds16) return FA_ERR_NULL;
  // head dim 256: dQ is always the streamed product over the 16-bit dS
  if (p->D == 256 && !(p->write_dbias && p->bias_kind == FA_BIAS_SAME) && !p->ds16) return FA_ERR_NULL;
  return FA_OK;
}

template <typename F>
int with_device(int device, F&& f) {
  DeviceGuard g(device);
  if (g.err != cudaSuccess) return FA_ERR_CUDA;
  int* status = device_status_ptr(device);
  if (!status) return FA_ERR_CUDA;
  return f(status);
}

}  // namespace
}  // namespace fa

using namespace fa;

extern "C" {

int fa_version(void) { return FA_ABI_VERSION; }

uint64_t fa_launch_count(void) { return g_kernel_launches.load(std::memory_order_relaxed); }

const char* fa_status_string(int code) {
  switch (code) {
    case FA_OK: return "ok";
    case FA_ERR_ABI: return "fa_params.struct_size does not match this library";
    case FA_ERR_NULL: return "a required pointer is null";
    case FA_ERR_SHAPE: return "bad shape (sizes must be >= 1, head dim in {16,32,64,128,256})";
    case FA_ERR_DTYPE: return "bad dtype or bias kind";
    case FA_ERR_ALIGN: return "pointer or stride is not a multiple of 16 bytes";
    case FA_ERR_CUDA: return "a CUDA call failed";
    case FA_ERR_DEVICE_WAIT: return "a kernel abandoned a bounded wait";
    case FA_ERR_UNSUPPORTED: return "not supported by this build";
    case FA_ERR_TOO_LARGE: return "size exceeds a limit of this entry point";
    default: return "unknown error code";
  }
}

int fa_fwd(const fa_params* p, void* stream) {
  int r = validate_common(p);
  if (r) return r;
  return with_device(p->device,
                     [&](int* st) { return launch_fwd(*p, static_cast<cudaStream_t>(stream), st); });
}

int fa_bwd_pre(const fa_params* p, void* stream) {
  int r = validate_bwd(p);
  if (r) return r;
  return with_device(p->device, [&](int* st) {
    return launch_bwd_pre(*p, static_cast<cudaStream_t>(stream), st);
  });
}

int fa_bwd_dkdv(const fa_params* p, void* stream) {
  int r = validate_bwd(p);
  if (r) return r;
  return with_device(p->device, [&](int* st) {
    return launch_bwd_dkdv(*p, static_cast<cudaStream_t>(stream), st);
  });
}

int fa_bwd_dq(const fa_params* p, void* stream) {
  int r = validate_bwd(p);
  if (r) return r;
  return with_device(p->device, [&](int* st) {
    return launch_bwd_dq(*p, static_cast<cudaStream_t>(stream), st);
  });
}

int fa_bwd(const fa_params* p, void* stream) {
  int r = validate_bwd(p);
  if (r) return r;
  return with_device(p->device, [&](int* st) {
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int e = launch_bwd_pre(*p, s, st);
    if (e) return e;
    e = launch_bwd_dkdv(*p, s, st);
    if (e) return e;
    return launch_bwd_dq(*p, s, st);
  });
}

int fa_last_device_status(int device, int32_t out[8]) {
  if (!out) return FA_ERR_NULL;
  return with_device(device, [&](int* st) {
    if (cudaDeviceSynchronize() != cudaSuccess) return (int)FA_ERR_CUDA;
    if (cudaMemcpy(out, st, 8 * sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess)
      return (int)FA_ERR_CUDA;
    return out[0] == 0 ? (int)FA_OK : (int)FA_ERR_DEVICE_WAIT;
  });
}

int fa_reset_device_status(int device) {
  return with_device(device, [&](int* st) {
    if (cudaDeviceSynchronize() != cudaSuccess) return (int)FA_ERR_CUDA;
    // words 6..7 (address of the host copy) stay
    if (cudaMemset(st, 0, 6 * sizeof(int)) != cudaSuccess) return (int)FA_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_status_mu);
    if (volatile int32_t* h = g_mirror_host[device])
      for (int i = 0; i < 6; ++i) h[i] = 0;
    return (int)FA_OK;
  });
}

int fa_set_status_mirror(int device, int32_t* host_words) {
  return with_device(device, [&](int* st) {
    unsigned long long dev_addr = 0;
    if (host_words) {
      void* d = nullptr;
      if (cudaHostGetDevicePointer(&d, host_words, 0) != cudaSuccess) return (int)FA_ERR_CUDA;
      dev_addr = reinterpret_cast<unsigned long long>(d);
      for (int i = 0; i < 8; ++i) host_words[i] = 0;
    }
    if (cudaDeviceSynchronize() != cudaSuccess) return (int)FA_ERR_CUDA;
    if (cudaMemcpy(st + 6, &dev_addr, sizeof(dev_addr), cudaMemcpyHostToDevice) != cudaSuccess)
      return (int)FA_ERR_CUDA;
    std::lock_guard<std::mutex> lock(g_status_mu);
    g_mirror_host[device] = host_words;
    return (int)FA_OK;
  });
}

int fa_selftest_wait_timeout(int device, uint32_t limit_us, void* stream) {
  if (limit_us < 1 || limit_us > 100000) return FA_ERR_SHAPE;
  return with_device(device, [&](int* st) {
    return launch_selftest_timeout(limit_us, static_cast<cudaStream_t>(stream), st);
  });
}

int fa_selftest_umma(int mode, int dtype, const void* a, const void* b, void* c, int device,
                     void* stream) {
  if (!a || !b || !c) return FA_ERR_NULL;
  if (mode < 0 || mode > 4) return FA_ERR_SHAPE;
  if (dtype != FA_F16 && dtype != FA_BF16) return FA_ERR_DTYPE;
  return with_device(device, [&](int* st) {
    return launch_selftest(mode, dtype, a, b, c, static_cast<cudaStream_t>(stream), st);
  });
}

}  // extern "C"
