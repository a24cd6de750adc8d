/*
 * C ABI of libfa_sm100.so: flash-attention forward and backward for NVIDIA B200
 * (sm_100a), with an optional (B,H,M,N) additive bias / bool mask and a bias
 * gradient written at full size.
 *
 * Every entry point takes plain pointers and sizes, enqueues work on the CUDA
 * stream it is given, never synchronises the device (except where noted), never
 * throws and never frees caller memory.  All tensors are owned by the caller.
 * A return value of 0 means "enqueued"; any other value is an fa_error code
 * (fa_status_string() turns it into text).
 *
 * The entry points replace, one for one, the host launchers of the reference
 * project's flash_attention.py (cited per function below as FA:<line>).
 */
#ifndef FA_SM100_H_
#define FA_SM100_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define FA_ABI_VERSION 2

enum fa_dtype { FA_F16 = 0, FA_BF16 = 1 };

/* What the `bias` pointer holds. */
enum fa_bias_kind {
  FA_BIAS_NONE = 0,
  FA_BIAS_SAME = 1, /* float bias in the same 16-bit dtype as q; added to q.k^T*scale      */
  FA_BIAS_BOOL = 2, /* one byte per element; 0 masks the score out, non-zero keeps it      */
  FA_BIAS_F32 = 3   /* fp32 bias with 16-bit q/k/v: streamed as fp32, never rounded to 16 bits;
                       the bias gradient, when asked for, is written in fp32 (FA:52, FA:292, FA:799) */
};

enum fa_error {
  FA_OK = 0,
  FA_ERR_ABI = 1,         /* struct_size does not match this library            */
  FA_ERR_NULL = 2,        /* a required pointer is null                         */
  FA_ERR_SHAPE = 3,       /* a dimension is < 1 or the head dim is unsupported  */
  FA_ERR_DTYPE = 4,       /* unknown dtype / bias kind, or unsupported mix      */
  FA_ERR_ALIGN = 5,       /* a base pointer or stride breaks the 16-byte rule   */
  FA_ERR_CUDA = 6,        /* a CUDA runtime/driver call failed                  */
  FA_ERR_DEVICE_WAIT = 7, /* a kernel gave up a bounded wait (see fa_last_device_status) */
  FA_ERR_UNSUPPORTED = 8, /* legal in the reference, not built in this library
                             (no input reaches it today: every head dim of FA:776 runs) */
  FA_ERR_TOO_LARGE = 9    /* a size exceeds a stated limit of the entry point   */
};

/*
 * One attention problem.  Layouts (element strides; the innermost stride of
 * every tensor must be 1):
 *   q, o, do, dq : (B, M, H, D)  strides {B, M, H}
 *   k, v, dk, dv : (B, N, H, D)  strides {B, N, H}
 *   bias, dbias  : (B, H, M, N)  strides {B, H, M}; a stride of 0 (an expanded
 *                  view) is accepted for B and H of `bias`.  dbias has the bias's
 *                  element type (16-bit for FA_BIAS_SAME, fp32 for FA_BIAS_F32).  With
 *                  FA_BIAS_F32 and causal = 1 the caller zero-fills dbias first: tiles
 *                  above the diagonal are not visited (with FA_BIAS_SAME the library
 *                  writes those zeros itself, except at D = 256, where the caller
 *                  zero-fills a causal dbias of either type)
 *   lse, delta   : (B, H, M) fp32, contiguous
 * Alignment: q/k/v/do base pointers and strides*2 bytes are multiples of 16; the
 * same holds for bias/dbias strides in bytes (the Python layer pads when a row
 * pitch does not qualify).
 */
typedef struct fa_params {
  uint32_t struct_size; /* sizeof(fa_params), checked against the library */
  int32_t device;       /* CUDA device ordinal all pointers live on       */
  int32_t B, H, M, N, D;
  int32_t dtype;       /* fa_dtype of q, k, v, o, do, dq, dk, dv          */
  int32_t bias_kind;   /* fa_bias_kind                                    */
  int32_t causal;      /* 1: key n is visible to query m iff n <= m       */
  int32_t write_dbias; /* backward only: 1 = store dS into dbias          */
  float sm_scale;      /* multiplies q.k^T (not the bias)                 */

  const void* q;
  const void* k;
  const void* v;
  void* o;         /* forward: out; backward: in                          */
  const void* d_o; /* backward in: gradient of o                          */
  void* dq;
  void* dk;
  void* dv;
  const void* bias;
  void* dbias;
  float* lse;   /* forward out / backward in: log2-domain log-sum-exp      */
  float* delta; /* backward scratch: rowsum(o * do), written by fa_bwd_pre */

  int64_t q_stride[3];
  int64_t k_stride[3];
  int64_t v_stride[3];
  int64_t o_stride[3];
  int64_t do_stride[3];
  int64_t dq_stride[3];
  int64_t dk_stride[3];
  int64_t dv_stride[3];
  int64_t bias_stride[3];
  int64_t dbias_stride[3];

  /* Backward with FA_BIAS_F32, and every backward at D = 256 except the one that writes a
   * 16-bit dbias (FA_BIAS_SAME with write_dbias = 1): a (B,H,M,N) scratch tensor in q's 16-bit
   * dtype, required in those cases, ignored otherwise.  The dK/dV stage leaves dS there for
   * the dQ stage (which consumes dS as a 16-bit tensor-core operand, exactly as the reference
   * rounds dS before its dQ product, FA:517).  Same stride rules as dbias.  Contents
   * afterwards: dS rounded to 16 bits at and below the causal diagonal, unspecified above it. */
  void* ds16;
  int64_t ds16_stride[3];
} fa_params;

/* Library / ABI version (FA_ABI_VERSION of the build). */
int fa_version(void);

/*
 * Number of attention kernels this library has launched since it was loaded (forward 1 per
 * call; backward 3: preprocess, dK/dV, dQ).  For benchmarks and tests that must show the
 * work ran here.  No counterpart in the reference.
 */
uint64_t fa_launch_count(void);

/* Text for an fa_error code; never null. */
const char* fa_status_string(int code);

/*
 * Forward: o = softmax(q.k^T * sm_scale + bias, masks) . v and the log2-domain
 * log-sum-exp of every row.  Replaces _flash_attn_fwd (FA:649-685) and the
 * _attn_fwd kernel (FA:88-194); the eager `bias * log2(e)` copy of FA:661-663 is
 * folded into the kernel.
 */
int fa_fwd(const fa_params* p, void* stream);

/*
 * Backward, all three stages in order on `stream`.  Replaces _flash_attn_bwd
 * (FA:688-763): the eager pre-scaled copies of k and bias (FA:699-704) and the
 * zero fill of dbias (FA:799) are folded into the kernels.
 */
int fa_bwd(const fa_params* p, void* stream);

/*
 * Backward for callers that cannot allocate device memory (a plugin living inside a
 * host runtime with a frozen memory plan, a real-time loop, a foreign-language
 * binding without an allocator).  Same as fa_bwd, except that `p->delta` is ignored:
 * the row-sum scratch lives in a fixed 8 MiB device array inside the library.
 *   - limit: B * H * M <= 2,097,152, else FA_ERR_TOO_LARGE;
 *   - the first call on a device resolves the array's device address; make it before
 *     any stream capture starts;
 *   - all calls on a device share the array: calls that overlap on the GPU race,
 *     nothing in it has to be cleared between calls;
 *   - no cudaMalloc / cudaFree or other allocating call is made.
 * This entry point has no counterpart in the reference (its launcher allocates
 * `delta` with torch.empty_like on every call).
 */
int fa_bwd_static_scratch(const fa_params* p, void* stream);

/*
 * The three backward stages on their own (per-kernel timing and tests).  Order matters:
 * fa_bwd_pre writes `delta`, which the other two read; and when write_dbias is 1 with a
 * 16-bit bias, fa_bwd_dq READS `dbias` (it forms dQ from the dS tiles fa_bwd_dkdv has just
 * stored there), so fa_bwd_dkdv must have run on the same stream before it.
 */
int fa_bwd_pre(const fa_params* p, void* stream);  /* _attn_bwd_preprocess FA:197-233 */
int fa_bwd_dkdv(const fa_params* p, void* stream); /* _attn_bwd_dkdv       FA:330-454 */
int fa_bwd_dq(const fa_params* p, void* stream);   /* _attn_bwd_dq         FA:538-646 */

/*
 * Reads the device-side status word of `device` into out[0..7] (synchronises the
 * device).  out[0] != 0 means a kernel abandoned a bounded wait; out[1..5] hold
 * kernel id, block x, block y, wait site and loop iteration.  Returns FA_OK or
 * FA_ERR_DEVICE_WAIT / FA_ERR_CUDA.  No counterpart in the reference.
 */
int fa_last_device_status(int device, int32_t out[8]);

/* Clears the status word of `device` and its host copy (synchronises the device). */
int fa_reset_device_status(int device);

/*
 * Registers `host_words` (8 x int32 of page-locked host memory, e.g. from cudaHostAlloc;
 * NULL to unregister) as a host copy of the status word of `device`: a kernel that abandons
 * a wait writes words 0..5 there as well, so the host can notice the failure by reading
 * host_words[0] before its next call, without synchronising.  The memory stays owned by
 * the caller and must outlive the registration.  Synchronises the device once.  No
 * counterpart in the reference (its kernels have no waits of their own).
 */
int fa_set_status_mirror(int device, int32_t* host_words);

/*
 * Failure-path self-test: launches one CTA that waits, for at most `limit_us`
 * microseconds (1..100000), on a barrier nothing ever completes.  The wait gives up, the
 * kernel returns, and the status word reads {1, kernel 101, block 0, 0, site 7, limit_us}.
 * Every later kernel of the library on this device then does no work until
 * fa_reset_device_status() is called.  Nothing hangs or faults.  No counterpart in the
 * reference.
 */
int fa_selftest_wait_timeout(int device, uint32_t limit_us, void* stream);

/*
 * Self-test of the tensor-core building blocks on one 128x128x128 tile:
 *   mode 0: c = a . b^T            (both operands K-major in shared memory)
 *   mode 1: c = a . b              (b MN-major)
 *   mode 2: c = a^T . b            (both MN-major)
 *   mode 3: c = a . b              (a staged through tensor memory, b MN-major)
 *   mode 4: c16 = a                (shared-memory rewrite + bulk tensor store, 16-bit out)
 * a, b: [128][128] 16-bit row-major device buffers of `dtype`; c: [128][128] fp32
 * (mode 4: 16-bit).  Used by the test-suite to pin descriptor encodings; no
 * counterpart in the reference.
 */
int fa_selftest_umma(int mode, int dtype, const void* a, const void* b, void* c, int device,
                     void* stream);

#ifdef __cplusplus
}
#endif
#endif /* FA_SM100_H_ */
