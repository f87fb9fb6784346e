// Shared host-side plumbing for the vkgrad_b200 C ABI: the device object, the
// thread-local error string, and launch checking.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <mutex>
#include <vector>

#include "../../include/vkgrad_b200.h"

// Error codes written by kernels into vkg_device::err_flag (host-mapped).
#define VKG_ERR_WAIT_TIMEOUT 1u   // a bounded mbarrier wait gave up

// One deferred final pass: out[c / D][c % D] (+)= sum over nchunk rows of partial[k][c], c < W,
// with up to three destinations of D columns each (W = D, 2 D or 3 D).
struct vkg_final_entry {
  const float* partial;
  float* dst[3];
  int W, D, nchunk, accumulate;
  int first_block, reserved;
};

struct vkg_device {
  int ordinal = 0;
  cudaStream_t stream = nullptr;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  int sm_count = 0;
  int cc_major = 0, cc_minor = 0;
  size_t total_bytes = 0;
  char name[128] = {0};
  // Host-mapped words kernels can write: [0] error code, [1] detail.
  volatile uint32_t* err_host = nullptr;
  uint32_t* err_dev = nullptr;
  bool capturing = false;
  // cuTensorMapEncodeTiled, resolved at run time so the library loads on a
  // machine without a driver.
  void* encode_tiled = nullptr;
  size_t gemm_smem_optin = 0;
  // cudaFuncSetAttribute(MaxDynamicSharedMemorySize) is per device: one flag per kernel family
  bool gemm_attr_set = false;
  bool group_attr_set = false;
  bool attn_fwd_attr_set = false;
  bool attn_bwd_attr_set = false;
  // programmatic dependent launch for the kernels of a training step (vkg_set_pdl)
  // GEMM epilogues without fused reads store C through tensor maps (VKG_TMA_STORE=0: per lane)
  bool tma_store = true;
  bool pdl = false;
  unsigned pdl_mask = 0xffffffffu;   // kernel families (VKG_K_*) it applies to
  // While a communicator is attached, host waits on this device poll against a deadline
  // instead of blocking: a collective whose peer never arrives must not hang the process.
  // on_async_error returns non-zero (and sets the error text) when the communicator reports a
  // failure; on_abort tears the communicator down so the stream can drain.
  void* wait_ctx = nullptr;
  int (*on_async_error)(void* ctx) = nullptr;
  void (*on_abort)(void* ctx) = nullptr;
  double wait_timeout_s = 60.0;
  std::vector<void*> comms;          // communicators attached to this device (comm.cu)
  // Persistent kernels (GEMMs, grouped GEMMs, attention backward) launch at most this many
  // CTAs; 0 = one per SM.  Lowered while a collective runs beside the compute stream so that
  // the collective's CTAs find free SMs instead of delaying a statically scheduled grid.
  int sm_limit = 0;
  // fused attention forward: one pass with a lazily rescaled running maximum (default), or
  // the two-pass kernel (VKG_TUNE_ATTN_ONE_PASS)
  bool attn_one_pass = true;
  bool pair192 = true;        // vkg_gemm may pick 256 x 192 CTA-pair tiles for N = 768-like outputs
  // vkg_gemm takes 256 x 256 CTA-pair tiles on its own (cta_pair == 0) from this many
  // tiles per CTA pair on, in tenths (VKG_TUNE_PAIR_MIN_WAVES)
  int pair_min_waves_x10 = 60;
  // vkg_finals_defer / vkg_finals_flush: final passes of two-stage column sums collected
  // instead of launched, then run as one launch
  bool defer_finals = false;
  std::vector<vkg_final_entry> finals;
};

static inline int vkg_persistent_ctas(const vkg_device* dev) {
  return dev->sm_limit > 0 && dev->sm_limit < dev->sm_count ? dev->sm_limit : dev->sm_count;
}

struct vkg_graph {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  int kernel_nodes = 0;
};

void vkg_set_error(const char* fmt, ...);

// The deadline loop of every host wait (runtime.cu).  query() returns 0 when the work is done,
// 1 when it is still running, anything else on a failure it has already described with
// vkg_set_error.  Without an abort hook the loop is a plain blocking wait on `query`.
struct vkg_wait_hooks {
  int (*query)(void* ctx);
  void* query_ctx;
  int (*async_error)(void* ctx);
  void (*abort)(void* ctx);
  void* comm_ctx;
  double timeout_s;
};
int vkg_wait_with_deadline(const vkg_wait_hooks* h, const char* what);
// Waits for the device's stream (ev == nullptr) or for an event recorded on it.
int vkg_wait_device(vkg_device* dev, cudaEvent_t ev, const char* what);

// ops.cu: sums[c] (+)= sum over nchunk rows of partial[k][c], rows added in a fixed order;
// collected for vkg_finals_flush while vkg_finals_defer is on
int vkg_launch_col_sum_final(vkg_device* dev, const float* partial, float* sums, int ncol, int nchunk,
                             int accumulate);

#define VKG_FAIL(...)            \
  do {                           \
    vkg_set_error(__VA_ARGS__);  \
    return 1;                    \
  } while (0)

#define VKG_CUDA(expr)                                                          \
  do {                                                                          \
    cudaError_t _e = (expr);                                                    \
    if (_e != cudaSuccess) {                                                    \
      vkg_set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),     \
                    __FILE__, __LINE__);                                        \
      return 1;                                                                 \
    }                                                                           \
  } while (0)

#define VKG_REQUIRE(cond, ...)   \
  do {                           \
    if (!(cond)) {               \
      vkg_set_error(__VA_ARGS__);\
      return 1;                  \
    }                            \
  } while (0)

// Makes `dev` current on this thread and checks the launch that just happened.
static inline int vkg_bind(vkg_device* dev) {
  if (!dev) {
    vkg_set_error("null device");
    return 1;
  }
  cudaError_t e = cudaSetDevice(dev->ordinal);
  if (e != cudaSuccess) {
    vkg_set_error("cudaSetDevice(%d): %s", dev->ordinal, cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

static inline int vkg_check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    vkg_set_error("launch of %s failed: %s", what, cudaGetErrorString(e));
    return 1;
  }
  return 0;
}

static inline unsigned vkg_blocks(int64_t n, int per_block, int64_t cap = (1ll << 31) - 1) {
  int64_t b = (n + per_block - 1) / per_block;
  if (b < 1) b = 1;
  if (b > cap) b = cap;
  return (unsigned)b;
}

// ---- programmatic dependent launch ------------------------------------------
//
// A kernel launched through vkg_launch() may become resident while the kernel before it on
// the stream is still draining: its CTAs take the SMs the predecessor's last CTAs leave, run
// their prologue (barrier set-up, TMEM allocation, tensor-map prefetch) and then block in
// pdl_wait() until the predecessor has completed and its writes are visible.  Rules every such
// kernel keeps: pdl_wait() is executed by every thread before its first global-memory access
// (loads, stores and TMA alike, so neither RAW nor WAR hazards arise), also by threads that
// would return early -- a kernel that could complete without waiting would let ITS successor
// overtake the predecessor; pdl_trigger() may come first, it only allows the successor to be
// scheduled once every CTA of this grid has started.  Both are no-ops for a plain launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() {
#ifndef VKG_PDL_NO_TRIGGER
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}

// Launch on the device's stream, with the programmatic-serialisation attribute when the
// device has it switched on (and `cluster` > 1 for a thread-block cluster along x).
enum : unsigned {
  VKG_K_GEMM = 1, VKG_K_GEMM_PAIR = 2, VKG_K_GEMM_GROUP = 4, VKG_K_ATTN_FWD = 8, VKG_K_ATTN_BWD = 16,
  VKG_K_LN = 32, VKG_K_LN_BWD = 64, VKG_K_CE = 128, VKG_K_ADAMW = 256, VKG_K_SMALL = 512
};

template <typename... KArgs, typename... Args>
static inline cudaError_t vkg_launch(vkg_device* dev, unsigned family, void (*kernel)(KArgs...),
                                     dim3 grid, dim3 block, size_t smem, int cluster, Args&&... args) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = dev->stream;
  cudaLaunchAttribute attr[2];
  memset(attr, 0, sizeof(attr));
  int n = 0;
  if (cluster > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = (unsigned)cluster;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (dev->pdl && (dev->pdl_mask & family)) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = (unsigned)n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- device helpers shared by the elementwise kernels ----------------------

// GELU in its tanh form (kernels.py:624-636) written through the logistic function:
//   0.5 x (1 + tanh(u)) = x * s,   s = 1 / (1 + e^{-2u}),   u = c (x + a x^3)
//   d/dx               = s + x s (1 - s) * 2c (1 + 3a x^2)
// Algebraically identical, no cancellation, and 7 / 10 instructions (one ex2 and one
// rcp on the special-function unit) instead of libm tanhf: the GEMM epilogues that call
// these are instruction-issue bound.
__device__ __forceinline__ float vkg_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float vkg_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// s = 1 / (1 + exp(-2 c (x + a x^3))), with -2 c log2(e) folded into the polynomial
__device__ __forceinline__ float vkg_gelu_gate(float x, float x2) {
  const float k1 = -2.0f * 0.7978845608028654f * 1.4426950408889634f;
  const float k3 = k1 * 0.044715f;
  return vkg_rcp(1.0f + vkg_ex2(x * fmaf(x2, k3, k1)));
}

__device__ __forceinline__ float vkg_gelu(float x) {
  return x * vkg_gelu_gate(x, x * x);
}

__device__ __forceinline__ float vkg_dgelu(float x) {
  const float c2 = 2.0f * 0.7978845608028654f;
  const float x2 = x * x;
  const float s = vkg_gelu_gate(x, x2);
  const float w = fmaf(x2, c2 * 3.0f * 0.044715f, c2);   // 2c (1 + 3a x^2)
  return fmaf(x * fmaf(-s, s, s), w, s);
}

__device__ __forceinline__ float vkg_act(float v, int act) {
  if (act == VKG_ACT_GELU) return vkg_gelu(v);
  if (act == VKG_ACT_RELU) return v > 0.0f ? v : 0.0f;
  return v;
}

__device__ __forceinline__ float vkg_dact(float z, int act) {
  if (act == VKG_ACT_GELU) return vkg_dgelu(z);
  if (act == VKG_ACT_RELU) return z > 0.0f ? 1.0f : 0.0f;
  return 1.0f;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
