// Runtime half of the C ABI: device, memory kinds, copies, event timing and
// CUDA-graph record/replay.  Stands where the reference's Vulkan runtime stood
// (vk.Device / vk.Buffer / vk.Graph); nothing here computes.
#include "common.cuh"

#include <chrono>
#include <cstdlib>
#include <thread>

static thread_local char g_err[1024] = "";

void vkg_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

extern "C" const char* vkg_last_error(void) { return g_err; }

extern "C" const char* vkg_version(void) { return "vkgrad_b200 0.1 (sm_100a)"; }

extern "C" int vkg_device_count(int* count) {
  if (!count) VKG_FAIL("null count");
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    cudaGetLastError();
    n = 0;
  }
  *count = n;
  return 0;
}

extern "C" int vkg_device_create(int ordinal, vkg_device** out) {
  if (!out) VKG_FAIL("null out");
  *out = nullptr;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
    cudaGetLastError();
    VKG_FAIL("no CUDA device is visible; this library has no CPU fallback");
  }
  VKG_REQUIRE(ordinal >= 0 && ordinal < n, "device ordinal %d out of range (%d devices)",
              ordinal, n);
  VKG_CUDA(cudaSetDevice(ordinal));
  cudaDeviceProp prop;
  VKG_CUDA(cudaGetDeviceProperties(&prop, ordinal));
  VKG_REQUIRE(prop.major == 10,
              "device %d is compute capability %d.%d; this library is built for sm_100a only",
              ordinal, prop.major, prop.minor);
  vkg_device* d = new vkg_device();
  d->ordinal = ordinal;
  d->sm_count = prop.multiProcessorCount;
  d->cc_major = prop.major;
  d->cc_minor = prop.minor;
  d->total_bytes = prop.totalGlobalMem;
  d->gemm_smem_optin = prop.sharedMemPerBlockOptin;
  snprintf(d->name, sizeof(d->name), "%.127s", prop.name);
  VKG_CUDA(cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking));
  VKG_CUDA(cudaEventCreate(&d->ev0));
  VKG_CUDA(cudaEventCreate(&d->ev1));
  void* host = nullptr;
  VKG_CUDA(cudaHostAlloc(&host, 64, cudaHostAllocMapped | cudaHostAllocPortable));
  memset(host, 0, 64);
  d->err_host = (volatile uint32_t*)host;
  VKG_CUDA(cudaHostGetDevicePointer((void**)&d->err_dev, host, 0));
  cudaDriverEntryPointQueryResult qres;
  void* fn = nullptr;
  cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
  if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !fn) {
    cudaGetLastError();
    delete d;
    VKG_FAIL("cuTensorMapEncodeTiled is not available from this driver");
  }
  d->encode_tiled = fn;
  const char* pdl = getenv("VKG_PDL");
  d->pdl = pdl && pdl[0] == '1';    // off unless asked for: it measured slower inside CUDA graphs
  const char* ts = getenv("VKG_TMA_STORE");
  d->tma_store = !(ts && ts[0] == '0');
  const char* a1 = getenv("VKG_ATTN_ONE_PASS");
  if (a1 && a1[0]) d->attn_one_pass = a1[0] == '1';
  const char* lim = getenv("VKG_SM_LIMIT");      // persistent kernels' grid cap, for experiments
  if (lim && lim[0]) d->sm_limit = atoi(lim);
  const char* mask = getenv("VKG_PDL_MASK");     // kernel families, for experiments
  if (mask && mask[0]) d->pdl_mask = (unsigned)strtoul(mask, nullptr, 0);
  *out = d;
  return 0;
}

extern "C" int vkg_set_pdl(vkg_device* dev, int on) {
  if (!dev) VKG_FAIL("null device");
  VKG_REQUIRE(!dev->capturing, "set_pdl: not while a graph is being recorded");
  dev->pdl = on != 0;
  return 0;
}

extern "C" int vkg_set_tuning(vkg_device* dev, int key, int64_t value) {
  if (!dev) VKG_FAIL("null device");
  // the SM limit is host state read when a launch is enqueued: it may change between the
  // launches of one recording
  VKG_REQUIRE(!dev->capturing || key == VKG_TUNE_SM_LIMIT,
              "set_tuning: not while a graph is being recorded");
  switch (key) {
    case VKG_TUNE_PDL: dev->pdl = value != 0; break;
    case VKG_TUNE_PDL_FAMILIES: dev->pdl_mask = (unsigned)value; break;
    case VKG_TUNE_TMA_STORE: dev->tma_store = value != 0; break;
    case VKG_TUNE_SM_LIMIT:
      VKG_REQUIRE(value >= 0, "set_tuning: the SM limit cannot be negative");
      dev->sm_limit = (int)value;
      break;
    case VKG_TUNE_PAIR_MIN_WAVES:
      VKG_REQUIRE(value >= 0, "set_tuning: the threshold cannot be negative");
      dev->pair_min_waves_x10 = (int)value;
      break;
    case VKG_TUNE_ATTN_ONE_PASS: dev->attn_one_pass = value != 0; break;
    case VKG_TUNE_PAIR_192: dev->pair192 = value != 0; break;
    case VKG_TUNE_WAIT_TIMEOUT_MS:
      VKG_REQUIRE(value > 0, "set_tuning: the wait limit must be positive");
      dev->wait_timeout_s = (double)value * 1e-3;
      break;
    default: VKG_FAIL("set_tuning: unknown key %d", key);
  }
  return 0;
}

extern "C" int vkg_device_destroy(vkg_device* dev) {
  if (!dev) return 0;
  cudaSetDevice(dev->ordinal);
  cudaStreamSynchronize(dev->stream);
  if (dev->ev0) cudaEventDestroy(dev->ev0);
  if (dev->ev1) cudaEventDestroy(dev->ev1);
  if (dev->err_host) cudaFreeHost((void*)dev->err_host);
  if (dev->stream) cudaStreamDestroy(dev->stream);
  delete dev;
  return 0;
}

extern "C" int vkg_device_info(vkg_device* dev, char* name, size_t name_cap, int* sm_count,
                               size_t* total_bytes, int* cc_major, int* cc_minor) {
  if (!dev) VKG_FAIL("null device");
  if (name && name_cap) snprintf(name, name_cap, "%s", dev->name);
  if (sm_count) *sm_count = dev->sm_count;
  if (total_bytes) *total_bytes = dev->total_bytes;
  if (cc_major) *cc_major = dev->cc_major;
  if (cc_minor) *cc_minor = dev->cc_minor;
  return 0;
}

extern "C" void* vkg_device_stream(vkg_device* dev) { return dev ? (void*)dev->stream : nullptr; }

static int check_err_flag(vkg_device* dev) {
  uint32_t code = dev->err_host[0];
  if (code != 0) {
    uint32_t detail = dev->err_host[1];
    dev->err_host[0] = 0;
    dev->err_host[1] = 0;
    VKG_FAIL("kernel reported error %u (detail 0x%x): a bounded device-side wait gave up",
             code, detail);
  }
  return 0;
}

// ---- host waits ------------------------------------------------------------------------
//
// The reference turns a fence that does not signal within 10 s into VkError (vk.py:884-888,
// 1335-1339).  Here a step can hang only in a collective whose peer never arrives, so waits
// on a device with a communicator poll against a deadline; on expiry the communicator is
// aborted (which lets the stream drain) and the call fails.
int vkg_wait_with_deadline(const vkg_wait_hooks* h, const char* what) {
  const auto t0 = std::chrono::steady_clock::now();
  for (long long polls = 0;; ++polls) {
    const int q = h->query(h->query_ctx);
    if (q == 0) return 0;
    if (q != 1) return 1;
    if (h->async_error && (polls & 63) == 63 && h->async_error(h->comm_ctx)) {
      if (h->abort) h->abort(h->comm_ctx);
      return 1;
    }
    const double waited = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if (h->abort && waited > h->timeout_s) {
      h->abort(h->comm_ctx);
      vkg_set_error("%s: the device did not finish within %.1f s (a collective whose peer never "
                    "arrived?); the communicator was aborted", what, h->timeout_s);
      return 1;
    }
    // spin for the first 200 us (a training step's tail), then yield the core
    if (waited > 200e-6) std::this_thread::sleep_for(std::chrono::microseconds(waited > 0.05 ? 500 : 20));
  }
}

namespace {
struct DeviceQuery {
  vkg_device* dev;
  cudaEvent_t ev;
};
int query_device(void* ctx) {
  DeviceQuery* q = static_cast<DeviceQuery*>(ctx);
  cudaError_t e = q->ev ? cudaEventQuery(q->ev) : cudaStreamQuery(q->dev->stream);
  if (e == cudaSuccess) return 0;
  if (e == cudaErrorNotReady) {
    cudaGetLastError();
    return 1;
  }
  vkg_set_error("device wait failed: %s", cudaGetErrorString(e));
  return 2;
}
}  // namespace

int vkg_wait_device(vkg_device* dev, cudaEvent_t ev, const char* what) {
  if (!dev->on_abort) {          // no communicator: nothing can hang, block in the driver
    if (ev) VKG_CUDA(cudaEventSynchronize(ev));
    else VKG_CUDA(cudaStreamSynchronize(dev->stream));
    return 0;
  }
  DeviceQuery q{dev, ev};
  vkg_wait_hooks h{query_device, &q, dev->on_async_error, dev->on_abort, dev->wait_ctx,
                   dev->wait_timeout_s};
  return vkg_wait_with_deadline(&h, what);
}

// The deadline loop against a scripted device, for tests without a GPU: the "stream" reports
// done after ready_after_polls queries (never, if negative), the "communicator" reports an
// asynchronous error from its async_error_at-th check on (never, if negative).  *aborted
// receives how often the abort hook ran.
namespace {
struct FakeWait {
  long long polls, ready_after, checks, error_at;
  int aborted;
};
int fake_query(void* ctx) {
  FakeWait* f = static_cast<FakeWait*>(ctx);
  return (f->ready_after >= 0 && f->polls++ >= f->ready_after) ? 0 : 1;
}
int fake_async_error(void* ctx) {
  FakeWait* f = static_cast<FakeWait*>(ctx);
  if (f->error_at >= 0 && f->checks++ >= f->error_at) {
    vkg_set_error("communicator reported an asynchronous error (scripted)");
    return 1;
  }
  return 0;
}
void fake_abort(void* ctx) { static_cast<FakeWait*>(ctx)->aborted++; }
}  // namespace

extern "C" int vkg_selftest_wait_deadline(int64_t ready_after_polls, int64_t async_error_at,
                                          double timeout_s, int* aborted) {
  FakeWait f{0, ready_after_polls, 0, async_error_at, 0};
  vkg_wait_hooks h{fake_query, &f, fake_async_error, fake_abort, &f, timeout_s};
  const int rc = vkg_wait_with_deadline(&h, "selftest");
  if (aborted) *aborted = f.aborted;
  return rc;
}

extern "C" int vkg_sync(vkg_device* dev) {
  if (vkg_bind(dev)) return 1;
  if (vkg_wait_device(dev, nullptr, "sync")) return 1;
  return check_err_flag(dev);
}

extern "C" int vkg_alloc(vkg_device* dev, size_t bytes, int kind, void** dptr, void** hptr) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(dptr && hptr, "null output pointer");
  *dptr = nullptr;
  *hptr = nullptr;
  if (bytes == 0) bytes = 16;
  if (kind == 0) {
    VKG_CUDA(cudaMalloc(dptr, bytes));
  } else if (kind == 1) {
    VKG_CUDA(cudaHostAlloc(hptr, bytes, cudaHostAllocMapped | cudaHostAllocPortable));
    memset(*hptr, 0, bytes);
    VKG_CUDA(cudaHostGetDevicePointer(dptr, *hptr, 0));
  } else if (kind == 2) {
    VKG_CUDA(cudaMalloc(dptr, bytes));
    cudaError_t e = cudaHostAlloc(hptr, bytes, cudaHostAllocPortable);
    if (e != cudaSuccess) {
      cudaFree(*dptr);
      *dptr = nullptr;
      VKG_FAIL("cudaHostAlloc(%zu) failed: %s", bytes, cudaGetErrorString(e));
    }
    memset(*hptr, 0, bytes);
  } else {
    VKG_FAIL("unknown memory kind %d", kind);
  }
  return 0;
}

extern "C" int vkg_free(vkg_device* dev, void* dptr, void* hptr, int kind) {
  if (vkg_bind(dev)) return 1;
  if (kind == 0) {
    if (dptr) VKG_CUDA(cudaFree(dptr));
  } else if (kind == 1) {
    if (hptr) VKG_CUDA(cudaFreeHost(hptr));
  } else if (kind == 2) {
    if (dptr) VKG_CUDA(cudaFree(dptr));
    if (hptr) VKG_CUDA(cudaFreeHost(hptr));
  } else {
    VKG_FAIL("unknown memory kind %d", kind);
  }
  return 0;
}

extern "C" int vkg_upload(vkg_device* dev, void* dptr, const void* hptr, size_t bytes) {
  if (vkg_bind(dev)) return 1;
  VKG_CUDA(cudaMemcpyAsync(dptr, hptr, bytes, cudaMemcpyHostToDevice, dev->stream));
  VKG_CUDA(cudaStreamSynchronize(dev->stream));
  return 0;
}

extern "C" int vkg_download(vkg_device* dev, void* hptr, const void* dptr, size_t bytes) {
  if (vkg_bind(dev)) return 1;
  VKG_CUDA(cudaMemcpyAsync(hptr, dptr, bytes, cudaMemcpyDeviceToHost, dev->stream));
  if (vkg_wait_device(dev, nullptr, "download")) return 1;
  return check_err_flag(dev);
}

extern "C" int vkg_copy(vkg_device* dev, void* dst, const void* src, size_t bytes) {
  if (vkg_bind(dev)) return 1;
  VKG_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDefault, dev->stream));
  return 0;
}

extern "C" int vkg_copy_h2d_async(vkg_device* dev, void* dptr, const void* hptr, size_t bytes) {
  if (vkg_bind(dev)) return 1;
  VKG_CUDA(cudaMemcpyAsync(dptr, hptr, bytes, cudaMemcpyHostToDevice, dev->stream));
  return 0;
}

extern "C" int vkg_copy_d2h_async(vkg_device* dev, void* hptr, const void* dptr, size_t bytes) {
  if (vkg_bind(dev)) return 1;
  VKG_CUDA(cudaMemcpyAsync(hptr, dptr, bytes, cudaMemcpyDeviceToHost, dev->stream));
  return 0;
}

extern "C" int vkg_memset0(vkg_device* dev, void* dptr, size_t bytes) {
  if (vkg_bind(dev)) return 1;
  VKG_CUDA(cudaMemsetAsync(dptr, 0, bytes, dev->stream));
  return 0;
}

extern "C" int vkg_timer_begin(vkg_device* dev) {
  if (vkg_bind(dev)) return 1;
  VKG_CUDA(cudaEventRecord(dev->ev0, dev->stream));
  return 0;
}

extern "C" int vkg_timer_end(vkg_device* dev, double* seconds) {
  if (vkg_bind(dev)) return 1;
  VKG_CUDA(cudaEventRecord(dev->ev1, dev->stream));
  if (vkg_wait_device(dev, dev->ev1, "timer_end")) return 1;
  float ms = 0.f;
  VKG_CUDA(cudaEventElapsedTime(&ms, dev->ev0, dev->ev1));
  if (seconds) *seconds = (double)ms * 1e-3;
  return check_err_flag(dev);
}

extern "C" int vkg_graph_begin(vkg_device* dev) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(!dev->capturing, "a graph is already being recorded on this device");
  VKG_CUDA(cudaStreamBeginCapture(dev->stream, cudaStreamCaptureModeThreadLocal));
  dev->capturing = true;
  return 0;
}

extern "C" int vkg_graph_end(vkg_device* dev, vkg_graph** out) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(out, "null out");
  VKG_REQUIRE(dev->capturing, "no graph is being recorded");
  dev->capturing = false;
  cudaGraph_t graph = nullptr;
  VKG_CUDA(cudaStreamEndCapture(dev->stream, &graph));
  VKG_REQUIRE(graph != nullptr, "capture produced no graph (an enqueue failed during recording)");
  vkg_graph* g = new vkg_graph();
  g->graph = graph;
  size_t n = 0;
  if (cudaGraphGetNodes(graph, nullptr, &n) == cudaSuccess && n > 0) {
    std::vector<cudaGraphNode_t> nodes(n);
    if (cudaGraphGetNodes(graph, nodes.data(), &n) == cudaSuccess) {
      for (size_t i = 0; i < n; ++i) {
        cudaGraphNodeType t;
        if (cudaGraphNodeGetType(nodes[i], &t) == cudaSuccess && t == cudaGraphNodeTypeKernel)
          g->kernel_nodes++;
      }
    }
  }
  cudaError_t e = cudaGraphInstantiate(&g->exec, graph, 0);
  if (e != cudaSuccess) {
    cudaGraphDestroy(graph);
    delete g;
    VKG_FAIL("cudaGraphInstantiate failed: %s", cudaGetErrorString(e));
  }
  *out = g;
  return 0;
}

extern "C" int vkg_graph_launch(vkg_device* dev, vkg_graph* g, double* seconds) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(g && g->exec, "graph is not finished");
  VKG_CUDA(cudaEventRecord(dev->ev0, dev->stream));
  VKG_CUDA(cudaGraphLaunch(g->exec, dev->stream));
  VKG_CUDA(cudaEventRecord(dev->ev1, dev->stream));
  if (vkg_wait_device(dev, dev->ev1, "graph_launch")) return 1;
  float ms = 0.f;
  VKG_CUDA(cudaEventElapsedTime(&ms, dev->ev0, dev->ev1));
  if (seconds) *seconds = (double)ms * 1e-3;
  return check_err_flag(dev);
}

extern "C" int vkg_graph_launch_async(vkg_device* dev, vkg_graph* g) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(g && g->exec, "graph is not finished");
  VKG_CUDA(cudaGraphLaunch(g->exec, dev->stream));
  return 0;
}

extern "C" int vkg_graph_destroy(vkg_graph* g) {
  if (!g) return 0;
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  delete g;
  return 0;
}

extern "C" int vkg_graph_kernel_count(vkg_graph* g, int* count) {
  VKG_REQUIRE(g && count, "null argument");
  *count = g->kernel_nodes;
  return 0;
}
