// Runtime half of the C ABI: device, memory kinds, copies, event timing and
// CUDA-graph record/replay.  Stands where the reference's Vulkan runtime stood
// (vk.Device / vk.Buffer / vk.Graph); nothing here computes.
#include "common.cuh"

#include <cstdlib>

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
  snprintf(d->name, sizeof(d->name), "%s", prop.name);
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
  d->pdl = !(pdl && pdl[0] == '0');
  *out = d;
  return 0;
}

extern "C" int vkg_set_pdl(vkg_device* dev, int on) {
  if (!dev) VKG_FAIL("null device");
  VKG_REQUIRE(!dev->capturing, "set_pdl: not while a graph is being recorded");
  dev->pdl = on != 0;
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

extern "C" int vkg_sync(vkg_device* dev) {
  if (vkg_bind(dev)) return 1;
  VKG_CUDA(cudaStreamSynchronize(dev->stream));
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
  VKG_CUDA(cudaStreamSynchronize(dev->stream));
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
  VKG_CUDA(cudaEventSynchronize(dev->ev1));
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
  VKG_CUDA(cudaEventSynchronize(dev->ev1));
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
