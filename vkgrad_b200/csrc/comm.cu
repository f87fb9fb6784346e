// Data-parallel gradient exchange: NCCL all-reduce over NVLink / NVSwitch in
// place of the reference's shared host arena + float atomicAdd
// (dataparallel.py:40-47, 119-126).  NCCL is opened with dlopen at first use so
// the library loads (and single-GPU work runs) on a machine without it.
#include <dlfcn.h>

#include <climits>

#include "common.cuh"

namespace {

typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
enum { NCCL_SUM = 0, NCCL_MAX = 2 };
enum { NCCL_FLOAT16 = 6, NCCL_FLOAT32 = 7, NCCL_FLOAT64 = 8, NCCL_BFLOAT16 = 9 };

struct NcclApi {
  void* handle = nullptr;
  int (*GetUniqueId)(ncclUniqueId*) = nullptr;
  int (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  int (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, void*) = nullptr;
  int (*CommDestroy)(ncclComm_t) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  const char* (*GetLastError)(ncclComm_t) = nullptr;
  int (*CommAbort)(ncclComm_t) = nullptr;
  int (*CommGetAsyncError)(ncclComm_t, int*) = nullptr;
};

// ncclConfig_t as NCCL 2.18 laid it out (later releases only append fields and accept the
// shorter structure, told apart by `size` and `version`).  Unset fields carry INT_MIN / NULL.
struct NcclConfig218 {
  size_t size;
  unsigned int magic;
  unsigned int version;
  int blocking;
  int cgaClusterSize;
  int minCTAs;
  int maxCTAs;
  const char* netName;
  int splitShare;
};

NcclApi g_nccl;
std::mutex g_nccl_mu;

int load_nccl() {
  std::lock_guard<std::mutex> lock(g_nccl_mu);
  if (g_nccl.handle) return 0;
  const char* names[] = {"libnccl.so.2", "libnccl.so"};
  void* h = nullptr;
  for (const char* n : names) {
    // RTLD_NOLOAD first: reuse a copy the process already holds.
    h = dlopen(n, RTLD_NOW | RTLD_NOLOAD);
    if (!h) h = dlopen(n, RTLD_NOW | RTLD_LOCAL);
    if (h) break;
  }
  if (!h) {
    vkg_set_error("NCCL not found (libnccl.so.2): %s", dlerror());
    return 1;
  }
  NcclApi api;
  api.handle = h;
  api.GetUniqueId = (int (*)(ncclUniqueId*))dlsym(h, "ncclGetUniqueId");
  api.CommInitRank = (int (*)(ncclComm_t*, int, ncclUniqueId, int))dlsym(h, "ncclCommInitRank");
  api.CommInitRankConfig =
      (int (*)(ncclComm_t*, int, ncclUniqueId, int, void*))dlsym(h, "ncclCommInitRankConfig");
  api.CommDestroy = (int (*)(ncclComm_t))dlsym(h, "ncclCommDestroy");
  api.AllReduce = (int (*)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t))dlsym(
      h, "ncclAllReduce");
  api.GetErrorString = (const char* (*)(int))dlsym(h, "ncclGetErrorString");
  api.GetLastError = (const char* (*)(ncclComm_t))dlsym(h, "ncclGetLastError");
  api.CommAbort = (int (*)(ncclComm_t))dlsym(h, "ncclCommAbort");
  api.CommGetAsyncError = (int (*)(ncclComm_t, int*))dlsym(h, "ncclCommGetAsyncError");
  if (!api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllReduce ||
      !api.GetErrorString) {
    vkg_set_error("libnccl is missing a required symbol");
    return 1;
  }
  g_nccl = api;
  return 0;
}

}  // namespace

constexpr int VKG_COMM_SLOTS = 16;

struct vkg_comm {
  vkg_device* dev = nullptr;
  ncclComm_t comm = nullptr;
  int rank = 0, nranks = 1;
  double* scratch_dev = nullptr;
  // a second stream for collectives that run beside the compute stream, and the events that
  // order the two (created at first use)
  cudaStream_t side = nullptr;
  cudaEvent_t ev_fork = nullptr;
  cudaEvent_t ev_done[VKG_COMM_SLOTS] = {};
};

// Hooks the device's host waits call while this communicator is attached (common.cuh).
// ctx is the device; every communicator attached to it is checked / aborted.
static int comm_async_error(void* ctx) {
  vkg_device* dev = static_cast<vkg_device*>(ctx);
  for (void* v : dev->comms) {
    vkg_comm* c = static_cast<vkg_comm*>(v);
    if (!c->comm || !g_nccl.CommGetAsyncError) continue;
    int state = 0;
    if (g_nccl.CommGetAsyncError(c->comm, &state) != 0 || state != 0) {
      vkg_set_error("NCCL reported an asynchronous error: %s",
                    g_nccl.GetErrorString ? g_nccl.GetErrorString(state) : "?");
      return 1;
    }
  }
  return 0;
}

static void comm_abort(void* ctx) {
  vkg_device* dev = static_cast<vkg_device*>(ctx);
  for (void* v : dev->comms) {
    vkg_comm* c = static_cast<vkg_comm*>(v);
    if (c->comm && g_nccl.CommAbort) g_nccl.CommAbort(c->comm);
    else if (c->comm) g_nccl.CommDestroy(c->comm);
    c->comm = nullptr;     // every later collective on it fails instead of hanging
  }
}

#define VKG_NCCL(expr)                                                              \
  do {                                                                              \
    int _r = (expr);                                                                \
    if (_r != 0) {                                                                  \
      vkg_set_error("%s failed: %s", #expr, g_nccl.GetErrorString(_r));             \
      return 1;                                                                     \
    }                                                                               \
  } while (0)

extern "C" int vkg_comm_unique_id(uint8_t id[128]) {
  if (!id) VKG_FAIL("null id");
  if (load_nccl()) return 1;
  ncclUniqueId uid;
  VKG_NCCL(g_nccl.GetUniqueId(&uid));
  memcpy(id, uid.internal, 128);
  return 0;
}

extern "C" int vkg_comm_create(vkg_device* dev, int rank, int nranks, const uint8_t id[128],
                               vkg_comm** out) {
  return vkg_comm_create_limited(dev, rank, nranks, id, 0, out);
}

extern "C" int vkg_comm_create_limited(vkg_device* dev, int rank, int nranks, const uint8_t id[128],
                                       int max_ctas, vkg_comm** out) {
  if (vkg_bind(dev)) return 1;
  VKG_REQUIRE(out && id, "comm_create: null argument");
  VKG_REQUIRE(nranks >= 1 && rank >= 0 && rank < nranks, "comm_create: rank %d of %d", rank, nranks);
  if (load_nccl()) return 1;
  ncclUniqueId uid;
  memcpy(uid.internal, id, 128);
  vkg_comm* c = new vkg_comm();
  c->dev = dev;
  c->rank = rank;
  c->nranks = nranks;
  int r;
  if (max_ctas > 0) {
    if (!g_nccl.CommInitRankConfig) {
      delete c;
      VKG_FAIL("comm_create: this NCCL has no ncclCommInitRankConfig (needed for max_ctas)");
    }
    NcclConfig218 cfg;
    cfg.size = sizeof(cfg);
    cfg.magic = 0xcafebeefu;
    cfg.version = 21800;
    cfg.blocking = cfg.cgaClusterSize = cfg.minCTAs = cfg.splitShare = INT_MIN;
    cfg.maxCTAs = max_ctas;
    cfg.netName = nullptr;
    r = g_nccl.CommInitRankConfig(&c->comm, nranks, uid, rank, &cfg);
  } else {
    r = g_nccl.CommInitRank(&c->comm, nranks, uid, rank);
  }
  if (r != 0) {
    delete c;
    VKG_FAIL("ncclCommInitRank failed: %s", g_nccl.GetErrorString(r));
  }
  cudaError_t e = cudaMalloc(&c->scratch_dev, 64);
  if (e != cudaSuccess) {
    g_nccl.CommDestroy(c->comm);
    delete c;
    VKG_FAIL("comm_create: %s", cudaGetErrorString(e));
  }
  // One small collective now, outside any capture: NCCL sets its channels up lazily
  // on the first call, which allocates and synchronises.
  cudaMemsetAsync(c->scratch_dev, 0, 64, dev->stream);
  r = g_nccl.AllReduce(c->scratch_dev, c->scratch_dev, 1, NCCL_FLOAT64, NCCL_MAX, c->comm, dev->stream);
  e = cudaStreamSynchronize(dev->stream);
  if (r != 0 || e != cudaSuccess) {
    cudaFree(c->scratch_dev);
    g_nccl.CommDestroy(c->comm);
    delete c;
    VKG_FAIL("comm_create: first collective failed (%s / %s)", r ? g_nccl.GetErrorString(r) : "ok",
             cudaGetErrorString(e));
  }
  dev->comms.push_back(c);
  dev->wait_ctx = dev;
  dev->on_async_error = comm_async_error;
  dev->on_abort = comm_abort;
  *out = c;
  return 0;
}

extern "C" int vkg_comm_destroy(vkg_comm* comm) {
  if (!comm) return 0;
  if (comm->dev) {
    std::vector<void*>& v = comm->dev->comms;
    for (size_t i = 0; i < v.size(); ++i)
      if (v[i] == comm) {
        v.erase(v.begin() + i);
        break;
      }
    if (v.empty()) {
      comm->dev->wait_ctx = nullptr;
      comm->dev->on_async_error = nullptr;
      comm->dev->on_abort = nullptr;
    }
  }
  if (comm->dev) cudaSetDevice(comm->dev->ordinal);
  if (comm->dev) cudaStreamSynchronize(comm->dev->stream);
  if (comm->side) {
    cudaStreamSynchronize(comm->side);
    for (int i = 0; i < VKG_COMM_SLOTS; ++i)
      if (comm->ev_done[i]) cudaEventDestroy(comm->ev_done[i]);
    if (comm->ev_fork) cudaEventDestroy(comm->ev_fork);
    cudaStreamDestroy(comm->side);
  }
  if (comm->scratch_dev) cudaFree(comm->scratch_dev);
  if (comm->comm) g_nccl.CommDestroy(comm->comm);
  delete comm;
  return 0;
}

extern "C" int vkg_allreduce_sum(vkg_comm* comm, void* buf, int64_t count, int dtype) {
  VKG_REQUIRE(comm && buf && count > 0, "allreduce: bad arguments");
  VKG_REQUIRE(comm->comm, "allreduce: the communicator was aborted");
  if (vkg_bind(comm->dev)) return 1;
  int t = dtype == VKG_F32 ? NCCL_FLOAT32 : dtype == VKG_F16 ? NCCL_FLOAT16 : dtype == VKG_BF16 ? NCCL_BFLOAT16 : -1;
  VKG_REQUIRE(t >= 0, "allreduce: unknown dtype %d", dtype);
  VKG_NCCL(g_nccl.AllReduce(buf, buf, (size_t)count, t, NCCL_SUM, comm->comm, comm->dev->stream));
  return 0;
}

// ---- collectives beside the compute stream -------------------------------------------------
//
// vkg_comm_side_begin: everything enqueued on the device's stream so far happens before what
// follows on the side stream.  vkg_allreduce_sum_side: the all-reduce on the side stream;
// `slot` names the event that marks its end.  vkg_comm_side_wait: the device's stream waits
// for that event -- so a finished part of the bucket is summed while the backward of the
// blocks below still runs, and the optimiser starts on the parts that have arrived.
static int side_init(vkg_comm* comm) {
  if (comm->side) return 0;
  VKG_CUDA(cudaStreamCreateWithFlags(&comm->side, cudaStreamNonBlocking));
  VKG_CUDA(cudaEventCreateWithFlags(&comm->ev_fork, cudaEventDisableTiming));
  for (int i = 0; i < VKG_COMM_SLOTS; ++i)
    VKG_CUDA(cudaEventCreateWithFlags(&comm->ev_done[i], cudaEventDisableTiming));
  return 0;
}

extern "C" int vkg_comm_side_begin(vkg_comm* comm) {
  VKG_REQUIRE(comm, "comm_side_begin: null communicator");
  if (vkg_bind(comm->dev)) return 1;
  if (side_init(comm)) return 1;
  VKG_CUDA(cudaEventRecord(comm->ev_fork, comm->dev->stream));
  VKG_CUDA(cudaStreamWaitEvent(comm->side, comm->ev_fork, 0));
  return 0;
}

extern "C" int vkg_allreduce_sum_side(vkg_comm* comm, void* buf, int64_t count, int dtype, int slot) {
  VKG_REQUIRE(comm && buf && count > 0 && slot >= 0 && slot < VKG_COMM_SLOTS,
              "allreduce_side: bad arguments (slot 0..%d)", VKG_COMM_SLOTS - 1);
  VKG_REQUIRE(comm->comm, "allreduce_side: the communicator was aborted");
  if (vkg_bind(comm->dev)) return 1;
  if (side_init(comm)) return 1;
  int t = dtype == VKG_F32 ? NCCL_FLOAT32 : dtype == VKG_F16 ? NCCL_FLOAT16 : dtype == VKG_BF16 ? NCCL_BFLOAT16 : -1;
  VKG_REQUIRE(t >= 0, "allreduce_side: unknown dtype %d", dtype);
  VKG_NCCL(g_nccl.AllReduce(buf, buf, (size_t)count, t, NCCL_SUM, comm->comm, comm->side));
  VKG_CUDA(cudaEventRecord(comm->ev_done[slot], comm->side));
  return 0;
}

extern "C" int vkg_comm_side_wait(vkg_comm* comm, int slot) {
  VKG_REQUIRE(comm && comm->side && slot >= 0 && slot < VKG_COMM_SLOTS, "comm_side_wait: bad arguments");
  if (vkg_bind(comm->dev)) return 1;
  VKG_CUDA(cudaStreamWaitEvent(comm->dev->stream, comm->ev_done[slot], 0));
  return 0;
}

extern "C" int vkg_comm_max_double(vkg_comm* comm, double* value) {
  VKG_REQUIRE(comm && value, "comm_max_double: bad arguments");
  VKG_REQUIRE(comm->comm, "comm_max_double: the communicator was aborted");
  if (vkg_bind(comm->dev)) return 1;
  cudaStream_t s = comm->dev->stream;
  VKG_CUDA(cudaMemcpyAsync(comm->scratch_dev, value, sizeof(double), cudaMemcpyHostToDevice, s));
  VKG_NCCL(g_nccl.AllReduce(comm->scratch_dev, comm->scratch_dev, 1, NCCL_FLOAT64, NCCL_MAX,
                            comm->comm, s));
  VKG_CUDA(cudaMemcpyAsync(value, comm->scratch_dev, sizeof(double), cudaMemcpyDeviceToHost, s));
  return vkg_wait_device(comm->dev, nullptr, "comm_max_double");
}

extern "C" int vkg_comm_barrier(vkg_comm* comm) {
  double v = 0.0;
  return vkg_comm_max_double(comm, &v);
}
