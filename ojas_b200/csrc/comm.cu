// Data-parallel exchange behind the C ABI: a communicator over NCCL, reached with dlopen so that the library itself links
// nothing but the CUDA runtime. New with this backend: the reference has no distributed code; the semantics it has to keep
// are those of K-micro-batch accumulation (ojas-model/src/trainer.rs:916-1001): every rank's backward is seeded 1/world,
// the f32 gradients are summed, then every rank runs the same clip and optimizer and holds the same bits.
//
// One communicator per backend, one stream of its own. A gradient bucket is all-reduced as soon as the event the step driver
// records behind the bucket's last gradient fires, so the exchange runs under the rest of backward; the backend's stream
// only waits for the last collective. Only NCCL's own kernels touch peer memory.
#include <dlfcn.h>

#include <chrono>
#include <thread>

#include "common.cuh"

namespace {

// The handful of NCCL entry points used, with the library's own value for each enum constant named here.
typedef struct ncclComm* nccl_comm_t;
typedef struct { char internal[128]; } nccl_unique_id;
enum { NCCL_SUCCESS = 0, NCCL_IN_PROGRESS = 7 };
enum { NCCL_SUM = 0, NCCL_MAX = 2, NCCL_MIN = 3 };
enum { NCCL_UINT64 = 5, NCCL_FLOAT32 = 7, NCCL_BFLOAT16 = 9 };

struct NcclApi {
  void* handle = nullptr;
  int (*GetUniqueId)(nccl_unique_id*) = nullptr;
  int (*CommInitRank)(nccl_comm_t*, int, nccl_unique_id, int) = nullptr;
  int (*CommDestroy)(nccl_comm_t) = nullptr;
  int (*CommAbort)(nccl_comm_t) = nullptr;
  int (*CommGetAsyncError)(nccl_comm_t, int*) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
  int (*Broadcast)(const void*, void*, size_t, int, int, nccl_comm_t, cudaStream_t) = nullptr;
  int (*GroupStart)() = nullptr;
  int (*GroupEnd)() = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
  std::string error;
};

NcclApi& nccl() {
  static NcclApi api;
  static bool tried = false;
  if (tried) return api;
  tried = true;
  // a copy the process already holds first (a host that also uses NCCL elsewhere must share it), then the loader's search path
  api.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);
  if (!api.handle) api.handle = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!api.handle) { api.error = std::string("libnccl.so.2 cannot be loaded: ") + (dlerror() ? dlerror() : "not found"); return api; }
  auto sym = [&](const char* name) -> void* {
    void* p = dlsym(api.handle, name);
    if (!p && api.error.empty()) api.error = std::string("libnccl.so.2 lacks ") + name;
    return p;
  };
  api.GetUniqueId = (decltype(api.GetUniqueId))sym("ncclGetUniqueId");
  api.CommInitRank = (decltype(api.CommInitRank))sym("ncclCommInitRank");
  api.CommDestroy = (decltype(api.CommDestroy))sym("ncclCommDestroy");
  api.CommAbort = (decltype(api.CommAbort))sym("ncclCommAbort");
  api.CommGetAsyncError = (decltype(api.CommGetAsyncError))sym("ncclCommGetAsyncError");
  api.AllReduce = (decltype(api.AllReduce))sym("ncclAllReduce");
  api.Broadcast = (decltype(api.Broadcast))sym("ncclBroadcast");
  api.GroupStart = (decltype(api.GroupStart))sym("ncclGroupStart");
  api.GroupEnd = (decltype(api.GroupEnd))sym("ncclGroupEnd");
  api.GetErrorString = (decltype(api.GetErrorString))sym("ncclGetErrorString");
  return api;
}

ojc_status nccl_check(int rc, const char* op) {
  if (rc == NCCL_SUCCESS) return OJC_OK;
  const char* text = nccl().GetErrorString ? nccl().GetErrorString(rc) : "unknown";
  return ojc_fail(OJC_ERR_BACKEND, op, std::string("NCCL: ") + text);
}

}  // namespace

struct ojc_comm {
  ojc_backend* be = nullptr;
  nccl_comm_t comm = nullptr;
  int rank = 0, world = 1;
  cudaStream_t stream = nullptr;
  cudaEvent_t done = nullptr, fork = nullptr;
};

extern "C" {

ojc_status ojc_comm_unique_id(uint8_t* id128) {
  const char* op = "comm_unique_id";
  if (!id128) return ojc_fail(OJC_ERR_BACKEND, op, "null id");
  NcclApi& api = nccl();
  if (!api.error.empty()) return ojc_fail(OJC_ERR_UNSUPPORTED, op, api.error);
  nccl_unique_id id;
  OJC_TRY(nccl_check(api.GetUniqueId(&id), op));
  memcpy(id128, id.internal, 128);
  return OJC_OK;
}

ojc_status ojc_comm_init(ojc_backend* be, int32_t rank, int32_t world, const uint8_t* id128, ojc_comm** out) {
  const char* op = "comm_init";
  OJC_ALIVE(be, op);
  if (!id128 || !out) return ojc_fail(OJC_ERR_BACKEND, op, "null argument");
  *out = nullptr;
  if (world < 1 || rank < 0 || rank >= world) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "rank must be in [0, world)");
  NcclApi& api = nccl();
  if (!api.error.empty()) return ojc_fail(OJC_ERR_UNSUPPORTED, op, api.error);
  ojc_comm* c = new ojc_comm();
  c->be = be; c->rank = rank; c->world = world;
  cudaSetDevice(be->device);
  nccl_unique_id id;
  memcpy(id.internal, id128, 128);
  ojc_status st = nccl_check(api.CommInitRank(&c->comm, world, id, rank), op);
  if (st == OJC_OK && (cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking) != cudaSuccess ||
                       cudaEventCreateWithFlags(&c->done, cudaEventDisableTiming) != cudaSuccess ||
                       cudaEventCreateWithFlags(&c->fork, cudaEventDisableTiming) != cudaSuccess))
    st = ojc_fail(OJC_ERR_BACKEND, op, "cannot create the exchange stream");
  if (st != OJC_OK) { ojc_comm_destroy(c); return st; }
  *out = c;
  return OJC_OK;
}

ojc_status ojc_comm_destroy(ojc_comm* c) {
  if (!c) return OJC_OK;
  if (c->stream) cudaStreamSynchronize(c->stream);
  if (c->comm) nccl().CommDestroy(c->comm);
  if (c->stream) cudaStreamDestroy(c->stream);
  if (c->done) cudaEventDestroy(c->done);
  if (c->fork) cudaEventDestroy(c->fork);
  delete c;
  return OJC_OK;
}

int32_t ojc_comm_rank(ojc_comm* c) { return c ? c->rank : 0; }
int32_t ojc_comm_world(ojc_comm* c) { return c ? c->world : 1; }

// An error NCCL found on its own threads since the last call (a peer that went away, a transport fault). Never blocks.
ojc_status ojc_comm_check(ojc_comm* c) {
  const char* op = "comm_check";
  if (!c) return ojc_fail(OJC_ERR_BACKEND, op, "null communicator");
  int async = NCCL_SUCCESS;
  OJC_TRY(nccl_check(nccl().CommGetAsyncError(c->comm, &async), op));
  if (async != NCCL_SUCCESS && async != NCCL_IN_PROGRESS) return nccl_check(async, op);
  return OJC_OK;
}

ojc_status ojc_allreduce_start(ojc_comm* c, ojc_trainer* tr) {
  const char* op = "allreduce_start";
  if (!c || !tr) return ojc_fail(OJC_ERR_BACKEND, op, "null argument");
  OJC_ALIVE(c->be, op);
  NcclApi& api = nccl();
  const int64_t n = ojc_trainer_bucket_count(tr);
  for (int64_t i = 0; i < n; ++i) {
    void *ptr = nullptr, *ev = nullptr;
    uint64_t floats = 0;
    OJC_TRY(ojc_trainer_bucket(tr, i, &ptr, &floats));
    OJC_TRY(ojc_trainer_bucket_ready_event(tr, i, &ev));
    OJC_CUDA(c->be, cudaStreamWaitEvent(c->stream, (cudaEvent_t)ev, 0), op);
    OJC_TRY(nccl_check(api.AllReduce(ptr, ptr, (size_t)floats, NCCL_FLOAT32, NCCL_SUM, c->comm, c->stream), op));
  }
  OJC_CUDA(c->be, cudaEventRecord(c->done, c->stream), op);
  return OJC_OK;
}

ojc_status ojc_allreduce_wait(ojc_comm* c, ojc_trainer* tr) {
  const char* op = "allreduce_wait";
  (void)tr;
  if (!c) return ojc_fail(OJC_ERR_BACKEND, op, "null communicator");
  OJC_ALIVE(c->be, op);
  OJC_CUDA(c->be, cudaStreamWaitEvent(c->be->stream, c->done, 0), op);   // the device waits; the host does not
  return ojc_comm_check(c);
}

// In-place collectives on device memory, ordered on the backend's own stream (loss mean, counts, checksums, parameter broadcasts).
ojc_status ojc_comm_allreduce(ojc_comm* c, void* data, uint64_t count, int32_t dtype, int32_t op_kind) {
  const char* op = "comm_allreduce";
  if (!c || !data) return ojc_fail(OJC_ERR_BACKEND, op, "null argument");
  OJC_ALIVE(c->be, op);
  const int dt = dtype == OJC_F32 ? NCCL_FLOAT32 : dtype == OJC_BF16 ? NCCL_BFLOAT16 : -1;
  const int red = op_kind == 0 ? NCCL_SUM : op_kind == 1 ? NCCL_MAX : op_kind == 2 ? NCCL_MIN : -1;
  if (dt < 0 || red < 0) return ojc_fail(OJC_ERR_UNSUPPORTED, op, "F32 or BF16 data; op 0 sum, 1 max, 2 min");
  OJC_TRY(nccl_check(nccl().AllReduce(data, data, (size_t)count, dt, red, c->comm, c->be->stream), op));
  return ojc_comm_check(c);
}

ojc_status ojc_comm_broadcast_many(ojc_comm* c, void* const* ptrs, const uint64_t* counts, const int32_t* roots, int64_t n, int32_t dtype) {
  const char* op = "comm_broadcast";
  if (!c || (n > 0 && (!ptrs || !counts || !roots))) return ojc_fail(OJC_ERR_BACKEND, op, "null argument");
  OJC_ALIVE(c->be, op);
  const int dt = dtype == OJC_F32 ? NCCL_FLOAT32 : dtype == OJC_BF16 ? NCCL_BFLOAT16 : -1;
  if (dt < 0) return ojc_fail(OJC_ERR_UNSUPPORTED, op, "F32 or BF16 data");
  NcclApi& api = nccl();
  OJC_TRY(nccl_check(api.GroupStart(), op));
  ojc_status st = OJC_OK;
  for (int64_t i = 0; i < n && st == OJC_OK; ++i) {
    if (roots[i] < 0 || roots[i] >= c->world) st = ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "root outside the communicator");
    else st = nccl_check(api.Broadcast(ptrs[i], ptrs[i], (size_t)counts[i], dt, roots[i], c->comm, c->be->stream), op);
  }
  ojc_status end = nccl_check(api.GroupEnd(), op);
  return st != OJC_OK ? st : end;
}

}  // extern "C"
