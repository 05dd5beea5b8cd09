// Device runtime: open/close with explicit errors, a budgeted caching
// allocator, bounded waits, the deferred fault word. Takes the seat of the
// reference's CudaRuntime + AllocBudget (ojas-cuda/src/runtime.rs, budget.rs),
// built ahead of time for sm_100a instead of NVRTC at run time.
#include <chrono>
#include <cstdio>
#include <cstring>
#include <thread>

#include "common.cuh"

static thread_local std::string g_last_error;

static const char* kStatusNames[] = {"Ok", "Shape", "Dtype", "OutOfRange", "NonFinite", "UnsupportedHeadDim",
                                     "CapacityExceeded", "Poisoned", "DeviceLost", "WaitTimeout", "Backend",
                                     "Unsupported", "Placement", "NoDevice"};
static const char* kOpNames[OP_COUNT] = {"none", "embedding", "linear", "rms_norm", "rope", "value_residual_blend",
                                         "causal_sdpa", "per_head_sigmoid_gate", "silu", "mul", "residual_add",
                                         "linear_cross_entropy_mean", "cross_entropy_mean", "accumulate_grad",
                                         "scale_grad", "clip_grad_norm", "adamw_step", "muon_ns5_step", "argmax_rows",
                                         "cast", "gemm_pipeline_wait", "cached_attention_forward", "topk_rows",
                                         "token id or target"};
const char* ojc_op_name(uint32_t op) { return op < OP_COUNT ? kOpNames[op] : "unknown"; }

ojc_status ojc_fail(ojc_status st, const char* op, const std::string& detail) {
  g_last_error = std::string(op) + ": " + detail;
  return st;
}

// Sticky driver errors poison the context: they map to DeviceLost, as in the
// reference's error table (ojas-cuda/src/error.rs:254-290).
static bool sticky(cudaError_t e) {
  switch (e) {
    case cudaErrorIllegalAddress: case cudaErrorLaunchFailure: case cudaErrorIllegalInstruction:
    case cudaErrorMisalignedAddress: case cudaErrorHardwareStackError: case cudaErrorAssert:
    case cudaErrorECCUncorrectable: case cudaErrorDevicesUnavailable: case cudaErrorLaunchTimeout:
      return true;
    default: return false;
  }
}

ojc_status ojc_cuda_check(ojc_backend* be, cudaError_t err, const char* op) {
  if (err == cudaSuccess) return OJC_OK;
  std::string detail = std::string(cudaGetErrorName(err)) + ": " + cudaGetErrorString(err);
  if (sticky(err)) { if (be) be->lost = true; return ojc_fail(OJC_ERR_DEVICE_LOST, op, detail); }
  if (err == cudaErrorMemoryAllocation) { cudaGetLastError(); return ojc_fail(OJC_ERR_CAPACITY_EXCEEDED, op, detail); }
  cudaGetLastError();
  return ojc_fail(OJC_ERR_BACKEND, op, detail);
}

ojc_status check_tensor(const char* op, const char* what, const ojc_tensor* t, bool need_contig) {
  if (!t) return ojc_fail(OJC_ERR_SHAPE, op, std::string(what) + " is null");
  if (t->rank < 0 || t->rank > OJC_MAX_RANK) return ojc_fail(OJC_ERR_SHAPE, op, std::string(what) + ": rank out of range");
  for (int i = 0; i < t->rank; ++i)
    if (t->shape[i] < 0) return ojc_fail(OJC_ERR_SHAPE, op, std::string(what) + ": negative extent");
  if (numel(t) > 0 && !t->data) return ojc_fail(OJC_ERR_PLACEMENT, op, std::string(what) + ": no device storage");
  if (need_contig && !contiguous(t)) return ojc_fail(OJC_ERR_SHAPE, op, std::string(what) + " is not contiguous");
  return OJC_OK;
}

static uint64_t round_block(uint64_t bytes) {
  if (bytes < 512) return 512;
  if (bytes <= (1u << 20)) return (bytes + 511) & ~uint64_t(511);
  return (bytes + (2u << 20) - 1) & ~uint64_t((2u << 20) - 1);
}

static void release_cache(ojc_backend* be) {
  for (auto& kv : be->free_blocks) { cudaFree(kv.second); be->block_size.erase(kv.second); }
  be->free_blocks.clear();
}

extern "C" {

const char* ojc_last_error(void) { return g_last_error.c_str(); }
// FNV-1a over host bytes, continuing from `hash` (the run id of ojas-model/src/trainer.rs:436-456 hashes every parameter)
uint64_t ojc_fnv1a64(uint64_t hash, const void* bytes, uint64_t count) {
  const uint8_t* p = static_cast<const uint8_t*>(bytes);
  for (uint64_t i = 0; i < count; ++i) hash = (hash ^ p[i]) * 0x100000001b3ull;
  return hash;
}

const char* ojc_status_name(int32_t s) { return (s >= 0 && s <= OJC_ERR_NO_DEVICE) ? kStatusNames[s] : "Unknown"; }

ojc_status ojc_open(int32_t ordinal, uint64_t budget_bytes, ojc_backend** out) {
  const char* op = "open";
  if (!out) return ojc_fail(OJC_ERR_BACKEND, op, "null out pointer");
  *out = nullptr;
  int count = 0;
  cudaError_t err = cudaGetDeviceCount(&count);
  if (err != cudaSuccess || count == 0) {
    cudaGetLastError();
    return ojc_fail(OJC_ERR_NO_DEVICE, op, err != cudaSuccess ? std::string("no CUDA device: ") + cudaGetErrorString(err)
                                                              : "no CUDA device is visible");
  }
  if (ordinal < 0 || ordinal >= count) return ojc_fail(OJC_ERR_NO_DEVICE, op, "device ordinal out of range");
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, ordinal) != cudaSuccess) { cudaGetLastError(); return ojc_fail(OJC_ERR_NO_DEVICE, op, "cannot read device properties"); }
  // The kernels are built for sm_100a only; any other part is refused by name, never emulated.
  if (prop.major != 10) {
    char buf[160];
    snprintf(buf, sizeof buf, "device %d is compute capability %d.%d; this library carries sm_100a code only", ordinal, prop.major, prop.minor);
    return ojc_fail(OJC_ERR_UNSUPPORTED, op, buf);
  }
  if (cudaSetDevice(ordinal) != cudaSuccess) { cudaGetLastError(); return ojc_fail(OJC_ERR_NO_DEVICE, op, "cudaSetDevice failed"); }
  ojc_backend* be = new ojc_backend();
  be->device = ordinal;
  be->cap = budget_bytes;
  be->sm_count = prop.multiProcessorCount;
  ojc_status st = OJC_OK;
  if ((st = ojc_cuda_check(be, cudaStreamCreateWithFlags(&be->stream, cudaStreamNonBlocking), op)) != OJC_OK ||
      (st = ojc_cuda_check(be, cudaEventCreateWithFlags(&be->sync_event, cudaEventDisableTiming), op)) != OJC_OK ||
      (st = ojc_cuda_check(be, cudaMalloc(&be->fault_dev, 8), op)) != OJC_OK ||
      (st = ojc_cuda_check(be, cudaMallocHost(&be->fault_host, 8), op)) != OJC_OK ||
      (st = ojc_cuda_check(be, cudaMemsetAsync(be->fault_dev, 0, 8, be->stream), op)) != OJC_OK) {
    ojc_close(be);
    return st == OJC_ERR_BACKEND ? ojc_fail(OJC_ERR_BACKEND, op, "runtime initialisation failed") : st;
  }
  cudaDriverEntryPointQueryResult qres;
  void* fn = nullptr;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess &&
      qres == cudaDriverEntryPointSuccess) be->tmap_encode = fn;
  else cudaGetLastError();
  *out = be;
  return OJC_OK;
}

ojc_status ojc_close(ojc_backend* be) {
  if (!be) return OJC_OK;
  cudaSetDevice(be->device);
  if (be->stream) cudaStreamSynchronize(be->stream);
  for (auto& s : be->gemm_samples) { cudaEventDestroy(s.start); cudaEventDestroy(s.stop); }
  for (auto& e : be->event_pool) { cudaEventDestroy(e.first); cudaEventDestroy(e.second); }
  for (auto& kv : be->live_blocks) cudaFree(kv.first);
  release_cache(be);
  if (be->scratch) cudaFree(be->scratch);
  if (be->fault_dev) cudaFree(be->fault_dev);
  if (be->fault_host) cudaFreeHost(be->fault_host);
  if (be->sync_event) cudaEventDestroy(be->sync_event);
  if (be->stream) cudaStreamDestroy(be->stream);
  cudaGetLastError();
  delete be;
  return OJC_OK;
}

ojc_status ojc_alloc(ojc_backend* be, uint64_t bytes, void** out) {
  const char* op = "alloc";
  OJC_ALIVE(be, op);
  if (!out) return ojc_fail(OJC_ERR_BACKEND, op, "null out pointer");
  *out = nullptr;
  // A refusal, never a clamp: the request is checked against the cap before any device call.
  if (bytes > be->cap || be->live > be->cap - bytes) {
    char buf[160];
    snprintf(buf, sizeof buf, "requested %llu bytes, cap %llu, live %llu", (unsigned long long)bytes,
             (unsigned long long)be->cap, (unsigned long long)be->live);
    return ojc_fail(OJC_ERR_CAPACITY_EXCEEDED, op, buf);
  }
  uint64_t real = round_block(bytes);
  void* ptr = nullptr;
  auto it = be->free_blocks.find(real);
  if (it != be->free_blocks.end()) { ptr = it->second; be->free_blocks.erase(it); }
  else {
    cudaSetDevice(be->device);
    cudaError_t err = cudaMalloc(&ptr, real);
    if (err == cudaErrorMemoryAllocation) { cudaGetLastError(); cudaStreamSynchronize(be->stream); release_cache(be); err = cudaMalloc(&ptr, real); }
    OJC_CUDA(be, err, op);
    be->block_size[ptr] = real;
  }
  be->live_blocks[ptr] = bytes;
  be->live += bytes;
  if (be->live > be->peak) be->peak = be->live;
  *out = ptr;
  return OJC_OK;
}

ojc_status ojc_free(ojc_backend* be, void* ptr) {
  if (!be || !ptr) return OJC_OK;
  auto it = be->live_blocks.find(ptr);
  if (it == be->live_blocks.end()) return ojc_fail(OJC_ERR_BACKEND, "free", "pointer was not allocated by this backend");
  be->live -= it->second;
  be->live_blocks.erase(it);
  // Work already queued on the one stream finishes before any later kernel reuses the block.
  be->free_blocks.emplace(be->block_size[ptr], ptr);
  return OJC_OK;
}

ojc_status ojc_budget(ojc_backend* be, uint64_t* cap, uint64_t* live, uint64_t* peak) {
  if (!be) return ojc_fail(OJC_ERR_BACKEND, "budget", "null backend");
  if (cap) *cap = be->cap;
  if (live) *live = be->live;
  if (peak) *peak = be->peak;
  return OJC_OK;
}
ojc_status ojc_reset_peak(ojc_backend* be) { if (be) be->peak = be->live; return OJC_OK; }
ojc_status ojc_readbacks(ojc_backend* be, uint64_t* count) { if (be && count) *count = be->readbacks; return OJC_OK; }
void* ojc_stream(ojc_backend* be) { return be ? (void*)be->stream : nullptr; }
uint64_t ojc_kernel_launches(ojc_backend* be) { return be ? be->launches : 0; }
ojc_status ojc_set_sync_timeout_ms(ojc_backend* be, uint64_t ms) { if (be) be->sync_timeout_ms = ms; return OJC_OK; }

ojc_status ojc_upload(ojc_backend* be, void* dst, const void* src, uint64_t bytes) {
  OJC_ALIVE(be, "upload");
  if (bytes == 0) return OJC_OK;
  OJC_CUDA(be, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, be->stream), "upload");
  // Pageable sources are staged by the driver before the call returns; pinned ones must outlive the copy,
  // so the upload completes here (the step's per-call cost is a few KB of token ids).
  OJC_CUDA(be, cudaStreamSynchronize(be->stream), "upload");
  return OJC_OK;
}

// Every host wait is bounded: poll the event until the deadline (poll_until,
// ojas-device/src/gpu.rs:17-34). A timeout is retryable; nothing is freed.
static ojc_status bounded_wait(ojc_backend* be, const char* op) {
  OJC_CUDA(be, cudaEventRecord(be->sync_event, be->stream), op);
  auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(be->sync_timeout_ms);
  int spins = 0;
  while (true) {
    cudaError_t q = cudaEventQuery(be->sync_event);
    if (q == cudaSuccess) break;
    if (q != cudaErrorNotReady) return ojc_cuda_check(be, q, op);
    if (std::chrono::steady_clock::now() > deadline) return ojc_fail(OJC_ERR_WAIT_TIMEOUT, op, "the device did not finish within the sync timeout");
    if (++spins > 2000) std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
  return OJC_OK;
}

static ojc_status report_fault(ojc_backend* be, const char* op) {
  uint32_t first = be->fault_host[0];
  if (first == 0) return OJC_OK;
  be->fault_host[0] = be->fault_host[1] = 0;
  cudaMemsetAsync(be->fault_dev, 0, 8, be->stream);
  if (first == OP_ID_RANGE) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "a token id or target on the device is outside the vocabulary");
  if (first == OP_GEMM_WAIT) return ojc_fail(OJC_ERR_WAIT_TIMEOUT, op, "a tensor-pipeline wait inside a GEMM kernel ran out");
  return ojc_fail(OJC_ERR_NON_FINITE, ojc_op_name(first), std::string("non-finite value raised on the device, reported at ") + op);
}

ojc_status ojc_sync(ojc_backend* be) {
  OJC_ALIVE(be, "sync");
  OJC_CUDA(be, cudaMemcpyAsync(be->fault_host, be->fault_dev, 8, cudaMemcpyDeviceToHost, be->stream), "sync");
  OJC_TRY(bounded_wait(be, "sync"));
  return report_fault(be, "sync");
}

ojc_status ojc_download(ojc_backend* be, void* dst, const void* src, uint64_t bytes) {
  OJC_ALIVE(be, "download");
  if (bytes) OJC_CUDA(be, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, be->stream), "download");
  OJC_CUDA(be, cudaMemcpyAsync(be->fault_host, be->fault_dev, 8, cudaMemcpyDeviceToHost, be->stream), "download");
  OJC_TRY(bounded_wait(be, "download"));
  be->readbacks++;
  return report_fault(be, "download");
}

ojc_status ojc_profile_gemm(ojc_backend* be, int32_t enable) {
  OJC_ALIVE(be, "profile_gemm");
  be->profile_gemm = enable != 0;
  return OJC_OK;
}

ojc_status ojc_profile_gemm_read_split(ojc_backend* be, double* plain_ms, double* plain_flops, uint64_t* plain_launches, double* epilogue_ms, double* epilogue_flops,
                                       uint64_t* epilogue_launches) {
  OJC_ALIVE(be, "profile_gemm_read");
  OJC_CUDA(be, cudaStreamSynchronize(be->stream), "profile_gemm_read");
  double ms[2] = {0.0, 0.0}, flops[2] = {0.0, 0.0};
  uint64_t count[2] = {0, 0};
  for (auto& s : be->gemm_samples) {
    float t = 0.0f;
    const int k = s.with_epilogue ? 1 : 0;
    if (cudaEventElapsedTime(&t, s.start, s.stop) == cudaSuccess) ms[k] += t; else cudaGetLastError();
    flops[k] += s.flops;
    ++count[k];
    be->event_pool.emplace_back(s.start, s.stop);
  }
  if (plain_ms) *plain_ms = ms[0];
  if (plain_flops) *plain_flops = flops[0];
  if (plain_launches) *plain_launches = count[0];
  if (epilogue_ms) *epilogue_ms = ms[1];
  if (epilogue_flops) *epilogue_flops = flops[1];
  if (epilogue_launches) *epilogue_launches = count[1];
  be->gemm_samples.clear();
  return OJC_OK;
}

ojc_status ojc_profile_gemm_read(ojc_backend* be, double* total_ms, double* total_flops, uint64_t* launches) {
  double ms[2], flops[2];
  uint64_t count[2];
  OJC_TRY(ojc_profile_gemm_read_split(be, &ms[0], &flops[0], &count[0], &ms[1], &flops[1], &count[1]));
  if (total_ms) *total_ms = ms[0] + ms[1];
  if (total_flops) *total_flops = flops[0] + flops[1];
  if (launches) *launches = count[0] + count[1];
  return OJC_OK;
}

ojc_status ojc_stream_wait_event(ojc_backend* be, void* cuda_stream, void* cuda_event) {
  OJC_ALIVE(be, "stream_wait_event");
  if (!cuda_event) return ojc_fail(OJC_ERR_BACKEND, "stream_wait_event", "null event");
  OJC_CUDA(be, cudaStreamWaitEvent(cuda_stream ? (cudaStream_t)cuda_stream : be->stream, (cudaEvent_t)cuda_event, 0), "stream_wait_event");
  return OJC_OK;
}

ojc_status ojc_fill_zero(ojc_backend* be, void* ptr, uint64_t bytes) {
  OJC_ALIVE(be, "fill_zero");
  if (bytes) OJC_CUDA(be, cudaMemsetAsync(ptr, 0, bytes, be->stream), "fill_zero");
  return OJC_OK;
}

}  // extern "C"

ojc_status ojc_partials(ojc_backend* be, uint64_t bytes, void** out, bool* on_lane) {
  ojc_backend::FinishLane& f = be->finish;
  const uint64_t need = (bytes + 255) & ~uint64_t(255);
  *on_lane = f.active && f.stream != be->stream && f.used + need <= f.pool_bytes;
  if (!*on_lane) return ojc_scratch(be, bytes, out);
  *out = f.pool + f.used;
  f.used += need;
  return OJC_OK;
}

ojc_status ojc_finish_stream(ojc_backend* be, bool on_lane, cudaStream_t* stream) {
  *stream = be->stream;
  if (!on_lane) return OJC_OK;
  OJC_CUDA(be, cudaEventRecord(be->finish.ev, be->stream), "finish_lane");
  OJC_CUDA(be, cudaStreamWaitEvent(be->finish.stream, be->finish.ev, 0), "finish_lane");
  *stream = be->finish.stream;
  return OJC_OK;
}

ojc_status ojc_scratch(ojc_backend* be, uint64_t bytes, void** out) {
  if (bytes > be->scratch_bytes) {
    // The old workspace may still be read by queued kernels: drain the stream before replacing it.
    OJC_CUDA(be, cudaStreamSynchronize(be->stream), "scratch");
    if (be->scratch) cudaFree(be->scratch);
    be->scratch = nullptr; be->scratch_bytes = 0;
    uint64_t want = (bytes + (1u << 20) - 1) & ~uint64_t((1u << 20) - 1);
    cudaError_t err = cudaMalloc(&be->scratch, want);
    if (err == cudaErrorMemoryAllocation) { cudaGetLastError(); release_cache(be); err = cudaMalloc(&be->scratch, want); }
    OJC_CUDA(be, err, "scratch");
    be->scratch_bytes = want;
  }
  *out = be->scratch;
  return OJC_OK;
}
