// Shared declarations of the sm_100a library: the backend object, status and
// fault plumbing, tensor-descriptor checks and small device helpers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/ojas_cuda.h"

typedef __nv_bfloat16 bf16;

// Op ids written into the deferred fault word (first faulting op wins), in the
// spirit of the reference's fault.wgsl / deferred-fault contract
// (ojas-core/src/backend.rs:963-973).
// Grids whose block count is also the number of partial sums of a reduction are sized from this constant (the B200's SM count),
// not from the opened device: the order a gradient is summed in, and so its bits, is then a function of the shape alone
// (the reference's rule for its device kernels: grid a function of shape, ojas-cuda/README.md:131-134).
constexpr int REDUCE_SMS = 148;

// Function attributes (dynamic shared-memory limits, cluster occupancy) belong to a device, not to the process: a flag or a
// value cached for them is kept per device ordinal, so a second backend opened on another GPU sets its own.
constexpr int OJC_MAX_DEVICES = 64;
struct PerDeviceFlag { bool set[OJC_MAX_DEVICES] = {}; bool& operator[](int device) { return set[(unsigned)device % OJC_MAX_DEVICES]; } };
struct PerDeviceInt { int v[OJC_MAX_DEVICES]; explicit PerDeviceInt(int init) { for (int& x : v) x = init; } int& operator[](int device) { return v[(unsigned)device % OJC_MAX_DEVICES]; } };

enum OjcOp : uint32_t {
  OP_NONE = 0, OP_EMBEDDING, OP_LINEAR, OP_RMS_NORM, OP_ROPE, OP_VRES, OP_SDPA, OP_GATE, OP_SILU, OP_MUL,
  OP_ADD, OP_LINEAR_CE, OP_CE, OP_ACCUMULATE, OP_SCALE, OP_CLIP, OP_ADAMW, OP_MUON, OP_ARGMAX, OP_CAST, OP_GEMM_WAIT,
  OP_CACHED_ATTN, OP_TOPK,
  OP_ID_RANGE,  // a token id or target outside the vocabulary: reported as OutOfRange
  OP_COUNT
};
const char* ojc_op_name(uint32_t op);

struct ojc_backend {
  int device = 0;
  cudaStream_t stream = nullptr;
  cudaEvent_t sync_event = nullptr;
  uint64_t cap = 0, live = 0, peak = 0, readbacks = 0, launches = 0;
  uint64_t sync_timeout_ms = 60000;
  bool lost = false;                       // a sticky CUDA error was seen: every later call is DeviceLost
  uint32_t* fault_dev = nullptr;           // [0] first op id, [1] op mask
  uint32_t* fault_host = nullptr;          // pinned
  std::unordered_map<void*, uint64_t> live_blocks;            // ptr -> charged bytes
  std::unordered_map<void*, uint64_t> block_size;             // ptr -> real (rounded) bytes
  std::multimap<uint64_t, void*> free_blocks;                 // rounded bytes -> ptr
  void* scratch = nullptr;                 // grows on demand; library-internal workspace (not charged to the caller's tensors)
  uint64_t scratch_bytes = 0;
  int sm_count = 148;                      // the opened device's; sizes persistent grids only (never a reduction's partial count, see REDUCE_SMS)
  void* tmap_encode = nullptr;             // cuTensorMapEncodeTiled, resolved once
  bool profile_gemm = false;               // bracket tensor-core GEMM launches with events
  struct GemmSample { cudaEvent_t start, stop; double flops; bool with_epilogue; };   // with_epilogue: the launch also ran SwiGLU in its epilogue
  std::vector<GemmSample> gemm_samples;
  std::vector<std::pair<cudaEvent_t, cudaEvent_t>> event_pool;
  // Finishing lane for two-stage reductions (per-block partials, then a few blocks that sum them into a weight gradient).
  // The finishing kernels are tiny and nothing reads their result before the optimizer, so a step driver may point this
  // at a second stream: the partials then come from the lane's own pool (the main workspace is reused by the next op) and
  // the finishing kernel runs on the lane's stream behind an event. The owner resets `used` wherever it joins the lane.
  struct FinishLane { cudaStream_t stream = nullptr; cudaEvent_t ev = nullptr; char* pool = nullptr; uint64_t pool_bytes = 0, used = 0; bool active = false; } finish;
};

ojc_status ojc_fail(ojc_status st, const char* op, const std::string& detail);
ojc_status ojc_cuda_check(ojc_backend* be, cudaError_t err, const char* op);
// Library workspace of at least `bytes` (256-byte aligned); contents are undefined.
ojc_status ojc_scratch(ojc_backend* be, uint64_t bytes, void** out);
// Workspace for the partials of a two-stage reduction and the stream its finishing kernel goes on. Without an active
// finishing lane (or when its pool is full) that is the main workspace and the main stream. With one, call
// ojc_finish_stream after the producing kernel was launched: it orders the lane behind the main stream's work so far.
ojc_status ojc_partials(ojc_backend* be, uint64_t bytes, void** out, bool* on_lane);
ojc_status ojc_finish_stream(ojc_backend* be, bool on_lane, cudaStream_t* stream);

#define OJC_TRY(expr) do { ojc_status st__ = (expr); if (st__ != OJC_OK) return st__; } while (0)
#define OJC_CUDA(be, expr, op) OJC_TRY(ojc_cuda_check((be), (expr), (op)))
#define OJC_LAUNCHED(be, op) do { (be)->launches++; OJC_TRY(ojc_cuda_check((be), cudaGetLastError(), (op))); } while (0)
#define OJC_ALIVE(be, op) do { if (!(be)) return ojc_fail(OJC_ERR_BACKEND, (op), "null backend"); \
    if ((be)->lost) return ojc_fail(OJC_ERR_DEVICE_LOST, (op), "the device was lost earlier"); } while (0)

// ---- tensor descriptor helpers
inline int64_t numel(const ojc_tensor* t) { int64_t n = 1; for (int i = 0; i < t->rank; ++i) n *= t->shape[i]; return n; }
inline bool contiguous(const ojc_tensor* t) {
  int64_t expect = 1;
  for (int i = t->rank - 1; i >= 0; --i) { if (t->shape[i] != 1 && t->stride[i] != expect) return false; expect *= t->shape[i]; }
  return true;
}
inline bool same_shape(const ojc_tensor* a, const ojc_tensor* b) {
  if (a->rank != b->rank) return false;
  for (int i = 0; i < a->rank; ++i) if (a->shape[i] != b->shape[i]) return false;
  return true;
}
inline size_t dtype_size(int32_t dt) { return dt == OJC_BF16 || dt == OJC_F16 ? 2 : 4; }
inline bool is_float(const ojc_tensor* t) { return t->dtype == OJC_F32 || t->dtype == OJC_BF16; }
ojc_status check_tensor(const char* op, const char* what, const ojc_tensor* t, bool need_contig = true);

// ---- device helpers
#ifdef __CUDACC__
__device__ __forceinline__ float ldf(const float* p, int64_t i) { return p[i]; }
__device__ __forceinline__ float ldf(const bf16* p, int64_t i) { return __bfloat162float(p[i]); }
__device__ __forceinline__ void stf(float* p, int64_t i, float v) { p[i] = v; }
__device__ __forceinline__ void stf(bf16* p, int64_t i, float v) { p[i] = __float2bfloat16_rn(v); }

// bf16 round-to-nearest-even on the integer bits; NaN keeps sign + payload and
// sets the quiet bit (ojas-core/src/autocast.rs:89-96).
__device__ __forceinline__ uint16_t f32_to_bf16_bits(float v) {
  uint32_t bits = __float_as_uint(v);
  if ((bits & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((bits >> 16) | 0x0040u);
  uint32_t round = 0x7FFFu + ((bits >> 16) & 1u);
  return (uint16_t)((bits + round) >> 16);
}
__device__ __forceinline__ float round_bf16(float v) { return __uint_as_float((uint32_t)f32_to_bf16_bits(v) << 16); }

__device__ __forceinline__ void raise_fault(uint32_t* fault, uint32_t op) {
  atomicCAS(&fault[0], 0u, op);
  atomicOr(&fault[1], 1u << (op & 31u));
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
// Block-wide sum in a fixed order (warp butterflies, then warp 0 over the warp
// partials): every thread returns the total. `red` holds >= 32 floats.
// Lets a kernel launched after this one with programmatic stream serialization (the tensor-core GEMMs are) set itself up on SMs
// this kernel's CTAs have already left; such a kernel touches no global memory before this one is complete. A no-op otherwise.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? red[lane] : 0.0f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < nwarps) ? red[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
#endif

// Grid for a grid-stride elementwise kernel: enough CTAs to fill the GPU, a
// multiple of the SM count.
inline int elementwise_grid(const ojc_backend* be, int64_t work_items, int threads) {
  int64_t blocks = (work_items + threads - 1) / threads;
  int64_t cap = (int64_t)be->sm_count * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}
