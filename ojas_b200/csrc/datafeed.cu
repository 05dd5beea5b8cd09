// Token windows out of a token stream that is resident in device memory: the device half of the data feed.
// The host keeps the sampler (which window comes next is a keyed permutation, ojas-data/src/sampler.rs:292-318); the stream
// itself sits in HBM once (u16 or u32 tokens as stored in the file), and a step's batch costs B window starts of host->device
// traffic instead of 2 x B x T ids: x[r] = tokens[start_r .. start_r + T), y[r] = tokens[start_r + 1 .. start_r + T + 1)
// (ojas-data/src/sampler.rs:245-290), widened to U32.
#include "common.cuh"

namespace {

constexpr int ROWS_PER_LAUNCH = 256;
struct WindowStarts { int64_t start[ROWS_PER_LAUNCH]; };

template <class TT>
__global__ void token_windows_kernel(const TT* __restrict__ tokens, const WindowStarts ws, int rows, int seq, uint32_t* __restrict__ x, uint32_t* __restrict__ y) {
  const int r = blockIdx.y;
  if (r >= rows) return;
  const TT* src = tokens + ws.start[r];
  uint32_t* xr = x + (int64_t)r * seq;
  uint32_t* yr = y + (int64_t)r * seq;
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i <= seq; i += gridDim.x * blockDim.x) {
    const uint32_t t = (uint32_t)src[i];
    if (i < seq) xr[i] = t;
    if (i > 0) yr[i - 1] = t;
  }
}

}  // namespace

extern "C" ojc_status ojc_gather_token_windows(ojc_backend* be, const void* tokens, int32_t bytes_per_token, uint64_t n_tokens, const int64_t* starts_host,
                                               int64_t rows, int64_t seq, ojc_tensor* x, ojc_tensor* y) {
  const char* op = "gather_token_windows";
  OJC_ALIVE(be, op);
  if (!tokens || !starts_host) return ojc_fail(OJC_ERR_BACKEND, op, "null argument");
  OJC_TRY(check_tensor(op, "x", x)); OJC_TRY(check_tensor(op, "y", y));
  if (bytes_per_token != 2 && bytes_per_token != 4) return ojc_fail(OJC_ERR_DTYPE, op, "tokens are u16 or u32");
  if (rows <= 0 || seq <= 0 || seq >= INT32_MAX) return ojc_fail(OJC_ERR_SHAPE, op, "rows and seq must be positive");
  if (x->dtype != OJC_U32 || y->dtype != OJC_U32) return ojc_fail(OJC_ERR_DTYPE, op, "x and y are U32");
  if (numel(x) != rows * seq || numel(y) != rows * seq || !contiguous(x) || !contiguous(y)) return ojc_fail(OJC_ERR_SHAPE, op, "x and y are contiguous [rows, seq]");
  for (int64_t r = 0; r < rows; ++r)   // every window is checked before the first launch (sampler.rs:297-302)
    if (starts_host[r] < 0 || (uint64_t)starts_host[r] + (uint64_t)seq + 1 > n_tokens)
      return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "token window [" + std::to_string(starts_host[r]) + ", +" + std::to_string(seq + 1) + ") past length " + std::to_string(n_tokens));
  const int bx = (int)std::min<int64_t>((seq + 1 + 255) / 256, 64);
  for (int64_t r0 = 0; r0 < rows; r0 += ROWS_PER_LAUNCH) {
    const int count = (int)std::min<int64_t>(ROWS_PER_LAUNCH, rows - r0);
    WindowStarts ws{};
    for (int i = 0; i < count; ++i) ws.start[i] = starts_host[r0 + i];
    uint32_t* xo = (uint32_t*)x->data + r0 * seq;
    uint32_t* yo = (uint32_t*)y->data + r0 * seq;
    if (bytes_per_token == 2) token_windows_kernel<uint16_t><<<dim3(bx, count), 256, 0, be->stream>>>((const uint16_t*)tokens, ws, count, (int)seq, xo, yo);
    else token_windows_kernel<uint32_t><<<dim3(bx, count), 256, 0, be->stream>>>((const uint32_t*)tokens, ws, count, (int)seq, xo, yo);
    OJC_LAUNCHED(be, op);
  }
  return OJC_OK;
}
