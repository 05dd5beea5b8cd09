/* ojas-cuda for B200: the C-ABI a Rust `impl Backend for CudaBackend` binds.
 *
 * One entry point per `ojas_core::Backend` method that one nanolab GPT training
 * step exercises (trait declarations: ojas-core/src/backend.rs:889-2634; the
 * reference's own CUDA backend refuses every one of them with `Unsupported`,
 * ojas-cuda/src/backend.rs:194-515). Plain pointers and sizes only.
 *
 * Conventions
 *  - Every call returns an ojc_status; the values are 1:1 with OjasError's
 *    variants (ojas-core/src/error.rs:18-118). ojc_last_error() gives the detail.
 *  - There is no host fallback: a device that cannot be opened is an explicit
 *    error from ojc_open (AGENTS.md:42-44 of the reference).
 *  - Tensors are descriptors over device memory obtained from ojc_alloc (which
 *    charges the backend's byte budget, as Tensor::from_device_reserved does,
 *    ojas-core/src/tensor.rs:1026). Outputs are caller-allocated descriptors.
 *  - dtype F32 is the storage of record; BF16 operands are accepted where
 *    Backend::bf16_operands() would say so (ojas-core/src/backend.rs:1029): a
 *    matmul-class op given BF16 operands runs on the tcgen05 tensor path with
 *    f32 accumulation, given F32 operands it runs the f32 tier.
 *  - Non-finite values found on the device are deferred: kernels raise a fault
 *    word that ojc_sync / ojc_download / ojc_clip_grad_norm report as
 *    OJC_ERR_NON_FINITE naming the first op (ojas-core/src/backend.rs:963-973).
 *  - A backend handle is single-owner-thread; all work is ordered on one stream
 *    (the reference runtime is `!Send`, ojas-cuda/src/backend.rs:27-31).
 */
#ifndef OJAS_CUDA_H
#define OJAS_CUDA_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

typedef enum ojc_status {
  OJC_OK = 0,
  OJC_ERR_SHAPE = 1,
  OJC_ERR_DTYPE = 2,
  OJC_ERR_OUT_OF_RANGE = 3,
  OJC_ERR_NON_FINITE = 4,
  OJC_ERR_UNSUPPORTED_HEAD_DIM = 5,
  OJC_ERR_CAPACITY_EXCEEDED = 6,
  OJC_ERR_POISONED = 7,
  OJC_ERR_DEVICE_LOST = 8,
  OJC_ERR_WAIT_TIMEOUT = 9,
  OJC_ERR_BACKEND = 10,
  OJC_ERR_UNSUPPORTED = 11,
  OJC_ERR_PLACEMENT = 12,
  OJC_ERR_NO_DEVICE = 13
} ojc_status;

typedef enum ojc_dtype { OJC_F32 = 0, OJC_BF16 = 1, OJC_F16 = 2, OJC_U32 = 3 } ojc_dtype; /* ojas-core/src/dtype.rs:5-10 */

#define OJC_MAX_RANK 6
/* Shape + dtype + device pointer (ojas-core/src/tensor.rs:20-55). Strides are in
 * elements; every op wants contiguous row-major tensors except the SDPA family,
 * which reads q/k/v/out through the strides (so a permuted view costs no copy). */
typedef struct ojc_tensor {
  void* data;
  int32_t dtype;
  int32_t rank;
  int64_t shape[OJC_MAX_RANK];
  int64_t stride[OJC_MAX_RANK];
} ojc_tensor;

typedef struct ojc_backend ojc_backend;

/* ---- lifetime, memory, transfers: BackendCore::{upload,download,sync} (backend.rs:917,939,971);
 *      open errors keep their kind (ojas-cuda/README.md:16-19). */
ojc_status ojc_open(int32_t device_ordinal, uint64_t budget_bytes, ojc_backend** out);
ojc_status ojc_close(ojc_backend* be);
const char* ojc_last_error(void);
const char* ojc_status_name(int32_t status);
/* FNV-1a (offset 0xcbf29ce484222325 to start) over host bytes, continuing from `hash`: the run id of Trainer::new
 * (ojas-model/src/trainer.rs:436-456) hashes the config texts and every parameter's f32 bytes. */
uint64_t ojc_fnv1a64(uint64_t hash, const void* bytes, uint64_t count);
ojc_status ojc_alloc(ojc_backend* be, uint64_t bytes, void** out);              /* charges the budget (budget.rs:65) */
ojc_status ojc_free(ojc_backend* be, void* ptr);                                /* refunds it */
ojc_status ojc_budget(ojc_backend* be, uint64_t* cap, uint64_t* live, uint64_t* peak); /* Budget::{cap,live,peak_bytes} budget.rs:19-240 */
ojc_status ojc_reset_peak(ojc_backend* be);
ojc_status ojc_upload(ojc_backend* be, void* dst_device, const void* src_host, uint64_t bytes);
ojc_status ojc_download(ojc_backend* be, void* dst_host, const void* src_device, uint64_t bytes); /* counts a readback (budget.rs:201) */
ojc_status ojc_sync(ojc_backend* be);                                           /* bounded wait; reports a deferred fault */
ojc_status ojc_set_sync_timeout_ms(ojc_backend* be, uint64_t ms);               /* RuntimeConfig::sync_timeout, ojas-cuda/src/runtime.rs:76 */
ojc_status ojc_readbacks(ojc_backend* be, uint64_t* count);
void* ojc_stream(ojc_backend* be);                                              /* the cudaStream_t all work is ordered on */
ojc_status ojc_fill_zero(ojc_backend* be, void* ptr, uint64_t bytes);
uint64_t ojc_kernel_launches(ojc_backend* be);                                  /* kernels launched by this backend so far */

/* ---- instrumentation (no counterpart in the reference): when enabled, every tensor-core GEMM launch is bracketed by CUDA
 *      events on the backend's stream; the read call waits for the stream, returns the summed device time, the summed
 *      2*m*n*k and the launch count since the last read, and resets them. */
ojc_status ojc_sdpa_forward_variant(int32_t variant);    /* attention kernels on the tensor cores. 0: the library's choice; 1: one CTA per tile (for timing the persistent kernels against it); 2: the 64-wide persistent kernels on at most three CTAs (tests: several tiles per CTA on small shapes); 3: the 128-wide backward kernels on at most three CTAs (likewise); 4: the 64-wide backward kernels by their own rule; 5: the 128-wide backward kernels at any head_dim */
ojc_status ojc_mlp_epilogue_variant(int32_t variant);    /* the step driver's MLP backward under bf16 autocast. 0: the library's choice (SwiGLU's forward runs in the epilogue of the gate/up product and its backward in that of the down projection's input-gradient product, where the shapes allow); 1: kernels of their own after the products (tests: both give the same bits) */
ojc_status ojc_ce_rows_variant(int32_t variant);         /* the fused cross-entropy's row kernel under bf16 autocast. 0: the library's choice (rows that fit twice in an SM's shared memory are worked on there: persistent CTAs streaming rows through two buffers for tiles of at least two rows per SM, else a CTA per row); 1: always the form that re-reads the row from L2; 2: always a CTA per row (tests: all three give the same bits) */
ojc_status ojc_profile_gemm(ojc_backend* be, int32_t enable);
ojc_status ojc_profile_gemm_read(ojc_backend* be, double* total_ms, double* total_flops, uint64_t* launches);
/* the same totals in two parts: the plain products, and the launches that also ran SwiGLU in their epilogue (they move 2-3x the bytes of the
 * plain product for the same 2*m*n*k, so their rate is not a tensor-core figure) */
ojc_status ojc_profile_gemm_read_split(ojc_backend* be, double* plain_ms, double* plain_flops, uint64_t* plain_launches, double* epilogue_ms, double* epilogue_flops,
                                       uint64_t* epilogue_launches);
ojc_status ojc_stream_wait_event(ojc_backend* be, void* cuda_stream, void* cuda_event);  /* cuda_stream waits for an event recorded by this backend (NULL stream: the backend's own) */

/* ---- owner-thread session: how a host whose calls come from many threads holds this single-owner-thread backend. ojas-capi does it for
 *      Metal with a thread that owns the device and a channel of requests (ojas-capi/src/owner.rs); its load path still refuses the CUDA
 *      device (ojas-capi/src/load.rs:41-56), partly because the CUDA runtime handle is `!Send`. ojc_session_open starts a thread that opens
 *      the backend and is the only thread that ever calls into it; the wait for the open is limited (open_timeout_ms), and a session
 *      abandoned at that limit closes whatever it opens later. ojc_session_call runs fn(backend, arg) on the owner thread and returns
 *      its status (the error text is copied to the caller's thread); calls from several threads are served in arrival order.
 *      ojc_session_train_open / _run / _close are the training requests (OP_TRAIN_OPEN, OP_TRAIN_STEP of ojas-capi/src/train.rs) as such calls. */
typedef struct ojc_session ojc_session;
typedef int32_t (*ojc_session_fn)(ojc_backend* be, void* arg);   /* returns an ojc_status value */
typedef struct ojc_model_spec ojc_model_spec;
typedef struct ojc_train_config ojc_train_config;
typedef struct ojc_step_report ojc_step_report;
typedef struct ojc_trainer ojc_trainer;
ojc_status ojc_session_open(int32_t device_ordinal, uint64_t budget_bytes, uint64_t open_timeout_ms, ojc_session** out);
ojc_status ojc_session_call(ojc_session* session, ojc_session_fn fn, void* arg);
ojc_status ojc_session_close(ojc_session* session);   /* answers every queued call, closes the backend on its own thread, joins it */
ojc_status ojc_session_train_open(ojc_session* session, const ojc_model_spec* spec, const ojc_train_config* cfg, int64_t batch, int64_t seq, ojc_trainer** out);
ojc_status ojc_session_train_run(ojc_session* session, ojc_trainer* trainer, const uint32_t* const* ids_host, const uint32_t* const* targets_host, int64_t k, ojc_step_report* report);
ojc_status ojc_session_train_close(ojc_session* session, ojc_trainer* trainer);

/* Self-test of the bounded device-side wait (no counterpart in the reference; its device-lost test traps the GPU, which this library
 * never does): one small kernel waits, with the helper every tensor-pipeline role uses, on a barrier that nothing arrives on, for at
 * most limit_cycles SM cycles (<= 2e8, about 0.1 s). Every thread must give up, the kernel ends in order, and the call returns
 * WaitTimeout from the fault word it raised; the backend stays usable (WaitTimeout is retryable, error.rs:47-95). */
ojc_status ojc_selftest_bounded_wait(ojc_backend* be, uint64_t limit_cycles, int32_t* threads_that_gave_up);

/* ---- casts: BackendCore::{cast_bf16,to_bf16,to_f32} (backend.rs:982,1042,1070); RNE on the integer bits,
 *      NaN keeps sign + payload and sets the quiet bit (autocast.rs:89-96). */
ojc_status ojc_cast_bf16(ojc_backend* be, const ojc_tensor* x, ojc_tensor* y);  /* F32 -> F32 storage holding bf16-exact values */
ojc_status ojc_to_bf16(ojc_backend* be, const ojc_tensor* x, ojc_tensor* y);    /* F32 -> BF16 */
ojc_status ojc_to_f32(ojc_backend* be, const ojc_tensor* x, ojc_tensor* y);     /* BF16 -> F32 */

/* ---- BackendModule ops of the block (backend.rs:1609-2634) */
/* Data feed, device half (next to the path: ojas-data/src/sampler.rs:245-290, BatchSampler::next_batch's read loop). The token
   stream is resident in device memory as stored (u16 or u32); the host sampler supplies `rows` window starts and the kernel writes
   x[r] = tokens[start_r, start_r + seq), y[r] = tokens[start_r + 1, start_r + seq + 1) as U32. Every window is bounds-checked first. */
ojc_status ojc_gather_token_windows(ojc_backend* be, const void* tokens_dev, int32_t bytes_per_token, uint64_t n_tokens, const int64_t* starts_host,
                                    int64_t rows, int64_t seq, ojc_tensor* x, ojc_tensor* y);
ojc_status ojc_embedding_forward(ojc_backend* be, const ojc_tensor* table, const ojc_tensor* ids, ojc_tensor* out);          /* :1615 */
ojc_status ojc_embedding_backward(ojc_backend* be, const ojc_tensor* table_shape, const ojc_tensor* ids, const ojc_tensor* grad_out, ojc_tensor* grad_table); /* :1621 */
ojc_status ojc_linear_forward(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* weight, ojc_tensor* y);               /* :1628 y = x W^T */
ojc_status ojc_linear_backward(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* weight, const ojc_tensor* grad_y, ojc_tensor* grad_x, ojc_tensor* grad_w); /* :1631 */
ojc_status ojc_linear_backward_input(ojc_backend* be, const ojc_tensor* weight, const ojc_tensor* grad_y, ojc_tensor* grad_x); /* :1648 */
ojc_status ojc_rms_norm_forward(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* weight, float eps, ojc_tensor* y);   /* :1658 */
ojc_status ojc_rms_norm_backward(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* weight, const ojc_tensor* grad_y, float eps, ojc_tensor* grad_x, ojc_tensor* grad_w); /* :1666 */
/* No counterpart in the reference. rms_norm_backward for hosts that must not let this library allocate: ojas charges every
 * device byte to one Budget before it is allocated (ojas-core/src/budget.rs), and a host that has handed all device memory
 * to that budget (or runs inside a region where cudaMalloc is forbidden) cannot let the regular entry point grow its
 * workspace. This variant takes raw F32 device pointers and a cudaStream_t, calls no allocator, and keeps the per-block
 * partial sums of grad_w in a fixed 2 MiB device array inside the library (held by every GPU that loads it). Limits:
 * dim <= 2048, F32 contiguous operands; larger row counts run on fewer, longer blocks. The first call on a device looks
 * up the array's address (make that call before any stream capture). All calls on a device share the array: calls that
 * overlap on the GPU (different streams) race; calls on one stream are safe. */
ojc_status ojc_rms_norm_backward_noalloc(void* cuda_stream, const float* x, const float* weight, const float* grad_y, int64_t rows, int64_t dim, float eps, float* grad_x, float* grad_w);
ojc_status ojc_rope_half_split_forward(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* cos_t, const ojc_tensor* sin_t, ojc_tensor* y);  /* :1674 x [B,T,H,dh], tables [T,dh] */
ojc_status ojc_rope_half_split_backward(ojc_backend* be, const ojc_tensor* grad_y, const ojc_tensor* cos_t, const ojc_tensor* sin_t, ojc_tensor* grad_x); /* :1681 */
ojc_status ojc_rms_qk_norm_forward(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* q_weight, const ojc_tensor* k_weight, float eps, ojc_tensor* q_out, ojc_tensor* k_out); /* :1688 per-head norm over the last axis */
ojc_status ojc_rms_qk_norm_backward(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* q_weight, const ojc_tensor* k_weight, const ojc_tensor* grad_q, const ojc_tensor* grad_k, float eps, ojc_tensor* grad_q_in, ojc_tensor* grad_k_in, ojc_tensor* grad_q_weight, ojc_tensor* grad_k_weight); /* :1700 */
ojc_status ojc_value_residual_blend_forward(ojc_backend* be, const ojc_tensor* v, const ojc_tensor* v0, const ojc_tensor* lambda, ojc_tensor* y); /* :1907 */
ojc_status ojc_value_residual_blend_backward(ojc_backend* be, const ojc_tensor* v, const ojc_tensor* v0, const ojc_tensor* lambda, const ojc_tensor* grad_y, ojc_tensor* grad_v, ojc_tensor* grad_v0, ojc_tensor* grad_lambda); /* :1914 */
ojc_status ojc_permute(ojc_backend* be, const ojc_tensor* x, const int32_t* dims, int32_t ndims, ojc_tensor* y);            /* :1131 only [0,2,1,3] on the path */
/* window < 0: full causal. q [B,H,T,dh]; k,v [B,Hkv,T,dh]; lse [B,H,T] F32. (:1753,1767,1781) */
ojc_status ojc_causal_sdpa_forward(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, int64_t window, ojc_tensor* out, ojc_tensor* lse);
ojc_status ojc_causal_sdpa_backward(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* out, const ojc_tensor* lse, const ojc_tensor* grad_out, int64_t window, ojc_tensor* grad_q, ojc_tensor* grad_k, ojc_tensor* grad_v);
ojc_status ojc_causal_sdpa_backward_recompute(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k, const ojc_tensor* v, const ojc_tensor* grad_out, int64_t window, ojc_tensor* grad_q, ojc_tensor* grad_k, ojc_tensor* grad_v);
/* scales (optional, [rows,H] F32) is the saved sigmoid of `_forward_saving` (:1860,1879) */
ojc_status ojc_per_head_sigmoid_gate_forward(ojc_backend* be, const ojc_tensor* input, const ojc_tensor* weight, const ojc_tensor* bias, const ojc_tensor* attn, ojc_tensor* out, ojc_tensor* scales);
/* saved_scales optional (`_backward_saved`, :1868,1894) */
ojc_status ojc_per_head_sigmoid_gate_backward(ojc_backend* be, const ojc_tensor* input, const ojc_tensor* weight, const ojc_tensor* bias, const ojc_tensor* attn, const ojc_tensor* grad_out, const ojc_tensor* saved_scales, ojc_tensor* grad_input, ojc_tensor* grad_weight, ojc_tensor* grad_bias, ojc_tensor* grad_attn);
ojc_status ojc_silu_forward(ojc_backend* be, const ojc_tensor* x, ojc_tensor* y);                                           /* :1151 */
ojc_status ojc_silu_backward(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* grad_y, ojc_tensor* grad_x);            /* :1153 */
ojc_status ojc_mul_forward(ojc_backend* be, const ojc_tensor* a, const ojc_tensor* b, ojc_tensor* y);                        /* :1155 */
ojc_status ojc_mul_backward(ojc_backend* be, const ojc_tensor* a, const ojc_tensor* b, const ojc_tensor* grad_y, ojc_tensor* grad_a, ojc_tensor* grad_b); /* :1158 */
ojc_status ojc_residual_add_forward(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* y, ojc_tensor* out);             /* :1165 */
ojc_status ojc_residual_add_backward(ojc_backend* be, const ojc_tensor* grad_out, ojc_tensor* grad_x, ojc_tensor* grad_y);   /* :1168 two copies */
/* CeChunk only bounds the reference's scratch; here it bounds the logits tile rows (cols are never chunked). has_ignore/ignore = Option<u32>.
 * grad_input / grad_weight may be NULL (CeGrads, backend.rs:3081-3136). loss: F32 [1]. (:2513) */
ojc_status ojc_linear_cross_entropy_mean(ojc_backend* be, const ojc_tensor* x, const ojc_tensor* weight, const ojc_tensor* targets, int32_t has_ignore, uint32_t ignore, int64_t chunk_rows, int64_t chunk_cols, ojc_tensor* loss, ojc_tensor* grad_input, ojc_tensor* grad_weight);
ojc_status ojc_cross_entropy_mean_forward(ojc_backend* be, const ojc_tensor* logits, const ojc_tensor* targets, int32_t has_ignore, uint32_t ignore, ojc_tensor* loss);      /* :2452 */
ojc_status ojc_cross_entropy_mean_backward(ojc_backend* be, const ojc_tensor* logits, const ojc_tensor* targets, int32_t has_ignore, uint32_t ignore, ojc_tensor* grad_logits); /* :2461 */
ojc_status ojc_argmax_rows(ojc_backend* be, const ojc_tensor* x, ojc_tensor* out_u32);                                       /* :1525 ties -> lowest column */
/* ---- decode / eval ops on the same backend (the "next" rows after the training step)
 * topk_rows (ojas-core/src/backend.rs:1553-1612): the k leaders of each row of x [rows, cols] by rank_logits (:186-195): value
 * descending with +0.0 and -0.0 one value and -inf after every finite value, then column ascending. values F32 [rows, k], ids U32
 * [rows, k]. NaN or +inf in a row surfaces as NonFinite at the next sync; k > 1024 is Unsupported (as the Metal and wgpu kernels).
 * kv_cache_write (:2556-2565): src [B, Tn, Hkv, D] into the ring cache [B, Tcap, Hkv, D], position at + t to slot (at + t) % Tcap.
 * cached_attention_forward (:2521-2554): q [B, Tq, H, D] against kv_len cached positions; query i sits at kv_len - Tq + i and sees
 * positions 0..=p or the last `window` of them (window -1: none), oldest first; head h reads KV head h / (H / Hkv); out [B, Tq, H, D]. */
ojc_status ojc_topk_rows(ojc_backend* be, const ojc_tensor* x, int64_t k, ojc_tensor* values, ojc_tensor* ids_u32);
ojc_status ojc_kv_cache_write(ojc_backend* be, ojc_tensor* cache, const ojc_tensor* src, uint64_t at);
ojc_status ojc_cached_attention_forward(ojc_backend* be, const ojc_tensor* q, const ojc_tensor* k_cache, const ojc_tensor* v_cache, uint64_t kv_len, int64_t window,
                                        ojc_tensor* out);

/* ---- gradient plumbing and optimizers */
ojc_status ojc_accumulate_grad(ojc_backend* be, ojc_tensor* acc, const ojc_tensor* grad);                                    /* :1483 acc += grad */
ojc_status ojc_scale_grad(ojc_backend* be, ojc_tensor* grad, float scale);                                                   /* :1502 */
/* Global L2 norm over `count` F32 tensors, then scale by min(1, max/(norm+1e-6)) only if < 1 (:1471; clip_scale :277-303).
 * One sync point: returns the norm on the host and reports any deferred fault. */
ojc_status ojc_clip_grad_norm(ojc_backend* be, ojc_tensor* const* grads, int64_t count, float max_norm, float* norm_out);
typedef struct ojc_adamw_config { double lr, beta1, beta2, eps, weight_decay; } ojc_adamw_config;                            /* AdamWConfig backend.rs:494 */
/* In place on param, m, v. The 7 f32 words are formed inside from step_before + config (AdamWScalars, backend.rs:371-476).
 * bf16_mirror (optional, BF16, same shape) is refreshed with the new parameter. */
ojc_status ojc_adamw_step(ojc_backend* be, ojc_tensor* param, const ojc_tensor* grad, ojc_tensor* m, ojc_tensor* v, uint64_t step_before, const ojc_adamw_config* cfg, ojc_tensor* bf16_mirror); /* :2470 */
typedef struct ojc_muon_config { double lr, momentum, weight_decay; int32_t nesterov; int32_t ns5_bf16; } ojc_muon_config;   /* MuonNs5Config backend.rs:548 */
ojc_status ojc_muon_ns5_step(ojc_backend* be, ojc_tensor* param, const ojc_tensor* grad, ojc_tensor* momentum, const ojc_muon_config* cfg, ojc_tensor* bf16_mirror); /* :2485 */
ojc_status ojc_optimizer_scratch_bytes(ojc_backend* be, int32_t kind /*0 AdamW, 1 Muon*/, int64_t rows, int64_t cols, uint64_t* bytes); /* :953 */

/* ---- whole-step driver: the op sequence of Trainer::step (ojas-model/src/trainer.rs:672-1046) replayed in C++ over
 *      the entry points above, so the path can be driven end to end without the Rust host. */
typedef struct ojc_model_spec {            /* ModelSpec, ojas-model/src/spec.rs:45 */
  int64_t vocab, n_embd, n_layer, n_head, n_kv_head, head_dim, hidden, max_seq;
  int64_t window;                          /* -1: full causal */
  double rope_base;
  float rms_eps;
} ojc_model_spec;
typedef struct ojc_train_config {          /* TrainConfig, ojas-model/src/trainer.rs:100-172 */
  int32_t autocast_bf16;                   /* 0: f32 tier, 1: bf16 autocast (Autocast<B>, autocast.rs:464) */
  int32_t optimizer;                       /* 0: AdamW on every tensor (lr = adam_lr, wd = adam_weight_decay); 1: Muon NS5 on rank-2 hidden weights + AdamW(wd 0) elsewhere (ojas-cpu/src/train.rs:54-62) */
  double adam_lr, adam_beta1, adam_beta2, adam_eps, adam_weight_decay;
  double matrix_lr, muon_momentum, muon_weight_decay;
  int32_t ns5_bf16;
  float grad_clip;                         /* <= 0: no clipping */
  int32_t has_ignore; uint32_t ignore_index;
  int64_t ce_chunk_rows;                   /* rows of one fused-CE logits tile (0: default) */
  float loss_seed;                         /* backward seed w_i (MicroWeights, trainer.rs:1083-1119); 1/world under data parallelism */
  int32_t checkpoint_blocks;               /* ActivationCheckpoint::Blocks (ojas-model/src/block.rs:323-336): keep only each block's input and recompute the block in
                                            * backward; same bits as without, about a third more forward work, activation memory of two blocks instead of n_layer */
  int32_t schedule;                        /* LrSchedule (ojas-cpu/src/schedule.rs:205-226): 0 none (multiplier 1 at every step), 1 Cosine, 2 Wsd */
  uint64_t warmup_steps, total_steps;      /* total_steps 0 is refused for Cosine and Wsd (schedule.rs:42-47,127-133) */
  double decay_frac;                       /* Wsd only, in [0, 1] (WSD_DECAY_FRAC 0.2, schedule.rs:94) */
  int32_t on_nonfinite;                    /* NonFinitePolicy (trainer.rs:85-91): 0 Abort (keep the data cursor), 1 SkipBatch (move it past the step's batches) */
} ojc_train_config;
/* StepReport (trainer.rs:281-297). loss is the token-weighted mean of the micro-batch losses, grad_norm the global norm before clipping,
 * lr_multiplier the schedule's factor on every group's peak learning rate, step the completed steps after this one. */
typedef struct ojc_step_report { float loss; float grad_norm; uint64_t step; uint64_t tokens; double lr_multiplier; } ojc_step_report;
typedef struct ojc_trainer ojc_trainer;
ojc_status ojc_trainer_open(ojc_backend* be, const ojc_model_spec* spec, const ojc_train_config* cfg, int64_t batch, int64_t seq, ojc_trainer** out);
ojc_status ojc_trainer_close(ojc_trainer* tr);
int64_t ojc_trainer_param_count(ojc_trainer* tr);
ojc_status ojc_trainer_param_info(ojc_trainer* tr, int64_t index, char* name, int64_t name_cap, int32_t* rank, int64_t* shape2, int32_t* group, int32_t* trains);
ojc_status ojc_trainer_set_param(ojc_trainer* tr, int64_t index, const float* host, uint64_t count);   /* also refreshes the bf16 mirror */
ojc_status ojc_trainer_get_param(ojc_trainer* tr, int64_t index, float* host, uint64_t count);
ojc_status ojc_trainer_get_grad(ojc_trainer* tr, int64_t index, float* host, uint64_t count);          /* after ojc_trainer_gradients */
/* Checkpoint support (Trainer::save / resume_from, ojas-model/src/checkpoint.rs:527-700): the optimizer state of one parameter and
 * the completed-step count. slot 0: Muon momentum of a matrix (optimizer 1) or AdamW first moment; slot 1: AdamW second moment.
 * A frozen parameter, or slot 1 of a Muon matrix, is OutOfRange. */
ojc_status ojc_trainer_get_moment(ojc_trainer* tr, int64_t index, int32_t slot, float* host, uint64_t count);
ojc_status ojc_trainer_set_moment(ojc_trainer* tr, int64_t index, int32_t slot, const float* host, uint64_t count);
uint64_t ojc_trainer_steps_done(ojc_trainer* tr);
ojc_status ojc_trainer_set_steps_done(ojc_trainer* tr, uint64_t step);
/* forward + fused CE + backward on host ids/targets [batch*seq] (copied in from the caller's pinned or pageable memory);
 * gradients stay on the device. loss_out may be NULL (no readback). */
ojc_status ojc_trainer_gradients(ojc_trainer* tr, const uint32_t* ids_host, const uint32_t* targets_host, float* loss_out);
ojc_status ojc_trainer_gradients_device(ojc_trainer* tr, const uint32_t* ids_dev, const uint32_t* targets_dev); /* inputs already resident */
ojc_status ojc_trainer_apply(ojc_trainer* tr, float* grad_norm_out);                                   /* clip + optimizer, step += 1 */
ojc_status ojc_trainer_finish(ojc_trainer* tr, ojc_step_report* report);                               /* Trainer::finish (trainer.rs:1031): sync + the one readback (loss, norm, fault word) */
ojc_status ojc_trainer_step(ojc_trainer* tr, const uint32_t* ids_host, const uint32_t* targets_host, ojc_step_report* report); /* gradients + apply + the one loss readback */
ojc_status ojc_trainer_step_device(ojc_trainer* tr, const uint32_t* ids_dev, const uint32_t* targets_dev, ojc_step_report* report);
/* Trainer::step_tokens / Trainer::run (trainer.rs:713-890): ONE optimizer step over k caller-supplied micro-batches of [batch, seq] host ids and
 * targets. Micro-batch i seeds its backward with MicroWeights' w_i (its share of the step's valid targets; 1/run when every non-empty micro-batch
 * counts the same, trainer.rs:1083-1119) times the config's loss_seed, gradients are summed in f32 in micro-batch order (accumulate_grad), a
 * micro-batch whose targets are all ignored only has its ids checked. Then clip, the schedule's learning rates, Muon / AdamW, and the one readback.
 * Refusals before any work: Poisoned, a step past a Wsd schedule or at u64::MAX (OutOfRange), k outside 1..=2^24 (OutOfRange), an id outside the
 * vocabulary (OutOfRange), no valid target at all (NonFinite), no room for the optimizer's scratch (CapacityExceeded). A non-finite loss or
 * gradient norm is found on the device before the first update: the optimizer kernels leave parameters, moments and the step count as they were,
 * the call returns NonFinite and the trainer stays Ready (trainer.rs:824-838). Only a failure inside the update poisons. */
ojc_status ojc_trainer_run(ojc_trainer* tr, const uint32_t* const* ids_host, const uint32_t* const* targets_host, int64_t k, ojc_step_report* report);
/* The first half of ojc_trainer_run (refusals, k forward/backward passes, accumulation), for callers that exchange gradient buckets between
 * it and ojc_trainer_apply + ojc_trainer_finish. */
ojc_status ojc_trainer_run_gradients(ojc_trainer* tr, const uint32_t* const* ids_host, const uint32_t* const* targets_host, int64_t k);
/* What Trainer::step does with a failed run (trainer.rs:686-708), for the host that owns the sampler: given the status ojc_trainer_run returned,
 * *advance_cursor says whether the data cursor moves past the step's batches (only a NonFinite on a Ready trainer under SkipBatch), and the return
 * value is the status to surface: run_status itself, or OutOfRange once 8 skips in a row (MAX_CONSECUTIVE_SKIPS, trainer.rs:81) were already
 * taken, in which case the cursor stays. Any committed step clears the count. */
ojc_status ojc_trainer_resolve_failure(ojc_trainer* tr, ojc_status run_status, int32_t* advance_cursor);
int32_t ojc_trainer_state(ojc_trainer* tr);                                                              /* TrainState (trainer.rs:93-98): 0 Ready, 1 Poisoned */
/* LrSchedule::multiplier at a 0-based step (schedule.rs:66-90,163-199), every operation in f64 in nanolab's order. */
ojc_status ojc_lr_multiplier(const ojc_train_config* cfg, uint64_t step, double* multiplier);
/* Host-made failure for tests of the trainer's state machine (the job of the reference's Probe<B> test double, ojas-model/tests/common/mod.rs:647:
 * fail the n-th call of a chosen op). where 1: the next gradient pass fails after its forward, before anything the trainer owns changed;
 * where 2: the next optimizer phase fails after its first update kernel. One shot; no device fault is involved. */
ojc_status ojc_trainer_inject_failure(ojc_trainer* tr, int32_t where);
ojc_status ojc_trainer_logits(ojc_trainer* tr, const uint32_t* ids_host, float* logits_host);          /* forward_logits, block.rs:407-416; [batch*seq, vocab] */
/* Data-parallel extension (new; the reference has no distributed code): gradients live in contiguous buckets; the
 * caller all-reduces each bucket (NCCL) between ojc_trainer_gradients and ojc_trainer_apply. */
/* Under bf16 autocast the weight-gradient GEMMs of backward run on a second stream beside the dX chain (same kernels, same
   results bit for bit). enable = 0 folds them back into the one stream, e.g. to time each GEMM with the GPU to itself. */
ojc_status ojc_trainer_overlap_weight_grads(ojc_trainer* tr, int32_t enable);
int64_t ojc_trainer_bucket_count(ojc_trainer* tr);
/* The communicator of the data-parallel step (no counterpart in the reference, which has no distributed code; what it keeps is the
 * arithmetic of K-micro-batch accumulation, trainer.rs:916-1001, with K = world). NCCL is loaded with dlopen at the first call, so a
 * host that never calls these needs no NCCL. One process per GPU: rank 0 makes a 128-byte id with ojc_comm_unique_id and hands it to
 * the other ranks by any means of its own (a file, a socket, an environment variable); every rank then calls ojc_comm_init.
 * ojc_allreduce_start queues one in-place f32 sum per gradient bucket on the communicator's own stream, each behind the bucket's
 * ready event, so the exchange runs under the rest of backward; ojc_allreduce_wait makes the backend's stream wait for the last one
 * (the host does not block) and reports an error NCCL met asynchronously. A collective that never completes surfaces as WaitTimeout
 * from the next bounded host wait (ojc_sync / ojc_download / ojc_trainer_finish). */
typedef struct ojc_comm ojc_comm;
ojc_status ojc_comm_unique_id(uint8_t* id128);
ojc_status ojc_comm_init(ojc_backend* be, int32_t rank, int32_t world, const uint8_t* id128, ojc_comm** out);
ojc_status ojc_comm_destroy(ojc_comm* comm);
int32_t ojc_comm_rank(ojc_comm* comm);
int32_t ojc_comm_world(ojc_comm* comm);
ojc_status ojc_comm_check(ojc_comm* comm);                                                              /* an asynchronous NCCL error since the last call; never blocks */
ojc_status ojc_allreduce_start(ojc_comm* comm, ojc_trainer* tr);
ojc_status ojc_allreduce_wait(ojc_comm* comm, ojc_trainer* tr);
ojc_status ojc_comm_allreduce(ojc_comm* comm, void* device_data, uint64_t count, int32_t dtype, int32_t op); /* in place on the backend's stream; op 0 sum, 1 max, 2 min */
ojc_status ojc_comm_broadcast_many(ojc_comm* comm, void* const* device_ptrs, const uint64_t* counts, const int32_t* roots, int64_t n, int32_t dtype); /* one group */
/* Gives the trainer the communicator: ojc_trainer_run / _step / _step_device then exchange the buckets themselves between backward and
 * the optimizer (the config's loss_seed should be 1/world). shard_muon != 0 also splits the Muon phase: matrix j of each shape group is
 * orthogonalised by rank j % world only and its new parameters are broadcast from there, so every rank holds the same parameters but a
 * matrix's momentum lives on its owner (ojc_trainer_sync_moments broadcasts the momenta, e.g. before a checkpoint). comm NULL detaches. */
ojc_status ojc_trainer_set_comm(ojc_trainer* tr, ojc_comm* comm, int32_t shard_muon);
ojc_status ojc_trainer_sync_moments(ojc_trainer* tr);
/* Device time the backend's stream spent waiting for the gradient exchange in the last finished step: from the end of backward to
 * the first optimizer kernel, minus nothing (with the exchange fully hidden under backward it is the launch gap only). */
ojc_status ojc_trainer_exposed_exchange_ms(ojc_trainer* tr, float* ms);
/* FNV-1a over every parameter's f32 bytes in table order (device -> host copies, then ojc_fnv1a64): equal on every rank of a healthy
 * data-parallel job. */
ojc_status ojc_trainer_param_checksum(ojc_trainer* tr, uint64_t* hash);
ojc_status ojc_trainer_bucket(ojc_trainer* tr, int64_t index, void** device_ptr, uint64_t* floats);
ojc_status ojc_trainer_bucket_ready_event(ojc_trainer* tr, int64_t index, void** cuda_event);          /* recorded when the bucket's last gradient is written */

#ifdef __cplusplus
}
#endif
#endif
