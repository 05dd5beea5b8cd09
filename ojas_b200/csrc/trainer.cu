// The nanolab GPT training step as a C++ driver over this library's ops.
//
// It replays what the reference's host layers do with a Backend:
//   parameters  ojas-model/src/names.rs:188-300 (param_table order and groups)
//   forward     ojas-model/src/block.rs:218-264 (block_with), 351-404 (hidden), 423-447 (forward_loss)
//   backward    the reverse walk of ojas-autograd/src/tape.rs:2004-2466, fan-in by accumulation (2565-2591)
//   optimizer   ojas-model/src/trainer.rs:754-1046 (clip, per-slot Muon / AdamW in table order, one readback)
// Under bf16 autocast the rounding points follow ojas-core/src/autocast.rs: the residual stream, norm statistics,
// loss, weight gradients and optimizer state stay f32; matmul-class operands and activation outputs are bf16.
// Permutes are views: attention reads and writes [B,T,H,dh] storage through [B,H,T,dh] strides.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "ce.cuh"
#include "common.cuh"
#include "linear.cuh"
#include "ops.cuh"
#include "optim.cuh"
#include "sdpa.cuh"

int g_mlp_epilogue_variant = 0;   // ojc_mlp_epilogue_variant: 0 SwiGLU inside the epilogues of the gate/up product and of the down projection's input-gradient product, 1 kernels of its own
extern "C" ojc_status ojc_mlp_epilogue_variant(int32_t variant) { g_mlp_epilogue_variant = variant == 1 ? 1 : 0; return OJC_OK; }

namespace {

enum { P_NORM1 = 0, P_Q, P_K, P_V, P_O, P_QN, P_KN, P_GW, P_GB, P_LAMBDA, P_NORM2, P_FG, P_FU, P_FD, P_PER_BLOCK };
enum { GROUP_ADAMW = 0, GROUP_MUON = 1 };

struct Param {
  std::string name;
  int rank; int64_t shape[2]; int64_t n; int group; bool trains;
  int64_t offset;  // floats into the flat buffers
};

struct LayerActs {
  void *h, *q, *k, *rawv, *qr, *kr, *v, *y, *yg, *h2, *a, *u, *m;  // activation dtype
  float *x, *x1, *lse, *scales;                                     // f32
};

ojc_tensor T1(void* p, int32_t dt, int64_t n) { ojc_tensor t{}; t.data = p; t.dtype = dt; t.rank = 1; t.shape[0] = n; t.stride[0] = 1; return t; }
ojc_tensor T2(void* p, int32_t dt, int64_t r, int64_t c) {
  ojc_tensor t{}; t.data = p; t.dtype = dt; t.rank = 2; t.shape[0] = r; t.shape[1] = c; t.stride[0] = c; t.stride[1] = 1; return t;
}
ojc_tensor T4(void* p, int32_t dt, int64_t a, int64_t b, int64_t c, int64_t d) {
  ojc_tensor t{}; t.data = p; t.dtype = dt; t.rank = 4; t.shape[0] = a; t.shape[1] = b; t.shape[2] = c; t.shape[3] = d;
  t.stride[3] = 1; t.stride[2] = d; t.stride[1] = c * d; t.stride[0] = b * c * d; return t;
}
// [B,T,H,dh] storage seen as [B,H,T,dh]
ojc_tensor TBHTD(void* p, int32_t dt, int64_t b, int64_t t, int64_t h, int64_t d, int64_t token_stride = 0) {
  const int64_t ts = token_stride ? token_stride : h * d;   // a column slice of a wider [tokens, ld] buffer keeps its row stride
  ojc_tensor x{}; x.data = p; x.dtype = dt; x.rank = 4; x.shape[0] = b; x.shape[1] = h; x.shape[2] = t; x.shape[3] = d;
  x.stride[0] = t * ts; x.stride[1] = d; x.stride[2] = ts; x.stride[3] = 1; return x;
}

}  // namespace

struct ojc_trainer {
  ojc_backend* be = nullptr;
  ojc_model_spec spec{};
  ojc_train_config cfg{};
  int64_t B = 0, T = 0, N = 0;
  std::vector<Param> params;
  int64_t flat_n = 0;
  float *w = nullptr, *g = nullptr, *m1 = nullptr, *m2 = nullptr;  // flat parameter-shaped buffers (m1 doubles as the Muon momentum)
  bf16* mirror = nullptr;
  int32_t act_dt = OJC_F32;
  std::vector<LayerActs> acts;
  std::vector<void*> owned;
  float *cos_t = nullptr, *sin_t = nullptr, *x_final = nullptr, *gx = nullptr, *g_h = nullptr, *g_h2 = nullptr, *gv0_acc = nullptr, *stats = nullptr;
  void *hf = nullptr, *gx_b = nullptr, *gx_b2 = nullptr, *g_m = nullptr, *g_a = nullptr, *g_u = nullptr, *g_yg = nullptr, *g_y = nullptr, *g_qr = nullptr, *g_kr = nullptr,
       *g_v = nullptr, *g_qn = nullptr, *g_kn = nullptr, *g_q = nullptr, *g_k = nullptr, *g_rawv = nullptr, *g_v0l = nullptr, *qn = nullptr, *kn = nullptr;
  uint32_t *ids = nullptr, *targets = nullptr;
  float* dr = nullptr;                          // [B, H, T] rowsum(dO . O): written by the gate's backward, read by the attention backward
  bf16 *gate_z = nullptr, *gate_gz = nullptr;   // [N, gate_ld] logits / logit gradients of the gate GEMMs (bf16 tier)
  float* gate_gw = nullptr;                     // [gate_ld, d] padded weight gradient
  int gate_ld = 0;                              // 0: the gate runs on the per-row kernels
  bool fused_qk = false;
  // bf16 tier: q/k/v come from one GEMM over the adjacent weight slots [q_proj; k_proj; v_proj] and ffn gate/up from one over
  // [gate; up]; the consumers read column slices with these row strides (0: separate buffers)
  bool fused_lin = false;
  int64_t ld_qkv = 0, ld_au = 0;
  uint64_t step = 0;
  bool poisoned = false, grads_ready = false;
  // One step over K micro-batches (Trainer::run): the running gradient sum of micro-batches 0..i-1 while micro-batch i's backward
  // writes g, the backward seed of the pass in flight, which stats slot holds the step's loss, and what the report needs.
  float* gacc = nullptr;
  float seed_now = 1.0f;
  int loss_slot = 0;
  double lr_mult = 1.0;
  float loss_div = 1.0f;
  uint64_t run_tokens = 0;
  uint32_t consecutive_skips = 0;
  bool eager_used = false;                      // this step's blocks were stepped during backward, before the norm was known
  int inject = 0;                               // ojc_trainer_inject_failure
  // data-parallel: the communicator the one-call steps exchange the buckets through, whether the Muon phase is split across
  // ranks, and the events that time how long the main stream waited for the exchange
  ojc_comm* comm = nullptr;
  bool shard_muon = false;
  cudaEvent_t ev_bwd_end = nullptr, ev_exchanged = nullptr;
  bool exchange_timed = false;
  // One-call steps with AdamW on every tensor and no clipping: a block's parameters are stepped on the side lane as soon as its
  // gradients are final, under the rest of backward (nothing later reads them); apply() then skips [eager_begin, eager_end).
  bool eager_request = false;
  int64_t eager_begin = 0, eager_end = 0;
  // Weight gradients (their GEMMs, split-K sums and copies) run on a second stream with its own workspace while the main
  // stream walks on through the dX chain: nothing downstream reads them before the optimizer.
  cudaStream_t side_stream = nullptr;
  bool side_enabled = true;
  cudaEvent_t ev_main = nullptr, ev_side = nullptr, ev_finish = nullptr;
  void* finish_pool = nullptr;                  // partial sums of the small weight-gradient reductions finished on the side stream
  static constexpr uint64_t FINISH_POOL_BYTES = 16ull << 20;
  void* side_scratch = nullptr;
  uint64_t side_scratch_bytes = 0;
  struct Bucket { int64_t offset, floats; int first_param; cudaEvent_t ready; bool recorded; };
  std::vector<Bucket> buckets;

  const Param& P(int64_t layer, int which) const { return params[1 + layer * P_PER_BLOCK + which]; }
  float* W(const Param& p) const { return w + p.offset; }
  float* G(const Param& p) const { return g + p.offset; }
  // the operand a matmul-class op reads: the bf16 mirror under autocast, the f32 master otherwise
  const void* WM(const Param& p) const { return act_dt == OJC_BF16 ? (const void*)(mirror + p.offset) : (const void*)(w + p.offset); }
};

namespace {

void build_table(ojc_trainer* tr) {
  const ojc_model_spec& s = tr->spec;
  const int64_t d = s.n_embd, q = s.n_head * s.head_dim, kv = s.n_kv_head * s.head_dim;
  int64_t off = 0;
  auto push = [&](std::string name, int rank, int64_t a, int64_t b, bool embedding, bool trains) {
    Param p; p.name = std::move(name); p.rank = rank; p.shape[0] = a; p.shape[1] = b; p.n = a * b;
    p.group = embedding ? GROUP_ADAMW : (rank >= 2 ? GROUP_MUON : GROUP_ADAMW);  // ojas-cpu/src/train.rs:54-62
    p.trains = trains; p.offset = off;
    off += (p.n + 63) & ~int64_t(63);  // 256-byte aligned slots; the padding stays zero
    tr->params.push_back(std::move(p));
  };
  push("tok_emb.weight", 2, s.vocab, d, true, true);
  for (int64_t i = 0; i < s.n_layer; ++i) {
    std::string p = "blocks." + std::to_string(i), m = p + ".mixer";
    push(p + ".norm1.weight", 1, d, 1, false, true);
    push(m + ".q_proj.weight", 2, q, d, false, true);
    push(m + ".k_proj.weight", 2, kv, d, false, true);
    push(m + ".v_proj.weight", 2, kv, d, false, true);
    push(m + ".o_proj.weight", 2, d, q, false, true);
    push(m + ".q_norm.weight", 1, s.head_dim, 1, false, true);
    push(m + ".k_norm.weight", 1, s.head_dim, 1, false, true);
    push(m + ".gate.weight", 2, s.n_head, d, false, true);
    push(m + ".gate.bias", 1, s.n_head, 1, false, true);
    push(m + ".vr_lambda", 1, 1, 1, false, i != 0);
    push(p + ".norm2.weight", 1, d, 1, false, true);
    push(p + ".ffn.gate.weight", 2, s.hidden, d, false, true);
    push(p + ".ffn.up.weight", 2, s.hidden, d, false, true);
    push(p + ".ffn.down.weight", 2, d, s.hidden, false, true);
  }
  push("norm_f.weight", 1, d, 1, false, true);
  tr->flat_n = off;
}

ojc_status take(ojc_trainer* tr, uint64_t bytes, void** out) {
  OJC_TRY(ojc_alloc(tr->be, bytes, out));
  tr->owned.push_back(*out);
  return OJC_OK;
}
template <class P> ojc_status take_as(ojc_trainer* tr, uint64_t bytes, P** out) { void* p = nullptr; OJC_TRY(take(tr, bytes, &p)); *out = (P*)p; return OJC_OK; }

void rope_tables_host(double base, int64_t len, int64_t dim, std::vector<float>& cos_t, std::vector<float>& sin_t) {
  // ojas-model/src/block.rs:62-85: f64 powf / sin_cos, then f32
  const int64_t half = dim / 2;
  cos_t.assign(len * dim, 0.0f); sin_t.assign(len * dim, 0.0f);
  for (int64_t row = 0; row < len; ++row)
    for (int64_t i = 0; i < half; ++i) {
      double inv = std::pow(base, -((double)(2 * i)) / (double)dim);
      double s = std::sin((double)row * inv), c = std::cos((double)row * inv);
      cos_t[row * dim + i] = (float)c; cos_t[row * dim + half + i] = (float)c;
      sin_t[row * dim + i] = (float)s; sin_t[row * dim + half + i] = (float)s;
    }
}

ojc_status refresh_mirror(ojc_trainer* tr, const Param& p) {
  if (tr->act_dt != OJC_BF16) return OJC_OK;
  ojc_tensor src = T1(tr->W(p), OJC_F32, p.n), dst = T1(tr->mirror + p.offset, OJC_BF16, p.n);
  return ojc_to_bf16(tr->be, &src, &dst);
}

// ---------------------------------------------------------------------------------------------- forward
// One block's forward from its saved input acts[l].x: writes the block's activations and the next block's input. Also the
// recompute step of activation checkpointing (ActivationCheckpoint::Blocks, ojas-model/src/block.rs:323-336), where it
// reproduces the same bits the forward pass wrote.
ojc_status block_forward(ojc_trainer* tr, int64_t l) {
  ojc_backend* be = tr->be;
  const ojc_model_spec& s = tr->spec;
  const int64_t d = s.n_embd, H = s.n_head, Hkv = s.n_kv_head, dh = s.head_dim, F = s.hidden, N = tr->N, B = tr->B, T = tr->T;
  const int64_t qw = H * dh, kvw = Hkv * dh, L = s.n_layer;
  const int32_t A = tr->act_dt;
  const float eps = s.rms_eps;
  ojc_tensor cos_t = T2(tr->cos_t, OJC_F32, T, dh), sin_t = T2(tr->sin_t, OJC_F32, T, dh);
  LayerActs& a = tr->acts[l];
  float* x_next = (l + 1 < L) ? tr->acts[l + 1].x : tr->x_final;
  ojc_tensor x = T2(a.x, OJC_F32, N, d), h = T2(a.h, A, N, d);
  ojc_tensor n1 = T1(tr->W(tr->P(l, P_NORM1)), OJC_F32, d);
  // bf16 tier: the residual stream's next buffer starts as a copy of this one and the projection adds into it (the
  // GEMM's adding tile stores), instead of reading a separate residual operand in the epilogue
  const bool add_in_place = A == OJC_BF16;
  OJC_TRY(rms_forward_impl(be, &x, &n1, eps, &h, add_in_place ? a.x1 : nullptr));
  const bool fl = tr->fused_lin;
  const int64_t sq = fl ? tr->ld_qkv : qw, skv = fl ? tr->ld_qkv : kvw;   // token strides of q and of k / raw v
  if (fl) {
    OJC_TRY(linear_forward_impl(be, a.h, A, tr->WM(tr->P(l, P_Q)), A, a.q, A, N, d, tr->ld_qkv, nullptr));
  } else {
    OJC_TRY(linear_forward_impl(be, a.h, A, tr->WM(tr->P(l, P_Q)), A, a.q, A, N, d, qw, nullptr));
    OJC_TRY(linear_forward_impl(be, a.h, A, tr->WM(tr->P(l, P_K)), A, a.k, A, N, d, kvw, nullptr));
    OJC_TRY(linear_forward_impl(be, a.h, A, tr->WM(tr->P(l, P_V)), A, a.rawv, A, N, d, kvw, nullptr));
  }
  if (tr->fused_qk) {
    OJC_TRY(qk_norm_rope_forward(be, (const bf16*)a.q, sq, tr->W(tr->P(l, P_QN)), tr->cos_t, tr->sin_t, (bf16*)a.qr, qw, N, (int)H, (int)dh, (int)T, eps));
    OJC_TRY(qk_norm_rope_forward(be, (const bf16*)a.k, skv, tr->W(tr->P(l, P_KN)), tr->cos_t, tr->sin_t, (bf16*)a.kr, kvw, N, (int)Hkv, (int)dh, (int)T, eps));
  } else {
    ojc_tensor q = T2(a.q, A, N * H, dh), qn = T2(tr->qn, A, N * H, dh), qnw = T1(tr->W(tr->P(l, P_QN)), OJC_F32, dh);
    ojc_tensor k = T2(a.k, A, N * Hkv, dh), kn = T2(tr->kn, A, N * Hkv, dh), knw = T1(tr->W(tr->P(l, P_KN)), OJC_F32, dh);
    OJC_TRY(rms_forward_impl(be, &q, &qnw, eps, &qn));
    OJC_TRY(rms_forward_impl(be, &k, &knw, eps, &kn));
    ojc_tensor qn4 = T4(tr->qn, A, B, T, H, dh), qr4 = T4(a.qr, A, B, T, H, dh), kn4 = T4(tr->kn, A, B, T, Hkv, dh), kr4 = T4(a.kr, A, B, T, Hkv, dh);
    OJC_TRY(rope_impl(be, "rope_half_split_forward", &qn4, &cos_t, &sin_t, &qr4, 0));
    OJC_TRY(rope_impl(be, "rope_half_split_forward", &kn4, &cos_t, &sin_t, &kr4, 0));
  }
  if (l > 0 && fl) {
    OJC_TRY(vres_rows_forward(be, (const bf16*)a.rawv, skv, (const bf16*)tr->acts[0].rawv, skv, tr->W(tr->P(l, P_LAMBDA)), (bf16*)a.v, N, kvw));
  } else if (l > 0) {
    ojc_tensor rv = T1(a.rawv, A, N * kvw), v0 = T1(tr->acts[0].rawv, A, N * kvw), lam = T1(tr->W(tr->P(l, P_LAMBDA)), OJC_F32, 1), v = T1(a.v, A, N * kvw);
    OJC_TRY(ojc_value_residual_blend_forward(be, &rv, &v0, &lam, &v));
  }
  {
    ojc_tensor q = TBHTD(a.qr, A, B, T, H, dh), k = TBHTD(a.kr, A, B, T, Hkv, dh), y = TBHTD(a.y, A, B, T, H, dh);
    ojc_tensor v = l > 0 ? TBHTD(a.v, A, B, T, Hkv, dh) : TBHTD(a.rawv, A, B, T, Hkv, dh, skv);
    ojc_tensor lse = T1(a.lse, OJC_F32, B * H * T);
    lse.rank = 3; lse.shape[0] = B; lse.shape[1] = H; lse.shape[2] = T; lse.stride[0] = H * T; lse.stride[1] = T; lse.stride[2] = 1;
    OJC_TRY(ojc_causal_sdpa_forward(be, &q, &k, &v, s.window, &y, &lse));
  }
  if (tr->gate_ld) {
    // gate logits as a skinny GEMM over the weight rows [0, gate_ld) (rows past H are the next parameters' mirror
    // values: their columns are never read), then the pointwise half
    OJC_TRY(linear_forward_impl(be, a.h, A, tr->WM(tr->P(l, P_GW)), A, tr->gate_z, A, N, d, tr->gate_ld, nullptr));
    OJC_TRY(gate_apply_forward(be, tr->gate_z, tr->gate_ld, tr->W(tr->P(l, P_GB)), (const bf16*)a.y, (bf16*)a.yg, a.scales, N, (int)H, (int)dh));
  } else {
    ojc_tensor h2d = T2(a.h, A, N, d), gw = T2((void*)tr->WM(tr->P(l, P_GW)), A, H, d), gb = T1(tr->W(tr->P(l, P_GB)), OJC_F32, H);
    ojc_tensor y = T2(a.y, A, N * H, dh), yg = T2(a.yg, A, N * H, dh), sc = T2(a.scales, OJC_F32, N, H);
    OJC_TRY(ojc_per_head_sigmoid_gate_forward(be, &h2d, &gw, &gb, &y, &yg, &sc));
  }
  OJC_TRY(linear_forward_impl(be, a.yg, A, tr->WM(tr->P(l, P_O)), A, a.x1, OJC_F32, N, qw, d, add_in_place ? nullptr : a.x, add_in_place));  // x1 = x + o_proj(yg)
  {
    ojc_tensor x1 = T2(a.x1, OJC_F32, N, d), h2 = T2(a.h2, A, N, d), n2 = T1(tr->W(tr->P(l, P_NORM2)), OJC_F32, d);
    OJC_TRY(rms_forward_impl(be, &x1, &n2, eps, &h2, add_in_place ? x_next : nullptr));
  }
  if (fl) {
    if (g_mlp_epilogue_variant == 0 && linear_forward_swiglu_eligible(be, a.h2, tr->WM(tr->P(l, P_FG)), a.a, a.m, tr->ld_au, N, d, F)) {
      OJC_TRY(linear_forward_swiglu_impl(be, a.h2, tr->WM(tr->P(l, P_FG)), a.a, a.m, tr->ld_au, N, d, F));   // a, u and m = silu(a) u from one product
    } else {
      OJC_TRY(linear_forward_impl(be, a.h2, A, tr->WM(tr->P(l, P_FG)), A, a.a, A, N, d, tr->ld_au, nullptr));
      OJC_TRY(swiglu_rows_forward(be, (const bf16*)a.a, tr->ld_au, (bf16*)a.m, N, F));
    }
    OJC_TRY(linear_forward_impl(be, a.m, A, tr->WM(tr->P(l, P_FD)), A, x_next, OJC_F32, N, F, d, nullptr, true));  // x2 = x1 + down(m)
    return OJC_OK;
  }
  OJC_TRY(linear_forward_impl(be, a.h2, A, tr->WM(tr->P(l, P_FG)), A, a.a, A, N, d, F, nullptr));
  OJC_TRY(linear_forward_impl(be, a.h2, A, tr->WM(tr->P(l, P_FU)), A, a.u, A, N, d, F, nullptr));
  if ((N * F) % 4 == 0) OJC_TRY(swiglu_forward_impl(be, a.a, a.u, a.m, A, N * F));
  else {
    ojc_tensor ta = T1(a.a, A, N * F), tu = T1(a.u, A, N * F), tm = T1(a.m, A, N * F);
    OJC_TRY(ojc_silu_forward(be, &ta, &tm));
    OJC_TRY(ojc_mul_forward(be, &tm, &tu, &tm));
  }
  OJC_TRY(linear_forward_impl(be, a.m, A, tr->WM(tr->P(l, P_FD)), A, x_next, OJC_F32, N, F, d, add_in_place ? nullptr : a.x1, add_in_place));  // x2 = x1 + down(m)
  return OJC_OK;
}

ojc_status forward_hidden(ojc_trainer* tr, const uint32_t* ids_dev) {
  ojc_backend* be = tr->be;
  const ojc_model_spec& s = tr->spec;
  const int64_t d = s.n_embd, H = s.n_head, Hkv = s.n_kv_head, dh = s.head_dim, F = s.hidden, N = tr->N, B = tr->B, T = tr->T;
  const int64_t qw = H * dh, kvw = Hkv * dh, L = s.n_layer;
  const int32_t A = tr->act_dt;
  const float eps = s.rms_eps;
  ojc_tensor cos_t = T2(tr->cos_t, OJC_F32, T, dh), sin_t = T2(tr->sin_t, OJC_F32, T, dh);
  {
    ojc_tensor table = T2(tr->w + tr->params[0].offset, OJC_F32, s.vocab, d), ids = T1((void*)ids_dev, OJC_U32, N), out = T2(tr->acts[0].x, OJC_F32, N, d);
    OJC_TRY(ojc_embedding_forward(be, &table, &ids, &out));
  }
  for (int64_t l = 0; l < L; ++l) OJC_TRY(block_forward(tr, l));
  ojc_tensor xf = T2(tr->x_final, OJC_F32, N, d), hf = T2(tr->hf, A, N, d), nf = T1(tr->W(tr->params.back()), OJC_F32, d);
  return rms_forward_impl(be, &xf, &nf, eps, &hf);
}

ojc_status record_ready(ojc_trainer* tr, int first_param_done) {
  // a bucket is complete once every parameter from its first one to the end of the table has its gradient
  for (auto& b : tr->buckets)
    if (!b.recorded && b.first_param >= first_param_done && b.first_param != 0) {
      OJC_CUDA(tr->be, cudaEventRecord(b.ready, tr->be->stream), "bucket_ready");
      b.recorded = true;
    }
  return OJC_OK;
}

// While alive, library calls issue on the trainer's side stream with the side workspace (the step driver is single-threaded).
struct SideLane {
  ojc_trainer* tr; bool profile;
  explicit SideLane(ojc_trainer* t) : tr(t), profile(t->be->profile_gemm) { swap(); tr->be->profile_gemm = false; }
  ~SideLane() { swap(); tr->be->profile_gemm = profile; }
  void swap() {
    std::swap(tr->be->stream, tr->side_stream);
    std::swap(tr->be->scratch, tr->side_scratch);
    std::swap(tr->be->scratch_bytes, tr->side_scratch_bytes);
  }
};

// ---------------------------------------------------------------------------------------------- backward
ojc_status backward(ojc_trainer* tr, const uint32_t* ids_dev, const uint32_t* targets_dev) {
  ojc_backend* be = tr->be;
  const ojc_model_spec& s = tr->spec;
  const int64_t d = s.n_embd, H = s.n_head, Hkv = s.n_kv_head, dh = s.head_dim, F = s.hidden, N = tr->N, B = tr->B, T = tr->T, V = s.vocab;
  const int64_t qw = H * dh, kvw = Hkv * dh, L = s.n_layer;
  const int32_t A = tr->act_dt;
  const bool bf = A == OJC_BF16;
  const float eps = s.rms_eps;
  ojc_tensor cos_t = T2(tr->cos_t, OJC_F32, T, dh), sin_t = T2(tr->sin_t, OJC_F32, T, dh);
  const Param& tok = tr->params[0];
  for (auto& b : tr->buckets) b.recorded = false;
  // fused tied-head loss: both gradients come out of the forward call (ojas-autograd/src/tape.rs:1766-1779)
  OJC_TRY(linear_ce_impl(be, tr->hf, A, tr->WM(tok), A, targets_dev, N, d, V, tr->cfg.has_ignore, tr->cfg.ignore_index, tr->cfg.ce_chunk_rows, tr->stats, tr->g_h,
                         OJC_F32, tr->G(tok), false, tr->seed_now));
  {
    ojc_tensor xf = T2(tr->x_final, OJC_F32, N, d), nf = T1(tr->W(tr->params.back()), OJC_F32, d), gy = T2(tr->g_h, OJC_F32, N, d), gx = T2(tr->gx, OJC_F32, N, d);
    ojc_tensor gnf = T1(tr->G(tr->params.back()), OJC_F32, d);
    OJC_TRY(rms_backward_impl(be, &xf, &nf, &gy, eps, &gx, &gnf, false, false, A == OJC_BF16 ? (bf16*)tr->gx_b : nullptr));
  }
  OJC_TRY(record_ready(tr, (int)tr->params.size() - 1));
  // the residual gradient as a matmul operand: f32 in the f32 tier, the bf16 copy the norm backward kernels write under autocast
  // Under autocast the bf16 copy alternates between two buffers: the one the block's second norm writes (read by the output
  // projection's gradients) and the one the first norm writes (read by the next block's down-projection gradients), so the
  // weight gradients still running on the side lane never read a buffer the main stream is about to rewrite mid-block.
  const void* gxo = bf ? tr->gx_b : (void*)tr->gx;
  bool have_v0 = false;
  // fn's inputs are final on the main stream now; run it on the side lane (or in place when there is none)
  const bool lane = bf && tr->side_stream != nullptr && tr->side_enabled;
  // (only under NonFinitePolicy::Abort: a non-finite gradient found after blocks were stepped poisons the trainer)
  const bool eager = lane && tr->eager_request && tr->cfg.optimizer == 0 && !(tr->cfg.grad_clip > 0.0f) && L > 0 && tr->cfg.on_nonfinite == 0 && !tr->comm;
  tr->eager_used = eager;
  tr->eager_begin = tr->eager_end = eager ? tr->params.back().offset : 0;   // grows downwards block by block
  auto on_side = [&](auto&& fn) -> ojc_status {
    if (!lane) return fn();
    OJC_CUDA(be, cudaEventRecord(tr->ev_main, be->stream), "side_lane");
    OJC_CUDA(be, cudaStreamWaitEvent(tr->side_stream, tr->ev_main, 0), "side_lane");
    SideLane guard(tr);
    return fn();
  };
  // the main stream goes no further until the side lane has drained (before a buffer the lane still reads is rewritten)
  auto join_side = [&]() -> ojc_status {
    if (!lane) return OJC_OK;
    OJC_CUDA(be, cudaEventRecord(tr->ev_side, tr->side_stream), "side_lane");
    OJC_CUDA(be, cudaStreamWaitEvent(be->stream, tr->ev_side, 0), "side_lane");
    be->finish.used = 0;     // every finishing kernel queued so far is ordered before what the main stream does next
    return OJC_OK;
  };
  // The small finishing reductions of the norm, QK-norm and gate-bias gradients (a few blocks each) go to the side lane too.
  struct FinishScope {
    ojc_backend* be;
    FinishScope(ojc_backend* b, ojc_trainer* t, bool on) : be(b) {
      if (on) { be->finish.stream = t->side_stream; be->finish.ev = t->ev_finish; be->finish.pool = (char*)t->finish_pool; be->finish.pool_bytes = ojc_trainer::FINISH_POOL_BYTES; be->finish.used = 0; be->finish.active = true; }
    }
    ~FinishScope() { be->finish.active = false; }
  } finish_scope(be, tr, lane);
  // a bucket's event must also cover the lane's work: join before the first event a call records
  auto ready = [&](int first_param_done) -> ojc_status {
    for (auto& b : tr->buckets)
      if (!b.recorded && b.first_param >= first_param_done && b.first_param != 0) { OJC_TRY(join_side()); break; }
    return record_ready(tr, first_param_done);
  };
  for (int64_t l = L - 1; l >= 0; --l) {
    LayerActs& a = tr->acts[l];
    // Activation checkpointing: only the block inputs were kept, every block works in the same activation buffers. The last
    // block's are still in place from the forward pass; the others are recomputed here (same kernels, same bits), after the
    // side lane has finished reading the previous occupant's. Block 0 keeps buffers of its own.
    if (tr->cfg.checkpoint_blocks && l + 1 < L && l > 0) {
      OJC_TRY(join_side());
      OJC_TRY(block_forward(tr, l));
    }
    // x2 = x1 + down(m)
    const bool fl = tr->fused_lin;
    // With gate and up side by side the SwiGLU gradient leaves the product's epilogue directly and g_m is never stored.
    const bool in_epilogue = fl && g_mlp_epilogue_variant == 0 &&
                             linear_backward_input_swiglu_eligible(be, tr->WM(tr->P(l, P_FD)), gxo, a.a, tr->g_a, tr->ld_au, N, F, d);
    if (in_epilogue) OJC_TRY(linear_backward_input_swiglu_impl(be, tr->WM(tr->P(l, P_FD)), gxo, a.a, tr->g_a, tr->ld_au, N, F, d));
    else OJC_TRY(linear_backward_input_impl(be, tr->WM(tr->P(l, P_FD)), A, gxo, A, tr->g_m, A, N, F, d, false));
    OJC_TRY(on_side([&] { return linear_backward_weight_impl(be, a.m, A, gxo, A, tr->G(tr->P(l, P_FD)), N, F, d, false); }));
    const int64_t sq = fl ? tr->ld_qkv : qw, skv = fl ? tr->ld_qkv : kvw;
    if (in_epilogue) {}
    else if (fl) OJC_TRY(swiglu_rows_backward(be, (const bf16*)a.a, (const bf16*)tr->g_m, (bf16*)tr->g_a, tr->ld_au, N, F));
    else if ((N * F) % 4 == 0) OJC_TRY(swiglu_backward_impl(be, a.a, a.u, tr->g_m, tr->g_a, tr->g_u, A, N * F));
    else {
      ojc_tensor ta = T1(a.a, A, N * F), tu = T1(a.u, A, N * F), gm = T1(tr->g_m, A, N * F), ga = T1(tr->g_a, A, N * F), gu = T1(tr->g_u, A, N * F);
      OJC_TRY(join_side());                // the down-projection's weight gradient on the side lane still reads m
      ojc_tensor sil = T1(a.m, A, N * F);  // silu(a) recomputed into the slot of m, which is no longer needed
      OJC_TRY(ojc_silu_forward(be, &ta, &sil));
      OJC_TRY(ojc_mul_backward(be, &sil, &tu, &gm, &ga, &gu));  // ga = g_silu for now
      OJC_TRY(ojc_silu_backward(be, &ta, &ga, &ga));
    }
    if (fl) {
      OJC_TRY(linear_backward_input_impl(be, tr->WM(tr->P(l, P_FG)), A, tr->g_a, A, tr->g_h2, OJC_F32, N, d, tr->ld_au, false));
      OJC_TRY(on_side([&] { return linear_backward_weight_impl(be, a.h2, A, tr->g_a, A, tr->G(tr->P(l, P_FG)), N, d, tr->ld_au, false); }));
    } else {
      OJC_TRY(linear_backward_input_impl(be, tr->WM(tr->P(l, P_FU)), A, tr->g_u, A, tr->g_h2, OJC_F32, N, d, F, false));
      OJC_TRY(on_side([&] { return linear_backward_weight_impl(be, a.h2, A, tr->g_u, A, tr->G(tr->P(l, P_FU)), N, d, F, false); }));
      OJC_TRY(linear_backward_input_impl(be, tr->WM(tr->P(l, P_FG)), A, tr->g_a, A, tr->g_h2, OJC_F32, N, d, F, true));
      OJC_TRY(on_side([&] { return linear_backward_weight_impl(be, a.h2, A, tr->g_a, A, tr->G(tr->P(l, P_FG)), N, d, F, false); }));
    }
    {
      ojc_tensor x1 = T2(a.x1, OJC_F32, N, d), n2 = T1(tr->W(tr->P(l, P_NORM2)), OJC_F32, d), gy = T2(tr->g_h2, OJC_F32, N, d), gx = T2(tr->gx, OJC_F32, N, d);
      ojc_tensor gn2 = T1(tr->G(tr->P(l, P_NORM2)), OJC_F32, d);
      OJC_TRY(rms_backward_impl(be, &x1, &n2, &gy, eps, &gx, &gn2, false, true, bf ? (bf16*)tr->gx_b2 : nullptr));  // gx now holds d/dx1
      if (bf) gxo = tr->gx_b2;
    }
    // x1 = x + o_proj(yg)
    OJC_TRY(linear_backward_input_impl(be, tr->WM(tr->P(l, P_O)), A, gxo, A, tr->g_yg, A, N, qw, d, false));
    OJC_TRY(on_side([&] { return linear_backward_weight_impl(be, a.yg, A, gxo, A, tr->G(tr->P(l, P_O)), N, qw, d, false); }));
    // the attention backward's operands, built early: when its tensor-core path will run, the gate's backward (which forms the
    // same dot product) hands it Dr = rowsum(dO . O) and the pass over O and dO that would compute it is dropped
    ojc_tensor at_q = TBHTD(a.qr, A, B, T, H, dh), at_k = TBHTD(a.kr, A, B, T, Hkv, dh), at_y = TBHTD(a.y, A, B, T, H, dh);
    ojc_tensor at_v = l > 0 ? TBHTD(a.v, A, B, T, Hkv, dh) : TBHTD(a.rawv, A, B, T, Hkv, dh, skv);
    ojc_tensor at_gy = TBHTD(tr->g_y, A, B, T, H, dh), at_gq = TBHTD(tr->g_qr, A, B, T, H, dh), at_gk = TBHTD(tr->g_kr, A, B, T, Hkv, dh), at_gv = TBHTD(tr->g_v, A, B, T, Hkv, dh);
    const bool dr_from_gate = tr->gate_ld && tr->dr && sdpa_backward_takes_dr(be, &at_q, &at_k, &at_v, &at_y, &at_gy, &at_gq, &at_gk, &at_gv, s.window);
    if (tr->gate_ld) {
      const int ld = tr->gate_ld;
      OJC_TRY(gate_apply_backward(be, a.scales, (const bf16*)a.y, (const bf16*)tr->g_yg, (bf16*)tr->g_y, tr->gate_gz, ld, tr->G(tr->P(l, P_GB)), N, (int)H, (int)dh,
                                  dr_from_gate ? tr->dr : nullptr, (int)T));
      OJC_TRY(linear_backward_input_impl(be, tr->WM(tr->P(l, P_GW)), A, tr->gate_gz, A, tr->g_h, OJC_F32, N, d, ld, false));   // d/dh = gz . Wg (padding columns of gz are zero)
      OJC_TRY(on_side([&]() -> ojc_status {
        OJC_TRY(linear_backward_weight_impl(be, a.h, A, tr->gate_gz, A, tr->gate_gw, N, d, ld, false));                        // [ld, d]; rows past H are zero
        OJC_CUDA(be, cudaMemcpyAsync(tr->G(tr->P(l, P_GW)), tr->gate_gw, (size_t)H * d * 4, cudaMemcpyDeviceToDevice, be->stream), "per_head_sigmoid_gate_backward");
        return OJC_OK;
      }));
    } else {
      ojc_tensor h = T2(a.h, A, N, d), gw = T2((void*)tr->WM(tr->P(l, P_GW)), A, H, d), gb = T1(tr->W(tr->P(l, P_GB)), OJC_F32, H);
      ojc_tensor y = T2(a.y, A, N * H, dh), gyg = T2(tr->g_yg, A, N * H, dh), sc = T2(a.scales, OJC_F32, N, H), gh = T2(tr->g_h, OJC_F32, N, d), gy = T2(tr->g_y, A, N * H, dh);
      OJC_TRY(gate_backward_impl(be, &h, &gw, &gb, &y, &gyg, &sc, &gh, tr->G(tr->P(l, P_GW)), tr->G(tr->P(l, P_GB)), &gy, false));
    }
    {
      ojc_tensor lse = T1(a.lse, OJC_F32, B * H * T);
      lse.rank = 3; lse.shape[0] = B; lse.shape[1] = H; lse.shape[2] = T; lse.stride[0] = H * T; lse.stride[1] = T; lse.stride[2] = 1;
      bool taken = false;
      if (dr_from_gate) OJC_TRY(sdpa_backward_with_dr(be, &at_q, &at_k, &at_v, &at_y, &lse, &at_gy, s.window, &at_gq, &at_gk, &at_gv, tr->dr, &taken));
      if (!taken) OJC_TRY(ojc_causal_sdpa_backward(be, &at_q, &at_k, &at_v, &at_y, &lse, &at_gy, s.window, &at_gq, &at_gk, &at_gv));
    }
    const void* g_rawv = tr->g_v;
    if (fl) {
      if (l > 0) {
        OJC_TRY(vres_rows_backward(be, (const bf16*)a.rawv, skv, (const bf16*)tr->acts[0].rawv, skv, tr->W(tr->P(l, P_LAMBDA)), (const bf16*)tr->g_v,
                                   (bf16*)tr->g_rawv, skv, tr->gv0_acc, !have_v0, tr->G(tr->P(l, P_LAMBDA)), N, kvw));
        have_v0 = true;
      } else {
        OJC_TRY(vres_root_backward(be, have_v0 ? tr->gv0_acc : nullptr, (const bf16*)tr->g_v, (bf16*)tr->g_rawv, skv, N, kvw));
      }
      g_rawv = tr->g_rawv;
    } else if (l > 0) {
      ojc_tensor rv = T1(a.rawv, A, N * kvw), v0 = T1(tr->acts[0].rawv, A, N * kvw), lam = T1(tr->W(tr->P(l, P_LAMBDA)), OJC_F32, 1), gv = T1(tr->g_v, A, N * kvw);
      ojc_tensor grv = T1(tr->g_rawv, A, N * kvw), gv0 = T1(tr->g_v0l, A, N * kvw);
      OJC_TRY(vres_backward_impl(be, &rv, &v0, &lam, &gv, &grv, &gv0, tr->G(tr->P(l, P_LAMBDA)), false));
      ojc_tensor acc = T1(tr->gv0_acc, OJC_F32, N * kvw);
      if (!have_v0) { OJC_TRY(ojc_fill_zero(be, tr->gv0_acc, (uint64_t)N * kvw * 4)); have_v0 = true; }
      OJC_TRY(ojc_residual_add_forward(be, &acc, &gv0, &acc));
      g_rawv = tr->g_rawv;
    } else if (have_v0) {
      // layer 0's raw v also fed every later layer's blend: add those contributions (gathered in reverse-walk order)
      ojc_tensor acc = T1(tr->gv0_acc, OJC_F32, N * kvw), gv = T1(tr->g_v, A, N * kvw), grv = T1(tr->g_rawv, A, N * kvw);
      OJC_TRY(ojc_residual_add_forward(be, &acc, &gv, &grv));
      g_rawv = tr->g_rawv;
    }
    if (tr->fused_qk) {
      OJC_TRY(qk_norm_rope_backward(be, (const bf16*)a.k, skv, tr->W(tr->P(l, P_KN)), tr->cos_t, tr->sin_t, (const bf16*)tr->g_kr, kvw, (bf16*)tr->g_k, skv,
                                    tr->G(tr->P(l, P_KN)), N, (int)Hkv, (int)dh, (int)T, eps));
      OJC_TRY(qk_norm_rope_backward(be, (const bf16*)a.q, sq, tr->W(tr->P(l, P_QN)), tr->cos_t, tr->sin_t, (const bf16*)tr->g_qr, qw, (bf16*)tr->g_q, sq,
                                    tr->G(tr->P(l, P_QN)), N, (int)H, (int)dh, (int)T, eps));
    } else {
      ojc_tensor gkr = T4(tr->g_kr, A, B, T, Hkv, dh), gkn = T4(tr->g_kn, A, B, T, Hkv, dh), gqr = T4(tr->g_qr, A, B, T, H, dh), gqn = T4(tr->g_qn, A, B, T, H, dh);
      OJC_TRY(rope_impl(be, "rope_half_split_backward", &gkr, &cos_t, &sin_t, &gkn, 1));
      OJC_TRY(rope_impl(be, "rope_half_split_backward", &gqr, &cos_t, &sin_t, &gqn, 1));
      ojc_tensor k = T2(a.k, A, N * Hkv, dh), knw = T1(tr->W(tr->P(l, P_KN)), OJC_F32, dh), gkn2 = T2(tr->g_kn, A, N * Hkv, dh), gk = T2(tr->g_k, A, N * Hkv, dh);
      ojc_tensor gknw = T1(tr->G(tr->P(l, P_KN)), OJC_F32, dh);
      OJC_TRY(rms_backward_impl(be, &k, &knw, &gkn2, eps, &gk, &gknw, false, false));
      ojc_tensor q = T2(a.q, A, N * H, dh), qnw = T1(tr->W(tr->P(l, P_QN)), OJC_F32, dh), gqn2 = T2(tr->g_qn, A, N * H, dh), gq = T2(tr->g_q, A, N * H, dh);
      ojc_tensor gqnw = T1(tr->G(tr->P(l, P_QN)), OJC_F32, dh);
      OJC_TRY(rms_backward_impl(be, &q, &qnw, &gqn2, eps, &gq, &gqnw, false, false));
    }
    if (fl) {
      // d/dh += [gq | gk | gv] . [Wq; Wk; Wv], and the three weight gradients as one [ld_qkv, d] block
      OJC_TRY(linear_backward_input_impl(be, tr->WM(tr->P(l, P_Q)), A, tr->g_q, A, tr->g_h, OJC_F32, N, d, tr->ld_qkv, true));
      OJC_TRY(on_side([&] { return linear_backward_weight_impl(be, a.h, A, tr->g_q, A, tr->G(tr->P(l, P_Q)), N, d, tr->ld_qkv, false); }));
    } else {
      OJC_TRY(linear_backward_input_impl(be, tr->WM(tr->P(l, P_V)), A, g_rawv, A, tr->g_h, OJC_F32, N, d, kvw, true));
      OJC_TRY(on_side([&] { return linear_backward_weight_impl(be, a.h, A, g_rawv, A, tr->G(tr->P(l, P_V)), N, d, kvw, false); }));
      OJC_TRY(linear_backward_input_impl(be, tr->WM(tr->P(l, P_K)), A, tr->g_k, A, tr->g_h, OJC_F32, N, d, kvw, true));
      OJC_TRY(on_side([&] { return linear_backward_weight_impl(be, a.h, A, tr->g_k, A, tr->G(tr->P(l, P_K)), N, d, kvw, false); }));
      OJC_TRY(linear_backward_input_impl(be, tr->WM(tr->P(l, P_Q)), A, tr->g_q, A, tr->g_h, OJC_F32, N, d, qw, true));
      OJC_TRY(on_side([&] { return linear_backward_weight_impl(be, a.h, A, tr->g_q, A, tr->G(tr->P(l, P_Q)), N, d, qw, false); }));
    }
    {
      ojc_tensor x = T2(a.x, OJC_F32, N, d), n1 = T1(tr->W(tr->P(l, P_NORM1)), OJC_F32, d), gy = T2(tr->g_h, OJC_F32, N, d), gx = T2(tr->gx, OJC_F32, N, d);
      ojc_tensor gn1 = T1(tr->G(tr->P(l, P_NORM1)), OJC_F32, d);
      OJC_TRY(join_side());   // every weight gradient of this layer is in: the buffers the lane read may be rewritten, the bucket events may fire
      OJC_TRY(rms_backward_impl(be, &x, &n1, &gy, eps, &gx, &gn1, false, true, bf ? (bf16*)tr->gx_b : nullptr));
      if (bf) gxo = tr->gx_b;
    }
    if (l == 0 && s.n_layer > 0) OJC_TRY(ojc_fill_zero(be, tr->G(tr->P(0, P_LAMBDA)), 4));  // layer 0's lambda never trains (names.rs:262-268)
    OJC_TRY(ready(1 + (int)l * P_PER_BLOCK));
    if (eager) {
      // this block's slots [begin, end) of the flat buffers; a frozen parameter (block 0's lambda) is stepped around
      const int first = 1 + (int)l * P_PER_BLOCK;
      const int64_t end = tr->params[first + P_PER_BLOCK].offset;
      int64_t begin = tr->params[first].offset;
      const ojc_adamw_config ac{tr->cfg.adam_lr * tr->lr_mult, tr->cfg.adam_beta1, tr->cfg.adam_beta2, tr->cfg.adam_eps, tr->cfg.adam_weight_decay};
      OJC_TRY(on_side([&]() -> ojc_status {
        auto run_range = [&](int64_t b0, int64_t b1) -> ojc_status {
          if (b1 <= b0) return OJC_OK;
          return adamw_device(be, tr->w + b0, tr->g + b0, tr->m1 + b0, tr->m2 + b0, tr->mirror ? tr->mirror + b0 : nullptr, b1 - b0, tr->step, ac, nullptr);
        };
        for (int i = first; i < first + P_PER_BLOCK; ++i) {
          const Param& q = tr->params[i];
          if (q.trains) continue;
          OJC_TRY(run_range(begin, q.offset));
          begin = tr->params[i + 1].offset;
        }
        return run_range(begin, end);
      }));
      tr->eager_begin = tr->params[first].offset;
    }
  }
  OJC_TRY(embedding_backward_impl(be, ids_dev, tr->gx, OJC_F32, tr->G(tok), N, V, d, true));
  OJC_TRY(join_side());   // the last finishing reductions: every gradient is final on the main stream from here
  for (auto& b : tr->buckets) if (b.first_param == 0) OJC_CUDA(be, cudaEventRecord(b.ready, be->stream), "bucket_ready");
  return OJC_OK;
}

// stats layout (device floats): [0] loss of the pass in flight, [1] gradient norm, [2] clip scale, or STEP_CALLED_OFF, [3] steps called
// off since the host last looked, [4] sum of the step's micro-batch losses.
constexpr float STEP_CALLED_OFF = -1.0f;

// Trainer::gradients' loss sum (trainer.rs:975-988): the first micro-batch's loss starts it, the others are added in f32;
// each is scaled by its weight first when the weights are not uniform.
__global__ void loss_sum_kernel(float* stats, float weight, int first, int scaled) {
  const float l = scaled ? stats[0] * weight : stats[0];
  stats[4] = first ? l : stats[4] + l;
}

// The reference finds a non-finite gradient in clip_grad_norm, before any update (trainer.rs:824-838). Here nothing waits for the
// host: when the norm or the loss is not finite, the scale every optimizer kernel reads becomes STEP_CALLED_OFF, which makes
// them return without writing, and the count of called-off steps goes up for the host's one readback.
__global__ void step_gate_kernel(float* stats, int loss_slot) {
  if (!isfinite(stats[1]) || !isfinite(stats[loss_slot])) { stats[2] = STEP_CALLED_OFF; stats[3] += 1.0f; }
}

// LrSchedule::multiplier (ojas-cpu/src/schedule.rs:66-90 cosine, 163-199 wsd): f64, nanolab's order of operations.
ojc_status schedule_multiplier(const ojc_train_config& c, uint64_t step, double* out) {
  const char* op = c.schedule == 2 ? "wsd_schedule" : "cosine_schedule";
  constexpr uint64_t F64_INT_MAX = 1ull << 53;
  constexpr double FLOOR = 0.1;    // COSINE_FLOOR_FRAC, schedule.rs:27
  *out = 1.0;
  if (c.schedule == 0) return OJC_OK;
  if (c.schedule != 1 && c.schedule != 2) return ojc_fail(OJC_ERR_UNSUPPORTED, "lr_schedule", "schedule must be 0 (none), 1 (cosine) or 2 (wsd)");
  if (c.total_steps == 0) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "total steps 0");
  if (c.warmup_steps > F64_INT_MAX || c.total_steps > F64_INT_MAX) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "a step count is not an exact f64 integer");
  if (c.schedule == 2 && !(std::isfinite(c.decay_frac) && c.decay_frac >= 0.0 && c.decay_frac <= 1.0)) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "decay fraction is outside [0, 1]");
  if (step == UINT64_MAX) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "step counter is u64::MAX");
  if (step + 1 > F64_INT_MAX) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "the step is not an exact f64 integer");
  const double step_f = (double)step, warmup = (double)c.warmup_steps;
  if (c.schedule == 2 && step > c.total_steps) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "the step is past the schedule's steps");
  if (step < c.warmup_steps) { *out = (step_f + 1.0) / warmup; return OJC_OK; }
  double m;
  if (c.schedule == 1) {
    const double span = (double)c.total_steps - warmup, denom = span < 1.0 ? 1.0 : span;
    double t = (step_f - warmup) / denom;
    t = t < 0.0 ? 0.0 : (t > 1.0 ? 1.0 : t);
    m = FLOOR + (1.0 - FLOOR) * 0.5 * (1.0 + std::cos(3.14159265358979323846 * t));
  } else {
    const uint64_t decay_steps = (uint64_t)(c.decay_frac * (double)c.total_steps), decay_start = c.total_steps - decay_steps;
    if (step < decay_start) return OJC_OK;
    const double frac = (double)(step - decay_start) / (double)std::max<uint64_t>(decay_steps, 1);
    m = FLOOR + (1.0 - FLOOR) * (1.0 - frac);
  }
  if (!std::isfinite(m)) return ojc_fail(OJC_ERR_NON_FINITE, op, "the multiplier is not finite");
  *out = m;
  return OJC_OK;
}

// scaled_lr (schedule.rs:235-245)
ojc_status scaled_lr(double initial, double mult, double* out) {
  const double lr = initial * mult;
  if (!(std::isfinite(initial) && std::isfinite(mult) && std::isfinite(lr))) return ojc_fail(OJC_ERR_NON_FINITE, "cosine_schedule", "a learning rate is not finite");
  *out = lr;
  return OJC_OK;
}

ojc_status check_ids(const uint32_t* ids, int64_t n, int64_t vocab) {
  // check_ids, ojas-model/src/trainer.rs:1054-1065 and ojas-cpu/src/pointwise.rs:285-295: refused on the host, before anything is launched
  for (int64_t i = 0; i < n; ++i) if (ids[i] >= (uint64_t)vocab) return ojc_fail(OJC_ERR_OUT_OF_RANGE, "embedding_forward", "token id outside the vocabulary");
  return OJC_OK;
}

ojc_status check_live(ojc_trainer* tr, const char* op) {
  if (!tr) return ojc_fail(OJC_ERR_BACKEND, op, "null trainer");
  OJC_ALIVE(tr->be, op);
  if (tr->poisoned) return ojc_fail(OJC_ERR_POISONED, op, "an earlier optimizer phase failed; the trainer state is not trustworthy (TrainState::Poisoned)");
  return OJC_OK;
}

}  // namespace

extern "C" {

ojc_status ojc_trainer_open(ojc_backend* be, const ojc_model_spec* spec, const ojc_train_config* cfg, int64_t batch, int64_t seq, ojc_trainer** out) {
  const char* op = "trainer_open";
  OJC_ALIVE(be, op);
  if (!spec || !cfg || !out) return ojc_fail(OJC_ERR_BACKEND, op, "null argument");
  *out = nullptr;
  const ojc_model_spec& s = *spec;
  if (s.vocab <= 0 || s.n_embd <= 0 || s.n_layer <= 0 || s.n_head <= 0 || s.n_kv_head <= 0 || s.head_dim <= 0 || s.hidden <= 0 || s.max_seq <= 0)
    return ojc_fail(OJC_ERR_SHAPE, op, "every ModelSpec extent must be positive");
  if (s.n_head % s.n_kv_head != 0 || s.head_dim % 2 != 0) return ojc_fail(OJC_ERR_SHAPE, op, "n_head must be a multiple of n_kv_head and head_dim even");
  if (batch <= 0 || seq <= 0 || seq > s.max_seq) return ojc_fail(OJC_ERR_SHAPE, op, "batch and seq must be positive and seq <= max_seq");
  ojc_trainer* tr = new ojc_trainer();
  tr->be = be; tr->spec = s; tr->cfg = *cfg; tr->B = batch; tr->T = seq; tr->N = batch * seq;
  tr->act_dt = cfg->autocast_bf16 ? OJC_BF16 : OJC_F32;
  if (tr->cfg.loss_seed == 0.0f) tr->cfg.loss_seed = 1.0f;
  {
    double m = 1.0;     // a schedule the first step would refuse (total 0, decay fraction outside [0, 1]) is refused here (CosineSchedule::new, schedule.rs:42-55)
    ojc_status sst = schedule_multiplier(tr->cfg, 0, &m);
    if (sst != OJC_OK) { delete tr; return sst; }
    if (cfg->on_nonfinite != 0 && cfg->on_nonfinite != 1) { delete tr; return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "on_nonfinite must be 0 (abort) or 1 (skip_batch)"); }
  }
  build_table(tr);
  const int64_t d = s.n_embd, H = s.n_head, Hkv = s.n_kv_head, dh = s.head_dim, F = s.hidden, N = tr->N, L = s.n_layer;
  const int64_t qw = H * dh, kvw = Hkv * dh;
  const uint64_t es = dtype_size(tr->act_dt);
  auto fail = [&](ojc_status st) { ojc_trainer_close(tr); return st; };
  ojc_status st = OJC_OK;
#define TAKE(ptr, bytes) do { if ((st = take_as(tr, (uint64_t)(bytes), &(ptr))) != OJC_OK) return fail(st); } while (0)
  TAKE(tr->w, tr->flat_n * 4); TAKE(tr->g, tr->flat_n * 4); TAKE(tr->m1, tr->flat_n * 4); TAKE(tr->m2, tr->flat_n * 4);
  if (tr->act_dt == OJC_BF16) { TAKE(tr->mirror, tr->flat_n * 2); }
  for (float* p : {tr->w, tr->g, tr->m1, tr->m2}) if ((st = ojc_fill_zero(be, p, (uint64_t)tr->flat_n * 4)) != OJC_OK) return fail(st);
  if (tr->mirror && (st = ojc_fill_zero(be, tr->mirror, (uint64_t)tr->flat_n * 2)) != OJC_OK) return fail(st);
  if (tr->act_dt == OJC_BF16) {
    tr->fused_qk = qk_norm_rope_supported((int)dh) && qw % 8 == 0 && kvw % 8 == 0;
    // the concatenated-weight GEMMs need the q/k/v (gate/up) slots back to back, i.e. no 64-float slot padding between them
    tr->fused_lin = tr->fused_qk && F % 8 == 0 && d % 8 == 0 && (qw * d) % 64 == 0 && (kvw * d) % 64 == 0 && (F * d) % 64 == 0;
    if (tr->fused_lin) { tr->ld_qkv = qw + 2 * kvw; tr->ld_au = 2 * F; }
  }
  const bool fl = tr->fused_lin;
  tr->acts.resize(L);
  for (int64_t l = 0; l < L; ++l) {
    LayerActs& a = tr->acts[l];
    if (tr->cfg.checkpoint_blocks && l > 0) {
      // every block shares block 1's buffers (block 0 keeps its own q / k / raw v: raw v of block 0 feeds every block's value
      // residual); only the block input is per block
      if (l > 1) { a = tr->acts[1]; TAKE(a.x, N * d * 4); continue; }
    }
    TAKE(a.x, N * d * 4); TAKE(a.x1, N * d * 4); TAKE(a.lse, tr->B * H * tr->T * 4); TAKE(a.scales, N * H * 4);
    TAKE(a.h, N * d * es); TAKE(a.qr, N * qw * es); TAKE(a.kr, N * kvw * es);
    if (fl) {
      TAKE(a.q, N * tr->ld_qkv * es); a.k = (bf16*)a.q + qw; a.rawv = (bf16*)a.q + qw + kvw;
      TAKE(a.a, N * tr->ld_au * es); a.u = (bf16*)a.a + F;
    } else {
      TAKE(a.q, N * qw * es); TAKE(a.k, N * kvw * es); TAKE(a.rawv, N * kvw * es); TAKE(a.a, N * F * es); TAKE(a.u, N * F * es);
    }
    a.v = nullptr;
    if (l > 0) { TAKE(a.v, N * kvw * es); }
    TAKE(a.y, N * qw * es); TAKE(a.yg, N * qw * es); TAKE(a.h2, N * d * es); TAKE(a.m, N * F * es);
  }
  TAKE(tr->x_final, N * d * 4); TAKE(tr->gx, N * d * 4); TAKE(tr->g_h, N * d * 4); TAKE(tr->g_h2, N * d * 4); TAKE(tr->gv0_acc, N * kvw * 4); TAKE(tr->stats, 256);
  TAKE(tr->hf, N * d * es); TAKE(tr->gx_b, N * d * 2); TAKE(tr->gx_b2, N * d * 2); TAKE(tr->g_m, N * F * es);
  TAKE(tr->g_yg, N * qw * es); TAKE(tr->g_y, N * qw * es); TAKE(tr->g_qr, N * qw * es); TAKE(tr->g_kr, N * kvw * es); TAKE(tr->g_v, N * kvw * es);
  if (fl) {
    TAKE(tr->g_a, N * tr->ld_au * es); tr->g_u = (bf16*)tr->g_a + F;
    TAKE(tr->g_q, N * tr->ld_qkv * es); tr->g_k = (bf16*)tr->g_q + qw; tr->g_rawv = (bf16*)tr->g_q + qw + kvw;
  } else {
    TAKE(tr->g_a, N * F * es); TAKE(tr->g_u, N * F * es);
    TAKE(tr->g_q, N * qw * es); TAKE(tr->g_k, N * kvw * es); TAKE(tr->g_rawv, N * kvw * es);
  }
  if (!tr->fused_qk) { TAKE(tr->g_qn, N * qw * es); TAKE(tr->g_kn, N * kvw * es); TAKE(tr->qn, N * qw * es); TAKE(tr->kn, N * kvw * es); }
  if (!fl) { TAKE(tr->g_v0l, N * kvw * es); }
  if (tr->act_dt == OJC_BF16) {
    const int64_t ld = (H + 7) & ~int64_t(7);
    const Param& gwp = tr->P(0, P_GW);
    const bool per_ok = dh % 8 == 0 && (dh / 8) <= 32 && (((dh / 8) & ((dh / 8) - 1)) == 0);
    if (per_ok && d % 8 == 0 && tr->P(L - 1, P_GW).offset + ld * d <= tr->flat_n && gwp.n == H * d) {
      tr->gate_ld = (int)ld;
      TAKE(tr->gate_z, N * ld * 2); TAKE(tr->gate_gz, N * ld * 2); TAKE(tr->gate_gw, ld * d * 4); TAKE(tr->dr, tr->B * H * tr->T * 4);
    }
  }
  TAKE(tr->cos_t, tr->T * dh * 4); TAKE(tr->sin_t, tr->T * dh * 4); TAKE(tr->ids, N * 4); TAKE(tr->targets, N * 4);
#undef TAKE
  std::vector<float> cos_h, sin_h;
  rope_tables_host(s.rope_base, tr->T, dh, cos_h, sin_h);
  if ((st = ojc_upload(be, tr->cos_t, cos_h.data(), cos_h.size() * 4)) != OJC_OK) return fail(st);
  if ((st = ojc_upload(be, tr->sin_t, sin_h.data(), sin_h.size() * 4)) != OJC_OK) return fail(st);
  if ((st = ojc_fill_zero(be, tr->stats, 256)) != OJC_OK) return fail(st);
  // gradient buckets of about 25 MB, filled from the end of the table (the order gradients become final)
  const int64_t bucket_floats = (25ll << 20) / 4;
  int64_t end = tr->flat_n;
  int last = (int)tr->params.size() - 1;
  while (last >= 0) {
    int first = last;
    while (first > 0 && end - tr->params[first].offset < bucket_floats) --first;
    ojc_trainer::Bucket b{tr->params[first].offset, end - tr->params[first].offset, first, nullptr, false};
    if (cudaEventCreateWithFlags(&b.ready, cudaEventDisableTiming) != cudaSuccess) return fail(ojc_fail(OJC_ERR_BACKEND, op, "cannot create an event"));
    tr->buckets.push_back(b);
    end = tr->params[first].offset;
    last = first - 1;
  }
  if (tr->act_dt == OJC_BF16) {
    if (cudaStreamCreateWithFlags(&tr->side_stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&tr->ev_main, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&tr->ev_side, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&tr->ev_finish, cudaEventDisableTiming) != cudaSuccess ||
        cudaMalloc(&tr->finish_pool, ojc_trainer::FINISH_POOL_BYTES) != cudaSuccess)
      return fail(ojc_fail(OJC_ERR_BACKEND, op, "cannot create the weight-gradient stream"));
  }
  *out = tr;
  return OJC_OK;
}

ojc_status ojc_trainer_close(ojc_trainer* tr) {
  if (!tr) return OJC_OK;
  if (tr->be && tr->be->stream) cudaStreamSynchronize(tr->be->stream);
  if (tr->side_stream) { cudaStreamSynchronize(tr->side_stream); cudaStreamDestroy(tr->side_stream); }
  if (tr->ev_main) cudaEventDestroy(tr->ev_main);
  if (tr->ev_side) cudaEventDestroy(tr->ev_side);
  if (tr->side_scratch) cudaFree(tr->side_scratch);
  if (tr->ev_finish) cudaEventDestroy(tr->ev_finish);
  if (tr->ev_bwd_end) cudaEventDestroy(tr->ev_bwd_end);
  if (tr->ev_exchanged) cudaEventDestroy(tr->ev_exchanged);
  if (tr->finish_pool) cudaFree(tr->finish_pool);
  for (void* p : tr->owned) ojc_free(tr->be, p);
  for (auto& b : tr->buckets) if (b.ready) cudaEventDestroy(b.ready);
  delete tr;
  return OJC_OK;
}

int64_t ojc_trainer_param_count(ojc_trainer* tr) { return tr ? (int64_t)tr->params.size() : 0; }

ojc_status ojc_trainer_param_info(ojc_trainer* tr, int64_t index, char* name, int64_t name_cap, int32_t* rank, int64_t* shape2, int32_t* group, int32_t* trains) {
  if (!tr || index < 0 || index >= (int64_t)tr->params.size()) return ojc_fail(OJC_ERR_OUT_OF_RANGE, "trainer_param_info", "parameter index out of range");
  const Param& p = tr->params[index];
  if (name && name_cap > 0) snprintf(name, (size_t)name_cap, "%s", p.name.c_str());
  if (rank) *rank = p.rank;
  if (shape2) { shape2[0] = p.shape[0]; shape2[1] = p.shape[1]; }
  if (group) *group = p.group;
  if (trains) *trains = p.trains ? 1 : 0;
  return OJC_OK;
}

ojc_status ojc_trainer_set_param(ojc_trainer* tr, int64_t index, const float* host, uint64_t count) {
  const char* op = "trainer_set_param";
  OJC_TRY(check_live(tr, op));
  if (index < 0 || index >= (int64_t)tr->params.size()) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "parameter index out of range");
  const Param& p = tr->params[index];
  if ((int64_t)count != p.n) return ojc_fail(OJC_ERR_SHAPE, op, "element count does not match the parameter");
  OJC_TRY(ojc_upload(tr->be, tr->W(p), host, count * 4));
  return refresh_mirror(tr, p);
}

ojc_status ojc_trainer_get_param(ojc_trainer* tr, int64_t index, float* host, uint64_t count) {
  const char* op = "trainer_get_param";
  if (!tr || index < 0 || index >= (int64_t)tr->params.size()) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "parameter index out of range");
  const Param& p = tr->params[index];
  if ((int64_t)count != p.n) return ojc_fail(OJC_ERR_SHAPE, op, "element count does not match the parameter");
  return ojc_download(tr->be, host, tr->W(p), count * 4);
}

ojc_status ojc_trainer_get_grad(ojc_trainer* tr, int64_t index, float* host, uint64_t count) {
  const char* op = "trainer_get_grad";
  if (!tr || index < 0 || index >= (int64_t)tr->params.size()) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "parameter index out of range");
  const Param& p = tr->params[index];
  if ((int64_t)count != p.n) return ojc_fail(OJC_ERR_SHAPE, op, "element count does not match the parameter");
  if (!tr->grads_ready) return ojc_fail(OJC_ERR_BACKEND, op, "no gradients have been computed yet");
  return ojc_download(tr->be, host, tr->G(p), count * 4);
}

// Optimizer state of one parameter for the checkpoint directory (ojas-model/src/checkpoint.rs:225-243): slot 0 is the Muon
// momentum of a matrix or the AdamW first moment of an embedding / vector, slot 1 the AdamW second moment.
static ojc_status moment_slot(ojc_trainer* tr, const char* op, int64_t index, int32_t slot, uint64_t count, float** out) {
  if (!tr || index < 0 || index >= (int64_t)tr->params.size()) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "parameter index out of range");
  const Param& p = tr->params[index];
  if ((int64_t)count != p.n) return ojc_fail(OJC_ERR_SHAPE, op, "element count does not match the parameter");
  if (!p.trains) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "a frozen parameter has no optimizer state");
  const bool muon = tr->cfg.optimizer == 1 && p.group == GROUP_MUON;
  if (slot < 0 || slot > 1 || (slot == 1 && muon)) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "no such moment for this parameter's optimizer group");
  *out = (slot == 0 ? tr->m1 : tr->m2) + p.offset;
  return OJC_OK;
}

ojc_status ojc_trainer_get_moment(ojc_trainer* tr, int64_t index, int32_t slot, float* host, uint64_t count) {
  float* dev = nullptr;
  OJC_TRY(moment_slot(tr, "trainer_get_moment", index, slot, count, &dev));
  return ojc_download(tr->be, host, dev, count * 4);
}

ojc_status ojc_trainer_set_moment(ojc_trainer* tr, int64_t index, int32_t slot, const float* host, uint64_t count) {
  OJC_TRY(check_live(tr, "trainer_set_moment"));
  float* dev = nullptr;
  OJC_TRY(moment_slot(tr, "trainer_set_moment", index, slot, count, &dev));
  return ojc_upload(tr->be, dev, host, count * 4);
}

uint64_t ojc_trainer_steps_done(ojc_trainer* tr) { return tr ? tr->step : 0; }

ojc_status ojc_trainer_set_steps_done(ojc_trainer* tr, uint64_t step) {
  OJC_TRY(check_live(tr, "trainer_set_steps_done"));
  if (step == UINT64_MAX) return ojc_fail(OJC_ERR_OUT_OF_RANGE, "trainer_set_steps_done", "step count u64::MAX has no successor");   // next_step, ojas-core/src/backend.rs:220-224
  tr->step = step;
  return OJC_OK;
}

// One forward + backward pass with the seed in tr->seed_now. A host-made failure (ojc_trainer_inject_failure, where 1) fires after
// the forward: nothing the trainer owns (parameters, moments, step count) has changed by then.
static ojc_status gradient_pass(ojc_trainer* tr, const uint32_t* ids_dev, const uint32_t* targets_dev) {
  OJC_TRY(forward_hidden(tr, ids_dev));
  if (tr->inject == 1) { tr->inject = 0; return ojc_fail(OJC_ERR_BACKEND, "trainer_gradients", "injected failure after the forward pass"); }
  return backward(tr, ids_dev, targets_dev);
}

// The schedule's multiplier for the step about to be taken; refusals leave everything unchanged (Trainer::run, trainer.rs:757-759).
static ojc_status begin_step(ojc_trainer* tr) {
  OJC_TRY(schedule_multiplier(tr->cfg, tr->step, &tr->lr_mult));
  if (tr->step == UINT64_MAX) return ojc_fail(OJC_ERR_OUT_OF_RANGE, "Trainer::step", "step count u64::MAX has no successor");   // next_step, ojas-core/src/backend.rs:220-224
  return OJC_OK;
}

ojc_status ojc_trainer_gradients_device(ojc_trainer* tr, const uint32_t* ids_dev, const uint32_t* targets_dev) {
  const char* op = "trainer_gradients";
  OJC_TRY(check_live(tr, op));
  if (!ids_dev || !targets_dev) return ojc_fail(OJC_ERR_PLACEMENT, op, "ids and targets must be device pointers");
  OJC_TRY(begin_step(tr));
  tr->seed_now = tr->cfg.loss_seed; tr->loss_slot = 0; tr->loss_div = 1.0f; tr->run_tokens = (uint64_t)tr->N;
  OJC_TRY(gradient_pass(tr, ids_dev, targets_dev));
  tr->grads_ready = true;
  return OJC_OK;
}

ojc_status ojc_trainer_gradients(ojc_trainer* tr, const uint32_t* ids_host, const uint32_t* targets_host, float* loss_out) {
  const char* op = "trainer_gradients";
  OJC_TRY(check_live(tr, op));
  if (!ids_host || !targets_host) return ojc_fail(OJC_ERR_BACKEND, op, "null ids or targets");
  OJC_TRY(check_ids(ids_host, tr->N, tr->spec.vocab));
  OJC_CUDA(tr->be, cudaMemcpyAsync(tr->ids, ids_host, (size_t)tr->N * 4, cudaMemcpyHostToDevice, tr->be->stream), op);
  OJC_CUDA(tr->be, cudaMemcpyAsync(tr->targets, targets_host, (size_t)tr->N * 4, cudaMemcpyHostToDevice, tr->be->stream), op);
  OJC_TRY(ojc_trainer_gradients_device(tr, tr->ids, tr->targets));
  if (loss_out) OJC_TRY(ojc_download(tr->be, loss_out, tr->stats, 4));
  return OJC_OK;
}

// MicroWeights::new (ojas-model/src/trainer.rs:1083-1119)
struct MicroWeights { std::vector<float> w; bool uniform = true; int64_t run = 0; };
static ojc_status micro_weights(const std::vector<uint64_t>& counts, MicroWeights* out) {
  const char* op = "Trainer::step";
  uint64_t total = 0, first = 0;
  for (uint64_t n : counts) {
    if (total + n < total) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "valid target count overflows u64");
    total += n;
    if (n > 0) { if (!first) first = n; out->run += 1; }
  }
  if (!first) return ojc_fail(OJC_ERR_NON_FINITE, op, "no micro-batch has a valid target: the mean has no denominator");
  for (uint64_t n : counts) out->uniform = out->uniform && (n == 0 || n == first);
  for (uint64_t n : counts) out->w.push_back(n == 0 ? 0.0f : (out->uniform ? 1.0f / (float)out->run : (float)((double)n / (double)total)));
  return OJC_OK;
}

ojc_status ojc_trainer_run_gradients(ojc_trainer* tr, const uint32_t* const* ids_host, const uint32_t* const* targets_host, int64_t k) {
  const char* op = "Trainer::step";
  OJC_TRY(check_live(tr, op));
  ojc_backend* be = tr->be;
  // every refusal that does not depend on the data comes before any work (trainer.rs:754-815)
  OJC_TRY(begin_step(tr));
  constexpr int64_t MAX_ACCUM = 1ll << 24;   // trainer.rs:75
  if (k <= 0 || k > MAX_ACCUM) return ojc_fail(OJC_ERR_OUT_OF_RANGE, op, "the number of micro-batches must be in 1..=2^24");
  if (!ids_host || !targets_host) return ojc_fail(OJC_ERR_BACKEND, op, "null ids or targets");
  for (int64_t i = 0; i < k; ++i) if (!ids_host[i] || !targets_host[i]) return ojc_fail(OJC_ERR_BACKEND, op, "null ids or targets");
  std::vector<uint64_t> counts((size_t)k);
  bool any = false;
  for (int64_t i = 0; i < k; ++i) {
    uint64_t n = 0;
    for (int64_t j = 0; j < tr->N; ++j) n += !(tr->cfg.has_ignore && targets_host[i][j] == tr->cfg.ignore_index);   // valid_targets, trainer.rs:1049-1051
    counts[i] = n; any = any || n > 0;
  }
  // with no valid target anywhere the ids are checked first, so a corrupt batch is OutOfRange and never a skippable NonFinite
  if (!any) for (int64_t i = 0; i < k; ++i) OJC_TRY(check_ids(ids_host[i], tr->N, tr->spec.vocab));
  MicroWeights mw;
  OJC_TRY(micro_weights(counts, &mw));
  for (int64_t i = 0; i < k; ++i) OJC_TRY(check_ids(ids_host[i], tr->N, tr->spec.vocab));
  if (tr->cfg.optimizer == 1) {
    // preflight (trainer.rs:401-426,801-806): the largest Muon group's scratch must fit the budget before any work
    uint64_t need = 0, cap = 0, live = 0;
    for (const Param& p : tr->params) if (p.trains && p.group == GROUP_MUON) need = std::max<uint64_t>(need, muon_scratch_bytes(p.shape[0], p.shape[1], tr->cfg.ns5_bf16 != 0));
    OJC_TRY(ojc_budget(be, &cap, &live, nullptr));
    if (need > cap - std::min(cap, live)) return ojc_fail(OJC_ERR_CAPACITY_EXCEEDED, op, "no room for the optimizer's scratch");
  }
  if (k > 1 && !tr->gacc) OJC_TRY(take_as(tr, (uint64_t)tr->flat_n * 4, &tr->gacc));
  tr->loss_slot = 4; tr->loss_div = mw.uniform ? (float)mw.run : 1.0f; tr->run_tokens = (uint64_t)k * (uint64_t)tr->N;
  tr->grads_ready = false;
  int64_t last = -1, done = 0;
  for (int64_t i = 0; i < k; ++i) if (mw.w[i] != 0.0f) last = i;
  ojc_tensor acc = T1(tr->gacc, OJC_F32, tr->flat_n), g = T1(tr->g, OJC_F32, tr->flat_n);
  for (int64_t i = 0; i < k; ++i) {
    if (mw.w[i] == 0.0f) continue;          // no valid target: contributes nothing and is not run (trainer.rs:925-931)
    OJC_CUDA(be, cudaMemcpyAsync(tr->ids, ids_host[i], (size_t)tr->N * 4, cudaMemcpyHostToDevice, be->stream), op);
    OJC_CUDA(be, cudaMemcpyAsync(tr->targets, targets_host[i], (size_t)tr->N * 4, cudaMemcpyHostToDevice, be->stream), op);
    tr->seed_now = mw.w[i] * tr->cfg.loss_seed;
    OJC_TRY(gradient_pass(tr, tr->ids, tr->targets));
    // accumulate_grad in micro-batch order (trainer.rs:969-974): the sum of the earlier micro-batches waits in gacc while a backward
    // writes g; the last one adds the two into g, where the buckets, the clip and the optimizer read (a + b == b + a bit for bit)
    if (done > 0 && i == last) OJC_TRY(ojc_accumulate_grad(be, &g, &acc));
    else if (done > 0) OJC_TRY(ojc_accumulate_grad(be, &acc, &g));
    else if (i != last) OJC_CUDA(be, cudaMemcpyAsync(tr->gacc, tr->g, (size_t)tr->flat_n * 4, cudaMemcpyDeviceToDevice, be->stream), op);
    loss_sum_kernel<<<1, 1, 0, be->stream>>>(tr->stats, mw.w[i], done == 0, !mw.uniform && mw.w[i] != 1.0f);
    OJC_LAUNCHED(be, op);
    done += 1;
  }
  // the bucket events of the last backward predate the final sum: a data-parallel exchange must wait for it
  if (done > 1) for (auto& b : tr->buckets) OJC_CUDA(be, cudaEventRecord(b.ready, be->stream), "bucket_ready");
  tr->grads_ready = true;
  return OJC_OK;
}

static ojc_status finish_step(ojc_trainer* tr, ojc_step_report* report);

// Sum the gradient buckets across the ranks of the trainer's communicator (nothing to do without one).
static ojc_status exchange(ojc_trainer* tr) {
  if (!tr->comm || ojc_comm_world(tr->comm) <= 1) return OJC_OK;
  ojc_backend* be = tr->be;
  if (!tr->ev_bwd_end) {
    OJC_CUDA(be, cudaEventCreate(&tr->ev_bwd_end), "exchange");
    OJC_CUDA(be, cudaEventCreate(&tr->ev_exchanged), "exchange");
  }
  OJC_CUDA(be, cudaEventRecord(tr->ev_bwd_end, be->stream), "exchange");
  OJC_TRY(ojc_allreduce_start(tr->comm, tr));
  OJC_TRY(ojc_allreduce_wait(tr->comm, tr));
  OJC_CUDA(be, cudaEventRecord(tr->ev_exchanged, be->stream), "exchange");
  tr->exchange_timed = true;
  return OJC_OK;
}

ojc_status ojc_trainer_apply(ojc_trainer* tr, float* grad_norm_out) {
  const char* op = "trainer_apply";
  OJC_TRY(check_live(tr, op));
  if (!tr->grads_ready) return ojc_fail(OJC_ERR_BACKEND, op, "no gradients to apply");
  ojc_backend* be = tr->be;
  const float* gp = tr->g;
  const int64_t glen = tr->flat_n;
  const bool clip = tr->cfg.grad_clip > 0.0f;
  // this step's learning rates (optimizer_configs, trainer.rs:860-883); a refusal here leaves everything unchanged
  OJC_TRY(begin_step(tr));
  double adam_lr = 0.0, matrix_lr = 0.0;
  OJC_TRY(scaled_lr(tr->cfg.adam_lr, tr->lr_mult, &adam_lr));
  OJC_TRY(scaled_lr(tr->cfg.matrix_lr, tr->lr_mult, &matrix_lr));
  // stats[0] loss, [1] grad norm, [2] clip scale. A failure from here on leaves parameters partly stepped: poison.
  auto run = [&]() -> ojc_status {
    OJC_TRY(grad_norm_device(be, &gp, &glen, 1, clip ? tr->cfg.grad_clip : -1.0f, tr->stats + 1));
    step_gate_kernel<<<1, 1, 0, be->stream>>>(tr->stats, tr->loss_slot);
    OJC_LAUNCHED(be, op);
    const float* scale = tr->stats + 2;     // 1 without clipping; STEP_CALLED_OFF when the norm or the loss is not finite
    bool first_update = true;
    auto injected = [&]() -> ojc_status {
      if (!first_update || tr->inject != 2) { first_update = false; return OJC_OK; }
      tr->inject = 0;
      return ojc_fail(OJC_ERR_BACKEND, op, "injected failure inside the optimizer phase");
    };
    // AdamW is element-wise with one configuration per group, so neighbouring AdamW slots go out as one launch over the
    // flat buffers (the zero padding between slots stays zero: p = g = m = v = 0 is a fixed point of the update).
    // the hybrid recipe runs AdamW without decay on embeddings and vectors (ADAM_HYBRID_WEIGHT_DECAY, ojas-cpu/src/train.rs:31-37)
    const ojc_adamw_config ac{adam_lr, tr->cfg.adam_beta1, tr->cfg.adam_beta2, tr->cfg.adam_eps, tr->cfg.optimizer == 1 ? 0.0 : tr->cfg.adam_weight_decay};
    int64_t run_begin = -1, run_end = -1;
    auto flush = [&]() -> ojc_status {
      if (run_begin < 0) return OJC_OK;
      bf16* mir = tr->mirror ? tr->mirror + run_begin : nullptr;
      ojc_status r = adamw_device(be, tr->w + run_begin, tr->g + run_begin, tr->m1 + run_begin, tr->m2 + run_begin, mir, run_end - run_begin, tr->step, ac, scale);
      run_begin = run_end = -1;
      if (r == OJC_OK) r = injected();
      return r;
    };
    // Muon matrices are stepped in groups of one shape (batched Newton-Schulz products): gather them here, in table order
    std::vector<std::pair<std::pair<int64_t, int64_t>, std::vector<const Param*>>> muon_groups;
    for (const Param& p : tr->params) {
      const int64_t slot_end = p.offset + ((p.n + 63) & ~int64_t(63));
      if (!p.trains || (p.offset >= tr->eager_begin && p.offset < tr->eager_end)) { OJC_TRY(flush()); continue; }   // frozen, or stepped during backward
      if (tr->cfg.optimizer == 1 && p.group == GROUP_MUON) {
        OJC_TRY(flush());
        const std::pair<int64_t, int64_t> shape{p.shape[0], p.shape[1]};
        auto it = std::find_if(muon_groups.begin(), muon_groups.end(), [&](const auto& gr) { return gr.first == shape; });
        if (it == muon_groups.end()) { muon_groups.push_back({shape, {}}); it = muon_groups.end() - 1; }
        it->second.push_back(&p);
      } else {
        if (run_begin < 0) run_begin = p.offset;
        else if (p.offset != run_end) { OJC_TRY(flush()); run_begin = p.offset; }
        run_end = slot_end;
      }
    }
    OJC_TRY(flush());
    const ojc_muon_config mc{matrix_lr, tr->cfg.muon_momentum, tr->cfg.muon_weight_decay, 1, tr->cfg.ns5_bf16};
    // Split across ranks: matrix j of a shape group belongs to rank j % world, which alone orthogonalises it; the others receive
    // its new parameters afterwards (every rank saw the same reduced gradient and the same clip scale, so the result is what an
    // unsplit step gives, and a called-off step broadcasts unchanged parameters).
    const int world = tr->comm ? ojc_comm_world(tr->comm) : 1, me = tr->comm ? ojc_comm_rank(tr->comm) : 0;
    const bool split = tr->shard_muon && world > 1;
    std::vector<void*> bc_ptr; std::vector<uint64_t> bc_count; std::vector<int32_t> bc_root; std::vector<const Param*> received;
    for (auto& gr : muon_groups) {
      if (split) {
        std::vector<const Param*> mine;
        for (size_t j = 0; j < gr.second.size(); ++j) {
          const Param* q = gr.second[j];
          const int owner = (int)(j % (size_t)world);
          bc_ptr.push_back(tr->W(*q)); bc_count.push_back((uint64_t)q->n); bc_root.push_back(owner);
          if (owner == me) mine.push_back(q); else received.push_back(q);
        }
        gr.second.swap(mine);
      }
      const size_t chunk = 48;   // the group kernels' pointer table
      for (size_t first = 0; first < gr.second.size(); first += chunk) {
        const size_t count = std::min(chunk, gr.second.size() - first);
        std::vector<float*> pp(count), mm(count); std::vector<const float*> gg(count); std::vector<bf16*> mir(count);
        for (size_t i = 0; i < count; ++i) {
          const Param& q = *gr.second[first + i];
          pp[i] = tr->W(q); gg[i] = tr->G(q); mm[i] = tr->m1 + q.offset; mir[i] = tr->mirror ? tr->mirror + q.offset : nullptr;
        }
        OJC_TRY(muon_group_device(be, pp.data(), gg.data(), mm.data(), tr->mirror ? mir.data() : nullptr, (int64_t)count, gr.first.first, gr.first.second, mc, scale));
        OJC_TRY(injected());
      }
    }
    if (split && !bc_ptr.empty()) {
      OJC_TRY(ojc_comm_broadcast_many(tr->comm, bc_ptr.data(), bc_count.data(), bc_root.data(), (int64_t)bc_ptr.size(), OJC_F32));
      for (const Param* q : received) OJC_TRY(refresh_mirror(tr, *q));
    }
    return OJC_OK;
  };
  ojc_status st = run();
  if (st != OJC_OK) { tr->poisoned = true; return st; }
  tr->step += 1;
  tr->grads_ready = false;
  tr->eager_begin = tr->eager_end = 0;
  if (grad_norm_out) {
    ojc_step_report rep{};
    st = finish_step(tr, &rep);
    *grad_norm_out = rep.grad_norm;
  }
  return st;
}

// The one readback of the step: loss, norm, the called-off count and the deferred fault word (Trainer::finish, trainer.rs:1031-1046).
static ojc_status finish_step(ojc_trainer* tr, ojc_step_report* report) {
  float host[5] = {0, 0, 1, 0, 0};
  ojc_status st = ojc_download(tr->be, host, tr->stats, 20);
  const uint64_t called_off = host[3] > 0.0f ? (uint64_t)host[3] : 0;
  if (report) {
    report->loss = host[tr->loss_slot] / tr->loss_div;     // MicroWeights::report (trainer.rs:1122-1129)
    report->grad_norm = host[1]; report->tokens = tr->run_tokens; report->lr_multiplier = tr->lr_mult;
  }
  if (called_off && (st == OJC_OK || st == OJC_ERR_NON_FINITE)) {
    // the optimizer kernels returned without writing: parameters, moments and the step count are what they were
    cudaMemsetAsync(tr->stats + 3, 0, 4, tr->be->stream);
    tr->step -= std::min<uint64_t>(called_off, tr->step);
    if (report) report->step = tr->step;
    if (tr->eager_used) tr->poisoned = true;               // some blocks had been stepped under backward already
    return st == OJC_OK ? ojc_fail(OJC_ERR_NON_FINITE, "Trainer::step", "the loss or the gradient norm is not finite; no parameter was updated") : st;
  }
  if (st != OJC_OK) { tr->poisoned = true; return st; }
  if (report) report->step = tr->step;
  if (!std::isfinite(host[tr->loss_slot])) { tr->poisoned = true; return ojc_fail(OJC_ERR_NON_FINITE, "Trainer::step", "the loss is not finite"); }
  tr->consecutive_skips = 0;     // any committed step ends a run of skips (trainer.rs:849-850)
  return OJC_OK;
}

ojc_status ojc_trainer_finish(ojc_trainer* tr, ojc_step_report* report) {
  OJC_TRY(check_live(tr, "trainer_finish"));
  return finish_step(tr, report);
}

ojc_status ojc_trainer_step_device(ojc_trainer* tr, const uint32_t* ids_dev, const uint32_t* targets_dev, ojc_step_report* report) {
  if (tr) tr->eager_request = true;        // gradients and apply in one call: the optimizer may start during backward
  ojc_status st = ojc_trainer_gradients_device(tr, ids_dev, targets_dev);
  if (tr) tr->eager_request = false;
  if (st != OJC_OK) { if (tr && tr->eager_end > tr->eager_begin) tr->poisoned = true; return st; }
  OJC_TRY(exchange(tr));
  OJC_TRY(ojc_trainer_apply(tr, nullptr));
  return finish_step(tr, report);
}

ojc_status ojc_trainer_step(ojc_trainer* tr, const uint32_t* ids_host, const uint32_t* targets_host, ojc_step_report* report) {
  if (tr) tr->eager_request = true;
  ojc_status st = ojc_trainer_gradients(tr, ids_host, targets_host, nullptr);
  if (tr) tr->eager_request = false;
  if (st != OJC_OK) { if (tr && tr->eager_end > tr->eager_begin) tr->poisoned = true; return st; }
  OJC_TRY(exchange(tr));
  OJC_TRY(ojc_trainer_apply(tr, nullptr));
  return finish_step(tr, report);
}

ojc_status ojc_trainer_run(ojc_trainer* tr, const uint32_t* const* ids_host, const uint32_t* const* targets_host, int64_t k, ojc_step_report* report) {
  OJC_TRY(ojc_trainer_run_gradients(tr, ids_host, targets_host, k));
  OJC_TRY(exchange(tr));
  OJC_TRY(ojc_trainer_apply(tr, nullptr));
  return finish_step(tr, report);
}

ojc_status ojc_trainer_resolve_failure(ojc_trainer* tr, ojc_status run_status, int32_t* advance_cursor) {
  if (advance_cursor) *advance_cursor = 0;
  if (!tr) return ojc_fail(OJC_ERR_BACKEND, "Trainer::step", "null trainer");
  if (run_status == OJC_OK) { if (advance_cursor) *advance_cursor = 1; return OJC_OK; }
  const bool skippable = !tr->poisoned && tr->cfg.on_nonfinite == 1 && run_status == OJC_ERR_NON_FINITE;
  if (!skippable) return run_status;
  constexpr uint32_t MAX_CONSECUTIVE_SKIPS = 8;   // trainer.rs:81
  if (tr->consecutive_skips >= MAX_CONSECUTIVE_SKIPS)
    return ojc_fail(OJC_ERR_OUT_OF_RANGE, "Trainer::step", "9 consecutive non-finite steps under SkipBatch; the run is not recovering");
  if (advance_cursor) *advance_cursor = 1;
  tr->consecutive_skips += 1;
  return run_status;
}

int32_t ojc_trainer_state(ojc_trainer* tr) { return tr && tr->poisoned ? 1 : 0; }

ojc_status ojc_lr_multiplier(const ojc_train_config* cfg, uint64_t step, double* multiplier) {
  if (!cfg || !multiplier) return ojc_fail(OJC_ERR_BACKEND, "lr_schedule", "null argument");
  return schedule_multiplier(*cfg, step, multiplier);
}

ojc_status ojc_trainer_inject_failure(ojc_trainer* tr, int32_t where) {
  OJC_TRY(check_live(tr, "trainer_inject_failure"));
  if (where < 0 || where > 2) return ojc_fail(OJC_ERR_OUT_OF_RANGE, "trainer_inject_failure", "where must be 0 (none), 1 (gradient pass) or 2 (optimizer phase)");
  tr->inject = where;
  return OJC_OK;
}

ojc_status ojc_trainer_set_comm(ojc_trainer* tr, ojc_comm* comm, int32_t shard_muon) {
  OJC_TRY(check_live(tr, "trainer_set_comm"));
  tr->comm = comm;
  tr->shard_muon = comm != nullptr && shard_muon != 0;
  return OJC_OK;
}

ojc_status ojc_trainer_sync_moments(ojc_trainer* tr) {
  OJC_TRY(check_live(tr, "trainer_sync_moments"));
  if (!tr->comm || !tr->shard_muon || ojc_comm_world(tr->comm) <= 1 || tr->cfg.optimizer != 1) return OJC_OK;
  const int world = ojc_comm_world(tr->comm);
  // the same walk as the optimizer phase: matrix j of a shape group belongs to rank j % world
  std::vector<std::pair<std::pair<int64_t, int64_t>, int64_t>> seen;
  std::vector<void*> ptr; std::vector<uint64_t> count; std::vector<int32_t> root;
  for (const Param& p : tr->params) {
    if (!p.trains || p.group != GROUP_MUON) continue;
    const std::pair<int64_t, int64_t> shape{p.shape[0], p.shape[1]};
    auto it = std::find_if(seen.begin(), seen.end(), [&](const auto& e) { return e.first == shape; });
    if (it == seen.end()) { seen.push_back({shape, 0}); it = seen.end() - 1; }
    ptr.push_back(tr->m1 + p.offset); count.push_back((uint64_t)p.n); root.push_back((int32_t)(it->second % world));
    it->second += 1;
  }
  return ojc_comm_broadcast_many(tr->comm, ptr.data(), count.data(), root.data(), (int64_t)ptr.size(), OJC_F32);
}

ojc_status ojc_trainer_exposed_exchange_ms(ojc_trainer* tr, float* ms) {
  const char* op = "trainer_exposed_exchange_ms";
  if (!tr || !ms) return ojc_fail(OJC_ERR_BACKEND, op, "null argument");
  *ms = 0.0f;
  if (!tr->exchange_timed) return OJC_OK;
  OJC_CUDA(tr->be, cudaEventSynchronize(tr->ev_exchanged), op);
  OJC_CUDA(tr->be, cudaEventElapsedTime(ms, tr->ev_bwd_end, tr->ev_exchanged), op);
  return OJC_OK;
}

ojc_status ojc_trainer_param_checksum(ojc_trainer* tr, uint64_t* hash) {
  const char* op = "trainer_param_checksum";
  if (!tr || !hash) return ojc_fail(OJC_ERR_BACKEND, op, "null argument");
  uint64_t h = 0xcbf29ce484222325ull;
  std::vector<float> host;
  for (const Param& p : tr->params) {
    host.resize((size_t)p.n);
    OJC_TRY(ojc_download(tr->be, host.data(), tr->W(p), (uint64_t)p.n * 4));
    h = ojc_fnv1a64(h, host.data(), (uint64_t)p.n * 4);
  }
  *hash = h;
  return OJC_OK;
}

ojc_status ojc_trainer_logits(ojc_trainer* tr, const uint32_t* ids_host, float* logits_host) {
  const char* op = "trainer_logits";
  OJC_TRY(check_live(tr, op));
  if (!ids_host || !logits_host) return ojc_fail(OJC_ERR_BACKEND, op, "null argument");
  for (int64_t i = 0; i < tr->N; ++i) if (ids_host[i] >= (uint64_t)tr->spec.vocab) return ojc_fail(OJC_ERR_OUT_OF_RANGE, "embedding_forward", "token id outside the vocabulary");
  OJC_TRY(ojc_upload(tr->be, tr->ids, ids_host, (uint64_t)tr->N * 4));
  OJC_TRY(forward_hidden(tr, tr->ids));
  const int64_t V = tr->spec.vocab, d = tr->spec.n_embd;
  void* logits = nullptr;
  OJC_TRY(ojc_alloc(tr->be, (uint64_t)tr->N * V * 4, &logits));
  ojc_status st = linear_forward_impl(tr->be, tr->hf, tr->act_dt, tr->WM(tr->params[0]), tr->act_dt, logits, OJC_F32, tr->N, d, V, nullptr);
  if (st == OJC_OK) st = ojc_download(tr->be, logits_host, logits, (uint64_t)tr->N * V * 4);
  ojc_free(tr->be, logits);
  return st;
}

ojc_status ojc_trainer_overlap_weight_grads(ojc_trainer* tr, int32_t enable) {
  OJC_TRY(check_live(tr, "trainer_overlap_weight_grads"));
  tr->side_enabled = enable != 0;
  return OJC_OK;
}

int64_t ojc_trainer_bucket_count(ojc_trainer* tr) { return tr ? (int64_t)tr->buckets.size() : 0; }
ojc_status ojc_trainer_bucket(ojc_trainer* tr, int64_t index, void** device_ptr, uint64_t* floats) {
  if (!tr || index < 0 || index >= (int64_t)tr->buckets.size()) return ojc_fail(OJC_ERR_OUT_OF_RANGE, "trainer_bucket", "bucket index out of range");
  if (device_ptr) *device_ptr = tr->g + tr->buckets[index].offset;
  if (floats) *floats = (uint64_t)tr->buckets[index].floats;
  return OJC_OK;
}
ojc_status ojc_trainer_bucket_ready_event(ojc_trainer* tr, int64_t index, void** cuda_event) {
  if (!tr || index < 0 || index >= (int64_t)tr->buckets.size()) return ojc_fail(OJC_ERR_OUT_OF_RANGE, "trainer_bucket", "bucket index out of range");
  if (cuda_event) *cuda_event = (void*)tr->buckets[index].ready;
  return OJC_OK;
}

}  // extern "C"
