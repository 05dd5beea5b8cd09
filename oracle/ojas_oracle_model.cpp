// CPU oracle, model level: TEST INFRASTRUCTURE ONLY (see ojas_oracle.cpp).
//
// The nanolab GPT forward loss and its reverse walk, written over the oracle's
// own ops in the order ojas records and replays them:
//   parameters      ojas-model/src/names.rs:188-300 (param_table order)
//   forward         ojas-model/src/block.rs:218-264 (block_with), 351-404 (hidden), 423-447 (forward_loss)
//   backward        ojas-autograd/src/tape.rs:2004-2466 (backward_one), fan-in by accumulate (2565-2591)
// Gradient fan-in adds contributions in reverse-walk order.

#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "ojas_oracle.h"

namespace {

struct Info { std::string name; int64_t rank; int64_t shape[2]; int init; int group; int trains; };

std::vector<Info> table(const orc_spec& s) {
  std::vector<Info> rows;
  const int64_t d = s.n_embd, q = s.n_head * s.head_dim, kv = s.n_kv_head * s.head_dim;
  auto push = [&](std::string name, int64_t rank, int64_t a, int64_t b, int init, bool embedding, bool trains) {
    // ojas-cpu/src/train.rs:54-62: embedding -> AdamW, rank >= 2 -> Muon, else AdamW
    int group = embedding ? ORC_GROUP_ADAMW : (rank >= 2 ? ORC_GROUP_MUON : ORC_GROUP_ADAMW);
    rows.push_back({std::move(name), rank, {a, b}, init, group, trains ? 1 : 0});
  };
  push("tok_emb.weight", 2, s.vocab, d, ORC_INIT_NORMAL, true, true);
  for (int64_t i = 0; i < s.n_layer; ++i) {
    std::string p = "blocks." + std::to_string(i), m = p + ".mixer";
    push(p + ".norm1.weight", 1, d, 1, ORC_INIT_ONES, false, true);
    push(m + ".q_proj.weight", 2, q, d, ORC_INIT_NORMAL, false, true);
    push(m + ".k_proj.weight", 2, kv, d, ORC_INIT_NORMAL, false, true);
    push(m + ".v_proj.weight", 2, kv, d, ORC_INIT_NORMAL, false, true);
    push(m + ".o_proj.weight", 2, d, q, ORC_INIT_ZEROS, false, true);
    push(m + ".q_norm.weight", 1, s.head_dim, 1, ORC_INIT_ONES, false, true);
    push(m + ".k_norm.weight", 1, s.head_dim, 1, ORC_INIT_ONES, false, true);
    push(m + ".gate.weight", 2, s.n_head, d, ORC_INIT_NORMAL, false, true);
    push(m + ".gate.bias", 1, s.n_head, 1, ORC_INIT_ZEROS, false, true);
    push(m + ".vr_lambda", 1, 1, 1, ORC_INIT_ZEROS, false, i != 0);
    push(p + ".norm2.weight", 1, d, 1, ORC_INIT_ONES, false, true);
    push(p + ".ffn.gate.weight", 2, s.hidden, d, ORC_INIT_NORMAL, false, true);
    push(p + ".ffn.up.weight", 2, s.hidden, d, ORC_INIT_NORMAL, false, true);
    push(p + ".ffn.down.weight", 2, d, s.hidden, ORC_INIT_ZEROS, false, true);
  }
  push("norm_f.weight", 1, d, 1, ORC_INIT_ONES, false, true);
  return rows;
}

// Offsets of one block's tensors inside the flat parameter list.
enum { P_NORM1 = 0, P_Q, P_K, P_V, P_O, P_QN, P_KN, P_GW, P_GB, P_LAMBDA, P_NORM2, P_FG, P_FU, P_FD, P_PER_BLOCK };

struct LayerActs {
  std::vector<float> x, h, q, k, rawv, qn, kn, qh, kh, vh, yh, lse, y, yg, x1, h2, a, s, u, m;
};

#define CHECK(expr) do { int st_ = (expr); if (st_ != ORC_OK) return st_; } while (0)

}  // namespace

extern "C" {

int64_t orc_param_count(const orc_spec* spec) { return 2 + P_PER_BLOCK * spec->n_layer; }

int orc_param_info(const orc_spec* spec, int64_t index, char* name, int64_t name_cap, int64_t* rank,
                   int64_t* shape2, int* init_kind, int* group, int* trains) {
  auto rows = table(*spec);
  if (index < 0 || index >= (int64_t)rows.size()) return ORC_OUT_OF_RANGE;
  const Info& r = rows[index];
  if (name && name_cap > 0) std::snprintf(name, (size_t)name_cap, "%s", r.name.c_str());
  if (rank) *rank = r.rank;
  if (shape2) { shape2[0] = r.shape[0]; shape2[1] = r.shape[1]; }
  if (init_kind) *init_kind = r.init;
  if (group) *group = r.group;
  if (trains) *trains = r.trains;
  return ORC_OK;
}

int orc_forward_loss(const orc_spec* sp, const float* const* params, const uint32_t* ids,
                     const uint32_t* targets, int64_t B, int64_t T, int has_ignore, uint32_t ignore,
                     float seed, float* loss, float* const* grads, float* logits_out) {
  const orc_spec& s = *sp;
  const int64_t d = s.n_embd, H = s.n_head, Hkv = s.n_kv_head, dh = s.head_dim, F = s.hidden, V = s.vocab;
  const int64_t L = s.n_layer, N = B * T, qw = H * dh, kvw = Hkv * dh;
  if (T > s.max_seq || B <= 0 || T <= 0) return ORC_SHAPE;
  std::vector<float> cos_t(T * dh), sin_t(T * dh);
  orc_rope_tables(s.rope_base, 0, T, dh, cos_t.data(), sin_t.data());
  const float eps = s.rms_eps;
  auto P = [&](int64_t layer, int which) { return params[1 + layer * P_PER_BLOCK + which]; };
  auto G = [&](int64_t layer, int which) { return grads[1 + layer * P_PER_BLOCK + which]; };
  const float* tok_emb = params[0];
  const float* norm_f = params[1 + L * P_PER_BLOCK];

  std::vector<LayerActs> acts(L);
  std::vector<float> x(N * d), tmp_q(N * qw), tmp_k(N * kvw), v(N * kvw);
  CHECK(orc_embedding_forward(tok_emb, ids, N, V, d, x.data()));
  for (int64_t l = 0; l < L; ++l) {
    LayerActs& a = acts[l];
    a.x = x;
    a.h.resize(N * d); a.q.resize(N * qw); a.k.resize(N * kvw); a.rawv.resize(N * kvw);
    a.qn.resize(N * qw); a.kn.resize(N * kvw); a.qh.resize(N * qw); a.kh.resize(N * kvw); a.vh.resize(N * kvw);
    a.yh.resize(N * qw); a.lse.resize(B * H * T); a.y.resize(N * qw); a.yg.resize(N * qw);
    a.x1.resize(N * d); a.h2.resize(N * d); a.a.resize(N * F); a.s.resize(N * F); a.u.resize(N * F); a.m.resize(N * F);
    CHECK(orc_rms_norm_forward(x.data(), P(l, P_NORM1), N, d, eps, a.h.data()));
    CHECK(orc_linear_forward(a.h.data(), P(l, P_Q), N, d, qw, a.q.data()));
    CHECK(orc_linear_forward(a.h.data(), P(l, P_K), N, d, kvw, a.k.data()));
    CHECK(orc_linear_forward(a.h.data(), P(l, P_V), N, d, kvw, a.rawv.data()));
    CHECK(orc_rms_norm_forward(a.q.data(), P(l, P_QN), N * H, dh, eps, a.qn.data()));
    CHECK(orc_rms_norm_forward(a.k.data(), P(l, P_KN), N * Hkv, dh, eps, a.kn.data()));
    CHECK(orc_rope(a.qn.data(), cos_t.data(), sin_t.data(), N * H, dh, T, H, 0, tmp_q.data()));
    CHECK(orc_rope(a.kn.data(), cos_t.data(), sin_t.data(), N * Hkv, dh, T, Hkv, 0, tmp_k.data()));
    if (l > 0) CHECK(orc_vres_forward(a.rawv.data(), acts[0].rawv.data(), P(l, P_LAMBDA)[0], N * kvw, v.data()));
    else v = a.rawv;
    CHECK(orc_permute_0213(tmp_q.data(), B, T, H, dh, a.qh.data()));
    CHECK(orc_permute_0213(tmp_k.data(), B, T, Hkv, dh, a.kh.data()));
    CHECK(orc_permute_0213(v.data(), B, T, Hkv, dh, a.vh.data()));
    CHECK(orc_causal_sdpa_forward(a.qh.data(), a.kh.data(), a.vh.data(), B, H, Hkv, T, dh, s.window,
                                  a.yh.data(), a.lse.data()));
    CHECK(orc_permute_0213(a.yh.data(), B, H, T, dh, a.y.data()));
    CHECK(orc_gate_forward(a.h.data(), P(l, P_GW), P(l, P_GB), a.y.data(), N, d, H, dh, a.yg.data(), nullptr));
    std::vector<float> o(N * d);
    CHECK(orc_linear_forward(a.yg.data(), P(l, P_O), N, qw, d, o.data()));
    CHECK(orc_add(x.data(), o.data(), N * d, a.x1.data()));
    CHECK(orc_rms_norm_forward(a.x1.data(), P(l, P_NORM2), N, d, eps, a.h2.data()));
    CHECK(orc_linear_forward(a.h2.data(), P(l, P_FG), N, d, F, a.a.data()));
    CHECK(orc_silu_forward(a.a.data(), N * F, a.s.data()));
    CHECK(orc_linear_forward(a.h2.data(), P(l, P_FU), N, d, F, a.u.data()));
    CHECK(orc_mul_forward(a.s.data(), a.u.data(), N * F, a.m.data()));
    CHECK(orc_linear_forward(a.m.data(), P(l, P_FD), N, F, d, o.data()));
    CHECK(orc_add(a.x1.data(), o.data(), N * d, x.data()));
  }
  std::vector<float> hf(N * d);
  CHECK(orc_rms_norm_forward(x.data(), norm_f, N, d, eps, hf.data()));
  if (logits_out) CHECK(orc_linear_forward(hf.data(), tok_emb, N, d, V, logits_out));
  if (!grads) {
    return orc_linear_cross_entropy_mean(hf.data(), tok_emb, targets, N, d, V, has_ignore, ignore, loss, nullptr, nullptr);
  }

  // ---- backward
  std::vector<float> g_hf(N * d);
  float* g_tok = grads[0];
  CHECK(orc_linear_cross_entropy_mean(hf.data(), tok_emb, targets, N, d, V, has_ignore, ignore, loss, g_hf.data(), g_tok));
  if (seed != 1.0f) {  // ojas-autograd/src/tape.rs:2442-2464
    orc_scale_grad(g_hf.data(), N * d, seed);
    orc_scale_grad(g_tok, V * d, seed);
  }
  std::vector<float> gx(N * d), g_v0;
  CHECK(orc_rms_norm_backward(x.data(), norm_f, g_hf.data(), N, d, eps, gx.data(), grads[1 + L * P_PER_BLOCK]));
  std::vector<float> g_m(N * F), g_s(N * F), g_u(N * F), g_a(N * F), g_h2(N * d), g_tmp(N * d), g_x1(N * d);
  std::vector<float> g_yg(N * qw), g_h(N * d), g_y(N * qw), g_yh(N * qw), g_qh(N * qw), g_kh(N * kvw), g_vh(N * kvw);
  std::vector<float> g_qr(N * qw), g_kr(N * kvw), g_v(N * kvw), g_qn(N * qw), g_kn(N * kvw), g_q(N * qw), g_k(N * kvw);
  std::vector<float> g_rawv(N * kvw), g_v0l(N * kvw);
  for (int64_t l = L - 1; l >= 0; --l) {
    LayerActs& a = acts[l];
    CHECK(orc_linear_backward(a.m.data(), P(l, P_FD), gx.data(), N, F, d, g_m.data(), G(l, P_FD)));
    CHECK(orc_mul_backward(a.s.data(), a.u.data(), g_m.data(), N * F, g_s.data(), g_u.data()));
    CHECK(orc_linear_backward(a.h2.data(), P(l, P_FU), g_u.data(), N, d, F, g_h2.data(), G(l, P_FU)));
    CHECK(orc_silu_backward(a.a.data(), g_s.data(), N * F, g_a.data()));
    CHECK(orc_linear_backward(a.h2.data(), P(l, P_FG), g_a.data(), N, d, F, g_tmp.data(), G(l, P_FG)));
    CHECK(orc_accumulate_grad(g_h2.data(), g_tmp.data(), N * d));
    CHECK(orc_rms_norm_backward(a.x1.data(), P(l, P_NORM2), g_h2.data(), N, d, eps, g_tmp.data(), G(l, P_NORM2)));
    g_x1 = gx;
    CHECK(orc_accumulate_grad(g_x1.data(), g_tmp.data(), N * d));
    CHECK(orc_linear_backward(a.yg.data(), P(l, P_O), g_x1.data(), N, qw, d, g_yg.data(), G(l, P_O)));
    CHECK(orc_gate_backward(a.h.data(), P(l, P_GW), P(l, P_GB), a.y.data(), g_yg.data(), N, d, H, dh,
                            g_h.data(), G(l, P_GW), G(l, P_GB), g_y.data()));
    CHECK(orc_permute_0213(g_y.data(), B, T, H, dh, g_yh.data()));
    CHECK(orc_causal_sdpa_backward(a.qh.data(), a.kh.data(), a.vh.data(), a.yh.data(), a.lse.data(), g_yh.data(),
                                   B, H, Hkv, T, dh, s.window, g_qh.data(), g_kh.data(), g_vh.data()));
    CHECK(orc_permute_0213(g_vh.data(), B, Hkv, T, dh, g_v.data()));
    CHECK(orc_permute_0213(g_kh.data(), B, Hkv, T, dh, g_kr.data()));
    CHECK(orc_permute_0213(g_qh.data(), B, H, T, dh, g_qr.data()));
    if (l > 0) {
      float gl = 0.0f;
      CHECK(orc_vres_backward(a.rawv.data(), acts[0].rawv.data(), g_v.data(), P(l, P_LAMBDA)[0], N * kvw,
                              g_rawv.data(), g_v0l.data(), &gl));
      G(l, P_LAMBDA)[0] = gl;
      if (g_v0.empty()) g_v0 = g_v0l; else CHECK(orc_accumulate_grad(g_v0.data(), g_v0l.data(), N * kvw));
    } else {
      if (g_v0.empty()) g_rawv = g_v;
      else { CHECK(orc_accumulate_grad(g_v0.data(), g_v.data(), N * kvw)); g_rawv = g_v0; }
      G(l, P_LAMBDA)[0] = 0.0f;  // layer 0's lambda never trains (names.rs:262-268)
    }
    CHECK(orc_rope(g_kr.data(), cos_t.data(), sin_t.data(), N * Hkv, dh, T, Hkv, 1, g_kn.data()));
    CHECK(orc_rope(g_qr.data(), cos_t.data(), sin_t.data(), N * H, dh, T, H, 1, g_qn.data()));
    CHECK(orc_rms_norm_backward(a.k.data(), P(l, P_KN), g_kn.data(), N * Hkv, dh, eps, g_k.data(), G(l, P_KN)));
    CHECK(orc_rms_norm_backward(a.q.data(), P(l, P_QN), g_qn.data(), N * H, dh, eps, g_q.data(), G(l, P_QN)));
    CHECK(orc_linear_backward(a.h.data(), P(l, P_V), g_rawv.data(), N, d, kvw, g_tmp.data(), G(l, P_V)));
    CHECK(orc_accumulate_grad(g_h.data(), g_tmp.data(), N * d));
    CHECK(orc_linear_backward(a.h.data(), P(l, P_K), g_k.data(), N, d, kvw, g_tmp.data(), G(l, P_K)));
    CHECK(orc_accumulate_grad(g_h.data(), g_tmp.data(), N * d));
    CHECK(orc_linear_backward(a.h.data(), P(l, P_Q), g_q.data(), N, d, qw, g_tmp.data(), G(l, P_Q)));
    CHECK(orc_accumulate_grad(g_h.data(), g_tmp.data(), N * d));
    CHECK(orc_rms_norm_backward(a.x.data(), P(l, P_NORM1), g_h.data(), N, d, eps, g_tmp.data(), G(l, P_NORM1)));
    gx = g_x1;
    CHECK(orc_accumulate_grad(gx.data(), g_tmp.data(), N * d));
  }
  std::vector<float> g_emb((size_t)V * d);
  CHECK(orc_embedding_backward(ids, gx.data(), N, V, d, g_emb.data()));
  CHECK(orc_accumulate_grad(g_tok, g_emb.data(), V * d));
  return ORC_OK;
}

}  // extern "C"
