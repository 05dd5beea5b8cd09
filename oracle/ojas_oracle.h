/* CPU oracle for the nanolab GPT training step: TEST INFRASTRUCTURE, not product.
 * Plain C ABI so tests and the CPU-baseline leg of bench.py can load it with ctypes.
 * Every function returns ORC_OK or an error class that mirrors ojas's
 * OjasError::{Shape, NonFinite, OutOfRange} (ojas-core/src/error.rs:18-118). */
#ifndef OJAS_ORACLE_H
#define OJAS_ORACLE_H
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

enum { ORC_OK = 0, ORC_SHAPE = 1, ORC_NONFINITE = 2, ORC_OUT_OF_RANGE = 3 };

/* generators (ojas-kernels/src/rng.rs, ojas-test-support/src/rng.rs, ojas-model/src/init.rs) */
uint64_t orc_splitmix_next(uint64_t* state);
void orc_splitmix_vec(uint64_t* state, int64_t n, float scale, float* out);
uint64_t orc_splitmix_below(uint64_t* state, uint64_t n);
uint64_t orc_fnv1a_bytes(const uint8_t* bytes, int64_t n);
uint64_t orc_fnv1a_f32(const float* v, int64_t n);
void orc_init_normal(const char* name, uint64_t seed, double stdev, int64_t n, float* out);
void orc_rope_tables(double base, int64_t start, int64_t len, int64_t dim, float* cos_t, float* sin_t);

/* scalar functions (ojas-core/src/exp_exact.rs, autocast.rs) */
float orc_exp_exact(float x);
float orc_log_sum_exp_exact(float max, float sum);
float orc_log1p_exact(float x);
float orc_sigmoid_exact(float x);
float orc_round_bf16(float x);
void orc_round_bf16_vec(const float* x, int64_t n, float* out);
float orc_sdpa_scale(int64_t head_dim);

/* ops, one per Backend method on the path (ojas-core/src/backend.rs) */
int orc_gemm(const float* a, int64_t ars, int64_t acs, const float* b, int64_t brs, int64_t bcs,
             float* c, int64_t m, int64_t k, int64_t n, int accumulate);
int orc_linear_forward(const float* x, const float* w, int64_t rows, int64_t kin, int64_t nout, float* y);
int orc_linear_backward(const float* x, const float* w, const float* gy, int64_t rows, int64_t kin,
                        int64_t nout, float* gx, float* gw);
int orc_rms_norm_forward(const float* x, const float* w, int64_t rows, int64_t dim, float eps, float* y);
int orc_rms_norm_backward(const float* x, const float* w, const float* gy, int64_t rows, int64_t dim,
                          float eps, float* gx, float* gw);
int orc_rope(const float* x, const float* cos_t, const float* sin_t, int64_t rows, int64_t dim,
             int64_t time, int64_t heads, int backward, float* y);
int orc_causal_sdpa_forward(const float* q, const float* k, const float* v, int64_t batch, int64_t heads,
                            int64_t kv_heads, int64_t time, int64_t dim, int64_t window, float* out,
                            float* lse);
int orc_causal_sdpa_backward(const float* q, const float* k, const float* v, const float* out,
                             const float* lse, const float* gy, int64_t batch, int64_t heads,
                             int64_t kv_heads, int64_t time, int64_t dim, int64_t window, float* gq,
                             float* gk, float* gv);
int orc_embedding_forward(const float* table, const uint32_t* ids, int64_t tokens, int64_t vocab,
                          int64_t dim, float* out);
int orc_embedding_backward(const uint32_t* ids, const float* grad, int64_t tokens, int64_t vocab,
                           int64_t dim, float* out);
int orc_silu_forward(const float* x, int64_t n, float* y);
int orc_silu_backward(const float* x, const float* gy, int64_t n, float* gx);
int orc_mul_forward(const float* a, const float* b, int64_t n, float* y);
int orc_mul_backward(const float* a, const float* b, const float* gy, int64_t n, float* ga, float* gb);
int orc_add(const float* a, const float* b, int64_t n, float* y);
int orc_accumulate_grad(float* acc, const float* g, int64_t n);
int orc_scale_grad(float* g, int64_t n, float s);
int orc_permute_0213(const float* x, int64_t d0, int64_t d1, int64_t d2, int64_t d3, float* y);
int orc_gate_forward(const float* input, const float* weight, const float* bias, const float* attn,
                     int64_t rows, int64_t din, int64_t heads, int64_t dh, float* y, float* scales);
int orc_gate_backward(const float* input, const float* weight, const float* bias, const float* attn,
                      const float* gy, int64_t rows, int64_t din, int64_t heads, int64_t dh, float* gx,
                      float* gw, float* gb, float* gattn);
int orc_vres_forward(const float* v, const float* v0, float lambda, int64_t n, float* y);
int orc_vres_backward(const float* v, const float* v0, const float* gy, float lambda, int64_t n,
                      float* gv, float* gv0, float* glambda);
int orc_cross_entropy_mean(const float* logits, const uint32_t* targets, int64_t rows, int64_t vocab,
                           int has_ignore, uint32_t ignore, float* loss, float* grad);
int orc_linear_cross_entropy_mean(const float* x, const float* w, const uint32_t* targets, int64_t rows,
                                  int64_t dim, int64_t vocab, int has_ignore, uint32_t ignore,
                                  float* loss, float* gx, float* gw);
int orc_argmax_rows(const float* x, int64_t rows, int64_t cols, uint32_t* out);
int orc_grad_norm(const float* const* parts, const int64_t* lens, int64_t count, float* norm);
int orc_clip_scale(float max_norm, float total_norm, float* scale);
int orc_clip_grad_norm(float* const* parts, const int64_t* lens, int64_t count, float max_norm, float* norm);
int orc_adamw_step(float* p, const float* g, float* m, float* v, int64_t n, uint64_t step_before,
                   double lr, double beta1, double beta2, double eps, double weight_decay);
int orc_newton_schulz5(float* update, int64_t rows, int64_t cols, int bf16);
int orc_muon_ns5_step(float* p, const float* g, float* mom, int64_t rows, int64_t cols, double lr,
                      double momentum, double weight_decay, int nesterov, int bf16);

/* the model: ojas-model/src/{spec,names,block}.rs and the reverse walk of ojas-autograd/src/tape.rs */
typedef struct {
  int64_t vocab, n_embd, n_layer, n_head, n_kv_head, head_dim, hidden, max_seq;
  int64_t window; /* -1: full causal */
  double rope_base;
  float rms_eps;
} orc_spec;

enum { ORC_INIT_ZEROS = 0, ORC_INIT_ONES = 1, ORC_INIT_NORMAL = 2 };
enum { ORC_GROUP_ADAMW = 0, ORC_GROUP_MUON = 1 };

/* Timed CPU baseline only: Numerics::Fast arithmetic (fused multiply-add products on 6 x 16 register tiles, f32 AdamW) instead of the
 * Exact contract every parity check uses, and the number of threads the parallel regions run on. */
void orc_set_fast(int on);
int orc_fast(void);
int orc_set_threads(int n);
int orc_max_threads(void);

int64_t orc_param_count(const orc_spec* spec);
int orc_param_info(const orc_spec* spec, int64_t index, char* name, int64_t name_cap, int64_t* rank,
                   int64_t* shape2, int* init_kind, int* group, int* trains);
/* loss (and, when grads != NULL, every parameter gradient for a backward seeded with `seed`).
 * params/grads: one pointer per parameter in param_table order. logits (optional): [B*T, vocab]. */
int orc_forward_loss(const orc_spec* spec, const float* const* params, const uint32_t* ids,
                     const uint32_t* targets, int64_t batch, int64_t seq, int has_ignore, uint32_t ignore,
                     float seed, float* loss, float* const* grads, float* logits);

#ifdef __cplusplus
}
#endif
#endif
