/*
 * oracle.h -- CPU restatement of sptorch's transformer-forward arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  Nothing in the shipped library links, loads or
 * calls this code; it exists so that tests, the smoke check and the bench's
 * CPU-baseline leg can compare the CUDA path with the reference's math.
 *
 * Every function restates, in f32 and in the reference's own evaluation
 * order, one function of the reference (file:line given at each).  Pinning:
 * the known-answer vectors of the reference's unit tests are replayed in
 * tests/test_oracle_kat.py, and the eleven ops that the reference's own C
 * file crates/hal-ffi/mock_npu/mock_npu.c implements are cross-checked
 * against that file compiled in place (oracle/_ref/libmock_npu.so).
 *
 * Parity UNPINNED for one thing: the summation order inside
 * matrixmultiply::sgemm (crate requirement "0.3", no lock file, not vendored;
 * call site crates/core-ops/src/lib.rs:240-263).  orc_matmul uses the plain
 * p = 0..k-1 order that the reference's CpuBackend and mock_npu.c use
 * (crates/hal/src/lib.rs:547-557); orc_matmul_f64 bounds the oracle's own
 * rounding error.  The reference's exact KATs at that boundary are
 * small-integer valued, hence order independent.
 */
#ifndef SPTORCH_ORACLE_H
#define SPTORCH_ORACLE_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif

/* ---- core-ops ---- */
void orc_add(const float* a, const float* b, float* out, size_t n);
void orc_mul(const float* a, const float* b, float* out, size_t n);
void orc_neg(const float* a, float* out, size_t n);
void orc_exp(const float* a, float* out, size_t n);
void orc_log(const float* a, float* out, size_t n);
void orc_relu(const float* a, float* out, size_t n);
void orc_gelu(const float* a, float* out, size_t n);
void orc_scale(const float* a, float s, float* out, size_t n);
float orc_sum(const float* a, size_t n);
void orc_broadcast_add(const float* a, const float* b, float* out, size_t a_len, size_t b_len);
void orc_masked_fill(const float* a, const uint8_t* mask, float fill, float* out, size_t n);
int  orc_embedding(const float* w, const int64_t* idx, float* out, size_t n_idx, size_t vocab, size_t dim);
void orc_transpose(const float* a, float* out, size_t rows, size_t cols);
void orc_matmul(const float* a, const float* b, float* out, size_t m, size_t k, size_t n);
void orc_matmul_f64(const float* a, const float* b, float* out, size_t m, size_t k, size_t n);
void orc_batch_matmul(const float* a, const float* b, float* out, size_t batch, size_t m, size_t k, size_t n);
void orc_softmax(const float* a, float* out, size_t rows, size_t cols);
void orc_softmax_hal(const float* a, float* out, size_t rows, size_t cols);
void orc_masked_softmax(const float* a, const uint8_t* keep, float* out, size_t rows, size_t cols, int rank1);
void orc_rms_norm(const float* x, const float* w, float* out, size_t rows, size_t dim, float eps);
void orc_swiglu(const float* x, const float* gate, float* out, size_t n);
float orc_cross_entropy(const float* logits, const int64_t* targets, size_t rows, size_t classes, int has_ignore,
                        int64_t ignore_index, int* bad);
void orc_sgd_update(float* p, const float* g, float lr, size_t n);
void orc_adam_update(float* p, const float* g, float* m, float* v, size_t n, float lr, float beta1,
                     float beta2, float eps, float weight_decay, float bc1, float bc2);

/* ---- nn ---- */
void orc_layernorm(const float* x, const float* gamma, const float* beta, float* out,
                   size_t rows, size_t dim, float eps);
/* y[M,N] = x[M,K] * W[N,K]^T (+ bias[N]); `fast`: 0 = strict p-order via a
 * materialised transpose as the reference does, 1 = blocked row-dot kernel
 * (8 partial sums), 2 = f64 accumulation. */
void orc_linear(const float* x, const float* w, const float* bias, float* y,
                size_t M, size_t K, size_t N, int fast);
void orc_reshape_to_heads(const float* x, float* out, size_t T, size_t H, size_t hd);
void orc_reshape_from_heads(const float* x, float* out, size_t T, size_t H, size_t hd);
void orc_batch_transpose(const float* x, float* out, size_t H, size_t T, size_t hd);
void orc_mha_causal(const float* x, const float* wq, const float* wk, const float* wv, const float* wo,
                    float* out, size_t T, size_t d, size_t H, int fast);

int  orc_rope(const float* data, float* out, size_t n_head, size_t seq_len, size_t head_dim, float rope_base,
              size_t position_offset, int inverse);
void orc_mha_causal_rope(const float* x, const float* wq, const float* wk, const float* wv, const float* wo,
                         float* out, size_t T, size_t d, size_t H, int fast, float rope_base, size_t position_offset);

void orc_attention_last_token(const float* q, const float* k, const float* v, float* out, size_t H, size_t n, size_t hd);

typedef struct {
    int vocab, d_model, n_layer, n_head, d_ff, seq_len;
    float eps;
} orc_gpt_config;

/* Flat parameter block in GPT::named_parameters order (crates/nn/src/lib.rs:1382-1392):
 * token_emb.weight[V,d], pos_emb.weight[S,d], then per block: ln1.gamma[d], ln1.beta[d],
 * attn.wq/wk/wv/wo.weight[d,d], ln2.gamma[d], ln2.beta[d], ffn_up.weight[F,d], ffn_up.bias[F],
 * ffn_down.weight[d,F], ffn_down.bias[d]; then ln_f.gamma[d], ln_f.beta[d], lm_head.weight[V,d]. */
size_t orc_gpt_param_count(const orc_gpt_config* c);

/* One sequence: ids[T] -> logits[T,V].  taps (optional, may be NULL): receives the residual
 * stream after the embedding and after every block, then ln_f output: (n_layer+2) * T * d floats.
 * Returns 0, or -1 if an id is out of range (the reference panics there). */
int orc_gpt_forward_ids(const orc_gpt_config* c, const float* params, const int64_t* ids, size_t T,
                        float* logits, float* taps, int fast);

/* Batch = independent calls (the reference has no batch dimension); OpenMP over sequences. */
int orc_gpt_forward_batch(const orc_gpt_config* c, const float* params, const int64_t* ids, size_t B,
                          size_t T, float* logits, float* taps, int fast, int threads);
/* QwenLikeGPT (crates/nn/src/lib.rs:1439-1467): parameter block in named_parameters order, see oracle.c */
size_t orc_qwen_param_count(const orc_gpt_config* c);
int orc_qwen_forward_ids(const orc_gpt_config* c, float rope_base, const float* params, const int64_t* ids, size_t T,
                         float* logits, float* taps, int fast);
int orc_qwen_forward_batch(const orc_gpt_config* c, float rope_base, const float* params, const int64_t* ids, size_t B,
                           size_t T, float* logits, float* taps, int fast, int threads);
/* ---- sampling (crates/nn/src/lib.rs:2381-2418) ---- */
void orc_filter_step_logits(const float* logits, size_t n, const int64_t* allowed, size_t n_allowed, float* out);
long orc_sampling_candidates(const float* logits, size_t n_logits, size_t vocab_size, float temperature, size_t top_k, float top_p,
                             float repetition_penalty, const int64_t* history, size_t n_history,
                             int64_t* out_ids, float* out_logits, float* out_probs);
int orc_max_threads(void);

#ifdef __cplusplus
}
#endif
#endif
