/*
 * oracle.c -- CPU restatement of sptorch's transformer-forward arithmetic.
 * TEST INFRASTRUCTURE ONLY (see oracle.h).  All arithmetic is IEEE f32 in the
 * reference's evaluation order unless a function says otherwise.  Compile
 * WITHOUT -ffast-math; -ffp-contract=off keeps a*b+c as two roundings, which
 * is what the reference's scalar Rust does.
 */
#include "oracle.h"
#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
static int omp_in_parallel_(void) { return omp_in_parallel(); }
#else
static int omp_in_parallel_(void) { return 1; }
#endif

/* ---------- elementwise (crates/core-ops/src/lib.rs:299-332, 1331-1358, 1376-1399;
 *            crates/hal/src/lib.rs:497-545 state the same kernels) ---------- */
void orc_add(const float* a, const float* b, float* out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = a[i] + b[i]; }
void orc_mul(const float* a, const float* b, float* out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = a[i] * b[i]; }
void orc_neg(const float* a, float* out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = -a[i]; }
void orc_exp(const float* a, float* out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = expf(a[i]); }
void orc_log(const float* a, float* out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = logf(a[i]); }
void orc_relu(const float* a, float* out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = a[i] > 0.0f ? a[i] : 0.0f; }
void orc_scale(const float* a, float s, float* out, size_t n) { for (size_t i = 0; i < n; i++) out[i] = a[i] * s; }

/* gelu: crates/core-ops/src/lib.rs:1338-1342.  k = sqrt(2/pi) evaluated in f32;
 * x.powi(3) lowers to (x*x)*x. */
void orc_gelu(const float* a, float* out, size_t n) {
    const float k = sqrtf(2.0f / 3.14159265358979323846f);
    for (size_t i = 0; i < n; i++) {
        float x = a[i];
        float x3 = (x * x) * x;
        out[i] = 0.5f * x * (1.0f + tanhf(k * (x + 0.044715f * x3)));
    }
}

/* sum: crates/hal/src/lib.rs:578-580 (sequential f32). */
float orc_sum(const float* a, size_t n) { float s = 0.0f; for (size_t i = 0; i < n; i++) s += a[i]; return s; }

/* broadcast_add: crates/hal/src/lib.rs:604-608; equal to the numpy-style broadcast of
 * crates/core-ops/src/lib.rs:107-147 for [M,N] + [N]. */
void orc_broadcast_add(const float* a, const float* b, float* out, size_t a_len, size_t b_len) {
    for (size_t i = 0; i < a_len; i++) out[i] = a[i] + b[i % b_len];
}

/* masked_fill: crates/core-ops/src/lib.rs:1682-1703, crates/hal/src/lib.rs:598-602 (true = overwrite). */
void orc_masked_fill(const float* a, const uint8_t* mask, float fill, float* out, size_t n) {
    for (size_t i = 0; i < n; i++) out[i] = mask[i] ? fill : a[i];
}

/* embedding_lookup: crates/core-ops/src/lib.rs:1220-1255 (row copy; index >= vocab panics there). */
int orc_embedding(const float* w, const int64_t* idx, float* out, size_t n_idx, size_t vocab, size_t dim) {
    for (size_t i = 0; i < n_idx; i++) {
        if (idx[i] < 0 || (size_t)idx[i] >= vocab) return -1;
        memcpy(out + i * dim, w + (size_t)idx[i] * dim, dim * sizeof(float));
    }
    return 0;
}

/* transpose: crates/core-ops/src/lib.rs:825-850. */
void orc_transpose(const float* a, float* out, size_t rows, size_t cols) {
    for (size_t r = 0; r < rows; r++)
        for (size_t c = 0; c < cols; c++) out[c * rows + r] = a[r * cols + c];
}

/* matmul: row-major A[m,k]*B[k,n], scalar accumulator over p = 0..k-1
 * (crates/hal/src/lib.rs:547-557; call site of the un-vendored sgemm crates/core-ops/src/lib.rs:240-263). */
void orc_matmul(const float* a, const float* b, float* out, size_t m, size_t k, size_t n) {
    for (size_t i = 0; i < m; i++)
        for (size_t j = 0; j < n; j++) {
            float s = 0.0f;
            for (size_t p = 0; p < k; p++) s += a[i * k + p] * b[p * n + j];
            out[i * n + j] = s;
        }
}

void orc_matmul_f64(const float* a, const float* b, float* out, size_t m, size_t k, size_t n) {
    for (size_t i = 0; i < m; i++)
        for (size_t j = 0; j < n; j++) {
            double s = 0.0;
            for (size_t p = 0; p < k; p++) s += (double)a[i * k + p] * (double)b[p * n + j];
            out[i * n + j] = (float)s;
        }
}

/* batch_matmul: crates/core-ops/src/lib.rs:1763-1799 (loop over batch, plain matmul each). */
void orc_batch_matmul(const float* a, const float* b, float* out, size_t batch, size_t m, size_t k, size_t n) {
    for (size_t z = 0; z < batch; z++) orc_matmul(a + z * m * k, b + z * k * n, out + z * m * n, m, k, n);
}

/* softmax, 2-D path: crates/core-ops/src/lib.rs:903-920.  max folded from -inf; exp evaluated
 * twice; a zero sum gives the uniform row. */
void orc_softmax(const float* a, float* out, size_t rows, size_t cols) {
    for (size_t r = 0; r < rows; r++) {
        const float* x = a + r * cols;
        float* y = out + r * cols;
        float mx = -INFINITY;
        for (size_t c = 0; c < cols; c++) mx = fmaxf(mx, x[c]);
        float s = 0.0f;
        for (size_t c = 0; c < cols; c++) s += expf(x[c] - mx);
        if (s == 0.0f) {
            float u = 1.0f / (float)cols;
            for (size_t c = 0; c < cols; c++) y[c] = u;
        } else {
            for (size_t c = 0; c < cols; c++) y[c] = expf(x[c] - mx) / s;
        }
    }
}

/* softmax as the HAL reference kernel states it: crates/hal/src/lib.rs:582-596
 * (exp stored once, then divided; no zero-sum branch). */
void orc_softmax_hal(const float* a, float* out, size_t rows, size_t cols) {
    for (size_t r = 0; r < rows; r++) {
        const float* x = a + r * cols;
        float* y = out + r * cols;
        float mx = -INFINITY;
        for (size_t c = 0; c < cols; c++) mx = fmaxf(mx, x[c]);
        float s = 0.0f;
        for (size_t c = 0; c < cols; c++) { float e = expf(x[c] - mx); y[c] = e; s += e; }
        for (size_t c = 0; c < cols; c++) y[c] /= s;
    }
}

/* masked_softmax: crates/core-ops/src/lib.rs:1601-1645.  keep != 0 means the entry takes part
 * (the opposite polarity of masked_fill).  rank1 != 0 applies the extra rule for 1-D inputs. */
void orc_masked_softmax(const float* a, const uint8_t* keep, float* out, size_t rows, size_t cols, int rank1) {
    size_t n = rows * cols;
    for (size_t i = 0; i < n; i++) out[i] = 0.0f;
    for (size_t r = 0; r < rows; r++) {
        size_t off = r * cols;
        float mx = -INFINITY;
        for (size_t c = 0; c < cols; c++) if (keep[off + c]) mx = fmaxf(mx, a[off + c]);
        if (mx == -INFINITY) continue;
        float s = 0.0f;
        for (size_t c = 0; c < cols; c++) if (keep[off + c]) { float e = expf(a[off + c] - mx); out[off + c] = e; s += e; }
        if (s > 0.0f) for (size_t c = 0; c < cols; c++) if (keep[off + c]) out[off + c] /= s;
    }
    if (rank1) {
        int all_zero = 1; size_t cnt = 0;
        for (size_t i = 0; i < n; i++) { if (out[i] != 0.0f) all_zero = 0; if (keep[i]) cnt++; }
        if (all_zero) for (size_t i = 0; i < n; i++) if (keep[i]) out[i] = 1.0f / (float)cnt;
    }
}

/* rms_norm: crates/core-ops/src/lib.rs:1453-1475 (sequential sum of squares, inv = 1/sqrt(mean_sq+eps), x*inv*w). */
void orc_rms_norm(const float* x, const float* w, float* out, size_t rows, size_t dim, float eps) {
    for (size_t r = 0; r < rows; r++) {
        const float* xr = x + r * dim; float* yr = out + r * dim;
        float ms = 0.0f;
        for (size_t i = 0; i < dim; i++) ms += xr[i] * xr[i];
        ms /= (float)dim;
        float inv = 1.0f / sqrtf(ms + eps);
        for (size_t i = 0; i < dim; i++) yr[i] = xr[i] * inv * w[i];
    }
}

/* swiglu: crates/core-ops/src/lib.rs:1529-1540 (s = 1/(1+exp(-g)); x*g*s). */
void orc_swiglu(const float* x, const float* gate, float* out, size_t n) {
    for (size_t i = 0; i < n; i++) { float s = 1.0f / (1.0f + expf(-gate[i])); out[i] = x[i] * gate[i] * s; }
}

/* cross_entropy_loss(_ignore_index), batched path: crates/core-ops/src/lib.rs:1131-1168.  Mean over the rows whose
 * target is not the ignore index (0 if none); returns -1 through *bad for an out-of-range target (the reference panics). */
float orc_cross_entropy(const float* logits, const int64_t* targets, size_t rows, size_t classes, int has_ignore,
                        int64_t ignore_index, int* bad) {
    float total = 0.0f; size_t active = 0;
    if (bad) *bad = 0;
    for (size_t r = 0; r < rows; r++) {
        const float* x = logits + r * classes;
        if (has_ignore && targets[r] == ignore_index) continue;
        if (targets[r] < 0 || (size_t)targets[r] >= classes) { if (bad) *bad = 1; return 0.0f; }
        float mx = -INFINITY;
        for (size_t c = 0; c < classes; c++) mx = fmaxf(mx, x[c]);
        float s = 0.0f;
        for (size_t c = 0; c < classes; c++) s += expf(x[c] - mx);
        float ls = logf(s);
        total += -(x[targets[r]] - mx - ls);
        active++;
    }
    return active == 0 ? 0.0f : total / (float)active;
}

/* optimizer kernels of the KernelProvider trait: crates/hal/src/lib.rs:616-646. */
void orc_sgd_update(float* p, const float* g, float lr, size_t n) { for (size_t i = 0; i < n; i++) p[i] -= lr * g[i]; }
void orc_adam_update(float* p, const float* g, float* m, float* v, size_t n, float lr, float beta1,
                     float beta2, float eps, float weight_decay, float bc1, float bc2) {
    for (size_t j = 0; j < n; j++) {
        if (weight_decay != 0.0f) p[j] *= 1.0f - lr * weight_decay;
        m[j] = beta1 * m[j] + (1.0f - beta1) * g[j];
        v[j] = beta2 * v[j] + (1.0f - beta2) * g[j] * g[j];
        float mh = m[j] / bc1, vh = v[j] / bc2;
        p[j] -= lr * mh / (sqrtf(vh) + eps);
    }
}

/* LayerNorm::forward: crates/nn/src/lib.rs:397-418 (two sequential passes, biased variance,
 * inv = 1/sqrt(var+eps), y = gamma*((x-mean)*inv) + beta). */
void orc_layernorm(const float* x, const float* gamma, const float* beta, float* out,
                   size_t rows, size_t dim, float eps) {
    for (size_t r = 0; r < rows; r++) {
        const float* xr = x + r * dim;
        float* yr = out + r * dim;
        float s = 0.0f;
        for (size_t i = 0; i < dim; i++) s += xr[i];
        float mean = s / (float)dim;
        float v = 0.0f;
        for (size_t i = 0; i < dim; i++) { float d = xr[i] - mean; v += d * d; }
        float var = v / (float)dim;
        float inv = 1.0f / sqrtf(var + eps);
        for (size_t i = 0; i < dim; i++) { float nrm = (xr[i] - mean) * inv; yr[i] = gamma[i] * nrm + beta[i]; }
    }
}

/* Blocked row-dot kernel for y = x W^T: both operands are contiguous along K, so the dot is
 * split into 8 interleaved partial sums (lane j takes p = j mod 8), reduced pairwise at the end.
 * The order is fixed and documented; it is NOT the reference's (which is unpinned anyway). */
static float dot8(const float* a, const float* b, size_t k) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    size_t p = 0;
    for (; p + 8 <= k; p += 8)
        for (int j = 0; j < 8; j++) acc[j] += a[p + j] * b[p + j];
    float t = 0.0f;
    for (; p < k; p++) t += a[p] * b[p];
    return (((acc[0] + acc[4]) + (acc[2] + acc[6])) + ((acc[1] + acc[5]) + (acc[3] + acc[7]))) + t;
}

/* Linear::forward: crates/nn/src/lib.rs:121-133 = transpose (ops:825-836) + matmul (ops:643-676)
 * + broadcast bias add (ops:1804-1806). */
void orc_linear(const float* x, const float* w, const float* bias, float* y,
                size_t M, size_t K, size_t N, int fast) {
    if (fast == 0) {
        float* wt = (float*)malloc(K * N * sizeof(float));
        orc_transpose(w, wt, N, K);
        orc_matmul(x, wt, y, M, K, N);
        free(wt);
    } else if (fast == 1) {
        /* rows are independent: split them over threads unless the caller already runs one sequence per thread */
        const long IB = 32, JB = 256, JI = 64;
        const long nib = ((long)M + IB - 1) / IB, njb = ((long)N + JB - 1) / JB;
#pragma omp parallel for collapse(2) schedule(dynamic, 1) if (!omp_in_parallel_())
        for (long ib = 0; ib < nib; ib++) {
            for (long jb = 0; jb < njb; jb++) {
                size_t i0 = (size_t)ib * IB, i1 = i0 + IB < M ? i0 + IB : M;
                size_t jb0 = (size_t)jb * JB, jb1 = jb0 + JB < N ? jb0 + JB : N;
                for (size_t j0 = jb0; j0 < jb1; j0 += JI) {
                    size_t j1 = j0 + JI < jb1 ? j0 + JI : jb1;
                    for (size_t i = i0; i < i1; i++)
                        for (size_t j = j0; j < j1; j++) y[i * N + j] = dot8(x + i * K, w + j * K, K);
                }
            }
        }
    } else {
        for (size_t i = 0; i < M; i++)
            for (size_t j = 0; j < N; j++) {
                double s = 0.0;
                for (size_t p = 0; p < K; p++) s += (double)x[i * K + p] * (double)w[j * K + p];
                y[i * N + j] = (float)s;
            }
    }
    if (bias) for (size_t i = 0; i < M; i++) for (size_t j = 0; j < N; j++) y[i * N + j] = y[i * N + j] + bias[j];
}

/* head permutations: crates/nn/src/lib.rs:763-793, 822-850, 879-903. */
void orc_reshape_to_heads(const float* x, float* out, size_t T, size_t H, size_t hd) {
    for (size_t h = 0; h < H; h++) for (size_t s = 0; s < T; s++) for (size_t e = 0; e < hd; e++)
        out[(h * T + s) * hd + e] = x[s * (H * hd) + h * hd + e];
}
void orc_reshape_from_heads(const float* x, float* out, size_t T, size_t H, size_t hd) {
    for (size_t h = 0; h < H; h++) for (size_t s = 0; s < T; s++) for (size_t e = 0; e < hd; e++)
        out[s * (H * hd) + h * hd + e] = x[(h * T + s) * hd + e];
}
void orc_batch_transpose(const float* x, float* out, size_t H, size_t T, size_t hd) {
    for (size_t h = 0; h < H; h++) for (size_t s = 0; s < T; s++) for (size_t e = 0; e < hd; e++)
        out[(h * hd + e) * T + s] = x[(h * T + s) * hd + e];
}

/* per-head matmul used inside attention.  fast==0: the reference's [m,k]x[k,n] p-order;
 * fast==1: same products, B pre-transposed so the 8-lane dot can run; fast==2: f64. */
static void head_matmul_nt(const float* a, const float* bt, float* out, size_t m, size_t k, size_t n, int fast) {
    /* a[m,k], bt[n,k] -> out[m,n] */
    for (size_t i = 0; i < m; i++)
        for (size_t j = 0; j < n; j++) {
            if (fast == 1) out[i * n + j] = dot8(a + i * k, bt + j * k, k);
            else if (fast == 2) { double s = 0; for (size_t p = 0; p < k; p++) s += (double)a[i * k + p] * (double)bt[j * k + p]; out[i * n + j] = (float)s; }
            else { float s = 0.0f; for (size_t p = 0; p < k; p++) s += a[i * k + p] * bt[j * k + p]; out[i * n + j] = s; }
        }
}

/* apply_rope_raw: crates/nn/src/lib.rs:930-961.  data, out: [n_head, seq_len, head_dim]; pairs (2p, 2p+1) of every head
 * are rotated by theta = absolute_pos / base^(2p/head_dim), all in f32 (powf, sinf, cosf as f32::powf / sin_cos). */
int orc_rope(const float* data, float* out, size_t n_head, size_t seq_len, size_t head_dim, float rope_base,
             size_t position_offset, int inverse) {
    if (head_dim % 2) return -1;                       /* the reference asserts an even head dimension */
    size_t half = head_dim / 2;
    for (size_t h = 0; h < n_head; h++)
        for (size_t pos = 0; pos < seq_len; pos++) {
            size_t off = h * seq_len * head_dim + pos * head_dim;
            size_t absolute_pos = position_offset + pos;
            for (size_t pair = 0; pair < half; pair++) {
                float theta = (float)absolute_pos / powf(rope_base, (float)(2 * pair) / (float)head_dim);
                float sn = sinf(theta), cs = cosf(theta);
                if (inverse) sn = -sn;
                float even = data[off + 2 * pair], odd = data[off + 2 * pair + 1];
                out[off + 2 * pair] = even * cs - odd * sn;
                out[off + 2 * pair + 1] = even * sn + odd * cs;
            }
        }
    return 0;
}

static void mha_causal_impl(const float* x, const float* wq, const float* wk, const float* wv, const float* wo,
                            float* out, size_t T, size_t d, size_t H, int fast, int use_rope, float rope_base, size_t position_offset);

/* MultiHeadAttention::forward_causal_impl: crates/nn/src/lib.rs:590-642. */
void orc_mha_causal(const float* x, const float* wq, const float* wk, const float* wv, const float* wo,
                    float* out, size_t T, size_t d, size_t H, int fast) {
    mha_causal_impl(x, wq, wk, wv, wo, out, T, d, H, fast, 0, 0.0f, 0);
}

/* MultiHeadAttention::forward_causal_rope_with_offset: crates/nn/src/lib.rs:655-661 (Q and K rotated after the head split, :606-609). */
void orc_mha_causal_rope(const float* x, const float* wq, const float* wk, const float* wv, const float* wo,
                         float* out, size_t T, size_t d, size_t H, int fast, float rope_base, size_t position_offset) {
    mha_causal_impl(x, wq, wk, wv, wo, out, T, d, H, fast, 1, rope_base, position_offset);
}

static void mha_causal_impl(const float* x, const float* wq, const float* wk, const float* wv, const float* wo,
                            float* out, size_t T, size_t d, size_t H, int fast, int use_rope, float rope_base, size_t position_offset) {
    size_t hd = d / H;
    float* q = (float*)malloc(T * d * sizeof(float));
    float* k = (float*)malloc(T * d * sizeof(float));
    float* v = (float*)malloc(T * d * sizeof(float));
    float* q3 = (float*)malloc(T * d * sizeof(float));
    float* k3 = (float*)malloc(T * d * sizeof(float));
    float* v3 = (float*)malloc(T * d * sizeof(float));
    float* vt = (float*)malloc(T * d * sizeof(float));
    float* sc = (float*)malloc(H * T * T * sizeof(float));
    float* pr = (float*)malloc(H * T * T * sizeof(float));
    float* o3 = (float*)malloc(T * d * sizeof(float));
    float* o2 = (float*)malloc(T * d * sizeof(float));
    orc_linear(x, wq, NULL, q, T, d, d, fast);
    orc_linear(x, wk, NULL, k, T, d, d, fast);
    orc_linear(x, wv, NULL, v, T, d, d, fast);
    orc_reshape_to_heads(q, q3, T, H, hd);
    orc_reshape_to_heads(k, k3, T, H, hd);
    orc_reshape_to_heads(v, v3, T, H, hd);
    if (use_rope) {
        /* q and k are free again after the head split: rotate into them and swap the roles */
        orc_rope(q3, q, H, T, hd, rope_base, position_offset, 0);
        orc_rope(k3, k, H, T, hd, rope_base, position_offset, 0);
        float* t_ = q3; q3 = q; q = t_;
        t_ = k3; k3 = k; k = t_;
    }
    /* scores = Q K^T: the reference materialises K^T [H,hd,T] and multiplies [T,hd]x[hd,T];
     * the products and their p-order are the same as dotting rows of Q with rows of K. */
#pragma omp parallel for schedule(static) if (!omp_in_parallel_())
    for (long h = 0; h < (long)H; h++) head_matmul_nt(q3 + h * T * hd, k3 + h * T * hd, sc + h * T * T, T, hd, T, fast);
    float scale = 1.0f / sqrtf((float)hd);
    for (size_t i = 0; i < H * T * T; i++) sc[i] = sc[i] * scale;
    for (size_t h = 0; h < H; h++) for (size_t i = 0; i < T; i++) for (size_t j = i + 1; j < T; j++)
        sc[(h * T + i) * T + j] = -INFINITY;
#pragma omp parallel for schedule(static) if (!omp_in_parallel_())
    for (long h = 0; h < (long)H; h++) orc_softmax(sc + h * T * T, pr + h * T * T, T, T);
    /* out = P V: [T,T]x[T,hd]; V^T lets the same row-dot helper run, order of p unchanged for fast==0 */
    orc_batch_transpose(v3, vt, H, T, hd);
#pragma omp parallel for schedule(static) if (!omp_in_parallel_())
    for (long h = 0; h < (long)H; h++) head_matmul_nt(pr + h * T * T, vt + h * hd * T, o3 + h * T * hd, T, T, hd, fast);
    orc_reshape_from_heads(o3, o2, T, H, hd);
    orc_linear(o2, wo, NULL, out, T, d, d, fast);
    free(q); free(k); free(v); free(q3); free(k3); free(v3); free(vt); free(sc); free(pr); free(o3); free(o2);
}

/* causal_attention_last_token, the cache part: crates/nn/src/lib.rs:727-755.  q[H*hd]; k, v cached as [H, n, hd];
 * out[H*hd].  Sequential dots, scale, max, exp, denominator, then out += (exp/denom) * v over positions. */
void orc_attention_last_token(const float* q, const float* k, const float* v, float* out, size_t H, size_t n, size_t hd) {
    float scale = 1.0f / sqrtf((float)hd);
    float* sc = (float*)malloc(n * sizeof(float));
    for (size_t h = 0; h < H; h++) {
        for (size_t p = 0; p < n; p++) {
            float dot = 0.0f;
            for (size_t d = 0; d < hd; d++) dot += q[h * hd + d] * k[(h * n + p) * hd + d];
            sc[p] = dot * scale;
        }
        float mx = -INFINITY;
        for (size_t p = 0; p < n; p++) mx = fmaxf(mx, sc[p]);
        float den = 0.0f;
        for (size_t p = 0; p < n; p++) { sc[p] = expf(sc[p] - mx); den += sc[p]; }
        for (size_t d = 0; d < hd; d++) out[h * hd + d] = 0.0f;
        for (size_t p = 0; p < n; p++) {
            float w = sc[p] / den;
            for (size_t d = 0; d < hd; d++) out[h * hd + d] += w * v[(h * n + p) * hd + d];
        }
    }
    free(sc);
}

size_t orc_gpt_param_count(const orc_gpt_config* c) {
    size_t V = c->vocab, d = c->d_model, F = c->d_ff, S = c->seq_len, L = c->n_layer;
    size_t per_block = 2 * d + 4 * d * d + 2 * d + F * d + F + d * F + d;
    return V * d + S * d + L * per_block + 2 * d + V * d;
}

/* GPT::forward_ids: crates/nn/src/lib.rs:1349-1364; TransformerBlock::forward_seq with dropout
 * in eval mode: crates/nn/src/lib.rs:1189-1214. */
int orc_gpt_forward_ids(const orc_gpt_config* c, const float* params, const int64_t* ids, size_t T,
                        float* logits, float* taps, int fast) {
    size_t V = c->vocab, d = c->d_model, F = c->d_ff, S = c->seq_len, L = c->n_layer, H = c->n_head;
    if (T > S) return -2;
    const float* tok = params;
    const float* pos = tok + V * d;
    const float* p = pos + S * d;
    float* x = (float*)malloc(T * d * sizeof(float));
    float* t0 = (float*)malloc(T * d * sizeof(float));
    float* t1 = (float*)malloc(T * d * sizeof(float));
    float* hbuf = (float*)malloc(T * F * sizeof(float));
    float* gbuf = (float*)malloc(T * F * sizeof(float));
    int64_t* posid = (int64_t*)malloc(T * sizeof(int64_t));
    int rc = 0;
    for (size_t i = 0; i < T; i++) posid[i] = (int64_t)i;
    if (orc_embedding(tok, ids, t0, T, V, d) != 0) { rc = -1; goto done; }
    orc_embedding(pos, posid, t1, T, S, d);
    orc_add(t0, t1, x, T * d);
    if (taps) memcpy(taps, x, T * d * sizeof(float));
    for (size_t l = 0; l < L; l++) {
        const float* ln1g = p;            const float* ln1b = ln1g + d;
        const float* wq = ln1b + d;       const float* wk = wq + d * d;
        const float* wv = wk + d * d;     const float* wo = wv + d * d;
        const float* ln2g = wo + d * d;   const float* ln2b = ln2g + d;
        const float* w1 = ln2b + d;       const float* b1 = w1 + F * d;
        const float* w2 = b1 + F;         const float* b2 = w2 + d * F;
        p = b2 + d;
        orc_layernorm(x, ln1g, ln1b, t0, T, d, c->eps);
        orc_mha_causal(t0, wq, wk, wv, wo, t1, T, d, H, fast);
        orc_add(x, t1, x, T * d);
        orc_layernorm(x, ln2g, ln2b, t0, T, d, c->eps);
        orc_linear(t0, w1, b1, hbuf, T, d, F, fast);
        orc_gelu(hbuf, gbuf, T * F);
        orc_linear(gbuf, w2, b2, t1, T, F, d, fast);
        orc_add(x, t1, x, T * d);
        if (taps) memcpy(taps + (l + 1) * T * d, x, T * d * sizeof(float));
    }
    {
        const float* lnfg = p; const float* lnfb = lnfg + d; const float* head = lnfb + d;
        orc_layernorm(x, lnfg, lnfb, t0, T, d, c->eps);
        if (taps) memcpy(taps + (L + 1) * T * d, t0, T * d * sizeof(float));
        orc_linear(t0, head, NULL, logits, T, d, V, fast);
    }
done:
    free(x); free(t0); free(t1); free(hbuf); free(gbuf); free(posid);
    return rc;
}

/* Flat parameter block of QwenLikeGPT in named_parameters order (crates/nn/src/lib.rs:1483-1492, block :1157-1166):
 * token_emb.weight[V,d]; per block norm1.weight[d], attn.wq/wk/wv/wo.weight[d,d], norm2.weight[d], ffn_up.weight[F,d], ffn_up.bias[F],
 * ffn_gate.weight[F,d], ffn_gate.bias[F], ffn_down.weight[d,F], ffn_down.bias[d]; then norm_f.weight[d], lm_head.weight[V,d]. */
size_t orc_qwen_param_count(const orc_gpt_config* c) {
    size_t V = c->vocab, d = c->d_model, F = c->d_ff, L = c->n_layer;
    return V * d + L * (2 * d + 4 * d * d + 2 * (F * d + F) + d * F + d) + d + V * d;
}

/* QwenLikeGPT::forward_ids (crates/nn/src/lib.rs:1454-1467) with QwenLikeBlock::forward_seq_inference (:1106-1117): dropout is
 * the identity in evaluation.  c->eps is the RMSNorm epsilon (1e-6, :468); rope_base 10000 (:1083).  taps as in orc_gpt_forward_ids. */
int orc_qwen_forward_ids(const orc_gpt_config* c, float rope_base, const float* params, const int64_t* ids, size_t T,
                         float* logits, float* taps, int fast) {
    size_t V = c->vocab, d = c->d_model, F = c->d_ff, L = c->n_layer, H = c->n_head;
    if (T > (size_t)c->seq_len) return -2;
    float* x = (float*)malloc(T * d * sizeof(float));
    float* t0 = (float*)malloc(T * d * sizeof(float));
    float* t1 = (float*)malloc(T * d * sizeof(float));
    float* up = (float*)malloc(T * F * sizeof(float));
    float* gate = (float*)malloc(T * F * sizeof(float));
    float* act = (float*)malloc(T * F * sizeof(float));
    int rc = 0;
    const float* p = params;
    const float* tok = p; p += V * d;
    if (orc_embedding(tok, ids, x, T, V, d) != 0) { rc = -1; goto done; }
    if (taps) memcpy(taps, x, T * d * sizeof(float));
    for (size_t l = 0; l < L; l++) {
        const float* n1 = p;              const float* wq = n1 + d;
        const float* wk = wq + d * d;     const float* wv = wk + d * d;     const float* wo = wv + d * d;
        const float* n2 = wo + d * d;     const float* wu = n2 + d;         const float* bu = wu + F * d;
        const float* wg = bu + F;         const float* bg = wg + F * d;
        const float* wd = bg + F;         const float* bd = wd + d * F;
        p = bd + d;
        orc_rms_norm(x, n1, t0, T, d, c->eps);
        orc_mha_causal_rope(t0, wq, wk, wv, wo, t1, T, d, H, fast, rope_base, 0);
        orc_add(x, t1, x, T * d);
        orc_rms_norm(x, n2, t0, T, d, c->eps);
        orc_linear(t0, wu, bu, up, T, d, F, fast);
        orc_linear(t0, wg, bg, gate, T, d, F, fast);
        orc_swiglu(up, gate, act, T * F);
        orc_linear(act, wd, bd, t1, T, F, d, fast);
        orc_add(x, t1, x, T * d);
        if (taps) memcpy(taps + (l + 1) * T * d, x, T * d * sizeof(float));
    }
    {
        const float* nf = p; const float* head = nf + d;
        orc_rms_norm(x, nf, t0, T, d, c->eps);
        if (taps) memcpy(taps + (L + 1) * T * d, t0, T * d * sizeof(float));
        orc_linear(t0, head, NULL, logits, T, d, V, fast);
    }
done:
    free(x); free(t0); free(t1); free(up); free(gate); free(act);
    return rc;
}

int orc_qwen_forward_batch(const orc_gpt_config* c, float rope_base, const float* params, const int64_t* ids, size_t B,
                           size_t T, float* logits, float* taps, int fast, int threads) {
    size_t V = c->vocab, d = c->d_model, L = c->n_layer;
    int rc = 0;
#ifdef _OPENMP
    if (threads >= 1) omp_set_num_threads(threads);
#endif
    /* sequences one after another; the rows and heads of each are split over the threads */
    for (size_t b = 0; b < B; b++) {
        int r = orc_qwen_forward_ids(c, rope_base, params, ids + b * T, T, logits + b * T * V, taps ? taps + b * (L + 2) * T * d : NULL, fast);
        if (r != 0) rc = r;
    }
    return rc;
}

/* sampling_candidates: crates/nn/src/lib.rs:2381-2418 (penalize_repeated_logit :2343-2352, normalize_candidates :2354-2374).
 * out_* hold up to vocab_size entries; returns the number of candidates, or -1 if vocab_size exceeds n_logits (the
 * reference asserts).  The sort is a stable merge sort, as Rust's sort_by. */
typedef struct { int64_t id; float v; } orc_cand;
static void cand_merge_sort(orc_cand* a, orc_cand* tmp, size_t n) {
    if (n < 2) return;
    size_t h = n / 2;
    cand_merge_sort(a, tmp, h);
    cand_merge_sort(a + h, tmp, n - h);
    size_t i = 0, j = h, k = 0;
    while (i < h && j < n) tmp[k++] = (a[j].v > a[i].v) ? a[j++] : a[i++];      /* descending; equal values keep their order */
    while (i < h) tmp[k++] = a[i++];
    while (j < n) tmp[k++] = a[j++];
    memcpy(a, tmp, n * sizeof(orc_cand));
}
static void cand_normalize(const orc_cand* c, size_t n, float* probs) {
    if (n == 0) return;
    float mx = -INFINITY;
    for (size_t i = 0; i < n; i++) mx = fmaxf(mx, c[i].v);
    float sum = 0.0f;
    for (size_t i = 0; i < n; i++) { probs[i] = expf(c[i].v - mx); sum += probs[i]; }
    for (size_t i = 0; i < n; i++) probs[i] = probs[i] / sum;
}
/* filtered_step_logits (crates/nn/src/lib.rs:2465-2480): tokens outside the constraint's allowed set become -inf */
void orc_filter_step_logits(const float* logits, size_t n, const int64_t* allowed, size_t n_allowed, float* out) {
    for (size_t t = 0; t < n; t++) {
        int in = 0;
        for (size_t a = 0; a < n_allowed && !in; a++) in = allowed[a] == (int64_t)t;
        out[t] = in ? logits[t] : -INFINITY;
    }
}

long orc_sampling_candidates(const float* logits, size_t n_logits, size_t vocab_size, float temperature, size_t top_k, float top_p,
                             float repetition_penalty, const int64_t* history, size_t n_history,
                             int64_t* out_ids, float* out_logits, float* out_probs) {
    if (vocab_size > n_logits) return -1;
    float temp = fmaxf(temperature, 1e-8f);
    float penalty = fmaxf(repetition_penalty, 1.0f);
    orc_cand* c = (orc_cand*)malloc((vocab_size + 1) * sizeof(orc_cand));
    orc_cand* tmp = (orc_cand*)malloc((vocab_size + 1) * sizeof(orc_cand));
    size_t n = 0;
    for (size_t t = 0; t < vocab_size; t++) {
        float x = logits[t];
        int seen = 0;
        for (size_t h = 0; h < n_history && !seen; h++) seen = history[h] == (int64_t)t;
        if (penalty != 1.0f && seen) x = signbit(x) ? x * penalty : x / penalty;
        x = x / temp;
        if (isfinite(x)) { c[n].id = (int64_t)t; c[n].v = x; n++; }
    }
    cand_merge_sort(c, tmp, n);
    if (top_k > 0 && n > top_k) n = top_k;
    cand_normalize(c, n, out_probs);
    float p = top_p < 0.0f ? 0.0f : (top_p > 1.0f ? 1.0f : top_p);
    if (top_p != top_p) p = 0.0f;        /* clamp of a NaN is not reachable from the reference's configs; treated as 0 */
    if (!(p >= 1.0f) && n > 1) {
        float cum = 0.0f;
        size_t kept = 0;
        for (size_t i = 0; i < n; i++) { cum += out_probs[i]; kept = i + 1; if (cum >= p) break; }
        n = kept;
        cand_normalize(c, n, out_probs);
    }
    for (size_t i = 0; i < n; i++) { out_ids[i] = c[i].id; out_logits[i] = c[i].v; }
    free(c); free(tmp);
    return (long)n;
}

int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

int orc_gpt_forward_batch(const orc_gpt_config* c, const float* params, const int64_t* ids, size_t B,
                          size_t T, float* logits, float* taps, int fast, int threads) {
    size_t V = c->vocab, d = c->d_model, L = c->n_layer;
    int rc = 0;
    if (threads < 1) threads = 1;
#ifdef _OPENMP
    omp_set_num_threads(threads);       /* also bounds the row / head loops inside one sequence (threads == 1: truly one thread) */
#endif
    if (B < (size_t)threads) {
        /* fewer sequences than threads: run them one after another and split the rows / heads of each over the threads */
        for (size_t b = 0; b < B; b++) {
            int r = orc_gpt_forward_ids(c, params, ids + b * T, T, logits + b * T * V, taps ? taps + b * (L + 2) * T * d : NULL, fast);
            if (r != 0) rc = r;
        }
        return rc;
    }
#pragma omp parallel for schedule(dynamic, 1) num_threads(threads)
    for (long b = 0; b < (long)B; b++) {
        int r = orc_gpt_forward_ids(c, params, ids + (size_t)b * T, T, logits + (size_t)b * T * V,
                                    taps ? taps + (size_t)b * (L + 2) * T * d : NULL, fast);
        if (r != 0) {
#pragma omp critical
            rc = r;
        }
    }
    return rc;
}
