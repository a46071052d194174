// gemm.h -- internal interface of the tcgen05 GEMM (used by the C-ABI entry points, attention and the GPT driver).
#pragma once
#include "common.h"
#include <cuda.h>

namespace spt {

enum MMMode : int { MM_TF32 = 0, MM_BF16 = 1, MM_F32 = 2 };
// EPI_SWIGLU: C = R * g * sigmoid(g) with g = alpha * A B^T + bias (R is the other factor of the reference's swiglu(x, gate), not a residual)
enum Epilogue : int { EPI_NONE = 0, EPI_GELU = 1, EPI_SWIGLU = 2 };

// C[z][m,n] = act(alpha * sum_k A[z][m,k] * B[z][n,k] + bias[n]) + R[z][m,n]
// Both operands are K-major (k contiguous).  z = z1 + nb1*z2 enumerates two batch dimensions with
// independent element strides per operand (a head index and a sequence index, for attention).
struct GemmDesc {
    const void* A = nullptr; const void* B = nullptr; void* C = nullptr;
    const float* bias = nullptr; const void* R = nullptr;
    int M = 0, N = 0, K = 0;
    long long lda = 0, ldb = 0, ldc = 0;          // row strides in elements
    int nb1 = 1, nb2 = 1;
    long long sA1 = 0, sA2 = 0, sB1 = 0, sB2 = 0, sC1 = 0, sC2 = 0;   // batch strides in elements (C strides apply to R too)
    float alpha = 1.0f;
    int epilogue = EPI_NONE;
    int mode = MM_BF16;      // MM_BF16: A,B bf16.  MM_TF32: A,B f32.
    int out_dtype = BF16;    // C and R element type
    int causal_lower = 0;    // 1: square per-batch output, tiles entirely above the diagonal are skipped (never written)
    int b_broadcast = 0;     // 1: B has no batch dims (one weight matrix for every batch entry)
    // 1: a problem of at most 64 rows may run the weight-streaming kernel (linear_few_rows.cu) instead of 128-row tiles.  Its sums
    // are taken in another order, so the caller must not need a row's bits to be the same whatever the number of rows
    // (the model forward does: it leaves this 0; the decode step and the stand-alone Linear set it).
    int few_rows_ok = 0;
    int causal_k = 0;        // 1: A is lower triangular per batch (A[m,k] = 0 for k > m): k-blocks past the tile's last row are skipped
    // LayerNorm folded into the product.  With W' = W * gamma (per input feature), s[n] = sum_k W'[n,k], c[n] = sum_k beta[k] W[n,k] + bias[n]:
    //   LN(x) W^T + bias = inv[m] * (x W'^T)[m,n] - (mean[m] inv[m]) * s[n] + c[n]
    // so the GEMM reads the un-normalised rows and the epilogue applies the row statistics.  norm_axis 1: the normalised operand
    // is A (statistics per output row, s / c per output column, c passed as `bias`).  stats[i] = (inv_std, mean * inv_std).
    // norm_s must be readable up to N rounded up to 32 elements.
    int norm_axis = 0;
    const float2* norm_stats = nullptr;
    const float* norm_s = nullptr;
    // Row reductions instead of the output (the LM head followed by a loss / an argmax): C is not written.  Every epilogue thread
    // reduces the part of its output row it holds -- the values rounded to out_dtype first, so that they are exactly the logits the
    // ordinary epilogue would have stored -- to (maximum, sum of exp(x - maximum)) and the column of the first maximum, and writes
    // them to red_part / red_arg at [row * red_parts + 2 * n_tile + half]; red_parts = 2 * ceil(N / 256).  When red_targets is given,
    // the thread that holds column red_targets[row] also writes that logit to red_tgt[row].  Needs N > 128, no batch dims.
    int reduce = 0;
    float2* red_part = nullptr;
    int* red_arg = nullptr;
    const long long* red_targets = nullptr;
    float* red_tgt = nullptr;
};
inline int gemm_reduce_parts(int N) { return 2 * ((N + 255) / 256); }

// A prepared launch: tensor maps are encoded once and can be replayed (the GPT driver caches these).
struct GemmPlan {
    CUtensorMap tmA, tmB, tmC;
    bool tma_store = false;
    GemmDesc d;
    int bn = 0, tiles_m = 0, tiles_n = 0, grid = 0, group_m = 8;
    size_t smem = 0;
    bool pair = false;       // two-CTA tiles (256 x 256, cta_group::2); grid counts CTAs, two per tile worker
    bool few_rows = false;   // M <= 64 bf16: the weight-streaming kernel of linear_few_rows.cu instead of 128-row tiles
    bool valid = false;
};

// Returns 0 and fills plan, or non-zero with the reason in last_error (e.g. strides TMA cannot express).
int gemm_plan(const GemmDesc& d, GemmPlan* plan);
int gemm_run(const GemmPlan& plan);
// true when the tcgen05 path can take this problem (alignment / stride rules of TMA)
bool gemm_supported(const GemmDesc& d, const char** why);

// Linear for at most 64 input rows (a decode step), bf16: a stream over the weight rows spread over all SMs (linear_few_rows.cu).
// gemm_plan / gemm_run route there by themselves.
// nrm: the rows of A are normalised on the fly (kind 1: LayerNorm with gamma / beta, kind 2: RMSNorm with gamma), which saves the
// stand-alone normalisation launch in front of a projection.  dependent: launched as a programmatic dependent of the previous
// kernel in the stream (see launch_dependent in common.h).
struct RowNorm { int kind = 0; const float* gamma = nullptr; const float* beta = nullptr; float eps = 0.0f; };
bool linear_few_rows_supported(const GemmDesc& d);
bool linear_few_rows_norm_supported(const GemmDesc& d, const RowNorm& nrm);
int linear_few_rows(const GemmDesc& d, const RowNorm* nrm = nullptr, bool dependent = false);
// the normalisation alone, for at most 64 bf16 rows (row counts the projection kernel does not normalise itself)
bool norm_few_rows_supported(const void* x, const void* out, int rows, int K, const RowNorm& nrm);
int norm_few_rows(const void* x, void* out, int rows, int K, const RowNorm& nrm, bool dependent);

// CUDA-core f32 FMA matmul for shapes the TMA path cannot express and for MM_F32.
// B is [K,N] row-major when b_is_kn, else [N,K].
int simt_matmul_f32(const float* A, const float* B, float* C, int batch, int M, int N, int K, bool b_is_kn,
                    const float* bias, const float* R, float alpha, int epilogue);

int layernorm_launch(const void* x, const void* gamma, const void* beta, void* out, size_t rows, size_t dim, float eps, int dtype);
// LayerNorm folded into the following GEMM (GemmDesc::norm_axis): per-row statistics, and the folded weights / vectors
bool layernorm_stats_supported(size_t dim, int dtype);
int layernorm_stats_launch(const void* x, float2* stats, size_t rows, size_t dim, float eps, int dtype);
int layernorm_fold_launch(const void* w, const float* gamma, const float* beta, const float* bias, void* w_folded, float* svec, float* cvec,
                          size_t N, size_t K, int dtype);

}  // namespace spt
