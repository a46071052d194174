// gpt.cu -- device-resident GPT forward (crates/nn/src/lib.rs:1332-1364, blocks :1174-1214, MHA :574-642).
//
// The reference runs one sequence per call and allocates + copies on every op; here a batch of
// sequences is one [B*T, d] activation matrix (every op of the path is row- or sequence-local, so the
// per-sequence results are unchanged) and a layer is seven launches:
//   LN1 | [Wq;Wk;Wv] GEMM | fused causal attention | Wo GEMM (+residual) | LN2 | W_up GEMM (+bias, GELU) |
//   W_down GEMM (+bias, +residual)
// (models the fused attention kernel does not take -- f32, head sizes other than 64 / 128 -- run the attention as
// V^T GEMM | S = Q K^T | causal softmax | O = P V instead: eleven launches)
// Dropout (nn/src/lib.rs:168-182) is the identity in eval mode and is not launched.
// Weights keep the reference's [out,in] layout; parameter names are GPT::named_parameters' (nn/src/lib.rs:1382-1392).
// Tensor parallel (tp_size > 1): wq/wk/wv/ffn_up split by output rows (heads / d_ff columns), wo/ffn_down
// split along K; each produces a partial [M,d] that a caller-supplied all-reduce sums.  Rank 0 alone folds
// the residual and the ffn_down bias into its partial so that the reduced sum is the new residual stream.
#include "gemm.h"
#include "../../include/sptorch_b200_hal.h"
#include "../../include/sptorch_b200_ext.h"
#include <string>
#include <vector>
#include <cstring>
#include <cstdio>

namespace spt {

int attention_materialized(const void* q, const void* k, const void* vt, long long vt_ld, long long vt_s_head, long long vt_s_batch,
                           void* out, void* scores, int B, int Tn, int H, int hd, long long ld_qk, long long ld_out, int dtype);
int attention_fused(const void* q, const void* k, const void* v, void* out, int B, int T, int H, int hd, long long ld_q, long long ld_k,
                    long long ld_v, long long ld_out);
bool attention_uses_fused(int dtype, int Tn, int hd, long long ld_q, long long ld_kv);
int rope_launch(void* x, long long rows, int Tn, int n_slots, int hd, long long ld, float base, int offset, int dtype, const int* offset_dev = nullptr);
int compact_rows_launch(const void* src, void* dst, size_t rows, size_t cols, size_t ld, int es);
int head_reduce_combine_launch(const float2* part, const int* arg, const float* tgt_logit, const long long* targets, size_t rows, int parts,
                               int classes, int has_ignore, long long ignore_index, int* argmax_out, float* row_loss);
int cross_entropy_mean_launch(float* row_loss, size_t rows);
int attention_last_token(const void* q, long long ld_q, const void* kc, const void* vc, void* out, long long ld_out, int B, int H, int hd,
                         int n, long long seq_stride, long long row_stride, int dtype, const int* state, int n_cap,
                         const void* fresh_k, const void* fresh_v, long long ld_fresh, int slot, bool dependent);
bool attention_last_token_takes_fresh(int hd, int dtype);
int decode_state_launch(int* state, int pos, int n, int slot, int pos_row);
int kv_append_launch(const void* qkv, void* kc, void* vc, int B, int dl, long long seq_stride, int slot, const int* state, int dtype);
int embedding_sum_launch(const void* tok_w, const void* pos_w, const void* ids, void* out, size_t n_tokens, size_t T, size_t vocab, size_t dim,
                         int dtype, const int* pos_row_dev);

struct Layer {
    float *ln1g, *ln1b, *ln2g, *ln2b, *b1, *b2;     // Qwen-like: ln1g / ln2g hold the RMSNorm weights, the betas are unused
    void *wqkv;                                      // [Wq; Wk; Wv] of this rank, one [3*d_loc, d] matrix
    void *wqk, *wv, *wo, *w1, *w2;                   // wqk = rows 0..2*d_loc of wqkv, wv = rows 2*d_loc..
    void* wg = nullptr; float* bg = nullptr;         // Qwen-like: gate projection of the SwiGLU MLP
    // LayerNorm folded into the GEMMs that consume it (bf16 GPT): weights times gamma, their row sums s, and c = W beta (+ bias)
    void *wqkv_f = nullptr, *w1_f = nullptr;
    float *s_qkv = nullptr, *c_qkv = nullptr, *s_1 = nullptr, *c_1 = nullptr;
};

struct Gpt {
    sptorch_gpt_config c;
    int es;                 // bytes per activation/weight element
    int d_loc, H_loc, F_loc;
    size_t ldl;             // logits row stride
    void *tok, *pos, *head;
    float *lnfg, *lnfb;
    std::vector<Layer> L;
    // activations for max_batch * seq_len tokens
    void *x, *y, *h, *qkv, *ao, *f;                // qkv: [tokens, 3*d_loc] = [q | k | v] of every token
    void *vt = nullptr, *scores = nullptr;          // materialised attention only (ensure_scores): V^T [d_loc, tokens], scores [batch, heads, T, T]
    size_t scores_elems = 0, vt_elems = 0;
    std::vector<void*> taps; bool taps_on = false;
    sptorch_allreduce_fn ar = nullptr; void* ar_user = nullptr;
    std::vector<void*> owned;
    // pipelined host call
    void* logits_dev[2] = {nullptr, nullptr}; int* ids_dev = nullptr; int ids_cap = 0; size_t logits_cap = 0;
    cudaEvent_t ev_compute[2] = {nullptr, nullptr}, ev_copy[2] = {nullptr, nullptr};
    cudaEvent_t ev_partial[2] = {nullptr, nullptr}, ev_reduced[2] = {nullptr, nullptr};     // tensor-parallel pipeline
    // key/value cache for incremental decode: [layer][sequence][position][d_loc], allocated by gpt_enable_kv_cache
    void *kcache = nullptr, *vcache = nullptr;
    int cache_ctx = 0, cached_len = 0, cache_batch = 0;
    long long window_start = 0;   // absolute position of the oldest cached token (grows once the cache is full and slides)
    int* dstate = nullptr;        // device words of the current decode step: position, valid positions, ring slot, position-table row
    struct DecodeKey {
        const void* ids; void* logits; int batch, append; cudaStream_t stream; uint64_t epoch;
        bool operator==(const DecodeKey& o) const { return ids == o.ids && logits == o.logits && batch == o.batch && append == o.append && stream == o.stream && epoch == o.epoch; }
    };
    DecodeKey dkey = {nullptr, nullptr, 0, 0, nullptr, 0};
    cudaGraphExec_t dexec = nullptr; int d_eager = 0;
    bool fill_cache = false;      // set while a prefill runs
    void *dq = nullptr;                  // decode scratch: [max_batch, 3*d_loc] = [q | k | v] of the new tokens
    // CUDA graph of one forward, keyed by everything that is baked into its kernel arguments
    // (the config epoch covers the process-wide setters that change which kernels or grids a forward launches)
    struct GraphKey {
        const void* ids; void* logits; int batch, T; bool taps; cudaStream_t stream; uint64_t epoch;
        const void *targets, *argmax, *row_loss; int has_ignore; long long ignore_index; bool reduce;      // fused LM head (HeadReduce)
        bool operator==(const GraphKey& o) const {
            return ids == o.ids && logits == o.logits && batch == o.batch && T == o.T && taps == o.taps && stream == o.stream && epoch == o.epoch &&
                   targets == o.targets && argmax == o.argmax && row_loss == o.row_loss && has_ignore == o.has_ignore &&
                   ignore_index == o.ignore_index && reduce == o.reduce;
        }
    };
    // a few keys are kept so that callers alternating between buffers (double buffering) replay instead of re-capturing
    struct GraphSlot { GraphKey key; cudaGraphExec_t exec = nullptr; int eager_runs = 0; uint64_t last_use = 0; };
    static constexpr int kGraphSlots = 4;
    GraphSlot gslots[kGraphSlots];
    uint64_t guse = 0;
    bool graphs = true;
    // folded LayerNorm (see forward): per-token statistics, the head's folded copy, and whether the copies are stale
    float2* ln_stats = nullptr; void* head_f = nullptr; float *s_h = nullptr, *c_h = nullptr;
    bool ln_fold = false, fold_ready = false, fold_dirty = true;     // opt-in: measured neutral (see sptorch_ext_gpt_enable_ln_fold)
    int tp_overlap = 2;        // tensor parallel: reduce one half of the batch while the other half computes: 0 never, 1 always, 2 from 4 ranks up
    // LM head fused with the loss / greedy choice: per-row partial reductions of the head GEMM's tiles
    float2* red_part = nullptr; int* red_arg = nullptr; float* red_tgt = nullptr; size_t red_rows = 0;
    // host-buffer loss call: targets, greedy tokens and row losses of the whole batch on the device
    long long* loss_targets = nullptr; int* loss_argmax = nullptr; float* loss_rows = nullptr; size_t loss_cap = 0;
};

static void drop_graphs(Gpt* g) {
    if (g->dexec) { cudaGraphExecDestroy(g->dexec); g->dexec = nullptr; }
    g->d_eager = 0;
    for (auto& sl : g->gslots) {
        if (sl.exec) cudaGraphExecDestroy(sl.exec);
        sl = Gpt::GraphSlot();
    }
}

// returns a block of the model to the pool before the model itself goes (buffers that are re-allocated larger)
static void gfree(Gpt* g, void* p) {
    if (!p) return;
    for (auto it = g->owned.begin(); it != g->owned.end(); ++it)
        if (*it == p) { g->owned.erase(it); break; }
    sptorch_free(p);
}

static void* galloc(Gpt* g, size_t bytes) {
    void* p = sptorch_ext_alloc_bytes(bytes);
    if (p) g->owned.push_back(p);
    return p;
}

static int upload_rows(Gpt* g, void* dst_model_dtype, const float* host, size_t n) {
    // host f32 -> device in the model dtype (bf16: round to nearest even on the device)
    if (g->c.dtype == SPT_F32) return sptorch_ext_copy_h2d_bytes(host, dst_model_dtype, n * 4);
    float* tmp = (float*)sptorch_ext_alloc_bytes(n * 4);
    if (!tmp) return 1;
    int rc = sptorch_ext_copy_h2d_bytes(host, tmp, n * 4);
    if (!rc) rc = sptorch_ext_f32_to_bf16(tmp, dst_model_dtype, n);
    if (!rc) rc = stream_wait();       // host buffer and tmp may be released after return
    sptorch_free(tmp);
    return rc;
}

// ---- tensor-parallel shard rule (host code, no device needed) ----
// Megatron split of the block's projections over tp_size ranks: wq / wk / wv / ffn_up (and the Qwen-like ffn_gate) are cut by
// OUTPUT rows (heads, d_ff columns), their biases with them; wo / ffn_down are cut along K (input columns) so that every rank
// produces a partial [M, d] sum; everything else is replicated.  Rank 0 alone adds the residual and the row-parallel bias
// (ffn_down.bias) to its partial, so that the all-reduced sum is the new residual stream.
enum TpKind : int { TP_REPLICATED = 0, TP_ROWS = 1, TP_COLS = 2 };
static int tp_kind_of(const std::string& name) {
    auto ends = [&](const char* suf) { const size_t n = strlen(suf); return name.size() >= n && name.compare(name.size() - n, n, suf) == 0; };
    if (name.compare(0, 7, "blocks.") != 0) return TP_REPLICATED;
    if (ends("attn.wq.weight") || ends("attn.wk.weight") || ends("attn.wv.weight") || ends("ffn_up.weight") || ends("ffn_up.bias") ||
        ends("ffn_gate.weight") || ends("ffn_gate.bias")) return TP_ROWS;
    if (ends("attn.wo.weight") || ends("ffn_down.weight")) return TP_COLS;
    return TP_REPLICATED;
}

}  // namespace spt

extern "C" {

int sptorch_ext_tp_param_shard(const char* name, int tp_rank, int tp_size, size_t rows, size_t cols, int* kind, size_t* begin, size_t* count) {
    using namespace spt;
    if (!name || !kind || !begin || !count) return fail_host("tp_param_shard: null argument");
    if (tp_size < 1 || tp_rank < 0 || tp_rank >= tp_size) return fail_host("tp_param_shard: rank %d of %d", tp_rank, tp_size);
    const int k = tp_kind_of(name);
    *kind = k;
    if (k == TP_REPLICATED) { *begin = 0; *count = rows; return 0; }
    const size_t extent = k == TP_ROWS ? rows : cols;
    if (extent % (size_t)tp_size) return fail_host("tp_param_shard(%s): extent %zu does not divide by tp_size %d", name, extent, tp_size);
    *count = extent / (size_t)tp_size;
    *begin = (size_t)tp_rank * *count;
    return 0;
}

int sptorch_ext_tp_slice_host(const float* full, size_t rows, size_t cols, int kind, size_t begin, size_t count, float* out) {
    using namespace spt;
    if (!full || !out) return fail_host("tp_slice_host: null argument");
    if (kind == TP_REPLICATED) { memcpy(out, full, rows * cols * sizeof(float)); return 0; }
    if (kind == TP_ROWS) {
        if (begin + count > rows) return fail_host("tp_slice_host: rows [%zu, %zu) outside %zu", begin, begin + count, rows);
        memcpy(out, full + begin * cols, count * cols * sizeof(float));
        return 0;
    }
    if (kind == TP_COLS) {
        if (begin + count > cols) return fail_host("tp_slice_host: columns [%zu, %zu) outside %zu", begin, begin + count, cols);
        for (size_t r = 0; r < rows; r++) memcpy(out + r * count, full + r * cols + begin, count * sizeof(float));
        return 0;
    }
    return fail_host("tp_slice_host: unknown kind %d", kind);
}

int sptorch_ext_tp_rank_folds_residual(int tp_rank) { return tp_rank == 0 ? 1 : 0; }

}  // extern "C"

namespace spt {

// this rank's shard of a full [R, C] host tensor (a vector is [R, 1]) -> device, in the model dtype (f32 for vectors)
static int upload_shard(Gpt* g, void* dst, const char* name, const float* host, size_t R, size_t C, bool as_f32) {
    int kind; size_t begin, count;
    if (sptorch_ext_tp_param_shard(name, g->c.tp_rank, g->c.tp_size, R, C, &kind, &begin, &count)) return fail("gpt_set_param(%s): no shard rule", name);
    const size_t n = kind == TP_COLS ? R * count : count * C;
    const float* src = host;
    std::vector<float> tmp;
    if (kind == TP_ROWS) src = host + begin * C;                        // contiguous
    else if (kind == TP_COLS && count != C) {
        tmp.resize(n);
        if (sptorch_ext_tp_slice_host(host, R, C, kind, begin, count, tmp.data())) return 1;
        src = tmp.data();
    }
    if (as_f32) return sptorch_ext_copy_h2d_bytes(src, dst, n * 4) || stream_wait();
    return upload_rows(g, dst, src, n);
}

static int linear(Gpt* g, const void* x, const void* w, const float* bias, const void* res, void* out, int M, int K, int N,
                  long long ldo, int epi) {
    GemmDesc d;
    d.A = x; d.B = w; d.C = out; d.bias = bias; d.R = res;
    d.M = M; d.N = N; d.K = K; d.lda = K; d.ldb = K; d.ldc = ldo;
    d.epilogue = epi;
    d.mode = g->c.dtype == SPT_BF16 ? MM_BF16 : MM_TF32;
    d.out_dtype = g->c.dtype;
    GemmPlan pl;
    if (gemm_plan(d, &pl)) return 1;
    ProfScope ps(PROF_LINEAR);
    return gemm_run(pl);
}

static int ln(const void* x, const float* g_, const float* b_, void* out, size_t rows, size_t dim, float eps, int dt) {
    ProfScope ps(PROF_LAYERNORM);
    return layernorm_launch(x, g_, b_, out, rows, dim, eps, dt);
}

static int allreduce(Gpt* g, void* buf, size_t n) {
    if (g->c.tp_size <= 1) return 0;
    if (!g->ar) return fail("gpt: tensor parallel forward needs an all-reduce hook (sptorch_ext_gpt_set_allreduce)");
    ProfScope ps(PROF_OTHER);
    if (g->ar(buf, n, g->c.dtype, (void*)rt().stream, g->ar_user)) return fail("gpt: all-reduce hook failed");
    note_submit();
    return 0;
}

// ---- LayerNorm folded into the GEMMs ----
// LN(x) W^T + b = inv * (x (W gamma)^T) - (mean inv) * s + c with s = rowsum(W gamma), c = W beta + b.  The forward then launches,
// instead of a LayerNorm pass that reads and writes every activation, a statistics pass that only reads them (8 bytes per token
// out), and the GEMMs consume the residual stream directly.  Used for bf16 GPT models whose GEMMs all take the 256-column tile.
static bool model_uses_fused(const Gpt* g, int T);
static bool fold_applicable(const Gpt* g, int M, int T) {
    const sptorch_gpt_config& c = g->c;
    return g->ln_fold && c.arch == SPT_ARCH_GPT && c.dtype == SPT_BF16 && !g->fill_cache && layernorm_stats_supported((size_t)c.d_model, c.dtype) &&
           3 * g->d_loc > 128 && g->F_loc > 128 && c.vocab > 128 && M > 128 && M % 2 == 0 && model_uses_fused(g, T);
}

static int fold_prepare(Gpt* g) {
    const sptorch_gpt_config& c = g->c;
    const size_t d = c.d_model, dl = g->d_loc, Fl = g->F_loc, V = c.vocab, es = g->es;
    auto pad32 = [](size_t n) { return (n + 31) / 32 * 32; };
    if (!g->fold_ready) {
        bool ok = true;
        auto A = [&](size_t bytes) { void* p = galloc(g, bytes); if (!p) ok = false; return p; };
        auto Z = [&](size_t n) { float* p = (float*)A(pad32(n) * 4); if (p && sptorch_ext_memset(p, 0, pad32(n) * 4)) ok = false; return p; };
        for (auto& w : g->L) {
            w.wqkv_f = A(3 * dl * d * es); w.w1_f = A(Fl * d * es);
            w.s_qkv = Z(3 * dl); w.c_qkv = Z(3 * dl); w.s_1 = Z(Fl); w.c_1 = Z(Fl);
        }
        g->head_f = A(V * d * es); g->s_h = Z(V); g->c_h = Z(V);
        g->ln_stats = (float2*)A(((size_t)c.max_batch * c.seq_len + 32) * sizeof(float2));
        if (ok && sptorch_ext_memset(g->ln_stats, 0, ((size_t)c.max_batch * c.seq_len + 32) * sizeof(float2))) ok = false;
        if (!ok) return 1;
        g->fold_ready = true; g->fold_dirty = true;
    }
    if (g->fold_dirty) {
        for (auto& w : g->L) {
            if (layernorm_fold_launch(w.wqkv, w.ln1g, w.ln1b, nullptr, w.wqkv_f, w.s_qkv, w.c_qkv, 3 * dl, d, c.dtype)) return 1;
            if (layernorm_fold_launch(w.w1, w.ln2g, w.ln2b, w.b1, w.w1_f, w.s_1, w.c_1, Fl, d, c.dtype)) return 1;
        }
        if (layernorm_fold_launch(g->head, g->lnfg, g->lnfb, nullptr, g->head_f, g->s_h, g->c_h, V, d, c.dtype)) return 1;
        g->fold_dirty = false;
    }
    return 0;
}

static int ln_stats(Gpt* g, const void* x, int M) {
    ProfScope ps(PROF_LAYERNORM);
    return layernorm_stats_launch(x, g->ln_stats, (size_t)M, (size_t)g->c.d_model, g->c.eps, g->c.dtype);
}

// y[M,N] = act(LN(x) W^T + b) from the un-normalised x and the folded constants
static int linear_folded(Gpt* g, const void* x, const void* wf, const float* cvec, const float* svec, void* out, int M, int K, int N, long long ldo, int epi) {
    GemmDesc d;
    d.A = x; d.B = wf; d.C = out; d.bias = cvec;
    d.M = M; d.N = N; d.K = K; d.lda = K; d.ldb = K; d.ldc = ldo;
    d.epilogue = epi; d.mode = MM_BF16; d.out_dtype = SPT_BF16;
    d.norm_axis = 1; d.norm_stats = g->ln_stats; d.norm_s = svec;
    GemmPlan pl;
    if (gemm_plan(d, &pl)) return 1;
    ProfScope ps(PROF_LINEAR);
    return gemm_run(pl);
}

// true when the blocks of this model run the fused attention kernel on sequences of T tokens
static bool model_uses_fused(const Gpt* g, int T) {
    return attention_uses_fused(g->c.dtype, T, g->c.d_model / g->c.n_head, 3 * g->d_loc, 3 * g->d_loc);
}

// The [batch, heads, T, T] score workspace and the V^T buffer exist only for the materialised attention (f32 models, head sizes
// other than 64 / 128, or sptorch_ext_set_attention_mode(1)); the fused kernel never touches them.  They are sized for the batch
// actually run and grown on demand, outside any graph capture.
static int ensure_scores(Gpt* g, int batch, int T) {
    if (model_uses_fused(g, T)) return 0;
    const size_t need = (size_t)batch * g->H_loc * T * T, need_vt = (size_t)g->d_loc * batch * T;
    if (need <= g->scores_elems && need_vt <= g->vt_elems) return 0;
    if (stream_wait()) return 1;                   // nothing in flight may still read the old workspace
    drop_graphs(g);                                // captured launches hold its address
    if (need > g->scores_elems) {
        gfree(g, g->scores);
        g->scores = galloc(g, need * g->es);
        g->scores_elems = g->scores ? need : 0;
        if (!g->scores) return 1;
    }
    if (need_vt > g->vt_elems) {
        gfree(g, g->vt);
        g->vt = galloc(g, need_vt * g->es);
        g->vt_elems = g->vt ? need_vt : 0;
        if (!g->vt) return 1;
    }
    return 0;
}

// One block's attention from the normalised rows h [M, d] (M = B*T tokens) to the merged heads ao [M, d_loc]:
//   [q | k | v] = h [Wq;Wk;Wv]^T  (one GEMM, N = 3*d_loc)  ->  (Qwen-like: RoPE on the q and k columns)  ->  causal attention.
// The fused kernel reads q, k and v in place from the [M, 3*d_loc] buffer.  The materialised form needs V^T as the K-major
// operand of P V, which one more GEMM with swapped operands produces (V^T = Wv h^T).
// During a prefill the (rotated) keys and the values of every position are also copied into the cache rows
// [sequence][position][d_loc] of layer l (project_kv_cache_with_offset, nn/src/lib.rs:672-683).
// qkv / ao / scores / vt: the buffers of this call (the pipelined tensor-parallel forward passes halves of them).
static int attention_block(Gpt* g, const Layer& w, int l, const void* h, void* qkv, void* ao, int B, int T, bool folded, const void* x_unnorm) {
    const sptorch_gpt_config& c = g->c;
    const int d = c.d_model, M = B * T, dl = g->d_loc, Hl = g->H_loc, hd = d / c.n_head, dt = c.dtype;
    const size_t es = g->es;
    if (folded) { if (linear_folded(g, x_unnorm, w.wqkv_f, w.c_qkv, w.s_qkv, qkv, M, d, 3 * dl, 3 * dl, EPI_NONE)) return 1; }
    else if (linear(g, h, w.wqkv, nullptr, nullptr, qkv, M, d, 3 * dl, 3 * dl, EPI_NONE)) return 1;
    if (c.arch == SPT_ARCH_QWEN_LIKE) { ProfScope ps(PROF_OTHER); if (rope_launch(qkv, M, T, 2 * Hl, hd, 3 * dl, c.rope_base, 0, dt)) return 1; }
    const uint8_t* qp = (const uint8_t*)qkv;
    const uint8_t* kp = qp + (size_t)dl * es;
    const uint8_t* vp = qp + (size_t)2 * dl * es;
    if (g->fill_cache) {
        const size_t lay = (size_t)l * c.max_batch * g->cache_ctx * dl * es;
        ProfScope ps(PROF_OTHER);
        for (int b = 0; b < B; b++) {
            const size_t dst = lay + (size_t)b * g->cache_ctx * dl * es, src = (size_t)b * T * 3 * dl * es;
            SPT_CUDA(cudaMemcpy2DAsync((uint8_t*)g->kcache + dst, (size_t)dl * es, kp + src, (size_t)3 * dl * es, (size_t)dl * es, (size_t)T,
                                       cudaMemcpyDeviceToDevice, rt().stream));
            SPT_CUDA(cudaMemcpy2DAsync((uint8_t*)g->vcache + dst, (size_t)dl * es, vp + src, (size_t)3 * dl * es, (size_t)dl * es, (size_t)T,
                                       cudaMemcpyDeviceToDevice, rt().stream));
        }
    }
    if (model_uses_fused(g, T)) return attention_fused(qp, kp, vp, ao, B, T, Hl, hd, 3 * dl, 3 * dl, 3 * dl, dl);
    if (folded) return fail("gpt: the folded LayerNorm runs with the fused attention only");
    if (linear(g, w.wv, h, nullptr, nullptr, g->vt, dl, d, M, M, EPI_NONE)) return 1;
    return attention_materialized(qp, kp, g->vt, /*vt_ld*/ M, /*head*/ (long long)hd * M, /*batch*/ T, ao, g->scores, B, T, Hl, hd, 3 * dl, dl, dt);
}

// What replaces the logits when the LM head is fused with the step after it (cross_entropy_loss(_ignore_index), core-ops/src/lib.rs:1079-1194;
// the greedy token = first candidate of sampling_candidates, nn/src/lib.rs:2381-2418): per-row loss and / or the column of the row maximum.
struct HeadReduce { const long long* targets; int has_ignore; long long ignore_index; int* argmax; float* row_loss; };

// partial-reduction buffers for `rows` tokens (grown outside any graph capture)
static int ensure_reduce(Gpt* g, size_t rows) {
    if (rows <= g->red_rows) return 0;
    if (stream_wait()) return 1;
    drop_graphs(g);
    const size_t parts = (size_t)gemm_reduce_parts(g->c.vocab);
    gfree(g, g->red_part); gfree(g, g->red_arg); gfree(g, g->red_tgt);
    g->red_part = (float2*)galloc(g, rows * parts * sizeof(float2));
    g->red_arg = (int*)galloc(g, rows * parts * sizeof(int));
    g->red_tgt = (float*)galloc(g, rows * sizeof(float));
    g->red_rows = (g->red_part && g->red_arg && g->red_tgt) ? rows : 0;
    return g->red_rows ? 0 : 1;
}

// logits = h head^T, or -- with hr -- the row reductions of that product without the [M, vocab] matrix ever reaching HBM
static int lm_head(Gpt* g, const void* h, int M, void* logits, const HeadReduce* hr) {
    const sptorch_gpt_config& c = g->c;
    if (!hr) return linear(g, h, g->head, nullptr, nullptr, logits, M, c.d_model, c.vocab, (long long)g->ldl, EPI_NONE);
    if ((size_t)M > g->red_rows) return fail("gpt: reduction buffers not prepared for %d rows", M);
    GemmDesc d;
    d.A = h; d.B = g->head; d.C = nullptr;
    d.M = M; d.N = c.vocab; d.K = c.d_model; d.lda = c.d_model; d.ldb = c.d_model; d.ldc = (long long)g->ldl;
    d.mode = c.dtype == SPT_BF16 ? MM_BF16 : MM_TF32; d.out_dtype = c.dtype;
    d.reduce = 1; d.red_part = g->red_part; d.red_arg = g->red_arg; d.red_targets = hr->row_loss ? hr->targets : nullptr; d.red_tgt = g->red_tgt;
    GemmPlan pl;
    if (gemm_plan(d, &pl)) return 1;
    { ProfScope ps(PROF_LINEAR); if (gemm_run(pl)) return 1; }
    ProfScope ps(PROF_OTHER);
    return head_reduce_combine_launch(g->red_part, g->red_arg, g->red_tgt, hr->targets, (size_t)M, gemm_reduce_parts(c.vocab), c.vocab, hr->has_ignore,
                                      hr->ignore_index, hr->argmax, hr->row_loss);
}

// Tensor-parallel forward with the all-reduces taken off the critical path: the batch is cut into two halves that go
// through each half-block alternately, the partial sums of one half are reduced on a second stream while the other
// half computes.  The persistent kernels must leave SMs free for the collective: unless the caller has set a reserve
// (sptorch_ext_set_sm_reserve), kTpOverlapReserve SMs are left free for the duration of the call.
// Measured on 4 x B200, 12 layers of the 1.3B shape (d 2048, 16 x 2048 tokens), ms per step: serial 25.7 (all-reduce 10.3);
// overlapped with 16 / 24 / 32 / 40 / 48 / 64 SMs free: 23.0 / 22.2 / 21.1 / 21.6 / 22.0 / 23.9.  On 2 GPUs the all-reduce is a
// fifth of the step and the SMs given up cost what the overlap hides (22.0 serial, 21.5 at best), hence from four ranks up.
constexpr int kTpOverlapReserve = 32;
constexpr int kTpOverlapFromRanks = 4;
struct SmReserveScope {
    int saved;
    SmReserveScope() : saved(rt().sm_reserve) { if (saved == 0) rt().sm_reserve = kTpOverlapReserve; }
    ~SmReserveScope() { rt().sm_reserve = saved; }
};
static int forward_tp_pipelined(Gpt* g, const void* ids, int B, int T, void* logits, const HeadReduce* hr) {
    const sptorch_gpt_config& c = g->c;
    const int d = c.d_model, M = B * T, dl = g->d_loc, Fl = g->F_loc, dt = c.dtype;
    const bool lead = c.tp_rank == 0;
    const size_t es = g->es;
    const int Bc = B / 2, Mc = Bc * T;
    cudaStream_t cs = rt().stream, ms = rt().copy_stream;
    for (int i = 0; i < 2; i++) {
        if (!g->ev_partial[i]) SPT_CUDA(cudaEventCreateWithFlags(&g->ev_partial[i], cudaEventDisableTiming));
        if (!g->ev_reduced[i]) SPT_CUDA(cudaEventCreateWithFlags(&g->ev_reduced[i], cudaEventDisableTiming));
    }
    { ProfScope ps(PROF_EMBED); if (sptorch_ext_embedding_sum(g->tok, g->pos, ids, g->x, (size_t)M, (size_t)T, (size_t)c.vocab, (size_t)d, dt)) return 1; }
    auto rows = [&](void* base, int ch, size_t width) { return (void*)((uint8_t*)base + (size_t)ch * Mc * width * es); };
    void* xb[2] = {rows(g->x, 0, d), rows(g->x, 1, d)};
    void* yb[2] = {rows(g->y, 0, d), rows(g->y, 1, d)};
    bool pending[2] = {false, false};             // a reduction of this half is in flight on the second stream
    {
    SmReserveScope reserve;                       // the blocks only: the final LayerNorm and the LM head run beside no collective
    auto reduce_async = [&](int ch) -> int {
        SPT_CUDA(cudaEventRecord(g->ev_partial[ch], cs));
        SPT_CUDA(cudaStreamWaitEvent(ms, g->ev_partial[ch], 0));
        if (g->ar(yb[ch], (size_t)Mc * d, dt, (void*)ms, g->ar_user)) return fail("gpt: all-reduce hook failed");
        SPT_CUDA(cudaEventRecord(g->ev_reduced[ch], ms));
        std::swap(xb[ch], yb[ch]);
        pending[ch] = true;
        return 0;
    };
    auto wait_reduced = [&](int ch) -> int {
        if (pending[ch]) { SPT_CUDA(cudaStreamWaitEvent(cs, g->ev_reduced[ch], 0)); pending[ch] = false; }
        return 0;
    };
    for (int l = 0; l < c.n_layer; l++) {
        const Layer& w = g->L[l];
        for (int ch = 0; ch < 2; ch++) {
            if (wait_reduced(ch)) return 1;
            void* h = rows(g->h, ch, d); void* qkv = rows(g->qkv, ch, 3 * dl); void* ao = rows(g->ao, ch, dl);
            if (ln(xb[ch], w.ln1g, w.ln1b, h, (size_t)Mc, (size_t)d, c.eps, dt)) return 1;
            if (attention_block(g, w, l, h, qkv, ao, Bc, T, false, nullptr)) return 1;
            if (linear(g, ao, w.wo, nullptr, lead ? xb[ch] : nullptr, yb[ch], Mc, dl, d, d, EPI_NONE)) return 1;
            if (reduce_async(ch)) return 1;
        }
        for (int ch = 0; ch < 2; ch++) {
            if (wait_reduced(ch)) return 1;
            void* h = rows(g->h, ch, d); void* f = rows(g->f, ch, Fl);
            if (ln(xb[ch], w.ln2g, w.ln2b, h, (size_t)Mc, (size_t)d, c.eps, dt)) return 1;
            if (linear(g, h, w.w1, w.b1, nullptr, f, Mc, d, Fl, Fl, EPI_GELU)) return 1;
            if (linear(g, f, w.w2, lead ? w.b2 : nullptr, lead ? xb[ch] : nullptr, yb[ch], Mc, Fl, d, d, EPI_NONE)) return 1;
            if (reduce_async(ch)) return 1;
        }
    }
    if (wait_reduced(0) || wait_reduced(1)) return 1;
    }
    // two swaps per layer and half: both halves are back in the same base buffer, contiguous
    void* x = xb[0];
    if (ln(x, g->lnfg, g->lnfb, g->h, (size_t)M, (size_t)d, c.eps, dt)) return 1;
    if (lm_head(g, g->h, M, logits, hr)) return 1;
    note_submit();
    return 0;
}

int rms_launch(const void* x, const float* w, void* out, size_t rows, size_t dim, float eps, int dt) {
    ProfScope ps(PROF_LAYERNORM);
    return sptorch_ext_rms_norm(x, w, out, rows, dim, eps, dt);
}

// QwenLikeGPT::forward_ids (nn/src/lib.rs:1454-1467) over a batch; block = QwenLikeBlock::forward_seq_inference (:1106-1117):
//   x += Wo attn(rope(q), rope(k), v) of rms(x);  x += Wdown (up * gate * sigmoid(gate)) + bdown of rms(x)
// Launches per layer: RMSNorm, [q|k|v] GEMM, RoPE over q and k, attention, Wo GEMM (+residual), RMSNorm, up GEMM (+bias),
// gate GEMM (+bias, SwiGLU product with the up output in the epilogue), down GEMM (+bias, +residual).
static int forward_qwen(Gpt* g, const void* ids, int B, int T, void* logits, const HeadReduce* hr) {
    const sptorch_gpt_config& c = g->c;
    const int d = c.d_model, M = B * T, dl = g->d_loc, Fl = g->F_loc, dt = c.dtype;
    const bool lead = c.tp_rank == 0;
    { ProfScope ps(PROF_EMBED); if (sptorch_ext_embedding_sum(g->tok, nullptr, ids, g->x, (size_t)M, (size_t)T, (size_t)c.vocab, (size_t)d, dt)) return 1; }
    void* x = g->x; void* y = g->y;
    auto tap = [&](int i, const void* src) -> int {
        if (!g->taps_on) return 0;
        SPT_CUDA(cudaMemcpyAsync(g->taps[i], src, (size_t)M * d * g->es, cudaMemcpyDeviceToDevice, rt().stream));
        return 0;
    };
    if (tap(0, x)) return 1;
    for (int l = 0; l < c.n_layer; l++) {
        const Layer& w = g->L[l];
        if (rms_launch(x, w.ln1g, g->h, (size_t)M, (size_t)d, c.eps, dt)) return 1;
        if (attention_block(g, w, l, g->h, g->qkv, g->ao, B, T, false, nullptr)) return 1;
        if (c.tp_size <= 1) {
            if (linear(g, g->ao, w.wo, nullptr, x, x, M, dl, d, d, EPI_NONE)) return 1;
        } else {
            if (linear(g, g->ao, w.wo, nullptr, lead ? x : nullptr, y, M, dl, d, d, EPI_NONE)) return 1;
            if (allreduce(g, y, (size_t)M * d)) return 1;
            std::swap(x, y);
        }
        if (rms_launch(x, w.ln2g, g->h, (size_t)M, (size_t)d, c.eps, dt)) return 1;
        if (linear(g, g->h, w.w1, w.b1, nullptr, g->f, M, d, Fl, Fl, EPI_NONE)) return 1;                 // up
        if (linear(g, g->h, w.wg, w.bg, g->f, g->f, M, d, Fl, Fl, EPI_SWIGLU)) return 1;                  // f = up * silu(gate)
        if (c.tp_size <= 1) {
            if (linear(g, g->f, w.w2, w.b2, x, x, M, Fl, d, d, EPI_NONE)) return 1;
        } else {
            if (linear(g, g->f, w.w2, lead ? w.b2 : nullptr, lead ? x : nullptr, y, M, Fl, d, d, EPI_NONE)) return 1;
            if (allreduce(g, y, (size_t)M * d)) return 1;
            std::swap(x, y);
        }
        if (tap(l + 1, x)) return 1;
    }
    if (rms_launch(x, g->lnfg, g->h, (size_t)M, (size_t)d, c.eps, dt)) return 1;
    if (tap(c.n_layer + 1, g->h)) return 1;
    return lm_head(g, g->h, M, logits, hr);
}

static int forward(Gpt* g, const void* ids, int B, int T, void* logits, const HeadReduce* hr = nullptr) {
    if (g->c.arch == SPT_ARCH_QWEN_LIKE) return forward_qwen(g, ids, B, T, logits, hr);
    const bool overlap = g->tp_overlap == 1 || (g->tp_overlap == 2 && g->c.tp_size >= kTpOverlapFromRanks);
    if (g->c.tp_size > 1 && g->ar && overlap && !g->taps_on && !g->fill_cache && B >= 2 && B % 2 == 0 && model_uses_fused(g, T))
        return forward_tp_pipelined(g, ids, B, T, logits, hr);
    const sptorch_gpt_config& c = g->c;
    const int d = c.d_model, M = B * T, dl = g->d_loc, Fl = g->F_loc;
    const int dt = c.dtype;
    const bool lead = c.tp_rank == 0;
    { ProfScope ps(PROF_EMBED); if (sptorch_ext_embedding_sum(g->tok, g->pos, ids, g->x, (size_t)M, (size_t)T, (size_t)c.vocab, (size_t)d, dt)) return 1; }
    void* x = g->x; void* y = g->y;
    auto tap = [&](int i, const void* src) -> int {
        if (!g->taps_on) return 0;
        SPT_CUDA(cudaMemcpyAsync(g->taps[i], src, (size_t)M * d * g->es, cudaMemcpyDeviceToDevice, rt().stream));
        return 0;
    };
    if (tap(0, x)) return 1;
    const bool fold = fold_applicable(g, M, T) && g->fold_ready && !g->fold_dirty;
    for (int l = 0; l < c.n_layer; l++) {
        const Layer& w = g->L[l];
        if (fold) {
            if (ln_stats(g, x, M)) return 1;
            if (attention_block(g, w, l, nullptr, g->qkv, g->ao, B, T, true, x)) return 1;
        } else {
            if (ln(x, w.ln1g, w.ln1b, g->h, (size_t)M, (size_t)d, c.eps, dt)) return 1;
            if (attention_block(g, w, l, g->h, g->qkv, g->ao, B, T, false, nullptr)) return 1;
        }
        if (c.tp_size <= 1) {
            if (linear(g, g->ao, w.wo, nullptr, x, x, M, dl, d, d, EPI_NONE)) return 1;       // x += attn
        } else {
            if (linear(g, g->ao, w.wo, nullptr, lead ? x : nullptr, y, M, dl, d, d, EPI_NONE)) return 1;
            if (allreduce(g, y, (size_t)M * d)) return 1;
            std::swap(x, y);
        }
        if (fold) {
            if (ln_stats(g, x, M)) return 1;
            if (linear_folded(g, x, w.w1_f, w.c_1, w.s_1, g->f, M, d, Fl, Fl, EPI_GELU)) return 1;
        } else {
            if (ln(x, w.ln2g, w.ln2b, g->h, (size_t)M, (size_t)d, c.eps, dt)) return 1;
            if (linear(g, g->h, w.w1, w.b1, nullptr, g->f, M, d, Fl, Fl, EPI_GELU)) return 1;
        }
        if (c.tp_size <= 1) {
            if (linear(g, g->f, w.w2, w.b2, x, x, M, Fl, d, d, EPI_NONE)) return 1;            // x += ffn
        } else {
            if (linear(g, g->f, w.w2, lead ? w.b2 : nullptr, lead ? x : nullptr, y, M, Fl, d, d, EPI_NONE)) return 1;
            if (allreduce(g, y, (size_t)M * d)) return 1;
            std::swap(x, y);
        }
        if (tap(l + 1, x)) return 1;
    }
    if (fold && !hr) {
        if (g->taps_on) {          // the tap of ln_f's output is the only reader of the normalised rows
            if (ln(x, g->lnfg, g->lnfb, g->h, (size_t)M, (size_t)d, c.eps, dt)) return 1;
            if (tap(c.n_layer + 1, g->h)) return 1;
        }
        if (ln_stats(g, x, M)) return 1;
        return linear_folded(g, x, g->head_f, g->c_h, g->s_h, logits, M, d, c.vocab, (long long)g->ldl, EPI_NONE);
    }
    if (ln(x, g->lnfg, g->lnfb, g->h, (size_t)M, (size_t)d, c.eps, dt)) return 1;
    if (tap(c.n_layer + 1, g->h)) return 1;
    return lm_head(g, g->h, M, logits, hr);
}

// GPT::named_parameters (nn/src/lib.rs:1382-1392) / QwenLikeGPT::named_parameters (:1483-1492) with the full (unsharded) shapes
struct ParamInfo { std::string name; std::vector<size_t> shape; };
std::vector<ParamInfo> gpt_param_table(void* gp) {
    const sptorch_gpt_config& c = ((Gpt*)gp)->c;
    const size_t d = c.d_model, V = c.vocab, S = c.seq_len, F = c.d_ff;
    const bool qwen = c.arch == SPT_ARCH_QWEN_LIKE;
    std::vector<ParamInfo> t;
    t.push_back({"token_emb.weight", {V, d}});
    if (!qwen) t.push_back({"pos_emb.weight", {S, d}});
    for (int l = 0; l < c.n_layer; l++) {
        const std::string p = "blocks." + std::to_string(l) + ".";
        if (qwen) t.push_back({p + "norm1.weight", {d}});
        else { t.push_back({p + "ln1.gamma", {d}}); t.push_back({p + "ln1.beta", {d}}); }
        for (const char* w : {"attn.wq.weight", "attn.wk.weight", "attn.wv.weight", "attn.wo.weight"}) t.push_back({p + w, {d, d}});
        if (qwen) t.push_back({p + "norm2.weight", {d}});
        else { t.push_back({p + "ln2.gamma", {d}}); t.push_back({p + "ln2.beta", {d}}); }
        t.push_back({p + "ffn_up.weight", {F, d}}); t.push_back({p + "ffn_up.bias", {F}});
        if (qwen) { t.push_back({p + "ffn_gate.weight", {F, d}}); t.push_back({p + "ffn_gate.bias", {F}}); }
        t.push_back({p + "ffn_down.weight", {d, F}}); t.push_back({p + "ffn_down.bias", {d}});
    }
    if (qwen) t.push_back({"norm_f.weight", {d}});
    else { t.push_back({"ln_f.gamma", {d}}); t.push_back({"ln_f.beta", {d}}); }
    t.push_back({"lm_head.weight", {V, d}});
    return t;
}

}  // namespace spt

using namespace spt;

extern "C" {

void* sptorch_ext_gpt_create(const sptorch_gpt_config* cfg) {
    if (enter()) return nullptr;
    if (!cfg) { fail("gpt_create: null config"); return nullptr; }
    sptorch_gpt_config c = *cfg;
    if (c.tp_size < 1) { c.tp_size = 1; c.tp_rank = 0; }
    if (c.vocab <= 0 || c.d_model <= 0 || c.n_layer < 0 || c.n_head <= 0 || c.d_ff <= 0 || c.seq_len <= 0 || c.max_batch <= 0) {
        fail("gpt_create: non-positive dimension"); return nullptr;
    }
    if (c.dtype != SPT_F32 && c.dtype != SPT_BF16) { fail("gpt_create: unknown dtype %d", c.dtype); return nullptr; }
    if (c.arch != SPT_ARCH_GPT && c.arch != SPT_ARCH_QWEN_LIKE) { fail("gpt_create: unknown architecture %d", c.arch); return nullptr; }
    if (c.arch == SPT_ARCH_QWEN_LIKE && !(c.rope_base > 0.0f)) c.rope_base = 10000.0f;
    if (c.d_model % c.n_head) { fail("gpt_create: d_model %% n_head != 0"); return nullptr; }
    if (c.n_head % c.tp_size || c.d_ff % c.tp_size || c.tp_rank < 0 || c.tp_rank >= c.tp_size) {
        fail("gpt_create: heads and d_ff must divide by tp_size"); return nullptr;
    }
    const int vec = c.dtype == SPT_BF16 ? 8 : 4;
    const int hd = c.d_model / c.n_head;
    if (c.d_model % vec || (c.d_ff / c.tp_size) % vec || hd % vec) { fail("gpt_create: d_model, d_ff/tp and head_dim must be multiples of %d", vec); return nullptr; }
    Gpt* g = new Gpt();
    g->c = c;
    g->es = c.dtype == SPT_BF16 ? 2 : 4;
    g->H_loc = c.n_head / c.tp_size;
    g->d_loc = g->H_loc * hd;
    g->F_loc = c.d_ff / c.tp_size;
    g->ldl = ((size_t)c.vocab + 63) / 64 * 64;
    const size_t es = g->es, d = c.d_model, V = c.vocab, S = c.seq_len, dl = g->d_loc, Fl = g->F_loc;
    const size_t Mmax = (size_t)c.max_batch * S;
    bool ok = true;
    auto A = [&](size_t bytes) { void* p = galloc(g, bytes); if (!p) ok = false; return p; };
    g->tok = A(V * d * es); g->pos = A(S * d * es); g->head = A(V * d * es);
    g->lnfg = (float*)A(d * 4); g->lnfb = (float*)A(d * 4);
    g->L.resize(c.n_layer);
    for (auto& w : g->L) {
        w.ln1g = (float*)A(d * 4); w.ln1b = (float*)A(d * 4); w.ln2g = (float*)A(d * 4); w.ln2b = (float*)A(d * 4);
        w.b1 = (float*)A(Fl * 4); w.b2 = (float*)A(d * 4);
        w.wqkv = A(3 * dl * d * es); w.wqk = w.wqkv; w.wv = w.wqkv ? (uint8_t*)w.wqkv + 2 * dl * d * es : nullptr; w.wo = A(d * dl * es); w.w1 = A(Fl * d * es); w.w2 = A(d * Fl * es);
        if (c.arch == SPT_ARCH_QWEN_LIKE) { w.wg = A(Fl * d * es); w.bg = (float*)A(Fl * 4); }
    }
    g->x = A(Mmax * d * es); g->y = A(Mmax * d * es); g->h = A(Mmax * d * es);
    g->qkv = A(Mmax * 3 * dl * es); g->ao = A(Mmax * dl * es); g->f = A(Mmax * Fl * es);
    if (!ok) { sptorch_ext_gpt_destroy(g); return nullptr; }
    return g;
}

void sptorch_ext_gpt_destroy(void* gp) {
    if (!gp) return;
    Gpt* g = (Gpt*)gp;
    if (!enter()) {
        cudaStreamSynchronize(rt().stream);
        cudaStreamSynchronize(rt().copy_stream);
        drop_graphs(g);
        for (void* p : g->owned) sptorch_free(p);
        for (int i = 0; i < 2; i++) {
            if (g->ev_compute[i]) cudaEventDestroy(g->ev_compute[i]);
            if (g->ev_copy[i]) cudaEventDestroy(g->ev_copy[i]);
            if (g->ev_partial[i]) cudaEventDestroy(g->ev_partial[i]);
            if (g->ev_reduced[i]) cudaEventDestroy(g->ev_reduced[i]);
        }
    }
    delete g;
}

int sptorch_ext_gpt_set_param(void* gp, const char* name, const float* host, size_t n) {
    if (enter()) return 1;
    if (!gp || !name || !host) return fail("gpt_set_param: null argument");
    Gpt* g = (Gpt*)gp;
    const sptorch_gpt_config& c = g->c;
    const size_t d = c.d_model, V = c.vocab, S = c.seq_len, F = c.d_ff, dl = g->d_loc, Fl = g->F_loc, es = g->es;
    auto need = [&](size_t want) { return n == want ? 0 : fail("gpt_set_param(%s): got %zu values, expected %zu", name, n, want); };
    auto f32 = [&](float* dst, size_t off, size_t cnt) { return sptorch_ext_copy_h2d_bytes(host + off, dst, cnt * 4) || stream_wait(); };
    std::string s(name);
    g->fold_dirty = true;                       // folded copies of the weights follow any parameter change
    const bool qwen = c.arch == SPT_ARCH_QWEN_LIKE;
    if (qwen && (s == "pos_emb.weight" || s == "ln_f.gamma" || s == "ln_f.beta")) return fail("gpt_set_param: '%s' is not a parameter of the Qwen-like model", name);
    if (qwen && s == "norm_f.weight") return need(d) || f32(g->lnfg, 0, d);
    if (s == "token_emb.weight") return need(V * d) || upload_rows(g, g->tok, host, n);
    if (s == "pos_emb.weight") return need(S * d) || upload_rows(g, g->pos, host, n);
    if (s == "lm_head.weight") return need(V * d) || upload_rows(g, g->head, host, n);
    if (s == "ln_f.gamma") return need(d) || f32(g->lnfg, 0, d);
    if (s == "ln_f.beta") return need(d) || f32(g->lnfb, 0, d);
    int li = -1; char rest[64] = "";
    if (sscanf(name, "blocks.%d.%63s", &li, rest) == 2 && li >= 0 && li < c.n_layer) {
        Layer& w = g->L[li];
        std::string t(rest);
        if (qwen) {
            // QwenLikeBlock::named_parameters (nn/src/lib.rs:1157-1166)
            if (t == "norm1.weight") return need(d) || f32(w.ln1g, 0, d);
            if (t == "norm2.weight") return need(d) || f32(w.ln2g, 0, d);
            if (t == "ffn_gate.weight") return need(F * d) || upload_shard(g, w.wg, name, host, F, d, false);
            if (t == "ffn_gate.bias") return need(F) || upload_shard(g, w.bg, name, host, F, 1, true);
            if (t.compare(0, 2, "ln") == 0) return fail("gpt_set_param: '%s' is not a parameter of the Qwen-like model", name);
        }
        if (t == "ln1.gamma") return need(d) || f32(w.ln1g, 0, d);
        if (t == "ln1.beta") return need(d) || f32(w.ln1b, 0, d);
        if (t == "ln2.gamma") return need(d) || f32(w.ln2g, 0, d);
        if (t == "ln2.beta") return need(d) || f32(w.ln2b, 0, d);
        // the shard of this rank (sptorch_ext_tp_param_shard): rows of wq / wk / wv / ffn_up, columns of wo / ffn_down
        if (t == "attn.wq.weight") return need(d * d) || upload_shard(g, w.wqkv, name, host, d, d, false);
        if (t == "attn.wk.weight") return need(d * d) || upload_shard(g, (uint8_t*)w.wqkv + dl * d * es, name, host, d, d, false);
        if (t == "attn.wv.weight") return need(d * d) || upload_shard(g, (uint8_t*)w.wqkv + 2 * dl * d * es, name, host, d, d, false);
        if (t == "attn.wo.weight") return need(d * d) || upload_shard(g, w.wo, name, host, d, d, false);
        if (t == "ffn_up.weight") return need(F * d) || upload_shard(g, w.w1, name, host, F, d, false);
        if (t == "ffn_up.bias") return need(F) || upload_shard(g, w.b1, name, host, F, 1, true);
        if (t == "ffn_down.weight") return need(d * F) || upload_shard(g, w.w2, name, host, d, F, false);
        if (t == "ffn_down.bias") return need(d) || f32(w.b2, 0, d);
    }
    return fail("gpt_set_param: unknown parameter name '%s'", name);
}

size_t sptorch_ext_gpt_logits_ld(void* gp) { return gp ? ((Gpt*)gp)->ldl : 0; }

static int check_shape(Gpt* g, int batch, int T) {
    if (batch <= 0 || T <= 0) return fail("gpt_forward: empty batch or sequence");
    if (T > g->c.seq_len) return fail("gpt_forward: T=%d exceeds seq_len=%d", T, g->c.seq_len);   // nn/src/lib.rs:1351 asserts the same
    if ((size_t)batch * T > (size_t)g->c.max_batch * g->c.seq_len) return fail("gpt_forward: batch*T exceeds the activation capacity");
    if (ensure_scores(g, batch, T)) return 1;      // outside any graph capture
    const int vec = 16 / g->es;
    if (T % vec) return fail("gpt_forward: T must be a multiple of %d for this dtype", vec);
    return 0;
}

// One forward, replayed as a CUDA graph when it repeats.  The launch-bound inner loop (about 90 kernels, each a few microseconds
// when the batch is sharded 8 ways) is captured once per key: the first forward of a given key runs eagerly (it also sets function
// attributes), the second is captured, later ones are a single cudaGraphLaunch.  Per-kernel timing and tensor-parallel hooks run
// eagerly.  The key holds everything that is baked into the captured kernel arguments.
static int forward_graphed(Gpt* g, const void* ids, int batch, int T, void* logits, const HeadReduce* hr) {
    const bool graph_ok = g->graphs && !prof_enabled() && g->c.tp_size <= 1;
    if (!graph_ok) return forward(g, ids, batch, T, logits, hr);
    Gpt::GraphKey key = {ids, logits, batch, T, g->taps_on, rt().stream, config_epoch(),
                         hr ? (const void*)hr->targets : nullptr, hr ? (const void*)hr->argmax : nullptr, hr ? (const void*)hr->row_loss : nullptr,
                         hr ? hr->has_ignore : 0, hr ? hr->ignore_index : 0, hr != nullptr};
    Gpt::GraphSlot* slot = nullptr;
    for (auto& sl : g->gslots) if ((sl.exec || sl.eager_runs) && sl.key == key) slot = &sl;
    if (!slot) {                                   // least recently used slot takes the new key
        slot = &g->gslots[0];
        for (auto& sl : g->gslots) if (sl.last_use < slot->last_use) slot = &sl;
        if (slot->exec) { cudaGraphExecDestroy(slot->exec); slot->exec = nullptr; }
        slot->key = key; slot->eager_runs = 0;
    }
    slot->last_use = ++g->guse;
    if (slot->exec) {
        SPT_CUDA(cudaGraphLaunch(slot->exec, rt().stream));
        note_submit();
        return 0;
    }
    if (slot->eager_runs++ == 0) return forward(g, ids, batch, T, logits, hr);
    cudaGraph_t graph = nullptr;
    SPT_CUDA(cudaStreamBeginCapture(rt().stream, cudaStreamCaptureModeThreadLocal));
    int rc = forward(g, ids, batch, T, logits, hr);
    cudaError_t e = cudaStreamEndCapture(rt().stream, &graph);
    if (rc != 0 || e != cudaSuccess || !graph) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        g->graphs = false;                                   // capture is not possible here: stay eager from now on
        if (rc != 0) return rc;
        return forward(g, ids, batch, T, logits, hr);
    }
    e = cudaGraphInstantiate(&slot->exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) { slot->exec = nullptr; g->graphs = false; cudaGetLastError(); return forward(g, ids, batch, T, logits, hr); }
    SPT_CUDA(cudaGraphLaunch(slot->exec, rt().stream));
    note_submit();
    return 0;
}

int sptorch_ext_gpt_forward(void* gp, const void* ids, int batch, int T, void* logits) {
    if (enter()) return 1;
    if (!gp || !ids || !logits) return fail("gpt_forward: null argument");
    Gpt* g = (Gpt*)gp;
    if (check_shape(g, batch, T)) return 1;
    if (fold_applicable(g, batch * T, T) && fold_prepare(g)) return 1;      // outside any graph capture
    return forward_graphed(g, ids, batch, T, logits, nullptr);
}

static int check_reduce(Gpt* g, const char* who) {
    if (g->c.vocab <= 128) return fail("%s: the fused LM head needs a vocabulary larger than 128", who);
    if (g->c.tp_size > 1) return fail("%s: not available with tensor parallel shards", who);
    return 0;
}

// Forward + the step after it without the logits: the LM head's epilogue reduces every 128 x 256 tile of logits to per-row partial
// (max, sum exp, first argmax, target logit) and a second small kernel merges them.  Same values as the unfused path: the logits
// are rounded to the model dtype before they are reduced.
int sptorch_ext_gpt_forward_loss(void* gp, const void* ids, const void* targets_i64, int batch, int T, int has_ignore, long long ignore_index,
                                 void* argmax_i32, void* row_loss_f32, float* host_mean) {
    if (enter()) return 1;
    if (host_mean) *host_mean = 0.0f;
    if (!gp || !ids) return fail("gpt_forward_loss: null argument");
    if (!argmax_i32 && !row_loss_f32) return fail("gpt_forward_loss: neither the greedy tokens nor the loss were asked for");
    if (row_loss_f32 && !targets_i64) return fail("gpt_forward_loss: a loss needs targets");
    Gpt* g = (Gpt*)gp;
    if (check_reduce(g, "gpt_forward_loss") || check_shape(g, batch, T)) return 1;
    if (ensure_reduce(g, (size_t)batch * T)) return 1;
    HeadReduce hr = {(const long long*)targets_i64, has_ignore, ignore_index, (int*)argmax_i32, (float*)row_loss_f32};
    if (forward_graphed(g, ids, batch, T, nullptr, &hr)) return 1;
    if (row_loss_f32) {
        if (cross_entropy_mean_launch((float*)row_loss_f32, (size_t)batch * T)) return 1;
        if (host_mean) return sptorch_ext_copy_d2h_bytes((float*)row_loss_f32 + (size_t)batch * T, host_mean, sizeof(float));
    }
    return 0;
}

// The same through host buffers: ids (and targets) in, greedy tokens and the mean loss out; the only device-to-host traffic is 4
// bytes per token.  Micro-batches of `chunk` sequences as in sptorch_ext_gpt_forward_host.
int sptorch_ext_gpt_forward_loss_host(void* gp, const int32_t* ids_host, const int64_t* targets_host, int batch, int T, int has_ignore,
                                      long long ignore_index, int32_t* argmax_host, float* host_mean, int chunk) {
    if (enter()) return 1;
    if (host_mean) *host_mean = 0.0f;
    if (!gp || !ids_host) return fail("gpt_forward_loss_host: null argument");
    if (!argmax_host && !targets_host) return fail("gpt_forward_loss_host: neither the greedy tokens nor the loss were asked for");
    if (targets_host && !host_mean) return fail("gpt_forward_loss_host: null result pointer for the loss");
    Gpt* g = (Gpt*)gp;
    if (chunk <= 0 || chunk > batch) chunk = batch;
    if (chunk > g->c.max_batch) chunk = g->c.max_batch;
    if (check_reduce(g, "gpt_forward_loss_host") || check_shape(g, chunk, T)) return 1;
    if (ensure_reduce(g, (size_t)chunk * T)) return 1;
    const size_t n = (size_t)batch * T;
    if (g->loss_cap < n) {
        if (g->loss_cap && stream_wait()) return 1;
        gfree(g, g->loss_targets); gfree(g, g->loss_argmax); gfree(g, g->loss_rows);
        g->loss_targets = (long long*)galloc(g, n * sizeof(long long));
        g->loss_argmax = (int*)galloc(g, n * sizeof(int));
        g->loss_rows = (float*)galloc(g, (n + 1) * sizeof(float));
        g->loss_cap = (g->loss_targets && g->loss_argmax && g->loss_rows) ? n : 0;
        if (!g->loss_cap) return 1;
    }
    if (g->ids_cap < batch * T) {
        if (g->ids_cap && stream_wait()) return 1;
        gfree(g, g->ids_dev);
        g->ids_dev = (int*)galloc(g, n * 4);
        if (!g->ids_dev) return 1;
        g->ids_cap = batch * T;
    }
    cudaStream_t cs = rt().stream;
    SPT_CUDA(cudaMemcpyAsync(g->ids_dev, ids_host, n * 4, cudaMemcpyHostToDevice, cs));
    if (targets_host) SPT_CUDA(cudaMemcpyAsync(g->loss_targets, targets_host, n * sizeof(long long), cudaMemcpyHostToDevice, cs));
    for (int b0 = 0; b0 < batch; b0 += chunk) {
        const int nb = batch - b0 < chunk ? batch - b0 : chunk;
        const size_t off = (size_t)b0 * T;
        HeadReduce hr = {targets_host ? g->loss_targets + off : nullptr, has_ignore, ignore_index, argmax_host ? g->loss_argmax + off : nullptr,
                         targets_host ? g->loss_rows + off : nullptr};
        if (forward_graphed(g, g->ids_dev + off, nb, T, nullptr, &hr)) return 1;
    }
    if (targets_host && cross_entropy_mean_launch(g->loss_rows, n)) return 1;
    if (argmax_host) SPT_CUDA(cudaMemcpyAsync(argmax_host, g->loss_argmax, n * sizeof(int), cudaMemcpyDeviceToHost, cs));
    if (targets_host) SPT_CUDA(cudaMemcpyAsync(host_mean, g->loss_rows + n, sizeof(float), cudaMemcpyDeviceToHost, cs));
    SPT_CUDA(cudaStreamSynchronize(cs));
    rt().retired.store(rt().submitted.load());
    return 0;
}

// ---- incremental decode (crates/nn/src/lib.rs:1540-1573 prefill_kv_cache / append_last_token_kv_cache,
// :1619-1646 decode_logits_from_cache, :706-760 causal_attention_last_token, :1205-1214 forward_last_token_incremental) ----
int sptorch_ext_gpt_enable_kv_cache(void* gp, int max_context) {
    if (enter()) return 1;
    if (!gp) return fail("gpt_enable_kv_cache: null model");
    Gpt* g = (Gpt*)gp;
    if (g->c.tp_size > 1) return fail("gpt_enable_kv_cache: not available with tensor parallel shards");
    if (max_context <= 0 || max_context > g->c.seq_len) max_context = g->c.seq_len;     // learned positions end at seq_len; forward_ids asserts it for both models
    if (g->kcache) return max_context == g->cache_ctx ? 0 : fail("gpt_enable_kv_cache: cache already allocated with %d positions", g->cache_ctx);
    const size_t bytes = (size_t)g->c.n_layer * g->c.max_batch * max_context * g->d_loc * g->es;
    g->kcache = galloc(g, bytes); g->vcache = galloc(g, bytes);
    g->dq = galloc(g, (size_t)g->c.max_batch * 3 * g->d_loc * g->es);
    g->dstate = (int*)galloc(g, 256);
    if (!g->kcache || !g->vcache || !g->dq || !g->dstate) return 1;
    g->cache_ctx = max_context; g->cached_len = 0; g->cache_batch = 0; g->window_start = 0;
    return 0;
}

int sptorch_ext_gpt_cached_len(void* gp) { return gp ? ((Gpt*)gp)->cached_len : 0; }
long long sptorch_ext_gpt_window_start(void* gp) { return gp ? ((Gpt*)gp)->window_start : 0; }

// prefill: the ordinary forward over ids [batch, T], which also fills the cache with K and V of all T positions.
// logits may be NULL (then an internal scratch of the activations is NOT available: pass a buffer if logits are wanted).
int sptorch_ext_gpt_prefill(void* gp, const void* ids, int batch, int T, void* logits) {
    if (enter()) return 1;
    if (!gp || !ids || !logits) return fail("gpt_prefill: null argument");
    Gpt* g = (Gpt*)gp;
    if (!g->kcache) return fail("gpt_prefill: call sptorch_ext_gpt_enable_kv_cache first");
    if (check_shape(g, batch, T)) return 1;
    if (T > g->cache_ctx) return fail("gpt_prefill: T=%d exceeds the cache of %d positions", T, g->cache_ctx);
    g->fill_cache = true;
    int rc = forward(g, ids, batch, T, logits);
    g->fill_cache = false;
    if (rc) return rc;
    g->cached_len = T; g->cache_batch = batch; g->window_start = 0;
    return 0;
}

// One incremental step for `batch` sequences that share a cached length.
//   append = 1: last_ids are NEW tokens: their K,V are appended at position cached_len, the logits are those of the new token
//               (append_last_token_kv_cache followed by decode_logits_from_cache);
//   append = 0: last_ids are the tokens already at position cached_len-1: nothing is written, the logits of that last
//               cached token are recomputed from the cache (decode_logits_from_cache right after a prefill).
// logits: [batch, ld] in the model dtype, ld = sptorch_ext_gpt_logits_ld.
// The launches of one decode step.  Everything that changes from step to step -- the token's position, the number of valid cached
// positions, the ring slot, the row of the position table -- is read by the kernels from the device words `g->dstate`, so the same
// sequence of launches serves every step and can be replayed as a CUDA graph.
// One projection of a decode step: out = act(norm(x) W^T + bias) (+ or * res).  With at most 64 sequences in bf16 it is one launch
// of the weight-streaming kernel (linear_few_rows.cu) with the normalisation applied to the rows on the fly, started as a
// programmatic dependent of the kernel before it; otherwise the stand-alone normalisation into g->h and the tcgen05 GEMM.
static int decode_linear(Gpt* g, const void* x, const RowNorm* nrm, const void* w, const float* bias, const void* res, void* out, int B, int K, int N,
                         long long ldo, int epi) {
    const sptorch_gpt_config& c = g->c;
    if (c.dtype == SPT_BF16) {
        GemmDesc d;
        d.A = x; d.B = w; d.C = out; d.bias = bias; d.R = res;
        d.M = B; d.N = N; d.K = K; d.lda = K; d.ldb = K; d.ldc = ldo;
        d.epilogue = epi; d.mode = MM_BF16; d.out_dtype = BF16;
        if (linear_few_rows_supported(d) && (!nrm || linear_few_rows_norm_supported(d, *nrm))) {
            ProfScope ps(PROF_LINEAR);
            return linear_few_rows(d, nrm, true);
        }
    }
    const void* a = x;
    if (nrm) {
        if (c.dtype == SPT_BF16 && norm_few_rows_supported(x, g->h, B, K, *nrm)) {
            ProfScope ps(PROF_LAYERNORM);
            if (norm_few_rows(x, g->h, B, K, *nrm, true)) return 1;
        } else if (nrm->kind == 2 ? rms_launch(x, nrm->gamma, g->h, (size_t)B, (size_t)K, nrm->eps, c.dtype)
                                  : ln(x, nrm->gamma, nrm->beta, g->h, (size_t)B, (size_t)K, nrm->eps, c.dtype)) return 1;
        a = g->h;
    }
    if (c.dtype == SPT_BF16) {
        GemmDesc d;
        d.A = a; d.B = w; d.C = out; d.bias = bias; d.R = res;
        d.M = B; d.N = N; d.K = K; d.lda = K; d.ldb = K; d.ldc = ldo;
        d.epilogue = epi; d.mode = MM_BF16; d.out_dtype = BF16;
        if (linear_few_rows_supported(d)) { ProfScope ps(PROF_LINEAR); return linear_few_rows(d, nullptr, true); }
    }
    return linear(g, a, w, bias, res, out, B, K, N, ldo, epi);
}

static int decode_launches(Gpt* g, const void* last_ids, int B, int append, void* logits) {
    const sptorch_gpt_config& c = g->c;
    const int d = c.d_model, dl = g->d_loc, Fl = g->F_loc, hd = d / c.n_head, dt = c.dtype;
    const size_t es = g->es;
    const bool qwen = c.arch == SPT_ARCH_QWEN_LIKE;     // QwenLikeBlock::forward_last_token_incremental, nn/src/lib.rs:1119-1131
    const int* st = g->dstate;
    auto norm_of = [&](const float* gamma, const float* beta) {
        RowNorm n; n.kind = qwen ? 2 : 1; n.gamma = gamma; n.beta = qwen ? nullptr : beta; n.eps = c.eps; return n;
    };
    { ProfScope ps(PROF_EMBED);
      if (embedding_sum_launch(g->tok, qwen ? nullptr : g->pos, last_ids, g->x, (size_t)B, 1, (size_t)c.vocab, (size_t)d, dt, st + 3)) return 1; }
    void* x = g->x;
    const long long row = dl, seq = (long long)g->cache_ctx * dl;
    const bool fresh = append && attention_last_token_takes_fresh(hd, dt);     // the attention kernel appends the token's key / value itself
    for (int l = 0; l < c.n_layer; l++) {
        const Layer& w = g->L[l];
        const size_t lay = (size_t)l * c.max_batch * g->cache_ctx * dl * es;
        uint8_t* kc = (uint8_t*)g->kcache + lay;
        uint8_t* vc = (uint8_t*)g->vcache + lay;
        const RowNorm n1 = norm_of(w.ln1g, w.ln1b), n2 = norm_of(w.ln2g, w.ln2b);
        if (decode_linear(g, x, &n1, w.wqkv, nullptr, nullptr, g->dq, B, d, 3 * dl, 3 * dl, EPI_NONE)) return 1;     // [q | k | v] of the token
        // the query (and the key about to be cached) are rotated to the token's absolute position (nn/src/lib.rs:718-721, 678-680)
        if (qwen) { ProfScope ps(PROF_OTHER); if (rope_launch(g->dq, B, 1, 2 * g->H_loc, hd, 3 * dl, c.rope_base, 0, dt, st + 0)) return 1; }
        if (append && !fresh) { ProfScope ps(PROF_OTHER); if (kv_append_launch(g->dq, kc, vc, B, dl, seq, 0, st, dt)) return 1; }      // one cache row per sequence and layer
        { ProfScope ps(PROF_ATTN_FUSED);
          const uint8_t* dq = (const uint8_t*)g->dq;
          if (attention_last_token(g->dq, 3 * dl, kc, vc, g->ao, dl, B, g->H_loc, hd, g->cache_ctx, seq, row, dt, st, g->cache_ctx,
                                   fresh ? dq + (size_t)dl * es : nullptr, fresh ? dq + (size_t)2 * dl * es : nullptr, 3 * dl, 0, true)) return 1; }
        if (decode_linear(g, g->ao, nullptr, w.wo, nullptr, x, x, B, dl, d, d, EPI_NONE)) return 1;
        if (qwen) {
            if (decode_linear(g, x, &n2, w.w1, w.b1, nullptr, g->f, B, d, Fl, Fl, EPI_NONE)) return 1;
            if (decode_linear(g, x, &n2, w.wg, w.bg, g->f, g->f, B, d, Fl, Fl, EPI_SWIGLU)) return 1;
        } else if (decode_linear(g, x, &n2, w.w1, w.b1, nullptr, g->f, B, d, Fl, Fl, EPI_GELU)) return 1;
        if (decode_linear(g, g->f, nullptr, w.w2, w.b2, x, x, B, Fl, d, d, EPI_NONE)) return 1;
    }
    const RowNorm nf = norm_of(g->lnfg, g->lnfb);
    return decode_linear(g, x, &nf, g->head, nullptr, nullptr, logits, B, d, c.vocab, (long long)g->ldl, EPI_NONE);
}

int sptorch_ext_gpt_decode(void* gp, const void* last_ids, int batch, int append, void* logits) {
    if (enter()) return 1;
    if (!gp || !last_ids || !logits) return fail("gpt_decode: null argument");
    Gpt* g = (Gpt*)gp;
    const sptorch_gpt_config& c = g->c;
    if (!g->kcache || g->cached_len <= 0) return fail("gpt_decode: the cache is empty (prefill first)");
    if (batch != g->cache_batch) return fail("gpt_decode: batch %d differs from the cached batch %d", batch, g->cache_batch);
    // The cache is a ring over absolute positions (slot = position % capacity): once it is full an appended token takes the slot
    // of the oldest one, which is how append_kv_tensor (nn/src/lib.rs:2165-2203) keeps the last max_context positions; the window
    // start then moves on by one (KvCacheWindowState::append, hal/src/lib.rs:129-239).  The attention reads the n valid slots;
    // their order in memory does not matter to a softmax-weighted sum.
    const bool full = g->cached_len >= g->cache_ctx;
    const long long apos = append ? g->window_start + g->cached_len : g->window_start + g->cached_len - 1;   // absolute position of the token
    if (apos > INT32_MAX) return fail("gpt_decode: position overflow");
    const int pos = (int)apos;
    const int slot = (int)(apos % g->cache_ctx);
    const int n = append ? (full ? g->cache_ctx : g->cached_len + 1) : g->cached_len;
    const int pos_row = pos < c.seq_len - 1 ? pos : c.seq_len - 1;            // last_pos.min(seq_len - 1), nn/src/lib.rs:1631
    if (decode_state_launch(g->dstate, pos, n, slot, pos_row)) return 1;      // by value: nothing of the host's is read later
    // Replay: a decode step is about a hundred small launches, host-bound when issued one by one.  The first step of a key runs
    // eagerly, the second is captured, later ones are one cudaGraphLaunch.
    Gpt::DecodeKey key = {last_ids, logits, batch, append, rt().stream, config_epoch()};
    const bool graph_ok = g->graphs && !prof_enabled();
    int rc;
    if (!graph_ok) rc = decode_launches(g, last_ids, batch, append, logits);
    else {
        if (!(g->dkey == key)) {
            if (g->dexec) { cudaGraphExecDestroy(g->dexec); g->dexec = nullptr; }
            g->dkey = key; g->d_eager = 0;
        }
        if (g->dexec) { SPT_CUDA(cudaGraphLaunch(g->dexec, rt().stream)); note_submit(); rc = 0; }
        else if (g->d_eager++ == 0) rc = decode_launches(g, last_ids, batch, append, logits);
        else {
            cudaGraph_t graph = nullptr;
            SPT_CUDA(cudaStreamBeginCapture(rt().stream, cudaStreamCaptureModeThreadLocal));
            rc = decode_launches(g, last_ids, batch, append, logits);
            cudaError_t e = cudaStreamEndCapture(rt().stream, &graph);
            if (rc == 0 && e == cudaSuccess && graph && cudaGraphInstantiate(&g->dexec, graph, 0) == cudaSuccess) {
                cudaGraphDestroy(graph);
                SPT_CUDA(cudaGraphLaunch(g->dexec, rt().stream));
                note_submit();
            } else {
                if (graph) cudaGraphDestroy(graph);
                cudaGetLastError();
                g->dexec = nullptr; g->graphs = false;                       // capture is not possible here: stay eager from now on
                if (rc == 0) rc = decode_launches(g, last_ids, batch, append, logits);
            }
        }
    }
    if (rc) return rc;
    if (append) { if (full) g->window_start++; else g->cached_len++; }
    return 0;
}

int sptorch_ext_gpt_enable_ln_fold(void* gp, int on) {
    if (!gp) return fail("gpt_enable_ln_fold: null model");
    Gpt* g = (Gpt*)gp;
    if (g->ln_fold != (on != 0)) {
        g->ln_fold = on != 0;
        drop_graphs(g);                          // the captured launches belong to the other path
    }
    return 0;
}

int sptorch_ext_gpt_enable_tp_overlap(void* gp, int on) {
    if (!gp) return fail("gpt_enable_tp_overlap: null model");
    if (on < 0 || on > 2) return fail("gpt_enable_tp_overlap: mode %d (0 never, 1 always, 2 from four ranks up)", on);
    ((Gpt*)gp)->tp_overlap = on;
    drop_graphs((Gpt*)gp);
    return 0;
}

int sptorch_ext_gpt_enable_graphs(void* gp, int on) {
    if (!gp) return fail("gpt_enable_graphs: null model");
    Gpt* g = (Gpt*)gp;
    g->graphs = on != 0;
    if (!on) drop_graphs(g);
    return 0;
}

int sptorch_ext_gpt_enable_taps(void* gp, int on) {
    if (enter()) return 1;
    if (!gp) return fail("gpt_enable_taps: null model");
    Gpt* g = (Gpt*)gp;
    if (on && g->taps.empty()) {
        size_t bytes = (size_t)g->c.max_batch * g->c.seq_len * g->c.d_model * g->es;
        for (int i = 0; i < g->c.n_layer + 2; i++) {
            void* p = galloc(g, bytes);
            if (!p) return 1;
            g->taps.push_back(p);
        }
    }
    g->taps_on = on != 0;
    return 0;
}

const void* sptorch_ext_gpt_tap(void* gp, int i) {
    Gpt* g = (Gpt*)gp;
    if (!g || i < 0 || i >= (int)g->taps.size()) return nullptr;
    return g->taps[i];
}

int sptorch_ext_gpt_set_allreduce(void* gp, sptorch_allreduce_fn fn, void* user) {
    if (!gp) return fail("gpt_set_allreduce: null model");
    ((Gpt*)gp)->ar = fn; ((Gpt*)gp)->ar_user = user;
    return 0;
}

int sptorch_ext_gpt_launches(void* gp, int batch, int T) {
    if (!gp) return 0;
    Gpt* g = (Gpt*)gp;
    (void)batch;
    const bool fused = model_uses_fused(g, T);
    // embedding + per layer (LN1, QKV, attention [1 fused | V^T, S, softmax, PV], Wo, LN2, up, down) + ln_f + head;
    // the Qwen-like block adds the RoPE pass and the gate projection
    return 1 + g->c.n_layer * ((fused ? 7 : 10) + (g->c.arch == SPT_ARCH_QWEN_LIKE ? 2 : 0)) + 2;
}

int sptorch_ext_gpt_forward_host(void* gp, const int32_t* ids_host, int batch, int T, void* logits_host, int chunk) {
    if (enter()) return 1;
    if (!gp || !ids_host || !logits_host) return fail("gpt_forward_host: null argument");
    Gpt* g = (Gpt*)gp;
    if (chunk <= 0 || chunk > batch) chunk = batch;
    if (chunk > g->c.max_batch) chunk = g->c.max_batch;
    if (check_shape(g, chunk, T)) return 1;
    if (fold_applicable(g, chunk * T, T) && fold_prepare(g)) return 1;
    const size_t es = g->es, V = g->c.vocab, ldl = g->ldl;
    // per slot: the padded logits the head GEMM writes ([rows, ldl]: TMA stores need a 16-byte row pitch) and the dense
    // [rows, V] copy of them that leaves the device (a strided 2-D device-to-host copy of 100 514-byte rows ran far below the
    // link's rate when several GPUs copied at once; one contiguous copy per chunk does not)
    const size_t need_padded = ((size_t)chunk * T * ldl * es + 255) / 256 * 256;
    const size_t need_logits = need_padded + ((size_t)chunk * T * V * es + 255) / 256 * 256;
    if (g->logits_cap < need_logits) {
        if (g->logits_cap) { SPT_CUDA(cudaStreamSynchronize(rt().copy_stream)); if (stream_wait()) return 1; }
        for (int i = 0; i < 2; i++) {
            gfree(g, g->logits_dev[i]);
            g->logits_dev[i] = galloc(g, need_logits);
            if (!g->logits_dev[i]) return 1;
        }
        g->logits_cap = need_logits;
    }
    if (g->ids_cap < batch * T) {
        if (g->ids_cap && stream_wait()) return 1;
        gfree(g, g->ids_dev);
        g->ids_dev = (int*)galloc(g, (size_t)batch * T * 4);
        if (!g->ids_dev) return 1;
        g->ids_cap = batch * T;
    }
    for (int i = 0; i < 2; i++) {
        if (!g->ev_compute[i]) SPT_CUDA(cudaEventCreateWithFlags(&g->ev_compute[i], cudaEventDisableTiming));
        if (!g->ev_copy[i]) SPT_CUDA(cudaEventCreateWithFlags(&g->ev_copy[i], cudaEventDisableTiming));
    }
    cudaStream_t cs = rt().stream, ds = rt().copy_stream;
    SPT_CUDA(cudaMemcpyAsync(g->ids_dev, ids_host, (size_t)batch * T * 4, cudaMemcpyHostToDevice, cs));
    int slot = 0, issued = 0;
    for (int b0 = 0; b0 < batch; b0 += chunk, slot ^= 1, issued++) {
        int nb = batch - b0 < chunk ? batch - b0 : chunk;
        if (issued >= 2) SPT_CUDA(cudaStreamWaitEvent(cs, g->ev_copy[slot], 0));      // buffer free again
        void* padded = g->logits_dev[slot];
        void* dense = (uint8_t*)g->logits_dev[slot] + need_padded;
        if (forward(g, g->ids_dev + (size_t)b0 * T, nb, T, padded)) return 1;
        if (ldl != V) { ProfScope ps(PROF_OTHER); if (compact_rows_launch(padded, dense, (size_t)nb * T, V, ldl, (int)es)) return 1; }
        else dense = padded;
        SPT_CUDA(cudaEventRecord(g->ev_compute[slot], cs));
        SPT_CUDA(cudaStreamWaitEvent(ds, g->ev_compute[slot], 0));
        SPT_CUDA(cudaMemcpyAsync((uint8_t*)logits_host + (size_t)b0 * T * V * es, dense, (size_t)nb * T * V * es, cudaMemcpyDeviceToHost, ds));
        SPT_CUDA(cudaEventRecord(g->ev_copy[slot], ds));
    }
    SPT_CUDA(cudaStreamSynchronize(ds));
    SPT_CUDA(cudaStreamSynchronize(cs));
    rt().retired.store(rt().submitted.load());
    return 0;
}

}  // extern "C"
