/*
 * sptorch_b200_ext.h -- additive entry points of libsptorch_b200.so.
 *
 * The 20 symbols of sptorch_b200_hal.h are what sptorch's loader binds today.  They cover
 * only 11 of the kernels that the forward pass of nn::GPT needs, and every one of them is
 * reached through host slices.  The functions below make a device-resident forward possible
 * behind the same library: the remaining KernelProvider kernels (crates/hal/src/lib.rs:374-458),
 * the nn-level ops that the reference computes inline on the host (LayerNorm, Linear, causal
 * attention, the embedding sum) and the whole GPT forward.  Same conventions as the base ABI:
 * int 0 = success, device handles are device addresses, sizes count elements, all work is
 * enqueued on the library's stream, no function allocates behind the caller's back unless it
 * says so.
 */
#ifndef SPTORCH_B200_EXT_H
#define SPTORCH_B200_EXT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* storage types of activations / weights */
#define SPT_F32  0
#define SPT_BF16 1

/* arithmetic of a contraction (accumulation is always f32) */
#define SPT_MM_TF32 0   /* f32 operands, tensor cores read them as TF32          */
#define SPT_MM_BF16 1   /* bf16 operands                                          */
#define SPT_MM_F32  2   /* f32 operands, f32 FMA on the CUDA cores (exact-order)  */

/* epilogue of sptorch_ext_linear: out = act(alpha * x W^T + bias) + residual */
#define SPT_EPI_NONE 0
#define SPT_EPI_GELU 1
#define SPT_EPI_SWIGLU 2   /* out = residual * g * sigmoid(g), g = alpha x W^T + bias: swiglu(x, gate) of core-ops/src/lib.rs:1529-1541 with the gate projection fused */

/* ---- runtime ---- */
const char* sptorch_ext_last_error(void);              /* text of the calling thread's last failure */
int   sptorch_ext_device(void);                        /* CUDA ordinal in use, -1 before init */
int   sptorch_ext_sm_count(void);
int   sptorch_ext_set_stream(void* cuda_stream);       /* adopt a caller's stream; NULL = library's own */
void* sptorch_ext_alloc_bytes(size_t bytes);           /* stream-ordered pool, 256-byte aligned */
void* sptorch_ext_alloc_pinned(size_t bytes);          /* page-locked host memory */
void  sptorch_ext_free_pinned(void* p);
int   sptorch_ext_copy_h2d_bytes(const void* host, void* device, size_t bytes);   /* async if host is pinned */
int   sptorch_ext_copy_d2h_bytes(const void* device, void* host, size_t bytes);   /* returns with host valid */
int   sptorch_ext_memset(void* device, int byte, size_t bytes);
int   sptorch_ext_set_alloc_budget(size_t bytes);      /* tests: allocations beyond this many live bytes fail; 0 = off */
/* persistent GEMM / attention kernels launch on (SM count - n) SMs, leaving room for a collective on another stream */
int   sptorch_ext_set_sm_reserve(int n);
int   sptorch_ext_timer_begin(void);                   /* CUDA event on the library stream */
int   sptorch_ext_timer_end(float* ms);                /* second event, waits for it, elapsed ms */
int   sptorch_ext_flush_l2(void);                      /* overwrites a 256 MiB scratch (allocated on first use) */
/* per-category device timing of the GPT forward (CUDA events around each launch on the library stream).
 * categories: 0 linear GEMM, 1 attention GEMMs, 2 causal softmax, 3 layernorm, 4 embedding, 5 other, 6 fused attention */
#define SPT_PROF_NCAT 7
int   sptorch_ext_prof_enable(int on);
int   sptorch_ext_prof_read(float* ms, uint32_t* launches, int ncat);  /* syncs, sums since last read, clears */
uint32_t sptorch_ext_device_status(void);              /* non-zero if a kernel's bounded wait ran out (sticky until sync) */

/* ---- dtype conversion ---- */
int sptorch_ext_f32_to_bf16(const void* in, void* out, size_t n);   /* round to nearest even */
int sptorch_ext_bf16_to_f32(const void* in, void* out, size_t n);

/* ---- rest of KernelProvider (crates/hal/src/lib.rs:430-457; reference kernels :578-646) ---- */
int sptorch_ext_sum_f32(const void* a, size_t n, float* host_result);
int sptorch_ext_masked_fill_f32(const void* a, const void* mask_u8, float fill, void* out, size_t n); /* mask!=0 -> fill */
int sptorch_ext_broadcast_add_f32(const void* a, const void* b, void* out, size_t a_len, size_t b_len); /* b[i % b_len] */
int sptorch_ext_embedding_lookup_f32(const void* weight, const void* idx_i64, void* out,
                                     size_t n_idx, size_t vocab, size_t dim);  /* ids validated on device: bad id -> error at sync, row zeroed */
int sptorch_ext_sgd_update_f32(void* params, const void* grad, float lr, size_t n);
int sptorch_ext_adam_update_f32(void* params, const void* grad, void* m, void* v, size_t n, float lr,
                                float beta1, float beta2, float eps, float weight_decay, float bc1, float bc2);

/* ---- core-ops / nn row kernels; dtype = SPT_F32 | SPT_BF16 for input and output alike ---- */
int sptorch_ext_add(const void* a, const void* b, void* out, size_t n, int dtype);          /* core-ops/src/lib.rs:299 */
int sptorch_ext_gelu(const void* a, void* out, size_t n, int dtype);                        /* core-ops/src/lib.rs:1331 */
int sptorch_ext_transpose_f32(const void* a, void* out, size_t rows, size_t cols);          /* core-ops/src/lib.rs:825 */
int sptorch_ext_layernorm(const void* x, const void* gamma_f32, const void* beta_f32, void* out,
                          size_t rows, size_t dim, float eps, int dtype);                   /* nn/src/lib.rs:397-418 */
/* scale -> masked_fill(j>i, -inf) -> row softmax over scores [batch, T, T]  (nn/src/lib.rs:612-632) */
int sptorch_ext_causal_softmax(const void* scores, void* out, size_t batch, size_t T, float scale, int dtype);
/* core-ops masked_softmax (core-ops/src/lib.rs:1601-1645): keep!=0 takes part, others give exactly 0 */
int sptorch_ext_masked_softmax_f32(const void* a, const void* keep_u8, void* out, size_t rows, size_t cols, int rank1);
/* out[t,:] = tok[ids[t],:] + pos[t % T,:]   (nn/src/lib.rs:1351-1356); ids are int32 on the device;
 * pos_w may be NULL: token rows only (QwenLikeGPT::forward_ids, nn/src/lib.rs:1458-1459) */
int sptorch_ext_embedding_sum(const void* tok_w, const void* pos_w, const void* ids_i32, void* out,
                              size_t n_tokens, size_t T, size_t vocab, size_t dim, int dtype);

/* ---- neighbours of the path (the Qwen-like blocks and the step after the forward) ---- */
int sptorch_ext_rms_norm(const void* x, const void* weight_f32, void* out, size_t rows, size_t dim, float eps, int dtype);   /* core-ops/src/lib.rs:1453 */
int sptorch_ext_swiglu(const void* x, const void* gate, void* out, size_t n, int dtype);
/* Rotary position embedding, in place (apply_rope_raw, nn/src/lib.rs:930-961, as MultiHeadAttention::forward_causal_impl applies it
 * to Q and K, :606-609).  x is token-major [rows, ld] with head h at columns h*head_dim (the reference's [n_head, seq_len, head_dim]
 * permute is not needed); row r has position position_offset + r % seq_len; pairs are (2p, 2p+1), theta = pos / base^(2p/head_dim). */
int sptorch_ext_rope(void* x, size_t rows, size_t seq_len, size_t n_heads, size_t head_dim, size_t ld, float rope_base,
                     size_t position_offset, int dtype);                                    /* core-ops/src/lib.rs:1529 */
/* cross_entropy_loss / cross_entropy_loss_ignore_index over logits [rows, ld] (core-ops/src/lib.rs:1079-1194): mean of
 * -(x[target] - logsumexp(x)) over the rows whose target differs from ignore_index (has_ignore = 0: every row).
 * row_loss_f32: device scratch of rows + 1 floats (per-row losses, then the mean); the mean is also copied to *host_mean.
 * A target outside [0, classes) is reported at the next sync (the reference panics). */
int sptorch_ext_cross_entropy(const void* logits, size_t ld, const void* targets_i64, size_t rows, size_t classes, int has_ignore,
                              long long ignore_index, void* row_loss_f32, float* host_mean, int dtype);

/* ---- Linear (nn/src/lib.rs:121-133): out[M,N] = act(alpha * x[M,K] W[N,K]^T + bias[N]) + residual[M,N] ----
 * W is consumed in its native [out,in] layout; the reference's transpose() copy does not exist here.
 * mode SPT_MM_BF16: x, W, residual, out are bf16 (out may be f32 with out_dtype); SPT_MM_TF32 / SPT_MM_F32: f32.
 * bias is always f32; bias and residual may be NULL.  ldo = row stride of out/residual in elements (0 = N). */
/* arithmetic of the f32 C-ABI contractions sptorch_matmul_f32 / sptorch_batch_matmul_f32:
 * SPT_MM_TF32 (default, tensor cores) or SPT_MM_F32 (CUDA cores, f32 FMA in k order) */
int sptorch_ext_set_matmul_mode(int mode);
/* tiles of the wide GEMMs: 3 (default) = pairs of CTAs on 256 x 256 tiles (tcgen05 cta_group::2, each SM loads half of the B tile)
 * where they measured faster (TF32 problems, bf16 problems with K >= 1536, from 2048 rows up), one CTA per 128 x 256 tile elsewhere;
 * 0 = one CTA per tile always; 1 = pairs wherever they apply; 2 = pairs for TF32 problems only.  Pairs give bit-identical results. */
int sptorch_ext_set_gemm_pair(int mode);

/* No counterpart in the reference.  sptorch_matmul_f32 for callers that must not allocate device memory (fixed,
 * audited memory budgets; loops that may not touch the allocator; an exhausted pool): the transposed-B scratch is a
 * static 8 MiB array inside the library, so k * n is limited to 2,097,152 elements and larger products are rejected.
 * No cudaMalloc/cudaFree/pool call is made.  The array's device address is resolved when the backend is initialised; if that
 * lookup failed, the first call repeats it, so the first call should come before any stream capture.  All calls share the
 * array (it keeps the last call's contents; none of it needs clearing) -- calls that overlap on the GPU, or that two host
 * threads issue at the same time (their transpose and product kernels can interleave on the stream), race. */
int sptorch_ext_matmul_f32_static(const void* a, const void* b, void* out, size_t m, size_t k, size_t n);

/* bf16 problems of at most 64 rows run a weight-streaming kernel (the projections of a decode step) whose sums are taken in
 * another order than the 128-row tensor-core tiles': the same row may differ in its last bit between a call with 64 rows and
 * one with more.  The model forward (sptorch_ext_gpt_forward*) never takes that kernel: a row of its output does not depend
 * on the batch. */
int sptorch_ext_linear(const void* x, const void* w, const void* bias_f32, const void* residual, void* out,
                       size_t M, size_t K, size_t N, size_t ldo, float alpha, int epilogue, int mode, int out_dtype);

/* ---- causal multi-head attention core (nn/src/lib.rs:600-637 without the four projections) ----
 * q, k, v: [B*T, ld] with head h at columns h*hd..; out [B*T, H*hd].  dtype BF16 runs the fused
 * kernel; F32 runs scores -> causal softmax -> PV through the TF32 GEMM with a caller-visible
 * workspace of sptorch_ext_attention_workspace() bytes. */
/* 0 (default): bf16 with head_dim 64 or 128 runs the fused kernel, everything else the materialised form; 1: always materialised */
int sptorch_ext_set_attention_mode(int mode);
size_t sptorch_ext_attention_workspace(size_t B, size_t T, size_t H, size_t hd, int dtype);
int sptorch_ext_attention_causal(const void* q, const void* k, const void* v, void* out, void* workspace,
                                 size_t B, size_t T, size_t H, size_t hd, size_t ld_qkv, int dtype);

/* ---- GPT forward (nn/src/lib.rs:1332-1364) ---- */
typedef struct {
    int32_t vocab, d_model, n_layer, n_head, d_ff, seq_len;
    int32_t dtype;        /* SPT_F32 (TF32 contractions) or SPT_BF16 */
    int32_t max_batch;    /* activations are sized for max_batch * seq_len tokens */
    float   eps;          /* 1e-5 in the reference (nn/src/lib.rs:383) */
    int32_t tp_rank, tp_size;   /* tensor parallel shard of this process; 0,1 = none */
    int32_t arch;         /* SPT_ARCH_GPT: nn::GPT (learned positions, LayerNorm, GELU MLP);
                           * SPT_ARCH_QWEN_LIKE: nn::QwenLikeGPT (nn/src/lib.rs:1439-1467: no position table, RMSNorm with eps 1e-6,
                           * RoPE on Q and K, SwiGLU MLP with up / gate / down projections, all three biased) */
    float   rope_base;    /* SPT_ARCH_QWEN_LIKE: 10000 in the reference (nn/src/lib.rs:1083); 0 selects that default */
} sptorch_gpt_config;
#define SPT_ARCH_GPT 0
#define SPT_ARCH_QWEN_LIKE 1

void* sptorch_ext_gpt_create(const sptorch_gpt_config* cfg);       /* allocates weights + activations; NULL on failure */
void  sptorch_ext_gpt_destroy(void* gpt);
/* name as in GPT::named_parameters (nn/src/lib.rs:1382-1392); host f32 values of the FULL
 * (unsharded) tensor; converted to the model dtype and sliced for this tp_rank on upload. */
int   sptorch_ext_gpt_set_param(void* gpt, const char* name, const float* host, size_t n);
size_t sptorch_ext_gpt_logits_ld(void* gpt);                       /* row stride of device logits (vocab padded to 64) */
/* ids_i32 [batch*T] on the device -> logits [batch*T, ld] on the device in the model dtype */
int   sptorch_ext_gpt_forward(void* gpt, const void* ids_i32, int batch, int T, void* logits);
/* residual stream after embedding (i=0), after block i (1..L), and ln_f output (L+1): [batch*T, d] model dtype */
/* CUDA-graph replay of sptorch_ext_gpt_forward (on by default; the third call with unchanged arguments is the first replay) */
int   sptorch_ext_gpt_enable_graphs(void* gpt, int on);
int   sptorch_ext_gpt_enable_taps(void* gpt, int on);
const void* sptorch_ext_gpt_tap(void* gpt, int i);
/* Host-buffer call, the shape of nn::GPT::forward_ids: ids on the host in, dense [batch*T, vocab]
 * logits on the host out (model dtype), copies included.  Processes micro-batches of `chunk`
 * sequences and overlaps the device->host copy of one chunk with the compute of the next. */
int   sptorch_ext_gpt_forward_host(void* gpt, const int32_t* ids_host, int batch, int T, void* logits_host, int chunk);
/* Forward fused with the step after it (cross_entropy_loss / cross_entropy_loss_ignore_index, core-ops/src/lib.rs:1079-1194; the
 * greedy token = the first candidate of sampling_candidates, nn/src/lib.rs:2381-2418): the [batch*T, vocab] logits are never
 * written.  The LM head's epilogue reduces every tile of logits -- rounded to the model dtype first, so the values are exactly
 * those sptorch_ext_gpt_forward would have stored -- to per-row partial (max, sum exp, first argmax, target logit), and a second
 * kernel merges them.  targets_i64 [batch*T] on the device (NULL: no loss); argmax_i32 [batch*T] on the device (NULL: not wanted);
 * row_loss_f32: device scratch of batch*T + 1 floats (per-row losses, then their mean; rows whose target equals ignore_index are
 * left out when has_ignore != 0); the mean is also copied to *host_mean.  Needs vocab > 128; not for tensor-parallel shards. */
int   sptorch_ext_gpt_forward_loss(void* gpt, const void* ids_i32, const void* targets_i64, int batch, int T, int has_ignore,
                                   long long ignore_index, void* argmax_i32, void* row_loss_f32, float* host_mean);
/* the same with host buffers: ids (and targets) in, greedy tokens [batch*T] and the mean loss out; 4 bytes per token leave the device */
int   sptorch_ext_gpt_forward_loss_host(void* gpt, const int32_t* ids_host, const int64_t* targets_host, int batch, int T, int has_ignore,
                                        long long ignore_index, int32_t* argmax_host, float* host_mean, int chunk);
/* ---- incremental decode with a key/value cache (nn/src/lib.rs:1540-1573, 1619-1646, 706-760) ----
 * enable_kv_cache allocates [layer][sequence][position][d_model] K and V caches for max_context positions (<= seq_len).
 * prefill = forward over ids [batch, T] that also fills the cache.  decode runs one token per sequence through the
 * blocks against the cache: append = 1 takes NEW tokens (their K,V are appended, logits of the new position);
 * append = 0 recomputes the logits of the last cached token (decode_logits_from_cache right after a prefill).
 * logits of decode: [batch, ld].  The cache is a ring: appending to a full cache replaces the oldest position, the last max_context
 * positions stay (append_kv_tensor, nn/src/lib.rs:2165-2203) and the window start moves on by one; nothing is copied or recomputed. */
int   sptorch_ext_gpt_enable_kv_cache(void* gpt, int max_context);
int   sptorch_ext_gpt_cached_len(void* gpt);
long long sptorch_ext_gpt_window_start(void* gpt);        /* absolute position of the oldest cached token (0 until the cache slides) */
int   sptorch_ext_gpt_prefill(void* gpt, const void* ids_i32, int batch, int T, void* logits);
int   sptorch_ext_gpt_decode(void* gpt, const void* last_ids_i32, int batch, int append, void* logits);
/* the attention of one new token over a cache (nn/src/lib.rs:706-760 without the projections): q [B, H*hd];
 * k_cache, v_cache [B, cache_positions, H*hd] of which the first n positions are valid; out [B, H*hd] */
int   sptorch_ext_attention_last_token(const void* q, const void* k_cache, const void* v_cache, void* out, size_t B, size_t H, size_t hd,
                                       size_t n, size_t cache_positions, int dtype);
/* number of kernels one sptorch_ext_gpt_forward call of this shape enqueues */
int   sptorch_ext_gpt_launches(void* gpt, int batch, int T);
/* tensor-parallel all-reduce hook: called on the library stream's behalf after the row-split
 * projections; the callee must enqueue a sum-all-reduce of n elements at buf onto cuda_stream. */
typedef int (*sptorch_allreduce_fn)(void* buf, size_t n, int dtype, void* cuda_stream, void* user);
/* 1: bf16 GPT models apply LayerNorm inside the epilogue of the GEMMs that consume it (weights pre-multiplied by gamma, a per-token
 * statistics pass instead of a normalising pass).  Default 0: on B200 the statistics passes save 0.57 ms per step of the
 * GPT-2-small-shape benchmark and the heavier epilogues cost 0.5 ms, so the step time does not move (19.2 ms either way). */
int   sptorch_ext_gpt_enable_ln_fold(void* gpt, int on);
/* tensor parallel: reduce one half of the batch on a second stream while the other half computes.  mode 0: never; 1: whenever
 * the batch is even; 2 (default): from four ranks up, where the all-reduces are two fifths of a step and hiding them gains more
 * than the SMs left free for the collective cost (4 x B200, 12 layers of the 1.3B shape: 25.7 -> 21.1 ms per step; on two ranks
 * 22.0 -> 21.5 at best).  The call leaves 32 SMs free for the collective unless sptorch_ext_set_sm_reserve has set a number. */
int   sptorch_ext_gpt_enable_tp_overlap(void* gpt, int on);
int   sptorch_ext_gpt_set_allreduce(void* gpt, sptorch_allreduce_fn fn, void* user);
/* The tensor-parallel shard rule that sptorch_ext_gpt_set_param applies (host code: usable without a GPU).  For the parameter
 * `name` (GPT::named_parameters, nn/src/lib.rs:1382-1392) of full shape [rows, cols] (a vector is [rows, 1]) and rank tp_rank of
 * tp_size: *kind = 0 replicated, 1 the rows [*begin, *begin + *count) (wq / wk / wv / ffn_up / ffn_gate and their biases: the
 * column-parallel projections), 2 the columns [*begin, *begin + *count) (wo / ffn_down: the row-parallel projections, whose partial
 * products one all-reduce per attention and per MLP block sums).  sptorch_ext_tp_slice_host copies that slice of a full host tensor
 * into out (rows: count * cols values; columns: rows * count values).  Only the rank for which
 * sptorch_ext_tp_rank_folds_residual is non-zero adds the residual and the ffn_down bias to its partial product, so that the
 * all-reduced sum is the new residual stream (the reference's split of work across workers: crates/distributed/src/data_parallel.rs:21-59
 * shards the batch; this is the same idea applied to the weight matrices). */
int   sptorch_ext_tp_param_shard(const char* name, int tp_rank, int tp_size, size_t rows, size_t cols, int* kind, size_t* begin, size_t* count);
int   sptorch_ext_tp_slice_host(const float* full, size_t rows, size_t cols, int kind, size_t begin, size_t count, float* out);
int   sptorch_ext_tp_rank_folds_residual(int tp_rank);

/* ---- the step after the forward: sampling candidates (nn/src/lib.rs:2381-2418) ----
 * One row of logits on the device (f32 or bf16, at least vocab_size values) -> candidates on the host in the reference's
 * order: repetition penalty (history tokens: negative values multiplied, others divided by max(penalty, 1)) and division by
 * max(temperature, 1e-8), non-finite values dropped, stable sort by value descending, top_k cut (0 = none), softmax, top_p cut
 * on the running sum (clamped to [0, 1], at least one candidate stays), softmax over the kept ones.  out_logits are the
 * scaled values the reference stores in TokenCandidate::logit.  The call synchronises; *count candidates are written
 * (an error if they exceed capacity; vocab_size always suffices). */
int       sptorch_ext_sampling_candidates(const void* logits, size_t n_logits, int dtype, size_t vocab_size, float temperature, size_t top_k,
                                          float top_p, float repetition_penalty, const int64_t* history, size_t n_history,
                                          int32_t* out_ids, float* out_logits, float* out_probs, size_t capacity, size_t* count);
/* the same with a TokenConstraint's allowed set applied first (filtered_step_logits, nn/src/lib.rs:2465-2480): every token outside
 * `allowed` counts as -inf; an empty set leaves no candidate */
int       sptorch_ext_sampling_candidates_constrained(const void* logits, size_t n_logits, int dtype, size_t vocab_size, float temperature,
                                                      size_t top_k, float top_p, float repetition_penalty, const int64_t* history,
                                                      size_t n_history, const int64_t* allowed, size_t n_allowed,
                                                      int32_t* out_ids, float* out_logits, float* out_probs, size_t capacity, size_t* count);
/* sample_from_candidates (nn/src/lib.rs:2420-2429) for the caller's uniform draw `threshold` in [0, 1); -1 without candidates */
long long sptorch_ext_sample_from_candidates(const int32_t* ids, const float* probs, size_t count, float threshold);

/* ---- on-disk weight formats of the reference (crates/serialize/src/lib.rs, safetensors.rs; crates/versioning/src/lib.rs:32-66) ----
 * Readers are host code and work without a GPU: a file is parsed into f32 entries (F16 / BF16 widened exactly as the
 * reference's f16_to_f32 / bf16_to_f32), then a loader checks it against the model's named parameters with the reference's
 * strictness (magic, version, schema, count, duplicate / missing names, shape, dtype) and uploads only if every check passed. */
#define SPT_WEIGHTS_AUTO 0          /* by content */
#define SPT_WEIGHTS_SPTC 1          /* binary checkpoint "SPTC": save_checkpoint / load_checkpoint, serialize/src/lib.rs:34-131 */
#define SPT_WEIGHTS_STATE_DICT 2    /* JSON state_dict "sptorch.state_dict.v1": serialize/src/lib.rs:315-328, 446-481 */
#define SPT_WEIGHTS_SAFETENSORS 3   /* serialize/src/safetensors.rs:25-73 */
void*        sptorch_ext_weights_open(const char* path, int format);      /* NULL on failure, reason in sptorch_ext_last_error */
void         sptorch_ext_weights_close(void* w);
int          sptorch_ext_weights_format(void* w);
size_t       sptorch_ext_weights_count(void* w);
const char*  sptorch_ext_weights_name(void* w, size_t i);                 /* "" in a binary checkpoint, which stores no names */
const char*  sptorch_ext_weights_dtype(void* w, size_t i);                /* dtype as stored: "F32", "F16", "BF16" */
size_t       sptorch_ext_weights_ndim(void* w, size_t i);
size_t       sptorch_ext_weights_dim(void* w, size_t i, size_t k);
size_t       sptorch_ext_weights_numel(void* w, size_t i);
const float* sptorch_ext_weights_data(void* w, size_t i);
/* named parameters of the model in the reference's order (GPT::named_parameters nn/src/lib.rs:1382-1392, QwenLikeGPT :1483-1492) */
size_t       sptorch_ext_gpt_param_count(void* gpt);
int          sptorch_ext_gpt_param_info(void* gpt, size_t i, char* name, size_t name_cap, size_t* dims, size_t* ndim /* in: capacity, out: rank */);
/* binary checkpoint: by position (load_checkpoint); state_dict: by name (load_state_dict, serialize/src/lib.rs:237-313);
 * safetensors: n_map pairs {model parameter name, name in the file} as SafeTensorsFile::load_into (safetensors.rs:85-116),
 * or mapping NULL / n_map 0: every model parameter under its own name */
int          sptorch_ext_gpt_load_weights(void* gpt, void* w, const char* const* mapping, size_t n_map);
/* JSON state_dict plus "<path>.manifest.json" (load_state_dict_bundle, serialize/src/lib.rs:366-441) */
int          sptorch_ext_gpt_load_bundle(void* gpt, const char* weights_path);

/* ---- NCCL over NVLink (replaces the gRPC star all-reduce of crates/distributed/src/coordinator.rs:73-116) ---- */
int sptorch_ext_nccl_unique_id(const char* libnccl_path, void* id128);                      /* rank 0: 128-byte id */
int sptorch_ext_nccl_init(const char* libnccl_path, const void* id128, int rank, int world);
int sptorch_ext_nccl_allreduce_sum(void* buf, size_t n, int dtype);                         /* in place, library stream */
int sptorch_ext_nccl_allreduce_avg_f32(void* buf, size_t n);                                /* sum then * 1/world: average_gradients semantics */
int sptorch_ext_nccl_shutdown(void);
int sptorch_ext_gpt_use_nccl(void* gpt);      /* install the NCCL all-reduce as the tensor-parallel hook */

#ifdef __cplusplus
}
#endif
#endif /* SPTORCH_B200_EXT_H */
