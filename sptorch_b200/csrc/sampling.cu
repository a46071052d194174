// sampling.cu -- the step after the forward: from one row of logits to the list of sampling candidates.
//
// Reference: sampling_candidates (crates/nn/src/lib.rs:2381-2418) with penalize_repeated_logit (:2343-2352) and
// normalize_candidates (:2354-2374); sample_from_candidates (:2420-2429).  Order of the reference: repetition penalty and
// temperature per token, drop non-finite values, stable sort by value (descending), top-k cut, softmax over what is left,
// top-p cut on the running sum (at least one candidate stays), softmax again over the kept ones.
//
// Here the row stays on the device until the candidates are known: one CTA marks the history in a shared-memory bitmap and
// writes (value, token) pairs, the pairs are sorted with CUB's stable radix sort (library code, as cuBLAS would be for a plain
// GEMM; this is not the forward's hot path), and one CTA finishes: exponentials in parallel, the two running sums by one
// thread in the reference's left-to-right f32 order, so that the top-p cut falls where the reference's does.
#include "common.h"
#include "../../include/sptorch_b200_hal.h"
#include "../../include/sptorch_b200_ext.h"
#include <cub/device/device_radix_sort.cuh>
#include <math_constants.h>
#include <vector>

namespace spt {

constexpr int kSampThreads = 1024;
constexpr int kMaxVocabBitmapWords = 8192;     // shared-memory bitmap: vocabularies up to 262144 tokens

template <typename T>
__global__ void __launch_bounds__(kSampThreads) sampling_prep_kernel(const T* __restrict__ logits, int vocab, float temperature, float penalty,
                                                                     const int* __restrict__ history, int n_hist,
                                                                     const int* __restrict__ allowed, int n_allowed,
                                                                     float* __restrict__ keys, int* __restrict__ ids, int* __restrict__ n_valid) {
    extern __shared__ uint32_t seen[];                     // one bit per token: appears in the history; then one bit per allowed token
    const int words = (vocab + 31) / 32;
    uint32_t* allow = seen + words;
    for (int w = threadIdx.x; w < words; w += blockDim.x) { seen[w] = 0u; if (allowed) allow[w] = 0u; }
    __shared__ int count;
    if (threadIdx.x == 0) count = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_hist; i += blockDim.x) {
        const int t = history[i];
        if (t >= 0 && t < vocab) atomicOr(&seen[t >> 5], 1u << (t & 31));
    }
    for (int i = threadIdx.x; i < n_allowed; i += blockDim.x) {
        const int t = allowed[i];
        if (t >= 0 && t < vocab) atomicOr(&allow[t >> 5], 1u << (t & 31));
    }
    __syncthreads();
    int mine = 0;
    for (int t = threadIdx.x; t < vocab; t += blockDim.x) {
        float x = (float)logits[t];
        if (allowed && !(allow[t >> 5] >> (t & 31) & 1u)) x = -CUDART_INF_F;      // filtered_step_logits: outside the constraint's set
        if (penalty != 1.0f && (seen[t >> 5] >> (t & 31) & 1u)) x = signbit(x) ? x * penalty : x / penalty;
        x = x / temperature;
        const bool ok = isfinite(x);
        keys[t] = ok ? x : -CUDART_INF_F;                  // dropped entries sort behind every kept one
        ids[t] = t;
        mine += ok ? 1 : 0;
    }
    atomicAdd(&count, mine);
    __syncthreads();
    if (threadIdx.x == 0) *n_valid = count;
}

// keys / ids sorted by value (descending, ties in token order).  out_probs doubles as the buffer of exponentials.
__global__ void __launch_bounds__(kSampThreads) sampling_finish_kernel(const float* __restrict__ keys, const int* __restrict__ n_valid, int top_k,
                                                                       float top_p, float* __restrict__ out_probs, int* __restrict__ out_count) {
    __shared__ int n_s;
    __shared__ float sum_s;
    if (threadIdx.x == 0) {
        int n = *n_valid;
        if (top_k > 0 && n > top_k) n = top_k;
        n_s = n;
    }
    __syncthreads();
    int n = n_s;
    if (n == 0) { if (threadIdx.x == 0) *out_count = 0; return; }
    const float mx = keys[0];                              // sorted: the first is the maximum
    for (int i = threadIdx.x; i < n; i += blockDim.x) out_probs[i] = expf(keys[i] - mx);
    __syncthreads();
    if (threadIdx.x == 0) {
        float s = 0.0f;
        for (int i = 0; i < n; i++) s += out_probs[i];     // left to right, as `exps.iter().sum()`
        sum_s = s;
    }
    __syncthreads();
    const float s1 = sum_s;
    if (top_p >= 1.0f || n <= 1) {
        for (int i = threadIdx.x; i < n; i += blockDim.x) out_probs[i] = out_probs[i] / s1;
        if (threadIdx.x == 0) *out_count = n;
        return;
    }
    if (threadIdx.x == 0) {
        float cum = 0.0f;
        int kept = 0;
        for (int i = 0; i < n; i++) {
            cum += out_probs[i] / s1;
            kept = i + 1;
            if (cum >= top_p) break;
        }
        float s = 0.0f;
        for (int i = 0; i < kept; i++) s += out_probs[i];  // the kept ones again, same maximum: the same exponentials
        sum_s = s;
        n_s = kept;
    }
    __syncthreads();
    n = n_s;
    const float s2 = sum_s;
    for (int i = threadIdx.x; i < n; i += blockDim.x) out_probs[i] = out_probs[i] / s2;
    if (threadIdx.x == 0) *out_count = n;
}

}  // namespace spt

using namespace spt;

extern "C" {

static int sampling_impl(const void* logits, size_t n_logits, int dtype, size_t vocab_size, float temperature, size_t top_k,
                         float top_p, float repetition_penalty, const int64_t* history, size_t n_history,
                         const int64_t* allowed, size_t n_allowed, bool constrained,
                         int32_t* out_ids, float* out_logits, float* out_probs, size_t capacity, size_t* count) {
    if (enter()) return 1;
    if (!count) return fail("sampling_candidates: null count");
    *count = 0;
    if (!logits) return fail("sampling_candidates: null logits");
    if (dtype != SPT_F32 && dtype != SPT_BF16) return fail("sampling_candidates: unknown dtype %d", dtype);
    if (vocab_size > n_logits) return fail("sampling_candidates: vocab_size must not exceed logits length");      // the reference asserts (nn/src/lib.rs:2382-2385)
    if (vocab_size == 0) return 0;
    if (vocab_size > (size_t)kMaxVocabBitmapWords * 32) return fail("sampling_candidates: vocabularies above %d tokens are not supported", kMaxVocabBitmapWords * 32);
    if (n_history && !history) return fail("sampling_candidates: null history");
    if (constrained && n_allowed && !allowed) return fail("sampling_candidates: null constraint set");
    if (constrained && (size_t)((vocab_size + 31) / 32) * 8 > 48 * 1024) return fail("sampling_candidates: a constraint set needs a vocabulary of at most 196608 tokens");
    const int V = (int)vocab_size;
    const float temp = temperature > 1e-8f ? temperature : 1e-8f;                       // `temperature.max(1e-8)`
    const float pen = repetition_penalty > 1.0f ? repetition_penalty : 1.0f;            // `repetition_penalty.max(1.0)`
    float tp = top_p;                                                                   // `top_p.clamp(0.0, 1.0)`
    if (!(tp >= 0.0f)) tp = 0.0f;
    if (tp > 1.0f) tp = 1.0f;
    const int k = top_k > (size_t)INT32_MAX ? INT32_MAX : (int)top_k;
    // history: token ids that fit the vocabulary, as int32 on the device
    std::vector<int> hist;
    hist.reserve(n_history);
    for (size_t i = 0; i < n_history; i++) if (history[i] >= 0 && history[i] < (int64_t)V) hist.push_back((int)history[i]);
    const size_t n_hist_kept = hist.size();
    if (constrained) for (size_t i = 0; i < n_allowed; i++) if (allowed[i] >= 0 && allowed[i] < (int64_t)V) hist.push_back((int)allowed[i]);   // one upload: history, then the set
    cudaStream_t st = rt().stream;
    size_t tmp_bytes = 0;
    SPT_CUDA(cub::DeviceRadixSort::SortPairsDescending(nullptr, tmp_bytes, (const float*)nullptr, (float*)nullptr, (const int*)nullptr, (int*)nullptr, V, 0, 32, st));
    const size_t arr = ((size_t)V * 4 + 255) & ~(size_t)255;
    const size_t hist_bytes = (hist.size() * 4 + 255) & ~(size_t)255;
    uint8_t* ws = (uint8_t*)sptorch_ext_alloc_bytes(5 * arr + hist_bytes + 256 + tmp_bytes);
    if (!ws) return 1;
    float* keys = (float*)ws; int* ids = (int*)(ws + arr); float* keys_s = (float*)(ws + 2 * arr); int* ids_s = (int*)(ws + 3 * arr);
    float* probs = (float*)(ws + 4 * arr); int* hist_d = (int*)(ws + 5 * arr); int* counters = (int*)(ws + 5 * arr + hist_bytes);
    void* tmp = ws + 5 * arr + hist_bytes + 256;
    int rc = 0;
    int h_count = 0;
    do {
        if (!hist.empty() && cudaMemcpyAsync(hist_d, hist.data(), hist.size() * 4, cudaMemcpyHostToDevice, st) != cudaSuccess) { rc = fail("sampling_candidates: history upload failed"); break; }
        const size_t smem = (size_t)((V + 31) / 32) * 4 * (constrained ? 2 : 1);
        // a constraint with an empty set leaves nothing: the pointer is what switches the filter on
        const int* allow_d = constrained ? hist_d + n_hist_kept : nullptr;
        const int n_allow = constrained ? (int)(hist.size() - n_hist_kept) : 0;
        if (dtype == SPT_BF16)
            sampling_prep_kernel<__nv_bfloat16><<<1, kSampThreads, smem, st>>>((const __nv_bfloat16*)logits, V, temp, pen, hist_d, (int)n_hist_kept, allow_d, n_allow, keys, ids, counters);
        else
            sampling_prep_kernel<float><<<1, kSampThreads, smem, st>>>((const float*)logits, V, temp, pen, hist_d, (int)n_hist_kept, allow_d, n_allow, keys, ids, counters);
        if (cudaGetLastError() != cudaSuccess) { rc = fail("sampling_candidates: prep launch failed"); break; }
        if (cub::DeviceRadixSort::SortPairsDescending(tmp, tmp_bytes, keys, keys_s, ids, ids_s, V, 0, 32, st) != cudaSuccess) { rc = fail("sampling_candidates: sort failed"); break; }
        sampling_finish_kernel<<<1, kSampThreads, 0, st>>>(keys_s, counters, k, tp, probs, counters + 1);
        if (cudaGetLastError() != cudaSuccess) { rc = fail("sampling_candidates: finish launch failed"); break; }
        if (cudaMemcpyAsync(&h_count, counters + 1, 4, cudaMemcpyDeviceToHost, st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess) { rc = fail("sampling_candidates: reading the count failed"); break; }
        if ((size_t)h_count > capacity) { rc = fail("sampling_candidates: %d candidates do not fit the capacity of %zu", h_count, capacity); break; }
        if (h_count > 0) {
            if ((out_ids && cudaMemcpyAsync(out_ids, ids_s, (size_t)h_count * 4, cudaMemcpyDeviceToHost, st) != cudaSuccess) ||
                (out_logits && cudaMemcpyAsync(out_logits, keys_s, (size_t)h_count * 4, cudaMemcpyDeviceToHost, st) != cudaSuccess) ||
                (out_probs && cudaMemcpyAsync(out_probs, probs, (size_t)h_count * 4, cudaMemcpyDeviceToHost, st) != cudaSuccess) ||
                cudaStreamSynchronize(st) != cudaSuccess) { rc = fail("sampling_candidates: reading the candidates failed"); break; }
        }
        *count = (size_t)h_count;
    } while (0);
    if (rc) cudaStreamSynchronize(st);          // the history vector must outlive its copy
    sptorch_free(ws);
    note_submit();
    return rc;
}

int sptorch_ext_sampling_candidates(const void* logits, size_t n_logits, int dtype, size_t vocab_size, float temperature, size_t top_k,
                                    float top_p, float repetition_penalty, const int64_t* history, size_t n_history,
                                    int32_t* out_ids, float* out_logits, float* out_probs, size_t capacity, size_t* count) {
    return sampling_impl(logits, n_logits, dtype, vocab_size, temperature, top_k, top_p, repetition_penalty, history, n_history, nullptr, 0, false,
                         out_ids, out_logits, out_probs, capacity, count);
}

int sptorch_ext_sampling_candidates_constrained(const void* logits, size_t n_logits, int dtype, size_t vocab_size, float temperature, size_t top_k,
                                                float top_p, float repetition_penalty, const int64_t* history, size_t n_history,
                                                const int64_t* allowed, size_t n_allowed,
                                                int32_t* out_ids, float* out_logits, float* out_probs, size_t capacity, size_t* count) {
    return sampling_impl(logits, n_logits, dtype, vocab_size, temperature, top_k, top_p, repetition_penalty, history, n_history, allowed, n_allowed, true,
                         out_ids, out_logits, out_probs, capacity, count);
}

// sample_from_candidates (nn/src/lib.rs:2420-2429) given the caller's uniform draw in [0, 1): host arithmetic only
long long sptorch_ext_sample_from_candidates(const int32_t* ids, const float* probs, size_t count, float threshold) {
    if (!ids || !probs || count == 0) return -1;
    for (size_t i = 0; i < count; i++) {
        threshold -= probs[i];
        if (threshold <= 0.0f) return ids[i];
    }
    return ids[count - 1];
}

}  // extern "C"
