// decode.cu -- single-token attention over a key/value cache (crates/nn/src/lib.rs:706-760, causal_attention_last_token).
//
// One warp per (sequence, head).  The query (hd values) sits in shared memory; lanes take cached positions p = lane,
// lane+32, ... for the scores (each reads one contiguous K row of hd elements), the scores are normalised with two warp
// reductions, and for the weighted sum every lane owns hd/32 output columns and walks the positions (coalesced V rows).
// HBM-bound: the cache is read once: 2 * n * hd * sizeof(T) bytes per (sequence, head).
// Cache layout: [layer][sequence][position][H*hd] (position-major rows, as the HAL spec describes for devices:
// crates/hal/src/lib.rs:129-303), so appending a token is one row write per layer.
#include "common.h"
#include "../../include/sptorch_b200_ext.h"
#include <math.h>

namespace spt {

constexpr int kDecThreads = 128;    // 4 warps = 4 (sequence, head) pairs per CTA

template <typename T>
__global__ void __launch_bounds__(kDecThreads) attention_last_token_kernel(const T* __restrict__ q, long long ld_q, const T* __restrict__ kc,
                                                                           const T* __restrict__ vc, T* __restrict__ out, long long ld_out,
                                                                           int B, int H, int hd, int n, long long seq_stride, long long row_stride,
                                                                           float scale) {
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* qs = sm + warp * (hd + n);
    float* sc = qs + hd;
    const int pair = blockIdx.x * (kDecThreads / 32) + warp;
    if (pair >= B * H) return;
    const int b = pair / H, h = pair % H;
    const T* qp = q + (long long)b * ld_q + (long long)h * hd;
    for (int d = lane; d < hd; d += 32) qs[d] = (float)qp[d];
    __syncwarp();
    const T* kb = kc + (long long)b * seq_stride + (long long)h * hd;
    const T* vb = vc + (long long)b * seq_stride + (long long)h * hd;
    float mx = -INFINITY;
    for (int p = lane; p < n; p += 32) {
        const T* kr = kb + (long long)p * row_stride;
        float dot = 0.0f;
        for (int d = 0; d < hd; d++) dot += qs[d] * (float)kr[d];
        dot *= scale;
        sc[p] = dot;
        mx = fmaxf(mx, dot);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float den = 0.0f;
    for (int p = lane; p < n; p += 32) { float e = expf(sc[p] - mx); sc[p] = e; den += e; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
    __syncwarp();
    const float inv = 1.0f / den;
    T* op = out + (long long)b * ld_out + (long long)h * hd;
    for (int d = lane; d < hd; d += 32) {
        float acc = 0.0f;
        for (int p = 0; p < n; p++) acc += (sc[p] * inv) * (float)vb[(long long)p * row_stride + d];
        op[d] = (T)acc;
    }
}

// q: [B, ld_q] (head h at columns h*hd); kc/vc: first cached row of this layer, rows of H*hd elements, sequences
// seq_stride apart; n cached positions (the newest included); out: [B, ld_out]
int attention_last_token(const void* q, long long ld_q, const void* kc, const void* vc, void* out, long long ld_out, int B, int H, int hd,
                         int n, long long seq_stride, long long row_stride, int dtype) {
    if (B <= 0 || H <= 0 || n <= 0) return fail("attention_last_token: empty cache or batch");
    const size_t smem = (size_t)(kDecThreads / 32) * (hd + n) * sizeof(float);
    if (smem > 200 * 1024) return fail("attention_last_token: %d cached positions exceed the shared-memory score buffer", n);
    const int grid = ceil_div((long long)B * H, kDecThreads / 32);
    const float scale = 1.0f / sqrtf((float)hd);
    if (dtype == BF16) {
        auto kern = attention_last_token_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) SPT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<grid, kDecThreads, smem, rt().stream>>>((const __nv_bfloat16*)q, ld_q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc,
                                                       (__nv_bfloat16*)out, ld_out, B, H, hd, n, seq_stride, row_stride, scale);
    } else {
        auto kern = attention_last_token_kernel<float>;
        if (smem > 48 * 1024) SPT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<grid, kDecThreads, smem, rt().stream>>>((const float*)q, ld_q, (const float*)kc, (const float*)vc, (float*)out, ld_out, B, H, hd, n,
                                                       seq_stride, row_stride, scale);
    }
    SPT_LAUNCH_CHECK("attention_last_token");
    return 0;
}

}  // namespace spt

using namespace spt;

extern "C" int sptorch_ext_attention_last_token(const void* q, const void* k_cache, const void* v_cache, void* out, size_t B, size_t H, size_t hd,
                                                size_t n, size_t cache_positions, int dtype) {
    if (enter()) return 1;
    if (!q || !k_cache || !v_cache || !out) return fail("attention_last_token: null handle");
    if (dtype != SPT_F32 && dtype != SPT_BF16) return fail("attention_last_token: unknown dtype %d", dtype);
    if (n == 0 || n > cache_positions) return fail("attention_last_token: n must be in 1..cache_positions");
    const long long d = (long long)(H * hd);
    return attention_last_token(q, d, k_cache, v_cache, out, d, (int)B, (int)H, (int)hd, (int)n, (long long)cache_positions * d, d, dtype);
}
