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
                                                                           float scale, const int* __restrict__ state, int n_cap) {
    extern __shared__ float sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // decode graphs: the number of valid positions lives in a device word; shared memory is sized for the cache capacity
    if (state) n = state[1];
    float* qs = sm + warp * (hd + (state ? n_cap : n));
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
// The same function for head sizes up to 128 whose rows are 16 .. 512 bytes (a power of two): the form the decode step uses.
// One CTA of four warps per (sequence, head).  A row of K or V is read by LPR = row bytes / 16 neighbouring lanes with one 16-byte
// load each, so a warp fetches 32 / LPR whole rows per instruction, fully coalesced, and several positions are in flight per lane;
// the dot product is finished with log2(LPR) shuffles.  Every row group keeps a running (maximum, sum, weighted value sum) over the
// positions it visits (online softmax: exp(s - max) / sum exp(s - max) evaluated incrementally), the groups of a warp and then the
// four warps are merged at the end.  Same result as the kernel above up to the order of the f32 sums.
// HBM traffic: 2 * n * hd * sizeof(T) bytes per (sequence, head), read once.
template <typename T>
__global__ void __launch_bounds__(128) attention_last_token_rows_kernel(const T* __restrict__ q, long long ld_q, const T* __restrict__ kc,
                                                                        const T* __restrict__ vc, T* __restrict__ out, long long ld_out, int H, int hd,
                                                                        int n, long long seq_stride, long long row_stride, float scale,
                                                                        const int* __restrict__ state) {
    constexpr int VE = 16 / (int)sizeof(T);              // elements per 16-byte segment
    __shared__ float sm[4 * 130];                         // per warp: maximum, sum, up to 128 value sums (f32 rows of 512 bytes, bf16 rows of 256)
    if (state) n = state[1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int lpr = hd / VE;                             // lanes per row
    const int rpi = 32 / lpr;                            // rows per warp instruction
    const int seg = lane % lpr, grp = lane / lpr;
    const int b = blockIdx.x / H, h = blockIdx.x % H;
    auto widen = [](uint4 raw, float (&f)[VE]) {
        if constexpr (sizeof(T) == 2) {
            const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; i++) { const float2 a = __bfloat1622float2(e[i]); f[2 * i] = a.x; f[2 * i + 1] = a.y; }
        } else {
            f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y); f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
        }
    };
    float qf[VE];
    widen(*reinterpret_cast<const uint4*>(q + (long long)b * ld_q + (long long)h * hd + seg * VE), qf);
    const T* kb = kc + (long long)b * seq_stride + (long long)h * hd + seg * VE;
    const T* vb = vc + (long long)b * seq_stride + (long long)h * hd + seg * VE;
    float m = -INFINITY, l = 0.0f, o[VE];
#pragma unroll
    for (int i = 0; i < VE; i++) o[i] = 0.0f;
    const int stride = 4 * rpi;
    auto visit = [&](uint4 kraw, uint4 vraw) {
        float kf[VE], vf[VE];
        widen(kraw, kf);
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < VE; i++) s += qf[i] * kf[i];
        for (int off = lpr >> 1; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        s *= scale;
        const float mn = fmaxf(m, s);
        const float corr = expf(m - mn), pr = expf(s - mn);        // m = -inf on the first visit: corr = 0, nothing accumulated yet
        widen(vraw, vf);
        l = l * corr + pr;
#pragma unroll
        for (int i = 0; i < VE; i++) o[i] = o[i] * corr + pr * vf[i];
        m = mn;
    };
    // The loops run on a warp-uniform base position (the shuffles inside visit() are warp-wide).  First the part where every row
    // group has two live positions, two rows per lane in flight; then what is left, one position per group and turn, where groups
    // past the end still take part in the shuffles with a dead value.
    int base = warp * rpi;
    for (; base + stride + rpi <= n; base += 2 * stride) {
        const long long p = base + grp;
        const uint4 k0 = *reinterpret_cast<const uint4*>(kb + p * row_stride), k1 = *reinterpret_cast<const uint4*>(kb + (p + stride) * row_stride);
        const uint4 v0 = *reinterpret_cast<const uint4*>(vb + p * row_stride), v1 = *reinterpret_cast<const uint4*>(vb + (p + stride) * row_stride);
        visit(k0, v0); visit(k1, v1);
    }
    for (; base < n; base += stride) {
        const bool live = base + grp < n;
        const long long pp = live ? base + grp : 0;
        const uint4 k0 = *reinterpret_cast<const uint4*>(kb + pp * row_stride), v0 = *reinterpret_cast<const uint4*>(vb + pp * row_stride);
        const float m_keep = m, l_keep = l;
        float o_keep[VE];
#pragma unroll
        for (int i = 0; i < VE; i++) o_keep[i] = o[i];
        visit(k0, v0);
        if (!live) {
            m = m_keep; l = l_keep;
#pragma unroll
            for (int i = 0; i < VE; i++) o[i] = o_keep[i];
        }
    }
    // merge the row groups of the warp (groups that saw no position carry m = -inf, l = 0)
    auto merge = [&](float mo, float lo, const float (&oo)[VE]) {
        const float mn = fmaxf(m, mo);
        const float ca = (m == -INFINITY) ? 0.0f : expf(m - mn), cb = (mo == -INFINITY) ? 0.0f : expf(mo - mn);
        l = l * ca + lo * cb;
#pragma unroll
        for (int i = 0; i < VE; i++) o[i] = o[i] * ca + oo[i] * cb;
        m = mn;
    };
    for (int off = lpr; off < 32; off <<= 1) {
        const float mo = __shfl_xor_sync(0xffffffffu, m, off), lo = __shfl_xor_sync(0xffffffffu, l, off);
        float oo[VE];
#pragma unroll
        for (int i = 0; i < VE; i++) oo[i] = __shfl_xor_sync(0xffffffffu, o[i], off);
        merge(mo, lo, oo);
    }
    // ... and the four warps
    float* mine = sm + warp * 130;
    if (grp == 0) {
        if (seg == 0) { mine[0] = m; mine[1] = l; }
#pragma unroll
        for (int i = 0; i < VE; i++) mine[2 + seg * VE + i] = o[i];
    }
    __syncthreads();
    if (warp == 0 && grp == 0) {
        for (int w = 1; w < 4; w++) {
            const float* other = sm + w * 130;
            float oo[VE];
#pragma unroll
            for (int i = 0; i < VE; i++) oo[i] = other[2 + seg * VE + i];
            merge(other[0], other[1], oo);
        }
        const float inv = 1.0f / l;
        T* op = out + (long long)b * ld_out + (long long)h * hd + seg * VE;
        uint4 raw;
        if constexpr (sizeof(T) == 2) {
            __nv_bfloat162* e = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; i++) e[i] = __floats2bfloat162_rn(o[2 * i] * inv, o[2 * i + 1] * inv);
        } else {
            raw = make_uint4(__float_as_uint(o[0] * inv), __float_as_uint(o[1] * inv), __float_as_uint(o[2] * inv), __float_as_uint(o[3] * inv));
        }
        *reinterpret_cast<uint4*>(op) = raw;
    }
}

// Device-resident state of a decode step replayed as a CUDA graph: {absolute position, valid cached positions (new token
// included), ring slot the new token's key / value go to, row of the position table}.
__global__ void decode_state_kernel(int* state, int pos, int n, int slot, int pos_row) {
    state[0] = pos; state[1] = n; state[2] = slot; state[3] = pos_row;
}
int decode_state_launch(int* state, int pos, int n, int slot, int pos_row) {
    decode_state_kernel<<<1, 1, 0, rt().stream>>>(state, pos, n, slot, pos_row);
    SPT_LAUNCH_CHECK("decode_state");
    return 0;
}

// key and value of the new token of every sequence ([q | k | v] rows of 3*dl elements) into cache row `slot` (slot_dev overrides)
template <typename T>
__global__ void __launch_bounds__(256) kv_append_kernel(const T* __restrict__ qkv, T* __restrict__ kc, T* __restrict__ vc, int B, int dl, long long seq_stride,
                                                        int slot, const int* __restrict__ state) {
    if (state) slot = state[2];
    const int vec = 16 / (int)sizeof(T);
    const int per_row = dl / vec;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < B * per_row; i += gridDim.x * blockDim.x) {
        const int b = i / per_row, c = (i - b * per_row) * vec;
        const T* src = qkv + (long long)b * 3 * dl;
        const long long dst = (long long)b * seq_stride + (long long)slot * dl + c;
        *reinterpret_cast<uint4*>(kc + dst) = *reinterpret_cast<const uint4*>(src + dl + c);
        *reinterpret_cast<uint4*>(vc + dst) = *reinterpret_cast<const uint4*>(src + 2 * dl + c);
    }
}
int kv_append_launch(const void* qkv, void* kc, void* vc, int B, int dl, long long seq_stride, int slot, const int* state, int dtype) {
    const int vec = dtype == BF16 ? 8 : 4;
    if (dl % vec) return fail("kv_append: row width %d is not a multiple of %d", dl, vec);
    const int work = B * (dl / vec);
    const int grid = (work + 255) / 256;
    if (dtype == BF16) kv_append_kernel<__nv_bfloat16><<<grid, 256, 0, rt().stream>>>((const __nv_bfloat16*)qkv, (__nv_bfloat16*)kc, (__nv_bfloat16*)vc, B, dl, seq_stride, slot, state);
    else kv_append_kernel<float><<<grid, 256, 0, rt().stream>>>((const float*)qkv, (float*)kc, (float*)vc, B, dl, seq_stride, slot, state);
    SPT_LAUNCH_CHECK("kv_append");
    return 0;
}

// state / n_cap: when state is given, n is read from state[1] at run time and shared memory is sized for n_cap positions
int attention_last_token(const void* q, long long ld_q, const void* kc, const void* vc, void* out, long long ld_out, int B, int H, int hd,
                         int n, long long seq_stride, long long row_stride, int dtype, const int* state, int n_cap) {
    if (B <= 0 || H <= 0 || n <= 0) return fail("attention_last_token: empty cache or batch");
    {
        // rows of 16 .. 512 bytes, a power of two, everything 16-byte aligned: the coalesced kernel
        const size_t es = dtype == BF16 ? 2 : 4;
        const size_t rb = (size_t)hd * es;
        const bool pow2 = rb >= 16 && rb <= 512 && hd <= 128 && (rb & (rb - 1)) == 0;
        const bool aligned = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kc) | reinterpret_cast<uintptr_t>(vc) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 &&
                             (ld_q * es) % 16 == 0 && (ld_out * es) % 16 == 0 && (seq_stride * es) % 16 == 0 && (row_stride * es) % 16 == 0;
        if (pow2 && aligned) {
            const float scale = 1.0f / sqrtf((float)hd);
            if (dtype == BF16)
                attention_last_token_rows_kernel<__nv_bfloat16><<<B * H, 128, 0, rt().stream>>>((const __nv_bfloat16*)q, ld_q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc,
                                                                                            (__nv_bfloat16*)out, ld_out, H, hd, n, seq_stride, row_stride, scale, state);
            else
                attention_last_token_rows_kernel<float><<<B * H, 128, 0, rt().stream>>>((const float*)q, ld_q, (const float*)kc, (const float*)vc, (float*)out, ld_out, H, hd, n,
                                                                                    seq_stride, row_stride, scale, state);
            SPT_LAUNCH_CHECK("attention_last_token");
            return 0;
        }
    }
    const size_t smem = (size_t)(kDecThreads / 32) * (hd + (state ? n_cap : n)) * sizeof(float);
    if (smem > 200 * 1024) return fail("attention_last_token: %d cached positions exceed the shared-memory score buffer", n);
    const int grid = ceil_div((long long)B * H, kDecThreads / 32);
    const float scale = 1.0f / sqrtf((float)hd);
    if (dtype == BF16) {
        auto kern = attention_last_token_kernel<__nv_bfloat16>;
        if (smem > 48 * 1024) SPT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<grid, kDecThreads, smem, rt().stream>>>((const __nv_bfloat16*)q, ld_q, (const __nv_bfloat16*)kc, (const __nv_bfloat16*)vc,
                                                       (__nv_bfloat16*)out, ld_out, B, H, hd, n, seq_stride, row_stride, scale, state, n_cap);
    } else {
        auto kern = attention_last_token_kernel<float>;
        if (smem > 48 * 1024) SPT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kern<<<grid, kDecThreads, smem, rt().stream>>>((const float*)q, ld_q, (const float*)kc, (const float*)vc, (float*)out, ld_out, B, H, hd, n,
                                                       seq_stride, row_stride, scale, state, n_cap);
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
    return attention_last_token(q, d, k_cache, v_cache, out, d, (int)B, (int)H, (int)hd, (int)n, (long long)cache_positions * d, d, dtype, nullptr, 0);
}
