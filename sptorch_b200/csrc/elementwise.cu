// elementwise.cu -- HBM-bound elementwise kernels: 128-bit loads/stores, grid sized in multiples
// of the SM count, four independent vectors in flight per thread.
//
// Replaces the NVRTC string kernels of the reference (crates/runtime-cuda/src/lib.rs:85-141: one
// scalar 32-bit load per thread, block 256, grid n/256) and restates the semantics of
// CpuBackend (crates/hal/src/lib.rs:497-545, 598-646).  Algorithmic bytes: 8 B/element for unary
// f32 ops, 12 B/element for binary ones.
#include "common.h"
#include "../../include/sptorch_b200_hal.h"
#include "../../include/sptorch_b200_ext.h"
#include <math.h>

namespace spt {

// ---- functors (f32 math; no fast-math: expf/logf/tanhf are the <=2 ulp device versions) ----
struct OpAdd  { __device__ float operator()(float a, float b) const { return a + b; } };
struct OpMul  { __device__ float operator()(float a, float b) const { return a * b; } };
struct OpNeg  { __device__ float operator()(float a) const { return -a; } };
struct OpExp  { __device__ float operator()(float a) const { return expf(a); } };
struct OpLog  { __device__ float operator()(float a) const { return logf(a); } };
struct OpRelu { __device__ float operator()(float a) const { return a > 0.0f ? a : 0.0f; } };
struct OpScale { float s; __device__ float operator()(float a) const { return a * s; } };
// gelu: crates/core-ops/src/lib.rs:1338-1342; k = sqrt(2/pi) rounded to f32 = 0.79788458f
__device__ __forceinline__ float gelu_tanh(float x) {
    const float k = 0.7978845608028654f;
    float x3 = (x * x) * x;
    return 0.5f * x * (1.0f + tanhf(k * (x + 0.044715f * x3)));
}
struct OpGelu { __device__ float operator()(float a) const { return gelu_tanh(a); } };
// bf16 storage: tanh.approx (max relative error 2^-11) is well inside one bf16 ulp (2^-8) of the result and
// keeps the kernel HBM-bound; the precise tanhf costs ~30 instructions per element, more than the memory time.
struct OpGeluBf16 {
    __device__ float operator()(float x) const {
        const float k = 0.7978845608028654f;
        float u = k * (x + 0.044715f * ((x * x) * x)), t;
        asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
        return 0.5f * x * (1.0f + t);
    }
};

// swiglu: crates/core-ops/src/lib.rs:1529-1540: s = 1/(1+exp(-g)); x*g*s
struct OpSwiglu { __device__ float operator()(float x, float g) const { float s = 1.0f / (1.0f + expf(-g)); return x * g * s; } };

constexpr int kThreads = 256;
constexpr int kUnroll = 4;

template <class Op>
__global__ void __launch_bounds__(kThreads) unary_f32_vec(const float4* __restrict__ a, float4* __restrict__ out,
                                                          size_t nvec, const float* a_s, float* out_s, size_t n, Op op) {
    size_t stride = (size_t)gridDim.x * kThreads;
    size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
    for (; i + (kUnroll - 1) * stride < nvec; i += kUnroll * stride) {
        float4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; u++) v[u] = __ldcs(a + i + u * stride);
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            float4 r = make_float4(op(v[u].x), op(v[u].y), op(v[u].z), op(v[u].w));
            __stcs(out + i + u * stride, r);
        }
    }
    for (; i < nvec; i += stride) {
        float4 v = __ldcs(a + i);
        __stcs(out + i, make_float4(op(v.x), op(v.y), op(v.z), op(v.w)));
    }
    // scalar tail (n % 4) by the first threads of block 0
    size_t t = nvec * 4 + (size_t)blockIdx.x * kThreads + threadIdx.x;
    if (blockIdx.x == 0 && t < n) out_s[t] = op(a_s[t]);
}

template <class Op>
__global__ void __launch_bounds__(kThreads) unary_f32_scalar(const float* __restrict__ a, float* __restrict__ out, size_t n, Op op) {
    size_t stride = (size_t)gridDim.x * kThreads;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) out[i] = op(a[i]);
}

template <class Op>
__global__ void __launch_bounds__(kThreads) binary_f32_vec(const float4* __restrict__ a, const float4* __restrict__ b,
                                                           float4* __restrict__ out, size_t nvec, const float* a_s,
                                                           const float* b_s, float* out_s, size_t n, Op op) {
    size_t stride = (size_t)gridDim.x * kThreads;
    size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
    for (; i + (kUnroll - 1) * stride < nvec; i += kUnroll * stride) {
        float4 x[kUnroll], y[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; u++) { x[u] = __ldcs(a + i + u * stride); y[u] = __ldcs(b + i + u * stride); }
#pragma unroll
        for (int u = 0; u < kUnroll; u++)
            __stcs(out + i + u * stride, make_float4(op(x[u].x, y[u].x), op(x[u].y, y[u].y), op(x[u].z, y[u].z), op(x[u].w, y[u].w)));
    }
    for (; i < nvec; i += stride) {
        float4 x = __ldcs(a + i), y = __ldcs(b + i);
        __stcs(out + i, make_float4(op(x.x, y.x), op(x.y, y.y), op(x.z, y.z), op(x.w, y.w)));
    }
    size_t t = nvec * 4 + (size_t)blockIdx.x * kThreads + threadIdx.x;
    if (blockIdx.x == 0 && t < n) out_s[t] = op(a_s[t], b_s[t]);
}

template <class Op>
__global__ void __launch_bounds__(kThreads) binary_f32_scalar(const float* __restrict__ a, const float* __restrict__ b,
                                                              float* __restrict__ out, size_t n, Op op) {
    size_t stride = (size_t)gridDim.x * kThreads;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) out[i] = op(a[i], b[i]);
}

// bf16 variants: 8 elements per 128-bit vector, math in f32, round-to-nearest-even on store
struct bf16x8 { __nv_bfloat162 v[4]; };

template <class Op>
__global__ void __launch_bounds__(kThreads) unary_bf16_vec(const uint4* __restrict__ a, uint4* __restrict__ out, size_t nvec,
                                                           const __nv_bfloat16* a_s, __nv_bfloat16* out_s, size_t n, Op op) {
    size_t stride = (size_t)gridDim.x * kThreads;
    size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
    for (; i + (kUnroll - 1) * stride < nvec; i += kUnroll * stride) {
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; u++) v[u] = __ldcs(a + i + u * stride);
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            bf16x8 x = *reinterpret_cast<bf16x8*>(&v[u]);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float2 f = bf16x2_to_float2(x.v[j]);
                x.v[j] = __floats2bfloat162_rn(op(f.x), op(f.y));
            }
            __stcs(out + i + u * stride, *reinterpret_cast<uint4*>(&x));
        }
    }
    for (; i < nvec; i += stride) {
        uint4 v = __ldcs(a + i);
        bf16x8 x = *reinterpret_cast<bf16x8*>(&v);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float2 f = bf16x2_to_float2(x.v[j]);
            x.v[j] = __floats2bfloat162_rn(op(f.x), op(f.y));
        }
        __stcs(out + i, *reinterpret_cast<uint4*>(&x));
    }
    size_t t = nvec * 8 + (size_t)blockIdx.x * kThreads + threadIdx.x;
    if (blockIdx.x == 0 && t < n) out_s[t] = __float2bfloat16_rn(op(__bfloat162float(a_s[t])));
}

template <class Op>
__global__ void __launch_bounds__(kThreads) binary_bf16_vec(const uint4* __restrict__ a, const uint4* __restrict__ b,
                                                            uint4* __restrict__ out, size_t nvec, const __nv_bfloat16* a_s,
                                                            const __nv_bfloat16* b_s, __nv_bfloat16* out_s, size_t n, Op op) {
    size_t stride = (size_t)gridDim.x * kThreads;
    size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
    for (; i < nvec; i += stride) {
        uint4 va = __ldcs(a + i), vb = __ldcs(b + i);
        bf16x8 x = *reinterpret_cast<bf16x8*>(&va), y = *reinterpret_cast<bf16x8*>(&vb);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float2 f = bf16x2_to_float2(x.v[j]), g = bf16x2_to_float2(y.v[j]);
            x.v[j] = __floats2bfloat162_rn(op(f.x, g.x), op(f.y, g.y));
        }
        __stcs(out + i, *reinterpret_cast<uint4*>(&x));
    }
    size_t t = nvec * 8 + (size_t)blockIdx.x * kThreads + threadIdx.x;
    if (blockIdx.x == 0 && t < n) out_s[t] = __float2bfloat16_rn(op(__bfloat162float(a_s[t]), __bfloat162float(b_s[t])));
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// grid: enough CTAs to cover the data once with kUnroll vectors per thread, capped at 8 waves of CTAs per SM
static inline int grid_for(size_t nvec) {
    size_t want = (nvec + (size_t)kThreads * kUnroll - 1) / ((size_t)kThreads * kUnroll);
    size_t cap = (size_t)rt().sm_count * 8;
    if (want < 1) want = 1;
    if (want > cap) want = cap;
    // round up to a multiple of the SM count when that does not exceed the work
    size_t sm = rt().sm_count;
    if (want > sm) want = ((want + sm - 1) / sm) * sm;
    return (int)want;
}

template <class Op>
static int run_unary_f32(const void* a, void* out, size_t n, Op op, const char* name) {
    if (enter()) return 1;
    if (n == 0) return 0;
    if (!a || !out) return fail("%s: null handle", name);
    if (aligned16(a) && aligned16(out)) {
        size_t nvec = n / 4;
        unary_f32_vec<Op><<<grid_for(nvec), kThreads, 0, rt().stream>>>((const float4*)a, (float4*)out, nvec, (const float*)a, (float*)out, n, op);
    } else {
        unary_f32_scalar<Op><<<grid_for(n / 4 + 1), kThreads, 0, rt().stream>>>((const float*)a, (float*)out, n, op);
    }
    SPT_LAUNCH_CHECK(name);
    return 0;
}

template <class Op>
static int run_binary_f32(const void* a, const void* b, void* out, size_t n, Op op, const char* name) {
    if (enter()) return 1;
    if (n == 0) return 0;
    if (!a || !b || !out) return fail("%s: null handle", name);
    if (aligned16(a) && aligned16(b) && aligned16(out)) {
        size_t nvec = n / 4;
        binary_f32_vec<Op><<<grid_for(nvec), kThreads, 0, rt().stream>>>((const float4*)a, (const float4*)b, (float4*)out, nvec,
                                                                          (const float*)a, (const float*)b, (float*)out, n, op);
    } else {
        binary_f32_scalar<Op><<<grid_for(n / 4 + 1), kThreads, 0, rt().stream>>>((const float*)a, (const float*)b, (float*)out, n, op);
    }
    SPT_LAUNCH_CHECK(name);
    return 0;
}

template <class Op>
static int run_unary_bf16(const void* a, void* out, size_t n, Op op, const char* name) {
    if (enter()) return 1;
    if (n == 0) return 0;
    if (!a || !out) return fail("%s: null handle", name);
    if (!aligned16(a) || !aligned16(out)) return fail("%s: bf16 buffers must be 16-byte aligned", name);
    size_t nvec = n / 8;
    unary_bf16_vec<Op><<<grid_for(nvec), kThreads, 0, rt().stream>>>((const uint4*)a, (uint4*)out, nvec, (const __nv_bfloat16*)a,
                                                                      (__nv_bfloat16*)out, n, op);
    SPT_LAUNCH_CHECK(name);
    return 0;
}

template <class Op>
static int run_binary_bf16(const void* a, const void* b, void* out, size_t n, Op op, const char* name) {
    if (enter()) return 1;
    if (n == 0) return 0;
    if (!a || !b || !out) return fail("%s: null handle", name);
    if (!aligned16(a) || !aligned16(b) || !aligned16(out)) return fail("%s: bf16 buffers must be 16-byte aligned", name);
    size_t nvec = n / 8;
    binary_bf16_vec<Op><<<grid_for(nvec), kThreads, 0, rt().stream>>>((const uint4*)a, (const uint4*)b, (uint4*)out, nvec,
                                                                       (const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                                       (__nv_bfloat16*)out, n, op);
    SPT_LAUNCH_CHECK(name);
    return 0;
}

// ---- misc KernelProvider kernels ----
__global__ void __launch_bounds__(kThreads) masked_fill_kernel(const float* __restrict__ a, const uint8_t* __restrict__ m,
                                                               float fill, float* __restrict__ out, size_t n) {
    size_t stride = (size_t)gridDim.x * kThreads;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) out[i] = m[i] ? fill : a[i];
}

__global__ void __launch_bounds__(kThreads) broadcast_add_kernel(const float* __restrict__ a, const float* __restrict__ b,
                                                                 float* __restrict__ out, size_t a_len, size_t b_len) {
    size_t stride = (size_t)gridDim.x * kThreads;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < a_len; i += stride) out[i] = a[i] + __ldg(b + (i % b_len));
}

// [rows, b_len] + [b_len] with b_len % 4 == 0: one float4 of a and of b per thread-iteration
__global__ void __launch_bounds__(kThreads) broadcast_add_vec_kernel(const float4* __restrict__ a, const float4* __restrict__ b,
                                                                     float4* __restrict__ out, size_t nvec, size_t bvec) {
    size_t stride = (size_t)gridDim.x * kThreads;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < nvec; i += stride) {
        float4 x = __ldcs(a + i), y = __ldg(b + (i % bvec));
        __stcs(out + i, make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w));
    }
}

// embedding_lookup (crates/hal/src/lib.rs:610-614; bounds rule of crates/core-ops/src/lib.rs:1229):
// one warp per row; a bad id zeroes the row and raises the device status word instead of trapping.
__global__ void __launch_bounds__(kThreads) embedding_f32_kernel(const float* __restrict__ w, const long long* __restrict__ idx,
                                                                 float* __restrict__ out, size_t n_idx, size_t vocab, size_t dim,
                                                                 uint32_t* status) {
    size_t warp = ((size_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
    int lane = threadIdx.x & 31;
    size_t nwarps = ((size_t)gridDim.x * kThreads) >> 5;
    for (size_t r = warp; r < n_idx; r += nwarps) {
        long long id = idx[r];
        bool ok = id >= 0 && (size_t)id < vocab;
        if (!ok && lane == 0) atomicOr(status, 0x100u);
        const float* src = w + (size_t)(ok ? id : 0) * dim;
        float* dst = out + r * dim;
        for (size_t c = lane; c < dim; c += 32) dst[c] = ok ? src[c] : 0.0f;
    }
}

__global__ void __launch_bounds__(kThreads) sgd_kernel(float* __restrict__ p, const float* __restrict__ g, float lr, size_t n) {
    size_t stride = (size_t)gridDim.x * kThreads;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) p[i] = p[i] - lr * g[i];
}

__global__ void __launch_bounds__(kThreads) adam_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
                                                        float* __restrict__ v, size_t n, float lr, float b1, float b2, float eps,
                                                        float wd, float bc1, float bc2) {
    size_t stride = (size_t)gridDim.x * kThreads;
    for (size_t j = (size_t)blockIdx.x * kThreads + threadIdx.x; j < n; j += stride) {
        float pj = p[j], gj = g[j];
        if (wd != 0.0f) pj = __fmul_rn(pj, 1.0f - lr * wd);
        float mj = __fadd_rn(__fmul_rn(b1, m[j]), __fmul_rn(1.0f - b1, gj));
        float vj = __fadd_rn(__fmul_rn(b2, v[j]), __fmul_rn(__fmul_rn(1.0f - b2, gj), gj));
        m[j] = mj; v[j] = vj;
        float mh = mj / bc1, vh = vj / bc2;
        p[j] = pj - __fmul_rn(lr, mh) / (sqrtf(vh) + eps);
    }
}

// sum: two-stage; partials in f32 per block, final pass in f64 on one block (order differs from the
// reference's sequential f32 sum; documented tolerance in the tests)
__global__ void __launch_bounds__(kThreads) sum_partial_kernel(const float* __restrict__ a, size_t n, double* __restrict__ partial) {
    __shared__ double sh[kThreads / 32];
    double acc = 0.0;
    size_t stride = (size_t)gridDim.x * kThreads;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) acc += (double)a[i];
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0.0;
        for (int w = 0; w < kThreads / 32; w++) t += sh[w];
        partial[blockIdx.x] = t;
    }
}
__global__ void sum_final_kernel(const double* __restrict__ partial, int nparts, float* __restrict__ out) {
    double t = 0.0;
    for (int i = 0; i < nparts; i++) t += partial[i];
    *out = (float)t;
}

__global__ void __launch_bounds__(kThreads) f32_to_bf16_kernel(const float* __restrict__ in, __nv_bfloat16* __restrict__ out, size_t n) {
    size_t stride = (size_t)gridDim.x * kThreads;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) out[i] = __float2bfloat16_rn(in[i]);
}
__global__ void __launch_bounds__(kThreads) bf16_to_f32_kernel(const __nv_bfloat16* __restrict__ in, float* __restrict__ out, size_t n) {
    size_t stride = (size_t)gridDim.x * kThreads;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) out[i] = __bfloat162float(in[i]);
}

// [rows, ld] (ld >= cols) -> dense [rows, cols], elements of ES bytes (2 or 4).  The dense matrix is produced in aligned 16-byte
// vectors (its rows need not be: cols may be odd); each vector's elements are fetched one by one from wherever they lie in the
// padded matrix, neighbouring threads reading neighbouring elements.  One HBM pass: rows * cols * ES bytes in and out.
template <typename E>
__global__ void __launch_bounds__(256) compact_rows_kernel(const E* __restrict__ src, E* __restrict__ dst, size_t rows, size_t cols, size_t ld) {
    constexpr int VE = 16 / (int)sizeof(E);
    const size_t total = rows * cols;
    const size_t nvec = total / VE;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) {
        const size_t f = v * VE;
        size_t r = f / cols, c = f - r * cols;
        E e[VE];
#pragma unroll
        for (int i = 0; i < VE; i++) {
            e[i] = src[r * ld + c];
            if (++c == cols) { c = 0; r++; }
        }
        *reinterpret_cast<uint4*>(dst + f) = *reinterpret_cast<const uint4*>(e);
    }
    if (blockIdx.x == 0 && threadIdx.x == 0) {          // the last, partial vector
        for (size_t f = nvec * VE; f < total; f++) { const size_t r = f / cols; dst[f] = src[r * ld + (f - r * cols)]; }
    }
}

int compact_rows_launch(const void* src, void* dst, size_t rows, size_t cols, size_t ld, int es) {
    if (rows == 0 || cols == 0) return 0;
    if (reinterpret_cast<uintptr_t>(dst) & 15) return fail("compact_rows: destination must be 16-byte aligned");
    const int grid = rt().sm_count * 8;
    if (es == 2) compact_rows_kernel<uint16_t><<<grid, 256, 0, rt().stream>>>((const uint16_t*)src, (uint16_t*)dst, rows, cols, ld);
    else compact_rows_kernel<uint32_t><<<grid, 256, 0, rt().stream>>>((const uint32_t*)src, (uint32_t*)dst, rows, cols, ld);
    SPT_LAUNCH_CHECK("compact_rows");
    return 0;
}

}  // namespace spt

using namespace spt;

extern "C" {

int sptorch_add_f32(const void* a, const void* b, void* out, size_t n) { return run_binary_f32(a, b, out, n, OpAdd{}, "add_f32"); }
int sptorch_mul_f32(const void* a, const void* b, void* out, size_t n) { return run_binary_f32(a, b, out, n, OpMul{}, "mul_f32"); }
int sptorch_neg_f32(const void* a, void* out, size_t n) { return run_unary_f32(a, out, n, OpNeg{}, "neg_f32"); }
int sptorch_exp_f32(const void* a, void* out, size_t n) { return run_unary_f32(a, out, n, OpExp{}, "exp_f32"); }
int sptorch_log_f32(const void* a, void* out, size_t n) { return run_unary_f32(a, out, n, OpLog{}, "log_f32"); }
int sptorch_relu_f32(const void* a, void* out, size_t n) { return run_unary_f32(a, out, n, OpRelu{}, "relu_f32"); }
int sptorch_gelu_f32(const void* a, void* out, size_t n) { return run_unary_f32(a, out, n, OpGelu{}, "gelu_f32"); }
int sptorch_scale_f32(const void* a, float s, void* out, size_t n) { return run_unary_f32(a, out, n, OpScale{s}, "scale_f32"); }

int sptorch_ext_add(const void* a, const void* b, void* out, size_t n, int dtype) {
    if (dtype == SPT_F32) return run_binary_f32(a, b, out, n, OpAdd{}, "add");
    if (dtype == SPT_BF16) return run_binary_bf16(a, b, out, n, OpAdd{}, "add_bf16");
    return fail("add: unknown dtype %d", dtype);
}
int sptorch_ext_gelu(const void* a, void* out, size_t n, int dtype) {
    if (dtype == SPT_F32) return run_unary_f32(a, out, n, OpGelu{}, "gelu");
    if (dtype == SPT_BF16) return run_unary_bf16(a, out, n, OpGeluBf16{}, "gelu_bf16");
    return fail("gelu: unknown dtype %d", dtype);
}

int sptorch_ext_swiglu(const void* x, const void* gate, void* out, size_t n, int dtype) {
    if (dtype == SPT_F32) return run_binary_f32(x, gate, out, n, OpSwiglu{}, "swiglu");
    if (dtype == SPT_BF16) return run_binary_bf16(x, gate, out, n, OpSwiglu{}, "swiglu_bf16");
    return fail("swiglu: unknown dtype %d", dtype);
}

int sptorch_ext_masked_fill_f32(const void* a, const void* mask, float fill, void* out, size_t n) {
    if (enter()) return 1;
    if (n == 0) return 0;
    if (!a || !mask || !out) return fail("masked_fill: null handle");
    masked_fill_kernel<<<grid_for(n / 4 + 1), kThreads, 0, rt().stream>>>((const float*)a, (const uint8_t*)mask, fill, (float*)out, n);
    SPT_LAUNCH_CHECK("masked_fill");
    return 0;
}

int sptorch_ext_broadcast_add_f32(const void* a, const void* b, void* out, size_t a_len, size_t b_len) {
    if (enter()) return 1;
    if (a_len == 0) return 0;
    if (!a || !b || !out) return fail("broadcast_add: null handle");
    if (b_len == 0) return fail("broadcast_add: b_len == 0");
    if (a_len % 4 == 0 && b_len % 4 == 0 && aligned16(a) && aligned16(b) && aligned16(out))
        broadcast_add_vec_kernel<<<grid_for(a_len / 4), kThreads, 0, rt().stream>>>((const float4*)a, (const float4*)b, (float4*)out, a_len / 4, b_len / 4);
    else
        broadcast_add_kernel<<<grid_for(a_len / 4 + 1), kThreads, 0, rt().stream>>>((const float*)a, (const float*)b, (float*)out, a_len, b_len);
    SPT_LAUNCH_CHECK("broadcast_add");
    return 0;
}

int sptorch_ext_embedding_lookup_f32(const void* w, const void* idx, void* out, size_t n_idx, size_t vocab, size_t dim) {
    if (enter()) return 1;
    if (n_idx == 0 || dim == 0) return 0;
    if (!w || !idx || !out) return fail("embedding_lookup: null handle");
    size_t blocks = (n_idx * 32 + kThreads - 1) / kThreads;
    size_t cap = (size_t)rt().sm_count * 8;
    embedding_f32_kernel<<<(int)(blocks < cap ? blocks : cap), kThreads, 0, rt().stream>>>((const float*)w, (const long long*)idx, (float*)out,
                                                                                          n_idx, vocab, dim, rt().dev_status);
    SPT_LAUNCH_CHECK("embedding_lookup");
    return 0;
}

int sptorch_ext_sgd_update_f32(void* p, const void* g, float lr, size_t n) {
    if (enter()) return 1;
    if (n == 0) return 0;
    if (!p || !g) return fail("sgd_update: null handle");
    sgd_kernel<<<grid_for(n / 4 + 1), kThreads, 0, rt().stream>>>((float*)p, (const float*)g, lr, n);
    SPT_LAUNCH_CHECK("sgd_update");
    return 0;
}

int sptorch_ext_adam_update_f32(void* p, const void* g, void* m, void* v, size_t n, float lr, float beta1, float beta2,
                                float eps, float weight_decay, float bc1, float bc2) {
    if (enter()) return 1;
    if (n == 0) return 0;
    if (!p || !g || !m || !v) return fail("adam_update: null handle");
    adam_kernel<<<grid_for(n / 4 + 1), kThreads, 0, rt().stream>>>((float*)p, (const float*)g, (float*)m, (float*)v, n, lr, beta1, beta2,
                                                                  eps, weight_decay, bc1, bc2);
    SPT_LAUNCH_CHECK("adam_update");
    return 0;
}

int sptorch_ext_sum_f32(const void* a, size_t n, float* host_result) {
    if (enter()) return 1;
    if (!host_result) return fail("sum: null result pointer");
    if (n == 0) { *host_result = 0.0f; return 0; }
    if (!a) return fail("sum: null handle");
    int blocks = grid_for(n / 4 + 1);
    double* partial = (double*)sptorch_ext_alloc_bytes((size_t)blocks * sizeof(double) + 256);
    if (!partial) return 1;
    float* dres = (float*)(partial + blocks);
    sum_partial_kernel<<<blocks, kThreads, 0, rt().stream>>>((const float*)a, n, partial);
    sum_final_kernel<<<1, 1, 0, rt().stream>>>(partial, blocks, dres);
    cudaError_t e = cudaGetLastError();
    int rc = 0;
    if (e != cudaSuccess) rc = fail("launch of sum failed: %s", cudaGetErrorString(e));
    else rc = sptorch_ext_copy_d2h_bytes(dres, host_result, sizeof(float));
    sptorch_free(partial);
    return rc;
}

int sptorch_ext_f32_to_bf16(const void* in, void* out, size_t n) {
    if (enter()) return 1;
    if (n == 0) return 0;
    if (!in || !out) return fail("f32_to_bf16: null handle");
    f32_to_bf16_kernel<<<grid_for(n / 4 + 1), kThreads, 0, rt().stream>>>((const float*)in, (__nv_bfloat16*)out, n);
    SPT_LAUNCH_CHECK("f32_to_bf16");
    return 0;
}
int sptorch_ext_bf16_to_f32(const void* in, void* out, size_t n) {
    if (enter()) return 1;
    if (n == 0) return 0;
    if (!in || !out) return fail("bf16_to_f32: null handle");
    bf16_to_f32_kernel<<<grid_for(n / 4 + 1), kThreads, 0, rt().stream>>>((const __nv_bfloat16*)in, (float*)out, n);
    SPT_LAUNCH_CHECK("bf16_to_f32");
    return 0;
}

}  // extern "C"
