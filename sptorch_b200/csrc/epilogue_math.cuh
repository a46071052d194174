// epilogue_math.cuh -- the activation functions the GEMM epilogues apply, shared by the tcgen05 GEMM and the few-rows Linear
// so that both produce the same bits for the same accumulator value.
#pragma once
#include <cuda_runtime.h>

namespace spt {

__device__ __forceinline__ float gelu_exact(float x) {
    const float k = 0.7978845608028654f;
    float x3 = (x * x) * x;
    return 0.5f * x * (1.0f + tanhf(k * (x + 0.044715f * x3)));
}
// bf16 outputs use tanh.approx (max rel. error 2^-11, far below one bf16 ulp of the result).
// two GELUs at once on packed f32 pairs (fma.rn.f32x2 / mul.rn.f32x2): y = hx + hx * tanh(k x (1 + 0.044715 x^2)), hx = x / 2.
// Six issue slots per pair instead of about sixteen; every instruction of the GELU GEMM's epilogue shows in its time.
__device__ __forceinline__ float2 gelu_fast2(float2 x) {
    // k (x + 0.044715 x^3) = x (k + (0.044715 k) x^2): one packed multiply less
    const float2 kc1 = make_float2(0.044715f * 0.7978845608028654f, 0.044715f * 0.7978845608028654f);
    const float2 k = make_float2(0.7978845608028654f, 0.7978845608028654f), half = make_float2(0.5f, 0.5f);
    float2 w = __ffma2_rn(__fmul2_rn(x, x), kc1, k);
    float2 u = __fmul2_rn(x, w);
    float2 t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t.x) : "f"(u.x));
    asm("tanh.approx.f32 %0, %1;" : "=f"(t.y) : "f"(u.y));
    float2 hx = __fmul2_rn(x, half);
    return __ffma2_rn(hx, t, hx);
}

// e^x through ex2.approx (relative error 2^-22); e^(-inf) = 0
__device__ __forceinline__ float exp_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
    return y;
}

// g * sigmoid(g) (core-ops/src/lib.rs:1537-1538: s = 1 / (1 + exp(-g)), the product with x follows in the caller)
__device__ __forceinline__ float silu_exact(float g) { return g * (1.0f / (1.0f + expf(-g))); }
// bf16 outputs: ex2.approx + rcp.approx, relative error 2^-21, below one bf16 ulp
__device__ __forceinline__ float silu_fast(float g) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * g));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return g * r;
}

}  // namespace spt
