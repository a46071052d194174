// rowops.cu -- HBM-bound row kernels: LayerNorm, row softmax, causal softmax, masked softmax,
// embedding gather + positional add, 2-D transpose.
//
// Common shape: a row (or a pair of rows) lives in the registers of TPR cooperating threads, is read
// from HBM exactly once with 128-bit loads, reduced with warp shuffles (plus one shared-memory hop when
// TPR > 32) and written once with 128-bit stores.  The reference computes all of these on the host
// (crates/nn/src/lib.rs:397-418; crates/core-ops/src/lib.rs:888-935, 1601-1645, 1220-1255, 825-850) and its
// CUDA backend round-trips through the host for them (crates/runtime-cuda/src/lib.rs:302-490).
#include "common.h"
#include "sm100.cuh"
#include <cstdlib>
#include "../../include/sptorch_b200_hal.h"
#include "../../include/sptorch_b200_ext.h"
#include <math.h>

namespace spt {

constexpr int kRowThreads = 256;
constexpr int kRowVecs = 8;        // 128-bit vectors a thread may hold of its row (unused slots are predicated off)

// ---- 128-bit vector access for f32 (4 lanes) and bf16 (8 lanes) ----
template <typename T> struct Vec;
template <> struct Vec<float> {
    static constexpr int N = 4;
    using Raw = float4;
    float v[4];
    __device__ static Raw load_raw(const float* p) { return __ldcs(reinterpret_cast<const float4*>(p)); }
    __device__ static Vec from_raw(Raw t) { return Vec{{t.x, t.y, t.z, t.w}}; }
    __device__ static Vec load(const float* p) { float4 t = __ldcs(reinterpret_cast<const float4*>(p)); return Vec{{t.x, t.y, t.z, t.w}}; }
    __device__ static Vec load_keep(const float* p) { float4 t = __ldg(reinterpret_cast<const float4*>(p)); return Vec{{t.x, t.y, t.z, t.w}}; }
    __device__ void store(float* p) const { __stcs(reinterpret_cast<float4*>(p), make_float4(v[0], v[1], v[2], v[3])); }
};
template <> struct Vec<__nv_bfloat16> {
    static constexpr int N = 8;
    using Raw = uint4;                  // rows are held packed in registers (half the registers of unpacked f32)
    float v[8];
    __device__ static Raw load_raw(const __nv_bfloat16* p) { return __ldcs(reinterpret_cast<const uint4*>(p)); }
    __device__ static Vec from_raw(Raw t) { return unpack(t); }
    __device__ static Vec unpack(uint4 t) {
        Vec r;
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&t);
#pragma unroll
        for (int j = 0; j < 4; j++) { float2 f = bf16x2_to_float2(h[j]); r.v[2 * j] = f.x; r.v[2 * j + 1] = f.y; }
        return r;
    }
    __device__ static Vec load(const __nv_bfloat16* p) { return unpack(__ldcs(reinterpret_cast<const uint4*>(p))); }
    __device__ static Vec load_keep(const __nv_bfloat16* p) { return unpack(__ldg(reinterpret_cast<const uint4*>(p))); }
    __device__ void store(__nv_bfloat16* p) const {
        uint4 t;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&t);
#pragma unroll
        for (int j = 0; j < 4; j++) h[j] = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
        __stcs(reinterpret_cast<uint4*>(p), t);
    }
};

// reduction over the TPR threads that share a row.  TPR <= 32: shuffles only.  TPR > 32: warp
// shuffle, then one value per warp through shared memory (sh holds kRowThreads/32 floats).
template <int TPR, bool IS_MAX>
__device__ __forceinline__ float row_reduce(float x, float* sh) {
    constexpr int W = TPR < 32 ? TPR : 32;
#pragma unroll
    for (int o = W / 2; o > 0; o >>= 1) {
        float y = __shfl_xor_sync(0xffffffffu, x, o);
        x = IS_MAX ? fmaxf(x, y) : x + y;
    }
    if (TPR > 32) {
        constexpr int WPR = TPR / 32;                    // warps per row
        int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        __syncthreads();                                 // previous use of sh is finished
        if (lane == 0) sh[warp] = x;
        __syncthreads();
        int first = (warp / WPR) * WPR;
        float r = sh[first];
#pragma unroll
        for (int w = 1; w < WPR; w++) r = IS_MAX ? fmaxf(r, sh[first + w]) : r + sh[first + w];
        x = r;
    }
    return x;
}

// ---------------- LayerNorm (crates/nn/src/lib.rs:397-418) ----------------
// mean = sum/d; var = sum((x-mean)^2)/d (biased); inv = 1/sqrt(var+eps); y = gamma*((x-mean)*inv)+beta.
// The two sums are tree reductions here, sequential in the reference: results agree to f32 rounding.
// Algorithmic bytes per row: 2*dim*sizeof(T) (+ gamma/beta once per CTA, L2 resident).
template <typename T, int TPR>
__global__ void __launch_bounds__(kRowThreads) layernorm_kernel(const T* __restrict__ x, const float* __restrict__ gamma,
                                                                const float* __restrict__ beta, T* __restrict__ out,
                                                                size_t rows, int dim, float eps) {
    using VT = Vec<T>;
    constexpr int N = VT::N;
    constexpr int V = kRowVecs;
    constexpr int RPB = kRowThreads / TPR;   // rows per CTA pass
    __shared__ float sh[kRowThreads / 32];
    const int t = threadIdx.x % TPR;
    const int rl = threadIdx.x / TPR;
    const int nvec = dim / N;
    // when TPR > 32 every thread of the CTA must take part in the block-wide barrier of row_reduce,
    // so the row loop is uniform per CTA and out-of-range rows are predicated, not skipped.
    for (size_t r0 = (size_t)blockIdx.x * RPB; r0 < rows; r0 += (size_t)gridDim.x * RPB) {
        size_t r = r0 + rl;
        bool live = r < rows;
        const T* xr = x + (live ? r : 0) * (size_t)dim;
        typename VT::Raw d[V];
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < V; i++) {
            int c = i * TPR + t;
            if (live && c < nvec) d[i] = VT::load_raw(xr + c * N);
        }
#pragma unroll
        for (int i = 0; i < V; i++) {
            int c = i * TPR + t;
            if (live && c < nvec) {
                VT u = VT::from_raw(d[i]);
#pragma unroll
                for (int j = 0; j < N; j++) s += u.v[j];
            }
        }
        float mean = row_reduce<TPR, false>(s, sh) / (float)dim;
        float q = 0.0f;
#pragma unroll
        for (int i = 0; i < V; i++) {
            int c = i * TPR + t;
            if (live && c < nvec) {
                VT u = VT::from_raw(d[i]);
#pragma unroll
                for (int j = 0; j < N; j++) { float e = u.v[j] - mean; q += e * e; }
            }
        }
        float var = row_reduce<TPR, false>(q, sh) / (float)dim;
        float inv = 1.0f / sqrtf(var + eps);
        T* yr = out + (live ? r : 0) * (size_t)dim;
#pragma unroll
        for (int i = 0; i < V; i++) {
            int c = i * TPR + t;
            if (live && c < nvec) {
                VT u = VT::from_raw(d[i]);
                VT y;
#pragma unroll
                for (int j4 = 0; j4 < N; j4 += 4) {
                    float4 g = __ldg(reinterpret_cast<const float4*>(gamma + c * N + j4));
                    float4 b = __ldg(reinterpret_cast<const float4*>(beta + c * N + j4));
                    y.v[j4 + 0] = g.x * ((u.v[j4 + 0] - mean) * inv) + b.x;
                    y.v[j4 + 1] = g.y * ((u.v[j4 + 1] - mean) * inv) + b.y;
                    y.v[j4 + 2] = g.z * ((u.v[j4 + 2] - mean) * inv) + b.z;
                    y.v[j4 + 3] = g.w * ((u.v[j4 + 3] - mean) * inv) + b.w;
                }
                y.store(yr + c * N);
            }
        }
    }
}

// bf16 rows, packed arithmetic.  ncu on the generic kernel above with bf16 rows of 768: issue slots 62 % busy, 64 registers
// (4 CTAs per SM), DRAM 40 %: with half the bytes per element the instruction stream, not HBM, sets the pace.  Here the
// three passes work on f32 pairs (add / mul / fma .f32x2), the row stays packed in registers (unpacking a pair is a shift and
// a mask), so a 16-byte vector costs about 60 instructions instead of about 90 at the same register budget.  The output
// multiply-add is fused: one f32 rounding less than gamma * t + beta in two steps, in a value that is then rounded to bf16.
template <int TPR>
__global__ void __launch_bounds__(kRowThreads, 4) layernorm_bf16_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma,
                                                                        const float* __restrict__ beta, __nv_bfloat16* __restrict__ out,
                                                                        size_t rows, int dim, float eps) {
    constexpr int N = 8, V = kRowVecs;
    constexpr int RPB = kRowThreads / TPR;
    __shared__ float sh[kRowThreads / 32];
    const int t = threadIdx.x % TPR;
    const int rl = threadIdx.x / TPR;
    const int nvec = dim / N;
    auto lo = [](uint32_t w) { return __uint_as_float(w << 16); };
    auto hi = [](uint32_t w) { return __uint_as_float(w & 0xffff0000u); };
    for (size_t r0 = (size_t)blockIdx.x * RPB; r0 < rows; r0 += (size_t)gridDim.x * RPB) {
        const size_t r = r0 + rl;
        const bool live = r < rows;
        const __nv_bfloat16* xr = x + (live ? r : 0) * (size_t)dim;
        uint4 d[V];
#pragma unroll
        for (int i = 0; i < V; i++) {
            const int c = i * TPR + t;
            if (live && c < nvec) d[i] = __ldcs(reinterpret_cast<const uint4*>(xr + c * N));
        }
        float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int i = 0; i < V; i++) {
            const int c = i * TPR + t;
            if (live && c < nvec) {
                const uint32_t w[4] = {d[i].x, d[i].y, d[i].z, d[i].w};
#pragma unroll
                for (int j = 0; j < 4; j++) acc = __fadd2_rn(acc, make_float2(lo(w[j]), hi(w[j])));
            }
        }
        const float mean = row_reduce<TPR, false>(acc.x + acc.y, sh) / (float)dim;
        const float2 nmean = make_float2(-mean, -mean);
        float2 qa = make_float2(0.0f, 0.0f);
#pragma unroll
        for (int i = 0; i < V; i++) {
            const int c = i * TPR + t;
            if (live && c < nvec) {
                const uint32_t w[4] = {d[i].x, d[i].y, d[i].z, d[i].w};
#pragma unroll
                for (int j = 0; j < 4; j++) { const float2 e = __fadd2_rn(make_float2(lo(w[j]), hi(w[j])), nmean); qa = __ffma2_rn(e, e, qa); }
            }
        }
        const float var = row_reduce<TPR, false>(qa.x + qa.y, sh) / (float)dim;
        const float inv = 1.0f / sqrtf(var + eps);
        const float2 inv2 = make_float2(inv, inv);
        __nv_bfloat16* yr = out + (live ? r : 0) * (size_t)dim;
#pragma unroll
        for (int i = 0; i < V; i++) {
            const int c = i * TPR + t;
            if (live && c < nvec) {
                const uint32_t w[4] = {d[i].x, d[i].y, d[i].z, d[i].w};
                const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + c * N)), g1 = __ldg(reinterpret_cast<const float4*>(gamma + c * N + 4));
                const float4 b0 = __ldg(reinterpret_cast<const float4*>(beta + c * N)), b1 = __ldg(reinterpret_cast<const float4*>(beta + c * N + 4));
                const float2 g[4] = {make_float2(g0.x, g0.y), make_float2(g0.z, g0.w), make_float2(g1.x, g1.y), make_float2(g1.z, g1.w)};
                const float2 b[4] = {make_float2(b0.x, b0.y), make_float2(b0.z, b0.w), make_float2(b1.x, b1.y), make_float2(b1.z, b1.w)};
                uint4 o;
                __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float2 e = __fadd2_rn(make_float2(lo(w[j]), hi(w[j])), nmean);
                    const float2 y = __ffma2_rn(g[j], __fmul2_rn(e, inv2), b[j]);
                    oh[j] = __floats2bfloat162_rn(y.x, y.y);
                }
                __stcs(reinterpret_cast<uint4*>(yr + c * N), o);
            }
        }
    }
}

// bf16 LayerNorm for rows of 768 / 1024 / 2048 elements with the memory traffic taken off the compute warps.
// The kernel above is bound by load latency (ncu: DRAM 44 %, 7.6 stall cycles on loads per issued instruction): its threads
// load, reduce and store in turn, so a CTA has bytes in flight only part of the time.  Here one CTA per SM runs a ring of
// shared-memory stages: warp 0 streams blocks of rows in with bulk asynchronous copies (rows are contiguous, a block of rows is
// ONE copy of 24..64 KB), sixteen compute warps normalise one row each of a stage in
// place, warp 1 streams finished stages out with bulk stores -- about 190 KB per SM are in flight at every moment, whatever the
// compute warps are doing.  A compute warp owns a whole row (lane l holds the 16-byte vectors l, l + 32, ...), so the two
// reductions are five shuffles each, and for 768-wide rows gamma / beta of the lane's columns stay in registers for the whole
// kernel (wider rows keep them in shared memory).  The kernel is used for every row count, so that a row's result does not depend on
// how many rows are normalised with it.
// Same arithmetic as above (mean, then centred variance, f32 pairs), only the order of the partial sums differs.
template <int VPL, int CW>
__global__ void __launch_bounds__(64 + 32 * CW, 1) layernorm_bf16_async_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma,
                                                                      const float* __restrict__ beta, __nv_bfloat16* __restrict__ out,
                                                                      size_t rows, float eps, int stages, uint32_t* status) {
    using namespace sm100;
    constexpr int DIM = VPL * 256;                 // 32 lanes x VPL vectors x 8 elements
    constexpr int R = CW;                          // rows per stage: one per compute warp
    constexpr uint32_t ROW_BYTES = DIM * 2, STAGE_BYTES = R * ROW_BYTES;
    constexpr bool GB_REGS = VPL <= 3;             // wider rows: the registers go to the row itself
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t base = smem_u32(smem);
    const uint32_t bars = base + stages * STAGE_BYTES;           // full[stages], done[stages], empty[stages]
    const uint32_t full = bars, done = bars + 8 * stages, empty = bars + 16 * stages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + (size_t)stages * STAGE_BYTES + 24 * stages);
    // wider rows: gamma and beta wait in shared memory (8 * DIM bytes) instead of being fetched through L1 for every row
    float* gb = reinterpret_cast<float*>(smem + (size_t)stages * STAGE_BYTES + 256);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if constexpr (!GB_REGS) {
        for (int i = threadIdx.x; i < DIM / 4; i += blockDim.x) {
            reinterpret_cast<float4*>(gb)[i] = __ldg(reinterpret_cast<const float4*>(gamma) + i);
            reinterpret_cast<float4*>(gb + DIM)[i] = __ldg(reinterpret_cast<const float4*>(beta) + i);
        }
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) { mbar_init(full + 8 * s, 1); mbar_init(done + 8 * s, CW); mbar_init(empty + 8 * s, 1); }
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();
    const size_t n_tiles = (rows + R - 1) / R;
    auto tile_bytes = [&](size_t tile) -> uint32_t {
        const size_t left = rows - tile * R;
        return (uint32_t)(left < (size_t)R ? left : (size_t)R) * ROW_BYTES;
    };
    if (warp == 0) {
        // ---- loads ----
        uint32_t i = 0;
        for (size_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, i++) {
            const uint32_t s = i % stages, ph = (i / stages) & 1;
            if (!mbar_wait(empty + 8 * s, ph ^ 1, abort_flag, status, kErrProducerWait)) break;
            if (lane == 0) {
                const uint32_t bytes = tile_bytes(tile);
                mbar_expect_tx(full + 8 * s, bytes);
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(base + s * STAGE_BYTES), "l"(reinterpret_cast<uint64_t>(x + tile * (size_t)R * DIM)), "r"(bytes), "r"(full + 8 * s)
                             : "memory");
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ---- stores ----
        uint32_t i = 0;
        for (size_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, i++) {
            const uint32_t s = i % stages, ph = (i / stages) & 1;
            if (!mbar_wait(done + 8 * s, ph, abort_flag, status, kErrEpilogueWait)) break;
            if (lane == 0) {
                asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                             ::"l"(reinterpret_cast<uint64_t>(out + tile * (size_t)R * DIM)), "r"(base + s * STAGE_BYTES), "r"(tile_bytes(tile))
                             : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");      // the stage has been read: it may be refilled
                mbar_arrive(empty + 8 * s);
            }
            __syncwarp();
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    } else {
        // ---- compute: warp w owns row w of every stage ----
        const int w = warp - 2;
        float2 g[GB_REGS ? VPL * 4 : 1], b[GB_REGS ? VPL * 4 : 1];
        if constexpr (GB_REGS) {
#pragma unroll
            for (int i = 0; i < VPL; i++) {
                const int c = (i * 32 + lane) * 8;
                const float4 g0 = __ldg(reinterpret_cast<const float4*>(gamma + c)), g1 = __ldg(reinterpret_cast<const float4*>(gamma + c + 4));
                const float4 b0 = __ldg(reinterpret_cast<const float4*>(beta + c)), b1 = __ldg(reinterpret_cast<const float4*>(beta + c + 4));
                g[4 * i] = make_float2(g0.x, g0.y); g[4 * i + 1] = make_float2(g0.z, g0.w); g[4 * i + 2] = make_float2(g1.x, g1.y); g[4 * i + 3] = make_float2(g1.z, g1.w);
                b[4 * i] = make_float2(b0.x, b0.y); b[4 * i + 1] = make_float2(b0.z, b0.w); b[4 * i + 2] = make_float2(b1.x, b1.y); b[4 * i + 3] = make_float2(b1.z, b1.w);
            }
        }
        uint32_t i = 0;
        bool ok = true;
        for (size_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, i++) {
            const uint32_t s = i % stages, ph = (i / stages) & 1;
            ok = mbar_wait(full + 8 * s, ph, abort_flag, status, kErrMmaWait);
            if (!ok) break;
            const size_t left = rows - tile * R;
            if ((size_t)w < left) {
                const int lr = w;
                uint8_t* rowp = smem + (size_t)s * STAGE_BYTES + (size_t)lr * ROW_BYTES;
                float2 e[VPL * 4];
                float2 acc = make_float2(0.0f, 0.0f);
#pragma unroll
                for (int v = 0; v < VPL; v++) {
                    const uint4 d = *reinterpret_cast<const uint4*>(rowp + (v * 32 + lane) * 16);
                    const uint32_t wd[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        e[4 * v + j] = make_float2(__uint_as_float(wd[j] << 16), __uint_as_float(wd[j] & 0xffff0000u));
                        acc = __fadd2_rn(acc, e[4 * v + j]);
                    }
                }
                float sum = acc.x + acc.y;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                const float mean = sum / (float)DIM;
                const float2 nmean = make_float2(-mean, -mean);
                float2 qa = make_float2(0.0f, 0.0f);
#pragma unroll
                for (int k = 0; k < VPL * 4; k++) { e[k] = __fadd2_rn(e[k], nmean); qa = __ffma2_rn(e[k], e[k], qa); }
                float sq = qa.x + qa.y;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                const float inv = 1.0f / sqrtf(sq / (float)DIM + eps);
                const float2 inv2 = make_float2(inv, inv);
#pragma unroll
                for (int v = 0; v < VPL; v++) {
                    float2 gg[4], bb[4];
                    if constexpr (GB_REGS) {
#pragma unroll
                        for (int j = 0; j < 4; j++) { gg[j] = g[4 * v + j]; bb[j] = b[4 * v + j]; }
                    } else {
                        const int c = (v * 32 + lane) * 8;
                        const float4 g0 = *reinterpret_cast<const float4*>(gb + c), g1 = *reinterpret_cast<const float4*>(gb + c + 4);
                        const float4 b0 = *reinterpret_cast<const float4*>(gb + DIM + c), b1 = *reinterpret_cast<const float4*>(gb + DIM + c + 4);
                        gg[0] = make_float2(g0.x, g0.y); gg[1] = make_float2(g0.z, g0.w); gg[2] = make_float2(g1.x, g1.y); gg[3] = make_float2(g1.z, g1.w);
                        bb[0] = make_float2(b0.x, b0.y); bb[1] = make_float2(b0.z, b0.w); bb[2] = make_float2(b1.x, b1.y); bb[3] = make_float2(b1.z, b1.w);
                    }
                    uint4 o;
                    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float2 y = __ffma2_rn(gg[j], __fmul2_rn(e[4 * v + j], inv2), bb[j]);
                        oh[j] = __floats2bfloat162_rn(y.x, y.y);
                    }
                    *reinterpret_cast<uint4*>(rowp + (v * 32 + lane) * 16) = o;
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // the rows written above -> visible to the bulk store
            __syncwarp();
            if (lane == 0) mbar_arrive(done + 8 * s);
        }
    }
    __syncthreads();
    if (*abort_flag) {
        // copies that may still be in flight must land before shared memory is released
        unsigned long long t0 = globaltimer();
        while (globaltimer() - t0 < 200000ull) { }
        __syncthreads();
    }
}

template <int VPL, int CW>
static int layernorm_bf16_async_launch(const __nv_bfloat16* x, const float* g, const float* b, __nv_bfloat16* out, size_t rows, float eps) {
    constexpr size_t stage = (size_t)CW * VPL * 256 * 2;
    constexpr size_t gb_bytes = VPL <= 3 ? 0 : (size_t)VPL * 256 * 8;          // gamma and beta in shared memory for the wider rows
    int stages = (int)((216 * 1024 - gb_bytes) / stage);
    if (stages > 8) stages = 8;
    const size_t smem = (size_t)stages * stage + 256 + gb_bytes;
    auto kern = layernorm_bf16_async_kernel<VPL, CW>;
    static bool attr_set = false;
    if (!attr_set) { SPT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); attr_set = true; }
    const size_t tiles = (rows + CW - 1) / CW;
    const int grid = (int)(tiles < (size_t)rt().sm_count ? tiles : (size_t)rt().sm_count);
    kern<<<grid, 64 + 32 * CW, smem, rt().stream>>>(x, g, b, out, rows, eps, stages, rt().dev_status);
    return 0;
}

// Row statistics only: stats[row] = (1/sqrt(var + eps), mean/sqrt(var + eps)), the two numbers a GEMM epilogue needs to apply
// LayerNorm to its un-normalised operand (GemmDesc::norm_axis).  Same mean-then-centred-variance arithmetic as the kernel
// above; reads the rows once and writes 8 bytes per row.
template <typename T, int TPR>
__global__ void __launch_bounds__(kRowThreads) layernorm_stats_kernel(const T* __restrict__ x, float2* __restrict__ stats, size_t rows, int dim, float eps) {
    using VT = Vec<T>;
    constexpr int N = VT::N;
    constexpr int V = kRowVecs;
    constexpr int RPB = kRowThreads / TPR;
    __shared__ float sh[kRowThreads / 32];
    const int t = threadIdx.x % TPR;
    const int rl = threadIdx.x / TPR;
    const int nvec = dim / N;
    for (size_t r0 = (size_t)blockIdx.x * RPB; r0 < rows; r0 += (size_t)gridDim.x * RPB) {
        size_t r = r0 + rl;
        bool live = r < rows;
        const T* xr = x + (live ? r : 0) * (size_t)dim;
        typename VT::Raw d[V];
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < V; i++) {
            int c = i * TPR + t;
            if (live && c < nvec) d[i] = VT::load_raw(xr + c * N);
        }
#pragma unroll
        for (int i = 0; i < V; i++) {
            int c = i * TPR + t;
            if (live && c < nvec) {
                VT u = VT::from_raw(d[i]);
#pragma unroll
                for (int j = 0; j < N; j++) s += u.v[j];
            }
        }
        float mean = row_reduce<TPR, false>(s, sh) / (float)dim;
        float q = 0.0f;
#pragma unroll
        for (int i = 0; i < V; i++) {
            int c = i * TPR + t;
            if (live && c < nvec) {
                VT u = VT::from_raw(d[i]);
#pragma unroll
                for (int j = 0; j < N; j++) { float e = u.v[j] - mean; q += e * e; }
            }
        }
        float var = row_reduce<TPR, false>(q, sh) / (float)dim;
        float inv = 1.0f / sqrtf(var + eps);
        if (live && t == 0) stats[r] = make_float2(inv, mean * inv);
    }
}

// W'[n,k] = W[n,k] * gamma[k] (rounded to T), s[n] = sum_k W'[n,k], c[n] = sum_k beta[k] W[n,k] (+ bias[n]): the constants of a
// Linear that follows a LayerNorm when the normalisation is applied in the GEMM epilogue.  One CTA per output feature n.
template <typename T>
__global__ void __launch_bounds__(256) layernorm_fold_kernel(const T* __restrict__ w, const float* __restrict__ gamma, const float* __restrict__ beta,
                                                             const float* __restrict__ bias, T* __restrict__ wf, float* __restrict__ svec,
                                                             float* __restrict__ cvec, int K) {
    __shared__ float red[2][8];
    const size_t n = blockIdx.x;
    float s = 0.0f, c = 0.0f;
    for (int k = threadIdx.x; k < K; k += blockDim.x) {
        const float wv = (float)w[n * K + k];
        const T folded = (T)(wv * gamma[k]);
        wf[n * K + k] = folded;
        s += (float)folded;                      // the sum of what the tensor cores will actually multiply
        c += beta[k] * wv;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { s += __shfl_xor_sync(0xffffffffu, s, o); c += __shfl_xor_sync(0xffffffffu, c, o); }
    if ((threadIdx.x & 31) == 0) { red[0][threadIdx.x >> 5] = s; red[1][threadIdx.x >> 5] = c; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float st = 0.0f, ct = 0.0f;
        for (int i = 0; i < 8; i++) { st += red[0][i]; ct += red[1][i]; }
        svec[n] = st;
        cvec[n] = ct + (bias ? bias[n] : 0.0f);
    }
}

// any dim (unaligned, or longer than the register path holds): one CTA per row, three passes that hit L1/L2
template <typename T>
__global__ void __launch_bounds__(kRowThreads) layernorm_generic_kernel(const T* __restrict__ x, const float* __restrict__ gamma,
                                                                        const float* __restrict__ beta, T* __restrict__ out,
                                                                        size_t rows, int dim, float eps) {
    __shared__ float sh[kRowThreads / 32];
    for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const T* xr = x + r * (size_t)dim;
        float s = 0.0f;
        for (int c = threadIdx.x; c < dim; c += kRowThreads) s += (float)xr[c];
        float mean = row_reduce<kRowThreads, false>(s, sh) / (float)dim;
        float q = 0.0f;
        for (int c = threadIdx.x; c < dim; c += kRowThreads) { float e = (float)xr[c] - mean; q += e * e; }
        float var = row_reduce<kRowThreads, false>(q, sh) / (float)dim;
        float inv = 1.0f / sqrtf(var + eps);
        T* yr = out + r * (size_t)dim;
        for (int c = threadIdx.x; c < dim; c += kRowThreads) yr[c] = (T)(gamma[c] * (((float)xr[c] - mean) * inv) + beta[c]);
    }
}

// ---------------- row softmax (crates/core-ops/src/lib.rs:903-920; crates/hal/src/lib.rs:582-596) ----------------
template <typename T, int TPR>
__global__ void __launch_bounds__(kRowThreads) softmax_kernel(const T* __restrict__ x, T* __restrict__ out, size_t rows, int cols) {
    using VT = Vec<T>;
    constexpr int N = VT::N;
    constexpr int V = kRowVecs;
    constexpr int RPB = kRowThreads / TPR;
    __shared__ float sh[kRowThreads / 32];
    const int t = threadIdx.x % TPR;
    const int rl = threadIdx.x / TPR;
    const int nvec = cols / N;
    for (size_t r0 = (size_t)blockIdx.x * RPB; r0 < rows; r0 += (size_t)gridDim.x * RPB) {
        size_t r = r0 + rl;
        bool live = r < rows;
        const T* xr = x + (live ? r : 0) * (size_t)cols;
        VT d[V];
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < V; i++) {
            int c = i * TPR + t;
            if (live && c < nvec) {
                d[i] = VT::load(xr + c * N);
#pragma unroll
                for (int j = 0; j < N; j++) mx = fmaxf(mx, d[i].v[j]);
            }
        }
        mx = row_reduce<TPR, true>(mx, sh);
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < V; i++) {
            int c = i * TPR + t;
            if (live && c < nvec) {
#pragma unroll
                for (int j = 0; j < N; j++) { d[i].v[j] = expf(d[i].v[j] - mx); s += d[i].v[j]; }
            }
        }
        s = row_reduce<TPR, false>(s, sh);
        T* yr = out + (live ? r : 0) * (size_t)cols;
        const float uniform = 1.0f / (float)cols;
#pragma unroll
        for (int i = 0; i < V; i++) {
            int c = i * TPR + t;
            if (live && c < nvec) {
#pragma unroll
                for (int j = 0; j < N; j++) d[i].v[j] = (s == 0.0f) ? uniform : d[i].v[j] / s;
                d[i].store(yr + c * N);
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads) softmax_generic_kernel(const T* __restrict__ x, T* __restrict__ out, size_t rows, int cols) {
    __shared__ float sh[kRowThreads / 32];
    for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const T* xr = x + r * (size_t)cols;
        float mx = -INFINITY;
        for (int c = threadIdx.x; c < cols; c += kRowThreads) mx = fmaxf(mx, (float)xr[c]);
        mx = row_reduce<kRowThreads, true>(mx, sh);
        float s = 0.0f;
        for (int c = threadIdx.x; c < cols; c += kRowThreads) s += expf((float)xr[c] - mx);
        s = row_reduce<kRowThreads, false>(s, sh);
        T* yr = out + r * (size_t)cols;
        const float uniform = 1.0f / (float)cols;
        for (int c = threadIdx.x; c < cols; c += kRowThreads) yr[c] = (T)((s == 0.0f) ? uniform : expf((float)xr[c] - mx) / s);
    }
}

// ---------------- causal softmax over scores [batch, T, T] (crates/nn/src/lib.rs:612-632) ----------------
// y[i,j] = softmax_j( scale*x[i,j] for j <= i ; -inf for j > i ).  Only the lower triangle is read;
// the strict upper triangle is written as exact zeros (exp(-inf)/S = 0).  One warp takes the row
// pair (p, T-1-p) so that every warp moves the same number of bytes.
// Algorithmic bytes per [T,T] matrix: (T(T+1)/2 + T^2) * sizeof(T).
template <typename T, int V>
__device__ __forceinline__ void causal_row(const T* __restrict__ xr, T* __restrict__ yr, int i, int Tn, float scale, int lane) {
    using VT = Vec<T>;
    constexpr int N = VT::N;
    const int nvec = Tn / N;
    const int live_vec = i / N + 1;      // vectors holding at least one j <= i
    typename VT::Raw raw[V];             // the row stays packed in registers
#pragma unroll
    for (int k = 0; k < V; k++) {
        int c = k * 32 + lane;
        if (c < live_vec) raw[k] = VT::load_raw(xr + c * N);
    }
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < V; k++) {
        int c = k * 32 + lane;
        if (c < live_vec) {
            VT u = VT::from_raw(raw[k]);
#pragma unroll
            for (int j = 0; j < N; j++) {
                float s = u.v[j] * scale;
                mx = fmaxf(mx, (c * N + j > i) ? -INFINITY : s);
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.0f;
    // exponentials are evaluated once; f32 rows put them back into the registers that held the input,
    // bf16 rows (half as many vectors for the same T) keep them unpacked
    constexpr bool kInPlace = sizeof(T) == 4;
    VT e[kInPlace ? 1 : V];
#pragma unroll
    for (int k = 0; k < V; k++) {
        int c = k * 32 + lane;
        if (c < live_vec) {
            VT u = VT::from_raw(raw[k]);
#pragma unroll
            for (int j = 0; j < N; j++) {
                float s = u.v[j] * scale;
                // bf16 storage: 2^x on the special-function unit (relative error 2^-22, far below a bf16 ulp) keeps the
                // kernel memory bound; f32 storage keeps the precise expf
                float ex;
                if constexpr (sizeof(T) == 2) { asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex) : "f"((s - mx) * 1.4426950408889634f)); }
                else ex = expf(s - mx);
                ex = (c * N + j > i) ? 0.0f : ex;
                u.v[j] = ex; sum += ex;
            }
            if constexpr (kInPlace) raw[k] = *reinterpret_cast<typename VT::Raw*>(&u); else e[k] = u;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv_sum = 1.0f / sum;
#pragma unroll
    for (int k = 0; k < V; k++) {
        int c = k * 32 + lane;
        if (c < nvec) {
            VT y;
            if (c < live_vec) {
                VT u;
                if constexpr (kInPlace) u = VT::from_raw(raw[k]); else u = e[k];
#pragma unroll
                for (int j = 0; j < N; j++) y.v[j] = (sizeof(T) == 2) ? u.v[j] * inv_sum : u.v[j] / sum;
            } else {
#pragma unroll
                for (int j = 0; j < N; j++) y.v[j] = 0.0f;
            }
            y.store(yr + c * N);
        }
    }
}

template <typename T, int V>
__global__ void __launch_bounds__(kRowThreads, sizeof(T) == 4 ? 4 : 3) causal_softmax_kernel(const T* __restrict__ x, T* __restrict__ out, size_t batch,
                                                                     int Tn, float scale) {
    const int lane = threadIdx.x & 31;
    const size_t warp = ((size_t)blockIdx.x * kRowThreads + threadIdx.x) >> 5;
    const size_t nwarps = ((size_t)gridDim.x * kRowThreads) >> 5;
    const int pairs = (Tn + 1) / 2;
    const size_t tasks = batch * (size_t)pairs;
    for (size_t task = warp; task < tasks; task += nwarps) {
        size_t b = task / pairs;
        int p = (int)(task % pairs);
        const T* xb = x + b * (size_t)Tn * Tn;
        T* yb = out + b * (size_t)Tn * Tn;
        // rows p and T-1-p: together T+1 live entries, so every warp moves the same number of bytes
#pragma unroll 1
        for (int half = 0; half < 2; half++) {
            int r = half == 0 ? p : Tn - 1 - p;
            if (half == 1 && r == p) break;
            causal_row<T, V>(xb + (size_t)r * Tn, yb + (size_t)r * Tn, r, Tn, scale, lane);
        }
    }
}

// bf16 causal softmax for T = 256 / 512 / 1024 / 2048 with the memory traffic taken off the compute warps (the structure of
// layernorm_bf16_async_kernel): one CTA per SM, a ring of shared-memory stages of 16 rows; warp 0 streams in, per row, only the
// live prefix (i + 1 scores, rounded up to 16 bytes) with one bulk asynchronous copy each, sixteen compute warps normalise one
// row each in place and fill the dead part with zeros, warp 1 streams whole stages out with one bulk store.  The register
// kernel above reaches 0.65 of the copy bandwidth on bf16 rows (a warp has one or two rows' loads in flight and then computes);
// here the copies of up to ~190 KB per SM are in flight whatever the compute warps do.
// Same arithmetic as causal_row<bf16>: 2^x on the special-function unit, e * (1 / sum).
template <int VPL, int CW>
__global__ void __launch_bounds__(64 + 32 * CW, 1) causal_softmax_bf16_async_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                                                            size_t rows, float scale, int stages, uint32_t* status) {
    using namespace sm100;
    constexpr int T = VPL * 256;                   // 32 lanes x VPL vectors x 8 elements
    constexpr int R = CW;                          // rows per stage: one per compute warp (T is a multiple of R: a stage never spans two matrices)
    constexpr uint32_t ROW_BYTES = T * 2, STAGE_BYTES = R * ROW_BYTES;
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t base = smem_u32(smem);
    const uint32_t bars = base + stages * STAGE_BYTES;           // full[stages], done[stages], empty[stages]
    const uint32_t full = bars, done = bars + 8 * stages, empty = bars + 16 * stages;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + (size_t)stages * STAGE_BYTES + 24 * stages);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; s++) { mbar_init(full + 8 * s, 1); mbar_init(done + 8 * s, CW); mbar_init(empty + 8 * s, 1); }
        *abort_flag = 0;
        fence_barrier_init();
    }
    __syncthreads();
    const size_t n_tiles = (rows + R - 1) / R;
    if (warp == 0) {
        // ---- loads: lane l fetches the live prefix of row l of the stage ----
        uint32_t i = 0;
        for (size_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, i++) {
            const uint32_t s = i % stages, ph = (i / stages) & 1;
            if (!mbar_wait(empty + 8 * s, ph ^ 1, abort_flag, status, kErrProducerWait)) break;
            const size_t r = tile * R + lane;
            const bool live = lane < R && r < rows;
            const uint32_t pos = (uint32_t)(r % T);
            const uint32_t bytes = live ? ((pos + 1) * 2 + 15) & ~15u : 0;
            uint32_t total = bytes;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
            if (lane == 0) mbar_expect_tx(full + 8 * s, total);
            __syncwarp();
            if (live)
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(base + s * STAGE_BYTES + lane * ROW_BYTES), "l"(reinterpret_cast<uint64_t>(x + r * (size_t)T)), "r"(bytes), "r"(full + 8 * s)
                             : "memory");
            __syncwarp();
        }
    } else if (warp == 1) {
        // ---- stores: a stage is one contiguous block of R rows ----
        uint32_t i = 0;
        for (size_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, i++) {
            const uint32_t s = i % stages, ph = (i / stages) & 1;
            if (!mbar_wait(done + 8 * s, ph, abort_flag, status, kErrEpilogueWait)) break;
            if (lane == 0) {
                const size_t left = rows - tile * R;
                const uint32_t bytes = (uint32_t)(left < (size_t)R ? left : (size_t)R) * ROW_BYTES;
                asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                             ::"l"(reinterpret_cast<uint64_t>(out + tile * (size_t)R * T)), "r"(base + s * STAGE_BYTES), "r"(bytes)
                             : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");      // the stage has been read: it may be refilled
                mbar_arrive(empty + 8 * s);
            }
            __syncwarp();
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    } else {
        // ---- compute: warp w owns row w of every stage ----
        const int w = warp - 2;
        uint32_t i = 0;
        bool ok = true;
        for (size_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, i++) {
            const uint32_t s = i % stages, ph = (i / stages) & 1;
            ok = mbar_wait(full + 8 * s, ph, abort_flag, status, kErrMmaWait);
            if (!ok) break;
            const size_t r = tile * R + w;
            if (r < rows) {
                const int pos = (int)(r % T);
                const int live_vec = pos / 8 + 1;
                uint8_t* rowp = smem + (size_t)s * STAGE_BYTES + (size_t)w * ROW_BYTES;
                float e[VPL][8];
                float mx = -INFINITY;
#pragma unroll
                for (int v = 0; v < VPL; v++) {
                    const int c = v * 32 + lane;
                    if (c < live_vec) {
                        const uint4 d = *reinterpret_cast<const uint4*>(rowp + c * 16);
                        const uint32_t wd[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            const float lo = __uint_as_float(wd[j] << 16) * scale, hi = __uint_as_float(wd[j] & 0xffff0000u) * scale;
                            e[v][2 * j] = (c * 8 + 2 * j > pos) ? -INFINITY : lo;
                            e[v][2 * j + 1] = (c * 8 + 2 * j + 1 > pos) ? -INFINITY : hi;
                            mx = fmaxf(mx, fmaxf(e[v][2 * j], e[v][2 * j + 1]));
                        }
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                float sum = 0.0f;
#pragma unroll
                for (int v = 0; v < VPL; v++) {
                    const int c = v * 32 + lane;
                    if (c < live_vec) {
#pragma unroll
                        for (int j = 0; j < 8; j++) {
                            float ex;
                            asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(ex) : "f"((e[v][j] - mx) * 1.4426950408889634f));      // 2^(-inf) = 0 for the dead entries
                            e[v][j] = ex; sum += ex;
                        }
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                const float inv_sum = 1.0f / sum;
#pragma unroll
                for (int v = 0; v < VPL; v++) {
                    const int c = v * 32 + lane;
                    uint4 o = make_uint4(0, 0, 0, 0);
                    if (c < live_vec) {
                        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                        for (int j = 0; j < 4; j++) oh[j] = __floats2bfloat162_rn(e[v][2 * j] * inv_sum, e[v][2 * j + 1] * inv_sum);
                    }
                    *reinterpret_cast<uint4*>(rowp + c * 16) = o;
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");       // the rows written above -> visible to the bulk store
            __syncwarp();
            if (lane == 0) mbar_arrive(done + 8 * s);
        }
    }
    __syncthreads();
    if (*abort_flag) {
        // copies that may still be in flight must land before shared memory is released
        unsigned long long t0 = globaltimer();
        while (globaltimer() - t0 < 200000ull) { }
        __syncthreads();
    }
}

template <int VPL>
static int causal_softmax_bf16_async_launch(const __nv_bfloat16* x, __nv_bfloat16* out, size_t rows, float scale) {
    constexpr int CW = 16;
    constexpr size_t stage = (size_t)CW * VPL * 256 * 2;
    int stages = (int)((216 * 1024) / stage);
    if (stages > 16) stages = 16;
    const size_t smem = (size_t)stages * stage + 512;
    auto kern = causal_softmax_bf16_async_kernel<VPL, CW>;
    static bool attr_set = false;
    if (!attr_set) { SPT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); attr_set = true; }
    const size_t tiles = (rows + CW - 1) / CW;
    const int grid = (int)(tiles < (size_t)rt().sm_count ? tiles : (size_t)rt().sm_count);
    kern<<<grid, 64 + 32 * CW, smem, rt().stream>>>(x, out, rows, scale, stages, rt().dev_status);
    return 0;
}

// any T: CTA per row, scalar accesses
template <typename T>
__global__ void __launch_bounds__(kRowThreads) causal_softmax_generic_kernel(const T* __restrict__ x, T* __restrict__ out,
                                                                             size_t batch, int Tn, float scale) {
    __shared__ float sh[kRowThreads / 32];
    size_t rows = batch * (size_t)Tn;
    for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
        int i = (int)(r % Tn);
        const T* xr = x + r * (size_t)Tn;
        T* yr = out + r * (size_t)Tn;
        float mx = -INFINITY;
        for (int c = threadIdx.x; c <= i; c += kRowThreads) mx = fmaxf(mx, (float)xr[c] * scale);
        mx = row_reduce<kRowThreads, true>(mx, sh);
        float s = 0.0f;
        for (int c = threadIdx.x; c <= i; c += kRowThreads) s += expf((float)xr[c] * scale - mx);
        s = row_reduce<kRowThreads, false>(s, sh);
        for (int c = threadIdx.x; c < Tn; c += kRowThreads) yr[c] = (T)(c <= i ? expf((float)xr[c] * scale - mx) / s : 0.0f);
    }
}

// ---------------- masked_softmax, arbitrary byte mask (crates/core-ops/src/lib.rs:1601-1645) ----------------
// keep != 0: entry takes part.  A row without kept entries stays all zero.  rank1: the 1-D rule (all-zero
// result -> uniform over kept) applies; with one row it can only trigger when the sum underflows.
__global__ void __launch_bounds__(kRowThreads) masked_softmax_kernel(const float* __restrict__ x, const uint8_t* __restrict__ keep,
                                                                     float* __restrict__ out, size_t rows, int cols, int rank1) {
    __shared__ float sh[kRowThreads / 32];
    for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const float* xr = x + r * (size_t)cols;
        const uint8_t* kr = keep + r * (size_t)cols;
        float* yr = out + r * (size_t)cols;
        float mx = -INFINITY, cnt = 0.0f;
        for (int c = threadIdx.x; c < cols; c += kRowThreads) if (kr[c]) { mx = fmaxf(mx, xr[c]); cnt += 1.0f; }
        mx = row_reduce<kRowThreads, true>(mx, sh);
        cnt = row_reduce<kRowThreads, false>(cnt, sh);
        if (mx == -INFINITY) {   // uniform over the CTA: no kept entry (or all kept are -inf)
            for (int c = threadIdx.x; c < cols; c += kRowThreads) yr[c] = (rank1 && kr[c]) ? 1.0f / cnt : 0.0f;
            continue;
        }
        float s = 0.0f;
        for (int c = threadIdx.x; c < cols; c += kRowThreads) if (kr[c]) s += expf(xr[c] - mx);
        s = row_reduce<kRowThreads, false>(s, sh);
        for (int c = threadIdx.x; c < cols; c += kRowThreads) {
            float e = kr[c] ? expf(xr[c] - mx) : 0.0f;
            yr[c] = (kr[c] && s > 0.0f) ? e / s : e;
        }
    }
}

// ---------------- embedding gather + positional add (crates/nn/src/lib.rs:1351-1356) ----------------
// out[t,:] = tok[ids[t],:] + pos[t % T,:].  One warp per token row, 128-bit accesses.  An id outside
// [0, vocab) zeroes the row and raises the device status word (the reference asserts: core-ops/src/lib.rs:1229).
// Algorithmic bytes per token: 2*dim*sizeof(T) + 4 (pos rows are L2 resident).
template <typename T>
__global__ void __launch_bounds__(kRowThreads) embedding_sum_kernel(const T* __restrict__ tok, const T* __restrict__ pos,
                                                                    const int* __restrict__ ids, T* __restrict__ out,
                                                                    size_t n_tokens, int Tn, int vocab, int dim, uint32_t* status,
                                                                    const int* __restrict__ pos_row_dev) {
    using VT = Vec<T>;
    constexpr int N = VT::N;
    const int lane = threadIdx.x & 31;
    // incremental decode replayed as a CUDA graph: every token takes the position row a device word names
    const int fixed_row = pos_row_dev ? *pos_row_dev : -1;
    const size_t warp = ((size_t)blockIdx.x * kRowThreads + threadIdx.x) >> 5;
    const size_t nwarps = ((size_t)gridDim.x * kRowThreads) >> 5;
    const int nvec = dim / N;
    for (size_t t = warp; t < n_tokens; t += nwarps) {
        int id = ids[t];
        bool ok = id >= 0 && id < vocab;
        if (!ok && lane == 0) atomicOr(status, 0x100u);
        const T* a = tok + (size_t)(ok ? id : 0) * dim;
        const T* b = pos ? pos + (size_t)(fixed_row >= 0 ? fixed_row : (int)(t % Tn)) * dim : nullptr;      // no position table: plain gather (RoPE models)
        T* y = out + t * (size_t)dim;
        for (int c = lane; c < nvec; c += 32) {
            VT u = VT::load_keep(a + c * N), r;
            if (b) {
                VT w = VT::load_keep(b + c * N);
#pragma unroll
                for (int j = 0; j < N; j++) r.v[j] = ok ? u.v[j] + w.v[j] : 0.0f;
            } else {
#pragma unroll
                for (int j = 0; j < N; j++) r.v[j] = ok ? u.v[j] : 0.0f;
            }
            r.store(y + c * N);
        }
        for (int c = nvec * N + lane; c < dim; c += 32) y[c] = (T)(ok ? (float)a[c] + (b ? (float)b[c] : 0.0f) : 0.0f);
    }
}

// ---------------- rms_norm (crates/core-ops/src/lib.rs:1453-1475) ----------------
// y = x * (1/sqrt(mean(x^2) + eps)) * w.  Same register-resident row scheme as LayerNorm; one reduction.
template <typename T, int TPR>
__global__ void __launch_bounds__(kRowThreads) rms_norm_kernel(const T* __restrict__ x, const float* __restrict__ w, T* __restrict__ out,
                                                               size_t rows, int dim, float eps) {
    using VT = Vec<T>;
    constexpr int N = VT::N;
    constexpr int V = kRowVecs;
    constexpr int RPB = kRowThreads / TPR;
    __shared__ float sh[kRowThreads / 32];
    const int t = threadIdx.x % TPR;
    const int rl = threadIdx.x / TPR;
    const int nvec = dim / N;
    for (size_t r0 = (size_t)blockIdx.x * RPB; r0 < rows; r0 += (size_t)gridDim.x * RPB) {
        size_t r = r0 + rl;
        bool live = r < rows;
        const T* xr = x + (live ? r : 0) * (size_t)dim;
        typename VT::Raw d[V];
#pragma unroll
        for (int i = 0; i < V; i++) {
            int c = i * TPR + t;
            if (live && c < nvec) d[i] = VT::load_raw(xr + c * N);
        }
        float q = 0.0f;
#pragma unroll
        for (int i = 0; i < V; i++) {
            int c = i * TPR + t;
            if (live && c < nvec) {
                VT u = VT::from_raw(d[i]);
#pragma unroll
                for (int j = 0; j < N; j++) q += u.v[j] * u.v[j];
            }
        }
        float ms = row_reduce<TPR, false>(q, sh) / (float)dim;
        float inv = 1.0f / sqrtf(ms + eps);
        T* yr = out + (live ? r : 0) * (size_t)dim;
#pragma unroll
        for (int i = 0; i < V; i++) {
            int c = i * TPR + t;
            if (live && c < nvec) {
                VT u = VT::from_raw(d[i]);
                VT y;
#pragma unroll
                for (int j4 = 0; j4 < N; j4 += 4) {
                    float4 g = __ldg(reinterpret_cast<const float4*>(w + c * N + j4));
                    y.v[j4 + 0] = u.v[j4 + 0] * inv * g.x; y.v[j4 + 1] = u.v[j4 + 1] * inv * g.y;
                    y.v[j4 + 2] = u.v[j4 + 2] * inv * g.z; y.v[j4 + 3] = u.v[j4 + 3] * inv * g.w;
                }
                y.store(yr + c * N);
            }
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(kRowThreads) rms_norm_generic_kernel(const T* __restrict__ x, const float* __restrict__ w, T* __restrict__ out,
                                                                       size_t rows, int dim, float eps) {
    __shared__ float sh[kRowThreads / 32];
    for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const T* xr = x + r * (size_t)dim;
        float q = 0.0f;
        for (int c = threadIdx.x; c < dim; c += kRowThreads) { float v = (float)xr[c]; q += v * v; }
        float ms = row_reduce<kRowThreads, false>(q, sh) / (float)dim;
        float inv = 1.0f / sqrtf(ms + eps);
        T* yr = out + r * (size_t)dim;
        for (int c = threadIdx.x; c < dim; c += kRowThreads) yr[c] = (T)((float)xr[c] * inv * w[c]);
    }
}

// ---------------- cross_entropy_loss (crates/core-ops/src/lib.rs:1131-1168) ----------------
// Per row: loss = -(x[target] - max - ln(sum exp(x - max))), one pass over the logits with a running (max, sum) pair
// per thread, merged across the CTA.  A row whose target equals the ignore index contributes nothing; a target outside
// [0, classes) raises the device status word (the reference asserts).  Algorithmic bytes: rows * classes * sizeof(T).
template <typename T>
__global__ void __launch_bounds__(kRowThreads) cross_entropy_rows_kernel(const T* __restrict__ logits, long long ld, const long long* __restrict__ targets,
                                                                         size_t rows, int classes, int has_ignore, long long ignore_index,
                                                                         float* __restrict__ row_loss, uint32_t* status) {
    __shared__ float sh[kRowThreads / 32];
    for (size_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const long long tgt = targets[r];
        if (has_ignore && tgt == ignore_index) { if (threadIdx.x == 0) row_loss[r] = -1.0f; continue; }   // marker: not counted
        const bool bad = tgt < 0 || tgt >= classes;
        if (bad) { if (threadIdx.x == 0) { atomicOr(status, 0x100u); row_loss[r] = -1.0f; } continue; }
        const T* x = logits + r * (size_t)ld;
        float m = -INFINITY, s = 0.0f;
        for (int c = threadIdx.x; c < classes; c += kRowThreads) {
            float v = (float)x[c];
            if (v > m) { s = s * expf(m - v) + 1.0f; m = v; } else s += expf(v - m);
        }
        float gm = row_reduce<kRowThreads, true>(m, sh);
        float part = (m == -INFINITY) ? 0.0f : s * expf(m - gm);
        float gs = row_reduce<kRowThreads, false>(part, sh);
        if (threadIdx.x == 0) row_loss[r] = -((float)x[tgt] - gm - logf(gs));
    }
}

__global__ void __launch_bounds__(kRowThreads) cross_entropy_mean_kernel(const float* __restrict__ row_loss, size_t rows, float* __restrict__ out) {
    __shared__ double sd[kRowThreads];
    __shared__ unsigned long long sc[kRowThreads];
    double t = 0.0; unsigned long long n = 0;
    for (size_t r = threadIdx.x; r < rows; r += kRowThreads) { float v = row_loss[r]; if (v >= 0.0f || v != -1.0f) { t += (double)v; n++; } }
    sd[threadIdx.x] = t; sc[threadIdx.x] = n;
    __syncthreads();
    for (int o = kRowThreads / 2; o > 0; o >>= 1) {
        if (threadIdx.x < o) { sd[threadIdx.x] += sd[threadIdx.x + o]; sc[threadIdx.x] += sc[threadIdx.x + o]; }
        __syncthreads();
    }
    if (threadIdx.x == 0) out[0] = sc[0] ? (float)(sd[0] / (double)sc[0]) : 0.0f;
}

// Second stage of the LM head fused with the loss / greedy choice (GemmDesc::reduce wrote, per row, `parts` partial results over
// ascending column ranges): one warp per row merges them into the row's maximum, the column of its FIRST maximum (what a stable
// descending sort puts first: nn/src/lib.rs:2381-2418) and log-sum-exp, and -- when targets are given -- the row's loss
// -(x[target] - max - ln(sum)) with the conventions of cross_entropy_rows_kernel (ignored row: marker -1; bad target: status word).
__global__ void __launch_bounds__(kRowThreads) head_reduce_combine_kernel(const float2* __restrict__ part, const int* __restrict__ arg,
                                                                          const float* __restrict__ tgt_logit, const long long* __restrict__ targets,
                                                                          size_t rows, int parts, int classes, int has_ignore, long long ignore_index,
                                                                          int* __restrict__ argmax_out, float* __restrict__ row_loss, uint32_t* status) {
    const int lane = threadIdx.x & 31;
    const size_t warp0 = ((size_t)blockIdx.x * kRowThreads + threadIdx.x) >> 5, nwarps = ((size_t)gridDim.x * kRowThreads) >> 5;
    for (size_t r = warp0; r < rows; r += nwarps) {
        const float2* pr = part + r * parts;
        float m = -INFINITY; int best = 0x7fffffff;              // (maximum, index of the first partial that attains it)
        for (int i = lane; i < parts; i += 32) { const float v = pr[i].x; if (v > m) { m = v; best = i; } }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float om = __shfl_xor_sync(0xffffffffu, m, o);
            const int ob = __shfl_xor_sync(0xffffffffu, best, o);
            if (om > m || (om == m && ob < best)) { m = om; best = ob; }
        }
        float s = 0.0f;
        for (int i = lane; i < parts; i += 32) { const float2 v = pr[i]; if (v.x != -INFINITY) s += v.y * expf(v.x - m); }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        if (lane == 0) {
            if (argmax_out) argmax_out[r] = best < parts ? arg[r * parts + best] : 0;
            if (row_loss) {
                const long long t = targets[r];
                if (has_ignore && t == ignore_index) row_loss[r] = -1.0f;
                else if (t < 0 || t >= classes) { atomicOr(status, 0x100u); row_loss[r] = -1.0f; }
                else row_loss[r] = -(tgt_logit[r] - m - logf(s));
            }
        }
    }
}

int head_reduce_combine_launch(const float2* part, const int* arg, const float* tgt_logit, const long long* targets, size_t rows, int parts,
                               int classes, int has_ignore, long long ignore_index, int* argmax_out, float* row_loss) {
    if (rows == 0) return 0;
    const size_t warps_per_cta = kRowThreads / 32;
    size_t ctas = (rows + warps_per_cta - 1) / warps_per_cta;
    const size_t cap = (size_t)rt().sm_count * 8;
    if (ctas > cap) ctas = cap;
    head_reduce_combine_kernel<<<(unsigned)ctas, kRowThreads, 0, rt().stream>>>(part, arg, tgt_logit, targets, rows, parts, classes, has_ignore, ignore_index,
                                                                              argmax_out, row_loss, rt().dev_status);
    SPT_LAUNCH_CHECK("head_reduce_combine");
    return 0;
}

// mean of the row losses that are not markers into row_loss[rows] (cross_entropy_loss / _ignore_index: core-ops/src/lib.rs:1079-1194)
int cross_entropy_mean_launch(float* row_loss, size_t rows) {
    cross_entropy_mean_kernel<<<1, kRowThreads, 0, rt().stream>>>(row_loss, rows, row_loss + rows);
    SPT_LAUNCH_CHECK("cross_entropy_mean");
    return 0;
}

// ---------------- transpose (crates/core-ops/src/lib.rs:825-836) ----------------
__global__ void transpose_kernel(const float* __restrict__ a, float* __restrict__ out, int rows, int cols) {
    __shared__ float tile[32][33];
    int bx = blockIdx.x * 32, by = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += 8) {
        int r = by + j, c = bx + threadIdx.x;
        if (r < rows && c < cols) tile[j][threadIdx.x] = a[(size_t)r * cols + c];
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8) {
        int c = bx + j, r = by + threadIdx.x;   // out[c, r]
        if (r < rows && c < cols) out[(size_t)c * rows + r] = tile[threadIdx.x][j];
    }
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// CTAs per SM of the grid-stride row kernels.  Measured on B200 (65536 rows): f32 rows gain from many short-lived CTAs
// (LayerNorm 0.86 / 0.91 / 0.93 of the HBM peak at 8 per SM, 0.90 / 0.94 / 0.98 at 32), bf16 rows lose (0.60 -> 0.56).
static inline int row_grid(size_t row_groups, int per_sm = 8) {
    size_t cap = (size_t)rt().sm_count * per_sm;
    size_t g = row_groups < cap ? row_groups : cap;
    return (int)(g < 1 ? 1 : g);
}

// TPR = the fewest cooperating threads (power of two, 8..256) that hold the row in kRowVecs vectors each: few threads
// per row means many bytes in flight per thread, which is what saturates HBM on short bf16 rows.
#define SPT_ROW_DISPATCH(KERNEL, T, nvec, ...)                                                              \
    do {                                                                                                   \
        int _tpr = 8;                                                                                       \
        while (_tpr * kRowVecs < (nvec)) _tpr *= 2;                                                         \
        int _rpb = kRowThreads / _tpr;                                                                      \
        int _grid = row_grid((rows + _rpb - 1) / _rpb, sizeof(T) == 4 ? 32 : 8);                            \
        switch (_tpr) {                                                                                     \
            case 8: KERNEL<T, 8><<<_grid, kRowThreads, 0, rt().stream>>>(__VA_ARGS__); break;               \
            case 16: KERNEL<T, 16><<<_grid, kRowThreads, 0, rt().stream>>>(__VA_ARGS__); break;             \
            case 32: KERNEL<T, 32><<<_grid, kRowThreads, 0, rt().stream>>>(__VA_ARGS__); break;             \
            case 64: KERNEL<T, 64><<<_grid, kRowThreads, 0, rt().stream>>>(__VA_ARGS__); break;             \
            case 128: KERNEL<T, 128><<<_grid, kRowThreads, 0, rt().stream>>>(__VA_ARGS__); break;           \
            default: KERNEL<T, 256><<<_grid, kRowThreads, 0, rt().stream>>>(__VA_ARGS__); break;            \
        }                                                                                                   \
    } while (0)

template <typename T>
static int layernorm_t(const void* x, const void* gamma, const void* beta, void* out, size_t rows, size_t dim, float eps) {
    constexpr int N = Vec<T>::N;
    const T* xp = (const T*)x; T* op = (T*)out;
    const float* g = (const float*)gamma; const float* b = (const float*)beta;
    bool fast = dim % N == 0 && dim / N <= 2048 && aligned16(x) && aligned16(out) && aligned16(gamma) && aligned16(beta);
    if (fast) {
        int nvec = (int)(dim / N);
        if constexpr (sizeof(T) == 2) {
            // rows of 768 / 1024 / 2048: the pipelined kernel; a 4096-wide row does not fit one warp's registers unpacked and
            // stays with the kernel below
            static const bool async_on = !(getenv("SPTORCH_B200_LN_ASYNC") && getenv("SPTORCH_B200_LN_ASYNC")[0] == '0');
            if (async_on && (dim == 768 || dim == 1024 || dim == 2048)) {
                int rc = dim == 768 ? layernorm_bf16_async_launch<3, 16>(xp, g, b, op, rows, eps)
                       : dim == 1024 ? layernorm_bf16_async_launch<4, 16>(xp, g, b, op, rows, eps)
                                     : layernorm_bf16_async_launch<8, 16>(xp, g, b, op, rows, eps);
                if (rc) return rc;
                SPT_LAUNCH_CHECK("layernorm (pipelined)");
                return 0;
            }
            int tpr = 8;
            while (tpr * kRowVecs < nvec) tpr *= 2;
            const int rpb = kRowThreads / tpr;
            const int grid = row_grid((rows + rpb - 1) / rpb, 4);         // 64 registers: four CTAs per SM are resident
            switch (tpr) {
                case 8: layernorm_bf16_kernel<8><<<grid, kRowThreads, 0, rt().stream>>>(xp, g, b, op, rows, (int)dim, eps); break;
                case 16: layernorm_bf16_kernel<16><<<grid, kRowThreads, 0, rt().stream>>>(xp, g, b, op, rows, (int)dim, eps); break;
                case 32: layernorm_bf16_kernel<32><<<grid, kRowThreads, 0, rt().stream>>>(xp, g, b, op, rows, (int)dim, eps); break;
                case 64: layernorm_bf16_kernel<64><<<grid, kRowThreads, 0, rt().stream>>>(xp, g, b, op, rows, (int)dim, eps); break;
                case 128: layernorm_bf16_kernel<128><<<grid, kRowThreads, 0, rt().stream>>>(xp, g, b, op, rows, (int)dim, eps); break;
                default: layernorm_bf16_kernel<256><<<grid, kRowThreads, 0, rt().stream>>>(xp, g, b, op, rows, (int)dim, eps); break;
            }
        } else {
            SPT_ROW_DISPATCH(layernorm_kernel, T, nvec, xp, g, b, op, rows, (int)dim, eps);
        }
    } else {
        layernorm_generic_kernel<T><<<row_grid(rows), kRowThreads, 0, rt().stream>>>(xp, g, b, op, rows, (int)dim, eps);
    }
    SPT_LAUNCH_CHECK("layernorm");
    return 0;
}

template <typename T>
static int softmax_t(const void* x, void* out, size_t rows, size_t cols) {
    constexpr int N = Vec<T>::N;
    const T* xp = (const T*)x; T* op = (T*)out;
    bool fast = cols % N == 0 && cols / N <= 2048 && aligned16(x) && aligned16(out);
    if (fast) {
        int nvec = (int)(cols / N);
        SPT_ROW_DISPATCH(softmax_kernel, T, nvec, xp, op, rows, (int)cols);
    } else {
        softmax_generic_kernel<T><<<row_grid(rows), kRowThreads, 0, rt().stream>>>(xp, op, rows, (int)cols);
    }
    SPT_LAUNCH_CHECK("softmax");
    return 0;
}

template <typename T>
static int causal_softmax_t(const void* x, void* out, size_t batch, size_t Tn, float scale) {
    constexpr int N = Vec<T>::N;
    const T* xp = (const T*)x; T* op = (T*)out;
    bool fast = Tn % N == 0 && Tn / N <= 256 && aligned16(x) && aligned16(out);
    if constexpr (sizeof(T) == 2) {
        // SPTORCH_B200_SOFTMAX_ASYNC=0 keeps the register kernel (experiments)
        static const bool async_on = [] { const char* e = getenv("SPTORCH_B200_SOFTMAX_ASYNC"); return !(e && e[0] == '0'); }();
        if (fast && async_on && batch * Tn >= 2048 && (Tn == 256 || Tn == 512 || Tn == 1024 || Tn == 2048)) {
            int rc;
            if (Tn == 256) rc = causal_softmax_bf16_async_launch<1>(xp, op, batch * Tn, scale);
            else if (Tn == 512) rc = causal_softmax_bf16_async_launch<2>(xp, op, batch * Tn, scale);
            else if (Tn == 1024) rc = causal_softmax_bf16_async_launch<4>(xp, op, batch * Tn, scale);
            else rc = causal_softmax_bf16_async_launch<8>(xp, op, batch * Tn, scale);
            if (rc) return rc;
            SPT_LAUNCH_CHECK("causal_softmax");
            return 0;
        }
    }
    if (fast) {
        int nvec = (int)(Tn / N);
        int v = (nvec + 31) / 32;
        size_t tasks = batch * ((Tn + 1) / 2);
        int grid = row_grid((tasks + kRowThreads / 32 - 1) / (kRowThreads / 32));
        if (v <= 1) causal_softmax_kernel<T, 1><<<grid, kRowThreads, 0, rt().stream>>>(xp, op, batch, (int)Tn, scale);
        else if (v <= 2) causal_softmax_kernel<T, 2><<<grid, kRowThreads, 0, rt().stream>>>(xp, op, batch, (int)Tn, scale);
        else if (v <= 4) causal_softmax_kernel<T, 4><<<grid, kRowThreads, 0, rt().stream>>>(xp, op, batch, (int)Tn, scale);
        else causal_softmax_kernel<T, 8><<<grid, kRowThreads, 0, rt().stream>>>(xp, op, batch, (int)Tn, scale);
    } else {
        causal_softmax_generic_kernel<T><<<row_grid(batch * Tn), kRowThreads, 0, rt().stream>>>(xp, op, batch, (int)Tn, scale);
    }
    SPT_LAUNCH_CHECK("causal_softmax");
    return 0;
}

// bf16 rows whose length the register path holds; the GPT driver checks `layernorm_stats_supported` before it relies on this
bool layernorm_stats_supported(size_t dim, int dtype) { return dtype == BF16 && dim % 8 == 0 && dim / 8 <= 2048; }
int layernorm_stats_launch(const void* x, float2* stats, size_t rows, size_t dim, float eps, int dtype) {
    if (rows == 0) return 0;
    if (!layernorm_stats_supported(dim, dtype) || !aligned16(x)) return fail("layernorm_stats: unsupported row length, dtype or alignment");
    const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
    const int nvec = (int)(dim / 8);
    const int per_sm = 8;
    int tpr = 8;
    while (tpr * kRowVecs < nvec) tpr *= 2;
    const int rpb = kRowThreads / tpr;
    const int grid = row_grid((rows + rpb - 1) / rpb, per_sm);
    switch (tpr) {
        case 8: layernorm_stats_kernel<__nv_bfloat16, 8><<<grid, kRowThreads, 0, rt().stream>>>(xp, stats, rows, (int)dim, eps); break;
        case 16: layernorm_stats_kernel<__nv_bfloat16, 16><<<grid, kRowThreads, 0, rt().stream>>>(xp, stats, rows, (int)dim, eps); break;
        case 32: layernorm_stats_kernel<__nv_bfloat16, 32><<<grid, kRowThreads, 0, rt().stream>>>(xp, stats, rows, (int)dim, eps); break;
        case 64: layernorm_stats_kernel<__nv_bfloat16, 64><<<grid, kRowThreads, 0, rt().stream>>>(xp, stats, rows, (int)dim, eps); break;
        case 128: layernorm_stats_kernel<__nv_bfloat16, 128><<<grid, kRowThreads, 0, rt().stream>>>(xp, stats, rows, (int)dim, eps); break;
        default: layernorm_stats_kernel<__nv_bfloat16, 256><<<grid, kRowThreads, 0, rt().stream>>>(xp, stats, rows, (int)dim, eps); break;
    }
    SPT_LAUNCH_CHECK("layernorm_stats");
    return 0;
}
int layernorm_fold_launch(const void* w, const float* gamma, const float* beta, const float* bias, void* wf, float* svec, float* cvec,
                          size_t N, size_t K, int dtype) {
    if (N == 0 || K == 0) return 0;
    if (dtype != BF16) return fail("layernorm_fold: bf16 weights only");
    layernorm_fold_kernel<__nv_bfloat16><<<(unsigned)N, 256, 0, rt().stream>>>((const __nv_bfloat16*)w, gamma, beta, bias, (__nv_bfloat16*)wf, svec, cvec, (int)K);
    SPT_LAUNCH_CHECK("layernorm_fold");
    return 0;
}

// used by the GPT driver (same translation-unit-independent entry points as the C-ABI below)
int layernorm_launch(const void* x, const void* gamma, const void* beta, void* out, size_t rows, size_t dim, float eps, int dtype) {
    if (rows == 0 || dim == 0) return 0;
    if (dim > (size_t)INT32_MAX) return fail("layernorm: dim too large");
    return dtype == BF16 ? layernorm_t<__nv_bfloat16>(x, gamma, beta, out, rows, dim, eps)
                         : layernorm_t<float>(x, gamma, beta, out, rows, dim, eps);
}

}  // namespace spt

using namespace spt;

extern "C" {

int sptorch_softmax_f32(const void* a, void* out, size_t rows, size_t cols) {
    if (enter()) return 1;
    if (rows == 0 || cols == 0) return 0;
    if (!a || !out) return fail("softmax_f32: null handle");
    if (cols > (size_t)INT32_MAX) return fail("softmax_f32: cols too large");
    return softmax_t<float>(a, out, rows, cols);
}

int sptorch_ext_layernorm(const void* x, const void* gamma, const void* beta, void* out, size_t rows, size_t dim, float eps, int dtype) {
    if (enter()) return 1;
    if (rows == 0 || dim == 0) return 0;
    if (!x || !gamma || !beta || !out) return fail("layernorm: null handle");
    if (dtype != SPT_F32 && dtype != SPT_BF16) return fail("layernorm: unknown dtype %d", dtype);
    return layernorm_launch(x, gamma, beta, out, rows, dim, eps, dtype);
}

int sptorch_ext_causal_softmax(const void* scores, void* out, size_t batch, size_t T, float scale, int dtype) {
    if (enter()) return 1;
    if (batch == 0 || T == 0) return 0;
    if (!scores || !out) return fail("causal_softmax: null handle");
    if (T > (size_t)1 << 20) return fail("causal_softmax: T too large");
    if (dtype == SPT_F32) return causal_softmax_t<float>(scores, out, batch, T, scale);
    if (dtype == SPT_BF16) return causal_softmax_t<__nv_bfloat16>(scores, out, batch, T, scale);
    return fail("causal_softmax: unknown dtype %d", dtype);
}

int sptorch_ext_masked_softmax_f32(const void* a, const void* keep, void* out, size_t rows, size_t cols, int rank1) {
    if (enter()) return 1;
    if (rows == 0 || cols == 0) return 0;
    if (!a || !keep || !out) return fail("masked_softmax: null handle");
    if (cols > (size_t)INT32_MAX) return fail("masked_softmax: cols too large");
    masked_softmax_kernel<<<row_grid(rows), kRowThreads, 0, rt().stream>>>((const float*)a, (const uint8_t*)keep, (float*)out, rows, (int)cols, rank1);
    SPT_LAUNCH_CHECK("masked_softmax");
    return 0;
}

}  // extern "C"

namespace spt {
// embedding sum with an optional device word that names the position row of every token (decode graphs); else row t % T
int embedding_sum_launch(const void* tok_w, const void* pos_w, const void* ids, void* out, size_t n_tokens, size_t T, size_t vocab, size_t dim,
                         int dtype, const int* pos_row_dev);
}

extern "C" {

int sptorch_ext_embedding_sum(const void* tok_w, const void* pos_w, const void* ids, void* out, size_t n_tokens, size_t T,
                              size_t vocab, size_t dim, int dtype) {
    if (enter()) return 1;
    return spt::embedding_sum_launch(tok_w, pos_w, ids, out, n_tokens, T, vocab, dim, dtype, nullptr);
}

}  // extern "C"

int spt::embedding_sum_launch(const void* tok_w, const void* pos_w, const void* ids, void* out, size_t n_tokens, size_t T, size_t vocab, size_t dim,
                              int dtype, const int* pos_row_dev) {
    if (n_tokens == 0 || dim == 0) return 0;
    if (!tok_w || !ids || !out) return fail("embedding_sum: null handle");     // pos_w may be null: token rows only
    if (T == 0) return fail("embedding_sum: T == 0");
    int grid = row_grid((n_tokens + kRowThreads / 32 - 1) / (kRowThreads / 32));
    if (dtype == SPT_F32) {
        if (dim % 4 || !aligned16(tok_w) || !aligned16(pos_w) || !aligned16(out)) return fail("embedding_sum: dim %% 4 != 0 or unaligned buffers");
        embedding_sum_kernel<float><<<grid, kRowThreads, 0, rt().stream>>>((const float*)tok_w, (const float*)pos_w, (const int*)ids, (float*)out,
                                                                          n_tokens, (int)T, (int)vocab, (int)dim, rt().dev_status, pos_row_dev);
    } else if (dtype == SPT_BF16) {
        if (dim % 8 || !aligned16(tok_w) || !aligned16(pos_w) || !aligned16(out)) return fail("embedding_sum: dim %% 8 != 0 or unaligned buffers");
        embedding_sum_kernel<__nv_bfloat16><<<grid, kRowThreads, 0, rt().stream>>>((const __nv_bfloat16*)tok_w, (const __nv_bfloat16*)pos_w,
                                                                                  (const int*)ids, (__nv_bfloat16*)out, n_tokens, (int)T,
                                                                                  (int)vocab, (int)dim, rt().dev_status, pos_row_dev);
    } else return fail("embedding_sum: unknown dtype %d", dtype);
    SPT_LAUNCH_CHECK("embedding_sum");
    return 0;
}

extern "C" {

int sptorch_ext_rms_norm(const void* x, const void* w, void* out, size_t rows, size_t dim, float eps, int dtype) {
    if (enter()) return 1;
    if (rows == 0 || dim == 0) return 0;
    if (!x || !w || !out) return fail("rms_norm: null handle");
    if (dim > (size_t)INT32_MAX) return fail("rms_norm: dim too large");
    if (dtype != SPT_F32 && dtype != SPT_BF16) return fail("rms_norm: unknown dtype %d", dtype);
    const int N = dtype == SPT_BF16 ? 8 : 4;
    const bool fast = dim % N == 0 && dim / N <= 2048 && aligned16(x) && aligned16(out) && aligned16(w);
    const float* wp = (const float*)w;
    if (dtype == SPT_BF16) {
        const __nv_bfloat16* xp = (const __nv_bfloat16*)x; __nv_bfloat16* op = (__nv_bfloat16*)out;
        if (fast) { int nvec = (int)(dim / N); SPT_ROW_DISPATCH(rms_norm_kernel, __nv_bfloat16, nvec, xp, wp, op, rows, (int)dim, eps); }
        else rms_norm_generic_kernel<__nv_bfloat16><<<row_grid(rows), kRowThreads, 0, rt().stream>>>(xp, wp, op, rows, (int)dim, eps);
    } else {
        const float* xp = (const float*)x; float* op = (float*)out;
        if (fast) { int nvec = (int)(dim / N); SPT_ROW_DISPATCH(rms_norm_kernel, float, nvec, xp, wp, op, rows, (int)dim, eps); }
        else rms_norm_generic_kernel<float><<<row_grid(rows), kRowThreads, 0, rt().stream>>>(xp, wp, op, rows, (int)dim, eps);
    }
    SPT_LAUNCH_CHECK("rms_norm");
    return 0;
}

int sptorch_ext_cross_entropy(const void* logits, size_t ld, const void* targets_i64, size_t rows, size_t classes, int has_ignore,
                              long long ignore_index, void* row_loss_f32, float* host_mean, int dtype) {
    if (enter()) return 1;
    if (!host_mean) return fail("cross_entropy: null result pointer");
    *host_mean = 0.0f;
    if (rows == 0 || classes == 0) return 0;
    if (!logits || !targets_i64 || !row_loss_f32) return fail("cross_entropy: null handle");
    if (ld == 0) ld = classes;
    if (ld < classes || classes > (size_t)INT32_MAX) return fail("cross_entropy: bad row stride or class count");
    if (dtype != SPT_F32 && dtype != SPT_BF16) return fail("cross_entropy: unknown dtype %d", dtype);
    float* rl = (float*)row_loss_f32;                      // rows floats + 1 for the mean
    if (dtype == SPT_BF16)
        cross_entropy_rows_kernel<__nv_bfloat16><<<row_grid(rows), kRowThreads, 0, rt().stream>>>((const __nv_bfloat16*)logits, (long long)ld, (const long long*)targets_i64,
                                                                                                 rows, (int)classes, has_ignore, ignore_index, rl, rt().dev_status);
    else
        cross_entropy_rows_kernel<float><<<row_grid(rows), kRowThreads, 0, rt().stream>>>((const float*)logits, (long long)ld, (const long long*)targets_i64, rows,
                                                                                         (int)classes, has_ignore, ignore_index, rl, rt().dev_status);
    SPT_LAUNCH_CHECK("cross_entropy_rows");
    cross_entropy_mean_kernel<<<1, kRowThreads, 0, rt().stream>>>(rl, rows, rl + rows);
    SPT_LAUNCH_CHECK("cross_entropy_mean");
    return sptorch_ext_copy_d2h_bytes(rl + rows, host_mean, sizeof(float));
}

int sptorch_ext_transpose_f32(const void* a, void* out, size_t rows, size_t cols) {
    if (enter()) return 1;
    if (rows == 0 || cols == 0) return 0;
    if (!a || !out) return fail("transpose: null handle");
    dim3 grid((unsigned)((cols + 31) / 32), (unsigned)((rows + 31) / 32));
    if (grid.y > 65535) return fail("transpose: too many rows for one launch");
    transpose_kernel<<<grid, dim3(32, 8), 0, rt().stream>>>((const float*)a, (float*)out, (int)rows, (int)cols);
    SPT_LAUNCH_CHECK("transpose");
    return 0;
}

}  // extern "C"
