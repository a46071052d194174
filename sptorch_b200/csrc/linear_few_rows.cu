// linear_few_rows.cu -- Linear for a handful of input rows: C[m, n] = act(alpha * sum_k A[m,k] W[n,k] + bias[n]) (+ / * R[m,n]),
// M <= 64, bf16 operands and output.  This is the shape of every projection of a decode step (M = sequences in flight;
// crates/nn/src/lib.rs:706-760 and 1119-1131 run them once per generated token).
//
// With so few rows the product is a stream over the weight matrix and nothing else: 2 * N * K bytes read once, a few FLOP per
// byte.  The 128-row tcgen05 tiles of gemm.cu put such a problem on N / 256 .. N / 64 SMs (3 to 48 of 148) with a pipeline
// prologue and a TMEM allocation in front of a few microseconds of work; here the weight rows are spread over N / 8 .. N / 32
// CTAs, every warp takes every eighth 32-element slice of K, issues its weight loads (16 bytes per lane, up to eight slices
// in flight) before it touches the activations, and multiplies with mma.sync m16n8k16 -- the tensor unit is idle either way,
// the warp-level instruction needs no allocation and no barrier.  The eight warps' partial sums meet in shared memory and are
// added in warp order (the result does not depend on scheduling).  Where the weight rows alone do not cover the SMs (the
// projections back to the model width: N = d, K up to 4 d) a cluster of 2 or 4 CTAs splits K and the CTAs' sums meet in the
// cluster's first CTA through distributed shared memory, again in a fixed order.  Up to 16 rows the LayerNorm / RMSNorm in front
// of a projection is applied to the rows on the fly; 17 .. 64 rows take norm_few_rows_kernel below as a launch of its own.
//
// k order inside a 32-element slice: lane t of a quad loads the 8 consecutive elements 8t .. 8t+7 of a weight row and of an
// activation row; the first mma takes elements 0..3 of every lane as its k = {2t, 2t+1, 2t+8, 2t+9}, the second elements 4..7.
// A sum over k does not care about the order as long as both operands use the same one.
#include "gemm.h"
#include "epilogue_math.cuh"
#include <cooperative_groups.h>

namespace spt {

namespace {

constexpr int kWarps = 8;
// Row counts up to this take the kernel by default (the limit of its four 16-row groups).  Decode step of a 12-layer, 768-wide
// model, this kernel against 128-row tcgen05 tiles: 32 sequences 0.59 vs 1.00 ms, 48 sequences 0.90 vs 0.93 ms, 64 sequences
// 0.92 vs 0.99 ms -- above 16 rows every CTA re-reads more activation bytes from L2 than it streams weight bytes, and the gap
// closes.
constexpr int kDefaultMaxRows = 64;

__device__ __forceinline__ uint4 ld_stream(const void* p) {     // weights: read once, do not keep in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16_16x8x16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Every CTA normalises all M rows itself: for a few rows that is noise, at 64 rows it cost more than the launch it saves
// (decode step of a 12-layer, 768-wide model at 64 sequences: 2.30 ms with, 1.0 ms without).
constexpr int kNormMaxRows = 16;

// Programmatic dependent launch: a kernel launched with launch_dependent() may start while its predecessor in the stream still
// runs.  pdl_release() lets the successor's CTAs be scheduled as soon as every CTA of this grid has called it (or exited);
// pdl_acquire() returns once the predecessor grid has completed and its writes are visible.  Everything a kernel does before
// pdl_acquire() may only touch memory no earlier kernel of the stream writes (weights); both are no-ops in an ordinary launch.
__device__ __forceinline__ void pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_acquire() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// MT: 16-row groups of A (M <= 16 MT); NT: 8-row groups of W per CTA; S: weight slices a warp has in flight.
// NORM: A holds un-normalised rows; every CTA normalises them itself into shared memory (kind 1: LayerNorm, gamma * ((x - mean) *
// inv) + beta with inv = 1 / sqrt(var + eps); kind 2: RMSNorm, x * inv * gamma with inv = 1 / sqrt(mean(x^2) + eps)), rounded to
// bf16 as the stand-alone kernels store them.  M rows of K values per CTA is little work next to the launch it saves.
template <int MT, int NT, int S, bool NORM>
__global__ void __launch_bounds__(kWarps * 32) linear_few_rows_kernel(const __nv_bfloat16* __restrict__ A, long long lda,
                                                                     const __nv_bfloat16* __restrict__ W, long long ldb,
                                                                     __nv_bfloat16* C, long long ldc, const float* __restrict__ bias,
                                                                     const __nv_bfloat16* R, int M, int N, int K, float alpha, int epilogue,
                                                                     RowNorm nrm, int ksplit) {
    __shared__ float red[kWarps][MT * 16][NT * 8 + 1];
    extern __shared__ __align__(16) uint8_t dyn[];                       // NORM: M rows of (K + 8) bf16
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    // ksplit > 1: a cluster of ksplit CTAs shares the weight rows of one block, CTA r of it takes the r-th part of K
    const int krank = blockIdx.x % ksplit;
    const int n0 = (blockIdx.x / ksplit) * (NT * 8);
    const int all_slices = K >> 5, per_cta = (all_slices + ksplit - 1) / ksplit;
    const int s_lo = krank * per_cta, slices = min(all_slices, s_lo + per_cta);
    pdl_release();

    const __nv_bfloat16* wrow[NT];
#pragma unroll
    for (int j = 0; j < NT; j++) wrow[j] = W + (long long)min(n0 + 8 * j + g, N - 1) * ldb + 8 * t;
    float acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; i++)
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
            for (int q = 0; q < 4; q++) acc[i][j][q] = 0.0f;

    uint4 wv[S][NT];
    auto load_weights = [&](int s0) {
#pragma unroll
        for (int u = 0; u < S; u++) {
            const int s = s0 + u * kWarps;
#pragma unroll
            for (int j = 0; j < NT; j++) wv[u][j] = s < slices ? ld_stream(wrow[j] + 32 * s) : make_uint4(0, 0, 0, 0);
        }
    };
    load_weights(s_lo + warp);       // the weights do not depend on the kernel before this one
    // the output elements this thread finishes at the end: their bias and residual are requested now, not after the reduction
    constexpr int EI = (MT * 16 * NT * 8 + kWarps * 32 - 1) / (kWarps * 32);
    float bpre[EI], rpre[EI];
#pragma unroll
    for (int it = 0; it < EI; it++) {
        const int e = tid + it * kWarps * 32, n = n0 + e % (NT * 8);
        bpre[it] = (bias && e < MT * 16 * NT * 8 && n < N) ? __ldg(bias + n) : 0.0f;
    }
    pdl_acquire();
#pragma unroll
    for (int it = 0; it < EI; it++) {
        const int e = tid + it * kWarps * 32, m = e / (NT * 8), n = n0 + e % (NT * 8);
        rpre[it] = (R && krank == 0 && m < M && n < N) ? __bfloat162float(R[(long long)m * ldc + n]) : 0.0f;
    }

    const long long a_ld = NORM ? (long long)(K + 8) : lda;
    const __nv_bfloat16* a_base = NORM ? reinterpret_cast<const __nv_bfloat16*>(dyn) : A;
    if constexpr (NORM) {
        // Warps are dealt over (row, part of the row): eight rows or more, one warp per row; a single row, eight warps on its eighths.
        // The partial sums of a row's parts meet in shared memory.
        __shared__ float part[kNormMaxRows][kWarps], part2[kNormMaxRows][kWarps];
        const int P = M >= 8 ? 1 : M >= 4 ? 2 : M >= 2 ? 4 : 8, RP = kWarps / P;
        const int my_p = warp % P, my_r = warp / P;
        const int nvec = K >> 3, per = (nvec + P - 1) / P;
        const int c_begin = my_p * per, c_end = min(nvec, c_begin + per);
        const bool ln = nrm.kind == 1;
#pragma unroll 1
        for (int r = my_r; r < M; r += RP) {
            const uint4* src = reinterpret_cast<const uint4*>(A + (long long)r * lda);
            uint4* row = reinterpret_cast<uint4*>(dyn + (size_t)r * (K + 8) * 2);
            float acc1 = 0.0f;                                      // LayerNorm: sum; RMSNorm: sum of squares
            for (int c = c_begin + lane; c < c_end; c += 32) {
                const uint4 d = src[c];
                row[c] = d;
                const uint32_t wd[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float lo = __uint_as_float(wd[j] << 16), hi = __uint_as_float(wd[j] & 0xffff0000u);
                    acc1 += ln ? lo + hi : lo * lo + hi * hi;
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) acc1 += __shfl_xor_sync(0xffffffffu, acc1, o);
            if (lane == 0) part[r][my_p] = acc1;
        }
        if (P == 1) __syncwarp(); else __syncthreads();      // one warp per row: its sums never leave the warp
        if (ln) {
#pragma unroll 1
            for (int r = my_r; r < M; r += RP) {
                float tot = 0.0f;
                for (int q = 0; q < P; q++) tot += part[r][q];
                const float mean = tot / (float)K;
                const uint4* row = reinterpret_cast<const uint4*>(dyn + (size_t)r * (K + 8) * 2);
                float var = 0.0f;                                   // centred second pass over this warp's part of the copy in shared memory
                for (int c = c_begin + lane; c < c_end; c += 32) {
                    const uint4 d = row[c];
                    const uint32_t wd[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float lo = __uint_as_float(wd[j] << 16) - mean, hi = __uint_as_float(wd[j] & 0xffff0000u) - mean;
                        var += lo * lo + hi * hi;
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
                if (lane == 0) part2[r][my_p] = var;
            }
            if (P == 1) __syncwarp(); else __syncthreads();
        }
#pragma unroll 1
        for (int r = my_r; r < M; r += RP) {
            float tot = 0.0f, tot2 = 0.0f;
            for (int q = 0; q < P; q++) { tot += part[r][q]; tot2 += part2[r][q]; }
            const float mean = ln ? tot / (float)K : 0.0f;
            const float inv = 1.0f / sqrtf((ln ? tot2 : tot) / (float)K + nrm.eps);
            uint4* row = reinterpret_cast<uint4*>(dyn + (size_t)r * (K + 8) * 2);
            for (int c = c_begin + lane; c < c_end; c += 32) {
                const uint4 d = row[c];
                const uint32_t wd[4] = {d.x, d.y, d.z, d.w};
                const float4 g0 = __ldg(reinterpret_cast<const float4*>(nrm.gamma + 8 * c)), g1 = __ldg(reinterpret_cast<const float4*>(nrm.gamma + 8 * c + 4));
                const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
                float bb[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                if (ln) {
                    const float4 b0 = __ldg(reinterpret_cast<const float4*>(nrm.beta + 8 * c)), b1 = __ldg(reinterpret_cast<const float4*>(nrm.beta + 8 * c + 4));
                    bb[0] = b0.x; bb[1] = b0.y; bb[2] = b0.z; bb[3] = b0.w; bb[4] = b1.x; bb[5] = b1.y; bb[6] = b1.z; bb[7] = b1.w;
                }
                uint4 o;
                __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float lo = __uint_as_float(wd[j] << 16), hi = __uint_as_float(wd[j] & 0xffff0000u);
                    float y0, y1;
                    if (ln) { y0 = fmaf(gg[2 * j], (lo - mean) * inv, bb[2 * j]); y1 = fmaf(gg[2 * j + 1], (hi - mean) * inv, bb[2 * j + 1]); }
                    else { y0 = lo * inv * gg[2 * j]; y1 = hi * inv * gg[2 * j + 1]; }
                    oh[j] = __floats2bfloat162_rn(y0, y1);
                }
                row[c] = o;
            }
        }
        __syncthreads();
    }

    for (int s0 = s_lo + warp; s0 < slices; s0 += kWarps * S) {
        if (s0 != s_lo + warp) load_weights(s0);
#pragma unroll
        for (int u = 0; u < S; u++) {
            const int s = s0 + u * kWarps;
            if (s >= slices) break;
#pragma unroll
            for (int i = 0; i < MT; i++) {
                const int r0 = 16 * i + g, r1 = r0 + 8;
                uint4 a0 = make_uint4(0, 0, 0, 0), a1 = make_uint4(0, 0, 0, 0);
                if (r0 < M) a0 = *reinterpret_cast<const uint4*>(a_base + (long long)r0 * a_ld + 32 * s + 8 * t);
                if (r1 < M) a1 = *reinterpret_cast<const uint4*>(a_base + (long long)r1 * a_ld + 32 * s + 8 * t);
#pragma unroll
                for (int j = 0; j < NT; j++) {
                    mma_bf16_16x8x16(acc[i][j], a0.x, a1.x, a0.y, a1.y, wv[u][j].x, wv[u][j].y);
                    mma_bf16_16x8x16(acc[i][j], a0.z, a1.z, a0.w, a1.w, wv[u][j].z, wv[u][j].w);
                }
            }
        }
    }

#pragma unroll
    for (int i = 0; i < MT; i++)
#pragma unroll
        for (int j = 0; j < NT; j++) {
            red[warp][16 * i + g][8 * j + 2 * t] = acc[i][j][0];
            red[warp][16 * i + g][8 * j + 2 * t + 1] = acc[i][j][1];
            red[warp][16 * i + g + 8][8 * j + 2 * t] = acc[i][j][2];
            red[warp][16 * i + g + 8][8 * j + 2 * t + 1] = acc[i][j][3];
        }
    __syncthreads();
    float tot[EI];
#pragma unroll
    for (int it = 0; it < EI; it++) {
        const int e = tid + it * kWarps * 32;
        const int m = e / (NT * 8), nn = e % (NT * 8);
        tot[it] = 0.0f;
        if (m < MT * 16) {
            float sum = red[0][m][nn];
#pragma unroll
            for (int w = 1; w < kWarps; w++) sum += red[w][m][nn];
            tot[it] = sum;
        }
    }
    if (ksplit > 1) {
        // the CTAs' sums meet in the cluster's first CTA, read through distributed shared memory and added in rank order
        namespace cg = cooperative_groups;
        cg::cluster_group cluster = cg::this_cluster();
        __syncthreads();                                  // every thread has read red[*] before red[0] is reused
#pragma unroll
        for (int it = 0; it < EI; it++) {
            const int e = tid + it * kWarps * 32;
            if (e < MT * 16 * NT * 8) red[0][e / (NT * 8)][e % (NT * 8)] = tot[it];
        }
        cluster.sync();
        if (krank == 0) {
            for (int r = 1; r < ksplit; r++) {
                const float* other = cluster.map_shared_rank(&red[0][0][0], r);
#pragma unroll
                for (int it = 0; it < EI; it++) {
                    const int e = tid + it * kWarps * 32;
                    if (e < MT * 16 * NT * 8) tot[it] += other[(e / (NT * 8)) * (NT * 8 + 1) + e % (NT * 8)];
                }
            }
        }
        cluster.sync();                                   // no CTA leaves while its shared memory may still be read
        if (krank != 0) return;
    }
#pragma unroll
    for (int it = 0; it < EI; it++) {
        const int e = tid + it * kWarps * 32;
        const int m = e / (NT * 8), nn = e % (NT * 8), n = n0 + nn;
        if (m >= M || n >= N || m >= MT * 16) continue;
        float v = fmaf(tot[it], alpha, bpre[it]);
        if (epilogue == EPI_GELU) v = gelu_fast2(make_float2(v, 0.0f)).x;
        else if (epilogue == EPI_SWIGLU) v = silu_fast(v);
        if (R) v = epilogue == EPI_SWIGLU ? v * rpre[it] : v + rpre[it];
        C[(long long)m * ldc + n] = __float2bfloat16_rn(v);
    }
}

constexpr size_t kNormSmemLimit = 160 * 1024;
size_t norm_smem(const GemmDesc& d) { return (size_t)d.M * (d.K + 8) * 2; }

template <int MT, int NT, bool NORM>
int launch(const GemmDesc& d, const RowNorm& nrm, bool dependent) {
    // Few weight rows and a long K (the projections back to the model width): clusters of 2 or 4 CTAs split K, so that the launch
    // still covers the SMs and a warp's share of K is one round of loads.
    int ksplit = 1;
    if constexpr (!NORM) {
        const long long blocks = ceil_div(d.N, NT * 8);
        while (ksplit < 4 && blocks * ksplit * 2 <= 3ll * rt().sm_count && d.K / (ksplit * 2) >= 32 * kWarps) ksplit *= 2;
    }
    constexpr int S = NT == 1 ? 8 : NT == 2 ? 4 : 2;
    auto kern = linear_few_rows_kernel<MT, NT, S, NORM>;
    const size_t smem = NORM ? norm_smem(d) : 0;
    if constexpr (NORM) {
        static bool granted = false;                                   // per instantiation
        if (!granted) { SPT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kNormSmemLimit)); granted = true; }
    }
    const int grid = ceil_div(d.N, NT * 8) * ksplit;
    SPT_CUDA(launch_dependent(kern, dim3(grid), dim3(kWarps * 32), smem, dependent, ksplit,
                              static_cast<const __nv_bfloat16*>(d.A), d.lda, static_cast<const __nv_bfloat16*>(d.B), d.ldb, static_cast<__nv_bfloat16*>(d.C), d.ldc,
                              d.bias, static_cast<const __nv_bfloat16*>(d.R), d.M, d.N, d.K, d.alpha, d.epilogue, nrm, ksplit));
    note_submit();
    return 0;
}

template <bool NORM>
int dispatch(const GemmDesc& d, const RowNorm& nrm, bool dependent) {
    // CTAs: 8, 16 or 32 weight rows each, the widest that still gives every SM two CTAs (a short kernel: spread first)
    const long long want = 2ll * rt().sm_count;
    const int mt = d.M <= 16 ? 1 : d.M <= 32 ? 2 : 4;
    int nt = 1;
    if (ceil_div(d.N, 16) >= want) nt = 2;
    if (mt <= 2 && ceil_div(d.N, 32) >= want) nt = 4;
    if constexpr (NORM) {            // at most kNormMaxRows = 16 rows: one row group
        return nt == 1 ? launch<1, 1, true>(d, nrm, dependent) : nt == 2 ? launch<1, 2, true>(d, nrm, dependent) : launch<1, 4, true>(d, nrm, dependent);
    } else {
        switch (mt * 10 + nt) {
            case 11: return launch<1, 1, false>(d, nrm, dependent);
            case 12: return launch<1, 2, false>(d, nrm, dependent);
            case 14: return launch<1, 4, false>(d, nrm, dependent);
            case 21: return launch<2, 1, false>(d, nrm, dependent);
            case 22: return launch<2, 2, false>(d, nrm, dependent);
            case 24: return launch<2, 4, false>(d, nrm, dependent);
            case 41: return launch<4, 1, false>(d, nrm, dependent);
            default: return launch<4, 2, false>(d, nrm, dependent);
        }
    }
}

// LayerNorm / RMSNorm of a handful of rows as a launch of its own (17 .. 64 rows, where normalising inside every CTA of the
// projection costs more than it saves): one warp per row, the row in registers, nothing else -- the pipelined kernel of
// rowops.cu spends longer setting up its ring than these rows take.
template <int VMAX>
__global__ void __launch_bounds__(256) norm_few_rows_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, int rows, int K, RowNorm nrm) {
    pdl_release();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r = blockIdx.x * 8 + warp;
    pdl_acquire();
    if (r >= rows) return;
    const int nvec = K >> 3;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)r * K);
    uint4 d[VMAX];
    float sum = 0.0f, sq = 0.0f;
#pragma unroll
    for (int i = 0; i < VMAX; i++) {
        const int c = i * 32 + lane;
        d[i] = c < nvec ? src[c] : make_uint4(0, 0, 0, 0);
        const uint32_t wd[4] = {d[i].x, d[i].y, d[i].z, d[i].w};
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float lo = __uint_as_float(wd[j] << 16), hi = __uint_as_float(wd[j] & 0xffff0000u);
            sum += lo + hi; sq += lo * lo + hi * hi;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { sum += __shfl_xor_sync(0xffffffffu, sum, o); sq += __shfl_xor_sync(0xffffffffu, sq, o); }
    const bool ln = nrm.kind == 1;
    float mean = 0.0f, inv;
    if (ln) {
        mean = sum / (float)K;
        float var = 0.0f;
#pragma unroll
        for (int i = 0; i < VMAX; i++) {
            if (i * 32 + lane < nvec) {
                const uint32_t wd[4] = {d[i].x, d[i].y, d[i].z, d[i].w};
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float lo = __uint_as_float(wd[j] << 16) - mean, hi = __uint_as_float(wd[j] & 0xffff0000u) - mean;
                    var += lo * lo + hi * hi;
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) var += __shfl_xor_sync(0xffffffffu, var, o);
        inv = 1.0f / sqrtf(var / (float)K + nrm.eps);
    } else {
        inv = 1.0f / sqrtf(sq / (float)K + nrm.eps);
    }
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)r * K);
#pragma unroll
    for (int i = 0; i < VMAX; i++) {
        const int c = i * 32 + lane;
        if (c < nvec) {
            const uint32_t wd[4] = {d[i].x, d[i].y, d[i].z, d[i].w};
            const float4 g0 = __ldg(reinterpret_cast<const float4*>(nrm.gamma + 8 * c)), g1 = __ldg(reinterpret_cast<const float4*>(nrm.gamma + 8 * c + 4));
            const float gg[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
            float bb[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            if (ln) {
                const float4 b0 = __ldg(reinterpret_cast<const float4*>(nrm.beta + 8 * c)), b1 = __ldg(reinterpret_cast<const float4*>(nrm.beta + 8 * c + 4));
                bb[0] = b0.x; bb[1] = b0.y; bb[2] = b0.z; bb[3] = b0.w; bb[4] = b1.x; bb[5] = b1.y; bb[6] = b1.z; bb[7] = b1.w;
            }
            uint4 o;
            __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float lo = __uint_as_float(wd[j] << 16), hi = __uint_as_float(wd[j] & 0xffff0000u);
                float y0, y1;
                if (ln) { y0 = fmaf(gg[2 * j], (lo - mean) * inv, bb[2 * j]); y1 = fmaf(gg[2 * j + 1], (hi - mean) * inv, bb[2 * j + 1]); }
                else { y0 = lo * inv * gg[2 * j]; y1 = hi * inv * gg[2 * j + 1]; }
                oh[j] = __floats2bfloat162_rn(y0, y1);
            }
            dst[c] = o;
        }
    }
}

}  // namespace

bool linear_few_rows_supported(const GemmDesc& d) {
    // SPTORCH_B200_FEW_ROWS: the largest row count that takes this kernel (0 = never; experiments)
    static const int max_rows = [] { const char* e = getenv("SPTORCH_B200_FEW_ROWS"); const int v = e ? atoi(e) : kDefaultMaxRows; return v < 0 ? 0 : v > 64 ? 64 : v; }();
    const auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    return d.mode == MM_BF16 && d.out_dtype == BF16 && d.M >= 1 && d.M <= max_rows && d.N >= 1 && d.K >= 32 && d.K % 32 == 0 && d.nb1 * d.nb2 == 1 &&
           !d.causal_lower && !d.causal_k && !d.norm_axis && !d.reduce && d.lda % 8 == 0 && d.ldb % 8 == 0 && d.lda >= d.K && d.ldb >= d.K &&
           d.ldc >= d.N && al16(d.A) && al16(d.B) && d.C != nullptr;
}

bool linear_few_rows_norm_supported(const GemmDesc& d, const RowNorm& nrm) {
    const auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    return linear_few_rows_supported(d) && (nrm.kind == 1 || nrm.kind == 2) && nrm.gamma && al16(nrm.gamma) && (nrm.kind == 2 || (nrm.beta && al16(nrm.beta))) &&
           d.M <= kNormMaxRows && norm_smem(d) <= kNormSmemLimit;
}

bool norm_few_rows_supported(const void* x, const void* out, int rows, int K, const RowNorm& nrm) {
    const auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
    return rows >= 1 && rows <= 64 && K % 8 == 0 && K >= 8 && K <= 8 * 32 * 16 && (nrm.kind == 1 || nrm.kind == 2) && nrm.gamma && al16(nrm.gamma) &&
           (nrm.kind == 2 || (nrm.beta && al16(nrm.beta))) && al16(x) && al16(out);
}

int norm_few_rows(const void* x, void* out, int rows, int K, const RowNorm& nrm, bool dependent) {
    if (!norm_few_rows_supported(x, out, rows, K, nrm)) return fail("norm_few_rows: unsupported problem");
    const int v = ceil_div(K / 8, 32);
    const dim3 grid(ceil_div(rows, 8)), block(256);
    const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
    __nv_bfloat16* op = static_cast<__nv_bfloat16*>(out);
    if (v <= 4) SPT_CUDA(launch_dependent(norm_few_rows_kernel<4>, grid, block, 0, dependent, 1, xp, op, rows, K, nrm));
    else if (v <= 8) SPT_CUDA(launch_dependent(norm_few_rows_kernel<8>, grid, block, 0, dependent, 1, xp, op, rows, K, nrm));
    else SPT_CUDA(launch_dependent(norm_few_rows_kernel<16>, grid, block, 0, dependent, 1, xp, op, rows, K, nrm));
    note_submit();
    return 0;
}

int linear_few_rows(const GemmDesc& d, const RowNorm* nrm, bool dependent) {
    if (nrm && nrm->kind) {
        if (!linear_few_rows_norm_supported(d, *nrm)) return fail("linear_few_rows: unsupported problem (normalised rows)");
        return dispatch<true>(d, *nrm, dependent);
    }
    if (!linear_few_rows_supported(d)) return fail("linear_few_rows: unsupported problem");
    return dispatch<false>(d, RowNorm{}, dependent);
}

}  // namespace spt
