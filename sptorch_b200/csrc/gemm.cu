// gemm.cu -- persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   C[m,n] = act(alpha * sum_k A[m,k] * B[n,k] + bias[n]) + R[m,n]        (both operands K-major)
//
// This is the Linear of the reference (crates/nn/src/lib.rs:121-133): W is consumed in its native
// [out,in] layout as the K-major B operand, so the transpose() copy the reference makes on every call
// (crates/core-ops/src/lib.rs:825-836) does not exist, and the bias add / GELU / residual add that the
// reference runs as separate passes (core-ops/src/lib.rs:1804, 1331, 299) are the epilogue.  It also
// serves the per-head products of attention (core-ops/src/lib.rs:1763-1799) through two batch dims.
//
// Structure of one CTA (320 threads, one CTA per SM, static round-robin over output tiles):
//   warp 0      TMA producer: 128 x BK tile of A and BN x BK tile of B per stage, 128-byte swizzle,
//               4-stage ring, completion on mbarriers (no multicast: every CTA loads its own tiles)
//   warp 1      allocates TMEM, issues tcgen05.mma (M=128, N=BN, K=32 bytes) from one lane; a stage is
//               handed back to the producer by tcgen05.commit; the accumulator (f32, BN columns of
//               TMEM) is double buffered so the epilogue of tile i overlaps the main loop of tile i+1
//   warps 2..9  epilogue: two warps per TMEM lane quarter, each taking half of the tile's 32-column chunks:
//               tcgen05.ld -> alpha/bias/GELU/residual in registers -> packed row into a swizzled 32x32
//               staging block -> one TMA store per chunk (the store clips at the matrix edge)
// Bound: tensor pipe.  Algorithmic work 2*M*N*K FLOP; bytes (M*K + N*K)*s_in + M*N*s_out.
#include "gemm.h"
#include "epilogue_math.cuh"
#include "sm100.cuh"
#include "../../include/sptorch_b200_hal.h"
#include "../../include/sptorch_b200_ext.h"
#include <math.h>
#include <cstdlib>

namespace spt {

using namespace sm100;

constexpr int BM = 128;
constexpr int kStageRowBytes = 128;          // one swizzle row: 64 bf16 or 32 f32 along K
constexpr int kStages = 4;
constexpr int kStagesPair = 6;               // pair kernel: a stage is 32 KB per CTA instead of 48 KB
constexpr int kGemmThreads = 320;           // producer warp + MMA warp + 8 epilogue warps
constexpr int kEpiThreads = 256;
constexpr int kGroupM = 8;                   // default m-tiles per rasterisation band (L2 reuse of the B tiles)
constexpr double kNarrowTileCost = 0.68;     // time of a 128 x 128 tile relative to a 128 x 256 tile of the same K (measured)

struct GemmParams {
    void* C; const float* bias; const void* R;
    int M, N, K;
    long long ldc;
    int nb1, nb2;
    long long sC1, sC2;
    float alpha;
    int epilogue;
    int tiles_m, tiles_n;
    int num_kb;
    int causal_lower;
    int causal_k;
    int b_broadcast;
    int group_m;        // m-tiles per rasterisation band
    int tma_store;      // 1: C is written through the tensor map tmC; 0: element-wise stores
    int r_vec;          // 1: residual rows can be read with 16-byte loads
    uint32_t* status;
};

// LayerNorm folded into the epilogue (see GemmDesc): a kernel argument of its own, read by the NORM variants only
struct NormArgs { const float2* stats; const float* s; };
// row reductions instead of the output (see GemmDesc::reduce): read by the REDUCE variants only
struct ReduceArgs { float2* part; int* arg; const long long* targets; float* tgt; int parts; };

// tile index -> (batch z, m-tile, n-tile): bands of kGroupM m-tiles, n outer / m inner inside a band
__device__ __forceinline__ void decode_tile(int t, int tiles_m, int tiles_n, int group_m, int& z, int& tm, int& tn) {
    int per_batch = tiles_m * tiles_n;
    z = t / per_batch;
    int r = t - z * per_batch;
    int band = r / (group_m * tiles_n);
    int first_m = band * group_m;
    int rows_in_band = min(group_m, tiles_m - first_m);
    int q = r - band * (group_m * tiles_n);
    tn = q / rows_in_band;
    tm = first_m + (q - tn * rows_in_band);
}

// what an epilogue thread keeps per tile for its output row when LayerNorm is folded into the product (nothing otherwise)
template <int NORM> struct NormRow {};
template <> struct NormRow<1> { float2 stat; };

// PAIR: two CTAs of a cluster work on one 256 x BN tile with cta_group::2 MMAs issued by the even CTA.  Each CTA loads its
// own 128 rows of A and its own half (BN/2 rows) of the B tile, keeps its 128 rows of the accumulator in its own TMEM and
// runs its own epilogue; per SM the operand traffic from L2 falls from (128 + BN) to (128 + BN/2) rows per k-block.
// Barriers: `full` lives in the even CTA and counts the bytes of both CTAs' loads; `empty` and `tmem_full` exist in both
// CTAs and are signalled by two commits of the issuing thread; `tmem_empty` lives in the even CTA and collects the
// epilogue threads of both.
template <bool TF32, typename TOut, int BN, bool PAIR, int NORM = 0, bool REDUCE = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const __grid_constant__ CUtensorMap tmC, const GemmParams p, const NormArgs na, const ReduceArgs ra) {
    constexpr int NSTG = PAIR ? kStagesPair : kStages;
    constexpr int TM = PAIR ? 2 * BM : BM;             // rows of one scheduled tile
    constexpr int B_ROWS = PAIR ? BN / 2 : BN;         // rows of B this CTA loads
    constexpr int A_BYTES = BM * kStageRowBytes;
    constexpr int B_BYTES = B_ROWS * kStageRowBytes;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr int BK = TF32 ? 32 : 64;                 // elements of K per stage
    constexpr uint32_t TMEM_COLS = BN <= 64 ? 128 : BN <= 128 ? 256 : 512;   // two accumulators of BN columns; a power of two >= 32
    constexpr uint32_t IDESC = make_idesc(TF32, TM, BN);

    // layout: [kStages x (A tile | B tile)] [8 x 4 KB epilogue staging] [2 x 1 KB bias tiles] [barriers, 256 B]
    // (operand tiles and staging blocks sit on 1024-byte boundaries: the TMA swizzle is a function of the address bits)
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t base = smem_u32(smem);
    if ((base & 1023u) != 0) {           // the 128-byte swizzle pattern must start at row 0 of every tile
        if (threadIdx.x == 0) atomicOr(p.status, 0x200u);
        return;
    }
    constexpr int OFF_STAGING = NSTG * STAGE_BYTES;
    constexpr int OFF_BIAS = OFF_STAGING + 8 * 4096;
    constexpr int OFF_BARS = OFF_BIAS + 2 * 1024;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_BARS);
    // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
    const uint32_t bar_full = base + OFF_BARS;
    const uint32_t bar_empty = bar_full + 8 * NSTG;
    const uint32_t bar_tfull = bar_empty + 8 * NSTG;
    const uint32_t bar_tempty = bar_tfull + 16;
    const uint32_t bar_bias = bar_tempty + 16;           // two barriers: bias tile of even / odd tiles is in place
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * NSTG + 6);
    static_assert(8 * (2 * NSTG + 6) + 8 <= 256, "barrier block overflows");
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;           // 0: the CTA that issues the MMAs
    const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int n_workers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;

    if (threadIdx.x == 0) {
        for (int s = 0; s < NSTG; s++) { mbar_init(bar_full + 8 * s, 1); mbar_init(bar_empty + 8 * s, 1); }
        for (int a = 0; a < 2; a++) {
            mbar_init(bar_tfull + 8 * a, 1); mbar_init(bar_tempty + 8 * a, PAIR ? 2 * kEpiThreads : kEpiThreads);
            mbar_init(bar_bias + 8 * a, kEpiThreads);
        }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) {
        if constexpr (PAIR) { tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish_pair(); }
        else { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    }
    tc_fence_before();
    __syncthreads();
    if constexpr (PAIR) cluster_sync();        // the peer's barriers are initialised before anything is sent to them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int total_tiles = p.tiles_m * p.tiles_n * p.nb1 * p.nb2;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) { tma_prefetch_desc(&tmA); tma_prefetch_desc(&tmB); tma_prefetch_desc(&tmC); }
        int stage = 0; uint32_t phase = 0;
        bool ok = true;
        for (int t = worker; t < total_tiles && ok; t += n_workers) {
            int z, tm, tn;
            decode_tile(t, p.tiles_m, p.tiles_n, p.group_m, z, tm, tn);
            const int m0 = tm * TM + (int)rank * BM, n0 = tn * BN;
            if constexpr (!PAIR) { if (p.causal_lower && n0 > m0 + BM - 1) continue; }
            const int z1 = z % p.nb1, z2 = z / p.nb1;
            const int kb_end = (!PAIR && p.causal_k) ? min(p.num_kb, (m0 + BM + BK - 1) / BK) : p.num_kb;
            for (int kb = 0; kb < kb_end; kb++) {
                ok = mbar_wait(bar_empty + 8 * stage, phase ^ 1, abort_flag, p.status, kErrProducerWait);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t sa = base + stage * STAGE_BYTES;
                    if constexpr (PAIR) {
                        const uint32_t full0 = mapa(bar_full + 8 * stage, 0);
                        if (rank == 0) mbar_expect_tx(bar_full + 8 * stage, 2 * STAGE_BYTES);
                        tma_load_4d_pair(sa, &tmA, full0, kb * BK, m0, z1, z2);
                        tma_load_4d_pair(sa + A_BYTES, &tmB, full0, kb * BK, n0 + (int)rank * B_ROWS, p.b_broadcast ? 0 : z1, p.b_broadcast ? 0 : z2);
                    } else {
                        mbar_expect_tx(bar_full + 8 * stage, STAGE_BYTES);
                        tma_load_4d(sa, &tmA, bar_full + 8 * stage, kb * BK, m0, z1, z2);
                        tma_load_4d(sa + A_BYTES, &tmB, bar_full + 8 * stage, kb * BK, n0, p.b_broadcast ? 0 : z1, p.b_broadcast ? 0 : z2);
                    }
                }
                __syncwarp();
                if (++stage == NSTG) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        int stage = 0; uint32_t phase = 0;
        int acc = 0; uint32_t acc_phase = 0;
        bool ok = rank == 0;                 // the odd CTA of a pair issues nothing: its tiles are driven from the even CTA
        for (int t = worker; t < total_tiles && ok; t += n_workers) {
            int z, tm, tn;
            decode_tile(t, p.tiles_m, p.tiles_n, p.group_m, z, tm, tn);
            if constexpr (!PAIR) { if (p.causal_lower && tn * BN > tm * BM + BM - 1) continue; }
            ok = mbar_wait(bar_tempty + 8 * acc, acc_phase ^ 1, abort_flag, p.status, kErrMmaWait);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * BN;
            const int kb_end = (!PAIR && p.causal_k) ? min(p.num_kb, (tm * BM + BM + BK - 1) / BK) : p.num_kb;
            for (int kb = 0; kb < kb_end; kb++) {
                ok = mbar_wait(bar_full + 8 * stage, phase, abort_flag, p.status, kErrMmaWait);
                if (!ok) break;
                tc_fence_after();
                if (elect_one_sync()) {
                    const uint32_t sa = base + stage * STAGE_BYTES;
                    const uint64_t adesc = make_kmajor_sw128_desc(sa);
                    const uint64_t bdesc = make_kmajor_sw128_desc(sa + A_BYTES);
                    if constexpr (PAIR) {
#pragma unroll
                        for (int k = 0; k < kStageRowBytes / 32; k++)
                            mma_ss_pair<TF32>(d_tmem, adesc + 2 * k, bdesc + 2 * k, IDESC, (kb | k) != 0 ? 1u : 0u);
                        // the stage is handed back to the producers of both CTAs, the finished accumulator to both epilogues
                        mma_commit_pair(mapa(bar_empty + 8 * stage, 0));
                        mma_commit_pair(mapa(bar_empty + 8 * stage, 1));
                        if (kb == kb_end - 1) { mma_commit_pair(mapa(bar_tfull + 8 * acc, 0)); mma_commit_pair(mapa(bar_tfull + 8 * acc, 1)); }
                    } else {
#pragma unroll
                        for (int k = 0; k < kStageRowBytes / 32; k++)
                            mma_ss<TF32>(d_tmem, adesc + 2 * k, bdesc + 2 * k, IDESC, (kb | k) != 0 ? 1u : 0u);
                        mma_commit(bar_empty + 8 * stage);            // stage reusable once these MMAs have read it
                        if (kb == kb_end - 1) mma_commit(bar_tfull + 8 * acc);   // accumulator complete
                    }
                }
                __syncwarp();
                if (++stage == NSTG) { stage = 0; phase ^= 1; }
            }
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
    } else {
        // ---------------- epilogue (warps 2..9; TMEM lane quarter = warp % 4, two warps per quarter) ----------------
        // Only the epilogue's own instruction stream limits it (one warp per scheduler cannot hide a dependent-issue
        // latency), so the work per element is kept small: thread i keeps ROW i of a 32x32 chunk, applies
        // alpha/bias/GELU/residual in place, packs the row and writes it once to a swizzled staging block; one lane
        // then hands the block to the TMA unit, which writes whole rows to HBM and clips at the matrix edge.
        // Loads the epilogue depends on are issued early: the bias slice before the accumulator is waited for, the
        // residual vectors of the next chunk before the current chunk is computed.
        const int ew = warp - 2;                             // 0..7
        const int quarter = warp & 3;
        const int half = ew >> 2;                            // which half of the tile's chunks this warp takes
        const int eidx = threadIdx.x - 64;                   // 0..255 over the epilogue threads
        constexpr int CPW = (BN / 32 + 1) / 2;               // chunks per warp
        constexpr int kOutVec = 16 / (int)sizeof(TOut);      // elements per 16-byte piece
        constexpr int NV = 32 / kOutVec;                     // 16-byte pieces per 32-column row: 4 (bf16) or 8 (f32)
        constexpr int STG_BYTES = 32 * 32 * (int)sizeof(TOut);
        constexpr int NBUF = 4096 / STG_BYTES;               // staging buffers per warp: 2 (bf16) or 1 (f32)
        uint8_t* stg = smem + OFF_STAGING + ew * 4096;
        float* bias_s = reinterpret_cast<float*>(smem + OFF_BIAS);
        const bool use_tma = p.tma_store != 0;
        int acc = 0; uint32_t acc_phase = 0;
        uint32_t chunk_seq = 0;                              // chunks this warp has staged so far (buffer parity)
        uint32_t tile_par = 0, tile_seq = 0;
        bool ok = true;
        const bool has_bias = p.bias != nullptr;
        const bool plain_acc = !has_bias && p.alpha == 1.0f;
        if (!has_bias) {
            bias_s[eidx] = 0.0f; bias_s[256 + eidx] = 0.0f;
            mbar_arrive(bar_bias);
            ok = mbar_wait(bar_bias, 0, abort_flag, p.status, kErrEpilogueWait);
        }
        const uint32_t tempty0 = PAIR ? mapa(bar_tempty, 0) : bar_tempty;     // where a drained accumulator is reported
        auto release_acc = [&](int a) {
            tc_fence_before();
            if constexpr (PAIR) mbar_arrive_cluster(tempty0 + 8 * a); else mbar_arrive(tempty0 + 8 * a);
        };
        for (int t = worker; t < total_tiles && ok; t += n_workers) {
            int z, tm, tn;
            decode_tile(t, p.tiles_m, p.tiles_n, p.group_m, z, tm, tn);
            const int m0 = tm * TM + (int)rank * BM, n0 = tn * BN;
            if constexpr (!PAIR) { if (p.causal_lower && n0 > m0 + BM - 1) continue; }
            const int z1 = z % p.nb1, z2 = z / p.nb1;
            const long long zoff = (long long)z1 * p.sC1 + (long long)z2 * p.sC2;
            TOut* cbase = reinterpret_cast<TOut*>(p.C) + zoff;
            const TOut* rbase = p.R ? reinterpret_cast<const TOut*>(p.R) + zoff : nullptr;
            const int row = m0 + quarter * 32 + lane;        // this thread's output row
            const bool row_ok = row < p.M;
            const int n_chunks = min(BN / 32, (p.N - n0 + 31) / 32);
            const int c_begin = min(half * CPW, n_chunks), c_end = min(c_begin + CPW, n_chunks);
            // bias slice of the tile: one value per epilogue thread, parked in shared memory after the barrier wait
            float bval = 0.0f;
            if (p.bias && eidx < BN && n0 + eidx < p.N) bval = __ldg(p.bias + n0 + eidx);
            // folded LayerNorm: what this thread's output row needs for the whole tile
            NormRow<NORM> nr;
            if constexpr (NORM == 1) { nr.stat = row_ok ? __ldg(na.stats + (long long)z * p.M + row) : make_float2(1.0f, 0.0f); }
            // row reductions: running (maximum, sum of exp(x - maximum)), column of the first maximum, and the target's logit
            float r_mx = -INFINITY, r_s = 0.0f; int r_arg = 0;
            long long r_tgt = -1;
            if constexpr (REDUCE) { if (ra.targets && row_ok) r_tgt = ra.targets[row]; }
            // residual row segment of one chunk (row-per-thread layout)
            uint4 rnext[NV];
            auto fetch_residual = [&](int c) {
                const int col0 = n0 + c * 32;
#pragma unroll
                for (int k = 0; k < NV; k++) rnext[k] = make_uint4(0u, 0u, 0u, 0u);
                if (rbase && row_ok) {
                    const TOut* rp = rbase + (long long)row * p.ldc + col0;
                    if (p.r_vec && col0 + 32 <= p.N) {
#pragma unroll
                        for (int k = 0; k < NV; k++) rnext[k] = *reinterpret_cast<const uint4*>(rp + k * kOutVec);
                    } else {
                        TOut tmp[32];
#pragma unroll
                        for (int j = 0; j < 32; j++) tmp[j] = (col0 + j < p.N) ? rp[j] : (TOut)0.0f;
#pragma unroll
                        for (int k = 0; k < NV; k++) rnext[k] = *reinterpret_cast<const uint4*>(&tmp[k * kOutVec]);
                    }
                }
            };
            if (c_begin < c_end) fetch_residual(c_begin);
            ok = mbar_wait(bar_tfull + 8 * acc, acc_phase, abort_flag, p.status, kErrEpilogueWait);
            if (!ok) break;
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * BN;
            uint32_t v[32];
            if (c_begin < c_end) tmem_ld_32x32(t_row + c_begin * 32, v);
            // publish the bias tile to the 8 epilogue warps (an mbarrier, not bar.sync: its wait is bounded).  Without a bias the
            // tiles were zeroed once before the loop and the eight warps need not meet at every tile.
            if (has_bias) {
                bias_s[tile_par * 256 + eidx] = bval;
                mbar_arrive(bar_bias + 8 * tile_par);
                ok = mbar_wait(bar_bias + 8 * tile_par, (tile_seq >> 1) & 1, abort_flag, p.status, kErrEpilogueWait);
                if (!ok) break;
                tile_seq++;
            }
            const float* bt = bias_s + tile_par * 256;
#pragma unroll 1
            for (int c = c_begin; c < c_end; c++) {
                const int col0 = n0 + c * 32;
                uint4 rcur[NV];
#pragma unroll
                for (int k = 0; k < NV; k++) rcur[k] = rnext[k];
                tmem_ld_wait();
                float f[32];
                if constexpr (NORM == 1) {
                    // y = inv[row] * acc + (c[n] - (mean inv)[row] * s[n]); c sits in the bias tile, s is read through L1 (one address per warp)
                    const float2 inv2 = make_float2(nr.stat.x, nr.stat.x), nmi2 = make_float2(-nr.stat.y, -nr.stat.y);
                    const float* sp = na.s + n0 + c * 32;
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const float4 b4 = *reinterpret_cast<const float4*>(bt + c * 32 + j);
                        const float4 s4 = __ldg(reinterpret_cast<const float4*>(sp + j));       // norm_s is readable up to N rounded up to 32
                        float2 lo = __ffma2_rn(make_float2(__uint_as_float(v[j]), __uint_as_float(v[j + 1])), inv2, __ffma2_rn(nmi2, make_float2(s4.x, s4.y), make_float2(b4.x, b4.y)));
                        float2 hi = __ffma2_rn(make_float2(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])), inv2, __ffma2_rn(nmi2, make_float2(s4.z, s4.w), make_float2(b4.z, b4.w)));
                        f[j] = lo.x; f[j + 1] = lo.y; f[j + 2] = hi.x; f[j + 3] = hi.y;
                    }
                } else if (plain_acc) {
                    // alpha 1, no bias: the accumulator is the value.  Every epilogue instruction shows up in the step time: without
                    // these 16 FMAs and 8 shared-memory loads per chunk the 49 Linear launches of a GPT-2-small-shape forward (three
                    // of five kinds have no bias) take 15.11 instead of 15.40 ms, measured twice in one call
#pragma unroll
                    for (int j = 0; j < 32; j++) f[j] = __uint_as_float(v[j]);
                } else {
                const float2 al2 = make_float2(p.alpha, p.alpha);
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    const float4 b4 = *reinterpret_cast<const float4*>(bt + c * 32 + j);      // same address in every lane: broadcast
                    float2 lo = __ffma2_rn(make_float2(__uint_as_float(v[j]), __uint_as_float(v[j + 1])), al2, make_float2(b4.x, b4.y));
                    float2 hi = __ffma2_rn(make_float2(__uint_as_float(v[j + 2]), __uint_as_float(v[j + 3])), al2, make_float2(b4.z, b4.w));
                    f[j] = lo.x; f[j + 1] = lo.y; f[j + 2] = hi.x; f[j + 3] = hi.y;
                }
                }
                if (c + 1 < c_end) { tmem_ld_32x32(t_row + (c + 1) * 32, v); fetch_residual(c + 1); }
                else release_acc(acc);                                            // this warp has drained its part of the accumulator
                if constexpr (REDUCE) {
                    float cm = -INFINITY; int ca = 0;
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        float x = f[j];
                        if constexpr (sizeof(TOut) == 2) x = __bfloat162float(__float2bfloat16_rn(x));       // the logit as it would be stored
                        if (col0 + j >= p.N) x = -INFINITY;
                        f[j] = x;
                        if (x > cm) { cm = x; ca = j; }
                    }
                    if (cm > r_mx) { r_s *= exp_fast(r_mx - cm); r_mx = cm; r_arg = col0 + ca; }
                    float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
                    for (int j = 0; j < 32; j += 2) { s0 += exp_fast(f[j] - r_mx); s1 += exp_fast(f[j + 1] - r_mx); }
                    r_s += s0 + s1;
                    const long long tj = r_tgt - col0;
                    if (tj >= 0 && tj < 32) {
                        float tv = 0.0f;
#pragma unroll
                        for (int j = 0; j < 32; j++) if (j == (int)tj) tv = f[j];
                        ra.tgt[row] = tv;
                    }
                    continue;
                }
                if (p.epilogue == EPI_GELU) {
                    if constexpr (sizeof(TOut) == 2) {
#pragma unroll
                        for (int j = 0; j < 32; j += 2) { float2 y = gelu_fast2(make_float2(f[j], f[j + 1])); f[j] = y.x; f[j + 1] = y.y; }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; j++) f[j] = gelu_exact(f[j]);
                    }
                } else if (p.epilogue == EPI_SWIGLU) {
#pragma unroll
                    for (int j = 0; j < 32; j++) f[j] = sizeof(TOut) == 2 ? silu_fast(f[j]) : silu_exact(f[j]);
                }
                if (rbase && p.epilogue == EPI_SWIGLU) {
                    // the R operand is the other factor: x * (g * sigmoid(g))
                    if constexpr (sizeof(TOut) == 2) {
#pragma unroll
                        for (int k = 0; k < NV; k++) {
                            const __nv_bfloat162* rh = reinterpret_cast<const __nv_bfloat162*>(&rcur[k]);
#pragma unroll
                            for (int q = 0; q < 4; q++) {
                                const uint32_t rw = *reinterpret_cast<const uint32_t*>(&rh[q]);
                                const float2 pr2 = __fmul2_rn(make_float2(f[8 * k + 2 * q], f[8 * k + 2 * q + 1]),
                                                              make_float2(__uint_as_float(rw << 16), __uint_as_float(rw & 0xffff0000u)));
                                f[8 * k + 2 * q] = pr2.x; f[8 * k + 2 * q + 1] = pr2.y;
                            }
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < NV; k++) {
                            f[4 * k] *= __uint_as_float(rcur[k].x); f[4 * k + 1] *= __uint_as_float(rcur[k].y);
                            f[4 * k + 2] *= __uint_as_float(rcur[k].z); f[4 * k + 3] *= __uint_as_float(rcur[k].w);
                        }
                    }
                } else if (rbase) {
                    if constexpr (sizeof(TOut) == 2) {
#pragma unroll
                        for (int k = 0; k < NV; k++) {
                            const __nv_bfloat162* rh = reinterpret_cast<const __nv_bfloat162*>(&rcur[k]);
#pragma unroll
                            for (int q = 0; q < 4; q++) {
                                // bf16 pair -> f32 pair is a shift and a mask; one packed add per pair
                                const uint32_t rw = *reinterpret_cast<const uint32_t*>(&rh[q]);
                                const float2 sum2 = __fadd2_rn(make_float2(f[8 * k + 2 * q], f[8 * k + 2 * q + 1]),
                                                               make_float2(__uint_as_float(rw << 16), __uint_as_float(rw & 0xffff0000u)));
                                f[8 * k + 2 * q] = sum2.x; f[8 * k + 2 * q + 1] = sum2.y;
                            }
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < NV; k++) {
                            const float2 lo2 = __fadd2_rn(make_float2(f[4 * k], f[4 * k + 1]), make_float2(__uint_as_float(rcur[k].x), __uint_as_float(rcur[k].y)));
                            const float2 hi2 = __fadd2_rn(make_float2(f[4 * k + 2], f[4 * k + 3]), make_float2(__uint_as_float(rcur[k].z), __uint_as_float(rcur[k].w)));
                            f[4 * k] = lo2.x; f[4 * k + 1] = lo2.y; f[4 * k + 2] = hi2.x; f[4 * k + 3] = hi2.y;
                        }
                    }
                }
                if (use_tma) {
                    uint8_t* buf = stg + (chunk_seq % NBUF) * STG_BYTES;
                    // the store that last read this buffer must have finished reading it
                    if (lane == 0) {
                        if (NBUF == 2) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
                        else asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    }
                    __syncwarp();
                    // row `lane` of the block; 16-byte piece k goes to the position the tensor map's swizzle expects
                    if constexpr (sizeof(TOut) == 2) {
                        uint8_t* rowp = buf + lane * 64;
                        const int sw = (lane >> 1) & 3;                        // 64-byte swizzle: piece ^= (row / 2) % 4
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            uint4 o;
                            __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                            for (int q = 0; q < 4; q++) oh[q] = __floats2bfloat162_rn(f[8 * k + 2 * q], f[8 * k + 2 * q + 1]);
                            *reinterpret_cast<uint4*>(rowp + ((k ^ sw) << 4)) = o;
                        }
                    } else {
                        uint8_t* rowp = buf + lane * 128;
                        const int sw = lane & 7;                               // 128-byte swizzle: piece ^= row % 8
#pragma unroll
                        for (int k = 0; k < 8; k++)
                            *reinterpret_cast<float4*>(rowp + ((k ^ sw) << 4)) = make_float4(f[4 * k], f[4 * k + 1], f[4 * k + 2], f[4 * k + 3]);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic-proxy writes -> visible to the TMA unit
                    __syncwarp();
                    if (lane == 0) {
                        asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                                     ::"l"(reinterpret_cast<uint64_t>(&tmC)), "r"(smem_u32(buf)), "r"(col0), "r"(m0 + quarter * 32), "r"(z1), "r"(z2)
                                     : "memory");
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                    chunk_seq++;
                } else if (row_ok) {
                    // output pitch or base that a tensor map cannot express: element-wise stores of this thread's row
                    TOut* cp = cbase + (long long)row * p.ldc + col0;
#pragma unroll
                    for (int j = 0; j < 32; j++) if (col0 + j < p.N) cp[j] = (TOut)f[j];
                }
            }
            if (c_begin >= c_end) release_acc(acc);
            if constexpr (REDUCE) {
                if (row_ok) {
                    const size_t slot = (size_t)row * ra.parts + 2 * tn + half;
                    ra.part[slot] = make_float2(r_mx, r_s);
                    ra.arg[slot] = r_arg;
                }
            }
            tile_par ^= 1;
            if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // staging must outlive its readers
        __syncwarp();
    }

    // teardown: every thread arrives here, also after an aborted wait
    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // give loads that may still be in flight time to land before shared memory is released
        unsigned long long t0 = globaltimer();
        while (globaltimer() - t0 < 200000ull) { }
        __syncthreads();
    }
    if constexpr (PAIR) cluster_sync();        // neither CTA leaves (or frees TMEM) while the other may still signal it
    if (warp == 1) {
        tc_fence_after();
        if constexpr (PAIR) tmem_dealloc_pair(tmem_base, TMEM_COLS); else tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------- host side ----------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// rank-4 map over a K-major operand: dims (K, rows, nb1, nb2), box (128 bytes of K, box_rows, 1, 1)
static int encode_operand(CUtensorMap* map, const void* ptr, bool tf32, int K, int rows, long long ld, int nb1, int nb2,
                          long long s1, long long s2, int box_rows) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return fail("cuTensorMapEncodeTiled is not available from this driver");
    const size_t es = tf32 ? 4 : 2;
    cuuint64_t dims[4] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)nb1, (cuuint64_t)nb2};
    // strides of dims 1..3 in bytes; a dim of extent 1 still needs a legal (multiple of 16) stride
    cuuint64_t st[3] = {(cuuint64_t)ld * es, (cuuint64_t)(nb1 > 1 ? s1 : ld) * es, (cuuint64_t)(nb2 > 1 ? s2 : ld) * es};
    cuuint32_t box[4] = {(cuuint32_t)(kStageRowBytes / es), (cuuint32_t)box_rows, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    // TFLOAT32 maps make the TMA unit round f32 to TF32 on the way into shared memory; a plain FLOAT32 map would leave
    // the tensor core to truncate the low 13 mantissa bits, a one-sided error three times larger (measured 7.5e-4 vs 2.5e-4).
    CUresult r = enc(map, tf32 ? CU_TENSOR_MAP_DATA_TYPE_TFLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, st,
                     box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled failed with CUresult %d (K=%d rows=%d ld=%lld)", (int)r, K, rows, ld);
    return 0;
}

// rank-4 map over the output: dims (N, M, nb1, nb2), box (32 columns, 32 rows, 1, 1)
static int encode_output(CUtensorMap* map, void* ptr, bool bf16, int N, int M, long long ld, int nb1, int nb2, long long s1, long long s2) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return fail("cuTensorMapEncodeTiled is not available from this driver");
    const size_t es = bf16 ? 2 : 4;
    cuuint64_t dims[4] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)nb1, (cuuint64_t)nb2};
    cuuint64_t st[3] = {(cuuint64_t)ld * es, (cuuint64_t)(nb1 > 1 ? s1 : ld) * es, (cuuint64_t)(nb2 > 1 ? s2 : ld) * es};
    cuuint32_t box[4] = {32, 32, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, ptr, dims, st, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, bf16 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled (output) failed with CUresult %d (N=%d M=%d ld=%lld)", (int)r, N, M, ld);
    return 0;
}

bool gemm_supported(const GemmDesc& d, const char** why) {
    static const char* ok = "";
    const long long es = d.mode == MM_TF32 ? 4 : 2;
    auto bad = [&](const char* w) { if (why) *why = w; return false; };
    if (d.mode != MM_TF32 && d.mode != MM_BF16) return bad("mode is not a tensor-core mode");
    if (d.M <= 0 || d.N <= 0 || d.K <= 0) return bad("empty problem");
    if ((reinterpret_cast<uintptr_t>(d.A) & 15) || (reinterpret_cast<uintptr_t>(d.B) & 15)) return bad("operand base not 16-byte aligned");
    if ((d.lda * es) % 16 || (d.ldb * es) % 16) return bad("operand row pitch not a multiple of 16 bytes");
    if (d.nb1 > 1 && ((d.sA1 * es) % 16 || (!d.b_broadcast && (d.sB1 * es) % 16))) return bad("batch stride not a multiple of 16 bytes");
    if (d.nb2 > 1 && ((d.sA2 * es) % 16 || (!d.b_broadcast && (d.sB2 * es) % 16))) return bad("batch stride not a multiple of 16 bytes");
    if (d.lda < d.K || d.ldb < d.K) return bad("row pitch smaller than K");
    if ((long long)d.lda * es >= (1ll << 40) || (long long)d.ldb * es >= (1ll << 40)) return bad("row pitch too large for a tensor map");
    if (d.mode == MM_TF32 && d.out_dtype != F32) return bad("TF32 mode writes f32 only");
    if (d.norm_axis) {
        if (d.norm_axis != 1) return bad("norm_axis is not 0 or 1");
        if (!d.norm_stats || !d.norm_s) return bad("folded LayerNorm needs its statistics and column sums");
        if ((reinterpret_cast<uintptr_t>(d.norm_stats) | reinterpret_cast<uintptr_t>(d.norm_s)) & 15) return bad("folded LayerNorm vectors must be 16-byte aligned");
        if (d.alpha != 1.0f) return bad("folded LayerNorm does not combine with alpha");
    }
    if (d.reduce) {
        if (d.norm_axis || d.R || d.epilogue != EPI_NONE) return bad("row reductions do not combine with a folded LayerNorm, a residual or an activation");
        if (d.N <= 128) return bad("row reductions need N > 128");
        if (d.nb1 != 1 || d.nb2 != 1 || d.causal_lower || d.causal_k) return bad("row reductions take one plain matrix product");
        if (!d.red_part || !d.red_arg || (d.red_targets && !d.red_tgt)) return bad("row reductions need their output buffers");
    }
    if (why) *why = ok;
    return true;
}

template <bool TF32, typename TOut, int BN>
static int launch_t(const GemmPlan& pl, const GemmParams& prm) {
    auto kern = gemm_tcgen05_kernel<TF32, TOut, BN, false>;
    static bool attr_set = false;   // per instantiation
    if (!attr_set) {
        SPT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
        attr_set = true;
    }
    kern<<<pl.grid, kGemmThreads, pl.smem, rt().stream>>>(pl.tmA, pl.tmB, pl.tmC, prm, NormArgs{nullptr, nullptr}, ReduceArgs{});
    SPT_LAUNCH_CHECK("gemm_tcgen05");
    return 0;
}

// folded-LayerNorm epilogues exist for the shape class that uses them: bf16 in and out, 256-column tiles, one CTA per tile
template <int NORM>
static int launch_norm_t(const GemmPlan& pl, const GemmParams& prm) {
    auto kern = gemm_tcgen05_kernel<false, __nv_bfloat16, 256, false, NORM>;
    static bool attr_set = false;
    if (!attr_set) {
        SPT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
        attr_set = true;
    }
    kern<<<pl.grid, kGemmThreads, pl.smem, rt().stream>>>(pl.tmA, pl.tmB, pl.tmC, prm, NormArgs{pl.d.norm_stats, pl.d.norm_s}, ReduceArgs{});
    SPT_LAUNCH_CHECK("gemm_tcgen05 (folded LayerNorm)");
    return 0;
}

// row-reduction epilogues exist for 256-column tiles, one CTA per tile: bf16 operands with the values rounded to bf16, or TF32 / f32
template <bool TF32, typename TOut>
static int launch_reduce_t(const GemmPlan& pl, const GemmParams& prm) {
    auto kern = gemm_tcgen05_kernel<TF32, TOut, 256, false, 0, true>;
    static bool attr_set = false;
    if (!attr_set) {
        SPT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
        attr_set = true;
    }
    const GemmDesc& d = pl.d;
    kern<<<pl.grid, kGemmThreads, pl.smem, rt().stream>>>(pl.tmA, pl.tmB, pl.tmC, prm, NormArgs{nullptr, nullptr},
                                                          ReduceArgs{d.red_part, d.red_arg, d.red_targets, d.red_tgt, gemm_reduce_parts(d.N)});
    SPT_LAUNCH_CHECK("gemm_tcgen05 (row reductions)");
    return 0;
}

static size_t smem_for(int bn) { return (size_t)kStages * (BM + bn) * kStageRowBytes + 256 /*barriers*/ + 8 * 4096 /*epilogue staging*/ + 2 * 1024 /*bias tiles*/; }
static size_t smem_for_pair() { return (size_t)kStagesPair * (BM + 128) * kStageRowBytes + 256 + 8 * 4096 + 2 * 1024; }

// pair kernel: clusters of two CTAs
template <bool TF32, typename TOut>
static int launch_pair_t(const GemmPlan& pl, const GemmParams& prm) {
    auto kern = gemm_tcgen05_kernel<TF32, TOut, 256, true>;
    static bool attr_set = false;
    if (!attr_set) {
        SPT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
        attr_set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)pl.grid); cfg.blockDim = dim3(kGemmThreads); cfg.dynamicSmemBytes = pl.smem; cfg.stream = rt().stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension; at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    SPT_CUDA(cudaLaunchKernelEx(&cfg, kern, pl.tmA, pl.tmB, pl.tmC, prm, NormArgs{nullptr, nullptr}, ReduceArgs{}));
    SPT_LAUNCH_CHECK("gemm_tcgen05 (pair)");
    return 0;
}

// how many two-CTA clusters of the pair kernel the device holds at once (0: unknown or none -> pair kernel not used)
static int max_pairs() {
    static int n = -1;
    static std::once_flag once;
    std::call_once(once, [] {
        auto kern = gemm_tcgen05_kernel<false, __nv_bfloat16, 256, true>;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_for_pair()) != cudaSuccess) { cudaGetLastError(); n = 0; return; }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * 512); cfg.blockDim = dim3(kGemmThreads); cfg.dynamicSmemBytes = smem_for_pair();
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension; at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cfg.attrs = at; cfg.numAttrs = 1;
        int c = 0;
        if (cudaOccupancyMaxActiveClusters(&c, kern, &cfg) != cudaSuccess) { cudaGetLastError(); c = 0; }
        n = c;
    });
    return n;
}

// 3 (default): CTA pairs where they measured faster -- TF32 problems, bf16 problems with K >= 1536, and bf16 problems with a plain
// epilogue -- from 2048 rows up;
// 0: one-CTA tiles only; 1: CTA pairs wherever they apply; 2: CTA pairs for TF32 problems only.  Measured on B200 (median of 10,
// L2 flushed, one CTA vs pairs): bf16 65536 x 3072 -> 768 0.223 vs 0.203 ms, 16384 x 4096 -> 4096 0.368 vs 0.343 ms (1603 TFLOP/s),
// 16384 x 3072 -> 768 0.072 vs 0.064 ms, but 65536 x 768 -> 3072 0.244 vs 0.244 ms and 4096 x 768 -> 768 0.0164 vs 0.0174 ms (a
// K = 768 tile is twelve k-blocks: its fixed cost, not the operand traffic the pair halves, sets its pace); TF32 16384 x 768 -> 3072
// 0.135 vs 0.119 ms, 16384 x 3072 -> 768 0.139 vs 0.115 ms.  (Pairs were slower everywhere while the MMAs were issued under
// `lane == 0`: their issue path is longer, and that path was the limit.)  SPTORCH_B200_GEMM_PAIR in the environment sets the
// initial value.
static std::atomic<int> g_pair_mode{[] { const char* e = getenv("SPTORCH_B200_GEMM_PAIR"); return (e && e[0] >= '0' && e[0] <= '3') ? e[0] - '0' : 3; }()};

int gemm_plan(const GemmDesc& d, GemmPlan* plan) {
    const char* why = nullptr;
    if (d.few_rows_ok && linear_few_rows_supported(d)) {
        plan->d = d;
        plan->few_rows = true;
        plan->valid = true;
        return 0;
    }
    plan->few_rows = false;
    if (!gemm_supported(d, &why)) return fail("gemm: %s", why);
    plan->d = d;
    int bn = d.N <= 64 ? 64 : d.N <= 128 ? 128 : 256;
    if (bn == 256 && !d.norm_axis && !d.reduce) {
        // Tile width by the number of waves the tiles make over the SMs.  A problem with few 128 x 256 tiles leaves most SMs idle in
        // its last wave (8192 x 768 -> 768: 192 tiles on 148 SMs are two waves, the second 30 % full); 128-column tiles cost
        // kNarrowTileCost of a 256-column tile each (they re-read the A tile twice as often and amortise the per-tile overhead
        // over half the work) but round up to fewer idle SMs.  SPTORCH_B200_GEMM_BN forces a width (experiments).
        static const int forced = getenv("SPTORCH_B200_GEMM_BN") ? atoi(getenv("SPTORCH_B200_GEMM_BN")) : 0;
        static const double narrow_cost = getenv("SPTORCH_B200_GEMM_NARROW_COST") ? atof(getenv("SPTORCH_B200_GEMM_NARROW_COST")) : kNarrowTileCost;
        const long long sms = compute_sms();
        const long long tm = (long long)ceil_div(d.M, BM) * d.nb1 * d.nb2;
        auto waves = [&](int w) { const long long tiles = tm * ceil_div(d.N, w); return (double)((tiles + sms - 1) / sms); };
        if (forced == 128 || forced == 256) bn = forced;
        else if (!d.causal_lower && !d.causal_k && waves(128) * narrow_cost < waves(256) * 0.97) bn = 128;
    }
    plan->bn = bn;
    // wide problems run on CTA pairs (each SM then loads half of the B tile); the triangular attention products do not
    int pairs = 0;
    const int pm = g_pair_mode.load();
    // ... and bf16 problems whose epilogue has nothing to add (no bias, no residual, alpha 1): with the plain epilogue the pair kernel
    // is ahead at K = 768 too (65536 x 768 -> 2304: 0.173 vs 0.156 ms; 32768 x 768 -> 50304: 1.778 vs 1.650 ms), while with a
    // residual it is behind (65536 x 768 -> 768 + residual: 0.098 vs 0.102 ms).  SPTORCH_B200_GEMM_PAIR_PLAIN=0 drops this clause.
    static const bool pair_plain = !(getenv("SPTORCH_B200_GEMM_PAIR_PLAIN") && atoi(getenv("SPTORCH_B200_GEMM_PAIR_PLAIN")) == 0);
    const bool plain = pair_plain && !d.bias && !d.R && d.alpha == 1.0f && d.epilogue == EPI_NONE;
    const bool pair_auto = pm == 3 && d.M >= 2048 && d.nb1 * d.nb2 == 1 && (d.mode == MM_TF32 || d.K >= 1536 || plain);
    if (!d.norm_axis && !d.reduce && (pm == 1 || (pm == 2 && d.mode == MM_TF32) || pair_auto) && bn == 256 && d.M > BM && !d.causal_lower && !d.causal_k) pairs = std::min(max_pairs(), compute_sms() / 2);
    plan->pair = pairs > 0;
    plan->tiles_m = ceil_div(d.M, plan->pair ? 2 * BM : BM);
    plan->tiles_n = ceil_div(d.N, bn);
    long long total = (long long)plan->tiles_m * plan->tiles_n * d.nb1 * d.nb2;
    if (total > INT32_MAX) return fail("gemm: too many tiles");
    if (plan->pair) {
        plan->grid = 2 * (int)(total < pairs ? total : pairs);
        plan->smem = smem_for_pair();
    } else {
        plan->grid = (int)(total < compute_sms() ? total : compute_sms());
        plan->smem = smem_for(bn);
    }
    // Rasterisation band: B tiles are re-read once per band of m-tiles.  A B operand that fits L2 beside the streams stays
    // resident whatever the band; a large one (the LM head: 77 MB of bf16 weights under 6.6 GB of output writes) is evicted
    // between bands and came from DRAM 64 times with 8-tile bands (ncu: 5.0 GB read for 0.18 GB of operands); 64-tile bands
    // cut the re-reads eightfold and the head GEMM from 4.85 to 4.26 ms, while small-B shapes measured 1 % slower with them.
    {
        const long long b_bytes = (long long)d.N * d.K * (d.mode == MM_TF32 ? 4 : 2);
        plan->group_m = b_bytes > (48ll << 20) ? 64 : kGroupM;
    }
    const bool tf32 = d.mode == MM_TF32;
    const int b_box = plan->pair ? bn / 2 : bn;
    if (encode_operand(&plan->tmA, d.A, tf32, d.K, d.M, d.lda, d.nb1, d.nb2, d.sA1, d.sA2, BM)) return 1;
    if (d.b_broadcast) { if (encode_operand(&plan->tmB, d.B, tf32, d.K, d.N, d.ldb, 1, 1, 0, 0, b_box)) return 1; }
    else if (encode_operand(&plan->tmB, d.B, tf32, d.K, d.N, d.ldb, d.nb1, d.nb2, d.sB1, d.sB2, b_box)) return 1;
    // output map: 32x32 boxes, swizzled to match the conflict-free staging layout of the epilogue
    const long long oes = d.out_dtype == BF16 ? 2 : 4;
    plan->tma_store = !d.reduce && ((reinterpret_cast<uintptr_t>(d.C) & 15) == 0) && (d.ldc * oes) % 16 == 0 && d.ldc >= d.N &&
                      (d.nb1 <= 1 || (d.sC1 * oes) % 16 == 0) && (d.nb2 <= 1 || (d.sC2 * oes) % 16 == 0);
    if (plan->tma_store) {
        if (encode_output(&plan->tmC, d.C, d.out_dtype == BF16, d.N, d.M, d.ldc, d.nb1, d.nb2, d.sC1, d.sC2)) return 1;
    } else {
        plan->tmC = plan->tmA;   // never dereferenced by the kernel in this mode
    }
    plan->valid = true;
    return 0;
}

int gemm_run(const GemmPlan& pl) {
    if (!pl.valid) return fail("gemm_run: plan not prepared");
    const GemmDesc& d = pl.d;
    if (pl.few_rows) return linear_few_rows(d);
    GemmParams prm;
    prm.C = d.C; prm.bias = d.bias; prm.R = d.R;
    prm.M = d.M; prm.N = d.N; prm.K = d.K; prm.ldc = d.ldc;
    prm.nb1 = d.nb1; prm.nb2 = d.nb2; prm.sC1 = d.sC1; prm.sC2 = d.sC2;
    prm.alpha = d.alpha; prm.epilogue = d.epilogue;
    prm.tiles_m = pl.tiles_m; prm.tiles_n = pl.tiles_n;
    prm.group_m = pl.group_m;
    prm.num_kb = ceil_div(d.K, d.mode == MM_TF32 ? 32 : 64);
    prm.causal_lower = d.causal_lower;
    prm.causal_k = d.causal_k;
    prm.b_broadcast = d.b_broadcast;
    prm.tma_store = pl.tma_store ? 1 : 0;
    {
        const long long oes = d.out_dtype == BF16 ? 2 : 4;
        prm.r_vec = d.R != nullptr && (reinterpret_cast<uintptr_t>(d.R) & 15) == 0 && (d.ldc * oes) % 16 == 0 &&
                    (d.nb1 <= 1 || (d.sC1 * oes) % 16 == 0) && (d.nb2 <= 1 || (d.sC2 * oes) % 16 == 0);
    }
    prm.status = rt().dev_status;
    const bool tf32 = d.mode == MM_TF32;
    const bool out_bf16 = d.out_dtype == BF16;
    if (d.reduce) {
        if (pl.bn != 256 || pl.pair) return fail("gemm_run: the row-reduction epilogue needs N > 128");
        if (tf32) return launch_reduce_t<true, float>(pl, prm);
        if (out_bf16) return launch_reduce_t<false, __nv_bfloat16>(pl, prm);
        return launch_reduce_t<false, float>(pl, prm);
    }
    if (d.norm_axis) {
        if (tf32 || !out_bf16 || pl.bn != 256 || pl.pair) return fail("gemm_run: the folded-LayerNorm epilogue needs bf16 operands and output and N > 128");
        return launch_norm_t<1>(pl, prm);
    }
    if (pl.pair) {
        if (tf32) return launch_pair_t<true, float>(pl, prm);
        if (out_bf16) return launch_pair_t<false, __nv_bfloat16>(pl, prm);
        return launch_pair_t<false, float>(pl, prm);
    }
#define SPT_GEMM_CASE(BN_)                                                                          \
    if (pl.bn == BN_) {                                                                             \
        if (tf32) return launch_t<true, float, BN_>(pl, prm);                                       \
        if (out_bf16) return launch_t<false, __nv_bfloat16, BN_>(pl, prm);                          \
        return launch_t<false, float, BN_>(pl, prm);                                                \
    }
    SPT_GEMM_CASE(64)
    SPT_GEMM_CASE(128)
    SPT_GEMM_CASE(256)
#undef SPT_GEMM_CASE
    return fail("gemm_run: no kernel for BN=%d", pl.bn);
}

// ---------------- CUDA-core f32 matmul (exact-order mode and shapes TMA cannot express) ----------------
// 64x64 output tile per CTA, 16x16 threads, 4x4 outputs per thread, K consumed in order p = 0..K-1 with
// one fused multiply-add per product.
__global__ void __launch_bounds__(256) simt_matmul_kernel(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                                                          int M, int N, int K, int b_is_kn, const float* __restrict__ bias,
                                                          const float* __restrict__ R, float alpha, int epilogue) {
    __shared__ float As[16][64 + 1];
    __shared__ float Bs[16][64 + 1];
    const int z = blockIdx.z;
    A += (size_t)z * M * K; B += (size_t)z * N * K; C += (size_t)z * M * N;
    if (R) R += (size_t)z * M * N;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            int r = i / 16, c = i % 16;                 // A tile: 64 rows x 16 k
            int gm = m0 + r, gk = k0 + c;
            As[c][r] = (gm < M && gk < K) ? A[(size_t)gm * K + gk] : 0.0f;
        }
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            int gk, gn, kk, nn;
            if (b_is_kn) { kk = i / 64; nn = i % 64; } else { nn = i / 16; kk = i % 16; }
            gk = k0 + kk; gn = n0 + nn;
            float v = 0.0f;
            if (gk < K && gn < N) v = b_is_kn ? B[(size_t)gk * N + gn] : B[(size_t)gn * K + gk];
            Bs[kk][nn] = v;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < 16; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { a[i] = As[kk][ty * 4 + i]; b[i] = Bs[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            int gm = m0 + ty * 4 + i, gn = n0 + tx * 4 + j;
            if (gm < M && gn < N) {
                float v = acc[i][j] * alpha;
                if (bias) v += bias[gn];
                if (epilogue == EPI_GELU) v = gelu_exact(v);
                if (epilogue == EPI_SWIGLU) { const float s_ = 1.0f / (1.0f + expf(-v)); v = R ? (R[(size_t)gm * N + gn] * v) * s_ : v * s_; }
                else if (R) v += R[(size_t)gm * N + gn];
                C[(size_t)gm * N + gn] = v;
            }
        }
}

int simt_matmul_f32(const float* A, const float* B, float* C, int batch, int M, int N, int K, bool b_is_kn, const float* bias,
                    const float* R, float alpha, int epilogue) {
    if (batch <= 0 || M <= 0 || N <= 0) return 0;
    dim3 grid((unsigned)ceil_div(N, 64), (unsigned)ceil_div(M, 64), (unsigned)batch);
    if (grid.y > 65535 || grid.z > 65535) return fail("simt_matmul: shape exceeds one launch (M tiles %u, batch %u)", grid.y, grid.z);
    simt_matmul_kernel<<<grid, 256, 0, rt().stream>>>(A, B, C, M, N, K, b_is_kn ? 1 : 0, bias, R, alpha, epilogue);
    SPT_LAUNCH_CHECK("simt_matmul");
    return 0;
}

static std::atomic<int> g_abi_mode{MM_TF32};

extern "C" int sptorch_ext_set_gemm_pair(int mode) {
    if (mode < 0 || mode > 3) return fail("set_gemm_pair: mode %d is not 0 .. 3", mode);
    g_pair_mode.store(mode);
    bump_config_epoch();
    return 0;
}

// C-ABI matmul: B arrives as [k,n] row-major.  Tensor-core path: transpose B once into a pool scratch
// (one HBM pass over B) so that both operands are K-major, then the TF32 GEMM.  Shapes whose pitches TMA
// cannot express, and MM_F32 mode, run on the CUDA cores.
static int abi_matmul(const void* a, const void* b, void* out, size_t batch, size_t m, size_t k, size_t n) {
    if (enter()) return 1;
    if (batch == 0 || m == 0 || n == 0) return 0;
    if (!a || !b || !out) return fail("matmul_f32: null handle");
    if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX || batch > 65535) return fail("matmul_f32: dimension too large");
    if (k == 0) return sptorch_ext_memset(out, 0, batch * m * n * sizeof(float));
    GemmDesc d;
    d.mode = MM_TF32; d.out_dtype = F32;
    d.M = (int)m; d.N = (int)n; d.K = (int)k;
    d.lda = (long long)k; d.ldb = (long long)k; d.ldc = (long long)n;
    d.nb1 = (int)batch; d.sA1 = (long long)(m * k); d.sB1 = (long long)(n * k); d.sC1 = (long long)(m * n);
    d.A = a; d.B = b /* placeholder for the support check */; d.C = out;
    const bool tc = g_abi_mode.load() == MM_TF32 && gemm_supported(d, nullptr) && (m * n * k >= (size_t)64 * 64 * 64);
    if (!tc) return simt_matmul_f32((const float*)a, (const float*)b, (float*)out, (int)batch, (int)m, (int)n, (int)k, true, nullptr, nullptr, 1.0f, EPI_NONE);
    float* bt = (float*)sptorch_ext_alloc_bytes(batch * n * k * sizeof(float));
    if (!bt) return 1;
    int rc = 0;
    for (size_t z = 0; z < batch && rc == 0; z++)
        rc = sptorch_ext_transpose_f32((const float*)b + z * k * n, bt + z * k * n, k, n);
    if (rc == 0) {
        d.B = bt;
        GemmPlan pl;
        rc = gemm_plan(d, &pl);
        if (rc == 0) rc = gemm_run(pl);
    }
    sptorch_free(bt);
    return rc;
}

// ---- matmul for callers that must not allocate ----
// Scratch for the transposed B operand lives in the library image instead of coming from the pool.
constexpr size_t kStaticScratchFloats = size_t(1) << 21;                 // 8 MiB: k * n <= 2,097,152
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];
static float* g_static_scratch_addr[64] = {};                            // device address per CUDA ordinal, filled on first use
static std::mutex g_static_scratch_mu;

// Device address of the array for the runtime's device; looked up once per CUDA ordinal with that device current.
// In host code the array's name is only a stand-in: a kernel must be given the address the runtime reports.
static float* static_scratch_address(int dev) {
    if (dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lk(g_static_scratch_mu);
    if (!g_static_scratch_addr[dev]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) { cudaGetLastError(); return nullptr; }
        g_static_scratch_addr[dev] = (float*)p;
    }
    return g_static_scratch_addr[dev];
}
// Called by the backend's initialisation (device current, nothing captured yet), so that later calls of
// sptorch_ext_matmul_f32_static find the address cached; a failure here is retried by the first call.
void static_scratch_prepare() { (void)static_scratch_address(rt().device); }

}  // namespace spt

using namespace spt;

extern "C" {

// sptorch_ext_matmul_f32_static: same result as sptorch_matmul_f32 (C = A[m,k] * B[k,n], row-major f32), for callers
// that cannot let the library allocate device memory while they run: a program whose memory budget is fixed up
// front and audited, a latency-critical loop that must not touch the allocator (an allocation can synchronise or
// fail at an arbitrary moment), or code running while the pool is deliberately exhausted.  The only scratch the
// tensor-core path needs -- B transposed to K-major -- is a fixed 8 MiB array inside the library image, so this
// call performs no cudaMalloc / cudaFree / pool allocation of any kind.
//   * limit: k * n <= 2,097,152 elements (for example 1024 x 2048); larger products are rejected with an error.
//     Every GPU that loads the library carries the 8 MiB until the process exits.
//   * the array's device address is looked up (cudaGetSymbolAddress) when the backend is initialised, with the
//     backend's device current; should that lookup have failed, the first call here repeats it, so make the first
//     call before starting any stream capture.
//   * all calls share the one array and it keeps the previous call's contents; nothing in it has to start at zero
//     (each call overwrites the k * n elements it then reads).  Two calls whose kernels overlap on the GPU -- from
//     different streams or threads -- would race on it: issue them on the library's stream, one after the other.
// a, b, out are device handles as for sptorch_matmul_f32; returns 0 on success.
int sptorch_ext_matmul_f32_static(const void* a, const void* b, void* out, size_t m, size_t k, size_t n) {
    if (enter()) return 1;
    if (m == 0 || n == 0) return 0;
    if (!a || !b || !out) return fail("matmul_f32_static: null handle");
    if (m > INT32_MAX || n > INT32_MAX || k > INT32_MAX) return fail("matmul_f32_static: dimension too large");
    if (k == 0) {
        SPT_CUDA(cudaMemsetAsync(out, 0, m * n * sizeof(float), rt().stream));
        note_submit();
        return 0;
    }
    if (k * n > kStaticScratchFloats)
        return fail("matmul_f32_static: k*n = %zu exceeds the static scratch of %zu elements; use sptorch_matmul_f32", k * n, (size_t)kStaticScratchFloats);
    const int dev = rt().device;
    if (dev < 0 || dev >= 64) return fail("matmul_f32_static: device ordinal %d out of range", dev);
    float* scratch = static_scratch_address(dev);
    if (!scratch) return fail("matmul_f32_static: cudaGetSymbolAddress could not resolve the static scratch on device %d", dev);
    GemmDesc d;
    d.mode = MM_TF32; d.out_dtype = F32;
    d.M = (int)m; d.N = (int)n; d.K = (int)k;
    d.lda = (long long)k; d.ldb = (long long)k; d.ldc = (long long)n;
    d.A = a; d.B = scratch; d.C = out;
    const bool tc = g_abi_mode.load() == MM_TF32 && gemm_supported(d, nullptr) && (m * n * k >= (size_t)64 * 64 * 64);
    if (!tc) return simt_matmul_f32((const float*)a, (const float*)b, (float*)out, 1, (int)m, (int)n, (int)k, true, nullptr, nullptr, 1.0f, EPI_NONE);
    if (sptorch_ext_transpose_f32(b, scratch, k, n)) return 1;
    GemmPlan pl;
    if (gemm_plan(d, &pl)) return 1;
    return gemm_run(pl);
}

int sptorch_matmul_f32(const void* a, const void* b, void* out, size_t m, size_t k, size_t n) { return abi_matmul(a, b, out, 1, m, k, n); }
int sptorch_batch_matmul_f32(const void* a, const void* b, void* out, size_t batch, size_t m, size_t k, size_t n) {
    return abi_matmul(a, b, out, batch, m, k, n);
}

int sptorch_ext_set_matmul_mode(int mode) {
    if (mode != SPT_MM_TF32 && mode != SPT_MM_F32) return fail("set_matmul_mode: the f32 C-ABI accepts SPT_MM_TF32 or SPT_MM_F32");
    g_abi_mode.store(mode);
    bump_config_epoch();
    return 0;
}

int sptorch_ext_linear(const void* x, const void* w, const void* bias, const void* residual, void* out, size_t M, size_t K, size_t N,
                       size_t ldo, float alpha, int epilogue, int mode, int out_dtype) {
    if (enter()) return 1;
    if (M == 0 || N == 0) return 0;
    if (!x || !w || !out) return fail("linear: null handle");
    if (M > INT32_MAX || N > INT32_MAX || K > INT32_MAX) return fail("linear: dimension too large");
    if (ldo == 0) ldo = N;
    if (ldo < N) return fail("linear: ldo < N");
    if (epilogue != SPT_EPI_NONE && epilogue != SPT_EPI_GELU && epilogue != SPT_EPI_SWIGLU) return fail("linear: unknown epilogue %d", epilogue);
    if (epilogue == SPT_EPI_SWIGLU && !residual) return fail("linear: the SwiGLU epilogue multiplies by the residual operand, which is null");
    if (mode == SPT_MM_F32 || K == 0) {
        if (out_dtype != SPT_F32 || ldo != N) return fail("linear: the CUDA-core f32 mode needs f32 output with ldo == N");
        return simt_matmul_f32((const float*)x, (const float*)w, (float*)out, 1, (int)M, (int)N, (int)K, false, (const float*)bias,
                               (const float*)residual, alpha, epilogue);
    }
    GemmDesc d;
    d.A = x; d.B = w; d.C = out; d.bias = (const float*)bias; d.R = residual;
    d.M = (int)M; d.N = (int)N; d.K = (int)K;
    d.lda = (long long)K; d.ldb = (long long)K; d.ldc = (long long)ldo;
    d.alpha = alpha; d.epilogue = epilogue; d.mode = mode; d.out_dtype = out_dtype;
    d.few_rows_ok = 1;
    if (mode == SPT_MM_TF32 && !gemm_supported(d, nullptr) && out_dtype == SPT_F32 && ldo == N)
        return simt_matmul_f32((const float*)x, (const float*)w, (float*)out, 1, (int)M, (int)N, (int)K, false, (const float*)bias,
                               (const float*)residual, alpha, epilogue);
    GemmPlan pl;
    if (gemm_plan(d, &pl)) return 1;
    return gemm_run(pl);
}

}  // extern "C"
