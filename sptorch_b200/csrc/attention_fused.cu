// attention_fused.cu -- fused causal attention for bf16, head_dim 64 or 128 (sm_100a, tcgen05 + TMEM + TMA).
//
// Same function as crates/nn/src/lib.rs:600-637 (scores = Q K^T * 1/sqrt(hd); entries j > i set to -inf; row
// softmax; P V; heads merged back) but the [T,T] score and probability matrices never reach HBM: one CTA owns
// one 128-row query tile of one (sequence, head) and walks the key/value tiles (64 keys each) up to the diagonal
// with a running row maximum and row sum (the softmax is exact; only the order of the sums differs).
//
//   warp 0      TMA: Q tile once, then K tile [64 keys, hd] and V^T tile [hd, 64 keys] per step, 3-stage ring
//   warp 1      tcgen05.mma: S_j = Q K_j^T (M128 N64) into one of two TMEM buffers, issued one step AHEAD of the
//               softmax; O_j = P_j V_j (M128 N=hd) into one of two TMEM buffers when P_j is ready
//   warps 2..9  two threads per query row (32 of the 64 key columns each): S_j from TMEM into registers, causal
//               mask on the diagonal tiles, running maximum agreed with the partner thread, exp2, P_j as bf16 into
//               one of two shared-memory buffers in the 128-byte-swizzled K-major layout the P V MMA reads; the
//               product O_{j-1} of the PREVIOUS step is folded into the register accumulator afterwards, so no
//               thread ever waits for the MMA it has just enabled
// Two CTAs are resident per SM for hd = 64 (97 KB of shared memory and 256 TMEM columns each).  Heavy (late)
// query tiles are scheduled first.
// Algorithmic work per (sequence, head): 2 * T(T+1) * hd FLOP; HBM traffic: Q, K, V read once per query tile
// (K/V re-reads hit L2), O written once.
#include "gemm.h"
#include "sm100.cuh"
#include "../../include/sptorch_b200_ext.h"
#include <algorithm>
#include <array>
#include <cstdlib>
#include <map>
#include <mutex>
#include <queue>
#include <vector>

namespace spt {

using namespace sm100;

constexpr int kAttnThreads = 320;           // TMA warp + MMA warp + 8 softmax warps
constexpr int kQTile = 128, kKvTile = 64;
constexpr int kKvStages = 3;

struct AttnParams {
    __nv_bfloat16* out;
    long long ld_out;       // row stride of out in elements
    int T, H, B;
    int n_qtiles;
    float scale_log2;       // 1/sqrt(hd) * log2(e)
    unsigned long long* prof;   // diagnostics: cycle counters of CTA 0 (softmax warp 2 lane 0: [0..7], MMA warp lane 0: [8..15]); may be null
    uint32_t* status;
    const int* sched;       // work schedule [sched_len][gridDim.x]: item of CTA c at step k, -1 past the end of its list
    int sched_len;
};

// 2^x on the special-function unit: one instruction, relative error 2^-22 (P is rounded to bf16 right after)
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

template <int HD>
struct AttnSmem {
    static constexpr int kQBytes = kQTile * HD * 2;
    static constexpr int kKBytes = kKvTile * HD * 2;          // HD/64 k-blocks of [64 keys x 128 B]
    static constexpr int kVBytes = HD * kKvTile * 2;          // [HD rows x 128 B]
    static constexpr int kStageBytes = kKBytes + kVBytes;
    static constexpr int kPBytes = kQTile * kKvTile * 2;      // [128 rows x 128 B]
    static constexpr int kQ = 0;
    static constexpr int kKV = kQ + kQBytes;
    static constexpr int kP = kKV + kKvStages * kStageBytes;
    static constexpr int kBars = kP + 2 * kPBytes;            // mbarriers + TMEM slot + abort flag (256 B)
    static constexpr int kX = kBars + 256;                    // running-maximum exchange: [parity][half][128] floats
    static constexpr int kTotal = kX + 2048;
};

// Persistent kernel: CTA c works through column c of a schedule built on the host (attention_schedule below), and all
// three roles run straight through item boundaries (barrier phases are driven by running counters), so the loads and
// the first Q K^T of the next item are in flight while the current one drains.
template <int HD, bool PROF>
__global__ void __launch_bounds__(kAttnThreads, HD == 64 ? 2 : 1)
attn_fused_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
    using L = AttnSmem<HD>;
    constexpr uint32_t TMEM_COLS = HD == 64 ? 256 : 512;    // S: 2 x 64 columns at 0; O: 2 x HD columns at 128
    constexpr uint32_t IDESC_S = make_idesc(false, 128, kKvTile);
    constexpr uint32_t IDESC_O = make_idesc(false, 128, HD);
    constexpr int KB_Q = HD / 64;                           // 128-byte k-blocks along head_dim
    constexpr int NS = kKvStages;

    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t base = smem_u32(smem);
    // barrier slots (8 bytes each)
    const uint32_t bar = base + L::kBars;
    const uint32_t q_full = bar;                    // 2
    const uint32_t q_free = q_full + 16;            // 2
    const uint32_t kv_full = q_free + 16;           // NS
    const uint32_t kv_empty = kv_full + 8 * NS;     // NS
    const uint32_t s_full = kv_empty + 8 * NS;      // 2
    const uint32_t s_free = s_full + 16;            // 2
    const uint32_t p_full = s_free + 16;            // 2
    const uint32_t o_full = p_full + 16;            // 2
    const uint32_t o_free = o_full + 16;            // 2
    const uint32_t mx_bar = o_free + 16;            // 4, one per TMEM lane quarter
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kBars + 240);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kBars + 244);
    static_assert(8 * (4 + 2 * NS + 10 + 4) <= 240, "barrier block overflows");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int BH = p.B * p.H;
    const int n_kv_seq = (p.T + kKvTile - 1) / kKvTile;

    if ((base & 1023u) != 0) {                                // swizzled tiles need 1024-byte alignment
        if (threadIdx.x == 0) atomicOr(p.status, 0x200u);
        return;
    }
    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; s++) { mbar_init(kv_full + 8 * s, 1); mbar_init(kv_empty + 8 * s, 1); }
        for (int i = 0; i < 2; i++) {
            mbar_init(q_full + 8 * i, 1); mbar_init(q_free + 8 * i, 1);
            mbar_init(s_full + 8 * i, 1); mbar_init(s_free + 8 * i, 8); mbar_init(p_full + 8 * i, 8);      // one arrival per softmax warp
            mbar_init(o_full + 8 * i, 1); mbar_init(o_free + 8 * i, 8);
        }
        for (int q = 0; q < 4; q++) mbar_init(mx_bar + 8 * q, 2);           // the two warps of a lane quarter
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;

    // step k of this CTA's list; the entry of the next step is fetched while the current item runs
    auto fetch = [&](int k) -> int { return k < p.sched_len ? __ldg(p.sched + (size_t)k * gridDim.x + blockIdx.x) : -1; };
    // work item -> (query tile, sequence, head, number of key tiles)
    auto decode = [&](int item, int& q0, int& bb, int& hh, int& n_kv) {
        const int qt = p.n_qtiles - 1 - item / BH;
        const int bh = item % BH;
        bb = bh / p.H; hh = bh % p.H;
        q0 = qt * kQTile;
        n_kv = min((q0 + kQTile + kKvTile - 1) / kKvTile, n_kv_seq);       // causal: keys 0 .. q0+127, clipped to the sequence
    };

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) { tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); }
        bool ok = true;
        uint32_t g = 0, it = 0;
        for (int k = 0, item = fetch(0); item >= 0 && ok; k++, it++) {
            const int item_next = fetch(k + 1);
            int q0, bb, hh, n_kv;
            decode(item, q0, bb, hh, n_kv);
            item = item_next;
            const uint32_t qb = 0;       // one Q buffer: reloaded as soon as the last Q K^T of the previous item has read it
            ok = mbar_wait(q_free + 8 * qb, (it & 1) ^ 1, abort_flag, p.status, kErrProducerWait);
            if (!ok) break;
            if (lane == 0) {
                mbar_expect_tx(q_full + 8 * qb, L::kQBytes);
                for (int kb = 0; kb < KB_Q; kb++) tma_load_4d(base + L::kQ + qb * L::kQBytes + kb * (kQTile * 128), &tmQ, q_full + 8 * qb, kb * 64, q0, hh, bb);
            }
            for (int j = 0; j < n_kv && ok; j++, g++) {
                const uint32_t s = g % NS, u = (g / NS) & 1;
                ok = mbar_wait(kv_empty + 8 * s, u ^ 1, abort_flag, p.status, kErrProducerWait);
                if (!ok) break;
                if (lane == 0) {
                    const int k0 = j * kKvTile;
                    const uint32_t dst = base + L::kKV + s * L::kStageBytes;
                    mbar_expect_tx(kv_full + 8 * s, L::kStageBytes);
                    for (int kb = 0; kb < KB_Q; kb++) tma_load_4d(dst + kb * (kKvTile * 128), &tmK, kv_full + 8 * s, kb * 64, k0, hh, bb);
                    tma_load_4d(dst + L::kKBytes, &tmV, kv_full + 8 * s, k0, 0, hh, bb);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        bool ok = true;
        uint32_t g = 0, it = 0;
        const bool pr = PROF && p.prof != nullptr && blockIdx.x == 0 && lane == 0;
        unsigned long long pc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        long long tprev = clock64();
#define SPT_TICK(i) do { if (PROF && pr) { long long _t = clock64(); pc[i] += (unsigned long long)(_t - tprev); tprev = _t; } } while (0)
        auto issue_s = [&](uint32_t gg, uint32_t qb) {        // S = Q K^T of global step gg into S buffer gg & 1
            const uint32_t kaddr = base + L::kKV + (gg % NS) * L::kStageBytes;
#pragma unroll
            for (int kb = 0; kb < KB_Q; kb++) {
                const uint64_t adesc = make_kmajor_sw128_desc(base + L::kQ + qb * L::kQBytes + kb * (kQTile * 128));
                const uint64_t bdesc = make_kmajor_sw128_desc(kaddr + kb * (kKvTile * 128));
#pragma unroll
                for (int k = 0; k < 4; k++) mma_ss<false>(tmem_s + (gg & 1) * kKvTile, adesc + 2 * k, bdesc + 2 * k, IDESC_S, (kb | k) != 0 ? 1u : 0u);
            }
            mma_commit(s_full + 8 * (gg & 1));
        };
        // waits until the operands of global step gg are loaded and its S buffer has been drained
        auto s_ready = [&](uint32_t gg) -> bool {
            return mbar_wait(kv_full + 8 * (gg % NS), (gg / NS) & 1, abort_flag, p.status, kErrMmaWait) &&
                   mbar_wait(s_free + 8 * (gg & 1), ((gg >> 1) & 1) ^ 1, abort_flag, p.status, kErrMmaWait);
        };
        for (int k = 0, item = fetch(0); item >= 0 && ok; k++, it++) {
            const int item_next = fetch(k + 1);
            int q0, bb, hh, n_kv;
            decode(item, q0, bb, hh, n_kv);
            item = item_next;
            const uint32_t qb = 0;
            SPT_TICK(7);
            ok = mbar_wait(q_full + 8 * qb, it & 1, abort_flag, p.status, kErrMmaWait) && s_ready(g);
            if (!ok) break;
            SPT_TICK(0);
            tc_fence_after();
            if (lane == 0) {
                issue_s(g, qb);
                if (n_kv == 1) mma_commit(q_free + 8 * qb);
            }
            __syncwarp();
            for (int j = 0; j < n_kv && ok; j++, g++) {
                const uint32_t u2 = (g >> 1) & 1;
                if (j + 1 < n_kv) {
                    // next scores while the softmax warps work on this step
                    SPT_TICK(7);
                    ok = s_ready(g + 1);
                    if (!ok) break;
                    SPT_TICK(1);
                    tc_fence_after();
                    if (lane == 0) {
                        issue_s(g + 1, qb);
                        if (j + 2 == n_kv) mma_commit(q_free + 8 * qb);   // last read of this item's Q
                    }
                    __syncwarp();
                }
                SPT_TICK(7);
                ok = mbar_wait(p_full + 8 * (g & 1), u2, abort_flag, p.status, kErrMmaWait);
                SPT_TICK(2);
                // the output accumulator of an item (buffer = item parity) is written for the first time: the item two back must
                // have been read out of it
                if (j == 0) ok = ok && mbar_wait(o_free + 8 * (it & 1), ((it >> 1) & 1) ^ 1, abort_flag, p.status, kErrMmaWait);
                if (!ok) break;
                SPT_TICK(3);
                tc_fence_after();
                if (lane == 0) {
                    const uint64_t adesc = make_kmajor_sw128_desc(base + L::kP + (g & 1) * L::kPBytes);
                    const uint64_t bdesc = make_kmajor_sw128_desc(base + L::kKV + (g % NS) * L::kStageBytes + L::kKBytes);
                    // O accumulates in TMEM over the key tiles of the item (the softmax warps rescale it in place when a row
                    // maximum grows enough)
#pragma unroll
                    for (int k = 0; k < 4; k++) mma_ss<false>(tmem_o + (it & 1) * HD, adesc + 2 * k, bdesc + 2 * k, IDESC_O, (j | k) != 0 ? 1u : 0u);
                    mma_commit(o_full + 8 * (g & 1));
                    mma_commit(kv_empty + 8 * (g % NS));
                }
                __syncwarp();
            }
        }
        if (pr) { for (int i = 0; i < 8; i++) p.prof[8 + i] = pc[i]; }
#undef SPT_TICK
    } else {
        // ---------------- softmax + accumulate: two threads per query row ----------------
        // Warps w and w+4 share a TMEM lane quarter.  Of query row r the thread in the lower warp owns key columns
        // 0..31 of every tile and the first half of the output columns, its partner the other halves.  The two only
        // have to agree on the running maximum (exchanged through shared memory); row sums stay per thread and are
        // added once at the end.
        const int quarter = warp & 3;
        const int ch = (warp - 2) >> 2;                          // column half
        const int r = quarter * 32 + lane;                       // row inside the tile = TMEM lane
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        constexpr int OC = HD / 2;                               // output columns per thread
        const int prow_off = (r >> 3) * 1024 + (r & 7) * 128;    // row r of a [128 x 128 B] swizzled block
        const int rx = r & 7;
        float* xmax = reinterpret_cast<float*>(smem + L::kX);
        const uint32_t pair_bar = mx_bar + 8 * quarter;
        bool ok = true;
        uint32_t g = 0, px = 0, it = 0;                          // global step; pair exchanges done so far; items done so far
        const bool pr = PROF && p.prof != nullptr && blockIdx.x == 0 && warp == 2 && lane == 0;
        unsigned long long pc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        long long tprev = clock64();
#define SPT_TICK(i) do { if (PROF && pr) { long long _t = clock64(); pc[i] += (unsigned long long)(_t - tprev); tprev = _t; } } while (0)
        // P V of global step gg has completed (its commit arrives on o_full[gg & 1]; a thread never waits for a step whose
        // successor two steps on could already have been committed, because that commit needs this thread's own P)
        auto pv_done = [&](uint32_t gg) -> bool {
            return mbar_wait(o_full + 8 * (gg & 1), (gg >> 1) & 1, abort_flag, p.status, kErrEpilogueWait);
        };
        for (int k = 0, item = fetch(0); item >= 0 && ok; k++) {
            const int item_next = fetch(k + 1);
            int q0, bb, hh, n_kv;
            decode(item, q0, bb, hh, n_kv);
            item = item_next;
            const int qrow = q0 + r;
            float m = -INFINITY, l = 0.0f;
            const uint32_t o_addr = tmem_o + lane_off + (it & 1) * HD + ch * OC;      // this thread's half of its output row
            for (int j = 0; j < n_kv && ok; j++, g++) {
                const uint32_t sb = g & 1;
                const int kcol0 = j * kKvTile + ch * 32;             // key index of this thread's first column
                const bool diag = (j * kKvTile + kKvTile - 1 > q0);  // tile reaches past the first row of the query tile
                SPT_TICK(7);
                ok = mbar_wait(s_full + 8 * sb, (g >> 1) & 1, abort_flag, p.status, kErrEpilogueWait);
                if (!ok) break;
                SPT_TICK(0);
                tc_fence_after();
                uint32_t v[32];
                tmem_ld_32x32(tmem_s + lane_off + sb * kKvTile + ch * 32, v);
                tmem_ld_wait();
                tc_fence_before();
                // One arrival per warp on every barrier of this role, after __syncwarp has ordered the lanes' accesses (per-thread
                // arrivals measured the same speed; this form issues 24 shared-memory atomics per step instead of 768).
                __syncwarp();
                if (lane == 0) mbar_arrive(s_free + 8 * sb);         // scores are in registers: the buffer can take the S after next
                SPT_TICK(1);
                float mx = -INFINITY;
                if (diag) {
#pragma unroll
                    for (int i = 0; i < 32; i++) if (kcol0 + i > qrow) v[i] = 0xff800000u;     // -inf
                }
                {   // four independent chains instead of one 16-deep dependent chain
                    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        m0 = max3(m0, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                        m1 = max3(m1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                        m2 = max3(m2, __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
                        m3 = max3(m3, __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
                    }
                    mx = fmaxf(max3(m0, m1, m2), m3);
                }
                // double buffered by exchange parity: the partner may still be reading the previous value
                float* xm = xmax + (px & 1) * 256;
                xm[ch * 128 + r] = mx;
                __syncwarp();
                if (lane == 0) mbar_arrive(pair_bar);
                ok = mbar_wait(pair_bar, px & 1, abort_flag, p.status, kErrEpilogueWait);
                if (!ok) break;
                px++;
                SPT_TICK(2);
                // Lazy rescaling: the reference maximum of a row only moves when the new maximum exceeds it by more than 8 in the
                // exponent (P then stays below 2^8, exact enough in bf16 and harmless in the f32 sums); the accumulated output
                // in TMEM and the row sum are multiplied by 2^(old - new) at that moment.  Both threads of a row see the same
                // maxima and take the same decision; tcgen05.ld / st are warp-wide, so a warp rescales when any of its rows does
                // (the others multiply by one).
                const float m_cand = fmaxf(m, fmaxf(mx, xm[(ch ^ 1) * 128 + r]));
                if (j == 0) m = m_cand;
                const bool grow = j > 0 && (m_cand - m) * p.scale_log2 > 8.0f;
                if (__any_sync(0xffffffffu, grow)) {
                    float alpha = 1.0f;
                    if (grow) { alpha = ex2_approx((m - m_cand) * p.scale_log2); m = m_cand; l *= alpha; }
                    ok = pv_done(g - 1);                               // every product accumulated so far is in place
                    if (!ok) break;
                    tc_fence_after();
#pragma unroll
                    for (int c = 0; c < OC / 32; c++) {
                        uint32_t o[32];
                        tmem_ld_32x32(o_addr + c * 32, o);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                        tmem_st_32x32(o_addr + c * 32, o);
                    }
                    tmem_st_wait();
                    tc_fence_before();
                }
                const float mb = m * p.scale_log2;
                // the softmax warps are bound by instruction issue: scale/subtract, the row sum and the accumulator
                // update run on pairs of floats (fma.rn.f32x2 / add.rn.f32x2), the maximum on three inputs at a time
                float2 sum2 = make_float2(0.0f, 0.0f), sum2b = make_float2(0.0f, 0.0f);
                const float2 c2 = make_float2(p.scale_log2, p.scale_log2), nmb2 = make_float2(-mb, -mb);
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float2 t = __ffma2_rn(make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1])), c2, nmb2);
                    float2 e = make_float2(ex2_approx(t.x), ex2_approx(t.y));                   // exp2(-inf) = 0 for masked entries
                    if (i & 2) sum2b = __fadd2_rn(sum2b, e); else sum2 = __fadd2_rn(sum2, e);     // two chains
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(e.x, e.y);
                    packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h2);
                }
                const float sum = (sum2.x + sum2.y) + (sum2b.x + sum2b.y);
                // P buffer sb was last read by the P V two steps back
                if (g >= 2) { ok = pv_done(g - 2); if (!ok) break; }
                uint8_t* prow = smem + L::kP + sb * L::kPBytes + prow_off;
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int chunk = (ch * 4 + q) ^ rx;               // 32 columns = 64 bytes = 16-byte chunks ch*4 .. ch*4+3
                    *reinterpret_cast<uint4*>(prow + chunk * 16) = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P visible to the MMA's async-proxy reads
                SPT_TICK(3);
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full + 8 * sb);
                l += sum;
                SPT_TICK(4);
            }
            if (!ok) break;
            SPT_TICK(5);
            // total row sum = own half + partner's half
            float* xm = xmax + (px & 1) * 256;
            xm[ch * 128 + r] = l;
            __syncwarp();
            if (lane == 0) mbar_arrive(pair_bar);
            ok = mbar_wait(pair_bar, px & 1, abort_flag, p.status, kErrEpilogueWait);
            if (!ok) break;
            px++;
            const float inv = 1.0f / (l + xm[(ch ^ 1) * 128 + r]);
            ok = pv_done(g - 1);                                       // the item's last product
            if (!ok) break;
            tc_fence_after();
            __nv_bfloat16* orow = p.out + ((long long)bb * p.T + qrow) * p.ld_out + (long long)hh * HD + ch * OC;
#pragma unroll
            for (int c = 0; c < OC / 32; c++) {
                uint32_t o[32];
                tmem_ld_32x32(o_addr + c * 32, o);
                tmem_ld_wait();
                if (qrow < p.T) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        uint4 w;
                        __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&w);
#pragma unroll
                        for (int q = 0; q < 4; q++) oh[q] = __floats2bfloat162_rn(__uint_as_float(o[i + 2 * q]) * inv, __uint_as_float(o[i + 2 * q + 1]) * inv);
                        *reinterpret_cast<uint4*>(orow + c * 32 + i) = w;
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(o_free + 8 * (it & 1));         // the accumulator may be overwritten by the item after next
            it++;
            SPT_TICK(6);
        }
        if (pr) { for (int i = 0; i < 8; i++) p.prof[i] = pc[i]; }
#undef SPT_TICK
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        unsigned long long t0 = globaltimer();
        while (globaltimer() - t0 < 200000ull) { }
        __syncthreads();
    }
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, TMEM_COLS); }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn attn_encode() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* q = nullptr;
        cudaDriverEntryPointQueryResult r;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &q, cudaEnableDefault, &r) == cudaSuccess && r == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)q;
    });
    return fn;
}

// bf16 rank-4 map: dims (d0, d1, H, B) with element strides (1, s1, sH, sB), box (64, box1, 1, 1), 128-byte swizzle
static int encode4(CUtensorMap* map, const void* ptr, long long d0, long long d1, int H, int B, long long s1, long long sH, long long sB, int box1) {
    EncodeTiledFn enc = attn_encode();
    if (!enc) return fail("cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[4] = {(cuuint64_t)d0, (cuuint64_t)d1, (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t st[3] = {(cuuint64_t)s1 * 2, (cuuint64_t)(H > 1 ? sH : s1) * 2, (cuuint64_t)(B > 1 ? sB : s1) * 2};
    cuuint32_t box[4] = {64, (cuuint32_t)box1, 1, 1};
    cuuint32_t es[4] = {1, 1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, st, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("attention: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return 0;
}

// diagnostics: when SPTORCH_B200_ATTN_PROF is set, CTA 0 of every fused-attention launch records where one softmax
// thread and the MMA thread spend their cycles (read back with sptorch_ext_debug_attn_prof)
static unsigned long long* g_attn_prof = nullptr;
static unsigned long long* attn_prof_buffer() {
    static const bool on = getenv("SPTORCH_B200_ATTN_PROF") != nullptr;
    if (!on) return nullptr;
    if (!g_attn_prof) { if (cudaMalloc(&g_attn_prof, 16 * sizeof(unsigned long long)) != cudaSuccess) g_attn_prof = nullptr; }
    return g_attn_prof;
}
extern "C" int sptorch_ext_debug_attn_prof(unsigned long long* host16) {
    if (enter() || !g_attn_prof || !host16) return 1;
    cudaStreamSynchronize(rt().stream);
    return cudaMemcpy(host16, g_attn_prof, 16 * sizeof(unsigned long long), cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : 1;
}

// Work schedule of the persistent kernel.  Items are (query tile, sequence*head); a query tile q reads the keys and values
// 0 .. 128 q + 127 of its pair, so the eight tiles of one pair re-read the same K/V.  The list is cut into groups of pairs
// whose K/V fit in L2 together, each group ordered longest tile first, and the items are dealt out in that order to the CTA
// that has the least work so far (list scheduling with cost = key tiles + 1): the tiles of a pair then run close together
// in time and their K/V come from L2 instead of DRAM, while the CTAs still finish together.
struct AttnSchedule { std::vector<int> host; int* dev = nullptr; int len = 0; };
static std::mutex g_sched_mu;
static std::map<std::array<int, 6>, AttnSchedule> g_sched;

static int attention_schedule(int B, int H, int T, int hd, int nq, int grid, const int** dev, int* len) {
    static const int l2_mb = getenv("SPTORCH_B200_ATTN_L2_MB") ? atoi(getenv("SPTORCH_B200_ATTN_L2_MB")) : 32;
    const int BH = B * H;
    const long long pair_bytes = 2LL * T * hd * 2;                       // K and V of one (sequence, head)
    long long group = l2_mb > 0 ? ((long long)l2_mb << 20) / pair_bytes : BH;
    group = group < 1 ? 1 : (group > BH ? BH : group);
    std::lock_guard<std::mutex> lk(g_sched_mu);
    AttnSchedule& s = g_sched[{B, H, T, hd, grid, (int)group}];
    if (!s.dev) {
        const int n_kv_seq = ceil_div(T, kKvTile);
        std::vector<std::vector<int>> lists(grid);
        using Slot = std::pair<long long, int>;                          // (work so far, CTA)
        std::priority_queue<Slot, std::vector<Slot>, std::greater<Slot>> heap;
        for (int c = 0; c < grid; c++) heap.push({0, c});
        for (int g0 = 0; g0 < BH; g0 += (int)group) {
            const int g1 = std::min<long long>(BH, g0 + group);
            for (int qt = nq - 1; qt >= 0; qt--) {
                const int n_kv = std::min(ceil_div(qt * kQTile + kQTile, kKvTile), n_kv_seq);
                for (int bh = g0; bh < g1; bh++) {
                    Slot t = heap.top(); heap.pop();
                    lists[t.second].push_back((nq - 1 - qt) * BH + bh);
                    heap.push({t.first + n_kv + 1, t.second});
                }
            }
        }
        size_t len_max = 0;
        for (auto& l : lists) len_max = std::max(len_max, l.size());
        s.len = (int)len_max;
        s.host.assign(len_max * grid, -1);
        for (int c = 0; c < grid; c++)
            for (size_t k = 0; k < lists[c].size(); k++) s.host[k * grid + c] = lists[c][k];
        SPT_CUDA(cudaMalloc(&s.dev, s.host.size() * sizeof(int)));
        // the host copy lives as long as the cache entry, so the copy may stay asynchronous
        SPT_CUDA(cudaMemcpyAsync(s.dev, s.host.data(), s.host.size() * sizeof(int), cudaMemcpyHostToDevice, rt().stream));
    }
    *dev = s.dev; *len = s.len;
    return 0;
}

bool attention_fused_supported(int T, int hd, long long ld_qk, long long vt_ld, long long vt_s_head, long long vt_s_batch) {
    return (hd == 64 || hd == 128) && T % 8 == 0 && ld_qk % 8 == 0 && vt_ld % 8 == 0 && vt_s_head % 8 == 0 && vt_s_batch % 8 == 0;
}

// q, k: [B*T, ld_qk] bf16, head h at columns h*hd; vt: V^T, element (b,h,e,t) at vt[b*vt_s_batch + h*vt_s_head + e*vt_ld + t];
// out: [B*T, ld_out] bf16, head h at columns h*hd.
int attention_fused(const void* q, const void* k, const void* vt, long long vt_ld, long long vt_s_head, long long vt_s_batch, void* out,
                    int B, int T, int H, int hd, long long ld_qk, long long ld_out) {
    if (!attention_fused_supported(T, hd, ld_qk, vt_ld, vt_s_head, vt_s_batch)) return fail("attention_fused: unsupported shape or stride");
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(vt) | reinterpret_cast<uintptr_t>(out)) & 15)
        return fail("attention_fused: buffers must be 16-byte aligned");
    if (ld_out % 8) return fail("attention_fused: ld_out must be a multiple of 8");
    CUtensorMap tq, tk, tv;
    if (encode4(&tq, q, hd, T, H, B, ld_qk, hd, (long long)T * ld_qk, kQTile)) return 1;
    if (encode4(&tk, k, hd, T, H, B, ld_qk, hd, (long long)T * ld_qk, kKvTile)) return 1;
    if (encode4(&tv, vt, T, hd, H, B, vt_ld, vt_s_head, vt_s_batch, hd)) return 1;
    AttnParams prm;
    prm.out = (__nv_bfloat16*)out; prm.ld_out = ld_out; prm.T = T; prm.H = H; prm.B = B;
    prm.n_qtiles = ceil_div(T, kQTile);
    prm.scale_log2 = (1.0f / sqrtf((float)hd)) * 1.4426950408889634f;
    prm.status = rt().dev_status;
    prm.prof = attn_prof_buffer();
    long long items = (long long)B * H * prm.n_qtiles;
    if (items > INT32_MAX) return fail("attention_fused: too many work items");
    const long long slots = (long long)compute_sms() * (hd == 64 ? 2 : 1);      // resident CTAs
    long long grid = items < slots ? items : slots;
    if (attention_schedule(B, H, T, hd, prm.n_qtiles, (int)grid, &prm.sched, &prm.sched_len)) return 1;
    ProfScope ps(PROF_ATTN_FUSED);
    auto launch = [&](auto kern, int smem_bytes) -> int {
        SPT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        kern<<<(unsigned)grid, kAttnThreads, smem_bytes, rt().stream>>>(tq, tk, tv, prm);
        return 0;
    };
    int lrc;
    if (hd == 64) lrc = prm.prof ? launch(attn_fused_kernel<64, true>, AttnSmem<64>::kTotal) : launch(attn_fused_kernel<64, false>, AttnSmem<64>::kTotal);
    else lrc = prm.prof ? launch(attn_fused_kernel<128, true>, AttnSmem<128>::kTotal) : launch(attn_fused_kernel<128, false>, AttnSmem<128>::kTotal);
    if (lrc) return lrc;
    SPT_LAUNCH_CHECK("attn_fused");
    return 0;
}

}  // namespace spt
