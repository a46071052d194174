// attention_fused.cu -- fused causal attention for bf16, head_dim 64 or 128 (sm_100a, tcgen05 + TMEM + TMA).
//
// Same function as crates/nn/src/lib.rs:600-637 (scores = Q K^T * 1/sqrt(hd); entries j > i set to -inf; row
// softmax; P V; heads merged back) but the [T,T] score and probability matrices never reach HBM, and the head
// split / merge and the K transpose (nn/src/lib.rs:763-793, 822-850, 879-903) are strides of the tensor maps.
//
// One CTA owns TWO 128-row query tiles of one (sequence, head) at a time and walks the 128-key tiles up to the
// diagonal with a running row maximum and row sum (the softmax is exact; only the order of the sums differs):
//
//   warp 0      TMA: both Q tiles once per work item, then per key tile K [128 keys, hd] and V [128 keys, hd]
//               (V in its natural token-major layout: it is the MN-major B operand of P V, no transposed copy)
//   warp 1      tcgen05.mma, one lane: S_g = Q_g K_j^T (M128 N128) into the TMEM buffer of tile g, and
//               O_g += P_g V_j with P read straight from TMEM; the two query tiles alternate, so the tensor
//               core works on one tile while the softmax warps work on the other
//   warps 2..5  softmax of query tile 0, warps 6..9 of query tile 1: ONE THREAD PER QUERY ROW.  A thread reads
//               its 128 scores from TMEM in four chunks of 32 (the next chunk's load in flight while one is worked on;
//               the running row maximum is the thread's own business, no other thread has a part in it), evaluates
//               2^(s*c - m*c) (part on the special-function unit, part as a cubic polynomial on the FMA pipe,
//               because the 16-per-clock exponential unit would otherwise be the limit), and writes P as bf16
//               back into the TMEM columns the scores came from
// O accumulates in TMEM over the key tiles of an item and is rescaled in place only when a row maximum grows by
// more than 2^8 (lazy rescaling).  TMEM, head size 128: S/P of tile 0 at columns 0..127, of tile 1 at 128..255, O_0 at 256,
// O_1 at 384 (512 columns, one CTA per SM).  Head size 64 (accumulators of 64 columns): THREE score buffers at 0 / 128 / 256
// that the Q K^T products take in turn, O_0 at 384, O_1 at 448 -- a tile's next scores are ready before its softmax warps
// have finished the current ones.
// Algorithmic work per (sequence, head): 2 * T(T+1) * hd FLOP; HBM traffic: Q, K, V read once per query tile
// (K/V re-reads hit L2 thanks to the work schedule below), O written once.
#include "gemm.h"
#include "sm100.cuh"
#include "../../include/sptorch_b200_ext.h"
#include <algorithm>
#include <array>
#include <type_traits>
#include <cstdlib>
#include <map>
#include <mutex>
#include <queue>
#include <vector>

namespace spt {

using namespace sm100;

constexpr int kAttnThreads = 320;           // TMA warp + MMA warp + 2 x 4 softmax warps
constexpr int kQTile = 128, kKvTile = 128;
constexpr int kQPair = 2 * kQTile;          // query rows per work item

struct AttnParams {
    __nv_bfloat16* out;
    long long ld_out;       // row stride of out in elements
    int T, H, B;
    int n_ptiles;           // 256-row query tile pairs per sequence
    float scale_log2;       // 1/sqrt(hd) * log2(e)
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

// 2^x for two values on the FMA pipe: x = n + f with n = round(x), f in [-0.5, 0.5]; 2^f by a cubic (relative error
// 7.5e-5 = 2^-13.7, far below the 2^-9 of the bf16 rounding that follows); n goes straight into the exponent field.
// x is clamped at -125 so that the exponent arithmetic cannot wrap (the result is then 2^-125, nothing in any sum).
__device__ __forceinline__ float2 ex2_poly2(float2 x) {
    const float kMagic = 12582912.0f;               // 1.5 * 2^23: adding it leaves round(x) in the low mantissa bits
    x.x = fmaxf(x.x, -125.0f); x.y = fmaxf(x.y, -125.0f);
    const float2 r = __fadd2_rn(x, make_float2(kMagic, kMagic));
    const float2 n = __fadd2_rn(r, make_float2(-kMagic, -kMagic));
    const float2 f = __ffma2_rn(n, make_float2(-1.0f, -1.0f), x);
    float2 p = __ffma2_rn(f, make_float2(0.055171654f, 0.055171654f), make_float2(0.24261113f, 0.24261113f));
    p = __ffma2_rn(p, f, make_float2(0.69326097f, 0.69326097f));
    p = __ffma2_rn(p, f, make_float2(0.99992806f, 0.99992806f));
    return make_float2(__int_as_float(__float_as_int(p.x) + (__float_as_int(r.x) << 23)),
                       __int_as_float(__float_as_int(p.y) + (__float_as_int(r.y) << 23)));
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// 32 lanes x 16 consecutive 32-bit columns: thread i of the warp owns lane (base_lane + i)
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// tcgen05.mma with the A operand in TMEM (rows = lanes, two bf16 per 32-bit column) and B in shared memory
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Shared-memory descriptor of an MN-major operand tile stored as k-rows of exactly 128 bytes (64 bf16 along the MN
// dimension) with the 128-byte swizzle: what a TMA box of {64 elements, rows} writes for a row-major [k, n] matrix.
//   leading byte offset = distance between 64-element chunks along MN (for N = 128: the second TMA box)
//   stride byte offset  = distance between groups of 8 k-rows = 1024 B
// Advancing along K by one MMA (16 rows) adds 2048 B to the start address.
__device__ __forceinline__ uint64_t make_mnmajor_sw128_desc(uint32_t smem_addr, uint32_t chunk_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(chunk_bytes >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

template <int HD>
struct AttnSmem {
    static constexpr int kStages = HD == 64 ? 4 : 2;
    static constexpr int kQTileBytes = kQTile * HD * 2;       // HD/64 k-blocks of [128 rows x 128 B]
    static constexpr int kKBytes = kKvTile * HD * 2;          // HD/64 k-blocks of [128 keys x 128 B]
    static constexpr int kVBytes = kKvTile * HD * 2;          // HD/64 chunks of [128 keys x 128 B] (64 head columns each)
    static constexpr int kStageBytes = kKBytes + kVBytes;
    static constexpr int kQ = 0;
    static constexpr int kKV = kQ + 2 * kQTileBytes;
    static constexpr int kBars = kKV + kStages * kStageBytes; // mbarriers + TMEM slot + abort flag (256 B)
    static constexpr int kTotal = kBars + 256;
};

// Persistent kernel: CTA c works through column c of a schedule built on the host (attention_schedule below), and all
// roles run straight through item boundaries (barrier phases are driven by running counters), so the loads and the
// first Q K^T of the next item are in flight while the current one drains.
template <int HD, int NPOLY, bool ROTP = true>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fused_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
    using L = AttnSmem<HD>;
    constexpr uint32_t TMEM_COLS = 512;
    constexpr uint32_t IDESC_S = make_idesc(false, 128, kKvTile);
    constexpr uint32_t IDESC_O = make_idesc(false, 128, HD) | (1u << 16);      // B operand (V) is MN-major
    constexpr int KB = HD / 64;                               // 128-byte blocks along head_dim
    constexpr int NS = L::kStages;

    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t base = smem_u32(smem);
    const uint32_t bar = base + L::kBars;
    const uint32_t q_full = bar;                    // 1
    const uint32_t q_free = q_full + 8;             // 1
    const uint32_t kv_full = q_free + 8;            // NS
    const uint32_t kv_empty = kv_full + 8 * NS;     // NS
    // Head size 64 leaves 128 TMEM columns free beside two score tiles and two 64-column accumulators: a THIRD score buffer.  The
    // three buffers go round robin to the Q K^T products in issue order (tile 0 / tile 1 alternating), so a query tile's next
    // scores are computed while its softmax warps are still on the current ones, and the softmax never waits for the tensor core
    // (ROT).  Head size 128 fills the 512 columns with two score tiles and two accumulators: buffer = query tile, as before.
    constexpr bool ROT = HD == 64 && ROTP;
    constexpr int NSB = ROT ? 3 : 2;                // score buffers
    constexpr uint32_t O_COL = ROT ? 384 : 256;     // first accumulator column
    constexpr uint32_t O_STRIDE = ROT ? 64 : 128;
    const uint32_t s_full = kv_empty + 8 * NS;      // NSB (per score buffer)
    const uint32_t p_full = s_full + 8 * 3;         // NSB
    // P V products done: two barriers per query tile, taken in turn by the tile's steps (index step & 1, phase step >> 1).  With
    // rotating score buffers a tile's softmax can finish step j before P V of step j - 1 has completed, so its wait for the
    // product of step j on a single barrier would be two phases ahead -- which a parity wait cannot tell from none; on the
    // barrier of its own parity class it is never more than one phase ahead (the product of step j + 2 needs this thread's P).
    const uint32_t pv_done = p_full + 8 * 3;        // 4: [query tile][step & 1]
    const uint32_t o_free = pv_done + 32;           // 2
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kBars + 240);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kBars + 244);
    static_assert(8 * (2 + 2 * NS + 12) <= 240, "barrier block overflows");

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int BH = p.B * p.H;
    const int n_kv_seq = (p.T + kKvTile - 1) / kKvTile;

    if ((base & 1023u) != 0) {                                // swizzled tiles need 1024-byte alignment
        if (threadIdx.x == 0) atomicOr(p.status, 0x200u);
        return;
    }
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1); mbar_init(q_free, 1);
        for (int s = 0; s < NS; s++) { mbar_init(kv_full + 8 * s, 1); mbar_init(kv_empty + 8 * s, 1); }
        for (int g = 0; g < 3; g++) {
            mbar_init(s_full + 8 * g, 1);
            mbar_init(p_full + 8 * g, 4);           // one arrival per softmax warp of the tile
        }
        for (int g = 0; g < 4; g++) mbar_init(pv_done + 8 * g, 1);
        for (int g = 0; g < 2; g++) mbar_init(o_free + 8 * g, 4);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    // step k of this CTA's list; the entry of the next step is fetched while the current item runs
    auto fetch = [&](int k) -> int { return k < p.sched_len ? __ldg(p.sched + (size_t)k * gridDim.x + blockIdx.x) : -1; };
    // work item -> (first query row, sequence, head, key tiles of query tile 0 and of query tile 1)
    auto decode = [&](int item, int& q0, int& bb, int& hh, int& n0, int& n1) {
        const int pt = p.n_ptiles - 1 - item / BH;
        const int bh = item % BH;
        bb = bh / p.H; hh = bh % p.H;
        q0 = pt * kQPair;
        n0 = min(q0 / kKvTile + 1, n_kv_seq);                             // causal: keys 0 .. q0+127
        n1 = (q0 + kQTile < p.T) ? min(q0 / kKvTile + 2, n_kv_seq) : 0;   // second tile exists only inside the sequence
    };

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) { tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); }
        bool ok = true;
        uint32_t g = 0, it = 0;
        for (int k = 0, item = fetch(0); item >= 0 && ok; k++, it++) {
            const int item_next = fetch(k + 1);
            int q0, bb, hh, n0, n1;
            decode(item, q0, bb, hh, n0, n1);
            item = item_next;
            const int nmax = max(n0, n1);
            ok = mbar_wait(q_free, (it & 1) ^ 1, abort_flag, p.status, kErrProducerWait);
            if (!ok) break;
            if (lane == 0) {
                mbar_expect_tx(q_full, 2 * L::kQTileBytes);
                for (int t = 0; t < 2; t++)
                    for (int kb = 0; kb < KB; kb++)
                        tma_load_4d(base + L::kQ + t * L::kQTileBytes + kb * (kQTile * 128), &tmQ, q_full, kb * 64, q0 + t * kQTile, hh, bb);
            }
            for (int j = 0; j < nmax && ok; j++, g++) {
                const uint32_t s = g % NS, u = (g / NS) & 1;
                ok = mbar_wait(kv_empty + 8 * s, u ^ 1, abort_flag, p.status, kErrProducerWait);
                if (!ok) break;
                if (lane == 0) {
                    const int k0 = j * kKvTile;
                    const uint32_t dst = base + L::kKV + s * L::kStageBytes;
                    mbar_expect_tx(kv_full + 8 * s, L::kStageBytes);
                    for (int kb = 0; kb < KB; kb++) tma_load_4d(dst + kb * (kKvTile * 128), &tmK, kv_full + 8 * s, kb * 64, k0, hh, bb);
                    for (int kb = 0; kb < KB; kb++) tma_load_4d(dst + L::kKBytes + kb * (kKvTile * 128), &tmV, kv_full + 8 * s, kb * 64, k0, hh, bb);
                }
                __syncwarp();
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        bool ok = true;
        uint32_t g = 0, it = 0;                 // key tiles loaded so far (stage ring position); items so far
        uint32_t steps[2] = {0, 0};             // softmax steps of each query tile so far (phases of p_full)
        // S_t = Q_t K^T with the key tile of ring position gg
        auto issue_s = [&](int t, uint32_t gg) {
            const uint32_t kaddr = base + L::kKV + (gg % NS) * L::kStageBytes;
#pragma unroll
            for (int kb = 0; kb < KB; kb++) {
                const uint64_t adesc = make_kmajor_sw128_desc(base + L::kQ + t * L::kQTileBytes + kb * (kQTile * 128));
                const uint64_t bdesc = make_kmajor_sw128_desc(kaddr + kb * (kKvTile * 128));
#pragma unroll
                for (int k = 0; k < 4; k++) mma_ss<false>(tmem_base + t * 128, adesc + 2 * k, bdesc + 2 * k, IDESC_S, (kb | k) != 0 ? 1u : 0u);
            }
            mma_commit(s_full + 8 * t);
        };
        // O_t (+)= P_t V with the value tile of ring position gg; P is read from the TMEM columns of S_t
        auto issue_pv = [&](int t, uint32_t gg, bool accumulate, uint32_t pvidx) {      // pvidx: which product of this tile (over the whole kernel)
            const uint64_t bdesc = make_mnmajor_sw128_desc(base + L::kKV + (gg % NS) * L::kStageBytes + L::kKBytes, kKvTile * 128);
#pragma unroll
            for (int k = 0; k < kKvTile / 16; k++)
                mma_ts(tmem_base + O_COL + t * O_STRIDE, tmem_base + t * 128 + 8 * k, bdesc + (uint64_t)(128 * k), IDESC_O, (accumulate || k != 0) ? 1u : 0u);
            mma_commit(pv_done + 8 * (2 * t + (pvidx & 1)));
        };
        auto kv_ready = [&](uint32_t gg) -> bool { return mbar_wait(kv_full + 8 * (gg % NS), (gg / NS) & 1, abort_flag, p.status, kErrMmaWait); };
        if constexpr (ROT) {
            // The products of an item in issue order ("entries"): key tile by key tile, query tile 0 before query tile 1 where both
            // still have that key tile.  Scores run up to two entries ahead of the P V product that is issued next; score number n
            // (counted over the whole kernel) lives in buffer n % 3, which P V number n - 3 -- issued earlier by this thread, and
            // the tensor pipe runs one thread's MMAs in order -- has finished reading.
            uint32_t G = 0;                     // scores issued in earlier items
            auto issue_s3 = [&](int t, uint32_t gg, uint32_t n) {
                const uint32_t buf = n % 3;
                const uint32_t kaddr = base + L::kKV + (gg % NS) * L::kStageBytes;
#pragma unroll
                for (int kb = 0; kb < KB; kb++) {
                    const uint64_t adesc = make_kmajor_sw128_desc(base + L::kQ + t * L::kQTileBytes + kb * (kQTile * 128));
                    const uint64_t bdesc = make_kmajor_sw128_desc(kaddr + kb * (kKvTile * 128));
#pragma unroll
                    for (int k = 0; k < 4; k++) mma_ss<false>(tmem_base + buf * 128, adesc + 2 * k, bdesc + 2 * k, IDESC_S, (kb | k) != 0 ? 1u : 0u);
                }
                mma_commit(s_full + 8 * buf);
            };
            auto issue_pv3 = [&](int t, uint32_t gg, uint32_t n, bool accumulate, uint32_t pvidx) {
                const uint32_t buf = n % 3;
                const uint64_t bdesc = make_mnmajor_sw128_desc(base + L::kKV + (gg % NS) * L::kStageBytes + L::kKBytes, kKvTile * 128);
#pragma unroll
                for (int k = 0; k < kKvTile / 16; k++)
                    mma_ts(tmem_base + O_COL + t * O_STRIDE, tmem_base + buf * 128 + 8 * k, bdesc + (uint64_t)(128 * k), IDESC_O, (accumulate || k != 0) ? 1u : 0u);
                mma_commit(pv_done + 8 * (2 * t + (pvidx & 1)));
            };
            for (int k = 0, item = fetch(0); item >= 0 && ok; k++, it++) {
                const int item_next = fetch(k + 1);
                int q0, bb, hh, n0, n1;
                decode(item, q0, bb, hh, n0, n1);
                item = item_next;
                const int E = n0 + n1, nmin = min(n0, n1), t_long = n1 > n0 ? 1 : 0;
                auto entry = [&](int e, int& t, int& j) {
                    if (e < 2 * nmin) { j = e >> 1; t = e & 1; } else { j = nmin + (e - 2 * nmin); t = t_long; }
                };
                ok = mbar_wait(q_full, it & 1, abort_flag, p.status, kErrMmaWait);
                if (!ok) break;
                int issued = 0, kv_seen = -1;
                for (int e = 0; e < E && ok; e++) {
                    while (issued < min(E, e + 3)) {
                        int ts, js;
                        entry(issued, ts, js);
                        if (js > kv_seen) { ok = kv_ready(g + js); kv_seen = js; if (!ok) break; }
                        tc_fence_after();
                        if (elect_one_sync()) {
                            issue_s3(ts, g + js, G + issued);
                            if (issued == E - 1) mma_commit(q_free);            // the item's last read of Q
                        }
                        __syncwarp();
                        issued++;
                    }
                    if (!ok) break;
                    int t, j;
                    entry(e, t, j);
                    const uint32_t n = G + e, buf = n % 3;
                    ok = mbar_wait(p_full + 8 * buf, (n / 3) & 1, abort_flag, p.status, kErrMmaWait);
                    // the item's first product overwrites the accumulator: the previous item's output must have been read
                    if (ok && j == 0) ok = mbar_wait(o_free + 8 * t, (it & 1) ^ 1, abort_flag, p.status, kErrMmaWait);
                    if (!ok) break;
                    tc_fence_after();
                    int tn = 0, jn = -1;
                    if (e + 1 < E) entry(e + 1, tn, jn);
                    if (elect_one_sync()) {
                        issue_pv3(t, g + j, n, j > 0, steps[t]);
                        if (jn != j) mma_commit(kv_empty + 8 * ((g + j) % NS));     // every MMA that reads this stage has been issued
                    }
                    __syncwarp();
                    steps[t]++;
                }
                g += max(n0, n1);
                G += E;
            }
        } else
        for (int k = 0, item = fetch(0); item >= 0 && ok; k++, it++) {
            const int item_next = fetch(k + 1);
            int q0, bb, hh, n0, n1;
            decode(item, q0, bb, hh, n0, n1);
            item = item_next;
            const int nt[2] = {n0, n1};
            const int nmax = max(n0, n1);
            const int last_t = n1 > 0 ? 1 : 0;             // the tile whose last Q K^T is the item's last read of Q
            ok = mbar_wait(q_full, it & 1, abort_flag, p.status, kErrMmaWait) && kv_ready(g);
            if (!ok) break;
            tc_fence_after();
            if (elect_one_sync()) {
                issue_s(0, g);
                if (n1 > 0) issue_s(1, g);
                if (nt[last_t] == 1) mma_commit(q_free);
            }
            __syncwarp();
            for (int j = 0; j < nmax && ok; j++, g++) {
                if (j + 1 < nmax) { ok = kv_ready(g + 1); if (!ok) break; }
                for (int t = 0; t < 2 && ok; t++) {
                    if (j >= nt[t]) continue;
                    ok = mbar_wait(p_full + 8 * t, steps[t] & 1, abort_flag, p.status, kErrMmaWait);
                    // the item's first product overwrites the accumulator: the previous item's output must have been read
                    if (ok && j == 0) ok = mbar_wait(o_free + 8 * t, (it & 1) ^ 1, abort_flag, p.status, kErrMmaWait);
                    if (!ok) break;
                    steps[t]++;
                    tc_fence_after();
                    if (elect_one_sync()) {
                        issue_pv(t, g, j > 0, steps[t] - 1);
                        // the next scores of this tile go into the columns P was just read from: the tensor pipe runs the
                        // MMAs of one thread in order, so the product above has consumed P before these overwrite it
                        if (j + 1 < nt[t]) {
                            issue_s(t, g + 1);
                            if (t == last_t && j + 2 == nt[t]) mma_commit(q_free);
                        }
                    }
                    __syncwarp();
                }
                if (ok && elect_one_sync()) mma_commit(kv_empty + 8 * (g % NS));     // every MMA that reads this stage has been issued
                __syncwarp();
            }
        }
    } else {
        // ---------------- softmax + output: one thread per query row ----------------
        const int t = (warp - 2) >> 2;                           // query tile of this warp
        const int quarter = warp & 3;                            // TMEM lane quarter a warp may access = warp index % 4
        const int r = quarter * 32 + lane;                       // row inside the tile = TMEM lane
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        const uint32_t o_addr = tmem_base + lane_off + O_COL + t * O_STRIDE;
        bool ok = true;
        uint32_t step = 0, it = 0;                               // softmax steps of this tile so far; items so far
        uint32_t G = 0;                                          // ROT: scores of earlier items (both tiles), as the MMA warp counts them
        for (int k = 0, item = fetch(0); item >= 0 && ok; k++, it++) {
            const int item_next = fetch(k + 1);
            int q0, bb, hh, n0, n1;
            decode(item, q0, bb, hh, n0, n1);
            item = item_next;
            const int n_kv = t == 0 ? n0 : n1;
            const int qrow = q0 + t * kQTile + r;
            float m = -INFINITY, l = 0.0f;
            for (int j = 0; j < n_kv && ok; j++, step++) {
                // ROT: this step's scores are number G + (entries of the item before (t, j)) of the kernel, in buffer number % 3
                const uint32_t sn = ROT ? G + (uint32_t)(min(j, n0) + min(j, n1) + ((t == 1 && j < n0) ? 1 : 0)) : step;
                const uint32_t sbuf = ROT ? sn % 3 : (uint32_t)t;
                const uint32_t s_addr = tmem_base + lane_off + sbuf * 128;          // scores, and P over their first 64 columns
                ok = mbar_wait(s_full + 8 * sbuf, (ROT ? sn / 3 : sn) & 1, abort_flag, p.status, kErrEpilogueWait);
                if (!ok) break;
                tc_fence_after();
                const bool diag = (j == n_kv - 1);               // the tile on the diagonal: keys q .. q+127 of rows q .. q+127
                // The 128 scores of the row are taken in four chunks of 32: the load of chunk c + 1 is in flight while chunk c is
                // worked on, and a chunk needs only 32 registers.  The reference maximum m of the row is allowed to lag the true
                // maximum by up to 2^8 (lazy rescaling): a chunk whose maximum exceeds m by more moves m, and everything already
                // accumulated under the old m -- the row sum, the output in TMEM, and the chunks of P of this tile that are already
                // written -- is multiplied by 2^(old - new) at that moment.  tcgen05.ld / st are warp-wide, so a warp rescales when any
                // of its rows does (the others multiply by one).
                float2 sum_a = make_float2(0.0f, 0.0f), sum_b = make_float2(0.0f, 0.0f);
                const float2 c2 = make_float2(p.scale_log2, p.scale_log2);
                uint32_t va[32], vb[32];
                tmem_ld_32x32(s_addr, va);
                auto chunk = [&](auto c_tag, uint32_t (&v)[32], uint32_t (&vnext)[32], auto npoly_tag, auto diag_tag) -> bool {
                    constexpr int c = decltype(c_tag)::value;
                    constexpr int NP = decltype(npoly_tag)::value;
                    constexpr bool DIAG = decltype(diag_tag)::value;
                    tmem_ld_wait();
                    if (c < 3) tmem_ld_32x32(s_addr + (c + 1) * 32, vnext);
                    if (DIAG) {
#pragma unroll
                        for (int i = 0; i < 32; i++) if (c * 32 + i > r) v[i] = 0xff800000u;       // -inf right of the diagonal
                    }
                    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        m0 = max3(m0, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                        m1 = max3(m1, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
                        m2 = max3(m2, __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
                        m3 = max3(m3, __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
                    }
                    const float mx = fmaxf(max3(m0, m1, m2), m3);
                    if (j == 0 && c == 0) m = mx;                    // the first chunk of a row always holds key 0: finite
                    const bool grow = (mx - m) * p.scale_log2 > 8.0f;
                    if (__any_sync(0xffffffffu, grow)) {
                        float alpha = 1.0f;
                        if (grow) { alpha = ex2_approx((m - mx) * p.scale_log2); m = mx; }
                        l *= alpha;
                        sum_a.x *= alpha; sum_a.y *= alpha; sum_b.x *= alpha; sum_b.y *= alpha;
                        if (j > 0) {
                            // every product accumulated so far is in place (the commit of step - 1; the next one needs this thread's P)
                            if (!mbar_wait(pv_done + 8 * (2 * t + ((step - 1) & 1)), ((step - 1) >> 1) & 1, abort_flag, p.status, kErrEpilogueWait)) return false;
                            tc_fence_after();
#pragma unroll
                            for (int cc = 0; cc < HD / 32; cc++) {
                                uint32_t o[32];
                                tmem_ld_32x32(o_addr + cc * 32, o);
                                tmem_ld_wait();
#pragma unroll
                                for (int i = 0; i < 32; i++) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                                tmem_st_32x32(o_addr + cc * 32, o);
                            }
                        }
                        if (c > 0) {
                            // the chunks of P of this tile written so far: 16 columns (32 bf16) each
                            uint32_t w[16];
#pragma unroll
                            for (int cc = 0; cc < c; cc++) {
                                tmem_ld_32x32b_x16(s_addr + cc * 16, w);
                                tmem_ld_wait();
#pragma unroll
                                for (int i = 0; i < 16; i++) {
                                    const float lo = __uint_as_float(w[i] << 16) * alpha, hi = __uint_as_float(w[i] & 0xffff0000u) * alpha;
                                    __nv_bfloat162 h2 = __floats2bfloat162_rn(lo, hi);
                                    w[i] = *reinterpret_cast<uint32_t*>(&h2);
                                }
                                tmem_st_32x32b_x16(s_addr + cc * 16, w);
                            }
                        }
                        tmem_st_wait();
                        // the load of the next chunk was issued before this branch: the wait of the next chunk() call still covers it
                    }
                    const float mb = m * p.scale_log2;
                    const float2 nmb2 = make_float2(-mb, -mb);
                    uint32_t packed[16];
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const float2 x = __ffma2_rn(make_float2(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1])), c2, nmb2);
                        float2 e;
                        if (i < NP) e = ex2_poly2(x);
                        else e = make_float2(ex2_approx(x.x), ex2_approx(x.y));
                        if (i & 1) sum_b = __fadd2_rn(sum_b, e); else sum_a = __fadd2_rn(sum_a, e);
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(e.x, e.y);
                        packed[i] = *reinterpret_cast<uint32_t*>(&h2);
                    }
                    // keys 32c .. 32c+31 of this row, two per column: columns 16c .. 16c+15, whose scores have been read (c' <= c)
                    tmem_st_32x32b_x16(s_addr + c * 16, packed);
                    return true;
                };
                auto tile = [&](auto npoly_tag, auto diag_tag) -> bool {
                    return chunk(std::integral_constant<int, 0>(), va, vb, npoly_tag, diag_tag) &&
                           chunk(std::integral_constant<int, 1>(), vb, va, npoly_tag, diag_tag) &&
                           chunk(std::integral_constant<int, 2>(), va, vb, npoly_tag, diag_tag) &&
                           chunk(std::integral_constant<int, 3>(), vb, va, npoly_tag, diag_tag);
                };
                ok = diag ? tile(std::integral_constant<int, 0>(), std::true_type()) : tile(std::integral_constant<int, NPOLY>(), std::false_type());
                if (!ok) break;
                tmem_st_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full + 8 * sbuf);
                l += (sum_a.x + sum_a.y) + (sum_b.x + sum_b.y);
            }
            G += (uint32_t)(n0 + n1);
            if (!ok) break;
            if (n_kv > 0) {
                const float inv = 1.0f / l;
                ok = mbar_wait(pv_done + 8 * (2 * t + ((step - 1) & 1)), ((step - 1) >> 1) & 1, abort_flag, p.status, kErrEpilogueWait);     // the item's last product
                if (!ok) break;
                tc_fence_after();
                __nv_bfloat16* orow = p.out + ((long long)bb * p.T + qrow) * p.ld_out + (long long)hh * HD;
#pragma unroll
                for (int c = 0; c < HD / 32; c++) {
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
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(o_free + 8 * t);              // the accumulator may be overwritten by the next item
        }
    }

    tc_fence_before();
    __syncthreads();
    if (*abort_flag) {
        // give loads that may still be in flight time to land before shared memory is released
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

// bf16 rank-4 map over a token-major [B*T, ld] matrix seen as (head_dim, T, H, B): box (64, 128, 1, 1), 128-byte swizzle.
// Rows past T read as zero (they belong to the next sequence in memory, but the T dimension of the map ends there).
static int encode_heads(CUtensorMap* map, const void* ptr, int hd, int T, int H, int B, long long ld) {
    EncodeTiledFn enc = attn_encode();
    if (!enc) return fail("cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[4] = {(cuuint64_t)hd, (cuuint64_t)T, (cuuint64_t)H, (cuuint64_t)B};
    cuuint64_t st[3] = {(cuuint64_t)ld * 2, (cuuint64_t)(H > 1 ? hd : ld) * 2, (cuuint64_t)(B > 1 ? (long long)T * ld : ld) * 2};
    cuuint32_t box[4] = {64, 128, 1, 1};
    cuuint32_t es[4] = {1, 1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, st, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("attention: cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return 0;
}

// Work schedule of the persistent kernel.  Items are (query tile pair, sequence*head); pair q reads the keys and values
// 0 .. 256 q + 255 of its (sequence, head), so the tiles of one (sequence, head) re-read the same K/V.  The list is cut into
// groups of (sequence, head)s whose K/V fit in L2 together, each group ordered longest item first, and the items are dealt out
// in that order to the CTA that has the least work so far (list scheduling, cost = key tiles of both query tiles + 1): the
// items of one (sequence, head) then run close together in time and their K/V come from L2 instead of DRAM, while the CTAs
// still finish together.  Schedules are cached per shape and released when the backend shuts down.
struct AttnSchedule { std::vector<int> host; int* dev = nullptr; int len = 0; };
static std::mutex g_sched_mu;
static std::map<std::array<int, 6>, AttnSchedule> g_sched;

static void attention_schedules_release() {
    std::lock_guard<std::mutex> lk(g_sched_mu);
    for (auto& kv : g_sched) if (kv.second.dev) cudaFree(kv.second.dev);
    g_sched.clear();
}

static int attention_schedule(int B, int H, int T, int hd, int npt, int grid, const int** dev, int* len) {
    static const int l2_mb = getenv("SPTORCH_B200_ATTN_L2_MB") ? atoi(getenv("SPTORCH_B200_ATTN_L2_MB")) : 32;
    const int BH = B * H;
    const long long pair_bytes = 2LL * T * hd * 2;                       // K and V of one (sequence, head)
    long long group = l2_mb > 0 ? ((long long)l2_mb << 20) / pair_bytes : BH;
    group = group < 1 ? 1 : (group > BH ? BH : group);
    std::lock_guard<std::mutex> lk(g_sched_mu);
    if (g_sched.size() > 64) {                                           // a bound on the cache: drop everything not in flight
        if (stream_wait()) return 1;
        for (auto& kv : g_sched) if (kv.second.dev) cudaFree(kv.second.dev);
        g_sched.clear();
    }
    AttnSchedule& s = g_sched[{B, H, T, hd, grid, (int)group}];
    if (!s.dev) {
        at_shutdown(attention_schedules_release);
        const int n_kv_seq = ceil_div(T, kKvTile);
        std::vector<std::vector<int>> lists(grid);
        using Slot = std::pair<long long, int>;                          // (work so far, CTA)
        std::priority_queue<Slot, std::vector<Slot>, std::greater<Slot>> heap;
        for (int c = 0; c < grid; c++) heap.push({0, c});
        for (int g0 = 0; g0 < BH; g0 += (int)group) {
            const int g1 = std::min<long long>(BH, g0 + group);
            for (int pt = npt - 1; pt >= 0; pt--) {
                const int q0 = pt * kQPair;
                const int n0 = std::min(q0 / kKvTile + 1, n_kv_seq);
                const int n1 = q0 + kQTile < T ? std::min(q0 / kKvTile + 2, n_kv_seq) : 0;
                for (int bh = g0; bh < g1; bh++) {
                    Slot t = heap.top(); heap.pop();
                    lists[t.second].push_back((npt - 1 - pt) * BH + bh);
                    heap.push({t.first + n0 + n1 + 1, t.second});
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

bool attention_fused_supported(int T, int hd, long long ld_q, long long ld_kv) {
    return (hd == 64 || hd == 128) && T > 0 && ld_q % 8 == 0 && ld_kv % 8 == 0;
}

// share of the exponentials evaluated on the FMA pipe (of every 16 pairs), per head size; tunable for experiments
static int attn_npoly(int hd) {
    static const int e64 = getenv("SPTORCH_B200_ATTN_NPOLY64") ? atoi(getenv("SPTORCH_B200_ATTN_NPOLY64")) : 0;
    static const int e128 = getenv("SPTORCH_B200_ATTN_NPOLY128") ? atoi(getenv("SPTORCH_B200_ATTN_NPOLY128")) : 0;
    return hd == 64 ? e64 : e128;
}

// q, k, v: [B*T, ld] bf16, head h at columns h*hd (token-major: the layout the QKV projection writes);
// out: [B*T, ld_out] bf16, head h at columns h*hd.
int attention_fused(const void* q, const void* k, const void* v, void* out, int B, int T, int H, int hd, long long ld_q, long long ld_k,
                    long long ld_v, long long ld_out) {
    if (!attention_fused_supported(T, hd, ld_q, ld_k) || ld_v % 8) return fail("attention_fused: unsupported shape or stride");
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out)) & 15)
        return fail("attention_fused: buffers must be 16-byte aligned");
    if (ld_out % 8) return fail("attention_fused: ld_out must be a multiple of 8");
    CUtensorMap tq, tk, tv;
    if (encode_heads(&tq, q, hd, T, H, B, ld_q)) return 1;
    if (encode_heads(&tk, k, hd, T, H, B, ld_k)) return 1;
    if (encode_heads(&tv, v, hd, T, H, B, ld_v)) return 1;
    AttnParams prm;
    prm.out = (__nv_bfloat16*)out; prm.ld_out = ld_out; prm.T = T; prm.H = H; prm.B = B;
    prm.n_ptiles = ceil_div(T, kQPair);
    prm.scale_log2 = (1.0f / sqrtf((float)hd)) * 1.4426950408889634f;
    prm.status = rt().dev_status;
    long long items = (long long)B * H * prm.n_ptiles;
    if (items > INT32_MAX) return fail("attention_fused: too many work items");
    const long long slots = compute_sms();                                      // one resident CTA per SM
    long long grid = items < slots ? items : slots;
    if (attention_schedule(B, H, T, hd, prm.n_ptiles, (int)grid, &prm.sched, &prm.sched_len)) return 1;
    ProfScope ps(PROF_ATTN_FUSED);
    auto launch = [&](auto kern, int smem_bytes) -> int {
        SPT_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
        kern<<<(unsigned)grid, kAttnThreads, smem_bytes, rt().stream>>>(tq, tk, tv, prm);
        return 0;
    };
    const int np = attn_npoly(hd);
    int lrc;
    if (hd == 64) {
        static const bool rot_off = getenv("SPTORCH_B200_ATTN_ROT") && atoi(getenv("SPTORCH_B200_ATTN_ROT")) == 0;
        if (rot_off) lrc = launch(attn_fused_kernel<64, 0, false>, AttnSmem<64>::kTotal);
        else if (np <= 0) lrc = launch(attn_fused_kernel<64, 0>, AttnSmem<64>::kTotal);
        else if (np <= 4) lrc = launch(attn_fused_kernel<64, 4>, AttnSmem<64>::kTotal);
        else if (np <= 5) lrc = launch(attn_fused_kernel<64, 5>, AttnSmem<64>::kTotal);
        else if (np <= 6) lrc = launch(attn_fused_kernel<64, 6>, AttnSmem<64>::kTotal);
        else lrc = launch(attn_fused_kernel<64, 8>, AttnSmem<64>::kTotal);
    } else {
        if (np <= 0) lrc = launch(attn_fused_kernel<128, 0>, AttnSmem<128>::kTotal);
        else lrc = launch(attn_fused_kernel<128, 4>, AttnSmem<128>::kTotal);
    }
    if (lrc) return lrc;
    SPT_LAUNCH_CHECK("attn_fused");
    return 0;
}

}  // namespace spt
