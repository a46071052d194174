// attention_fused.cu -- fused causal attention for bf16, head_dim 64 or 128 (sm_100a, tcgen05 + TMEM + TMA).
//
// Same function as crates/nn/src/lib.rs:600-637 (scores = Q K^T * 1/sqrt(hd); entries j > i set to -inf; row
// softmax; P V; heads merged back) but the [T,T] score and probability matrices never reach HBM: one CTA owns
// one 128-row query tile of one (sequence, head) and walks the key/value tiles 0..diagonal with a running
// row maximum and row sum (the softmax is computed exactly; only the order of the sums differs).
//
//   warp 0      TMA: Q tile once, then K tile [128 keys, hd] and V^T tile [hd, 128 keys] per step, 2-stage ring
//   warp 1      tcgen05.mma: S = Q K^T (M128 N128) into TMEM, later O_j = P V (M128 N=hd) into TMEM
//   warps 2..5  one thread per query row: tcgen05.ld S twice (row max, then exp2), causal mask on the diagonal
//               tile, P written to shared memory as bf16 in the 128-byte-swizzled K-major layout that the P V
//               MMA reads, O_j read back from TMEM and folded into a register accumulator with the rescale factor
// Two CTAs are resident per SM for hd = 64 (112 KB of shared memory and 256 TMEM columns each), so one CTA's
// softmax overlaps the other's MMAs.  Heavy (late) query tiles are scheduled first.
// Algorithmic work per (sequence, head): 2 * T(T+1) * hd FLOP; HBM traffic Q, K, V read once per query tile pass
// (K/V re-reads hit L2), O written once.
#include "gemm.h"
#include "sm100.cuh"
#include "../../include/sptorch_b200_ext.h"

namespace spt {

using namespace sm100;

constexpr int kAttnThreads = 192;
constexpr int kQTile = 128, kKvTile = 128;

struct AttnParams {
    __nv_bfloat16* out;
    long long ld_out;       // row stride of out in elements
    int T, H, B;
    int n_qtiles;
    float scale_log2;       // 1/sqrt(hd) * log2(e)
    uint32_t* status;
};

// 2^x on the special-function unit: one instruction, relative error 2^-22 (P is rounded to bf16 right after)
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int HD>
struct AttnSmem {
    static constexpr int kQBytes = kQTile * HD * 2;
    static constexpr int kKBytes = kKvTile * HD * 2;
    static constexpr int kVBytes = HD * kKvTile * 2;
    static constexpr int kPBytes = kQTile * kKvTile * 2;
    static constexpr int kQ = 0;
    static constexpr int kK = kQ + kQBytes;
    static constexpr int kV = kK + 2 * kKBytes;
    static constexpr int kP = kV + 2 * kVBytes;
    static constexpr int kBars = kP + kPBytes;
    static constexpr int kTotal = kBars + 128;
};

template <int HD>
__global__ void __launch_bounds__(kAttnThreads, HD == 64 ? 2 : 1)
attn_fused_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                  const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
    using L = AttnSmem<HD>;
    constexpr uint32_t TMEM_COLS = 256;                     // S: columns [0,128), O_j: [128, 128+HD)
    constexpr uint32_t IDESC_S = make_idesc(false, 128, kKvTile);
    constexpr uint32_t IDESC_O = make_idesc(false, 128, HD);
    constexpr int KB_Q = HD / 64;                           // 128-byte k-blocks along head_dim
    constexpr int KB_P = kKvTile / 64;                      // 128-byte k-blocks along the keys

    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t base = smem_u32(smem);
    // barrier slots (8 bytes each)
    const uint32_t bar = base + L::kBars;
    const uint32_t q_full = bar, k_full = bar + 8, v_full = bar + 24, kv_empty = bar + 40, s_full = bar + 56, s_free = bar + 64,
                   p_full = bar + 72, o_full = bar + 80, o_free = bar + 88;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + L::kBars + 96);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + L::kBars + 100);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int BH = p.B * p.H;
    const int qt = p.n_qtiles - 1 - (int)(blockIdx.x / BH);   // heavy tiles first
    const int bh = (int)(blockIdx.x % BH);
    const int b = bh / p.H, h = bh % p.H;
    const int q0 = qt * kQTile;
    const int n_kv = qt + 1;                                  // causal: key tiles 0..qt

    if ((base & 1023u) != 0) {                                // swizzled tiles need 1024-byte alignment
        if (threadIdx.x == 0) atomicOr(p.status, 0x200u);
        return;
    }
    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int s = 0; s < 2; s++) { mbar_init(k_full + 8 * s, 1); mbar_init(v_full + 8 * s, 1); mbar_init(kv_empty + 8 * s, 1); }
        mbar_init(s_full, 1); mbar_init(s_free, 128); mbar_init(p_full, 128); mbar_init(o_full, 1); mbar_init(o_free, 128);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + 128;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV);
            mbar_expect_tx(q_full, L::kQBytes);
            for (int kb = 0; kb < KB_Q; kb++) tma_load_4d(base + L::kQ + kb * (kQTile * 128), &tmQ, q_full, kb * 64, q0, h, b);
        }
        bool ok = true;
        for (int j = 0; j < n_kv && ok; j++) {
            const int s = j & 1; const uint32_t ph = (j >> 1) & 1;
            ok = mbar_wait(kv_empty + 8 * s, ph ^ 1, abort_flag, p.status, kErrProducerWait);
            if (!ok) break;
            if (lane == 0) {
                const int k0 = j * kKvTile;
                mbar_expect_tx(k_full + 8 * s, L::kKBytes);
                for (int kb = 0; kb < KB_Q; kb++) tma_load_4d(base + L::kK + s * L::kKBytes + kb * (kKvTile * 128), &tmK, k_full + 8 * s, kb * 64, k0, h, b);
                mbar_expect_tx(v_full + 8 * s, L::kVBytes);
                for (int kb = 0; kb < KB_P; kb++) tma_load_4d(base + L::kV + s * L::kVBytes + kb * (HD * 128), &tmV, v_full + 8 * s, k0 + kb * 64, 0, h, b);
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        bool ok = mbar_wait(q_full, 0, abort_flag, p.status, kErrMmaWait);
        for (int j = 0; j < n_kv && ok; j++) {
            const int s = j & 1; const uint32_t ph = (j >> 1) & 1, it = j & 1;
            ok = mbar_wait(k_full + 8 * s, ph, abort_flag, p.status, kErrMmaWait) &&
                 mbar_wait(s_free, it ^ 1, abort_flag, p.status, kErrMmaWait);
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
#pragma unroll
                for (int kb = 0; kb < KB_Q; kb++) {
                    const uint64_t adesc = make_kmajor_sw128_desc(base + L::kQ + kb * (kQTile * 128));
                    const uint64_t bdesc = make_kmajor_sw128_desc(base + L::kK + s * L::kKBytes + kb * (kKvTile * 128));
#pragma unroll
                    for (int k = 0; k < 4; k++) mma_ss<false>(tmem_s, adesc + 2 * k, bdesc + 2 * k, IDESC_S, (kb | k) != 0 ? 1u : 0u);
                }
                mma_commit(s_full);
            }
            __syncwarp();
            ok = mbar_wait(p_full, it, abort_flag, p.status, kErrMmaWait) &&
                 mbar_wait(v_full + 8 * s, ph, abort_flag, p.status, kErrMmaWait) &&
                 mbar_wait(o_free, it ^ 1, abort_flag, p.status, kErrMmaWait);
            if (!ok) break;
            tc_fence_after();
            if (lane == 0) {
#pragma unroll
                for (int kb = 0; kb < KB_P; kb++) {
                    const uint64_t adesc = make_kmajor_sw128_desc(base + L::kP + kb * (kQTile * 128));
                    const uint64_t bdesc = make_kmajor_sw128_desc(base + L::kV + s * L::kVBytes + kb * (HD * 128));
#pragma unroll
                    for (int k = 0; k < 4; k++) mma_ss<false>(tmem_o, adesc + 2 * k, bdesc + 2 * k, IDESC_O, (kb | k) != 0 ? 1u : 0u);
                }
                mma_commit(o_full);
                mma_commit(kv_empty + 8 * s);
            }
            __syncwarp();
        }
    } else {
        // ---------------- softmax + accumulate: thread owns one query row ----------------
        const int quarter = warp & 3;
        const int r = quarter * 32 + lane;                       // row inside the tile = TMEM lane
        const uint32_t lane_off = (uint32_t)(quarter * 32) << 16;
        const int qrow = q0 + r;
        float m = -INFINITY, l = 0.0f;
        float O[HD];
#pragma unroll
        for (int i = 0; i < HD; i++) O[i] = 0.0f;
        uint8_t* prow = smem + L::kP + (r >> 3) * 1024 + (r & 7) * 128;   // row r of a 128-row, 128-byte-pitch swizzled block
        const int rx = r & 7;
        bool ok = true;
        for (int j = 0; j < n_kv && ok; j++) {
            const uint32_t it = j & 1;
            const bool diag = (j == qt);
            const int k0 = j * kKvTile;
            ok = mbar_wait(s_full, it, abort_flag, p.status, kErrEpilogueWait);
            if (!ok) break;
            tc_fence_after();
            // pass 1: row maximum of the unmasked entries
            float mx = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < kKvTile / 32; c++) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_s + lane_off + c * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    float sv = __uint_as_float(v[i]);
                    if (diag && (k0 + c * 32 + i > qrow)) sv = -INFINITY;
                    mx = fmaxf(mx, sv);
                }
            }
            const float m_new = fmaxf(m, mx);
            const float alpha = ex2_approx((m - m_new) * p.scale_log2);       // 0 on the first tile (m = -inf)
            const float mb = m_new * p.scale_log2;
            // pass 2: p = exp2(s*c - m*c), row sum, bf16 P into shared memory
            float sum = 0.0f;
#pragma unroll 1
            for (int c = 0; c < kKvTile / 32; c++) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_s + lane_off + c * 32, v);
                tmem_ld_wait();
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float a0 = __uint_as_float(v[i]), a1 = __uint_as_float(v[i + 1]);
                    float e0 = ex2_approx(fmaf(a0, p.scale_log2, -mb)), e1 = ex2_approx(fmaf(a1, p.scale_log2, -mb));
                    if (diag) {
                        if (k0 + c * 32 + i > qrow) e0 = 0.0f;
                        if (k0 + c * 32 + i + 1 > qrow) e1 = 0.0f;
                    }
                    sum += e0 + e1;
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(e0, e1);
                    packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h2);
                }
                // columns c*32 .. c*32+31 = 64 bytes = four 16-byte chunks of k-block (c/2), chunk index (c%2)*4 + q
                uint8_t* blk = prow + (c >> 1) * (kQTile * 128);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int chunk = ((c & 1) * 4 + q) ^ rx;
                    *reinterpret_cast<uint4*>(blk + chunk * 16) = make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
                }
            }
            tc_fence_before();
            mbar_arrive(s_free);                                   // S may be overwritten by the next Q K^T
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // P visible to the MMA's async-proxy reads
            mbar_arrive(p_full);
            l = l * alpha + sum;
            m = m_new;
            ok = mbar_wait(o_full, it, abort_flag, p.status, kErrEpilogueWait);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < HD / 32; c++) {
                uint32_t v[32];
                tmem_ld_32x32(tmem_o + lane_off + c * 32, v);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; i++) O[c * 32 + i] = fmaf(O[c * 32 + i], alpha, __uint_as_float(v[i]));
            }
            tc_fence_before();
            mbar_arrive(o_free);
        }
        if (ok && qrow < p.T) {
            const float inv = 1.0f / l;
            __nv_bfloat16* orow = p.out + ((long long)b * p.T + qrow) * p.ld_out + (long long)h * HD;
#pragma unroll
            for (int i = 0; i < HD; i += 8) {
                uint4 o;
                __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                for (int q = 0; q < 4; q++) oh[q] = __floats2bfloat162_rn(O[i + 2 * q] * inv, O[i + 2 * q + 1] * inv);
                *reinterpret_cast<uint4*>(orow + i) = o;
            }
        }
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
    long long grid = (long long)B * H * prm.n_qtiles;
    if (grid > INT32_MAX) return fail("attention_fused: grid too large");
    ProfScope ps(PROF_ATTN_FUSED);
    if (hd == 64) {
        static bool set = false;
        if (!set) { SPT_CUDA(cudaFuncSetAttribute(attn_fused_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem<64>::kTotal)); set = true; }
        attn_fused_kernel<64><<<(unsigned)grid, kAttnThreads, AttnSmem<64>::kTotal, rt().stream>>>(tq, tk, tv, prm);
    } else {
        static bool set = false;
        if (!set) { SPT_CUDA(cudaFuncSetAttribute(attn_fused_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem<128>::kTotal)); set = true; }
        attn_fused_kernel<128><<<(unsigned)grid, kAttnThreads, AttnSmem<128>::kTotal, rt().stream>>>(tq, tk, tv, prm);
    }
    SPT_LAUNCH_CHECK("attn_fused");
    return 0;
}

}  // namespace spt
