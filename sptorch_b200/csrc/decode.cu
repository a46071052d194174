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
#include <cooperative_groups.h>

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
// One CTA of 4 or 16 warps per (sequence, head).  A row of K or V is read by LPR = row bytes / 16 neighbouring lanes with one
// 16-byte load each, so a warp fetches 32 / LPR whole rows per instruction, fully coalesced, and four positions are in flight per
// lane (sixteen warps cover 256 positions of 128-byte rows per turn: the walk over a 1024-position cache is four dependent
// rounds of loads, not thirty); the dot product is finished with log2(LPR) shuffles.  Every row group keeps a running (maximum,
// sum, weighted value sum) over the positions it visits (online softmax), the groups of a warp and then the warps are merged at
// the end.  Same result as the kernel above up to the order of the f32 sums.
// fresh_k / fresh_v (optional): the newest token's key / value, still in the projection output (rows of ld_fresh elements, head h
// at columns h*hd).  The CTA copies its head's part into cache row `slot` and uses the fresh rows for that position, which
// saves the append launch in front of the attention.
// The first round of cache rows is requested before the programmatic-launch wait: cache rows other than `slot` were written by
// earlier steps, only q and the fresh rows come from the kernel before this one.
// HBM traffic: 2 * n * hd * sizeof(T) bytes per (sequence, head), read once.
constexpr int kRowsMaxWarps = 16;
// NW: warps per CTA.  Four-warp CTAs are held to 80 registers so that six share an SM (888 CTA slots: the 768 (sequence, head)
// pairs of 64 sequences x 12 heads run as one wave; at 92 registers and five per SM they made two).
template <typename T, int NW>
__global__ void __launch_bounds__(NW * 32, NW == 4 ? 6 : 1) attention_last_token_rows_kernel(const T* __restrict__ q, long long ld_q, const T* __restrict__ kc,
                                                                                      const T* __restrict__ vc, T* __restrict__ out, long long ld_out, int H, int hd,
                                                                                      int n, long long seq_stride, long long row_stride, float scale,
                                                                                      const int* __restrict__ state, const T* __restrict__ fresh_k,
                                                                                      const T* __restrict__ fresh_v, long long ld_fresh, int slot, T* kc_w, T* vc_w, int splits) {
    constexpr int VE = 16 / (int)sizeof(T);              // elements per 16-byte segment
    constexpr int U = 4;                                 // positions in flight per row group
    __shared__ float res[132];                           // this CTA's merged (maximum, sum, value sums): read by the cluster's first CTA
    __shared__ float sm[NW * 130];                       // per warp: maximum, sum, up to 128 value sums (f32 rows of 512 bytes, bf16 rows of 256)
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (state) { n = state[1]; slot = state[2]; }        // written before the step's first kernel was launched
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int nw = NW;
    const int lpr = hd / VE;                             // lanes per row
    const int rpi = 32 / lpr;                            // rows per warp instruction
    const int seg = lane % lpr, grp = lane / lpr;
    // a cluster of `splits` CTAs shares one (sequence, head): CTA r of it walks the r-th part of the positions
    const int pair = blockIdx.x / splits, rank = blockIdx.x % splits;
    const int b = pair / H, h = pair % H;
    const int part = (n + splits - 1) / splits, lo = rank * part, hi = min(n, lo + part);
    auto widen = [](uint4 raw, float (&f)[VE]) {
        if constexpr (sizeof(T) == 2) {
            const __nv_bfloat162* e = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; i++) { const float2 a = __bfloat1622float2(e[i]); f[2 * i] = a.x; f[2 * i + 1] = a.y; }
        } else {
            f[0] = __uint_as_float(raw.x); f[1] = __uint_as_float(raw.y); f[2] = __uint_as_float(raw.z); f[3] = __uint_as_float(raw.w);
        }
    };
    const T* kb = kc + (long long)b * seq_stride + (long long)h * hd + seg * VE;
    const T* vb = vc + (long long)b * seq_stride + (long long)h * hd + seg * VE;
    const int stride = nw * rpi;
    uint4 kr[U], vr[U];
    auto fetch = [&](int base) {                         // dead positions read row 0 (always valid) and are discarded by visit()
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int p = base + u * stride + grp;
            const long long pp = p < hi ? p : 0;
            kr[u] = *reinterpret_cast<const uint4*>(kb + pp * row_stride);
            vr[u] = *reinterpret_cast<const uint4*>(vb + pp * row_stride);
        }
    };
    const int first = lo + warp * rpi;
    if (first < hi) fetch(first);
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float qf[VE];
    widen(*reinterpret_cast<const uint4*>(q + (long long)b * ld_q + (long long)h * hd + seg * VE), qf);
    uint4 fk = make_uint4(0, 0, 0, 0), fv = fk;
    if (fresh_k) {
        fk = *reinterpret_cast<const uint4*>(fresh_k + (long long)b * ld_fresh + (long long)h * hd + seg * VE);
        fv = *reinterpret_cast<const uint4*>(fresh_v + (long long)b * ld_fresh + (long long)h * hd + seg * VE);
        if (rank == 0 && warp == 0 && grp == 0) {
            const long long dst = (long long)b * seq_stride + (long long)slot * row_stride + (long long)h * hd + seg * VE;
            *reinterpret_cast<uint4*>(kc_w + dst) = fk;
            *reinterpret_cast<uint4*>(vc_w + dst) = fv;
        }
    }
    float m = -INFINITY, l = 0.0f, o[VE];
#pragma unroll
    for (int i = 0; i < VE; i++) o[i] = 0.0f;
    auto visit = [&](uint4 kraw, uint4 vraw, bool live) {
        float kf[VE], vf[VE];
        widen(kraw, kf);
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < VE; i++) s += qf[i] * kf[i];
        for (int off = lpr >> 1; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        s *= scale;
        const float mn = live ? fmaxf(m, s) : m;
        const float corr = live ? expf(m - mn) : 1.0f;             // m = -inf on the first live visit: corr = 0, nothing accumulated yet
        const float pr = live ? expf(s - mn) : 0.0f;
        widen(vraw, vf);
        l = l * corr + pr;
#pragma unroll
        for (int i = 0; i < VE; i++) o[i] = o[i] * corr + pr * vf[i];
        m = mn;
    };
    // warp-uniform trip count (the shuffles inside visit() are warp-wide)
    for (int base = first; base < hi; base += U * stride) {
        if (base != first) fetch(base);
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int p = base + u * stride + grp;
            const bool is_fresh = fresh_k != nullptr && p == slot;
            visit(is_fresh ? fk : kr[u], is_fresh ? fv : vr[u], p < hi);
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
    // ... and the warps
    float* mine = sm + warp * 130;
    if (grp == 0) {
        if (seg == 0) { mine[0] = m; mine[1] = l; }
#pragma unroll
        for (int i = 0; i < VE; i++) mine[2 + seg * VE + i] = o[i];
    }
    __syncthreads();
    if (warp == 0 && grp == 0) {
        for (int w = 1; w < nw; w++) {
            const float* other = sm + w * 130;
            float oo[VE];
#pragma unroll
            for (int i = 0; i < VE; i++) oo[i] = other[2 + seg * VE + i];
            merge(other[0], other[1], oo);
        }
    }
    if (splits > 1) {
        // the parts meet in the first CTA of the cluster, which reads the others' results through distributed shared memory
        namespace cg = cooperative_groups;
        cg::cluster_group cluster = cg::this_cluster();
        if (warp == 0 && grp == 0) {
            if (seg == 0) { res[0] = m; res[1] = l; }
#pragma unroll
            for (int i = 0; i < VE; i++) res[2 + seg * VE + i] = o[i];
        }
        cluster.sync();
        if (rank == 0 && warp == 0 && grp == 0) {
            for (int r = 1; r < splits; r++) {
                const float* other = cluster.map_shared_rank(res, r);
                float oo[VE];
#pragma unroll
                for (int i = 0; i < VE; i++) oo[i] = other[2 + seg * VE + i];
                merge(other[0], other[1], oo);
            }
        }
        cluster.sync();                                  // no CTA leaves while its shared memory may still be read
    }
    if (rank == 0 && warp == 0 && grp == 0) {
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

// true when the coalesced kernel (the one that can also take the newest token's key / value rows straight from the projection
// output) serves this head size: rows of 16 .. 512 bytes, a power of two
bool attention_last_token_takes_fresh(int hd, int dtype) {
    const size_t rb = (size_t)hd * (dtype == BF16 ? 2 : 4);
    return rb >= 16 && rb <= 512 && hd <= 128 && (rb & (rb - 1)) == 0;
}

// state / n_cap: when state is given, n and the ring slot are read from state[1] / state[2] at run time; n_cap is the cache capacity
// fresh_k / fresh_v / ld_fresh / slot: see the kernel; dependent: launched as a programmatic dependent of the kernel before it
int attention_last_token(const void* q, long long ld_q, const void* kc, const void* vc, void* out, long long ld_out, int B, int H, int hd,
                         int n, long long seq_stride, long long row_stride, int dtype, const int* state, int n_cap,
                         const void* fresh_k, const void* fresh_v, long long ld_fresh, int slot, bool dependent) {
    if (B <= 0 || H <= 0 || n <= 0) return fail("attention_last_token: empty cache or batch");
    {
        // rows of 16 .. 512 bytes, a power of two, everything 16-byte aligned: the coalesced kernel
        const size_t es = dtype == BF16 ? 2 : 4;
        const bool aligned = ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kc) | reinterpret_cast<uintptr_t>(vc) | reinterpret_cast<uintptr_t>(out) |
                               reinterpret_cast<uintptr_t>(fresh_k) | reinterpret_cast<uintptr_t>(fresh_v)) & 15) == 0 &&
                             (ld_q * es) % 16 == 0 && (ld_out * es) % 16 == 0 && (seq_stride * es) % 16 == 0 && (row_stride * es) % 16 == 0 && (ld_fresh * es) % 16 == 0;
        if (attention_last_token_takes_fresh(hd, dtype) && aligned) {
            const float scale = 1.0f / sqrtf((float)hd);
            // Few (sequence, head) pairs: a cluster of up to eight CTAs shares each pair, with four or sixteen warps per CTA -- whichever
            // combination walks the cache in the fewest dependent rounds of loads while all CTAs are resident at once (a 16-warp CTA
            // is alone on its SM at 90 registers, six 4-warp CTAs share one).  One sequence of 12 heads: 48 CTAs of 16 warps, one
            // round; 8 sequences: 96 CTAs of 16 warps, no split; 64 sequences: 768 CTAs of 4 warps, no split.
            const int span = state ? n_cap : n;
            const long long pairs = (long long)B * H;
            const int per_warp_round = (32 / (hd / (16 / (int)es))) * 4;      // rows per warp instruction x positions in flight
            int splits = 1, threads = 128, best = INT32_MAX;
            for (int sp = 1; sp <= 8; sp *= 2)
                for (int nw = 4; nw <= kRowsMaxWarps; nw *= 4) {
                    const long long ctas = pairs * sp, cap = (long long)rt().sm_count * (nw == 4 ? 6 : 1);
                    if (ctas > cap && !(sp == 1 && nw == 4)) continue;
                    const int rounds = ceil_div(span, (long long)sp * nw * per_warp_round);
                    // a round of loads costs about as much as 1.3 doublings of the cluster size (measured at 8 sequences x 12 heads over
                    // a 1024-position cache: 96 CTAs of 16 warps, four rounds, 0.411 ms per step; 96 clusters of eight 4-warp CTAs, two
                    // rounds, 0.443 ms)
                    const int log2sp = sp == 1 ? 0 : sp == 2 ? 1 : sp == 4 ? 2 : 3;
                    const int score = rounds * 8 + (nw == 4 ? 0 : 2) + 6 * log2sp;
                    if (score < best) { best = score; splits = sp; threads = nw * 32; }
                }
#define SPT_ROWS_LAUNCH(T_, NW_)                                                                                                                      \
    SPT_CUDA(launch_dependent(attention_last_token_rows_kernel<T_, NW_>, dim3(B * H * splits), dim3(NW_ * 32), 0, dependent, splits, (const T_*)q, ld_q,   \
                              (const T_*)kc, (const T_*)vc, (T_*)out, ld_out, H, hd, n, seq_stride, row_stride, scale, state, (const T_*)fresh_k,         \
                              (const T_*)fresh_v, ld_fresh, slot, (T_*)const_cast<void*>(kc), (T_*)const_cast<void*>(vc), splits))
            if (dtype == BF16) { if (threads == 128) SPT_ROWS_LAUNCH(__nv_bfloat16, 4); else SPT_ROWS_LAUNCH(__nv_bfloat16, kRowsMaxWarps); }
            else { if (threads == 128) SPT_ROWS_LAUNCH(float, 4); else SPT_ROWS_LAUNCH(float, kRowsMaxWarps); }
#undef SPT_ROWS_LAUNCH
            note_submit();
            return 0;
        }
    }
    if (fresh_k || fresh_v) return fail("attention_last_token: the newest token's rows can only be taken from the projection output for 16 .. 512-byte head rows");
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
    return attention_last_token(q, d, k_cache, v_cache, out, d, (int)B, (int)H, (int)hd, (int)n, (long long)cache_positions * d, d, dtype, nullptr, 0,
                                nullptr, nullptr, 0, 0, false);
}
