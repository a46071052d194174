// attention.cu -- causal multi-head attention core (crates/nn/src/lib.rs:600-637).
//
// Reference composition: reshape_to_heads x3 -> batch_transpose(K) -> batch_matmul(Q,K^T) -> scale ->
// masked_fill(j>i,-inf) -> softmax rows -> batch_matmul(P,V) -> reshape_from_heads, each a separate host
// pass with its own copy.  Here the head permutations are strides of the tensor maps (no kernel, no
// copy), and the "materialised" form below runs three launches per layer:
//   S = Q K^T      batched tcgen05 GEMM over (head, sequence), tiles above the diagonal skipped
//   P = causal_softmax(scale * S)   in place, reads only j <= i
//   O = P V        batched tcgen05 GEMM, k-blocks above the diagonal skipped, V supplied as V^T [hd, T]
#include "gemm.h"
#include "../../include/sptorch_b200_ext.h"

namespace spt {

// v [B*T, ld] (head h at columns h*hd..) -> vt [B, H, hd, T]
template <typename T>
__global__ void head_transpose_kernel(const T* __restrict__ v, T* __restrict__ vt, int Tn, int H, int hd, long long ld) {
    __shared__ T tile[32][33];
    const int bh = blockIdx.z, b = bh / H, h = bh % H;
    const int t0 = blockIdx.x * 32, e0 = blockIdx.y * 32;
    const T* src = v + ((long long)b * Tn) * ld + (long long)h * hd;
    T* dst = vt + (long long)bh * hd * Tn;
    for (int j = threadIdx.y; j < 32; j += 8) {
        int t = t0 + j, e = e0 + threadIdx.x;
        if (t < Tn && e < hd) tile[j][threadIdx.x] = src[(long long)t * ld + e];
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8) {
        int e = e0 + j, t = t0 + threadIdx.x;
        if (t < Tn && e < hd) dst[(long long)e * Tn + t] = tile[threadIdx.x][j];
    }
}

int attention_materialized(const void* q, const void* k, const void* vt, long long vt_ld, long long vt_s_head, long long vt_s_batch,
                           void* out, void* scores, int B, int Tn, int H, int hd, long long ld_qk, long long ld_out, int dtype);
bool attention_fused_supported(int T, int hd, long long ld_q, long long ld_kv);
int attention_fused(const void* q, const void* k, const void* v, void* out, int B, int T, int H, int hd, long long ld_q, long long ld_k,
                    long long ld_v, long long ld_out);

static std::atomic<int> g_attn_mode{0};   // 0 = fused kernel whenever it applies, 1 = always the materialised three-launch form
int attention_mode() { return g_attn_mode.load(); }

// true when the fused kernel takes this problem (bf16, head_dim 64 or 128, 16-byte aligned row pitches, not switched off)
bool attention_uses_fused(int dtype, int Tn, int hd, long long ld_q, long long ld_kv) {
    return dtype == BF16 && g_attn_mode.load() == 0 && attention_fused_supported(Tn, hd, ld_q, ld_kv);
}

// q,k: [B*T, ld_qk]; vt: V^T with element (b,h,e,t) at vt[b*vt_s_batch + h*vt_s_head + e*vt_ld + t];
// scores: workspace of B*H*T*T elements; out: [B*T, ld_out]
int attention_materialized(const void* q, const void* k, const void* vt, long long vt_ld, long long vt_s_head, long long vt_s_batch,
                           void* out, void* scores, int B, int Tn, int H, int hd, long long ld_qk, long long ld_out, int dtype) {
    const int mode = dtype == BF16 ? MM_BF16 : MM_TF32;
    GemmDesc s;
    s.A = q; s.B = k; s.C = scores;
    s.M = Tn; s.N = Tn; s.K = hd;
    s.lda = ld_qk; s.ldb = ld_qk; s.ldc = Tn;
    s.nb1 = H; s.nb2 = B;
    s.sA1 = hd; s.sA2 = (long long)Tn * ld_qk;
    s.sB1 = hd; s.sB2 = (long long)Tn * ld_qk;
    s.sC1 = (long long)Tn * Tn; s.sC2 = (long long)H * Tn * Tn;
    s.mode = mode; s.out_dtype = dtype; s.causal_lower = 1;
    GemmPlan ps;
    if (gemm_plan(s, &ps)) return 1;
    { ProfScope pr(PROF_ATTN_GEMM); if (gemm_run(ps)) return 1; }
    // scale -> mask -> softmax exactly in the reference's order (crates/nn/src/lib.rs:614-632)
    { ProfScope pr(PROF_SOFTMAX); if (sptorch_ext_causal_softmax(scores, scores, (size_t)B * H, (size_t)Tn, 1.0f / sqrtf((float)hd), dtype)) return 1; }
    GemmDesc o;
    o.A = scores; o.B = vt; o.C = out;
    o.M = Tn; o.N = hd; o.K = Tn;
    o.lda = Tn; o.ldb = vt_ld; o.ldc = ld_out;
    o.nb1 = H; o.nb2 = B;
    o.sA1 = (long long)Tn * Tn; o.sA2 = (long long)H * Tn * Tn;
    o.sB1 = vt_s_head; o.sB2 = vt_s_batch;
    o.sC1 = hd; o.sC2 = (long long)Tn * ld_out;
    o.mode = mode; o.out_dtype = dtype; o.causal_k = 1;
    GemmPlan po;
    if (gemm_plan(o, &po)) return 1;
    { ProfScope pr(PROF_ATTN_GEMM); if (gemm_run(po)) return 1; }
    return 0;
}

}  // namespace spt

using namespace spt;

extern "C" {

size_t sptorch_ext_attention_workspace(size_t B, size_t T, size_t H, size_t hd, int dtype) {
    size_t es = dtype == SPT_BF16 ? 2 : 4;
    size_t scores = ((B * H * T * T * es + 255) / 256) * 256;
    size_t vt = ((B * H * hd * T * es + 255) / 256) * 256;
    return scores + vt;
}

int sptorch_ext_attention_causal(const void* q, const void* k, const void* v, void* out, void* workspace, size_t B, size_t T, size_t H,
                                 size_t hd, size_t ld_qkv, int dtype) {
    if (enter()) return 1;
    if (B == 0 || T == 0 || H == 0 || hd == 0) return 0;
    if (!q || !k || !v || !out || !workspace) return fail("attention: null handle");
    if (dtype != SPT_F32 && dtype != SPT_BF16) return fail("attention: unknown dtype %d", dtype);
    if (B * H > 65535) return fail("attention: B*H exceeds one launch of the V transpose");
    size_t es = dtype == SPT_BF16 ? 2 : 4;
    const bool fused = attention_uses_fused(dtype, (int)T, (int)hd, (long long)ld_qkv, (long long)ld_qkv);
    if (!fused && (T * es) % 16) return fail("attention: T must be a multiple of %zu for this dtype", 16 / es);
    size_t scores_bytes = ((B * H * T * T * es + 255) / 256) * 256;
    void* scores = workspace;
    void* vt = (uint8_t*)workspace + scores_bytes;
    if (fused)
        return attention_fused(q, k, v, out, (int)B, (int)T, (int)H, (int)hd, (long long)ld_qkv, (long long)ld_qkv, (long long)ld_qkv, (long long)(H * hd));
    dim3 grid((unsigned)((T + 31) / 32), (unsigned)((hd + 31) / 32), (unsigned)(B * H));
    if (dtype == SPT_BF16)
        head_transpose_kernel<__nv_bfloat16><<<grid, dim3(32, 8), 0, rt().stream>>>((const __nv_bfloat16*)v, (__nv_bfloat16*)vt, (int)T, (int)H, (int)hd, (long long)ld_qkv);
    else
        head_transpose_kernel<float><<<grid, dim3(32, 8), 0, rt().stream>>>((const float*)v, (float*)vt, (int)T, (int)H, (int)hd, (long long)ld_qkv);
    SPT_LAUNCH_CHECK("head_transpose");
    return attention_materialized(q, k, vt, (long long)T, (long long)(hd * T), (long long)(H * hd * T), out, scores, (int)B, (int)T, (int)H,
                                  (int)hd, (long long)ld_qkv, (long long)(H * hd), dtype);
}

int sptorch_ext_set_attention_mode(int mode) {
    if (mode != 0 && mode != 1) return fail("set_attention_mode: 0 = fused when possible, 1 = materialised");
    g_attn_mode.store(mode);
    bump_config_epoch();          // a captured forward holds the other path's launches
    return 0;
}

}  // extern "C"
