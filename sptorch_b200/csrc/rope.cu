// rope.cu -- rotary position embedding applied in place to the head slots of a token-major buffer.
//
// Reference: apply_rope_raw (crates/nn/src/lib.rs:930-961), called on Q and K of [n_head, seq_len, head_dim] by
// MultiHeadAttention::forward_causal_impl (nn/src/lib.rs:606-609).  For pair p of a head at absolute position s:
//   theta = s / base^(2p / head_dim);  (even, odd) <- (even cos - odd sin, even sin + odd cos)
// Here Q and K live side by side in one [rows, ld] buffer, head h at columns h*head_dim, so one pass rotates both and
// the head permutes of the reference do not exist.  The denominators base^(2p/head_dim) are evaluated on the host with
// the same powf the reference uses and cached per (head_dim, base); sine and cosine come from sincosf (2 ulp).
// One thread owns one 16-byte vector position of the head and walks over all head slots of its row, so a sine/cosine
// pair is computed once per (position, pair) and reused 2 * n_head times.
// Bound: HBM (one read and one write of the Q and K columns).
#include "common.h"
#include "../../include/sptorch_b200_ext.h"
#include <cmath>
#include <map>
#include <vector>

namespace spt {

template <typename T> struct RopeVec;
template <> struct RopeVec<float> { static constexpr int N = 4; };
template <> struct RopeVec<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T>
__global__ void __launch_bounds__(256) rope_kernel(T* __restrict__ x, const float* __restrict__ denom, long long rows, int Tn, int n_slots,
                                                   int hd, long long ld, int offset, const int* __restrict__ offset_dev) {
    constexpr int N = RopeVec<T>::N;
    if (offset_dev) offset = *offset_dev;                      // decode graphs: the position lives in a device word
    const int vec_per_head = hd / N;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * vec_per_head) return;
    const long long row = idx / vec_per_head;
    const int v = (int)(idx - row * vec_per_head);
    const float pos = (float)(offset + (int)(row % Tn));       // `absolute_pos as f32`
    float sn[N / 2], cs[N / 2];
#pragma unroll
    for (int i = 0; i < N / 2; i++) {
        const float theta = pos / denom[v * (N / 2) + i];
        sincosf(theta, &sn[i], &cs[i]);
    }
    T* p = x + row * ld + (long long)v * N;
    for (int h = 0; h < n_slots; h++, p += hd) {
        uint4 raw = *reinterpret_cast<const uint4*>(p);
        if constexpr (sizeof(T) == 4) {
            float* e = reinterpret_cast<float*>(&raw);
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const float ev = e[2 * i], od = e[2 * i + 1];
                e[2 * i] = ev * cs[i] - od * sn[i];
                e[2 * i + 1] = ev * sn[i] + od * cs[i];
            }
        } else {
            __nv_bfloat162* e = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 a = __bfloat1622float2(e[i]);
                e[i] = __floats2bfloat162_rn(a.x * cs[i] - a.y * sn[i], a.x * sn[i] + a.y * cs[i]);
            }
        }
        *reinterpret_cast<uint4*>(p) = raw;
    }
}

// element-wise form for head dims or strides that 16-byte vectors cannot take
template <typename T>
__global__ void __launch_bounds__(256) rope_generic_kernel(T* __restrict__ x, const float* __restrict__ denom, long long rows, int Tn,
                                                           int n_slots, int hd, long long ld, int offset, const int* __restrict__ offset_dev) {
    const int half = hd / 2;
    if (offset_dev) offset = *offset_dev;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * half) return;
    const long long row = idx / half;
    const int pr = (int)(idx - row * half);
    const float theta = (float)(offset + (int)(row % Tn)) / denom[pr];
    float sn, cs;
    sincosf(theta, &sn, &cs);
    T* p = x + row * ld + 2 * pr;
    for (int h = 0; h < n_slots; h++, p += hd) {
        const float ev = (float)p[0], od = (float)p[1];
        p[0] = (T)(ev * cs - od * sn);
        p[1] = (T)(ev * sn + od * cs);
    }
}

// base^(2p/hd), p = 0 .. hd/2-1, on the device; cached for the life of the process (a few hundred bytes per entry)
struct RopeTable { std::vector<float> host; float* dev = nullptr; };
static std::mutex g_rope_mu;
static std::map<std::pair<int, uint32_t>, RopeTable> g_rope;

static const float* rope_denominators(int hd, float base) {
    uint32_t bits;
    memcpy(&bits, &base, 4);
    std::lock_guard<std::mutex> lk(g_rope_mu);
    RopeTable& t = g_rope[{hd, bits}];
    if (!t.dev) {
        t.host.resize(hd / 2);
        for (int p = 0; p < hd / 2; p++) t.host[p] = powf(base, (float)(2 * p) / (float)hd);      // nn/src/lib.rs:948
        if (cudaMalloc(&t.dev, t.host.size() * sizeof(float)) != cudaSuccess) { t.dev = nullptr; cudaGetLastError(); return nullptr; }
        if (cudaMemcpyAsync(t.dev, t.host.data(), t.host.size() * sizeof(float), cudaMemcpyHostToDevice, rt().stream) != cudaSuccess) return nullptr;
    }
    return t.dev;
}

int rope_launch(void* x, long long rows, int Tn, int n_slots, int hd, long long ld, float base, int offset, int dtype, const int* offset_dev) {
    if (rows == 0 || n_slots == 0) return 0;
    if (hd <= 0 || hd % 2) return fail("rope: head_dim %d is not even", hd);          // the reference asserts (nn/src/lib.rs:938)
    const float* den = rope_denominators(hd, base);
    if (!den) return fail("rope: cannot stage the frequency table");
    const int N = dtype == SPT_BF16 ? 8 : 4;
    const size_t es = dtype == SPT_BF16 ? 2 : 4;
    const bool vec = hd % N == 0 && (ld * es) % 16 == 0 && (reinterpret_cast<uintptr_t>(x) & 15) == 0;
    const long long work = rows * (vec ? hd / N : hd / 2);
    const unsigned grid = (unsigned)((work + 255) / 256);
    if (dtype == SPT_BF16) {
        if (vec) rope_kernel<__nv_bfloat16><<<grid, 256, 0, rt().stream>>>((__nv_bfloat16*)x, den, rows, Tn, n_slots, hd, ld, offset, offset_dev);
        else rope_generic_kernel<__nv_bfloat16><<<grid, 256, 0, rt().stream>>>((__nv_bfloat16*)x, den, rows, Tn, n_slots, hd, ld, offset, offset_dev);
    } else {
        if (vec) rope_kernel<float><<<grid, 256, 0, rt().stream>>>((float*)x, den, rows, Tn, n_slots, hd, ld, offset, offset_dev);
        else rope_generic_kernel<float><<<grid, 256, 0, rt().stream>>>((float*)x, den, rows, Tn, n_slots, hd, ld, offset, offset_dev);
    }
    SPT_LAUNCH_CHECK("rope");
    return 0;
}

}  // namespace spt

extern "C" int sptorch_ext_rope(void* x, size_t rows, size_t seq_len, size_t n_heads, size_t head_dim, size_t ld, float rope_base,
                                size_t position_offset, int dtype) {
    using namespace spt;
    if (enter()) return 1;
    if (rows == 0 || n_heads == 0) return 0;
    if (!x) return fail("rope: null handle");
    if (dtype != SPT_F32 && dtype != SPT_BF16) return fail("rope: unknown dtype %d", dtype);
    if (seq_len == 0 || rows % seq_len) return fail("rope: rows must be a multiple of seq_len");
    if (ld == 0) ld = n_heads * head_dim;
    if (ld < n_heads * head_dim) return fail("rope: ld smaller than n_heads * head_dim");
    if (head_dim > 65536 || n_heads > 65536 || position_offset + seq_len > (size_t)1 << 24) return fail("rope: dimension too large");
    return rope_launch(x, (long long)rows, (int)seq_len, (int)n_heads, (int)head_dim, (long long)ld, rope_base, (int)position_offset, dtype, nullptr);
}
