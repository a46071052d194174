// common.h -- process-global runtime state shared by every translation unit of libsptorch_b200.so.
//
// The reference's C-ABI has no context argument (crates/hal-ffi/include/sptorch_hal.h:21-85), so the
// state is process-global: one device, one stream, one stream-ordered memory pool.  This replaces
// runtime-cuda's CudaBackend/GpuTensor layer (crates/runtime-cuda/src/lib.rs:26-81), which copies
// synchronously around every op and zero-fills every output.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stddef.h>
#include <cstdlib>
#include <atomic>
#include <mutex>

namespace spt {

enum DType : int { F32 = 0, BF16 = 1 };

struct Runtime {
    std::mutex mu;
    int refcount = 0;
    int device = -1;
    int sm_count = 0;
    int sm_reserve = 0;                 // SMs the persistent kernels leave free (for a collective running beside them)
    cudaStream_t stream = nullptr;      // the stream every op is enqueued on
    cudaStream_t own_stream = nullptr;  // created at init; `stream` may be swapped for a caller's
    cudaStream_t copy_stream = nullptr; // second stream for overlapped device->host copies
    cudaMemPool_t pool = nullptr;
    std::atomic<int> sticky{0};         // first failure since the last sync; reported again by sync
    std::atomic<uint64_t> submitted{0}, retired{0};
    size_t budget = 0;                  // 0 = unlimited; otherwise sptorch_alloc fails past it (tests)
    std::atomic<size_t> in_use{0};
    uint32_t* dev_status = nullptr;     // device word written by kernels whose bounded waits ran out
    cudaEvent_t t0 = nullptr, t1 = nullptr;
};

Runtime& rt();

// Records msg as the thread's and the process's last error, marks the sticky flag, returns 1.
int fail(const char* fmt, ...);
// Same, for host-only work (file parsing): nothing was submitted to the device, so the sticky flag stays clear.
int fail_host(const char* fmt, ...);
// Makes the runtime's device current for the calling thread; non-zero if the library is not initialised.
int enter();
// Waits for the library stream without consuming the sticky error flag (internal uploads use this).
int stream_wait();
// Registers a callback run once at backend shutdown, while the device is still current (frees per-process device caches).
void at_shutdown(void (*fn)());
// Counter bumped by every setter that changes which kernels or grids a forward launches (attention mode, GEMM tile mode,
// matmul arithmetic, SM reserve): a captured CUDA graph is only replayed while the counter still has the value it was captured at.
uint64_t config_epoch();
void bump_config_epoch();
// Resolves the device address of the allocation-free matmul's static scratch for the runtime's device (gemm.cu).
void static_scratch_prepare();
inline void note_submit() { rt().submitted.fetch_add(1, std::memory_order_relaxed); }

#define SPT_CUDA(expr)                                                                     \
    do {                                                                                   \
        cudaError_t _e = (expr);                                                           \
        if (_e != cudaSuccess) return ::spt::fail("%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

#define SPT_LAUNCH_CHECK(name)                                                             \
    do {                                                                                   \
        cudaError_t _e = cudaGetLastError();                                               \
        if (_e != cudaSuccess) return ::spt::fail("launch of %s failed: %s", name, cudaGetErrorString(_e)); \
        ::spt::note_submit();                                                              \
    } while (0)

// Launch on the library stream, optionally as a programmatic dependent of the kernel before it in the stream: the grid may then
// begin (and run whatever precedes its griddepcontrol.wait) while that kernel is still running.  Only kernels that execute
// griddepcontrol.wait before they touch anything an earlier kernel writes may be launched with dependent = true.
// SPTORCH_B200_PDL=0 in the environment turns every such launch into an ordinary one.
inline bool dependent_launch_enabled() {
    static const bool on = [] { const char* e = getenv("SPTORCH_B200_PDL"); return !(e && e[0] == '0'); }();
    return on;
}
// cluster: CTAs per thread-block cluster along x (1 = none; the grid's x extent must be a multiple of it).
template <typename... KArgs, typename... Args>
cudaError_t launch_dependent(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, bool dependent, int cluster, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = rt().stream;
    cudaLaunchAttribute at[2];
    int na = 0;
    if (dependent && dependent_launch_enabled()) {
        at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    if (cluster > 1) {
        at[na].id = cudaLaunchAttributeClusterDimension;
        at[na].val.clusterDim.x = (unsigned)cluster; at[na].val.clusterDim.y = 1; at[na].val.clusterDim.z = 1;
        na++;
    }
    cfg.attrs = at; cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// bf16 pair -> f32 pair as a shift and a mask (a bf16 is the upper half of an f32): two integer instructions on any pipe, where
// the conversion intrinsic may compile to conversion instructions.  In the residual add of the GEMM epilogue this form (with a
// packed add) took a 65536 x 768 -> 768 launch from 0.098 to 0.084 ms.
__device__ __forceinline__ float2 bf16x2_to_float2(__nv_bfloat162 h) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(&h);
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}

// Per-category device timing (CUDA events around launches on the library stream); off by default.
enum ProfCat : int { PROF_LINEAR = 0, PROF_ATTN_GEMM = 1, PROF_SOFTMAX = 2, PROF_LAYERNORM = 3, PROF_EMBED = 4, PROF_OTHER = 5, PROF_ATTN_FUSED = 6, PROF_NCAT = 7 };
bool prof_enabled();
void prof_begin(int cat);
void prof_end(int cat);
struct ProfScope { int c; explicit ProfScope(int cat) : c(cat) { prof_begin(c); } ~ProfScope() { prof_end(c); } };

// SMs the persistent GEMM / attention kernels may fill
inline int compute_sms() { int n = rt().sm_count - rt().sm_reserve; return n < 1 ? 1 : n; }

inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }

}  // namespace spt
