// runtime.cu -- lifecycle, stream-ordered memory pool, copies, sync, telemetry, timers.
//
// Replaces the reference's CudaBackend / GpuTensor layer (crates/runtime-cuda/src/lib.rs:26-81:
// htod_sync_copy / dtoh_sync_copy around every op, alloc_zeros for every output) with one stream
// and a cudaMallocAsync pool whose blocks are recycled without returning to the driver.
#include "common.h"
#include "../../include/sptorch_b200_hal.h"
#include "../../include/sptorch_b200_ext.h"
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <unordered_map>
#include <vector>

namespace spt {

static Runtime g_rt;
static thread_local char tl_error[512] = "";
static std::mutex g_sizes_mu;
static std::unordered_map<void*, size_t> g_sizes;   // live pool blocks -> bytes (for the test budget)
static void* g_flush = nullptr;
static const size_t kFlushBytes = 256u << 20;

Runtime& rt() { return g_rt; }

// ---- per-category event timing ----
struct ProfRec { int cat; cudaEvent_t e0, e1; };
static bool g_prof_on = false;
static std::vector<ProfRec> g_prof_recs;
static std::vector<cudaEvent_t> g_prof_free;
static std::mutex g_prof_mu;
static thread_local cudaEvent_t tl_open_e0 = nullptr;

static cudaEvent_t prof_event() {
    if (!g_prof_free.empty()) { cudaEvent_t e = g_prof_free.back(); g_prof_free.pop_back(); return e; }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}
bool prof_enabled() { return g_prof_on; }
void prof_begin(int) {
    if (!g_prof_on) return;
    std::lock_guard<std::mutex> lk(g_prof_mu);
    tl_open_e0 = prof_event();
    cudaEventRecord(tl_open_e0, g_rt.stream);
}
void prof_end(int cat) {
    if (!g_prof_on || !tl_open_e0) return;
    std::lock_guard<std::mutex> lk(g_prof_mu);
    cudaEvent_t e1 = prof_event();
    cudaEventRecord(e1, g_rt.stream);
    g_prof_recs.push_back({cat, tl_open_e0, e1});
    tl_open_e0 = nullptr;
}

int fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
    va_end(ap);
    g_rt.sticky.store(1);
    return 1;
}

int fail_host(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(tl_error, sizeof(tl_error), fmt, ap);
    va_end(ap);
    return 1;
}

int enter() {
    if (g_rt.refcount <= 0 || g_rt.device < 0) {
        snprintf(tl_error, sizeof(tl_error), "sptorch_b200: backend not initialised");
        return 1;
    }
    static thread_local int current = -1;
    if (current != g_rt.device) {
        if (cudaSetDevice(g_rt.device) != cudaSuccess) return fail("cudaSetDevice(%d) failed", g_rt.device);
        current = g_rt.device;
    }
    return 0;
}

int stream_wait() {
    cudaError_t e = cudaStreamSynchronize(g_rt.stream);
    g_rt.retired.store(g_rt.submitted.load());
    if (e != cudaSuccess) return fail("stream synchronize failed: %s", cudaGetErrorString(e));
    return 0;
}

static int pick_device() {
    const char* e = getenv("SPTORCH_B200_DEVICE");
    if (!e) e = getenv("LOCAL_RANK");
    if (e && *e) return atoi(e);
    int d = 0;
    if (cudaGetDevice(&d) != cudaSuccess) return 0;
    return d;
}

static int do_init() {
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0)
        return fail("sptorch_b200: no CUDA device (%s); this backend has no CPU path", cudaGetErrorString(e));
    int dev = pick_device();
    if (dev < 0 || dev >= n) return fail("sptorch_b200: device ordinal %d out of range (%d devices)", dev, n);
    cudaDeviceProp p;
    SPT_CUDA(cudaGetDeviceProperties(&p, dev));
    if (p.major != 10)
        return fail("sptorch_b200: device %d is sm_%d%d; the kernels are built for sm_100a only", dev, p.major, p.minor);
    SPT_CUDA(cudaSetDevice(dev));
    g_rt.device = dev;
    g_rt.sm_count = p.multiProcessorCount;
    SPT_CUDA(cudaStreamCreateWithFlags(&g_rt.own_stream, cudaStreamNonBlocking));
    SPT_CUDA(cudaStreamCreateWithFlags(&g_rt.copy_stream, cudaStreamNonBlocking));
    g_rt.stream = g_rt.own_stream;
    // A pool of the library's own: the device's default pool stays as the process's other users configured it.
    cudaMemPoolProps props = {};
    props.allocType = cudaMemAllocationTypePinned;
    props.handleTypes = cudaMemHandleTypeNone;
    props.location.type = cudaMemLocationTypeDevice;
    props.location.id = dev;
    SPT_CUDA(cudaMemPoolCreate(&g_rt.pool, &props));
    uint64_t keep = UINT64_MAX;   // never hand cached blocks back to the driver between ops
    SPT_CUDA(cudaMemPoolSetAttribute(g_rt.pool, cudaMemPoolAttrReleaseThreshold, &keep));
    SPT_CUDA(cudaMalloc(&g_rt.dev_status, 256));
    SPT_CUDA(cudaMemset(g_rt.dev_status, 0, 256));
    SPT_CUDA(cudaEventCreate(&g_rt.t0));
    SPT_CUDA(cudaEventCreate(&g_rt.t1));
    g_rt.sticky.store(0);
    static_scratch_prepare();     // the allocation-free matmul's scratch address, resolved while no capture can be open
    return 0;
}

// callbacks that release per-process device caches of other translation units (attention schedules, ...) at shutdown
static std::vector<void (*)()> g_shutdown_hooks;
void at_shutdown(void (*fn)()) {
    for (auto f : g_shutdown_hooks) if (f == fn) return;
    g_shutdown_hooks.push_back(fn);
}

static std::atomic<uint64_t> g_config_epoch{0};
uint64_t config_epoch() { return g_config_epoch.load(); }
void bump_config_epoch() { g_config_epoch.fetch_add(1); }

}  // namespace spt

using namespace spt;

extern "C" {

int sptorch_backend_init(void) {
    std::lock_guard<std::mutex> lk(g_rt.mu);
    if (g_rt.refcount > 0) { g_rt.refcount++; return 0; }
    if (do_init() != 0) { g_rt.device = -1; return 1; }
    g_rt.refcount = 1;
    return 0;
}

void sptorch_backend_shutdown(void) {
    std::lock_guard<std::mutex> lk(g_rt.mu);
    if (g_rt.refcount <= 0) return;
    if (--g_rt.refcount > 0) return;
    cudaSetDevice(g_rt.device);
    cudaStreamSynchronize(g_rt.stream);
    for (auto fn : g_shutdown_hooks) fn();
    if (g_flush) { cudaFree(g_flush); g_flush = nullptr; }
    if (g_rt.dev_status) { cudaFree(g_rt.dev_status); g_rt.dev_status = nullptr; }
    if (g_rt.t0) cudaEventDestroy(g_rt.t0);
    if (g_rt.t1) cudaEventDestroy(g_rt.t1);
    g_rt.t0 = g_rt.t1 = nullptr;
    if (g_rt.own_stream) cudaStreamDestroy(g_rt.own_stream);
    if (g_rt.copy_stream) cudaStreamDestroy(g_rt.copy_stream);
    g_rt.own_stream = g_rt.copy_stream = g_rt.stream = nullptr;
    if (g_rt.pool) { cudaMemPoolDestroy(g_rt.pool); g_rt.pool = nullptr; }
    g_rt.device = -1;
}

const char* sptorch_backend_name(void) { return "sptorch_b200"; }

void* sptorch_ext_alloc_bytes(size_t bytes) {
    if (enter()) return nullptr;
    size_t rounded = (bytes + 255) & ~size_t(255);
    if (rounded == 0) rounded = 256;
    if (g_rt.budget && g_rt.in_use.load() + rounded > g_rt.budget) {
        fail("sptorch_alloc: %zu bytes would exceed the allocation budget of %zu", rounded, g_rt.budget);
        g_rt.sticky.store(0);   // a refused allocation is reported by NULL, not by a poisoned stream
        return nullptr;
    }
    void* p = nullptr;
    cudaError_t e = cudaMallocFromPoolAsync(&p, rounded, g_rt.pool, g_rt.stream);
    if (e != cudaSuccess) {
        cudaGetLastError();
        fail("cudaMallocAsync(%zu) failed: %s", rounded, cudaGetErrorString(e));
        g_rt.sticky.store(0);
        return nullptr;
    }
    g_rt.in_use.fetch_add(rounded);
    {
        std::lock_guard<std::mutex> lk(g_sizes_mu);
        g_sizes[p] = rounded;
    }
    return p;
}

void* sptorch_alloc(size_t n) {
    if (n > (size_t(1) << 40)) { fail("sptorch_alloc: %zu elements is not a plausible size", n); g_rt.sticky.store(0); return nullptr; }
    return sptorch_ext_alloc_bytes(n * sizeof(float));
}

void sptorch_free(void* handle) {
    if (!handle || enter()) return;
    size_t bytes = 0;
    {
        std::lock_guard<std::mutex> lk(g_sizes_mu);
        auto it = g_sizes.find(handle);
        if (it == g_sizes.end()) return;   // not ours (or freed twice): ignore rather than corrupt the pool
        bytes = it->second;
        g_sizes.erase(it);
    }
    g_rt.in_use.fetch_sub(bytes);
    cudaFreeAsync(handle, g_rt.stream);
}

int sptorch_ext_copy_h2d_bytes(const void* host, void* device, size_t bytes) {
    if (enter()) return 1;
    if (bytes == 0) return 0;
    if (!host || !device) return fail("copy_h2d: null pointer");
    SPT_CUDA(cudaMemcpyAsync(device, host, bytes, cudaMemcpyHostToDevice, g_rt.stream));
    note_submit();
    return 0;
}

int sptorch_ext_copy_d2h_bytes(const void* device, void* host, size_t bytes) {
    if (enter()) return 1;
    if (bytes == 0) return 0;
    if (!host || !device) return fail("copy_d2h: null pointer");
    SPT_CUDA(cudaMemcpyAsync(host, device, bytes, cudaMemcpyDeviceToHost, g_rt.stream));
    SPT_CUDA(cudaStreamSynchronize(g_rt.stream));
    g_rt.retired.store(g_rt.submitted.load());
    return 0;
}

int sptorch_copy_h2d(const float* host, void* device, size_t n) { return sptorch_ext_copy_h2d_bytes(host, device, n * sizeof(float)); }
int sptorch_copy_d2h(const void* device, float* host, size_t n) { return sptorch_ext_copy_d2h_bytes(device, host, n * sizeof(float)); }

int sptorch_ext_memset(void* device, int byte, size_t bytes) {
    if (enter()) return 1;
    if (bytes == 0) return 0;
    SPT_CUDA(cudaMemsetAsync(device, byte, bytes, g_rt.stream));
    note_submit();
    return 0;
}

int sptorch_sync(void) {
    if (enter()) return 1;
    cudaError_t e = cudaStreamSynchronize(g_rt.stream);
    g_rt.retired.store(g_rt.submitted.load());
    if (e != cudaSuccess) return fail("stream synchronize failed: %s", cudaGetErrorString(e));
    uint32_t st = 0;
    if (g_rt.dev_status) {
        SPT_CUDA(cudaMemcpy(&st, g_rt.dev_status, sizeof(st), cudaMemcpyDeviceToHost));
        if (st) {
            cudaMemset(g_rt.dev_status, 0, 256);
            g_rt.sticky.store(0);
            fail("a kernel reported device status 0x%x (bounded wait ran out or an index was rejected)", st);
            g_rt.sticky.store(0);
            return 1;
        }
    }
    int s = g_rt.sticky.exchange(0);
    return s ? 1 : 0;
}

int sptorch_query_runtime(uint32_t* queue_depth, uint32_t* online) {
    if (enter()) { if (queue_depth) *queue_depth = 0; if (online) *online = 0; return 1; }
    cudaError_t q = cudaStreamQuery(g_rt.stream);
    uint64_t sub = g_rt.submitted.load();
    if (q == cudaSuccess) g_rt.retired.store(sub);
    uint64_t depth = sub - g_rt.retired.load();
    if (queue_depth) *queue_depth = depth > 0xFFFFFFFFull ? 0xFFFFFFFFu : (uint32_t)depth;
    bool healthy = (q == cudaSuccess || q == cudaErrorNotReady) && g_rt.sticky.load() == 0;
    if (online) *online = healthy ? 1u : 0u;
    return 0;
}

const char* sptorch_ext_last_error(void) { return tl_error; }
int sptorch_ext_device(void) { return g_rt.refcount > 0 ? g_rt.device : -1; }
int sptorch_ext_sm_count(void) { return g_rt.refcount > 0 ? g_rt.sm_count : 0; }

int sptorch_ext_set_stream(void* s) {
    if (enter()) return 1;
    SPT_CUDA(cudaStreamSynchronize(g_rt.stream));
    g_rt.stream = s ? (cudaStream_t)s : g_rt.own_stream;
    return 0;
}

void* sptorch_ext_alloc_pinned(size_t bytes) {
    if (enter()) return nullptr;
    void* p = nullptr;
    if (cudaHostAlloc(&p, bytes ? bytes : 1, cudaHostAllocDefault) != cudaSuccess) {
        cudaGetLastError();
        fail("cudaHostAlloc(%zu) failed", bytes);
        g_rt.sticky.store(0);
        return nullptr;
    }
    return p;
}
void sptorch_ext_free_pinned(void* p) { if (p && !enter()) cudaFreeHost(p); }

int sptorch_ext_set_alloc_budget(size_t bytes) { g_rt.budget = bytes; return 0; }

int sptorch_ext_set_sm_reserve(int n) {
    if (n < 0 || (g_rt.sm_count > 0 && n >= g_rt.sm_count)) return fail("set_sm_reserve: %d is outside 0..%d", n, g_rt.sm_count - 1);
    g_rt.sm_reserve = n;
    bump_config_epoch();          // grid sizes of captured launches depend on it
    return 0;
}

int sptorch_ext_timer_begin(void) {
    if (enter()) return 1;
    SPT_CUDA(cudaEventRecord(g_rt.t0, g_rt.stream));
    return 0;
}
int sptorch_ext_timer_end(float* ms) {
    if (enter()) return 1;
    SPT_CUDA(cudaEventRecord(g_rt.t1, g_rt.stream));
    SPT_CUDA(cudaEventSynchronize(g_rt.t1));
    g_rt.retired.store(g_rt.submitted.load());
    float t = 0;
    SPT_CUDA(cudaEventElapsedTime(&t, g_rt.t0, g_rt.t1));
    if (ms) *ms = t;
    return 0;
}

int sptorch_ext_flush_l2(void) {
    if (enter()) return 1;
    if (!g_flush) SPT_CUDA(cudaMalloc(&g_flush, kFlushBytes));
    SPT_CUDA(cudaMemsetAsync(g_flush, 0x5a, kFlushBytes, g_rt.stream));
    return 0;
}

int sptorch_ext_prof_enable(int on) {
    if (enter()) return 1;
    std::lock_guard<std::mutex> lk(g_prof_mu);
    g_prof_on = on != 0;
    return 0;
}

// Waits for the stream, adds up the elapsed time and launch count of every category since the last
// read into ms[PROF_NCAT] / launches[PROF_NCAT], and clears the records.
int sptorch_ext_prof_read(float* ms, uint32_t* launches, int ncat) {
    if (enter()) return 1;
    SPT_CUDA(cudaStreamSynchronize(g_rt.stream));
    std::lock_guard<std::mutex> lk(g_prof_mu);
    for (int i = 0; i < ncat; i++) { if (ms) ms[i] = 0.0f; if (launches) launches[i] = 0; }
    for (auto& r : g_prof_recs) {
        float t = 0.0f;
        cudaEventElapsedTime(&t, r.e0, r.e1);
        if (r.cat >= 0 && r.cat < ncat) { if (ms) ms[r.cat] += t; if (launches) launches[r.cat] += 1; }
        g_prof_free.push_back(r.e0); g_prof_free.push_back(r.e1);
    }
    g_prof_recs.clear();
    return 0;
}

uint32_t sptorch_ext_device_status(void) {
    if (enter() || !g_rt.dev_status) return 0;
    uint32_t st = 0;
    cudaStreamSynchronize(g_rt.stream);
    cudaMemcpy(&st, g_rt.dev_status, sizeof(st), cudaMemcpyDeviceToHost);
    return st;
}

}  // extern "C"
