// nccl_comm.cu -- NCCL over NVLink / NVSwitch, bound at run time with dlopen so that the library has
// no link-time dependency and shares the one NCCL the host process already loaded.
//
// Replaces the reference's gRPC star all-reduce (crates/distributed/src/coordinator.rs:73-116: every
// worker sends its f32 vector to a coordinator that returns sum / world_size) and the host-side
// average_gradients (crates/distributed/src/allreduce.rs:4-20).  One process per GPU; rank 0 creates
// the unique id and the host program hands it to the other ranks (torch.distributed store, MPI, a file).
// Data always lands in this GPU's own HBM before a kernel of ours reads it; no kernel here touches a
// peer's memory.
#include "common.h"
#include "../../include/sptorch_b200_ext.h"
#include <nccl.h>
#include <dlfcn.h>
#include <cstring>
#include <cstdlib>

namespace spt {

struct NcclApi {
    void* h = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*) = nullptr;      // optional
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};
static NcclApi g_nccl;
static ncclComm_t g_comm = nullptr;
static int g_world = 1, g_rank = 0;

static int load_nccl(const char* path) {
    if (g_nccl.h) return 0;
    const char* cands[] = {path, "libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (const char* c : cands) {
        if (!c || !*c) continue;
        h = dlopen(c, RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
    }
    if (!h) return fail("nccl: could not dlopen libnccl (%s)", dlerror());
    g_nccl.h = h;
    g_nccl.GetUniqueId = (decltype(g_nccl.GetUniqueId))dlsym(h, "ncclGetUniqueId");
    g_nccl.CommInitRank = (decltype(g_nccl.CommInitRank))dlsym(h, "ncclCommInitRank");
    g_nccl.CommInitRankConfig = (decltype(g_nccl.CommInitRankConfig))dlsym(h, "ncclCommInitRankConfig");
    g_nccl.AllReduce = (decltype(g_nccl.AllReduce))dlsym(h, "ncclAllReduce");
    g_nccl.CommDestroy = (decltype(g_nccl.CommDestroy))dlsym(h, "ncclCommDestroy");
    g_nccl.GetErrorString = (decltype(g_nccl.GetErrorString))dlsym(h, "ncclGetErrorString");
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.AllReduce || !g_nccl.CommDestroy || !g_nccl.GetErrorString) {
        g_nccl = NcclApi();
        return fail("nccl: libnccl lacks a required symbol");
    }
    return 0;
}

#define SPT_NCCL(expr)                                                                                   \
    do {                                                                                                 \
        ncclResult_t _r = (expr);                                                                        \
        if (_r != ncclSuccess) return ::spt::fail("%s failed: %s", #expr, g_nccl.GetErrorString(_r));    \
    } while (0)

int nccl_allreduce_on_stream(void* buf, size_t n, int dtype, void* stream, void*) {
    if (!g_comm) return fail("nccl: communicator not initialised");
    SPT_NCCL(g_nccl.AllReduce(buf, buf, n, dtype == BF16 ? ncclBfloat16 : ncclFloat32, ncclSum, g_comm, (cudaStream_t)stream));
    return 0;
}

__global__ void scale_inplace_kernel(float* p, float s, size_t n) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = p[i] * s;
}

}  // namespace spt

using namespace spt;

extern "C" {

int sptorch_ext_nccl_unique_id(const char* libnccl_path, void* id128) {
    if (enter()) return 1;
    if (!id128) return fail("nccl_unique_id: null output");
    if (load_nccl(libnccl_path)) return 1;
    ncclUniqueId id;
    SPT_NCCL(g_nccl.GetUniqueId(&id));
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
    memcpy(id128, &id, 128);
    return 0;
}

int sptorch_ext_nccl_init(const char* libnccl_path, const void* id128, int rank, int world) {
    if (enter()) return 1;
    if (!id128 || world < 1 || rank < 0 || rank >= world) return fail("nccl_init: bad arguments (rank %d of %d)", rank, world);
    if (g_comm) return fail("nccl_init: already initialised");
    if (load_nccl(libnccl_path)) return 1;
    ncclUniqueId id;
    memcpy(&id, id128, 128);
    // SPTORCH_B200_NCCL_MAX_CTAS caps the CTAs a collective of this communicator may use, so that a collective running beside the
    // persistent GEMM / attention kernels (sptorch_ext_set_sm_reserve leaves it that many SMs) fits into the SMs left free
    const char* cap = getenv("SPTORCH_B200_NCCL_MAX_CTAS");
    if (cap && atoi(cap) > 0 && g_nccl.CommInitRankConfig) {
        ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
        cfg.maxCTAs = atoi(cap);
        cfg.minCTAs = 1;
        SPT_NCCL(g_nccl.CommInitRankConfig(&g_comm, world, id, rank, &cfg));
    } else {
        SPT_NCCL(g_nccl.CommInitRank(&g_comm, world, id, rank));
    }
    g_world = world; g_rank = rank;
    return 0;
}

int sptorch_ext_nccl_allreduce_sum(void* buf, size_t n, int dtype) {
    if (enter()) return 1;
    if (n == 0) return 0;
    if (!buf) return fail("nccl_allreduce: null buffer");
    if (dtype != SPT_F32 && dtype != SPT_BF16) return fail("nccl_allreduce: unknown dtype %d", dtype);
    if (nccl_allreduce_on_stream(buf, n, dtype, (void*)rt().stream, nullptr)) return 1;
    note_submit();
    return 0;
}

// average_gradients semantics of the reference: sum over ranks, then multiply by 1/world
int sptorch_ext_nccl_allreduce_avg_f32(void* buf, size_t n) {
    if (sptorch_ext_nccl_allreduce_sum(buf, n, SPT_F32)) return 1;
    if (n == 0) return 0;
    int grid = rt().sm_count * 4;
    scale_inplace_kernel<<<grid, 256, 0, rt().stream>>>((float*)buf, 1.0f / (float)g_world, n);
    SPT_LAUNCH_CHECK("allreduce_avg_scale");
    return 0;
}

int sptorch_ext_nccl_shutdown(void) {
    if (g_comm) {
        if (!enter()) cudaStreamSynchronize(rt().stream);
        g_nccl.CommDestroy(g_comm);
        g_comm = nullptr;
    }
    g_world = 1; g_rank = 0;
    return 0;
}

// route the tensor-parallel partial sums of a GPT through the NCCL communicator
int sptorch_ext_gpt_use_nccl(void* gpt) {
    if (!g_comm) return fail("gpt_use_nccl: call sptorch_ext_nccl_init first");
    return sptorch_ext_gpt_set_allreduce(gpt, nccl_allreduce_on_stream, nullptr);
}

}  // extern "C"
