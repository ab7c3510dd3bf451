// Tensor-parallel plumbing: one process per GPU, NCCL over NVLink for the exchanges between the sharded
// projections.  The reference has one device per model (src/tensomite/device.cr); this is the sharding its
// large models need on several GPUs.  NCCL is bound at run time (dlopen of libnccl.so.2, or the path in
// TSM_NCCL_LIBRARY), so the library itself links the CUDA runtime only and single-GPU hosts need no NCCL.
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

namespace tsm {

namespace {

struct NcclId {
    char bytes[128];
};
typedef int (*GetUniqueId)(NcclId*);
typedef int (*CommInitRank)(void**, int, NcclId, int);
typedef int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef int (*CommDestroy)(void*);
typedef const char* (*GetErrorString)(int);

struct Nccl {
    void* handle = nullptr;
    GetUniqueId get_unique_id = nullptr;
    CommInitRank comm_init_rank = nullptr;
    AllGather all_gather = nullptr;
    AllReduce all_reduce = nullptr;
    CommDestroy comm_destroy = nullptr;
    GetErrorString error_string = nullptr;
    std::string problem;
};

Nccl& nccl() {
    static Nccl lib = [] {
        Nccl n;
        const char* path = getenv("TSM_NCCL_LIBRARY");
        n.handle = dlopen(path ? path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!n.handle) {
            n.problem = std::string("NCCL could not be loaded: ") + dlerror();
            return n;
        }
        n.get_unique_id = (GetUniqueId)dlsym(n.handle, "ncclGetUniqueId");
        n.comm_init_rank = (CommInitRank)dlsym(n.handle, "ncclCommInitRank");
        n.all_gather = (AllGather)dlsym(n.handle, "ncclAllGather");
        n.all_reduce = (AllReduce)dlsym(n.handle, "ncclAllReduce");
        n.comm_destroy = (CommDestroy)dlsym(n.handle, "ncclCommDestroy");
        n.error_string = (GetErrorString)dlsym(n.handle, "ncclGetErrorString");
        if (!n.get_unique_id || !n.comm_init_rank || !n.all_gather || !n.all_reduce || !n.comm_destroy) n.problem = "the NCCL library lacks an entry point";
        return n;
    }();
    return lib;
}

int nccl_fail(tsm_ctx* ctx, int rc, const char* call) {
    Nccl& n = nccl();
    return fail(ctx, TSM_ERR_EXECUTION, std::string(call) + ": " + (n.error_string ? n.error_string(rc) : "NCCL error " + std::to_string(rc)));
}

constexpr int kNcclInt8 = 0;  // ncclDataType_t: bytes are gathered, whatever they hold
constexpr int kNcclFloat32 = 7, kNcclSum = 0;

// dst[t, seg * width + j] (+)= src[seg, t, j]: the ranks' column slices, as an all-gather leaves them, back in row order.
template <bool ADD>
__global__ void interleave_kernel(const float* __restrict__ src, float* dst, int rows, int width, int parts) {
    chained_kernel_entry();
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = (int64_t)rows * width * parts;
    if (i >= total) return;
    int full = width * parts;
    int t = (int)(i / full), c = (int)(i % full);
    int seg = c / width, j = c % width;
    float v = src[((int64_t)seg * rows + t) * width + j];
    dst[i] = ADD ? __fadd_rn(dst[i], v) : v;
}

}  // namespace

// Every rank's `bytes` at buffer + rank * bytes become visible to all, in place.
int tp_all_gather(tsm_ctx* ctx, void* buffer, int64_t bytes) {
    if (ctx->tp_world <= 1) return TSM_OK;
    Nccl& n = nccl();
    int rc = n.all_gather((const char*)buffer + (int64_t)ctx->tp_rank * bytes, buffer, (size_t)bytes, kNcclInt8, ctx->comm, ctx->stream);
    if (rc != 0) return nccl_fail(ctx, rc, "ncclAllGather");
    ctx->counters.host_ops++;
    return TSM_OK;
}

// Every rank's `count` floats are replaced by their sum over the ranks, in NCCL's order of addition.
int tp_all_reduce_sum(tsm_ctx* ctx, float* buffer, int64_t count) {
    if (ctx->tp_world <= 1) return TSM_OK;
    int rc = nccl().all_reduce(buffer, buffer, (size_t)count, kNcclFloat32, kNcclSum, ctx->comm, ctx->stream);
    if (rc != 0) return nccl_fail(ctx, rc, "ncclAllReduce");
    ctx->counters.host_ops++;
    return TSM_OK;
}

int launch_interleave(tsm_ctx* ctx, const float* gathered, float* dst, int rows, int width, int parts, bool add) {
    int64_t total = (int64_t)rows * width * parts;
    if (total == 0) return TSM_OK;
    unsigned grid = (unsigned)((total + 255) / 256);
    if (add) TSM_CUDA(ctx, launch_chained(ctx, interleave_kernel<true>, dim3(grid), dim3(256), 0, gathered, dst, rows, width, parts));
    else TSM_CUDA(ctx, launch_chained(ctx, interleave_kernel<false>, dim3(grid), dim3(256), 0, gathered, dst, rows, width, parts));
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

void tp_release(tsm_ctx* ctx) {
    if (ctx->comm) nccl().comm_destroy(ctx->comm);
    ctx->comm = nullptr, ctx->tp_world = 1, ctx->tp_rank = 0;
}

}  // namespace tsm

extern "C" {

int tsm_tp_unique_id(uint8_t* out) {
    if (!out) return TSM_ERR_ARG;
    tsm::Nccl& n = tsm::nccl();
    if (!n.problem.empty()) return TSM_ERR_UNSUPPORTED;
    tsm::NcclId id;
    if (n.get_unique_id(&id) != 0) return TSM_ERR_EXECUTION;
    memcpy(out, id.bytes, 128);
    return TSM_OK;
}

int tsm_tp_init(tsm_ctx* ctx, int rank, int world, const uint8_t* id) {
    if (!ctx) return TSM_ERR_ARG;
    tsm::DeviceGuard guard(ctx->ordinal);
    if (world < 1 || rank < 0 || rank >= world || (world > 1 && !id)) return tsm::fail(ctx, TSM_ERR_ARG, "rank " + std::to_string(rank) + " of " + std::to_string(world));
    if (ctx->comm) return tsm::fail(ctx, TSM_ERR_ARG, "this context already belongs to a group");
    if (world == 1) return TSM_OK;
    tsm::Nccl& n = tsm::nccl();
    if (!n.problem.empty()) return tsm::fail(ctx, TSM_ERR_UNSUPPORTED, n.problem);
    tsm::NcclId uid;
    memcpy(uid.bytes, id, 128);
    void* comm = nullptr;
    int rc = n.comm_init_rank(&comm, world, uid, rank);
    if (rc != 0) return tsm::nccl_fail(ctx, rc, "ncclCommInitRank");
    ctx->comm = comm, ctx->tp_rank = rank, ctx->tp_world = world;
    return TSM_OK;
}

int tsm_tp_variant(tsm_ctx* ctx, int variant) {
    if (!ctx) return TSM_ERR_ARG;
    if (variant != TSM_TP_GATHER && variant != TSM_TP_REDUCE) return tsm::fail(ctx, TSM_ERR_ARG, "unknown tensor-parallel variant");
    ctx->tp_variant = variant;
    return TSM_OK;
}

int tsm_tp_info(tsm_ctx* ctx, int* rank, int* world) {
    if (!ctx) return TSM_ERR_ARG;
    if (rank) *rank = ctx->tp_rank;
    if (world) *world = ctx->tp_world;
    return TSM_OK;
}

}  // extern "C"
