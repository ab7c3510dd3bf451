// Tensor-parallel plumbing: one process per GPU, NCCL over NVLink for the exchanges between the sharded
// projections.  The reference has one device per model (src/tensomite/device.cr); this is the sharding its
// large models need on several GPUs.  NCCL is bound at run time (dlopen of libnccl.so.2, or the path in
// TSM_NCCL_LIBRARY), so the library itself links the CUDA runtime only and single-GPU hosts need no NCCL.
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

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
typedef int (*CommAbort)(void*);
typedef int (*CommGetAsyncError)(void*, int*);
typedef int (*ReduceScatter)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef const char* (*GetErrorString)(int);

struct Nccl {
    void* handle = nullptr;
    GetUniqueId get_unique_id = nullptr;
    CommInitRank comm_init_rank = nullptr;
    AllGather all_gather = nullptr;
    AllReduce all_reduce = nullptr;
    CommDestroy comm_destroy = nullptr;
    CommAbort comm_abort = nullptr;                   // optional: absent from a stub, the communicator is then only dropped
    CommGetAsyncError comm_async_error = nullptr;     // optional
    ReduceScatter reduce_scatter = nullptr;           // optional
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
        n.comm_abort = (CommAbort)dlsym(n.handle, "ncclCommAbort");
        n.comm_async_error = (CommGetAsyncError)dlsym(n.handle, "ncclCommGetAsyncError");
        n.reduce_scatter = (ReduceScatter)dlsym(n.handle, "ncclReduceScatter");
        n.error_string = (GetErrorString)dlsym(n.handle, "ncclGetErrorString");
        if (!n.get_unique_id || !n.comm_init_rank || !n.all_gather || !n.all_reduce || !n.comm_destroy) n.problem = "the NCCL library lacks an entry point";
        return n;
    }();
    return lib;
}

// Every failure of the communicator is TSM_ERR_COMM: the group is no longer usable and the host has to drop it
// (tsm_tp_abort) and rebuild, whatever NCCL's own code said.
int nccl_fail(tsm_ctx* ctx, int rc, const char* call) {
    Nccl& n = nccl();
    ctx->comm_failed = true;
    return fail(ctx, TSM_ERR_COMM, std::string(call) + ": " + (n.error_string ? n.error_string(rc) : "NCCL error " + std::to_string(rc)));
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
    OpTimer timer(ctx, "AllGather", bytes);
    if (ctx->tp_world <= 1) return TSM_OK;
    if (ctx->comm_failed || !ctx->comm) return fail(ctx, TSM_ERR_COMM, "the tensor-parallel group has failed or was left");
    Nccl& n = nccl();
    int rc = n.all_gather((const char*)buffer + (int64_t)ctx->tp_rank * bytes, buffer, (size_t)bytes, kNcclInt8, ctx->comm, ctx->stream);
    if (rc != 0) return nccl_fail(ctx, rc, "ncclAllGather");
    ctx->counters.collectives++;
    return TSM_OK;
}

// Every rank's `count` floats are replaced by their sum over the ranks, in NCCL's order of addition.
int tp_all_reduce_sum(tsm_ctx* ctx, float* buffer, int64_t count) {
    OpTimer timer(ctx, "AllReduce", count);
    if (ctx->tp_world <= 1) return TSM_OK;
    if (ctx->comm_failed || !ctx->comm) return fail(ctx, TSM_ERR_COMM, "the tensor-parallel group has failed or was left");
    int rc = nccl().all_reduce(buffer, buffer, (size_t)count, kNcclFloat32, kNcclSum, ctx->comm, ctx->stream);
    if (rc != 0) return nccl_fail(ctx, rc, "ncclAllReduce");
    ctx->counters.collectives++;
    return TSM_OK;
}

// Waits for the context's stream the way a member of a group has to: never without a limit.  The stream is polled; between
// polls the communicator is asked whether it has failed behind the host's back (a peer that died, a link error), and after
// `TSM_TP_TIMEOUT_MS` (default 60 s) without progress the wait gives up.  Either way the communicator is aborted, so that no
// kernel of it keeps spinning on the GPU, and the call returns TSM_ERR_COMM (failure) or TSM_ERR_TIMEOUT (no progress).
int tp_stream_wait(tsm_ctx* ctx) {
    if (ctx->tp_world <= 1 || !ctx->comm) {
        TSM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        return TSM_OK;
    }
    static const double limit_ms = getenv("TSM_TP_TIMEOUT_MS") ? atof(getenv("TSM_TP_TIMEOUT_MS")) : 60000.0;
    Nccl& n = nccl();
    timespec t0;
    clock_gettime(CLOCK_MONOTONIC, &t0);
    for (unsigned poll = 0;; poll++) {
        cudaError_t state = cudaStreamQuery(ctx->stream);
        if (state == cudaSuccess) return TSM_OK;
        if (state != cudaErrorNotReady) return cuda_fail(ctx, state, "cudaStreamQuery");
        if ((poll & 63) == 63) {
            int async = 0;
            if (n.comm_async_error && n.comm_async_error(ctx->comm, &async) == 0 && async != 0) {
                tp_abort(ctx);
                return fail(ctx, TSM_ERR_COMM, std::string("the communicator failed while a step was running: ") +
                                                   (n.error_string ? n.error_string(async) : "NCCL error " + std::to_string(async)));
            }
            timespec t1;
            clock_gettime(CLOCK_MONOTONIC, &t1);
            double ms = (t1.tv_sec - t0.tv_sec) * 1e3 + (t1.tv_nsec - t0.tv_nsec) * 1e-6;
            if (ms > limit_ms) {
                tp_abort(ctx);
                return fail(ctx, TSM_ERR_TIMEOUT, "a tensor-parallel step made no progress for " + std::to_string((int)limit_ms) + " ms: a rank is missing");
            }
        }
        if (poll > 2000) {  // a step takes milliseconds: after the first spins, stop burning the core
            timespec nap{0, 20000};
            nanosleep(&nap, nullptr);
        }
    }
}

// Drops the communicator without waiting for its peers (ncclCommAbort); later exchanges fail with TSM_ERR_COMM.
void tp_abort(tsm_ctx* ctx) {
    if (ctx->comm) {
        Nccl& n = nccl();
        if (n.comm_abort) n.comm_abort(ctx->comm);
        ctx->comm = nullptr;
    }
    ctx->comm_failed = true;
}

int launch_interleave(tsm_ctx* ctx, const float* gathered, float* dst, int rows, int width, int parts, bool add) {
    OpTimer timer(ctx, "Interleave", rows, width * parts);
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
    ctx->comm = nullptr, ctx->tp_world = 1, ctx->tp_rank = 0, ctx->comm_failed = false;
}

}  // namespace tsm

extern "C" {

int tsm_tp_unique_id(uint8_t* out) {
    if (!out) return TSM_ERR_ARG;
    tsm::Nccl& n = tsm::nccl();
    if (!n.problem.empty()) return TSM_ERR_UNSUPPORTED;
    tsm::NcclId id;
    if (n.get_unique_id(&id) != 0) return TSM_ERR_COMM;
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

int tsm_tp_abort(tsm_ctx* ctx) {
    if (!ctx) return TSM_ERR_ARG;
    tsm::DeviceGuard guard(ctx->ordinal);
    tsm::tp_abort(ctx);
    return TSM_OK;
}

int tsm_tp_info(tsm_ctx* ctx, int* rank, int* world) {
    if (!ctx) return TSM_ERR_ARG;
    if (rank) *rank = ctx->tp_rank;
    if (world) *world = ctx->tp_world;
    return TSM_OK;
}

}  // extern "C"
