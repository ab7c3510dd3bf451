// The fused exchange of the tensor-parallel step: partial products of all ranks -> residual add -> norm -> 8-bit activations
// on every rank, as ONE kernel per GPU over peer memory (NVLink loads and stores), in place of
// ncclAllReduce + add + norm on full rows.
//
// Under TSM_TP_REDUCE the o and down projections are split by input columns, so every rank holds a partial [tokens, width]
// product.  The rows (tokens) are dealt out to the ranks (row t belongs to rank t % ranks); the owner of a row
//   1. reads that row of every rank's partial product straight from the peers' memory and adds them in rank order
//      (a fixed order: the same bits on every run and every rank, which NCCL's reduction does not promise),
//   2. adds the residual stream's row (which only the owner keeps up to date) and folds the row's norm in the host's order,
//   3. quantises the normed row (quantize_block_q8) and stores the int8 values and block scales into EVERY rank's activation
//      buffer: 1.4 bytes per element cross NVLink instead of the 4 an all-reduce of floats moves.
// Two counters in each rank's exchange region order the ranks: "my partial product is complete" (one arrival per rank and
// exchange, waited for before step 1) and "row delivered" (one arrival per row and exchange on every rank, waited for before
// the kernel ends, so the product that follows reads complete rows).  Arrivals are system-scope atomic adds into the
// peers' regions; the counters only grow, and the targets are kept beside them on the device, so a captured graph replays
// the kernel unchanged.  Every wait is bounded: when it runs out the kernel sets the error record's timeout word and
// returns; nothing traps and no GPU is left spinning.  Plain peer loads and stores only: no multimem, no multicast.
// Where a row's 26 us go on two GPUs (clock64 around the phases): waiting for the peers' arrival 3-4, the peers' partial rows
// 2.7 (every rank's loads issued before the first add), the ordered sum of 4096 squares 9.3, norm and quantiser 3.2 (the
// norm's weights fetched before the sum), stores 0.8, the releasing arrival 3.5, waiting for the other rows 1.5-2.
//
// The regions are cudaMalloc'ed, exported with cudaIpcGetMemHandle, carried between the processes by an NCCL all-gather and
// opened with cudaIpcOpenMemHandle.  Where that is not possible (no peer access) the step keeps using NCCL's all-reduce.
#include <stdlib.h>

#include "model.cuh"
#include "row_helpers.cuh"

namespace tsm {

namespace {

constexpr int kXchgRows = 256;                 // most tokens of a step the fused exchange takes (more: NCCL's all-reduce)
constexpr int64_t kXchgHeader = 4096;
constexpr unsigned long long kXchgSpins = 40ull << 20;   // polls of ~0.25 us: about ten seconds

// The head of a rank's region.  `ready` and `delivered` are written by the peers; the targets by this GPU only.
struct XchgHeader {
    unsigned ready;          // arrivals "a rank's partial product is complete"
    unsigned pad0[31];
    unsigned delivered;      // arrivals "a row has been stored here"
    unsigned pad1[31];
    unsigned ready_target;   // `ready` as it stood when the last exchange had finished (what the running one adds to)
    unsigned delivered_target;
    unsigned finished;       // CTAs of the running exchange that are done (the last one moves the targets on)
    unsigned pad2[29];
};

struct XchgParams {
    unsigned char* regions[8];   // every rank's region as this process sees it ([rank] is its own)
    int ranks, rank;
    int total, width;            // tokens of the step, floats per row
    int64_t partial_at, quant_at;
    float* x;                    // the residual stream [total, width]: rows this rank owns are current
    const float* bias;           // added once to the summed row (GPT-2's projection bias), or null
    const float* norm_w;
    const float* norm_b;
    float eps;
    ErrorRecord* errors;
    unsigned long long spins;
    int chunked_sum;             // the norm's sum of squares chunk by chunk (chunked_sum_of_terms)
};

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_sys(unsigned* p, unsigned v) {
    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Waits until *counter has reached `target` (counters wrap with the targets: compare by difference).  Bounded.
__device__ __forceinline__ bool wait_counter(const unsigned* counter, unsigned target, unsigned long long limit) {
    for (unsigned long long spin = 0; spin < limit; spin++) {
        if ((int)(ld_acquire_sys(counter) - target) >= 0) return true;
        __nanosleep(spin < 64 ? 20 : 200);
    }
    return false;
}

// One CTA per row this rank owns (CTA c: row c * ranks + rank), at least one CTA per rank.
template <bool LAYER>
__global__ void tp_reduce_norm_kernel(XchgParams p) {
    chained_kernel_entry();
    extern __shared__ __align__(16) float row[];   // [width], then the terms of the ordered sums
    __shared__ float scratch[32];
    __shared__ SumScratch sum_scratch;
    __shared__ int proceed;
    const int n = p.width;
    float* terms = row + ((n + 3) & ~3);
    XchgHeader* mine = (XchgHeader*)p.regions[p.rank];
    const int t = blockIdx.x * p.ranks + p.rank;
    // what the counters will read once every rank has arrived for this exchange and every row of it has been stored here
    const unsigned ready_target = mine->ready_target + (unsigned)p.ranks, delivered_target = mine->delivered_target + (unsigned)p.total;

    // "my partial product is complete": the kernel before this one on the stream wrote it
    // (the release of the add itself orders everything the kernel before this one wrote: a separate system fence in front
    // of it cost a second 3.7 us)
    if (blockIdx.x == 0 && threadIdx.x < p.ranks) red_release_sys(&((XchgHeader*)p.regions[threadIdx.x])->ready, 1u);
    // what phase 3 needs of the norm's weight (and bias): fetched now, so that the loads are long back when the ordered
    // sums end (fetched after them they cost a trip to L2 per block of the row)
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int blocks = n >> 5;
    constexpr int kKeep = 8;
    const bool kept = blocks <= kKeep * warps;
    float wv[kKeep], bv[kKeep];
    if (kept) {
#pragma unroll
        for (int i = 0; i < kKeep; i++) {
            const int j = (warp + i * warps) * 32 + lane;
            wv[i] = j < n && p.norm_w ? p.norm_w[j] : 1.0f;
            bv[i] = LAYER && j < n ? p.norm_b[j] : 0.0f;
        }
    }
    if (threadIdx.x == 0) {
        bool ok = wait_counter(&mine->ready, ready_target, p.spins);
        if (!ok) atomicExch(&p.errors->timeout, 1);
        proceed = ok ? 1 : 0;
    }
    __syncthreads();
    const bool ok = proceed != 0;

    if (ok && t < p.total) {
        // 1. the row of every rank's partial product, added in rank order; 2. the residual
        float* xr = p.x + (int64_t)t * n;
        // two 16-byte pieces per thread and pass, every rank's loads of both issued before the first add: one trip over
        // NVLink per pass instead of one per piece
        const int step = blockDim.x * 4;
        for (int j0 = threadIdx.x * 4; j0 < n; j0 += 2 * step) {
            const int j1 = j0 + step;
            const bool two = j1 < n;
            float4 part[2][8], x4[2], b4[2];
#pragma unroll
            for (int q = 0; q < 8; q++) {
                if (q < p.ranks) {
                    const float* src = (const float*)(p.regions[q] + p.partial_at) + (int64_t)t * n;
                    part[0][q] = *(const float4*)(src + j0);
                    part[1][q] = two ? *(const float4*)(src + j1) : make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            x4[0] = *(const float4*)(xr + j0);
            x4[1] = two ? *(const float4*)(xr + j1) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (p.bias) {
                b4[0] = *(const float4*)(p.bias + j0);
                b4[1] = two ? *(const float4*)(p.bias + j1) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int k = 0; k < 2; k++) {
                if (k == 1 && !two) break;
                float4 sum = part[k][0];
#pragma unroll
                for (int q = 1; q < 8; q++) {
                    if (q < p.ranks) {
                        sum.x = __fadd_rn(sum.x, part[k][q].x), sum.y = __fadd_rn(sum.y, part[k][q].y);
                        sum.z = __fadd_rn(sum.z, part[k][q].z), sum.w = __fadd_rn(sum.w, part[k][q].w);
                    }
                }
                if (p.bias) {
                    sum.x = __fadd_rn(sum.x, b4[k].x), sum.y = __fadd_rn(sum.y, b4[k].y), sum.z = __fadd_rn(sum.z, b4[k].z), sum.w = __fadd_rn(sum.w, b4[k].w);
                }
                float4 v = x4[k];
                v.x = __fadd_rn(v.x, sum.x), v.y = __fadd_rn(v.y, sum.y), v.z = __fadd_rn(v.z, sum.z), v.w = __fadd_rn(v.w, sum.w);
                const int j = k == 0 ? j0 : j1;
                *(float4*)(xr + j) = v;
                *(float4*)(row + j) = v;
            }
        }
        __syncthreads();
        // the norm, in the host's order of addition (rmsnorm_row / the LayerNorm rows branch, devices/host.cr:348-403)
        const float count = (float)n;
        float mean = 0.0f;
        if (LAYER) mean = __fdiv_rn(ordered_sum<false>(row, terms, n, 0.0f, scratch), count);
        const float squares = ordered_sum_squares(row, terms, n, mean, scratch, &sum_scratch, p.chunked_sum != 0);
        const float denom = __fsqrt_rn(__fadd_rn(__fdiv_rn(squares, count), p.eps));
        // 3. quantised (staged in shared memory, over the terms, which are no longer needed), then stored to every rank in
        //    16-byte pieces
        // the normed values go to shared memory (over the sums' terms, 4 pad floats per block), then one thread per block
        // quantises them into the staging rows behind
        float* ybuf = terms;
        int8_t* q8 = (int8_t*)(terms + (n + (n >> 5) * 4 + 4));   // [n]
        float* head = (float*)(q8 + n);                    // [3][blocks]: scales, sums, totals (as bits)
        if (kept) {
#pragma unroll
            for (int i = 0; i < kKeep; i++) {
                const int j = (warp + i * warps) * 32 + lane;
                if (j < n) {
                    float c = LAYER ? __fsub_rn(row[j], mean) : row[j];
                    float y = __fdiv_rn(c, denom);
                    if (p.norm_w) y = __fmul_rn(y, wv[i]);
                    if (LAYER) y = __fadd_rn(y, bv[i]);
                    ybuf[j + (j >> 5) * 4] = y;
                }
            }
        } else {
            for (int j = threadIdx.x; j < n; j += blockDim.x) {
                float c = LAYER ? __fsub_rn(row[j], mean) : row[j];
                float y = __fdiv_rn(c, denom);
                if (p.norm_w) y = __fmul_rn(y, p.norm_w[j]);
                if (LAYER) y = __fadd_rn(y, p.norm_b[j]);
                ybuf[j + (j >> 5) * 4] = y;
            }
        }
        __syncthreads();
        for (int blk = threadIdx.x; blk < blocks; blk += blockDim.x)
            quantize_block_by_thread(ybuf + blk * 36, head + blk, head + blocks + blk, (int*)head + 2 * blocks + blk, q8 + blk * 32, true);
        __syncthreads();
        const int64_t all_blocks = (int64_t)p.total * blocks;
        const int64_t qs_at = (all_blocks * 12 + 255) / 256 * 256;   // quant_scratch_layout
        for (int q = 0; q < p.ranks; q++) {
            unsigned char* base = p.regions[q] + p.quant_at;
            uint4* dst = (uint4*)(base + qs_at + (int64_t)t * n);
            for (int i = threadIdx.x; i < n / 16; i += blockDim.x) dst[i] = ((const uint4*)q8)[i];
            for (int i = threadIdx.x; i < 3 * blocks; i += blockDim.x) {
                const int part = i / blocks, blk = i % blocks;
                ((float*)base)[part * all_blocks + (int64_t)t * blocks + blk] = head[i];
            }
        }
        __syncthreads();
        // "row delivered", on every rank
        // (the barrier above makes the CTA's stores this thread's to release; no fence of its own in front of the add)
        if (threadIdx.x < p.ranks) red_release_sys(&((XchgHeader*)p.regions[threadIdx.x])->delivered, 1u);
    }
    // the kernel ends when every row of the step has arrived here
    if (threadIdx.x == 0) {
        if (ok && !wait_counter(&mine->delivered, delivered_target, p.spins)) atomicExch(&p.errors->timeout, 1);
        __threadfence();
        if (atomicAdd(&mine->finished, 1u) == gridDim.x - 1) {   // the last CTA: the next exchange's targets
            mine->finished = 0;
            mine->ready_target = ready_target;
            mine->delivered_target = delivered_target;
        }
    }
}

}  // namespace

int64_t xchg_region_bytes(int width) {
    return kXchgHeader + (int64_t)kXchgRows * width * 4 + quant_scratch_bytes(kXchgRows, width) + 256;
}

// Allocates this rank's region, opens the peers', and zeroes the counters.  Collective: every rank of the group calls it
// at the same point (while the model is built).  Leaves m->xchg.ready false, without an error, when peer memory cannot be
// mapped: the step then exchanges through NCCL.
int xchg_setup(tsm_model* m) {
    tsm_ctx* ctx = m->ctx;
    Exchange& x = m->xchg;
    x = Exchange{};
    static const bool off = getenv("TSM_TP_FUSED") && getenv("TSM_TP_FUSED")[0] == '0';
    if (m->tp <= 1 || m->tp > 8 || !m->tp_reduce || off || m->cfg.width % 32 != 0) return TSM_OK;
    x.width = m->cfg.width, x.rows = kXchgRows;
    x.bytes = xchg_region_bytes(x.width);
    x.partial_at = kXchgHeader;
    x.quant_at = kXchgHeader + (int64_t)kXchgRows * x.width * 4;
    void* local = nullptr;
    cudaError_t err = cudaMalloc(&local, (size_t)x.bytes);
    if (err != cudaSuccess) return cuda_fail(ctx, err, "cudaMalloc of the exchange region");
    cudaMemsetAsync(local, 0, (size_t)x.bytes, ctx->stream);   // counters and targets start at zero on every rank
    // handles of all ranks, through a small device buffer and the group's all-gather; a rank that could not export its
    // region sends zeros, and then no rank uses the fused exchange
    cudaIpcMemHandle_t handle;
    memset(&handle, 0, sizeof(handle));
    bool exported = cudaIpcGetMemHandle(&handle, local) == cudaSuccess;
    if (!exported) cudaGetLastError(), memset(&handle, 0, sizeof(handle));
    const int64_t slot = 128;   // a handle is 64 bytes; a flag follows it
    unsigned char* table = nullptr;
    int rc = pool_alloc(ctx, slot * m->tp, (void**)&table);
    if (rc != TSM_OK) {
        cudaFree(local);
        return rc;
    }
    unsigned char mine[128] = {0};
    memcpy(mine, &handle, sizeof(handle));
    mine[64] = exported ? 1 : 0;
    cudaMemcpyAsync(table + slot * m->tp_rank, mine, (size_t)slot, cudaMemcpyHostToDevice, ctx->stream);
    rc = tp_all_gather(ctx, table, slot);
    std::vector<unsigned char> all((size_t)(slot * m->tp));
    if (rc == TSM_OK) {
        cudaMemcpyAsync(all.data(), table, all.size(), cudaMemcpyDeviceToHost, ctx->stream);
        rc = tp_stream_wait(ctx);
    }
    pool_release(ctx, table);
    if (rc != TSM_OK) {
        cudaFree(local);
        return rc;
    }
    bool usable = true;
    for (int q = 0; q < m->tp; q++) usable = usable && all[(size_t)(slot * q + 64)] == 1;
    for (int q = 0; q < m->tp && usable; q++) {
        if (q == m->tp_rank) {
            x.regions[q] = (unsigned char*)local;
            continue;
        }
        cudaIpcMemHandle_t theirs;
        memcpy(&theirs, &all[(size_t)(slot * q)], sizeof(theirs));
        void* mapped = nullptr;
        if (cudaIpcOpenMemHandle(&mapped, theirs, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            cudaGetLastError();
            usable = false;
            break;
        }
        x.regions[q] = (unsigned char*)mapped;
    }
    // every rank must come to the same decision: one more (tiny) all-gather of the outcome
    unsigned char* votes = nullptr;
    rc = pool_alloc(ctx, 4 * m->tp, (void**)&votes);
    int all_usable = 0;
    if (rc == TSM_OK) {
        int vote = usable ? 1 : 0;
        cudaMemcpyAsync(votes + 4 * m->tp_rank, &vote, 4, cudaMemcpyHostToDevice, ctx->stream);
        rc = tp_all_gather(ctx, votes, 4);
        std::vector<int> seen((size_t)m->tp, 0);
        if (rc == TSM_OK) {
            cudaMemcpyAsync(seen.data(), votes, (size_t)(4 * m->tp), cudaMemcpyDeviceToHost, ctx->stream);
            rc = tp_stream_wait(ctx);
        }
        all_usable = 1;
        for (int v : seen) all_usable = all_usable && v == 1;
        pool_release(ctx, votes);
    }
    x.local = local;
    if (rc != TSM_OK || !all_usable) {
        xchg_release(m);
        return rc;
    }
    x.ready = true;
    return TSM_OK;
}

// Closes the peers' regions, then frees this rank's once every rank has closed its view of it (the ranks free a model
// together, as they built it together; a group that has failed skips the rendezvous).
void xchg_release(tsm_model* m) {
    Exchange& x = m->xchg;
    tsm_ctx* ctx = m->ctx;
    bool mapped = false;
    for (int q = 0; q < 8; q++)
        if (x.regions[q] && x.regions[q] != (unsigned char*)x.local) cudaIpcCloseMemHandle(x.regions[q]), mapped = true;
    if (mapped && ctx->comm && !ctx->comm_failed) {
        unsigned char* token = nullptr;
        if (pool_alloc(ctx, 4 * m->tp, (void**)&token) == TSM_OK) {
            if (tp_all_gather(ctx, token, 4) == TSM_OK) tp_stream_wait(ctx);
            pool_release(ctx, token);
        }
    }
    if (x.local) cudaFree(x.local);
    cudaGetLastError();
    x = Exchange{};
}

bool xchg_takes(const tsm_model* m, int total) { return m->xchg.ready && total >= 1 && total <= m->xchg.rows; }

// Where the partial product of this rank goes, and where the quantised rows arrive (laid out as quant_scratch_layout
// for `total` rows of `width`).
float* xchg_partial(tsm_model* m) { return (float*)(m->xchg.regions[m->tp_rank] + m->xchg.partial_at); }
void* xchg_quantized(tsm_model* m) { return m->xchg.regions[m->tp_rank] + m->xchg.quant_at; }

// Queues one fused exchange over the step's `total` rows: partial products (already in xchg_partial on every rank) ->
// residual stream x -> norm with (w, b) -> quantised rows in xchg_quantized on every rank.
int launch_xchg_reduce_norm(tsm_model* m, int total, float* x, const float* bias, bool layer, const float* w, const float* b, float eps) {
    tsm_ctx* ctx = m->ctx;
    OpTimer timer(ctx, layer ? "Exchange reduce+LayerNorm" : "Exchange reduce+RMSNorm", total, m->xchg.width);
    if (ctx->comm_failed) return fail(ctx, TSM_ERR_COMM, "the tensor-parallel group has failed or was left");
    const Exchange& e = m->xchg;
    XchgParams p{};
    for (int q = 0; q < 8; q++) p.regions[q] = e.regions[q];
    p.ranks = m->tp, p.rank = m->tp_rank, p.total = total, p.width = e.width;
    p.partial_at = e.partial_at, p.quant_at = e.quant_at;
    p.x = x, p.bias = bias, p.norm_w = w, p.norm_b = b, p.eps = eps, p.errors = ctx->errors;
    p.spins = ctx->wait_spins ? ctx->wait_spins : kXchgSpins;
    static const int chunked = getenv("TSM_PLAIN_ORDERED_SUM") ? 0 : 1;
    p.chunked_sum = chunked;
    const int n = e.width;
    const int ctas = std::max(1, (total - m->tp_rank + m->tp - 1) / m->tp);
    const int threads = n >= 2048 ? 512 : n >= 512 ? 256 : 128;
    // the row; the terms of its ordered sums, later the normed values (36 floats per block); the quantised row and its scales
    const size_t smem = (size_t)(((n + 3) & ~3) + std::max((n + 15) & ~15, n + (n >> 5) * 4 + 4)) * 4 + (size_t)n + (size_t)(n >> 5) * 12 + 16;
    if (smem > 200 * 1024) return fail(ctx, TSM_ERR_UNSUPPORTED, "rows too wide for the fused exchange");
    if (layer) {
        if (smem > 48 * 1024) TSM_CUDA(ctx, cudaFuncSetAttribute(tp_reduce_norm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024));
        TSM_CUDA(ctx, launch_chained(ctx, tp_reduce_norm_kernel<true>, dim3(ctas), dim3(threads), smem, p));
    } else {
        if (smem > 48 * 1024) TSM_CUDA(ctx, cudaFuncSetAttribute(tp_reduce_norm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024));
        TSM_CUDA(ctx, launch_chained(ctx, tp_reduce_norm_kernel<false>, dim3(ctas), dim3(threads), smem, p));
    }
    count_launch(ctx);
    ctx->counters.collectives++;
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

}  // namespace tsm
