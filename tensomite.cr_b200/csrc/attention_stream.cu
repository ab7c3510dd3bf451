// Ordered ("exact") ragged attention for head width 128 and 4 query heads per key/value head, built to keep the
// memory system busy: the same arithmetic, in the same order, as attention_exact_kernel (the host's sequential
// sums, Tensor attention in the reference's CPU device), but
//   * keys and values arrive through ONE ring of shared-memory stages filled by a producer thread with tiled
//     tensor copies (cp.async.bulk.tensor.2d, 128-byte swizzle, four boxes of 32 floats x 32 positions per tile)
//     that complete on an mbarrier; the producer runs ahead through the whole key pass and straight on into the
//     value pass, so the softmax phase in between does not drain the ring;
//   * scores do not live in shared memory: they go to a scratch array in global memory (it stays in L2), are turned
//     into exp values in place, and come back tile by tile as weights;
//   * the score phase is a pipeline over the four quarters of the width: a warp keeps its quarter of the four heads'
//     queries in registers and its lanes are the positions of a tile, so keys are read once, with 16-byte loads that
//     hit 32 distinct rows, and no query is ever re-read from shared memory (a 16-byte shared load costs four
//     wavefronts even when every lane reads the same address, which is what bounded the earlier kernels);
//   * consumer warps synchronise among themselves with a named barrier only where data is exchanged (maximum,
//     denominator, a tile's weights), never with the producer.
// One CTA per (token, key/value head): 128 consumer threads + one producer warp.  The output rows can be written
// quantised for the product that follows (QuantSink).  Further down: the same arithmetic as three launches
// (attention_scores_kernel, attention_weights_kernel, attention_values_kernel) for calls that cannot fill the GPU.
#include "common.cuh"
#include "row_helpers.cuh"

namespace tsm {

namespace {

constexpr int kTP = 32;            // positions per tile
constexpr int kRing = 4;           // stages of the split-path and prefill kernels' rings
constexpr int kConsumers = 128;
constexpr unsigned kSpinLimit = 4u << 20;
constexpr int kWideDeep = 6;       // stages of 4 KB in attention_values_wide_kernel's ring

struct StreamParams {
    const float* q;
    int64_t q_stride;
    int heads, rows, kv_heads, capacity;
    const int* table;
    float scale;
    float* out;
    ErrorRecord* errors;
    const int* order;
    float* scratch;  // [tokens][heads][capacity]: scores, then exp values (split path: then weights)
    int splits;      // split path: CTAs that share one (token, kv head)'s key positions
    QuantSink sink;  // where the output rows also go quantised (or nulls)
    unsigned wait_hint;  // nanoseconds a waiting thread may sleep per poll (0: plain polling)
};

struct StreamMaps {
    CUtensorMap k, v;  // f32 [rows * kv_heads * capacity, width], box 32 x kTP, 128-byte swizzle
};

__device__ __forceinline__ unsigned s_smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void s_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s_smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void s_mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void s_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool s_mbar_try_wait(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(s_smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// The same poll, but the thread may be suspended for up to `hint_ns` while the phase has not completed: a waiting warp then
// leaves its issue slots to the warps that have work.
__device__ __forceinline__ bool s_mbar_try_wait_sleeping(uint64_t* bar, unsigned parity, unsigned hint_ns) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(s_smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
// Bounded: gives up after kSpinLimit polls, or soon after another warp has raised the CTA's abort flag.  abort_flag[2] holds
// the suspend hint in nanoseconds (0: plain polling).
__device__ __forceinline__ bool s_mbar_wait(uint64_t* bar, unsigned parity, volatile int* abort_flag) {
    if (s_mbar_try_wait(bar, parity)) return true;
    const unsigned hint = (unsigned)abort_flag[2];
    for (unsigned spin = 0; spin < kSpinLimit; spin++) {
        if (hint ? s_mbar_try_wait_sleeping(bar, parity, hint) : s_mbar_try_wait(bar, parity)) return true;
        if (hint || spin > 256) {
            if (*abort_flag) return false;
            if (!hint) __nanosleep(64);
        }
    }
    return false;
}
__device__ __forceinline__ void s_tensor_load(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     s_smem_u32(dst)),
                 "l"(map), "r"(x), "r"(y), "r"(s_smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory"); }

// attention_stream_kernel's shared memory before the ring: 1 KB of barriers and flags, then 12 KB that hold the score
// pipeline's hand-over slots (3 warps x RING x 512 bytes) and, once all scores are made, the exp values of a chunk and the
// weights of the tiles being folded.
constexpr int kSEChunk = 512;          // positions whose exp values are staged at once for the denominator's chain
constexpr int kStreamHeader = 1024 + 12288;

template <int WIDTH, int RING>
__global__ void __launch_bounds__(kConsumers + 32, 2) attention_stream_kernel(StreamParams p, const __grid_constant__ StreamMaps maps) {
    chained_kernel_entry();
    constexpr int G = 4;
    constexpr int BOXES = WIDTH / 32;              // 128-byte wide boxes per row
    constexpr int BOX_BYTES = kTP * 128;
    constexpr int STAGE_BYTES = BOXES * BOX_BYTES;
    constexpr int QP = WIDTH + 4;                  // query row pitch: the four heads' 16-byte reads fall in distinct banks
    static_assert(WIDTH == kConsumers && BOXES == kConsumers / 32, "one folding thread per column, one box per warp");
    static_assert(RING >= 2 && RING <= 6, "the header is laid out for at most 6 stages");
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (s_smem_u32(smem_raw) & 1023u)) & 1023u);  // an offset from the shared array: the address space stays known
    // RING stages of 16 KB: measured 262, 239 and 233 us for 3, 4 and 5 stages at the headline shape (two CTAs still fit an
    // SM at 5).  A ring per box (each warp's quarter refilled as soon as that warp is done with it, since the last warp of the
    // score pipeline runs three tiles behind the first) measured 3 % slower at every depth than one barrier pair per stage.
    uint64_t* full = (uint64_t*)smem;              // [RING], bytes 0..63
    uint64_t* empty = (uint64_t*)(smem + 64);      // [RING], bytes 64..127
    uint64_t* ready = (uint64_t*)(smem + 512);     // [3 warps][RING], bytes 512..703: a tile's running sums are in `hand`
    volatile int* abort_flag = (volatile int*)(smem + 896);   // [1] stays 0
    float* maxes = (float*)(smem + 912);           // [4]
    float* totals = (float*)(smem + 928);          // [4]
    float* hand = (float*)(smem + 1024);           // [3 warps][RING][32 positions][4 heads]: the score phase only
    float* ebuf = (float*)(smem + 1024);           // [G][kSEChunk]: after the score phase (a barrier of all consumers lies between)
    float* wbuf = ebuf + G * kSEChunk;             // [2][4 tiles][kTP][G]
    static_assert(3 * RING * 512 <= 12288 && (G * kSEChunk + 2 * 4 * kTP * G) * 4 <= 12288, "both uses fit the 12 KB");
    unsigned char* stages = smem + kStreamHeader;  // [RING][BOXES][kTP][128 bytes], swizzled
    float* qs = (float*)(stages + RING * STAGE_BYTES);   // [G][QP]

    const int token = p.order ? p.order[blockIdx.y] : blockIdx.y;  // longest tokens first when an order is given
    const int per_kv = p.heads / p.kv_heads, groups_per_kv = per_kv / G;
    const int kvh = blockIdx.x / groups_per_kv;
    const int head0 = kvh * per_kv + (blockIdx.x % groups_per_kv) * G;
    const int row = p.table[3 * token], limit = p.table[3 * token + 1];
    if (row < 0 || row >= p.rows || limit < 0 || limit >= p.capacity) {
        if (threadIdx.x == 0 && blockIdx.x == 0) report_bad_index(p.errors, limit, p.capacity);
        return;
    }
    const int len = limit + 1;
    const int tiles = (len + kTP - 1) / kTP;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    if (tid == 0) {
        for (int i = 0; i < RING; i++) s_mbar_init(&full[i], 1), s_mbar_init(&empty[i], BOXES);
        for (int i = 0; i < 3 * RING; i++) s_mbar_init(&ready[i], 1);
        abort_flag[0] = 0, abort_flag[1] = 0, abort_flag[2] = (int)p.wait_hint, abort_flag[3] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    {
        // the four heads' queries: every thread's loads issued before its first store (one per pass, each waited for, cost a
        // trip to L2 per pass)
        const float* qsrc = p.q + (int64_t)token * p.q_stride + (int64_t)head0 * WIDTH;
        constexpr int kPasses = (G * WIDTH + kConsumers + 31) / (kConsumers + 32);
        float qv[kPasses];
#pragma unroll
        for (int u = 0; u < kPasses; u++) {
            const int i = tid + u * (kConsumers + 32);
            qv[u] = i < G * WIDTH ? qsrc[i] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < kPasses; u++) {
            const int i = tid + u * (kConsumers + 32);
            if (i < G * WIDTH) qs[(i / WIDTH) * QP + i % WIDTH] = qv[u];
        }
    }
    __syncthreads();

    if (warp == kConsumers / 32) {
        // ------------------------------------------------------------ producer: keys, then values, one ring
        if (lane != 0) return;
        const int plane = (row * p.kv_heads + kvh) * p.capacity;   // first row of this (stream, kv head) in the maps
        int issued = 0;
        bool ok = true;
        for (int j = 0; j < 2 * tiles; j++) {
            int s = j % RING;
            if (j >= RING) ok = s_mbar_wait(&empty[s], (unsigned)((j / RING - 1) & 1), abort_flag);
            if (!ok) break;
            const CUtensorMap* map = j < tiles ? &maps.k : &maps.v;
            int y = plane + (j < tiles ? j : j - tiles) * kTP;
            unsigned char* dst = stages + (size_t)s * STAGE_BYTES;
            s_mbar_expect_tx(&full[s], STAGE_BYTES);
#pragma unroll
            for (int b = 0; b < BOXES; b++) s_tensor_load(dst + b * BOX_BYTES, map, 32 * b, y, &full[s]);
            issued = j + 1;
        }
        if (!ok) {
            // the consumers stopped arriving: say so, then see the copies already issued land before leaving
            *abort_flag = 1;
            atomicExch(&p.errors->timeout, 1);
            for (int j = max(0, issued - RING); j < issued; j++) s_mbar_wait(&full[j % RING], (unsigned)((j / RING) & 1), abort_flag + 1);
        }
        return;
    }

    // ---------------------------------------------------------------- consumers
    // A wait that gives up raises the abort flag and the thread carries on with whatever the stage holds, so that
    // every named barrier below is still reached by all 128 threads; the results are then dropped.
    bool ok = true;
    const int sp = tid >> 2, shd = tid & 3;        // in the output phase: the position within a tile and the head whose weight this thread makes
    float* srow = p.scratch + ((int64_t)token * p.heads + head0) * p.capacity;   // + h * capacity + position

    // ---- 1. scores: a pipeline over the four quarters of the width ----
    // Warp w owns columns [32 w, 32 w + 32): its lanes are the 32 positions of a tile, and each thread keeps its
    // quarter of the four heads' queries in registers.  A position's dot products start in warp 0, which folds
    // columns 0..31 and hands the four running sums to warp 1 through shared memory, and so on: the adds happen in
    // column order, as one chain, but every warp works on a different tile at any moment.  Keys are read once per
    // position and quarter with 16-byte loads that hit 32 distinct rows (no broadcast traffic, no query loads).
    float top[G] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
    {
        float qreg[G][32];
#pragma unroll
        for (int h = 0; h < G; h++)
#pragma unroll
            for (int j = 0; j < 32; j++) qreg[h][j] = qs[h * QP + 32 * warp + j];
        const int sw = lane & 7;
        for (int tile = 0; tile < tiles; tile++) {
            const int s = tile % RING;
            const unsigned parity = (unsigned)((tile / RING) & 1);
            if (!s_mbar_wait(&full[s], parity, abort_flag)) ok = false, *abort_flag = 1;
            float acc[G] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (warp > 0) {
                if (!s_mbar_wait(&ready[(warp - 1) * RING + s], parity, abort_flag)) ok = false, *abort_flag = 1;
                float4 in = *(const float4*)(hand + (((warp - 1) * RING + s) * 32 + lane) * 4);
                acc[0] = in.x, acc[1] = in.y, acc[2] = in.z, acc[3] = in.w;
            }
            const unsigned char* rowp = stages + (size_t)s * STAGE_BYTES + warp * BOX_BYTES + lane * 128;
#pragma unroll
            for (int c = 0; c < 8; c++) {
                float4 kv4 = *(const float4*)(rowp + ((c ^ sw) << 4));
#pragma unroll
                for (int h = 0; h < G; h++) {
                    acc[h] = __fadd_rn(acc[h], __fmul_rn(qreg[h][4 * c + 0], kv4.x));
                    acc[h] = __fadd_rn(acc[h], __fmul_rn(qreg[h][4 * c + 1], kv4.y));
                    acc[h] = __fadd_rn(acc[h], __fmul_rn(qreg[h][4 * c + 2], kv4.z));
                    acc[h] = __fadd_rn(acc[h], __fmul_rn(qreg[h][4 * c + 3], kv4.w));
                }
            }
            __syncwarp();
            if (lane == 0) s_mbar_arrive(&empty[s]);
            if (warp < 3) {
                *(float4*)(hand + ((warp * RING + s) * 32 + lane) * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
                __syncwarp();
                if (lane == 0) s_mbar_arrive(&ready[warp * RING + s]);
            } else {
                int pos = tile * kTP + lane;
                if (pos < len) {
#pragma unroll
                    for (int h = 0; h < G; h++) {
                        float sc = __fadd_rn(__fmul_rn(acc[h], p.scale), 0.0f);
                        srow[(int64_t)h * p.capacity + pos] = sc;
                        top[h] = fmaxf(top[h], sc);
                    }
                }
            }
        }
    }
    // ---- 2. softmax: maximum, exp in place, the denominator folded in position order ----
    if (warp == 3) {
#pragma unroll
        for (int h = 0; h < G; h++) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) top[h] = fmaxf(top[h], __shfl_xor_sync(0xffffffffu, top[h], off));
            if (lane == 0) maxes[h] = top[h];
        }
    }
    consumers_sync();
    {
        float total = 0.0f;  // lane 0 of warp h folds head h
        for (int e0 = 0; e0 < len; e0 += kSEChunk) {
            int count = min(kSEChunk, len - e0);
            // eight loads in flight per thread: the scores come back from L2
            for (int i0 = 0; i0 < count; i0 += 2 * kConsumers) {
                float sv[2][G];
#pragma unroll
                for (int u = 0; u < 2; u++)
#pragma unroll
                    for (int h = 0; h < G; h++) {
                        int i = i0 + u * kConsumers + tid;
                        sv[u][h] = i < count ? srow[(int64_t)h * p.capacity + e0 + i] : 0.0f;
                    }
#pragma unroll
                for (int u = 0; u < 2; u++)
#pragma unroll
                    for (int h = 0; h < G; h++) {
                        int i = i0 + u * kConsumers + tid;
                        if (i < count) {
                            float e = exact_exp(__fsub_rn(sv[u][h], maxes[h]));
                            srow[(int64_t)h * p.capacity + e0 + i] = e;
                            ebuf[h * kSEChunk + i] = e;
                        }
                    }
            }
            consumers_sync();
            if (lane == 0) {
                const float* eh = ebuf + warp * kSEChunk;
                int i = 0;
                for (; i + 8 <= count; i += 8) {
                    float4 a = *(const float4*)(eh + i), b = *(const float4*)(eh + i + 4);
                    total = __fadd_rn(total, a.x), total = __fadd_rn(total, a.y), total = __fadd_rn(total, a.z), total = __fadd_rn(total, a.w);
                    total = __fadd_rn(total, b.x), total = __fadd_rn(total, b.y), total = __fadd_rn(total, b.z), total = __fadd_rn(total, b.w);
                }
                for (; i < count; i++) total = __fadd_rn(total, eh[i]);
            }
            consumers_sync();
        }
        if (lane == 0) totals[warp] = total;
    }
    consumers_sync();
    // ---- 3. outputs: thread `tid` folds column `tid` of all four heads over positions in order ----
    {
        const float total = totals[shd];
        const float* erow = srow + (int64_t)shd * p.capacity + sp;   // this thread makes the weights of positions sp + 32 j, head shd
        constexpr int kBatch = 4;                  // tiles whose weights are made at once: one barrier per 128 positions
        float e_next[kBatch];
#pragma unroll
        for (int j = 0; j < kBatch; j++) e_next[j] = sp + kTP * j < len ? erow[kTP * j] : 0.0f;
        const int col = tid;
        const unsigned char* colp = stages + (col >> 5) * BOX_BYTES + (col & 3) * 4;
        const int piece = (col & 31) >> 2;  // a value's 16-byte piece of its 128-byte row sits at piece ^ (position & 7)
        int voff[8];
#pragma unroll
        for (int u = 0; u < 8; u++) voff[u] = u * 128 + ((piece ^ u) << 4);
        float acc[G];
#pragma unroll
        for (int i = 0; i < G; i++) acc[i] = 0.0f;
        for (int tile0 = 0; tile0 < tiles; tile0 += kBatch) {
            float* wb = wbuf + ((tile0 / kBatch) & 1) * kBatch * kTP * G;
#pragma unroll
            for (int j = 0; j < kBatch; j++) wb[(kTP * j + sp) * G + shd] = __fdiv_rn(e_next[j], total);
#pragma unroll
            for (int j = 0; j < kBatch; j++) {  // the exp values of the next batch travel from L2 while this one is folded
                int next = (tile0 + kBatch + j) * kTP + sp;
                e_next[j] = next < len ? erow[(tile0 + kBatch + j) * kTP] : 0.0f;
            }
            consumers_sync();  // this batch's weights are written; the other half of wbuf is no longer read
            const int last = min(tiles, tile0 + kBatch);
            for (int tile = tile0; tile < last; tile++) {
                const float* wt = wb + (tile - tile0) * kTP * G;
                int j = tiles + tile, s = j % RING;
                if (!s_mbar_wait(&full[s], (unsigned)((j / RING) & 1), abort_flag)) ok = false, *abort_flag = 1;
                const unsigned char* vt = colp + (size_t)s * STAGE_BYTES;
                int count = min(kTP, len - tile * kTP);
                int pos = 0;
                if (count == kTP) {
                    // a whole tile: the loads of the next 8 positions are in flight while the current 8 are folded (a
                    // warp may be alone on its scheduler, so nothing else would hide a shared-memory load's latency)
                    float vv[2][8];
                    float4 ww[2][8];
#pragma unroll
                    for (int u = 0; u < 8; u++) vv[0][u] = *(const float*)(vt + voff[u]), ww[0][u] = *(const float4*)(wt + u * G);
#pragma unroll
                    for (int group = 0; group < kTP / 8; group++) {
                        const int cur = group & 1;
                        if (group + 1 < kTP / 8) {
#pragma unroll
                            for (int u = 0; u < 8; u++) {
                                vv[cur ^ 1][u] = *(const float*)(vt + (group + 1) * 8 * 128 + voff[u]);
                                ww[cur ^ 1][u] = *(const float4*)(wt + ((group + 1) * 8 + u) * G);
                            }
                        }
#pragma unroll
                        for (int u = 0; u < 8; u++) {
                            acc[0] = __fadd_rn(acc[0], __fmul_rn(ww[cur][u].x, vv[cur][u]));
                            acc[1] = __fadd_rn(acc[1], __fmul_rn(ww[cur][u].y, vv[cur][u]));
                            acc[2] = __fadd_rn(acc[2], __fmul_rn(ww[cur][u].z, vv[cur][u]));
                            acc[3] = __fadd_rn(acc[3], __fmul_rn(ww[cur][u].w, vv[cur][u]));
                        }
                    }
                    pos = kTP;
                }
                for (; pos < count; pos++) {
                    float vv = *(const float*)(vt + pos * 128 + ((piece ^ (pos & 7)) << 4));  // no indexing of voff by a variable: it would move to local memory
                    float4 w4 = *(const float4*)(wt + pos * G);
                    acc[0] = __fadd_rn(acc[0], __fmul_rn(w4.x, vv));
                    acc[1] = __fadd_rn(acc[1], __fmul_rn(w4.y, vv));
                    acc[2] = __fadd_rn(acc[2], __fmul_rn(w4.z, vv));
                    acc[3] = __fadd_rn(acc[3], __fmul_rn(w4.w, vv));
                }
                __syncwarp();
                if (lane == 0) s_mbar_arrive(&empty[s]);
            }
        }
        if (!ok || *abort_flag) {
            if (tid == 0) atomicExch(&p.errors->timeout, 1);
            return;
        }
#pragma unroll
        for (int i = 0; i < G; i++) {  // a warp holds one 32-column block of each head
            int64_t at = ((int64_t)token * p.heads + head0 + i) * WIDTH + col;
            if (p.out) p.out[at] = acc[i];
            if (p.sink.qs) quantize_block_q8(acc[i], lane, p.sink.scales + (at >> 5), p.sink.sums + (at >> 5), p.sink.totals + (at >> 5), p.sink.qs + at);
        }
    }
}


// ---- the same attention as three launches, for calls with fewer (token, kv head) pairs than SMs ------------------
// One CTA per pair walks up to `capacity` positions alone, so a launch that cannot fill the GPU (a tensor-parallel rank
// with one or two kv heads, a handful of long streams) lasts as long as its longest stream takes on one SM.  Here the
// score pass is cut by position ranges and the value pass by quarters of the width, with the softmax in between; every
// sum is made in the same order as in the single launch, so the bits are the same.

// Scores of the positions of tiles [first, last) of one (token, kv head): the quarter pipeline of the kernel above.
template <int WIDTH>
__global__ void __launch_bounds__(kConsumers + 32, 2) attention_scores_kernel(StreamParams p, const __grid_constant__ StreamMaps maps) {
    chained_kernel_entry();
    constexpr int G = 4;
    constexpr int BOXES = WIDTH / 32;
    constexpr int BOX_BYTES = kTP * 128;
    constexpr int STAGE_BYTES = BOXES * BOX_BYTES;
    constexpr int QP = WIDTH + 4;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (s_smem_u32(smem_raw) & 1023u)) & 1023u);  // an offset from the shared array: the address space stays known
    uint64_t* full = (uint64_t*)smem;
    uint64_t* empty = (uint64_t*)(smem + 64);
    uint64_t* ready = (uint64_t*)(smem + 128);
    volatile int* abort_flag = (volatile int*)(smem + 320);
    float* hand = (float*)(smem + 512);
    unsigned char* stages = smem + 8192;
    float* qs = (float*)(stages + kRing * STAGE_BYTES);    // [G][QP]

    const int token = p.order ? p.order[blockIdx.y] : blockIdx.y;
    const int per_kv = p.heads / p.kv_heads, groups_per_kv = per_kv / G;
    const int kvh = blockIdx.x / groups_per_kv;
    const int head0 = kvh * per_kv + (blockIdx.x % groups_per_kv) * G;
    const int row = p.table[3 * token], limit = p.table[3 * token + 1];
    if (row < 0 || row >= p.rows || limit < 0 || limit >= p.capacity) {
        if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.z == 0) report_bad_index(p.errors, limit, p.capacity);
        return;
    }
    const int len = limit + 1;
    const int all_tiles = (len + kTP - 1) / kTP;
    const int first = (int)((int64_t)blockIdx.z * all_tiles / p.splits), last = (int)((int64_t)(blockIdx.z + 1) * all_tiles / p.splits);
    const int tiles = last - first;
    if (tiles <= 0) return;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    if (tid == 0) {
        for (int s = 0; s < kRing; s++) {
            s_mbar_init(&full[s], 1);
            s_mbar_init(&empty[s], kConsumers / 32);
            for (int w2 = 0; w2 < 3; w2++) s_mbar_init(&ready[w2 * kRing + s], 1);
        }
        abort_flag[0] = 0, abort_flag[1] = 0, abort_flag[2] = (int)p.wait_hint, abort_flag[3] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    {
        // the four heads' queries: every thread's loads issued before its first store (one per pass, each waited for, cost a
        // trip to L2 per pass)
        const float* qsrc = p.q + (int64_t)token * p.q_stride + (int64_t)head0 * WIDTH;
        constexpr int kPasses = (G * WIDTH + kConsumers + 31) / (kConsumers + 32);
        float qv[kPasses];
#pragma unroll
        for (int u = 0; u < kPasses; u++) {
            const int i = tid + u * (kConsumers + 32);
            qv[u] = i < G * WIDTH ? qsrc[i] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < kPasses; u++) {
            const int i = tid + u * (kConsumers + 32);
            if (i < G * WIDTH) qs[(i / WIDTH) * QP + i % WIDTH] = qv[u];
        }
    }
    __syncthreads();

    if (warp == kConsumers / 32) {
        if (lane != 0) return;
        const int plane = (row * p.kv_heads + kvh) * p.capacity;
        int issued = 0;
        bool ok = true;
        for (int j = 0; j < tiles; j++) {
            int s = j % kRing;
            if (j >= kRing) ok = s_mbar_wait(&empty[s], (unsigned)((j / kRing - 1) & 1), abort_flag);
            if (!ok) break;
            unsigned char* dst = stages + (size_t)s * STAGE_BYTES;
            s_mbar_expect_tx(&full[s], STAGE_BYTES);
#pragma unroll
            for (int b = 0; b < BOXES; b++) s_tensor_load(dst + b * BOX_BYTES, &maps.k, 32 * b, plane + (first + j) * kTP, &full[s]);
            issued = j + 1;
        }
        if (!ok) {
            *abort_flag = 1;
            atomicExch(&p.errors->timeout, 1);
            for (int j = max(0, issued - kRing); j < issued; j++) s_mbar_wait(&full[j % kRing], (unsigned)((j / kRing) & 1), abort_flag + 1);
        }
        return;
    }

    float* srow = p.scratch + ((int64_t)token * p.heads + head0) * p.capacity;
    float qreg[G][32];
#pragma unroll
    for (int h = 0; h < G; h++)
#pragma unroll
        for (int j = 0; j < 32; j++) qreg[h][j] = qs[h * QP + 32 * warp + j];
    const int sw = lane & 7;
    bool ok = true;
    for (int tile = 0; tile < tiles; tile++) {
        const int s = tile % kRing;
        const unsigned parity = (unsigned)((tile / kRing) & 1);
        if (!s_mbar_wait(&full[s], parity, abort_flag)) ok = false, *abort_flag = 1;
        float acc[G] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (warp > 0) {
            if (!s_mbar_wait(&ready[(warp - 1) * kRing + s], parity, abort_flag)) ok = false, *abort_flag = 1;
            float4 in = *(const float4*)(hand + (((warp - 1) * kRing + s) * 32 + lane) * 4);
            acc[0] = in.x, acc[1] = in.y, acc[2] = in.z, acc[3] = in.w;
        }
        const unsigned char* rowp = stages + (size_t)s * STAGE_BYTES + warp * BOX_BYTES + lane * 128;
#pragma unroll
        for (int c = 0; c < 8; c++) {
            float4 kv4 = *(const float4*)(rowp + ((c ^ sw) << 4));
#pragma unroll
            for (int h = 0; h < G; h++) {
                acc[h] = __fadd_rn(acc[h], __fmul_rn(qreg[h][4 * c + 0], kv4.x));
                acc[h] = __fadd_rn(acc[h], __fmul_rn(qreg[h][4 * c + 1], kv4.y));
                acc[h] = __fadd_rn(acc[h], __fmul_rn(qreg[h][4 * c + 2], kv4.z));
                acc[h] = __fadd_rn(acc[h], __fmul_rn(qreg[h][4 * c + 3], kv4.w));
            }
        }
        __syncwarp();
        if (lane == 0) s_mbar_arrive(&empty[s]);
        if (warp < 3) {
            *(float4*)(hand + ((warp * kRing + s) * 32 + lane) * 4) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            __syncwarp();
            if (lane == 0) s_mbar_arrive(&ready[warp * kRing + s]);
        } else {
            int pos = (first + tile) * kTP + lane;
            if (pos < len) {
#pragma unroll
                for (int h = 0; h < G; h++) srow[(int64_t)h * p.capacity + pos] = __fadd_rn(__fmul_rn(acc[h], p.scale), 0.0f);
            }
        }
    }
    if (!ok && lane == 0) atomicExch(&p.errors->timeout, 1);
}

// One (token, head): maximum, exp, the denominator folded in position order, weights = exp / denominator in place.
// A stream of up to kWeightKeep * 256 positions stays in registers from its one read to its one write (as three passes
// over the scratch array, each thread waiting for one load per pass and step, the kernel took 18 us); the exp values are
// staged in shared memory and summed chunk by chunk (chunked_sum_of_terms: the sequential sum's bits).  Longer streams go
// segment by segment through the scratch array, every segment's loads issued before their first use.
constexpr int kWeightSegment = kSumChunk * kSumMaxChunks;   // positions staged at once
constexpr int kWeightKeep = 20;

__device__ __forceinline__ float weights_sum(float* ebuf, int count, int padded, float start, float* sum_out, SumScratch* ss, int chunked) {
    // ebuf[0, padded) holds `count` exp values and +0 behind them; all threads call
    if (chunked && padded >= 8 * kSumChunk) return chunked_sum_of_terms(ebuf, padded, start, sum_out, ss);
    if (threadIdx.x == 0) {
        float acc = start;
        int i = 0;
        for (; i + 8 <= count; i += 8) {
            float4 a = *(const float4*)(ebuf + i), b = *(const float4*)(ebuf + i + 4);
            acc = __fadd_rn(acc, a.x), acc = __fadd_rn(acc, a.y), acc = __fadd_rn(acc, a.z), acc = __fadd_rn(acc, a.w);
            acc = __fadd_rn(acc, b.x), acc = __fadd_rn(acc, b.y), acc = __fadd_rn(acc, b.z), acc = __fadd_rn(acc, b.w);
        }
        for (; i < count; i++) acc = __fadd_rn(acc, ebuf[i]);
        sum_out[0] = acc;
    }
    __syncthreads();
    return sum_out[0];
}

__global__ void __launch_bounds__(256) attention_weights_kernel(StreamParams p, int chunked) {
    chained_kernel_entry();
    extern __shared__ __align__(16) float ebuf[];   // min(kWeightSegment, the capacity rounded up to whole chunks)
    __shared__ float red[8];
    __shared__ float sum_out[1];
    __shared__ SumScratch sum_scratch;
    const int token = p.order ? p.order[blockIdx.y] : blockIdx.y, head = blockIdx.x;
    const int row = p.table[3 * token], limit = p.table[3 * token + 1];
    if (row < 0 || row >= p.rows || limit < 0 || limit >= p.capacity) return;  // reported by the score kernel
    const int len = limit + 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float* sr = p.scratch + ((int64_t)token * p.heads + head) * p.capacity;
    auto block_max = [&](float top) {
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, off));
        if (lane == 0) red[warp] = top;
        __syncthreads();
        top = red[0];
#pragma unroll
        for (int w2 = 1; w2 < 8; w2++) top = fmaxf(top, red[w2]);
        return top;
    };
    if (len <= kWeightKeep * 256) {
        float sv[kWeightKeep];
#pragma unroll
        for (int u = 0; u < kWeightKeep; u++) sv[u] = u * 256 + tid < len ? sr[u * 256 + tid] : -INFINITY;
        float top = sv[0];
#pragma unroll
        for (int u = 1; u < kWeightKeep; u++) top = fmaxf(top, sv[u]);
        top = block_max(top);
        const int padded = (len + kSumChunk - 1) / kSumChunk * kSumChunk;   // +0 behind the last value: it changes no sum
#pragma unroll
        for (int u = 0; u < kWeightKeep; u++) {
            const int i = u * 256 + tid;
            sv[u] = i < len ? exact_exp(__fsub_rn(sv[u], top)) : 0.0f;
            if (i < padded) ebuf[i] = sv[u];
        }
        __syncthreads();
        const float total = weights_sum(ebuf, len, padded, 0.0f, sum_out, &sum_scratch, chunked);
#pragma unroll
        for (int u = 0; u < kWeightKeep; u++)
            if (u * 256 + tid < len) sr[u * 256 + tid] = __fdiv_rn(sv[u], total);
        return;
    }
    // long streams: eight loads in flight per thread in every pass
    float top = -INFINITY;
    for (int i0 = 0; i0 < len; i0 += 8 * 256) {
        float sv[8];
#pragma unroll
        for (int u = 0; u < 8; u++) sv[u] = i0 + u * 256 + tid < len ? sr[i0 + u * 256 + tid] : -INFINITY;
#pragma unroll
        for (int u = 0; u < 8; u++) top = fmaxf(top, sv[u]);
    }
    top = block_max(top);
    float total = 0.0f;
    for (int e0 = 0; e0 < len; e0 += kWeightSegment) {
        const int count = min(kWeightSegment, len - e0);
        const int padded = (count + kSumChunk - 1) / kSumChunk * kSumChunk;
        for (int i0 = 0; i0 < padded; i0 += 8 * 256) {
            float sv[8];
#pragma unroll
            for (int u = 0; u < 8; u++) sv[u] = i0 + u * 256 + tid < count ? sr[e0 + i0 + u * 256 + tid] : 0.0f;
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int i = i0 + u * 256 + tid;
                float e = 0.0f;
                if (i < count) {
                    e = exact_exp(__fsub_rn(sv[u], top));
                    sr[e0 + i] = e;
                }
                if (i < padded) ebuf[i] = e;
            }
        }
        __syncthreads();
        total = weights_sum(ebuf, count, padded, total, sum_out, &sum_scratch, chunked);
        __syncthreads();   // the next segment overwrites ebuf
    }
    for (int i0 = 0; i0 < len; i0 += 8 * 256) {
        float sv[8];
#pragma unroll
        for (int u = 0; u < 8; u++) sv[u] = i0 + u * 256 + tid < len ? sr[i0 + u * 256 + tid] : 0.0f;
#pragma unroll
        for (int u = 0; u < 8; u++)
            if (i0 + u * 256 + tid < len) sr[i0 + u * 256 + tid] = __fdiv_rn(sv[u], total);
    }
}

// Outputs of one quarter of the width (32 columns) of one (token, kv head): one consumer warp folds weight * value over all
// positions in order, its box of every value tile arriving through a ring; the weights come from the scratch array.
template <int WIDTH>
__global__ void __launch_bounds__(64) attention_values_kernel(StreamParams p, const __grid_constant__ StreamMaps maps) {
    chained_kernel_entry();
    constexpr int G = 4;
    constexpr int BOX_BYTES = kTP * 128;
    constexpr int kDeep = 6;                       // stages of 4 KB
    __shared__ __align__(1024) unsigned char stages[kDeep * BOX_BYTES];
    __shared__ __align__(16) float wbuf[2][kTP * G];
    __shared__ uint64_t full[kDeep], empty[kDeep];
    __shared__ int abort_words[4];
    volatile int* abort_flag = abort_words;

    const int token = blockIdx.y;
    const int per_kv = p.heads / p.kv_heads, groups_per_kv = per_kv / G;
    const int quarter = blockIdx.x & 3, group = blockIdx.x >> 2;
    const int kvh = group / groups_per_kv;
    const int head0 = kvh * per_kv + (group % groups_per_kv) * G;
    const int row = p.table[3 * token], limit = p.table[3 * token + 1];
    if (row < 0 || row >= p.rows || limit < 0 || limit >= p.capacity) return;
    const int len = limit + 1;
    const int tiles = (len + kTP - 1) / kTP;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        for (int s = 0; s < kDeep; s++) s_mbar_init(&full[s], 1), s_mbar_init(&empty[s], 1);
        abort_words[0] = 0, abort_words[1] = 0, abort_words[2] = (int)p.wait_hint, abort_words[3] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == 1) {
        if (lane != 0) return;
        const int plane = (row * p.kv_heads + kvh) * p.capacity;
        int issued = 0;
        bool ok = true;
        for (int j = 0; j < tiles; j++) {
            int s = j % kDeep;
            if (j >= kDeep) ok = s_mbar_wait(&empty[s], (unsigned)((j / kDeep - 1) & 1), abort_flag);
            if (!ok) break;
            s_mbar_expect_tx(&full[s], BOX_BYTES);
            s_tensor_load(stages + s * BOX_BYTES, &maps.v, 32 * quarter, plane + j * kTP, &full[s]);
            issued = j + 1;
        }
        if (!ok) {
            *abort_flag = 1;
            atomicExch(&p.errors->timeout, 1);
            for (int j = max(0, issued - kDeep); j < issued; j++) s_mbar_wait(&full[j % kDeep], (unsigned)((j / kDeep) & 1), abort_flag + 1);
        }
        return;
    }
    // consumer warp: lane = column 32 quarter + lane
    const float* wrow = p.scratch + ((int64_t)token * p.heads + head0) * p.capacity;   // weights [h][position]
    const int piece = lane >> 2;
    int voff[8];
#pragma unroll
    for (int u = 0; u < 8; u++) voff[u] = u * 128 + ((piece ^ u) << 4) + (lane & 3) * 4;
    float acc[G] = {0.0f, 0.0f, 0.0f, 0.0f};
    float w_next[G];   // lane's position of the next tile, four heads
#pragma unroll
    for (int h = 0; h < G; h++) w_next[h] = lane < len ? wrow[(int64_t)h * p.capacity + lane] : 0.0f;
    bool ok = true;
    for (int tile = 0; tile < tiles; tile++) {
        float* wt = wbuf[tile & 1];
        *(float4*)(wt + lane * G) = make_float4(w_next[0], w_next[1], w_next[2], w_next[3]);
        int next = (tile + 1) * kTP + lane;
#pragma unroll
        for (int h = 0; h < G; h++) w_next[h] = next < len ? wrow[(int64_t)h * p.capacity + next] : 0.0f;
        __syncwarp();
        int s = tile % kDeep;
        if (!s_mbar_wait(&full[s], (unsigned)((tile / kDeep) & 1), abort_flag)) ok = false, *abort_flag = 1;
        const unsigned char* vt = stages + s * BOX_BYTES;
        int count = min(kTP, len - tile * kTP);
        int pos = 0;
        for (; pos + 8 <= count; pos += 8) {
            float vv[8];
            float4 ww[8];
#pragma unroll
            for (int u = 0; u < 8; u++) vv[u] = *(const float*)(vt + pos * 128 + voff[u]), ww[u] = *(const float4*)(wt + (pos + u) * G);
#pragma unroll
            for (int u = 0; u < 8; u++) {
                acc[0] = __fadd_rn(acc[0], __fmul_rn(ww[u].x, vv[u]));
                acc[1] = __fadd_rn(acc[1], __fmul_rn(ww[u].y, vv[u]));
                acc[2] = __fadd_rn(acc[2], __fmul_rn(ww[u].z, vv[u]));
                acc[3] = __fadd_rn(acc[3], __fmul_rn(ww[u].w, vv[u]));
            }
        }
        for (; pos < count; pos++) {
            float vv = *(const float*)(vt + pos * 128 + ((piece ^ (pos & 7)) << 4) + (lane & 3) * 4);
            float4 w4 = *(const float4*)(wt + pos * G);
            acc[0] = __fadd_rn(acc[0], __fmul_rn(w4.x, vv));
            acc[1] = __fadd_rn(acc[1], __fmul_rn(w4.y, vv));
            acc[2] = __fadd_rn(acc[2], __fmul_rn(w4.z, vv));
            acc[3] = __fadd_rn(acc[3], __fmul_rn(w4.w, vv));
        }
        __syncwarp();
        if (lane == 0) s_mbar_arrive(&empty[s]);
    }
    if (!ok) {
        if (lane == 0) atomicExch(&p.errors->timeout, 1);
        return;
    }
#pragma unroll
    for (int i = 0; i < G; i++) {
        int64_t at = ((int64_t)token * p.heads + head0 + i) * WIDTH + 32 * quarter + lane;
        if (p.out) p.out[at] = acc[i];
        if (p.sink.qs) quantize_block_q8(acc[i], lane, p.sink.scales + (at >> 5), p.sink.sums + (at >> 5), p.sink.totals + (at >> 5), p.sink.qs + at);
    }
}

// The value pass for launches with few (token, kv head) pairs, cut as finely as the ordered sums allow: every output column
// of every head is its own chain over the positions, so a warp takes 8 columns x 4 heads (lane = head * 8 + column) and four
// such warps share one 32-column box of every value tile.  A lane then carries ONE chain (two instructions per position
// beside its two shared-memory loads), and a stream of 4096 positions is done in about as many times the add latency,
// where the kernel above, with four chains per lane and one warp per box, takes four times as long on a quarter of the warps.
template <int WIDTH, int DEEP>
__global__ void __launch_bounds__(160) attention_values_wide_kernel(StreamParams p, const __grid_constant__ StreamMaps maps) {
    chained_kernel_entry();
    constexpr int G = 4;
    constexpr int BOX_BYTES = kTP * 128;
    // The ring's depth bounds how fast one CTA's stream arrives (a copy takes about a microsecond to land): 6 stages when
    // the launch has CTAs enough to fill every SM several times over, 16 when it has few and long streams.
    constexpr int kDeep = DEEP;
    constexpr int kWarps = 4;
    extern __shared__ unsigned char wide_raw[];
    unsigned char* stages = wide_raw + ((1024u - (s_smem_u32(wide_raw) & 1023u)) & 1023u);   // [kDeep][BOX_BYTES], swizzled boxes
    float* wbuf_all = (float*)(stages + kDeep * BOX_BYTES);   // [kWarps][2 chunks][256 positions][G]: each warp's weights
    __shared__ uint64_t full[kDeep], empty[kDeep];
    __shared__ int abort_words[4];
    volatile int* abort_flag = abort_words;

    const int token = p.order ? p.order[blockIdx.y] : blockIdx.y;
    const int per_kv = p.heads / p.kv_heads, groups_per_kv = per_kv / G;
    const int quarter = blockIdx.x & 3, group = blockIdx.x >> 2;
    const int kvh = group / groups_per_kv;
    const int head0 = kvh * per_kv + (group % groups_per_kv) * G;
    const int row = p.table[3 * token], limit = p.table[3 * token + 1];
    if (row < 0 || row >= p.rows || limit < 0 || limit >= p.capacity) return;   // reported by the score kernel
    const int len = limit + 1;
    const int tiles = (len + kTP - 1) / kTP;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    if (tid == 0) {
        for (int s = 0; s < kDeep; s++) s_mbar_init(&full[s], 1), s_mbar_init(&empty[s], kWarps);
        abort_words[0] = 0, abort_words[1] = 0, abort_words[2] = (int)p.wait_hint, abort_words[3] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (warp == kWarps) {
        if (lane != 0) return;
        const int plane = (row * p.kv_heads + kvh) * p.capacity;
        int issued = 0;
        bool ok = true;
        for (int j = 0; j < tiles; j++) {
            int s = j % kDeep;
            if (j >= kDeep) ok = s_mbar_wait(&empty[s], (unsigned)((j / kDeep - 1) & 1), abort_flag);
            if (!ok) break;
            s_mbar_expect_tx(&full[s], BOX_BYTES);
            s_tensor_load(stages + s * BOX_BYTES, &maps.v, 32 * quarter, plane + j * kTP, &full[s]);
            issued = j + 1;
        }
        if (!ok) {
            *abort_flag = 1;
            atomicExch(&p.errors->timeout, 1);
            for (int j = max(0, issued - kDeep); j < issued; j++) s_mbar_wait(&full[j % kDeep], (unsigned)((j / kDeep) & 1), abort_flag + 1);
        }
        return;
    }
    // consumer warp `warp`: columns 32 quarter + 8 warp + (lane & 7), head head0 + (lane >> 3)
    const int h = lane >> 3, c8 = 8 * warp + (lane & 7);
    const float* wrow = p.scratch + ((int64_t)token * p.heads + head0) * p.capacity;   // weights [head][position]
    const int piece = c8 >> 2, within = (c8 & 3) * 4;
    float acc = 0.0f;
    // The weights of kWChunk positions at a time, fetched a whole chunk ahead: they come from L2, whose latency is several
    // times what a warp needs to fold a tile, so a fetch one tile ahead left every tile waiting for its weights.
    // Each warp keeps its own copy ([2 chunks][position][head]), so the warps need no barrier among themselves.
    constexpr int kWChunk = 256;
    constexpr int kPerLane = kWChunk / 32;
    float4* wchunk = (float4*)wbuf_all + (size_t)warp * 2 * kWChunk;
    auto fetch = [&](int chunk, float (&w4)[kPerLane][G]) {
#pragma unroll
        for (int u = 0; u < kPerLane; u++) {
            int pos = chunk * kWChunk + u * 32 + lane;
#pragma unroll
            for (int i = 0; i < G; i++) w4[u][i] = pos < len ? wrow[(int64_t)i * p.capacity + pos] : 0.0f;
        }
    };
    auto stash = [&](int chunk, const float (&w4)[kPerLane][G]) {
        float4* dst = wchunk + (size_t)(chunk & 1) * kWChunk;
#pragma unroll
        for (int u = 0; u < kPerLane; u++) dst[u * 32 + lane] = make_float4(w4[u][0], w4[u][1], w4[u][2], w4[u][3]);
    };
    float w_next[kPerLane][G];
    fetch(0, w_next);
    stash(0, w_next);
    const int chunks = (len + kWChunk - 1) / kWChunk;
    if (chunks > 1) fetch(1, w_next);
    __syncwarp();
    bool ok = true;
    for (int tile = 0; tile < tiles; tile++) {
        const int chunk = tile / (kWChunk / kTP);
        if (tile % (kWChunk / kTP) == 0 && tile > 0) {
            // entering chunk `chunk`: its weights were fetched while the chunk before it was folded; store them and start
            // fetching the chunk after it
            stash(chunk, w_next);
            if (chunk + 1 < chunks) fetch(chunk + 1, w_next);
            __syncwarp();
        }
        const float* wt = (const float*)(wchunk + (size_t)(chunk & 1) * kWChunk + (tile % (kWChunk / kTP)) * kTP);
        int s = tile % kDeep;
        if (!s_mbar_wait(&full[s], (unsigned)((tile / kDeep) & 1), abort_flag)) ok = false, *abort_flag = 1;
        const unsigned char* vt = stages + s * BOX_BYTES + within;
        const float* wh = wt + h;
        int count = min(kTP, len - tile * kTP);
        if (count == kTP) {
            float vv[kTP], ww[kTP];   // every load of the tile is issued before the chain starts
#pragma unroll
            for (int u = 0; u < kTP; u++) vv[u] = *(const float*)(vt + u * 128 + ((piece ^ (u & 7)) << 4)), ww[u] = wh[u * G];
#pragma unroll
            for (int u = 0; u < kTP; u++) acc = __fadd_rn(acc, __fmul_rn(ww[u], vv[u]));
        } else {
            for (int pos = 0; pos < count; pos++) {
                float vv = *(const float*)(vt + pos * 128 + ((piece ^ (pos & 7)) << 4));
                acc = __fadd_rn(acc, __fmul_rn(wh[pos * G], vv));
            }
        }
        __syncwarp();
        if (lane == 0) s_mbar_arrive(&empty[s]);
    }
    if (!ok && lane == 0) atomicExch(&p.errors->timeout, 1);
    // a block of 32 columns lies across the CTA's four warps: the rows go out through shared memory so that the quantiser's
    // warp-per-block arithmetic (quantize_block_q8) sees a block's 32 columns in one warp's lanes
    __shared__ float rows_out[G][32];
    rows_out[h][c8] = acc;
    asm volatile("bar.sync 2, 128;" ::: "memory");   // the four consumer warps only; reached by all of them, gave up or not
    if (*abort_flag) return;
    const float mine = rows_out[warp][lane];          // warp = head, lane = column of the quarter
    int64_t at = ((int64_t)token * p.heads + head0 + warp) * WIDTH + 32 * quarter + lane;
    if (p.out) p.out[at] = mine;
    if (p.sink.qs) quantize_block_q8(mine, lane, p.sink.scales + (at >> 5), p.sink.sums + (at >> 5), p.sink.totals + (at >> 5), p.sink.qs + at);
}

// ---- prefill: many consecutive tokens of one stream --------------------------------------------------------------
// A prompt's tokens attend over the same keys and values, each up to its own position.  The kernels above take one query
// token per CTA, so a prompt of n tokens reads its keys and values n times.  Here a CTA takes a tile of 16 consecutive tokens
// of one stream (x 4 query heads of one key/value head = 64 query rows) and streams the keys, then the values, ONCE for all
// of them, through the same ring of tiled tensor copies.  Every sum keeps the host's order, so a token's bits are those of
// the decode kernels (prefill == decode, spec/block_matmul_spec.cr:253-260):
//   scores   register tiles of 4 query rows x 4 positions per thread over a tile of 32 positions, the 128 products of a score
//            added in column order; the two halves of the CTA take alternate key tiles.  Scores go to the scratch array
//            (which stays in L2), masked by each row's own last position;
//   softmax  maximum per row, exp in place by all threads, then one thread per row folds its denominator in position order;
//   values   register tiles of 4 query rows x 8 columns per thread; a position's weights (exp / denominator) are made once per
//            tile into shared memory.  Positions a row must not see have weight +0, and +-0 never changes a running sum
//            that started at +0, so they cost nothing but the issue slots.
constexpr int kQT = 16;                // query tokens per CTA
constexpr int kQRows = kQT * 4;        // query rows: token-major, head-minor
constexpr int kPrefillConsumers = 256;

struct PrefillParams {
    StreamParams s;
    const int* qtiles;   // [tiles][2]: first token of the tile (in packed order), tokens in it (<= kQT)
};

template <int WIDTH>
__global__ void __launch_bounds__(kPrefillConsumers + 32, 2) attention_prefill_kernel(PrefillParams pp, const __grid_constant__ StreamMaps maps) {
    chained_kernel_entry();
    const StreamParams& p = pp.s;
    constexpr int G = 4;
    constexpr int BOXES = WIDTH / 32;
    constexpr int BOX_BYTES = kTP * 128;
    constexpr int STAGE_BYTES = BOXES * BOX_BYTES;
    constexpr int QP = WIDTH + 4;                  // pitch of a query row, and of an output row staged for the quantiser
    static_assert(WIDTH == 128, "the thread tiles below are laid out for 128 columns");
    extern __shared__ unsigned char prefill_raw[];
    unsigned char* smem = prefill_raw + ((1024u - (s_smem_u32(prefill_raw) & 1023u)) & 1023u);
    uint64_t* full = (uint64_t*)smem;              // [kRing]
    uint64_t* empty = (uint64_t*)(smem + 64);      // [kRing]
    volatile int* abort_flag = (volatile int*)(smem + 128);
    int* limits = (int*)(smem + 256);              // [kQRows] last visible position of each query row, -1: no such row
    float* tops = (float*)(smem + 512);            // [kQRows]
    float* tots = (float*)(smem + 768);            // [kQRows]
    unsigned char* stages = smem + 1024;           // [kRing][BOXES][kTP][128 bytes], swizzled
    float* qs = (float*)(stages + kRing * STAGE_BYTES);     // [kQRows][QP]; later the outputs
    float* wbuf = qs + kQRows * QP;                // [kQRows][kTP + 1] weights of one value tile; first the partial maxima

    const int tile_first = pp.qtiles[2 * blockIdx.y], tile_count = pp.qtiles[2 * blockIdx.y + 1];
    const int per_kv = p.heads / p.kv_heads, groups_per_kv = per_kv / G;
    const int kvh = blockIdx.x / groups_per_kv;
    const int head0 = kvh * per_kv + (blockIdx.x % groups_per_kv) * G;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int row = p.table[3 * tile_first];
    const int last_limit = p.table[3 * (tile_first + tile_count - 1) + 1];
    if (row < 0 || row >= p.rows || last_limit < 0 || last_limit >= p.capacity || tile_count < 1 || tile_count > kQT) {
        if (tid == 0 && blockIdx.x == 0) report_bad_index(p.errors, last_limit, p.capacity);
        return;
    }
    const int len = last_limit + 1;                // positions the tile's last token sees
    const int tiles = (len + kTP - 1) / kTP;

    if (tid == 0) {
        for (int s = 0; s < kRing; s++) {
            s_mbar_init(&full[s], 1);
            s_mbar_init(&empty[s], kPrefillConsumers / 32);
        }
        abort_flag[0] = 0, abort_flag[1] = 0, abort_flag[2] = (int)p.wait_hint, abort_flag[3] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i0 = tid; i0 < kQRows * WIDTH; i0 += 8 * blockDim.x) {   // eight loads per thread in flight, then their stores
        float qv[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int i = i0 + u * blockDim.x;
            const int r = i / WIDTH, d = i % WIDTH, t = r >> 2, h = r & 3;
            qv[u] = i < kQRows * WIDTH && t < tile_count ? p.q[(int64_t)(tile_first + t) * p.q_stride + (int64_t)(head0 + h) * WIDTH + d] : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int i = i0 + u * blockDim.x;
            if (i < kQRows * WIDTH) qs[(i / WIDTH) * QP + i % WIDTH] = qv[u];
        }
    }
    for (int r = tid; r < kQRows; r += blockDim.x) {
        int t = r >> 2;
        // a token of another stream, or out of order, would break the tile: such a row is left out
        bool mine = t < tile_count && p.table[3 * (tile_first + t)] == row;
        int limit = mine ? p.table[3 * (tile_first + t) + 1] : -1;
        limits[r] = limit >= 0 && limit <= last_limit ? limit : -1;
    }
    __syncthreads();

    if (warp == kPrefillConsumers / 32) {
        // ------------------------------------------------------------ producer: keys, then values, one ring
        if (lane != 0) return;
        const int plane = (row * p.kv_heads + kvh) * p.capacity;
        int issued = 0;
        bool ok = true;
        for (int j = 0; j < 2 * tiles; j++) {
            int s = j % kRing;
            if (j >= kRing) ok = s_mbar_wait(&empty[s], (unsigned)((j / kRing - 1) & 1), abort_flag);
            if (!ok) break;
            const CUtensorMap* map = j < tiles ? &maps.k : &maps.v;
            int y = plane + (j < tiles ? j : j - tiles) * kTP;
            unsigned char* dst = stages + (size_t)s * STAGE_BYTES;
            s_mbar_expect_tx(&full[s], STAGE_BYTES);
#pragma unroll
            for (int b = 0; b < BOXES; b++) s_tensor_load(dst + b * BOX_BYTES, map, 32 * b, y, &full[s]);
            issued = j + 1;
        }
        if (!ok) {
            *abort_flag = 1;
            atomicExch(&p.errors->timeout, 1);
            for (int j = max(0, issued - kRing); j < issued; j++) s_mbar_wait(&full[j % kRing], (unsigned)((j / kRing) & 1), abort_flag + 1);
        }
        return;
    }

    // ---------------------------------------------------------------- consumers (256 threads; every named barrier below is
    // reached by all of them, whether a wait gave up or not)
    auto consumers_barrier = [] { asm volatile("bar.sync 3, %0;" ::"n"(kPrefillConsumers) : "memory"); };
    bool ok = true;
    float* srow0 = p.scratch + ((int64_t)tile_first * p.heads + head0) * p.capacity;   // row r = 4 t + h: + (t * heads + h) * capacity
    auto score_row = [&](int r) { return srow0 + ((int64_t)(r >> 2) * p.heads + (r & 3)) * p.capacity; };

    // ---- 1. scores ----
    {
        const int half = warp >> 2;                // which key tiles this half of the CTA takes
        const int u = tid & 127, rg = u >> 3, pg = u & 7;   // rows 4 rg .. 4 rg + 3, positions pg + 8 j of the tile
        float top[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        int lim[4];
#pragma unroll
        for (int i = 0; i < 4; i++) lim[i] = limits[4 * rg + i];
        for (int tile = 0; tile < tiles; tile++) {
            const int s = tile % kRing;
            if (!s_mbar_wait(&full[s], (unsigned)((tile / kRing) & 1), abort_flag)) ok = false, *abort_flag = 1;
            if ((tile & 1) == half) {
                float acc[4][4];
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
                const unsigned char* st = stages + (size_t)s * STAGE_BYTES;
#pragma unroll 4
                for (int c = 0; c < WIDTH / 4; c++) {   // four columns at a time, in column order
                    float4 kq[4], qq[4];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const int pos = pg + 8 * j;   // pos & 7 == pg: the eight lanes of a load's phase hit eight different banks
                        kq[j] = *(const float4*)(st + (c >> 3) * BOX_BYTES + pos * 128 + (((c & 7) ^ pg) << 4));
                    }
#pragma unroll
                    for (int i = 0; i < 4; i++) qq[i] = *(const float4*)(qs + (4 * rg + i) * QP + 4 * c);
#pragma unroll
                    for (int i = 0; i < 4; i++)
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(qq[i].x, kq[j].x));
                            acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(qq[i].y, kq[j].y));
                            acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(qq[i].z, kq[j].z));
                            acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(qq[i].w, kq[j].w));
                        }
                }
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    float* sr = score_row(4 * rg + i);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const int pos = tile * kTP + pg + 8 * j;
                        if (pos <= lim[i]) {
                            float sc = __fadd_rn(__fmul_rn(acc[i][j], p.scale), 0.0f);
                            sr[pos] = sc;
                            top[i] = fmaxf(top[i], sc);
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) s_mbar_arrive(&empty[s]);
        }
        // a row's maximum: 16 threads hold a part of it (8 position groups x 2 halves)
#pragma unroll
        for (int i = 0; i < 4; i++) wbuf[(4 * rg + i) * 16 + half * 8 + pg] = top[i];
    }
    consumers_barrier();
    if (tid < kQRows) {
        float top = wbuf[tid * 16];
#pragma unroll
        for (int i = 1; i < 16; i++) top = fmaxf(top, wbuf[tid * 16 + i]);
        tops[tid] = top;
    }
    consumers_barrier();
    // ---- 2. softmax: exp in place by everyone, then one thread per row folds the denominator in position order ----
    for (int r = warp; r < kQRows; r += kPrefillConsumers / 32) {
        const int limit = limits[r];
        float* sr = score_row(r);
        const float top = tops[r];
        // eight loads per lane in flight: one per pass, each waited for before its exp, cost a trip to L2 per 32 positions
        for (int p0 = lane; p0 <= limit; p0 += 8 * 32) {
            float sv[8];
#pragma unroll
            for (int u = 0; u < 8; u++) sv[u] = p0 + 32 * u <= limit ? sr[p0 + 32 * u] : 0.0f;
#pragma unroll
            for (int u = 0; u < 8; u++)
                if (p0 + 32 * u <= limit) sr[p0 + 32 * u] = exact_exp(__fsub_rn(sv[u], top));
        }
    }
    consumers_barrier();
    if (tid < kQRows) {
        const int limit = limits[tid];
        const float* sr = score_row(tid);
        float total = 0.0f;
        int pos = 0;
        // a row starts on a 16-byte boundary when the capacity is a multiple of 4; otherwise plain loads
        if ((((uintptr_t)sr) & 15) == 0) {
            // the exp values come back from L2: 32 positions are on their way while the 32 before them are added
            constexpr int kAhead = 8;   // 16-byte pieces per step
            const int whole = (limit + 1) / (4 * kAhead);
            float4 cur[kAhead], nxt[kAhead];
            if (whole > 0) {
#pragma unroll
                for (int u = 0; u < kAhead; u++) cur[u] = *(const float4*)(sr + 4 * u);
            }
            for (int g = 0; g < whole; g++) {
                if (g + 1 < whole) {
#pragma unroll
                    for (int u = 0; u < kAhead; u++) nxt[u] = *(const float4*)(sr + (g + 1) * 4 * kAhead + 4 * u);
                }
#pragma unroll
                for (int u = 0; u < kAhead; u++) {
                    total = __fadd_rn(total, cur[u].x), total = __fadd_rn(total, cur[u].y);
                    total = __fadd_rn(total, cur[u].z), total = __fadd_rn(total, cur[u].w);
                }
                if (g + 1 < whole) {
#pragma unroll
                    for (int u = 0; u < kAhead; u++) cur[u] = nxt[u];
                }
            }
            pos = whole * 4 * kAhead;
        }
        for (; pos <= limit; pos++) total = __fadd_rn(total, sr[pos]);
        tots[tid] = total;
    }
    consumers_barrier();
    // ---- 3. outputs ----
    {
        const int rg = tid >> 4, cg = tid & 15;    // rows 4 rg .. + 3, columns 8 cg .. + 7
        float acc[4][8];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int c = 0; c < 8; c++) acc[i][c] = 0.0f;
        // as a maker of weights, the thread takes position `lane` of each tile for the eight rows warp + 8 e: a warp's loads
        // of exp values are then 128 consecutive bytes of one row of the scratch array
        constexpr int WP = kTP + 1;                 // pitch of a row's weights in shared memory: [row][position]
        int wlimit[8];
        float wtot[8];
        const float* wsr[8];
        float e_next[8];
#pragma unroll
        for (int e = 0; e < 8; e++) {
            const int wr = warp + 8 * e;
            wlimit[e] = limits[wr], wtot[e] = tots[wr], wsr[e] = score_row(wr);
            e_next[e] = lane <= wlimit[e] ? wsr[e][lane] : 0.0f;
        }
        const int box = cg >> 2, piece0 = (cg & 3) * 2;   // the thread's 8 columns are two 16-byte pieces of box `box`
        for (int tile = 0; tile < tiles; tile++) {
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const int pos = tile * kTP + lane;
                // a position the row must not see weighs +0 (the host masks it to -inf before the softmax: exp gives 0f)
                wbuf[(warp + 8 * e) * WP + lane] = pos <= wlimit[e] ? __fdiv_rn(e_next[e], wtot[e]) : 0.0f;
            }
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const int pos = (tile + 1) * kTP + lane;
                e_next[e] = pos <= wlimit[e] ? wsr[e][pos] : 0.0f;
            }
            consumers_barrier();   // the tile's weights are in place
            const int j = tiles + tile, s = j % kRing;
            if (!s_mbar_wait(&full[s], (unsigned)((j / kRing) & 1), abort_flag)) ok = false, *abort_flag = 1;
            const unsigned char* vt = stages + (size_t)s * STAGE_BYTES + box * BOX_BYTES;
            const int count = min(kTP, len - tile * kTP);
            for (int pos = 0; pos < count; pos++) {
                const float ws[4] = {wbuf[(4 * rg) * WP + pos], wbuf[(4 * rg + 1) * WP + pos], wbuf[(4 * rg + 2) * WP + pos], wbuf[(4 * rg + 3) * WP + pos]};
                const float4 va = *(const float4*)(vt + pos * 128 + ((piece0 ^ (pos & 7)) << 4));
                const float4 vb = *(const float4*)(vt + pos * 128 + (((piece0 + 1) ^ (pos & 7)) << 4));
                const float vs[8] = {va.x, va.y, va.z, va.w, vb.x, vb.y, vb.z, vb.w};
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int c = 0; c < 8; c++) acc[i][c] = __fadd_rn(acc[i][c], __fmul_rn(ws[i], vs[c]));
            }
            __syncwarp();
            if (lane == 0) s_mbar_arrive(&empty[s]);
            consumers_barrier();   // everyone is done with the weights before the next tile's overwrite them
        }
        // the rows go out through shared memory (over the queries), so that a warp holds one 32-column block for the quantiser
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int c = 0; c < 8; c++) qs[(4 * rg + i) * QP + 8 * cg + c] = acc[i][c];
    }
    consumers_barrier();
    if (!ok || *abort_flag) {
        if (tid == 0) atomicExch(&p.errors->timeout, 1);
        return;
    }
    for (int item = warp; item < kQRows * (WIDTH / 32); item += kPrefillConsumers / 32) {
        const int r = item / (WIDTH / 32), blk = item % (WIDTH / 32);
        if (limits[r] < 0) continue;
        const float v = qs[r * QP + 32 * blk + lane];
        const int64_t at = ((int64_t)(tile_first + (r >> 2)) * p.heads + head0 + (r & 3)) * WIDTH + 32 * blk + lane;
        if (p.out) p.out[at] = v;
        if (p.sink.qs) quantize_block_q8(v, lane, p.sink.scales + (at >> 5), p.sink.sums + (at >> 5), p.sink.totals + (at >> 5), p.sink.qs + at);
    }
}

}  // namespace

int64_t attention_stream_scratch_bytes(int tokens, int heads, int capacity) { return (int64_t)tokens * heads * capacity * 4 + 256; }

// Whether the streaming kernel takes this call.  `scratch` must hold attention_stream_scratch_bytes.
bool attention_stream_fits(tsm_ctx* ctx, int tokens, int heads, int width, int kv_heads, const float* q, int64_t q_stride, const float* k,
                           const float* v) {
    // Measured on B200 against attention_exact_kernel: 341 against 360 us for 64 ragged streams of up to 4096
    // positions, 230 against 258 us for 16.  TSM_ATTN_STREAM=0 selects the other kernel, for timing it.
    static const char* forced = getenv("TSM_ATTN_STREAM");
    if (forced && forced[0] == '0') return false;
    (void)ctx, (void)tokens;
    bool aligned = (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) == 0 && q_stride % 4 == 0;
    return width == 128 && kv_heads > 0 && heads % kv_heads == 0 && (heads / kv_heads) % 4 == 0 && aligned && tensor_maps_available();
}

// The prefill kernel over `tile_count` query tiles (pairs first token, count in device memory, longest first).
int launch_attention_prefill(tsm_ctx* ctx, const float* q, int64_t q_stride, int tokens, int heads, const float* k, const float* v, int rows,
                             int kv_heads, int capacity, const int* table, float scale, float* out, float* scratch, QuantSink sink,
                             const int* qtiles, int tile_count) {
    constexpr int WIDTH = 128;
    (void)tokens;
    PrefillParams pp{StreamParams{q, q_stride, heads, rows, kv_heads, capacity, table, scale, out, ctx->errors, nullptr, scratch, 1, sink, ctx->wait_hint}, qtiles};
    StreamMaps maps;
    uint64_t plane_rows = (uint64_t)rows * kv_heads * capacity;
    TSM_TRY(make_tensor_map_2d(ctx, &maps.k, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, k, WIDTH, plane_rows, WIDTH * 4, 32, kTP, CU_TENSOR_MAP_SWIZZLE_128B));
    TSM_TRY(make_tensor_map_2d(ctx, &maps.v, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, v, WIDTH, plane_rows, WIDTH * 4, 32, kTP, CU_TENSOR_MAP_SWIZZLE_128B));
    const size_t smem = 1024 + 1024 + (size_t)kRing * kTP * WIDTH * 4 + (size_t)kQRows * (WIDTH + 4) * 4 + (size_t)kQRows * (kTP + 1) * 4;
    auto kernel = attention_prefill_kernel<WIDTH>;
    {
        static std::mutex lock;
        static std::map<int, bool> done;
        std::lock_guard<std::mutex> guard(lock);
        if (!done.count(ctx->ordinal)) {
            TSM_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            done[ctx->ordinal] = true;
        }
    }
    const int groups = kv_heads * (heads / kv_heads / 4);
    TSM_CUDA(ctx, launch_chained(ctx, kernel, dim3(groups, tile_count), dim3(kPrefillConsumers + 32), smem, pp, maps));
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

int launch_attention_stream(tsm_ctx* ctx, const float* q, int64_t q_stride, int tokens, int heads, const float* k, const float* v,
                            int rows, int kv_heads, int capacity, const int* table, float scale, float* out, const int* order,
                            float* scratch, QuantSink sink) {
    constexpr int WIDTH = 128;
    StreamParams p{q, q_stride, heads, rows, kv_heads, capacity, table, scale, out, ctx->errors, order, scratch, 1, sink, ctx->wait_hint};
    StreamMaps maps;
    uint64_t plane_rows = (uint64_t)rows * kv_heads * capacity;
    TSM_TRY(make_tensor_map_2d(ctx, &maps.k, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, k, WIDTH, plane_rows, WIDTH * 4, 32, kTP, CU_TENSOR_MAP_SWIZZLE_128B));
    TSM_TRY(make_tensor_map_2d(ctx, &maps.v, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, v, WIDTH, plane_rows, WIDTH * 4, 32, kTP, CU_TENSOR_MAP_SWIZZLE_128B));
    const int groups = kv_heads * (heads / kv_heads / 4);
    // At most one (token, kv head) pair per SM and long caches: three launches that cut the score pass by positions and the
    // value pass by quarters of the width, so that the longest stream does not set the time alone (the single launch lasts
    // as long as one CTA takes for the longest stream: 163 us for 4224 positions).  Measured, 64 streams of up to 4224
    // positions on 1, 2, 4 and 8 kv heads (64 to 512 pairs): 106 against 163 us, 130 against 166, 195 against 184, and 433
    // against 231, where the single launch stays.  TSM_ATTN_SPLIT=0 / 1 forces the choice.
    static const char* forced = getenv("TSM_ATTN_SPLIT");
    bool split = (int64_t)tokens * groups <= (int64_t)ctx->sm_count && capacity >= 1024;
    if (forced) split = forced[0] == '1';
    if (split) {
        size_t smem_scores = 1024 + 8192 + (size_t)kRing * kTP * WIDTH * 4 + 4 * (WIDTH + 4) * 4;
        {
            static std::mutex lock;
            static std::map<int, bool> done;
            std::lock_guard<std::mutex> guard(lock);
            if (!done.count(ctx->ordinal)) {
                TSM_CUDA(ctx, cudaFuncSetAttribute(attention_scores_kernel<WIDTH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_scores));
                done[ctx->ordinal] = true;
            }
        }
        int64_t pairs = (int64_t)tokens * groups;
        // enough position ranges for about four CTAs per SM, none shorter than 8 tiles
        int64_t longest = ((int64_t)capacity + kTP - 1) / kTP;
        p.splits = (int)std::max<int64_t>(1, std::min<int64_t>(std::min<int64_t>(16, longest / 8), (4 * (int64_t)ctx->sm_count + pairs - 1) / pairs));
        TSM_CUDA(ctx, launch_chained(ctx, attention_scores_kernel<WIDTH>, dim3(groups, tokens, p.splits), dim3(kConsumers + 32), smem_scores, p, maps));
        count_launch(ctx);
        TSM_LAUNCH_CHECK(ctx);
        static const int chunked = getenv("TSM_PLAIN_ORDERED_SUM") ? 0 : 1;   // the term-by-term sum instead, for timing it
        const size_t smem_weights = (size_t)std::min(kWeightSegment, (capacity + kSumChunk - 1) / kSumChunk * kSumChunk) * 4;
        TSM_CUDA(ctx, launch_chained(ctx, attention_weights_kernel, dim3(heads, tokens), dim3(256), smem_weights, p, chunked));
        count_launch(ctx);
        TSM_LAUNCH_CHECK(ctx);
        static const char* narrow = getenv("TSM_ATTN_VALUES_NARROW");   // the one-warp-per-box value pass, for timing it
        if (narrow && narrow[0] == '1') TSM_CUDA(ctx, launch_chained(ctx, attention_values_kernel<WIDTH>, dim3(groups * 4, tokens), dim3(64), 0, p, maps));
        else {
            const bool deep = (int64_t)groups * 4 * tokens <= 3 * (int64_t)ctx->sm_count;
            const size_t smem_wide = 1024 + (size_t)(deep ? 16 : kWideDeep) * kTP * 128 + (size_t)4 * 2 * 256 * 4 * 4;   // the ring, then the warps' weights
            auto wide = deep ? attention_values_wide_kernel<WIDTH, 16> : attention_values_wide_kernel<WIDTH, kWideDeep>;
            static std::mutex wide_lock;
            static std::map<std::pair<int, bool>, bool> wide_done;
            {
                std::lock_guard<std::mutex> guard(wide_lock);
                if (!wide_done.count({ctx->ordinal, deep})) {
                    TSM_CUDA(ctx, cudaFuncSetAttribute(wide, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_wide));
                    wide_done[{ctx->ordinal, deep}] = true;
                }
            }
            TSM_CUDA(ctx, launch_chained(ctx, wide, dim3(groups * 4, tokens), dim3(160), smem_wide, p, maps));
        }
        count_launch(ctx);
        TSM_LAUNCH_CHECK(ctx);
        return TSM_OK;
    }
    // TSM_ATTN_RING = 3 .. 6 stages (of 16 KB) per CTA, for timing one depth against another; two CTAs fit an SM up to 6
    static const int ring = getenv("TSM_ATTN_RING") ? atoi(getenv("TSM_ATTN_RING")) : 5;
    const int depth = ring >= 3 && ring <= 6 ? ring : 5;
    size_t smem = 1024 + (size_t)kStreamHeader + (size_t)depth * kTP * WIDTH * 4 + 4 * (WIDTH + 4) * 4;
    auto kernel = depth == 3 ? attention_stream_kernel<WIDTH, 3> : depth == 4 ? attention_stream_kernel<WIDTH, 4>
                : depth == 6 ? attention_stream_kernel<WIDTH, 6> : attention_stream_kernel<WIDTH, 5>;
    {
        static std::mutex lock;
        static std::map<int, bool> done;
        std::lock_guard<std::mutex> guard(lock);
        if (!done.count(ctx->ordinal)) {
            TSM_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            done[ctx->ordinal] = true;
        }
    }
    dim3 grid(groups, tokens);
    TSM_CUDA(ctx, launch_chained(ctx, kernel, grid, dim3(kConsumers + 32), smem, p, maps));
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

}  // namespace tsm
