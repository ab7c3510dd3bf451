// Decode attention over the in-place KV cache [rows, kv_heads, capacity, width] (F32), one query per
// token, ragged lengths (Tensor.ragged_attention, tensor/composite.cr:210-227; the host composite of
// devices/host.cr:368-387, 700-721 is the arithmetic being matched).
//
// fast path (mode TSM_FAST, head width 64 or 128): split-K with online softmax.  Positions are cut
//   into chunks of 256 at fixed absolute offsets; one CTA takes (chunk, kv head, token), scores all the
//   query heads that share the kv head while the keys pass through registers once, and writes the
//   chunk's (max, sum, unnormalised output).  A second kernel merges a token's chunks in chunk order,
//   so a stream's bits depend neither on the batch around it nor on other streams' lengths.
//
// ordered path (mode TSM_EXACT, or any other head width): the host's order of arithmetic — each score
//   a dot product folded over the width from 0f, the host's own exp polynomial, the denominator
//   folded over positions in order, each output column folded over positions in order — run as many
//   independent chains in parallel (positions for scores, columns for outputs), which gives the host's
//   bits.
#include <math.h>
#include <stdlib.h>

#include "common.cuh"
#include "row_helpers.cuh"

namespace tsm {

constexpr int kChunk = 256;

struct QuantOutA {
    float* scales;
    float* sums;
    int* totals;
    int8_t* qs;
};

// ---- fast path --------------------------------------------------------------------------------------

template <int WIDTH, int GROUP>
__global__ void __launch_bounds__(256) attention_chunk_kernel(const float* __restrict__ q, int64_t q_stride, int heads,
                                                              const float* __restrict__ k, const float* __restrict__ v,
                                                              int rows, int kv_heads, int capacity,
                                                              const int* __restrict__ table, float scale, int chunks,
                                                              float* part_o, float* part_ml, ErrorRecord* errors) {
    chained_kernel_entry();
    constexpr int LPP = WIDTH / 16;  // lanes per position in the score phase (16 values each)
    constexpr int PPW = 32 / LPP;    // positions per warp iteration
    constexpr int TPR = WIDTH / 4;   // threads per value row in the output phase
    constexpr int PG = 256 / TPR;    // position groups in the output phase
    __shared__ float scores[GROUP][kChunk];
    __shared__ __align__(16) float red[PG][GROUP][WIDTH];
    __shared__ float stat[GROUP][2];
    __shared__ float wred[8][GROUP];

    const int chunk = blockIdx.x, token = blockIdx.z;
    const int groups_per_kv = (heads / kv_heads) / GROUP;
    const int kvh = blockIdx.y / groups_per_kv;
    const int head0 = kvh * (heads / kv_heads) + (blockIdx.y % groups_per_kv) * GROUP;
    const int row = table[3 * token], limit = table[3 * token + 1];
    if (row < 0 || row >= rows || limit < 0 || limit >= capacity) {
        if (threadIdx.x == 0 && chunk == 0 && blockIdx.y == 0) report_bad_index(errors, limit, capacity);
        return;
    }
    const int len = limit + 1;
    const int c0 = chunk * kChunk;
    if (c0 >= len) return;
    const int cnt = min(kChunk, len - c0);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* kbase = k + (((int64_t)row * kv_heads + kvh) * capacity + c0) * WIDTH;
    const float* vbase = v + (((int64_t)row * kv_heads + kvh) * capacity + c0) * WIDTH;

    // queries: lane holds values d = 4*(lane % LPP) + 4*LPP*i + {0..3}, i < 4, of each head
    float4 qr[GROUP][4];
    {
        const float* qt = q + (int64_t)token * q_stride + (int64_t)head0 * WIDTH;
#pragma unroll
        for (int h = 0; h < GROUP; h++)
#pragma unroll
            for (int i = 0; i < 4; i++) qr[h][i] = *(const float4*)(qt + h * WIDTH + 4 * (lane % LPP) + 4 * LPP * i);
    }
    // scores
    for (int base = warp * PPW; base < kChunk; base += 8 * PPW) {
        int p = base + lane / LPP;
        float dot[GROUP];
#pragma unroll
        for (int h = 0; h < GROUP; h++) dot[h] = 0.0f;
        if (p < cnt) {
            const float* kp = kbase + (int64_t)p * WIDTH + 4 * (lane % LPP);
            float4 kv4[4];
#pragma unroll
            for (int i = 0; i < 4; i++) kv4[i] = *(const float4*)(kp + 4 * LPP * i);
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int h = 0; h < GROUP; h++)
                    dot[h] += qr[h][i].x * kv4[i].x + qr[h][i].y * kv4[i].y + qr[h][i].z * kv4[i].z + qr[h][i].w * kv4[i].w;
        }
#pragma unroll
        for (int off = LPP / 2; off > 0; off >>= 1)
#pragma unroll
            for (int h = 0; h < GROUP; h++) dot[h] += __shfl_xor_sync(0xffffffffu, dot[h], off);
        if (lane % LPP == 0) {
#pragma unroll
            for (int h = 0; h < GROUP; h++) scores[h][p] = p < cnt ? dot[h] * scale : -INFINITY;
        }
    }
    __syncthreads();
    // chunk maximum and exponentials (each thread owns one position)
    float sv[GROUP], mx[GROUP];
#pragma unroll
    for (int h = 0; h < GROUP; h++) {
        sv[h] = scores[h][tid];
        mx[h] = sv[h];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], off));
        if (lane == 0) wred[warp][h] = mx[h];
    }
    __syncthreads();
    float ev[GROUP], sm[GROUP];
#pragma unroll
    for (int h = 0; h < GROUP; h++) {
        float m = wred[0][h];
#pragma unroll
        for (int w2 = 1; w2 < 8; w2++) m = fmaxf(m, wred[w2][h]);
        mx[h] = m;
        ev[h] = expf(sv[h] - m);  // -inf beyond the chunk's end gives 0
        sm[h] = ev[h];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) sm[h] += __shfl_xor_sync(0xffffffffu, sm[h], off);
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < GROUP; h++) {
        scores[h][tid] = ev[h];
        if (lane == 0) wred[warp][h] = sm[h];
    }
    __syncthreads();
    if (tid < GROUP) {
        float l = 0.0f;
        for (int w2 = 0; w2 < 8; w2++) l += wred[w2][tid];
        stat[tid][0] = mx[tid];
        stat[tid][1] = l;
    }
    // weighted values: thread (pg, cg) folds positions pg, pg + PG, ... for 4 columns of every head
    const int pg = tid / TPR, cg = tid % TPR;
    float4 acc[GROUP];
#pragma unroll
    for (int h = 0; h < GROUP; h++) acc[h] = make_float4(0.f, 0.f, 0.f, 0.f);
    int p = pg;
    for (; p + 3 * PG < cnt; p += 4 * PG) {
        float4 vv[4];
#pragma unroll
        for (int u = 0; u < 4; u++) vv[u] = *(const float4*)(vbase + (int64_t)(p + u * PG) * WIDTH + 4 * cg);
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int h = 0; h < GROUP; h++) {
                float w = scores[h][p + u * PG];
                acc[h].x += w * vv[u].x, acc[h].y += w * vv[u].y, acc[h].z += w * vv[u].z, acc[h].w += w * vv[u].w;
            }
    }
    for (; p < cnt; p += PG) {
        float4 vv = *(const float4*)(vbase + (int64_t)p * WIDTH + 4 * cg);
#pragma unroll
        for (int h = 0; h < GROUP; h++) {
            float w = scores[h][p];
            acc[h].x += w * vv.x, acc[h].y += w * vv.y, acc[h].z += w * vv.z, acc[h].w += w * vv.w;
        }
    }
#pragma unroll
    for (int h = 0; h < GROUP; h++) *(float4*)&red[pg][h][4 * cg] = acc[h];
    __syncthreads();
    for (int i = tid; i < GROUP * WIDTH; i += 256) {
        int h = i / WIDTH, c = i % WIDTH;
        float total = 0.0f;
#pragma unroll 4
        for (int g = 0; g < PG; g++) total += red[g][h][c];
        part_o[(((int64_t)token * heads + head0 + h) * chunks + chunk) * WIDTH + c] = total;
    }
    if (tid < GROUP) {
        float* ml = part_ml + (((int64_t)token * heads + head0 + tid) * chunks + chunk) * 2;
        ml[0] = stat[tid][0];
        ml[1] = stat[tid][1];
    }
}

// Merges a token's chunks in chunk order; one warp per 32 output columns so that the block quantiser
// for the product that follows can run in registers.
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, int heads,
                                       int width, int chunks, const int* __restrict__ table, int capacity, float* out,
                                       QuantOutA qo) {
    chained_kernel_entry();
    int token = blockIdx.y;
    int lane = threadIdx.x & 31;
    int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);  // 32-column block of the token's [heads*width]
    int total = heads * width;
    if (item * 32 >= total) return;
    int col = item * 32 + lane;
    int limit = table[3 * token + 1];
    float y = 0.0f;
    if (col < total && limit >= 0 && limit < capacity) {
        int head = col / width, c = col % width;
        int used = limit / kChunk + 1;
        const float* ml = part_ml + ((int64_t)token * heads + head) * chunks * 2;
        const float* po = part_o + ((int64_t)token * heads + head) * chunks * width + c;
        float m = ml[0];
        for (int i = 1; i < used; i++) m = fmaxf(m, ml[2 * i]);
        float l = 0.0f, o = 0.0f;
        for (int i = 0; i < used; i++) {
            float f = expf(ml[2 * i] - m);
            l += ml[2 * i + 1] * f;
            o += po[(int64_t)i * width] * f;
        }
        y = o / l;
        if (out) out[(int64_t)token * total + col] = y;
    }
    if (qo.qs) {
        int64_t at = (int64_t)token * (total >> 5) + item;
        quantize_block_q8(y, lane, qo.scales + at, qo.sums + at, qo.totals + at, qo.qs + (int64_t)token * total + col);
    }
}

// ---- ordered path ----------------------------------------------------------------------------------

// One CTA per (query head, token).  Shared memory holds the row's scores (len floats).
__global__ void attention_ordered_kernel(const float* __restrict__ q, int64_t q_stride, int heads, int width,
                                         const float* __restrict__ k, const float* __restrict__ v, int rows, int kv_heads,
                                         int capacity, const int* __restrict__ table, float scale, float* out,
                                         ErrorRecord* errors) {
    chained_kernel_entry();
    extern __shared__ float sh[];
    float* qs = sh;              // width
    float* scores = sh + width;  // len
    __shared__ float wmax[32];
    __shared__ float total_s;
    const int head = blockIdx.x, token = blockIdx.y;
    const int row = table[3 * token], limit = table[3 * token + 1];
    if (row < 0 || row >= rows || limit < 0 || limit >= capacity) {
        if (threadIdx.x == 0 && head == 0) report_bad_index(errors, limit, capacity);
        return;
    }
    const int len = limit + 1;
    const int kvh = head / (heads / kv_heads);
    const float* kb = k + ((int64_t)row * kv_heads + kvh) * capacity * width;
    const float* vb = v + ((int64_t)row * kv_heads + kvh) * capacity * width;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, warps = blockDim.x >> 5;
    for (int d = tid; d < width; d += blockDim.x) qs[d] = q[(int64_t)token * q_stride + (int64_t)head * width + d];
    __syncthreads();
    float top = -INFINITY;
    for (int p = tid; p < len; p += blockDim.x) {
        const float* kp = kb + (int64_t)p * width;
        float dot = 0.0f;
        for (int d = 0; d < width; d++) dot = __fadd_rn(dot, __fmul_rn(qs[d], kp[d]));
        float s = __fadd_rn(__fmul_rn(dot, scale), 0.0f);
        scores[p] = s;
        top = fmaxf(top, s);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, off));
    if (lane == 0) wmax[warp] = top;
    __syncthreads();
    top = wmax[0];
    for (int w2 = 1; w2 < warps; w2++) top = fmaxf(top, wmax[w2]);
    for (int p = tid; p < len; p += blockDim.x) scores[p] = exact_exp(__fsub_rn(scores[p], top));
    __syncthreads();
    if (tid == 0) {
        float total = 0.0f;
        for (int p = 0; p < len; p++) total = __fadd_rn(total, scores[p]);
        total_s = total;
    }
    __syncthreads();
    float total = total_s;
    for (int p = tid; p < len; p += blockDim.x) scores[p] = __fdiv_rn(scores[p], total);
    __syncthreads();
    for (int c = tid; c < width; c += blockDim.x) {
        float acc = 0.0f;
        for (int p = 0; p < len; p++) acc = __fadd_rn(acc, __fmul_rn(scores[p], vb[(int64_t)p * width + c]));
        out[((int64_t)token * heads + head) * width + c] = acc;
    }
}

// The ordered path for head widths 64 and 128, built for throughput: one CTA per (token, group of G
// query heads that share a kv head).
//  1. scores: keys arrive in tiles of 64 or 128 positions through a ring of cp.async stages into shared memory rows padded by
//     16 bytes (so that threads walking different rows hit different banks); thread (position, head)
//     folds its dot product over the width in index order.
//  2. the maximum, the host's exp of each score, then one thread per head folds the denominator over
//     positions in order (loads run ahead of the adds), then every weight is divided by it.
//  3. outputs: thread (column, heads) folds weight * value over positions in order, values read
//     coalesced from the cache.
// Scores live in shared memory interleaved by head: sc[p * GS + h], GS = 1, 2 or 4.

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int WIDTH, int G, int THREADS, int TP, int STAGES, int UNROLL>
__global__ void __launch_bounds__(THREADS) attention_exact_kernel(const float* __restrict__ q, int64_t q_stride, int heads,
                                                                  const float* __restrict__ k, const float* __restrict__ v,
                                                                  int rows, int kv_heads, int capacity,
                                                                  const int* __restrict__ table, float scale, float* out,
                                                                  ErrorRecord* errors, const int* __restrict__ order, QuantSink sink,
                                                                  int fresh, FreshRows fresh_rows) {
    chained_kernel_entry();
    constexpr int GS = G == 3 ? 4 : G;          // interleave stride of the scores
    constexpr int PITCH = WIDTH + 4;            // floats per staged key row
    constexpr int CHUNKS = WIDTH / 4;           // 16-byte pieces per key row
    constexpr int WARPS = THREADS / 32;
    static_assert(THREADS / GS >= TP && THREADS % GS == 0 && THREADS >= WIDTH, "thread mapping");
    extern __shared__ __align__(16) float sh[];
    float* qs = sh;                         // [GS][PITCH]
    float* kt = qs + GS * PITCH;            // [STAGES][TP][PITCH]
    float* sc = kt + STAGES * TP * PITCH;   // [capacity * GS]
    __shared__ float wred[WARPS][4];
    __shared__ float totals[4];
    __shared__ __align__(16) float fresh_k[WIDTH], fresh_v[WIDTH];  // the token's own key and value (FreshRows)

    const int token = order ? order[blockIdx.y] : blockIdx.y;  // longest tokens first when an order is given
    const int per_kv = heads / kv_heads, groups_per_kv = per_kv / G;
    const int kvh = blockIdx.x / groups_per_kv;
    const int head0 = kvh * per_kv + (blockIdx.x % groups_per_kv) * G;
    const int row = table[3 * token], limit = table[3 * token + 1];
    if (row < 0 || row >= rows || limit < 0 || limit >= capacity) {
        if (threadIdx.x == 0 && blockIdx.x == 0) report_bad_index(errors, limit, capacity);
        return;
    }
    const int len = limit + 1;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* kb = k + ((int64_t)row * kv_heads + kvh) * capacity * WIDTH;
    const float* vb = v + ((int64_t)row * kv_heads + kvh) * capacity * WIDTH;

    if (fresh) {
        // q is the token's joined [q; k; v] row as the projection left it: rotate this CTA's query heads and the kv head's key
        // on the way in (rope_append_kernel's arithmetic), keep key and value for position `limit`, and let the first CTA of
        // the kv head append them to the cache
        constexpr int HALF = WIDTH / 2;
        const float* joined = q + (int64_t)token * q_stride;
        const float* cs = fresh_rows.cos_table ? fresh_rows.cos_table + (int64_t)limit * WIDTH : nullptr;
        const float* sn = fresh_rows.cos_table ? fresh_rows.sin_table + (int64_t)limit * WIDTH : nullptr;
        if (cs && limit >= fresh_rows.context) {
            if (threadIdx.x == 0 && blockIdx.x == 0) report_bad_index(errors, limit, fresh_rows.context);
            return;
        }
        for (int i = tid; i < (G + 2) * HALF; i += THREADS) {
            int h = i / HALF, col = i % HALF;  // h < G: a query head; G: the key; G + 1: the value
            const float* src = joined + (int64_t)(h < G ? head0 + h : h == G ? heads + kvh : heads + kv_heads + kvh) * WIDTH;
            float a = src[col], b = src[col + HALF];
            if (cs && h <= G) {
                float ra, rb;
                rotate_pair(a, b, cs, sn, col, HALF, &ra, &rb);
                a = ra, b = rb;
            }
            float* dst = h < G ? qs + h * PITCH : h == G ? fresh_k : fresh_v;
            dst[col] = a, dst[col + HALF] = b;
            if (h >= G && blockIdx.x % groups_per_kv == 0) {
                float* cache_row = const_cast<float*>(h == G ? kb : vb) + (int64_t)limit * WIDTH;
                cache_row[col] = a, cache_row[col + HALF] = b;
            }
        }
    } else {
        for (int i = tid; i < G * WIDTH; i += THREADS)
            qs[(i / WIDTH) * PITCH + i % WIDTH] = q[(int64_t)token * q_stride + (int64_t)head0 * WIDTH + i];
    }

    const int tiles = (len + TP - 1) / TP;
    // Tile loads: thread tid always copies 16-byte piece (tid % CHUNKS) of rows (tid / CHUNKS) + n * (THREADS / CHUNKS),
    // so the addresses are a fixed base plus a constant stride.
    constexpr int RPP = THREADS / CHUNKS;  // rows covered by one pass of all threads
    static_assert(THREADS % CHUNKS == 0 && TP % RPP == 0, "tile load mapping");
    const int lrow = tid / CHUNKS, lpiece = tid % CHUNKS;
    auto load_rows = [&](const float* src, int tile) {  // always commits a group, so that group t is tile t
        if (tile < tiles) {
            int p0 = tile * TP;
            int count = min(TP, len - p0);
            float* dst = kt + (tile % STAGES) * TP * PITCH + lrow * PITCH + 4 * lpiece;
            const float* from = src + (int64_t)(p0 + lrow) * WIDTH + 4 * lpiece;
#pragma unroll
            for (int n = 0; n < TP / RPP; n++)
                if (lrow + n * RPP < count) cp_async16(dst + n * RPP * PITCH, from + (int64_t)n * RPP * WIDTH);
        }
        cp_async_commit();
    };
    auto load_tile = [&](int tile) { load_rows(kb, tile); };

    // ---- 1. scores ----
    const int sp = tid / GS, shd = tid % GS;  // this thread's position within a tile and its head
    float top = -INFINITY;
#pragma unroll
    for (int t = 0; t < STAGES - 1; t++) load_tile(t);
    for (int tile = 0; tile < tiles; tile++) {
        load_tile(tile + STAGES - 1);  // into the stage read in the previous iteration (a barrier ended it)
        cp_async_wait<STAGES - 1>();
        __syncthreads();
        if (fresh && tile == tiles - 1) {  // the last position is this token's own key: whatever the cache held there is replaced
            if (tid < WIDTH) kt[((tile % STAGES) * TP + (limit - tile * TP)) * PITCH + tid] = fresh_k[tid];
            __syncthreads();
        }
        int p = tile * TP + sp;
        if (sp < TP && shd < G && p < len) {
            const float4* kr = (const float4*)(kt + ((tile % STAGES) * TP + sp) * PITCH);
            const float4* qr = (const float4*)(qs + shd * PITCH);
            float dot = 0.0f;
#pragma unroll 8
            for (int c = 0; c < CHUNKS; c++) {
                float4 kv4 = kr[c], qv = qr[c];
                dot = __fadd_rn(dot, __fmul_rn(qv.x, kv4.x));
                dot = __fadd_rn(dot, __fmul_rn(qv.y, kv4.y));
                dot = __fadd_rn(dot, __fmul_rn(qv.z, kv4.z));
                dot = __fadd_rn(dot, __fmul_rn(qv.w, kv4.w));
            }
            float s = __fadd_rn(__fmul_rn(dot, scale), 0.0f);
            sc[p * GS + shd] = s;
            top = fmaxf(top, s);
        }
        __syncthreads();
    }
    // ---- 2. softmax weights ----
    // threads of one head are GS apart, so a butterfly over offsets >= GS keeps heads separate
#pragma unroll
    for (int off = 16; off >= GS; off >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, off));
    if (lane < GS) wred[warp][lane] = top;
    __syncthreads();
    {
        // THREADS % GS == 0, so in the flat walk below a thread always meets its own head
        float m = wred[0][shd];
#pragma unroll
        for (int w2 = 1; w2 < WARPS; w2++) m = fmaxf(m, wred[w2][shd]);
        if (shd < G)
            for (int i = tid; i < len * GS; i += THREADS) sc[i] = exact_exp(__fsub_rn(sc[i], m));
    }
    __syncthreads();
    if (tid < G) {
        float total = 0.0f;
        int p = 0;
        for (; p + 8 <= len; p += 8) {
            float e[8];
#pragma unroll
            for (int u = 0; u < 8; u++) e[u] = sc[(p + u) * GS + tid];
#pragma unroll
            for (int u = 0; u < 8; u++) total = __fadd_rn(total, e[u]);
        }
        for (; p < len; p++) total = __fadd_rn(total, sc[p * GS + tid]);
        totals[tid] = total;
    }
    __syncthreads();
    if (shd < G) {
        float total = totals[shd];
        for (int i = tid; i < len * GS; i += THREADS) sc[i] = __fdiv_rn(sc[i], total);
    }
    __syncthreads();
    // ---- 3. outputs: values pass through the same ring of stages (rows unpadded reads are conflict-free:
    //         consecutive threads read consecutive columns) ----
    // One thread per column folds all G heads' chains (the weights of a position are one 16-byte broadcast
    // load); the other threads only help to fetch.
    const int col = tid;
    const bool folds = tid < WIDTH;
    auto load_values = [&](int tile) { load_rows(vb, tile); };
    float acc[G];
#pragma unroll
    for (int i = 0; i < G; i++) acc[i] = 0.0f;
#pragma unroll
    for (int t = 0; t < STAGES - 1; t++) load_values(t);
    for (int tile = 0; tile < tiles; tile++) {
        load_values(tile + STAGES - 1);
        cp_async_wait<STAGES - 1>();
        __syncthreads();
        if (fresh && tile == tiles - 1) {
            if (tid < WIDTH) kt[((tile % STAGES) * TP + (limit - tile * TP)) * PITCH + tid] = fresh_v[tid];
            __syncthreads();
        }
        if (folds) {
            const float* vt = kt + (tile % STAGES) * TP * PITCH + col;
            const float* wt = sc + (int64_t)tile * TP * GS;
            int count = min(TP, len - tile * TP);
            int p = 0;
            for (; p + 8 <= count; p += 8) {
                float vv[8];
#pragma unroll
                for (int u = 0; u < 8; u++) vv[u] = vt[(p + u) * PITCH];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    float w[GS];
                    if (GS == 4) {
                        float4 w4 = *(const float4*)(wt + (p + u) * 4);
                        w[0] = w4.x, w[1] = w4.y, w[2] = w4.z, w[3] = w4.w;
                    } else if (GS == 2) {
                        float2 w2 = *(const float2*)(wt + (p + u) * 2);
                        w[0] = w2.x, w[1] = w2.y;
                    } else {
                        w[0] = wt[p + u];
                    }
#pragma unroll
                    for (int i = 0; i < G; i++) acc[i] = __fadd_rn(acc[i], __fmul_rn(w[i], vv[u]));
                }
            }
            for (; p < count; p++) {
                float vv = vt[p * PITCH];
#pragma unroll
                for (int i = 0; i < G; i++) acc[i] = __fadd_rn(acc[i], __fmul_rn(wt[p * GS + i], vv));
            }
        }
        __syncthreads();
    }
    if (folds) {  // warps 0 .. WIDTH / 32 - 1, all lanes: a warp holds one 32-column block of each of its heads
#pragma unroll
        for (int i = 0; i < G; i++) {
            int64_t at = ((int64_t)token * heads + head0 + i) * WIDTH + col;
            if (out) out[at] = acc[i];
            if (sink.qs) quantize_block_q8(acc[i], lane, sink.scales + (at >> 5), sink.sums + (at >> 5), sink.totals + (at >> 5), sink.qs + at);
        }
    }
}

// Ranks tokens by visible positions, most first: with one long-running CTA per (token, kv group) and ragged
// lengths, starting the longest first keeps the last wave short.
__global__ void length_order_kernel(const int* __restrict__ table, int tokens, int* order) {
    chained_kernel_entry();
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= tokens) return;
    int mine = table[3 * t + 1], rank = 0;
    for (int u = 0; u < tokens; u++) {
        int other = table[3 * u + 1];
        rank += (other > mine || (other == mine && u < t)) ? 1 : 0;
    }
    order[rank] = t;
}

int launch_length_order(tsm_ctx* ctx, const int* table, int tokens, int* order) {
    OpTimer timer(ctx, "Attention order", tokens);
    if (tokens == 0) return TSM_OK;
    TSM_CUDA(ctx, launch_chained(ctx, length_order_kernel, dim3((tokens + 255) / 256), dim3(256), 0, table, tokens, order));
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

// ---- host side -----------------------------------------------------------------------------------

int64_t attention_scratch_bytes(int tokens, int heads, int width, int capacity) {
    int chunks = (capacity + kChunk - 1) / kChunk;
    return (int64_t)tokens * heads * chunks * (width + 2) * 4 + 256;
}

template <int WIDTH>
static int launch_fast(tsm_ctx* ctx, const float* q, int64_t q_stride, int tokens, int heads, const float* k, const float* v,
                       int rows, int kv_heads, int capacity, const int* table, float scale, float* out,
                       const QuantizedActs* quantized) {
    int chunks = (capacity + kChunk - 1) / kChunk;
    int64_t need = attention_scratch_bytes(tokens, heads, WIDTH, capacity);
    TSM_TRY(ensure_scratch(ctx, ctx->attn, need));
    float* part_o = (float*)ctx->attn.ptr;
    float* part_ml = part_o + (int64_t)tokens * heads * chunks * WIDTH;
    int per_kv = heads / kv_heads;
    int group = per_kv <= 4 ? per_kv : (per_kv % 4 == 0 ? 4 : (per_kv % 2 == 0 ? 2 : 1));
    dim3 grid(chunks, kv_heads * (per_kv / group), tokens);
#define TSM_ATTN(G)                                                                                                      \
    TSM_CUDA(ctx, launch_chained(ctx, attention_chunk_kernel<WIDTH, G>, grid, dim3(256), 0, q, q_stride, heads, k, v, rows, kv_heads, \
                                 capacity, table, scale, chunks, part_o, part_ml, ctx->errors))
    if (group == 1) TSM_ATTN(1);
    else if (group == 2) TSM_ATTN(2);
    else if (group == 3) TSM_ATTN(3);
    else TSM_ATTN(4);
#undef TSM_ATTN
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    QuantOutA qo{nullptr, nullptr, nullptr, nullptr};
    if (quantized) qo = QuantOutA{(float*)quantized->scales, (float*)quantized->sums, (int*)quantized->totals, (int8_t*)quantized->qs};
    int items = (heads * WIDTH + 31) / 32;
    dim3 mgrid((items + 3) / 4, tokens);
    TSM_CUDA(ctx, launch_chained(ctx, attention_merge_kernel, mgrid, dim3(128), 0, part_o, part_ml, heads, WIDTH, chunks, table, capacity, out, qo));
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

int launch_attention(tsm_ctx* ctx, const float* q, int64_t q_stride, int tokens, int heads, int width, const float* k,
                     const float* v, int rows, int kv_heads, int capacity, const int* table, float scale, float* out,
                     const QuantizedActs* quantized, const int* order, const FreshRows* fresh) {
    OpTimer timer(ctx, fresh ? "Rope+WriteRows+RaggedAttention" : "RaggedAttention", tokens, heads, width);
    if (kv_heads <= 0 || heads % kv_heads != 0)
        return fail(ctx, TSM_ERR_ARG, std::to_string(heads) + " query heads do not group into " + std::to_string(kv_heads) + " key and value heads");
    if (tokens == 0) return TSM_OK;
    bool aligned = (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) == 0 && q_stride % 4 == 0;
    // FreshRows is served by attention_exact_kernel alone; every other kernel gets the separate rope + append launch first
    static const bool no_fresh = getenv("TSM_NO_FRESH_ROWS") != nullptr;  // time the separate launch instead
    auto settle_fresh = [&]() -> int {
        if (!fresh) return TSM_OK;
        const FreshRows* f = fresh;
        fresh = nullptr;
        return launch_rope_append(ctx, const_cast<float*>(q), tokens, heads, kv_heads, width, f->cos_table, f->sin_table, f->context, table,
                                  const_cast<float*>(k), const_cast<float*>(v), rows, capacity);
    };
    if (no_fresh || (ctx->mode == TSM_FAST && aligned && (width == 64 || width == 128))) TSM_TRY(settle_fresh());
    if (ctx->mode == TSM_FAST && aligned && width == 64)
        return launch_fast<64>(ctx, q, q_stride, tokens, heads, k, v, rows, kv_heads, capacity, table, scale, out, quantized);
    if (ctx->mode == TSM_FAST && aligned && width == 128)
        return launch_fast<128>(ctx, q, q_stride, tokens, heads, k, v, rows, kv_heads, capacity, table, scale, out, quantized);
    if (!out) return fail(ctx, TSM_ERR_ARG, "ordered attention needs an F32 output");
    bool launched = false;
    const QuantSink sink = quant_sink(quantized);  // the kernels for widths 64 and 128 quantise their rows themselves
    if (attention_stream_fits(ctx, tokens, heads, width, kv_heads, q, q_stride, k, v)) {
        TSM_TRY(settle_fresh());
        TSM_TRY(ensure_scratch(ctx, ctx->attn, attention_stream_scratch_bytes(tokens, heads, capacity)));
        static const bool no_prefill = getenv("TSM_NO_PREFILL_KERNEL") != nullptr;   // prompts through the decode kernels, for timing
        if (ctx->prefill_tiles && ctx->prefill_tile_count > 0 && !no_prefill)   // a step that holds prompts: keys and values once per 16 tokens
            return launch_attention_prefill(ctx, q, q_stride, tokens, heads, k, v, rows, kv_heads, capacity, table, scale, out,
                                            (float*)ctx->attn.ptr, sink, ctx->prefill_tiles, ctx->prefill_tile_count);
        return launch_attention_stream(ctx, q, q_stride, tokens, heads, k, v, rows, kv_heads, capacity, table, scale, out, order,
                                       (float*)ctx->attn.ptr, sink);
    }
    const int fresh_on = fresh ? 1 : 0;
    const FreshRows fresh_rows = fresh ? *fresh : FreshRows{nullptr, nullptr, 0};
    if (aligned && (width == 64 || width == 128)) {
        int per_kv = heads / kv_heads;
        int pitch = width + 4;
        for (int g = 4; g >= 1 && !launched; g--) {
            if (per_kv % g != 0) continue;
            int gs = g == 3 ? 4 : g;
            bool small = width == 64 && g == 1;  // few chains per CTA: smaller CTAs, more of them per SM
            int tp = width == 128 ? 64 : (small ? 64 : 128);
            for (int stages = 3; stages >= 2 && !launched; stages--) {
                size_t smem = ((size_t)gs * pitch + (size_t)stages * tp * pitch + (size_t)capacity * gs) * 4;
                if (smem > 200 * 1024) continue;
                dim3 grid(kv_heads * (per_kv / g), tokens);
#define TSM_EXACT_ATTN(W, G, T, TP, S, U)                                                                                 \
    do {                                                                                                                  \
        auto kernel = attention_exact_kernel<W, G, T, TP, S, U>;                                                          \
        if (smem > 48 * 1024) TSM_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)); \
        TSM_CUDA(ctx, launch_chained(ctx, kernel, grid, dim3(T), smem, q, q_stride, heads, k, v, rows, kv_heads, capacity, table, scale, \
                                     out, ctx->errors, order, sink, fresh_on, fresh_rows));                               \
    } while (0)
#define TSM_EXACT_STAGES(W, G, T, TP, U)          \
    do {                                          \
        if (stages == 3) TSM_EXACT_ATTN(W, G, T, TP, 3, U); \
        else TSM_EXACT_ATTN(W, G, T, TP, 2, U);   \
    } while (0)
                static const bool one_cta = getenv("TSM_ATTN_ONE_CTA") != nullptr;  // the 512-thread shape everywhere, for timing it
                if (width == 64) {
                    if (g == 4) TSM_EXACT_STAGES(64, 4, 512, 128, 16);
                    else if (g == 3) TSM_EXACT_STAGES(64, 3, 512, 128, 16);
                    else if (g == 2) TSM_EXACT_STAGES(64, 2, 512, 128, 16);
                    else TSM_EXACT_STAGES(64, 1, 128, 64, 32);
                } else if (!one_cta && g == 4 && ((size_t)gs * pitch + 2 * (size_t)32 * pitch + (size_t)capacity * gs) * 4 <= 110 * 1024) {
                    // two CTAs of 256 threads per SM overlap one's serial phases with the other's streaming: measured
                    // faster than one CTA of 512 threads with a deeper ring
                    smem = ((size_t)gs * pitch + 2 * (size_t)32 * pitch + (size_t)capacity * gs) * 4;
                    TSM_EXACT_ATTN(128, 4, 256, 32, 2, 16);
                } else {
                    if (g == 4) TSM_EXACT_STAGES(128, 4, 512, 64, 16);
                    else if (g == 3) TSM_EXACT_STAGES(128, 3, 512, 64, 16);
                    else if (g == 2) TSM_EXACT_STAGES(128, 2, 512, 64, 16);
                    else TSM_EXACT_STAGES(128, 1, 512, 64, 16);
                }
#undef TSM_EXACT_STAGES
#undef TSM_EXACT_ATTN
                launched = true;
            }
        }
    }
    const bool fused_quantiser = launched;
    if (!launched) {
        TSM_TRY(settle_fresh());
        size_t smem = (size_t)(width + capacity) * 4;
        if (smem > 200 * 1024) return fail(ctx, TSM_ERR_UNSUPPORTED, "ordered attention over more than 51000 positions");
        if (smem > 48 * 1024)
            TSM_CUDA(ctx, cudaFuncSetAttribute(attention_ordered_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
        dim3 grid(heads, tokens);
        int threads = capacity >= 1024 ? 256 : 128;
        TSM_CUDA(ctx, launch_chained(ctx, attention_ordered_kernel, grid, dim3(threads), smem, q, q_stride, heads, width, k, v, rows, kv_heads,
                                     capacity, table, scale, out, ctx->errors));
    }
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    if (quantized && !fused_quantiser) {
        TSM_TRY(launch_quantize_rows(ctx, out, tokens, heads * width, (int64_t)heads * width, (float*)quantized->scales,
                                     (float*)quantized->sums, (int*)quantized->totals, (int8_t*)quantized->qs));
    }
    return TSM_OK;
}

}  // namespace tsm
