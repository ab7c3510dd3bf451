// The quantised product x . w^T over ggml block weights, with the reference's bits
// (Quant.matmul_reference, quant.cr:122-142; block_matmul_lanes_f32, kernels.cu:1286-1328).
//
// Each output is the sum, IN BLOCK ORDER from 0f, of one float contribution per 32-element block;
// a block's integer dot product may be taken in any order (it is exact), the float sum may not.
//
// streamed kernel (rows of activations <= 4, the decode case)
//   The weight matrix is one contiguous run of blocks.  It is cut into tiles of whole rows; a tile's
//   bytes, widened to whole groups of 8 blocks (4 for Q4_1) so that both ends fall on 16-byte
//   boundaries, arrive in shared memory through one bulk asynchronous copy (cp.async.bulk, completion
//   counted on an mbarrier) into a ring of stages, so HBM sees long sequential reads and no thread
//   spends instructions on loads.  Each compute thread takes one group: 9 / 17 / 5 aligned 16-byte
//   shared loads (group sizes 144 / 272 / 80 bytes are odd multiples of 16, so a quarter-warp's loads
//   fall in distinct banks), unpacks scales and quants with byte permutes, multiplies with __dp4a
//   against the quantised activations held in shared memory, and writes the group's float
//   contributions to a staging array.  A fifth warp folds each row's contributions in block order
//   (one lane per row) while the compute warps work on the next tile, and issues the copies.
//   Two variants of the tile: rows too long for several to fit a stage are taken in pieces (the fold
//   lanes carry their running sums from piece to piece), and with a single row of activations whose
//   length divides what one sweep of the compute threads covers, every thread keeps its activation
//   blocks in registers instead of re-reading them from shared memory for every weight block.
//
// generic kernel (any row count, any alignment down to 2 bytes)
//   One warp per output; lane l takes blocks l, l+32, ...; contributions are folded in block order
//   through shuffles.  It is the fallback for shapes the streamed kernel does not take.
#include <stdlib.h>

#include "common.cuh"

namespace tsm {

template <int KIND> struct Fmt;
template <> struct Fmt<TSM_Q8_0> { static constexpr int B = 34, G = 8, GB = 272, WORDS = 68, CAP = 128; };
template <> struct Fmt<TSM_Q4_0> { static constexpr int B = 18, G = 8, GB = 144, WORDS = 36, CAP = 128; };
template <> struct Fmt<TSM_Q4_1> { static constexpr int B = 20, G = 4, GB = 80, WORDS = 20, CAP = 256; };

constexpr int kComputeThreads = 128;
constexpr int kThreads = 160;  // 4 compute warps + 1 fold/producer warp
constexpr unsigned kWaitSpins = 4u << 20;

struct MatvecParams {
    const uint8_t* w;
    int n, nb;
    QuantizedActs acts;
    const float* bias;
    const float* residual;
    float* out;
    int rows_per_tile, num_tiles;
    int cap, stages;    // groups a stage holds, stages in the ring
    int segments;       // > 1: long rows, a tile is `rows_per_tile` rows x one of `segments` equal pieces of a row (see below)
    int seg_blocks, seg_groups;   // blocks and groups of a piece (the host divides, once)
    unsigned nb_magic;  // floor(2^32 / nb) + 1: x / nb = umulhi(x, nb_magic) for the small x used here
    ErrorRecord* errors;
    const float* plain;   // not null: the rows come as F32, `plain_stride` apart, and every CTA quantises them itself
    int64_t plain_stride;
    int plain_vector;     // they may be read in 16-byte loads
};

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Waits for the phase with a bounded number of tries; false when it ran out.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity) {
    for (unsigned spin = 0; spin < kWaitSpins; spin++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (spin > 4096) __nanosleep(64);
    }
    return false;
}
// Dot product of four unsigned bytes of a with four signed bytes of b, plus c.
__device__ __forceinline__ int dp4a_us(unsigned a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Staging index of a tile-relative block: one pad word per 32, so that lanes folding different rows
// (a whole number of blocks apart) read different banks.
__host__ __device__ __forceinline__ int part_index(int p) { return p + (p >> 5); }
// Byte offset of activation block kb in shared memory: 16 pad bytes per 8 blocks, so that lanes on
// consecutive groups (256 bytes apart) read different banks.
__host__ __device__ __forceinline__ int act_offset(int kb) { return kb * 32 + (kb >> 3) * 16; }

// MODE 0: rows that are not whole groups; 1: whole groups; 2: whole groups, long rows in pieces; 3: whole groups, one row of
// activations, and a row length that divides the blocks one sweep of the compute threads covers: a thread then meets the same
// G activation blocks in every group it takes, and keeps them (values, scales, totals) in registers
template <int KIND, int C, int MODE>
__global__ void __launch_bounds__(kThreads) matvec_stream_kernel(MatvecParams p) {
    constexpr bool ALIGNED = MODE >= 1;
    constexpr bool KEPT = MODE == 3;
    // Q4_0 with kept activations: a thread takes HALF a group (4 blocks, 72 bytes, read in 8-byte loads), so that it keeps 32
    // activation registers and not 64 (with 64 the kernel needed 121 registers and a CTA less fitted an SM)
    constexpr bool HALVES = KEPT && KIND == TSM_Q4_0;
    constexpr int GG = HALVES ? 4 : Fmt<KIND>::G;   // blocks a thread takes at a time
    static_assert(!KEPT || C == 1, "kept activations: one row");
    using F = Fmt<KIND>;
    extern __shared__ __align__(128) unsigned char smem[];
    const int nb = p.nb;
    const int act_bytes = (act_offset(nb) + 15) & ~15;
    const int pcap = part_index(p.cap * F::G) + 1;
    const int kStages = p.stages;
    uint64_t* full = (uint64_t*)smem;                        // one barrier per stage
    int* abort_flag = (int*)(smem + 64);
    unsigned char* acts_q = smem + 128;                      // C x act_bytes
    float* acts_scale = (float*)(acts_q + C * act_bytes);    // C x nb
    float* acts_aux = acts_scale + C * nb;                   // C x nb (Q4_0: totals as int; Q4_1: sums)
    float* parts = acts_aux + C * nb;                        // 2 x C x pcap
    size_t stage_off = (size_t)((unsigned char*)(parts + 2 * C * pcap) - smem);
    stage_off = (stage_off + 127) & ~(size_t)127;
    unsigned char* stages = smem + stage_off;                // stages x cap x GB
    const int kStageBytes = p.cap * F::GB;

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const bool producer = (tid == kComputeThreads);

    auto tile_span = [&](int tile, int& r0, int& r1, int64_t& g0, int& groups) {
        r0 = tile * p.rows_per_tile;
        r1 = min(p.n, r0 + p.rows_per_tile);
        int64_t fb0 = (int64_t)r0 * nb, fb1 = (int64_t)r1 * nb;
        g0 = fb0 / F::G;
        groups = (int)((fb1 + F::G - 1) / F::G - g0);
    };
    // Long rows (p.segments > 1): a whole row fills most of a stage, so whole-row tiles hold 4 rows and the fold warp adds with
    // 4 of its lanes while the rest of the CTA waits for it.  A tile is then `rows_per_tile` rows x ONE of `segments` equal
    // pieces of a row: one copy per row, each row's piece contiguous in the stage; pass `it` of a CTA is piece it % segments
    // of its row tile it / segments, and the fold warp's lanes (one per row, up to 32) keep their running sums from piece to
    // piece, so every output still adds its blocks in order.
    const int S = MODE == 2 ? p.segments : 1;   // a constant 1 in the other modes: the pieces' code and registers drop out
    const int nbs = p.seg_blocks;           // blocks of a piece
    const int gps = p.seg_groups;           // groups of a piece
    auto issue = [&](int it) {
        if (S > 1) {
            int tile = blockIdx.x + (it / S) * gridDim.x, seg = it % S;
            if (tile >= p.num_tiles) return;
            int r0 = tile * p.rows_per_tile, rows = min(p.n, r0 + p.rows_per_tile) - r0;
            int s = it % kStages;
            const unsigned piece = (unsigned)gps * F::GB;
            mbar_expect_tx(&full[s], piece * (unsigned)rows);
            for (int i = 0; i < rows; i++)
                bulk_load(stages + (size_t)s * kStageBytes + (size_t)i * piece, p.w + ((int64_t)(r0 + i) * nb + (int64_t)seg * nbs) * F::B, piece, &full[s]);
            return;
        }
        int tile = blockIdx.x + it * gridDim.x;
        if (tile >= p.num_tiles) return;
        int r0, r1, groups;
        int64_t g0;
        tile_span(tile, r0, r1, g0, groups);
        int s = it % kStages;
        unsigned bytes = (unsigned)groups * F::GB;
        mbar_expect_tx(&full[s], bytes);
        bulk_load(stages + (size_t)s * kStageBytes, p.w + g0 * F::GB, bytes, &full[s]);
    };

    if (tid == 0) {
        for (int s = 0; s < kStages; s++) mbar_init(&full[s], 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (producer)
        for (int it = 0; it < kStages; it++) issue(it);

    // The weights' first stages are on their way; everything below reads what the kernel before this one wrote.
    chained_kernel_wait();
    if (p.plain) {
        // F32 rows: one thread per block of 32 with the quantiser's arithmetic (quantize_block_q8: amax, d = amax / 127,
        // id = 1 / d, round half away, f16 scale)
        for (int c = 0; c < C; c++) {
            const float* xr = p.plain + (int64_t)c * p.plain_stride;
            for (int blk = tid; blk < nb; blk += kThreads) {
                float v[32];
                if (p.plain_vector) {
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        float4 t = ((const float4*)(xr + blk * 32))[u];
                        v[4 * u] = t.x, v[4 * u + 1] = t.y, v[4 * u + 2] = t.z, v[4 * u + 3] = t.w;
                    }
                } else {
#pragma unroll
                    for (int u = 0; u < 32; u++) v[u] = xr[blk * 32 + u];
                }
                float amax = fabsf(v[0]);
#pragma unroll
                for (int u = 1; u < 32; u++) amax = fmaxf(amax, fabsf(v[u]));
                float d = __fdiv_rn(amax, 127.0f);
                float id = d == 0.0f ? 0.0f : __fdiv_rn(1.0f, d);
                int total = 0;
                unsigned words[8];
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    unsigned word = 0;
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        int q = (int)(signed char)(int)roundf(__fmul_rn(v[4 * u + e], id));
                        total += q;
                        word |= (unsigned)(q & 0xff) << (8 * e);
                    }
                    words[u] = word;
                }
                unsigned char* dst = acts_q + c * act_bytes + act_offset(blk);
                *(uint4*)dst = make_uint4(words[0], words[1], words[2], words[3]);
                *(uint4*)(dst + 16) = make_uint4(words[4], words[5], words[6], words[7]);
                acts_scale[c * nb + blk] = round_to_half(d);
                if (KIND == TSM_Q4_0) ((int*)acts_aux)[c * nb + blk] = total;
                if (KIND == TSM_Q4_1) acts_aux[c * nb + blk] = round_to_half(__fmul_rn((float)total, d));
            }
        }
    } else {
    // quantised activations -> shared memory (every CTA reads them once; they stay in L2).
    if (nb <= kThreads) {
    // short rows: a thread has at most two pieces and one block's scale to fetch, and Q4_0's totals come from the same global
    // words, so everything is one round of independent loads and one barrier
    for (int c = 0; c < C; c++) {
        const int4* src = (const int4*)(p.acts.qs + (int64_t)c * nb * 32);
        for (int i = tid; i < nb * 2; i += kThreads) {
            int kb = i >> 1;
            *(int4*)(acts_q + c * act_bytes + act_offset(kb) + (i & 1) * 16) = src[i];
        }
        for (int i = tid; i < nb; i += kThreads) {
            acts_scale[c * nb + i] = p.acts.scales[(int64_t)c * nb + i];
            if (KIND == TSM_Q4_0) {
                // the block's integer sum of quantised activations, for the -8 offset of Q4_0's nibbles
                const int* words = (const int*)(p.acts.qs + ((int64_t)c * nb + i) * 32);
                int total = 0;
#pragma unroll
                for (int u = 0; u < 8; u++) total = __dp4a(0x01010101, words[u], total);
                ((int*)acts_aux)[c * nb + i] = total;
            }
            if (KIND == TSM_Q4_1) acts_aux[c * nb + i] = p.acts.sums[(int64_t)c * nb + i];
        }
    }
    } else {
    // long rows: up to eight loads per thread are issued before the first store: one load per pass, each waited for, cost a
    // trip to L2 per 160 pieces (six trips for rows of 14336 values)
    for (int c = 0; c < C; c++) {
        const int4* src = (const int4*)(p.acts.qs + (int64_t)c * nb * 32);
        for (int i0 = tid; i0 < nb * 2; i0 += kThreads * 8) {
            int4 v[8];
#pragma unroll
            for (int u = 0; u < 8; u++)
                if (i0 + u * kThreads < nb * 2) v[u] = src[i0 + u * kThreads];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int i = i0 + u * kThreads;
                if (i < nb * 2) *(int4*)(acts_q + c * act_bytes + act_offset(i >> 1) + (i & 1) * 16) = v[u];
            }
        }
        for (int i0 = tid; i0 < nb; i0 += kThreads * 4) {
            float sc[4], au[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int i = i0 + u * kThreads;
                sc[u] = i < nb ? p.acts.scales[(int64_t)c * nb + i] : 0.0f;
                au[u] = KIND == TSM_Q4_1 && i < nb ? p.acts.sums[(int64_t)c * nb + i] : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int i = i0 + u * kThreads;
                if (i < nb) {
                    acts_scale[c * nb + i] = sc[u];
                    if (KIND == TSM_Q4_1) acts_aux[c * nb + i] = au[u];
                }
            }
        }
    }
    if (KIND == TSM_Q4_0) {
        // the block's integer sum of quantised activations, for the -8 offset of Q4_0's nibbles: from the copy just made
        __syncthreads();
        for (int c = 0; c < C; c++)
            for (int i = tid; i < nb; i += kThreads) {
                const int4* words = (const int4*)(acts_q + c * act_bytes + act_offset(i));
                const int4 lo = words[0], hi = words[1];
                int total = __dp4a(0x01010101, lo.x, 0);
                total = __dp4a(0x01010101, lo.y, total), total = __dp4a(0x01010101, lo.z, total), total = __dp4a(0x01010101, lo.w, total);
                total = __dp4a(0x01010101, hi.x, total), total = __dp4a(0x01010101, hi.y, total);
                total = __dp4a(0x01010101, hi.z, total), total = __dp4a(0x01010101, hi.w, total);
                ((int*)acts_aux)[c * nb + i] = total;
            }
    }
    }
    }
    __syncthreads();

    // Kept activations: the shared-memory copy is read once.  Read per block instead, the activations are 32 of the 50-odd
    // bytes a 4-bit block moves through shared memory, and that data path, not HBM, was what the kernel filled.
    unsigned kept_q[KEPT ? GG * 8 : 1];
    float kept_dx[KEPT ? GG : 1], kept_aux[KEPT ? GG : 1];
    if (KEPT && tid < kComputeThreads) {
        const int kb = (tid * GG) % nb;
        const uint4* ap = (const uint4*)(acts_q + act_offset(kb));
#pragma unroll
        for (int i = 0; i < GG * 2; i++) {
            const uint4 v = ap[i];
            kept_q[4 * i] = v.x, kept_q[4 * i + 1] = v.y, kept_q[4 * i + 2] = v.z, kept_q[4 * i + 3] = v.w;
        }
#pragma unroll
        for (int j = 0; j < GG; j++) {
            kept_dx[j] = acts_scale[kb + j];
            kept_aux[j] = KIND != TSM_Q8_0 ? acts_aux[kb + j] : 0.0f;
        }
    }

    int prev_r0 = 0, prev_r1 = 0, prev_base = 0, prev_seg = 0;  // the tile whose contributions wait to be folded
    bool have_prev = false;
    float run[C];                                 // segmented tiles: the fold lane's running sums of its row
#pragma unroll
    for (int c = 0; c < C; c++) run[c] = 0.0f;
    int seg = 0, row_tile = blockIdx.x;           // segmented tiles: the piece and the row tile of pass `it`, counted up
    for (int it = 0;; it++) {
        const int tile = S > 1 ? row_tile : blockIdx.x + it * gridDim.x;
        bool valid = tile < p.num_tiles;
        int r0 = 0, r1 = 0, groups = 0;
        int64_t g0 = 0;
        if (valid) {
            if (S > 1) {
                r0 = tile * p.rows_per_tile, r1 = min(p.n, r0 + p.rows_per_tile);
                groups = (r1 - r0) * gps;
            } else {
                tile_span(tile, r0, r1, g0, groups);
            }
        }
        float* cur = parts + (it & 1) * C * pcap;
        if (warp < 4) {
            if (valid) {
                int s = it % kStages;
                bool arrived = mbar_wait(&full[s], (unsigned)((it / kStages) & 1));
                if (!arrived) *abort_flag = 1;
                const unsigned char* stage = stages + (size_t)s * kStageBytes;
                // first activation block of the tile's first group: tiles start on a row, so the group that holds
                // the row's block 0 starts (r0 * nb) mod G blocks earlier, i.e. inside the previous row
                int lead = (int)(((int64_t)r0 * nb) & (F::G - 1));
                int kb_first = ALIGNED || lead == 0 ? 0 : nb - lead;
                // gi counts groups, or half groups (HALVES)
                for (int gi = tid; gi < (HALVES ? 2 * groups : groups) && arrived; gi += kComputeThreads) {
                    unsigned W[HALVES ? F::WORDS / 2 : F::WORDS];
                    if (HALVES) {
                        const uint2* gp = (const uint2*)(stage + (size_t)gi * (F::GB / 2));
#pragma unroll
                        for (int i = 0; i < F::WORDS / 4; i++) {
                            uint2 v = gp[i];
                            W[2 * i] = v.x, W[2 * i + 1] = v.y;
                        }
                    } else {
                        const uint4* gp = (const uint4*)(stage + (size_t)gi * F::GB);
#pragma unroll
                        for (int i = 0; i < F::WORDS / 4; i++) {
                            uint4 v = gp[i];
                            W[4 * i] = v.x, W[4 * i + 1] = v.y, W[4 * i + 2] = v.z, W[4 * i + 3] = v.w;
                        }
                    }
                    // first activation block of the group: (kb_first + gi * G) mod nb by a reciprocal multiply
                    unsigned x = (unsigned)(kb_first + gi * F::G);
                    int kb = (int)(x - __umulhi(x, p.nb_magic) * (unsigned)nb);
                    if (S > 1) kb = seg * nbs + (gi % gps) * F::G;   // group gi is group gi % gps of row gi / gps's piece
                    float* dst = cur + gi * GG + ((gi * GG) >> 5);  // part_index(gi * GG), then + j within the same 32
                    // the group's activation scales (and totals or sums) in 16-byte loads when the group lies in one row
                    float dxs[C][F::G], auxs[C][F::G];
                    if (KEPT) {
#pragma unroll
                        for (int j = 0; j < GG; j++) dxs[0][j] = kept_dx[j], auxs[0][j] = kept_aux[j];
                    } else if (ALIGNED) {
#pragma unroll
                        for (int c = 0; c < C; c++)
#pragma unroll
                            for (int v4 = 0; v4 < F::G / 4; v4++) {
                                float4 d4 = *(const float4*)(acts_scale + c * nb + kb + 4 * v4);
                                dxs[c][4 * v4] = d4.x, dxs[c][4 * v4 + 1] = d4.y, dxs[c][4 * v4 + 2] = d4.z, dxs[c][4 * v4 + 3] = d4.w;
                                if (KIND != TSM_Q8_0) {
                                    float4 a4 = *(const float4*)(acts_aux + c * nb + kb + 4 * v4);
                                    auxs[c][4 * v4] = a4.x, auxs[c][4 * v4 + 1] = a4.y, auxs[c][4 * v4 + 2] = a4.z, auxs[c][4 * v4 + 3] = a4.w;
                                }
                            }
                    }
#pragma unroll
                    for (int j = 0; j < GG; j++) {
                        int kbj = kb + j;
                        if (!ALIGNED && kbj >= nb) kbj -= nb;  // a group may run over the end of a row (rows hold >= G blocks)
                        float dw, mw = 0.0f;
                        unsigned q[8];  // Q8_0: 8 words of int8; Q4: q[0..3] low nibbles, q[4..7] high nibbles still times 16
                        if (KIND == TSM_Q8_0) {
                            const int base = 17 * (j >> 1);
                            if ((j & 1) == 0) {
                                dw = half_bits_to_float(W[base] & 0xffffu);
#pragma unroll
                                for (int i = 0; i < 8; i++) q[i] = __byte_perm(W[base + i], W[base + i + 1], 0x5432);
                            } else {
                                dw = half_bits_to_float(W[base + 8] >> 16);
#pragma unroll
                                for (int i = 0; i < 8; i++) q[i] = W[base + 9 + i];
                            }
                        } else if (KIND == TSM_Q4_0) {
                            const int base = 9 * (j >> 1);
                            unsigned nib[4];
                            if ((j & 1) == 0) {
                                dw = half_bits_to_float(W[base] & 0xffffu);
#pragma unroll
                                for (int i = 0; i < 4; i++) nib[i] = __byte_perm(W[base + i], W[base + i + 1], 0x5432);
                            } else {
                                dw = half_bits_to_float(W[base + 4] >> 16);
#pragma unroll
                                for (int i = 0; i < 4; i++) nib[i] = W[base + 5 + i];
                            }
#pragma unroll
                            for (int i = 0; i < 4; i++) q[i] = nib[i] & 0x0f0f0f0fu, q[4 + i] = nib[i] & 0xf0f0f0f0u;
                        } else {
                            const int base = 5 * j;
                            dw = half_bits_to_float(W[base] & 0xffffu);
                            mw = half_bits_to_float(W[base] >> 16);
#pragma unroll
                            for (int i = 0; i < 4; i++) q[i] = W[base + 1 + i] & 0x0f0f0f0fu, q[4 + i] = W[base + 1 + i] & 0xf0f0f0f0u;
                        }
#pragma unroll
                        for (int c = 0; c < C; c++) {
                            const uint4* ap = ALIGNED ? (const uint4*)(acts_q + c * act_bytes + act_offset(kb)) + 2 * j
                                                      : (const uint4*)(acts_q + c * act_bytes + act_offset(kbj));
                            uint4 a0, a1;
                            if (KEPT) {
                                a0 = make_uint4(kept_q[8 * j], kept_q[8 * j + 1], kept_q[8 * j + 2], kept_q[8 * j + 3]);
                                a1 = make_uint4(kept_q[8 * j + 4], kept_q[8 * j + 5], kept_q[8 * j + 6], kept_q[8 * j + 7]);
                            } else {
                                a0 = ap[0], a1 = ap[1];
                            }
                            int total;
                            if (KIND == TSM_Q8_0) {
                                total = __dp4a((int)q[0], (int)a0.x, 0);
                                total = __dp4a((int)q[1], (int)a0.y, total);
                                total = __dp4a((int)q[2], (int)a0.z, total);
                                total = __dp4a((int)q[3], (int)a0.w, total);
                                total = __dp4a((int)q[4], (int)a1.x, total);
                                total = __dp4a((int)q[5], (int)a1.y, total);
                                total = __dp4a((int)q[6], (int)a1.z, total);
                                total = __dp4a((int)q[7], (int)a1.w, total);
                            } else {
                                // low nibbles as they are; high nibbles as unsigned bytes worth 16 each, divided out after
                                int low = __dp4a((int)q[0], (int)a0.x, 0);
                                low = __dp4a((int)q[1], (int)a0.y, low);
                                low = __dp4a((int)q[2], (int)a0.z, low);
                                low = __dp4a((int)q[3], (int)a0.w, low);
                                int high = dp4a_us(q[4], (int)a1.x, 0);
                                high = dp4a_us(q[5], (int)a1.y, high);
                                high = dp4a_us(q[6], (int)a1.z, high);
                                high = dp4a_us(q[7], (int)a1.w, high);
                                total = low + (high >> 4);
                            }
                            float dx = ALIGNED ? dxs[c][j] : acts_scale[c * nb + kbj];
                            float contribution;
                            if (KIND == TSM_Q8_0) {
                                contribution = __fmul_rn((float)total, __fmul_rn(dw, dx));
                            } else if (KIND == TSM_Q4_0) {
                                int xt = ALIGNED ? __float_as_int(auxs[c][j]) : ((const int*)acts_aux)[c * nb + kbj];
                                contribution = __fmul_rn(__fmul_rn((float)(total - 8 * xt), dw), dx);
                            } else {
                                float sx = ALIGNED ? auxs[c][j] : acts_aux[c * nb + kbj];
                                contribution = __fadd_rn(__fmul_rn(__fmul_rn(dw, dx), (float)total), __fmul_rn(mw, sx));
                            }
                            dst[c * pcap + j] = contribution;
                        }
                    }
                }
            }
        } else if (have_prev && S > 1) {
            // the previous pass's piece: lane i adds row i's nbs contributions onto its running sums
            const float* old = parts + ((it - 1) & 1) * C * pcap;
            const int r = prev_r0 + lane;
            if (r < prev_r1) {
                if (prev_seg == 0) {
#pragma unroll
                    for (int c = 0; c < C; c++) run[c] = 0.0f;
                }
                const int at = lane * nbs;
                for (int b = 0; b < nbs; b += 8) {   // nbs is a multiple of 8: 8 consecutive blocks never straddle a pad word
                    float v[C][8];
                    const float* src = old + part_index(at + b);
#pragma unroll
                    for (int u = 0; u < 8; u++)
#pragma unroll
                        for (int c = 0; c < C; c++) v[c][u] = src[c * pcap + u];
#pragma unroll
                    for (int u = 0; u < 8; u++)
#pragma unroll
                        for (int c = 0; c < C; c++) run[c] = __fadd_rn(run[c], v[c][u]);
                }
                if (prev_seg == S - 1) {
#pragma unroll
                    for (int c = 0; c < C; c++) {
                        float v = run[c];
                        if (p.bias) v = __fadd_rn(v, p.bias[r]);
                        if (p.residual) v = __fadd_rn(p.residual[(int64_t)c * p.n + r], v);
                        p.out[(int64_t)c * p.n + r] = v;
                    }
                }
            }
        } else if (have_prev) {
            // fold the previous tile: lane per row, each row's blocks in order from 0f
            const float* old = parts + ((it - 1) & 1) * C * pcap;
            for (int r = prev_r0 + lane; r < prev_r1; r += 32) {
                int at = prev_base + (r - prev_r0) * nb;
                float sum[C];
#pragma unroll
                for (int c = 0; c < C; c++) sum[c] = 0.0f;
                // loads run ahead of the adds: 8 contributions are fetched, then folded in order
                int b = 0;
                for (; b + 8 <= nb; b += 8) {
                    float v[C][8];
                    // when rows hold a multiple of 8 blocks, 8 consecutive blocks never straddle a pad word
                    const float* src = old + part_index(at + b);
#pragma unroll
                    for (int u = 0; u < 8; u++) {
                        int idx = part_index(at + b + u);
#pragma unroll
                        for (int c = 0; c < C; c++) v[c][u] = ALIGNED ? src[c * pcap + u] : old[c * pcap + idx];
                    }
#pragma unroll
                    for (int u = 0; u < 8; u++)
#pragma unroll
                        for (int c = 0; c < C; c++) sum[c] = __fadd_rn(sum[c], v[c][u]);
                }
                for (; b < nb; b++) {
                    int idx = part_index(at + b);
#pragma unroll
                    for (int c = 0; c < C; c++) sum[c] = __fadd_rn(sum[c], old[c * pcap + idx]);
                }
#pragma unroll
                for (int c = 0; c < C; c++) {
                    float v = sum[c];
                    if (p.bias) v = __fadd_rn(v, p.bias[r]);
                    if (p.residual) v = __fadd_rn(p.residual[(int64_t)c * p.n + r], v);
                    p.out[(int64_t)c * p.n + r] = v;
                }
            }
        }
        __syncthreads();
        if (*abort_flag) break;
        if (!valid) break;
        have_prev = true;
        prev_r0 = r0, prev_r1 = r1, prev_seg = seg;
        if (S > 1 && ++seg == S) seg = 0, row_tile += gridDim.x;
        prev_base = (int)((int64_t)r0 * nb - g0 * F::G);
        if (producer) issue(it + kStages);
    }
    if (*abort_flag && tid == 0) {
        atomicExch(&p.errors->timeout, 1);
        // give copies still in flight a bounded chance to land before the shared memory is released
        for (int s = 0; s < kStages; s++) mbar_wait(&full[s], 0), mbar_wait(&full[s], 1);
    }
}

// ---- generic kernel ------------------------------------------------------------------------------

__device__ __forceinline__ unsigned load_u32_2(const uint8_t* p) {  // p is 2-byte aligned
    const unsigned short* h = (const unsigned short*)p;
    return (unsigned)h[0] | ((unsigned)h[1] << 16);
}

template <int KIND>
__global__ void matvec_generic_kernel(const uint8_t* __restrict__ w, int n, int nb, QuantizedActs acts, int rows,
                                      const float* __restrict__ bias, const float* __restrict__ residual, float* out) {
    chained_kernel_entry();
    constexpr int B = Fmt<KIND>::B;
    int lane = threadIdx.x & 31;
    int64_t col = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (col >= n) return;
    const uint8_t* wrow = w + col * (int64_t)nb * B;
    for (int row = 0; row < rows; row++) {
        const int8_t* qs = acts.qs + (int64_t)row * nb * 32;
        float sum = 0.0f;
        for (int start = 0; start < nb; start += 32) {
            int block = start + lane;
            float contribution = 0.0f;
            if (block < nb) {
                const uint8_t* blk = wrow + (int64_t)block * B;
                const int* a = (const int*)(qs + block * 32);
                float dw = half_bits_to_float(*(const unsigned short*)blk);
                float dx = acts.scales[(int64_t)row * nb + block];
                int total = 0;
                if (KIND == TSM_Q8_0) {
#pragma unroll
                    for (int i = 0; i < 8; i++) total = __dp4a((int)load_u32_2(blk + 2 + 4 * i), a[i], total);
                    contribution = __fmul_rn((float)total, __fmul_rn(dw, dx));
                } else {
                    const uint8_t* packed = blk + (KIND == TSM_Q4_0 ? 2 : 4);
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        unsigned word = load_u32_2(packed + 4 * i);
                        total = __dp4a((int)(word & 0x0f0f0f0fu), a[i], total);
                        total = __dp4a((int)((word >> 4) & 0x0f0f0f0fu), a[4 + i], total);
                    }
                    if (KIND == TSM_Q4_0) {
                        int xt = 0;
#pragma unroll
                        for (int i = 0; i < 8; i++) xt = __dp4a(0x01010101, a[i], xt);
                        contribution = __fmul_rn(__fmul_rn((float)(total - 8 * xt), dw), dx);
                    } else {
                        float mw = half_bits_to_float(*(const unsigned short*)(blk + 2));
                        float sx = acts.sums[(int64_t)row * nb + block];
                        contribution = __fadd_rn(__fmul_rn(__fmul_rn(dw, dx), (float)total), __fmul_rn(mw, sx));
                    }
                }
            }
            int run = min(32, nb - start);
            for (int j = 0; j < run; j++) sum = __fadd_rn(sum, __shfl_sync(0xffffffffu, contribution, j));
        }
        if (lane == 0) {
            float v = sum;
            if (bias) v = __fadd_rn(v, bias[col]);
            if (residual) v = __fadd_rn(residual[(int64_t)row * n + col], v);
            out[(int64_t)row * n + col] = v;
        }
    }
}

// ---- host side -----------------------------------------------------------------------------------

template <int KIND, int C>
static size_t stream_smem_bytes(int nb, int cap, int stages) {
    using F = Fmt<KIND>;
    size_t act_bytes = (size_t)((act_offset(nb) + 15) & ~15);
    size_t pcap = (size_t)(part_index(cap * F::G) + 1);
    size_t bytes = 128 + C * act_bytes + (size_t)2 * C * nb * 4 + 2 * C * pcap * 4;
    bytes = (bytes + 127) & ~(size_t)127;
    return bytes + (size_t)stages * cap * F::GB;
}

template <int KIND, int C>
static int launch_stream(tsm_ctx* ctx, const QuantizedActs& a, const float* plain, int64_t plain_stride, int k, const uint8_t* w, int n, const float* bias,
                         const float* residual, float* out, bool* taken) {
    using F = Fmt<KIND>;
    *taken = false;
    int nb = k / 32;
    if (((uintptr_t)w & 15) != 0 || ((int64_t)n * nb) % F::G != 0) return TSM_OK;
    if (!plain && ((uintptr_t)a.qs & 15) != 0) return TSM_OK;
    if (nb < F::G) return TSM_OK;  // rows shorter than a group: the generic kernel takes them
    // A stage holds `cap` groups.  Short rows: 128 groups (one per compute thread).  Long rows: 256 groups, so
    // that a tile still holds several rows for the fold warp to fold side by side.
    int per_thread = F::CAP / 128;  // groups per thread of the small configuration (Q4_1's groups are half as large)
    bool long_rows = nb / F::G > 32 * per_thread;
    bool aligned = nb % F::G == 0;
    // Long rows in pieces (see the kernel): the fewest pieces of at most 128 blocks that are whole groups and multiples of 8
    // blocks, as many rows per tile as give every CTA slot one row tile, at most 32 (a fold lane per row) and a stage's worth.
    static const bool whole_rows = getenv("TSM_MATVEC_WHOLE_ROWS") != nullptr;   // whole-row tiles for long rows too, for timing them
    int segments = 1;
    // Pieces of at most 128 blocks; for Q8_0 and Q4_1 of at most 64 when no more than 8 (Q4_1: 16) such pieces make a row.
    // Measured on 4096 x 14336: eight pieces of 56 blocks instead of four of 112 took Q8_0 from 25.7 to 21.6 us and Q4_1 from
    // 23.6 to 19.8, Q4_0 from 17.6 to 19.7; on 4096 x 28672 sixteen pieces of 56 took Q4_1 from 42.3 to 34.2 and Q8_0 from
    // 42.8 to 58.8.
    static const int env_pieces = getenv("TSM_MATVEC_PIECES") ? atoi(getenv("TSM_MATVEC_PIECES")) : 0;   // start the search at this many pieces
    bool small_pieces = false;
    if (long_rows && aligned && !whole_rows) {
        auto search = [&](int first, int last, int piece_most) {
            for (int pieces = first; pieces <= last && segments == 1; pieces *= 2) {
                int nbs = nb / pieces;
                if (nb % pieces == 0 && nbs % 8 == 0 && nbs % F::G == 0 && nbs <= piece_most) segments = pieces;
            }
        };
        if (env_pieces > 0) {
            search(env_pieces, 16, 128);
        } else {
            if (KIND != TSM_Q4_0) search(2, KIND == TSM_Q8_0 ? 8 : 16, 64);
            small_pieces = segments > 1;
            search(2, 16, 128);
        }
    }
    // One row of activations whose length divides a sweep of the compute threads: the activations stay in registers (mode 3 of
    // the kernel).  TSM_MATVEC_KEPT=0 turns the mode off, for timing the two against each other.
    static const bool kept_on = !(getenv("TSM_MATVEC_KEPT") && atoi(getenv("TSM_MATVEC_KEPT")) == 0);
    const int sweep = kComputeThreads * (KIND == TSM_Q4_0 ? 4 : F::G);   // Q4_0: a thread takes half a group there
    const bool kept = C == 1 && kept_on && aligned && segments == 1 && sweep % nb == 0;
    static const int env_long_cap = getenv("TSM_MATVEC_LONG_CAP") ? atoi(getenv("TSM_MATVEC_LONG_CAP")) : 0;   // long rows' stage, in halves of the default short one
    // rows in pieces: the stage that measured fastest with them (same shape): the short rows' for Q8_0, half as much again for Q4_1
    const int long_cap = !small_pieces ? 2 * F::CAP : KIND == TSM_Q8_0 ? F::CAP : F::CAP * 3 / 2;
    int cap = long_rows ? (env_long_cap >= 2 && env_long_cap <= 6 ? F::CAP * env_long_cap / 2 : long_cap) : F::CAP, stages = 2;  // two stages measured faster than three: more CTAs fit an SM
    if (kept && KIND == TSM_Q4_0 && !long_rows) cap = F::CAP * 6 / 4;   // three half-group sweeps per stage measured fastest (49 against 54 us for 128256 x 4096)
    // TSM_MATVEC_CAP / TSM_MATVEC_STAGES override the tile size (in units of the format's default) and ring depth, so
    // that variants can be timed without rebuilding (as TENSOMITE_BLOCK_MATMUL does in the reference, quant.cr:36-41)
    static const int env_cap = getenv("TSM_MATVEC_CAP") ? atoi(getenv("TSM_MATVEC_CAP")) : 0;
    static const int env_stages = getenv("TSM_MATVEC_STAGES") ? atoi(getenv("TSM_MATVEC_STAGES")) : 0;
    if (env_cap > 0 && !long_rows) cap = F::CAP * env_cap / 4;  // quarters of the default
    if (env_stages >= 1 && env_stages <= 4) stages = env_stages;
    int max_rows = ((cap - 2) * F::G) / nb;   // (filling a stage to the last group with rows of whole groups measured no faster)
    if (max_rows < 1) return TSM_OK;
    size_t smem = stream_smem_bytes<KIND, C>(nb, cap, stages);
    if (smem > 200 * 1024) return TSM_OK;
    auto kernel = segments > 1 ? matvec_stream_kernel<KIND, C, 2> : aligned ? matvec_stream_kernel<KIND, C, 1> : matvec_stream_kernel<KIND, C, 0>;
    if constexpr (C == 1) {
        if (kept) kernel = matvec_stream_kernel<KIND, C, 3>;
    }
    static std::mutex attr_lock;  // the attribute is per device and per function
    static std::map<std::pair<int, const void*>, size_t> attr_set;
    {
        std::lock_guard<std::mutex> guard(attr_lock);
        auto key = std::make_pair(ctx->ordinal, (const void*)kernel);
        auto found = attr_set.find(key);
        if (found == attr_set.end()) {
            TSM_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            attr_set[key] = 200 * 1024;
        }
    }
    int per_sm = 0;
    TSM_CUDA(ctx, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, smem));
    if (per_sm < 1) return TSM_OK;
    int slots = per_sm * ctx->sm_count;
    if (segments > 1) {
        const int gps = nb / segments / F::G;
        const int most = std::min(32, cap / gps);
        int rows_per_tile = std::max(1, std::min(most, (n + slots - 1) / slots));
        int tiles = (n + rows_per_tile - 1) / rows_per_tile;
        int grid = std::min(tiles, slots);
        MatvecParams p;
        p.w = w, p.n = n, p.nb = nb, p.acts = a, p.bias = bias, p.residual = residual, p.out = out;
        p.rows_per_tile = rows_per_tile, p.num_tiles = tiles, p.errors = ctx->errors;
        p.cap = cap, p.stages = stages, p.segments = segments, p.seg_blocks = nb / segments, p.seg_groups = gps;
        p.nb_magic = (unsigned)((1ull << 32) / (unsigned)nb) + 1u;
        p.plain = plain, p.plain_stride = plain_stride;
        p.plain_vector = plain && ((uintptr_t)plain & 15) == 0 && plain_stride % 4 == 0;
        TSM_CUDA(ctx, launch_chained(ctx, kernel, dim3(grid), dim3(kThreads), smem, p));
        count_launch(ctx);
        TSM_LAUNCH_CHECK(ctx);
        *taken = true;
        return TSM_OK;
    }
    int tiles = (n + max_rows - 1) / max_rows;
    if (tiles < ctx->sm_count) {
        // a small matrix: full tiles would leave most SMs without work, and the kernel's time is then one CTA's latency
        // chain over many rows; tiles of a few rows (at least 4) give every SM one
        int few = std::max(4, (n + ctx->sm_count - 1) / ctx->sm_count);
        if (few < max_rows) max_rows = few, tiles = (n + max_rows - 1) / max_rows;
    }
    int grid = tiles < slots ? tiles : slots;
    int per_cta = (tiles + grid - 1) / grid;
    int rows_per_tile = (n + grid * per_cta - 1) / (grid * per_cta);
    if (rows_per_tile > max_rows) rows_per_tile = max_rows;
    if (rows_per_tile < 1) rows_per_tile = 1;
    tiles = (n + rows_per_tile - 1) / rows_per_tile;
    if (grid > tiles) grid = tiles;
    MatvecParams p;
    p.w = w, p.n = n, p.nb = nb, p.acts = a, p.bias = bias, p.residual = residual, p.out = out;
    p.rows_per_tile = rows_per_tile, p.num_tiles = tiles, p.errors = ctx->errors;
    p.cap = cap, p.stages = stages, p.segments = 1, p.seg_blocks = nb, p.seg_groups = nb / F::G;
    p.nb_magic = (unsigned)((1ull << 32) / (unsigned)nb) + 1u;
    p.plain = plain, p.plain_stride = plain_stride;
    p.plain_vector = plain && ((uintptr_t)plain & 15) == 0 && plain_stride % 4 == 0;
    TSM_CUDA(ctx, launch_chained(ctx, kernel, dim3(grid), dim3(kThreads), smem, p));
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    *taken = true;
    return TSM_OK;
}

template <int KIND>
static int launch_kind(tsm_ctx* ctx, const QuantizedActs& a, int rows, int k, const uint8_t* w, int n, const float* bias,
                       const float* residual, float* out) {
    bool taken = false;
    if (rows == 1) TSM_TRY((launch_stream<KIND, 1>(ctx, a, nullptr, 0, k, w, n, bias, residual, out, &taken)));
    else if (rows == 2) TSM_TRY((launch_stream<KIND, 2>(ctx, a, nullptr, 0, k, w, n, bias, residual, out, &taken)));
    else if (rows == 3) TSM_TRY((launch_stream<KIND, 3>(ctx, a, nullptr, 0, k, w, n, bias, residual, out, &taken)));
    else if (rows == 4) TSM_TRY((launch_stream<KIND, 4>(ctx, a, nullptr, 0, k, w, n, bias, residual, out, &taken)));
    if (taken) return TSM_OK;
    if (rows == 1 && k >= 32) {
        // One row of activations and a matrix that is not a whole number of groups (GPT-2's 50257 x 1600 vocabulary head): the
        // streamed kernel takes the rows up to the last whole group, the generic kernel the few that are left (it alone took
        // 49 us for that head, the streamed kernel 20 us for 50256 of its rows).
        using F = Fmt<KIND>;
        const int nb = k / 32;
        int unit = F::G;   // rows that make a whole number of groups: G / gcd(nb, G)
        for (int d = F::G; d >= 1; d /= 2)
            if (nb % d == 0) { unit = F::G / d; break; }
        const int main = n - n % unit;
        if (main >= 1024 && main < n) {
            TSM_TRY((launch_stream<KIND, 1>(ctx, a, nullptr, 0, k, w, main, bias, residual, out, &taken)));
            if (taken) {
                const int left = n - main;
                TSM_CUDA(ctx, launch_chained(ctx, matvec_generic_kernel<KIND>, dim3((unsigned)((left + 3) / 4)), dim3(128), 0,
                                             w + (int64_t)main * nb * F::B, left, nb, a, 1, bias ? bias + main : (const float*)nullptr,
                                             residual ? residual + main : (const float*)nullptr, out + main));
                count_launch(ctx);
                TSM_LAUNCH_CHECK(ctx);
                return TSM_OK;
            }
        }
    }
    if (rows > 4 && umma_product_fits(a, rows, k, w, KIND, n)) return launch_block_matmul_umma(ctx, a, rows, k, w, KIND, n, bias, residual, out);
    if (rows > 4 && pipe_product_fits(a, rows, k, w, KIND, n)) return launch_block_matmul_pipe(ctx, a, rows, k, w, KIND, n, bias, residual, out);
    if (rows > 4 && mma_product_fits(a, rows, k, w, KIND, n)) return launch_block_matmul_mma(ctx, a, rows, k, w, KIND, n, bias, residual, out);
    int nb = k / 32;
    int64_t grid = ((int64_t)n + 3) / 4;
    TSM_CUDA(ctx, launch_chained(ctx, matvec_generic_kernel<KIND>, dim3((unsigned)grid), dim3(128), 0, w, n, nb, a, rows, bias, residual, out));
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

template <int KIND>
static int launch_plain_kind(tsm_ctx* ctx, const float* x, int64_t x_stride, int rows, int k, const uint8_t* w, int n, const float* bias,
                             const float* residual, float* out, bool* taken) {
    QuantizedActs none{nullptr, nullptr, nullptr, nullptr};
    switch (rows) {
        case 1: return launch_stream<KIND, 1>(ctx, none, x, x_stride, k, w, n, bias, residual, out, taken);
        case 2: return launch_stream<KIND, 2>(ctx, none, x, x_stride, k, w, n, bias, residual, out, taken);
        case 3: return launch_stream<KIND, 3>(ctx, none, x, x_stride, k, w, n, bias, residual, out, taken);
        case 4: return launch_stream<KIND, 4>(ctx, none, x, x_stride, k, w, n, bias, residual, out, taken);
    }
    return TSM_OK;
}

int launch_block_matvec_plain(tsm_ctx* ctx, const float* x, int64_t x_stride, int rows, int k, const uint8_t* w, int kind, int n,
                              const float* bias, const float* residual, float* out, bool* taken) {
    *taken = false;
    static const bool off = getenv("TSM_SEPARATE_QUANTISER") != nullptr;  // time the two launches instead
    if (off || rows < 1 || rows > 4 || n == 0 || k <= 0 || k % 32 != 0 || ((uintptr_t)w & 1) != 0) return TSM_OK;
    OpTimer timer(ctx, kind == TSM_Q8_0 ? "BlockMatMul q8_0" : kind == TSM_Q4_0 ? "BlockMatMul q4_0" : "BlockMatMul q4_1", rows, k, n);
    int rc = TSM_OK;
    switch (kind) {
        case TSM_Q8_0: rc = launch_plain_kind<TSM_Q8_0>(ctx, x, x_stride, rows, k, w, n, bias, residual, out, taken); break;
        case TSM_Q4_0: rc = launch_plain_kind<TSM_Q4_0>(ctx, x, x_stride, rows, k, w, n, bias, residual, out, taken); break;
        case TSM_Q4_1: rc = launch_plain_kind<TSM_Q4_1>(ctx, x, x_stride, rows, k, w, n, bias, residual, out, taken); break;
    }
    timer.dropped = !*taken;
    return rc;
}

int launch_block_matmul(tsm_ctx* ctx, const QuantizedActs& a, int rows, int k, const uint8_t* w, int kind, int n,
                        const float* bias, const float* residual, float* out) {
    OpTimer timer(ctx, kind == TSM_Q8_0 ? "BlockMatMul q8_0" : kind == TSM_Q4_0 ? "BlockMatMul q4_0" : "BlockMatMul q4_1", rows, k, n);
    if (k <= 0 || k % 32 != 0) return fail(ctx, TSM_ERR_ARG, "rows of " + std::to_string(k) + " do not split into blocks of 32");
    if (((uintptr_t)w & 1) != 0) return fail(ctx, TSM_ERR_ARG, "block weights must start at an even address");
    if (rows == 0 || n == 0) return TSM_OK;
    switch (kind) {
        case TSM_Q8_0: return launch_kind<TSM_Q8_0>(ctx, a, rows, k, w, n, bias, residual, out);
        case TSM_Q4_0: return launch_kind<TSM_Q4_0>(ctx, a, rows, k, w, n, bias, residual, out);
        case TSM_Q4_1: return launch_kind<TSM_Q4_1>(ctx, a, rows, k, w, n, bias, residual, out);
    }
    return fail(ctx, TSM_ERR_UNSUPPORTED, "not a block format");
}

}  // namespace tsm
