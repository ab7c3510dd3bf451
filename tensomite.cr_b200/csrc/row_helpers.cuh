// Device helpers shared by the kernels that fold a row's sum in the host's order (the norms, and the tensor-parallel
// exchange that ends in one).
#pragma once
#include "common.cuh"

namespace tsm {

// Σ f(row[j]) in index order from 0f, each step rounded (the host's fold, devices/host.cr:391-403,
// 348-361); every thread receives the result.  All threads first write the terms ((row[j] - shift)² or
// row[j]) to `terms`, padded to a multiple of 16 with +0 (adding +0 to a sum that started at +0 and only ever
// had such terms added never changes it: the running sum is never -0); one thread then folds them with
// 16-byte loads running ahead of the dependent adds, so a step costs the latency of one add.
template <bool SQUARE>
__device__ __forceinline__ float ordered_sum(const float* row, float* terms, int n, float shift, float* scratch) {
    const int padded = (n + 15) & ~15;
    for (int j = threadIdx.x; j < padded; j += blockDim.x) {
        float v = 0.0f;
        if (j < n) {
            v = SQUARE ? __fsub_rn(row[j], shift) : row[j];
            if (SQUARE) v = __fmul_rn(v, v);
        }
        terms[j] = v;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float acc = 0.0f;
        const float4* t4 = (const float4*)terms;
        float4 a = t4[0], b = t4[1], c = t4[2], d = t4[3];
        for (int j = 0; j < padded; j += 16) {
            float4 na = a, nb = b, nc = c, nd = d;
            if (j + 16 < padded) na = t4[(j >> 2) + 4], nb = t4[(j >> 2) + 5], nc = t4[(j >> 2) + 6], nd = t4[(j >> 2) + 7];
            acc = __fadd_rn(acc, a.x), acc = __fadd_rn(acc, a.y), acc = __fadd_rn(acc, a.z), acc = __fadd_rn(acc, a.w);
            acc = __fadd_rn(acc, b.x), acc = __fadd_rn(acc, b.y), acc = __fadd_rn(acc, b.z), acc = __fadd_rn(acc, b.w);
            acc = __fadd_rn(acc, c.x), acc = __fadd_rn(acc, c.y), acc = __fadd_rn(acc, c.z), acc = __fadd_rn(acc, c.w);
            acc = __fadd_rn(acc, d.x), acc = __fadd_rn(acc, d.y), acc = __fadd_rn(acc, d.z), acc = __fadd_rn(acc, d.w);
            a = na, b = nb, c = nc, d = nd;
        }
        scratch[0] = acc;
    }
    __syncthreads();
    return scratch[0];
}

// The same sum of squares, with the same bits, in about a third of the time.  A sequential float sum of NON-NEGATIVE terms is
// integer arithmetic for as long as the running sum s stays in one binade: s is then S ulps (2^23 <= S < 2^24) and adding a
// term t = m * 2^e moves it by floor(m / 2^shift) ulps, plus one if the bits shifted out are more than half an ulp
// (shift = exponent of s - exponent of t; a term below half an ulp adds nothing).  Integer additions may be made in any order,
// so the row is cut into chunks of 64 terms whose increments are summed by a warp each, under the exponent the running sum is
// PREDICTED to have when it reaches the chunk (from tree sums of the chunks before it).  One thread then walks the chunks with
// the exact running sum: where the prediction holds, no term of the chunk was a tie (bits shifted out exactly half an ulp: the
// rounding then depends on S's parity), was larger than an ulp of the next binade, infinite or NaN, and the sum stays inside
// the binade, the chunk costs one integer addition; otherwise its 64 terms are added one by one as before.  Every shortcut is
// checked against the exact running sum, so the result is the sequential sum's for any input; rows of normal activations take
// the slow way for about 9 of 64 chunks (the first ones, and those in which the sum crosses a power of two).
constexpr int kSumChunk = 64;
constexpr int kSumMaxChunks = 128;   // rows of up to 8192 terms; longer rows are folded term by term
struct SumScratch {
    float part[kSumMaxChunks];       // tree sum of each chunk, then the predicted running sum at its start
    int2 step[kSumMaxChunks];        // (predicted exponent or -1 when the chunk must be replayed, increment in ulps)
};

// `terms` [n] lie in shared memory, n a multiple of kSumChunk up to kSumChunk * kSumMaxChunks, every term >= 0 (or a NaN); the
// sum continues from `start` (the same in every thread); every thread of the CTA calls and receives the result.
__device__ __forceinline__ float chunked_sum_of_terms(const float* terms, int n, float start, float* scratch, SumScratch* ss) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int chunks = n / kSumChunk;
    // 1. a tree sum per chunk (any order: it only predicts an exponent)
    for (int c = warp; c < chunks; c += warps) {
        float2 t2 = ((const float2*)(terms + c * kSumChunk))[lane];
        float s = t2.x + t2.y;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
        if (lane == 0) ss->part[c] = s;
    }
    __syncthreads();
    // 2. the predicted running sum at each chunk's start: an exclusive scan by one warp, four chunks per lane
    if (warp == 0) {
        float mine[4], total = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int c = lane * 4 + i;
            mine[i] = c < chunks ? ss->part[c] : 0.0f;
            total += mine[i];
        }
        float before = total;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            float up = __shfl_up_sync(0xffffffffu, before, off);
            if (lane >= off) before += up;
        }
        before = before - total + start;   // what precedes this lane's chunks
#pragma unroll
        for (int i = 0; i < 4; i++) {
            int c = lane * 4 + i;
            if (c < chunks) ss->part[c] = before;
            before += mine[i];
        }
    }
    __syncthreads();
    // 3. every chunk's increment in ulps of its predicted binade
    for (int c = warp; c < chunks; c += warps) {
        const int E = (int)((__float_as_uint(ss->part[c]) >> 23) & 0xffu);
        float2 t2 = ((const float2*)(terms + c * kSumChunk))[lane];
        int inc = 0;
        bool bad = E == 0 || E == 255;
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const unsigned bits = __float_as_uint(k == 0 ? t2.x : t2.y);
            const int et = (int)((bits >> 23) & 0xffu);
            const unsigned man = bits & 0x7fffffu;
            const unsigned m = et == 0 ? man : (man | 0x800000u);
            const int sh = E - (et == 0 ? 1 : et);
            if ((bits >> 31) != 0 || et == 255 || (sh < 1 && m != 0)) bad = true;   // negative zero aside, terms are >= 0
            else if (m != 0 && sh <= 24) {
                const unsigned low = m & ((1u << sh) - 1u), half = 1u << (sh - 1);
                if (low == half) bad = true;
                inc += (int)(m >> sh) + (low > half ? 1 : 0);
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) inc += __shfl_xor_sync(0xffffffffu, inc, off);
        const bool any_bad = __any_sync(0xffffffffu, bad);
        if (lane == 0) ss->step[c] = make_int2(any_bad ? -1 : E, inc);
    }
    __syncthreads();
    // 4. one thread, the exact running sum
    if (threadIdx.x == 0) {
        unsigned ab = __float_as_uint(start);   // bits of the running sum
        int2 next = ss->step[0];
        for (int c = 0; c < chunks; c++) {
            const int2 st = next;
            if (c + 1 < chunks) next = ss->step[c + 1];
            const int Ea = (int)(ab >> 23);                      // the sign bit is clear unless the sum is a NaN: no match then
            const unsigned Sa = (ab & 0x7fffffu) | 0x800000u;
            if (st.x == Ea && Sa + (unsigned)st.y < (1u << 24)) {
                ab = ((unsigned)Ea << 23) | (Sa + (unsigned)st.y - 0x800000u);
            } else {
                float acc = __uint_as_float(ab);
                const float4* t4 = (const float4*)(terms + c * kSumChunk);
                float4 v[kSumChunk / 4];
#pragma unroll
                for (int i = 0; i < kSumChunk / 4; i++) v[i] = t4[i];
#pragma unroll
                for (int i = 0; i < kSumChunk / 4; i++) {
                    acc = __fadd_rn(acc, v[i].x), acc = __fadd_rn(acc, v[i].y), acc = __fadd_rn(acc, v[i].z), acc = __fadd_rn(acc, v[i].w);
                }
                ab = __float_as_uint(acc);
            }
        }
        scratch[0] = __uint_as_float(ab);
    }
    __syncthreads();
    return scratch[0];
}

// The sum of squares of a norm: the chunked form where it applies (`fast`, whole chunks, a block of at least four warps).
__device__ __forceinline__ float ordered_sum_squares(const float* row, float* terms, int n, float shift, float* scratch, SumScratch* ss, bool fast) {
    // (rows under 1024 terms are quicker term by term: the chunked form's four barriers cost more than the short chain)
    if (fast && n % kSumChunk == 0 && n >= 16 * kSumChunk && n <= kSumChunk * kSumMaxChunks && blockDim.x >= 128) {
        for (int j = threadIdx.x; j < n; j += blockDim.x) {
            float v = __fsub_rn(row[j], shift);
            terms[j] = __fmul_rn(v, v);
        }
        __syncthreads();
        return chunked_sum_of_terms(terms, n, 0.0f, scratch, ss);
    }
    return ordered_sum<true>(row, terms, n, shift, scratch);
}

// One THREAD quantises one block of 32 values that lie in shared memory (16-byte aligned; rows there are stored with 4 pad
// floats per block, so that threads on consecutive blocks read distinct banks), with quantize_block_q8's arithmetic: the
// maximum of 32 magnitudes in any order is the same number, the rest is element by element.  A row of 128 blocks costs the
// 128 threads about 600 cycles this way; one warp per block, eight blocks per warp one after the other, each with two chains
// of five shuffles, cost 3.2 us.  `vector`: q_out may be written in two 16-byte pieces.
__device__ __forceinline__ void quantize_block_by_thread(const float* y, float* scale, float* sum, int* total, int8_t* q_out, bool vector) {
    float v[32];
#pragma unroll
    for (int u = 0; u < 8; u++) {
        float4 t = ((const float4*)y)[u];
        v[4 * u] = t.x, v[4 * u + 1] = t.y, v[4 * u + 2] = t.z, v[4 * u + 3] = t.w;
    }
    float amax = fabsf(v[0]);
#pragma unroll
    for (int u = 1; u < 32; u++) amax = fmaxf(amax, fabsf(v[u]));
    float d = __fdiv_rn(amax, 127.0f);
    float id = d == 0.0f ? 0.0f : __fdiv_rn(1.0f, d);
    int t = 0;
    unsigned words[8];
#pragma unroll
    for (int u = 0; u < 8; u++) {
        unsigned word = 0;
#pragma unroll
        for (int e = 0; e < 4; e++) {
            int q = (int)(signed char)(int)roundf(__fmul_rn(v[4 * u + e], id));
            t += q;
            word |= (unsigned)(q & 0xff) << (8 * e);
        }
        words[u] = word;
    }
    if (vector) {
        ((uint4*)q_out)[0] = make_uint4(words[0], words[1], words[2], words[3]);
        ((uint4*)q_out)[1] = make_uint4(words[4], words[5], words[6], words[7]);
    } else {
#pragma unroll
        for (int u = 0; u < 32; u++) q_out[u] = (int8_t)(words[u >> 2] >> (8 * (u & 3)));
    }
    *scale = round_to_half(d);
    *sum = round_to_half(__fmul_rn((float)t, d));
    *total = t;
}

// One rotary pair (host.cr:448-466): x*cos + rotate_half(x)*sin, three roundings per element.
__device__ __forceinline__ void rotate_pair(float a, float b, const float* c, const float* s, int i, int half, float* oa,
                                            float* ob) {
    // a = x[i] (first half), b = x[i + half]
    *oa = __fadd_rn(__fmul_rn(a, c[i]), __fmul_rn(__fmul_rn(b, -1.0f), s[i]));
    *ob = __fadd_rn(__fmul_rn(b, c[i + half]), __fmul_rn(a, s[i + half]));
}

// kernels.cr:4,18 through the tape of kernel.cr:259-300: every step rounded on its own.
__device__ __forceinline__ float swiglu_value(float gate, float up) {
    float t1 = exact_exp(-gate);
    float t2 = __fadd_rn(t1, 1.0f);
    float t3 = __fdiv_rn(gate, t2);
    return __fmul_rn(t3, up);
}

__device__ __forceinline__ float gelu_value(float x) {
    const float c = 0.7978845608028654f;  // f32(sqrt(2 / pi))
    float t0 = __fmul_rn(x, 0.5f);
    float t1 = __fmul_rn(x, x);
    float t2 = __fmul_rn(t1, x);
    float t3 = __fmul_rn(t2, 0.044715f);
    float t4 = __fadd_rn(x, t3);
    float t5 = __fmul_rn(t4, c);
    float t6 = exact_tanh(t5);
    float t7 = __fadd_rn(t6, 1.0f);
    return __fmul_rn(t0, t7);
}

}  // namespace tsm
