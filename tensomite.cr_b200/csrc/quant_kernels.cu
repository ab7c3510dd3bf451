// Block-format kernels: the activation quantiser, the weight quantisers and dequantisers, the
// embedding gather and the seeded normal fill used to make synthetic models on the device.
#include "common.cuh"

namespace tsm {

// ---- activation quantiser (quantize_block_q8 in common.cuh): one warp per block of 32 -------------
__global__ void quantize_rows_kernel(const float* __restrict__ x, int rows, int k, int64_t x_stride, float* scales,
                                     float* sums, int* totals, int8_t* qs) {
    chained_kernel_entry();
    int lane = threadIdx.x & 31;
    int64_t warp = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int nb = k >> 5;
    int64_t blocks = (int64_t)rows * nb;
    if (warp >= blocks) return;
    int row = (int)(warp / nb), block = (int)(warp % nb);
    float v = x[(int64_t)row * x_stride + block * 32 + lane];
    quantize_block_q8(v, lane, scales + warp, sums + warp, totals + warp, qs + (int64_t)row * k + block * 32 + lane);
}

int64_t quant_scratch_bytes(int rows, int k) {
    int64_t blocks = (int64_t)rows * (k / 32);
    int64_t bytes = (blocks * 12 + 255) / 256 * 256 + (int64_t)rows * k;
    return (bytes + 255) / 256 * 256;
}

QuantizedActs quant_scratch_layout(void* base, int rows, int k) {
    int64_t blocks = (int64_t)rows * (k / 32);
    char* p = (char*)base;
    QuantizedActs a;
    a.scales = (const float*)p;
    a.sums = (const float*)(p + blocks * 4);
    a.totals = (const int*)(p + blocks * 8);
    a.qs = (const int8_t*)(p + (blocks * 12 + 255) / 256 * 256);  // 16-byte aligned for vector loads
    return a;
}

int launch_quantize_rows(tsm_ctx* ctx, const float* x, int rows, int k, int64_t x_stride, float* scales, float* sums,
                         int* totals, int8_t* qs) {
    OpTimer timer(ctx, "QuantizeRows", rows, k);
    if (k % 32 != 0 || rows < 0) return fail(ctx, TSM_ERR_ARG, "rows of " + std::to_string(k) + " do not split into blocks of 32");
    int64_t blocks = (int64_t)rows * (k / 32);
    if (blocks == 0) return TSM_OK;
    int64_t grid = (blocks + 7) / 8;
    TSM_CUDA(ctx, launch_chained(ctx, quantize_rows_kernel, dim3((unsigned)grid), dim3(256), 0, x, rows, k, x_stride, scales, sums, totals, qs));
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

// ---- weight quantisers (Quant.quantize, quant.cr:499-535): one warp per block ------------------

__global__ void quantize_blocks_kernel(const float* __restrict__ x, int64_t blocks, int kind, uint8_t* out) {
    int lane = threadIdx.x & 31;
    int64_t block = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (block >= blocks) return;
    float v = x[block * 32 + lane];
    const unsigned full = 0xffffffffu;
    if (kind == TSM_Q8_0) {
        uint8_t* t = out + block * 34;
        float amax = fabsf(v);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(full, amax, off));
        float d = __fdiv_rn(amax, 127.0f);
        float id = d == 0.0f ? 0.0f : __fdiv_rn(1.0f, d);
        t[2 + lane] = (uint8_t)(signed char)(int)roundf(__fmul_rn(v, id));
        if (lane == 0) *(__half*)t = __float2half_rn(d);
        return;
    }
    if (kind == TSM_Q4_0) {
        uint8_t* t = out + block * 18;
        // the value of largest magnitude, the first of equals (quant.cr:510-511)
        float best = v;
        int at = lane;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            float other = __shfl_xor_sync(full, best, off);
            int other_at = __shfl_xor_sync(full, at, off);
            bool take = fabsf(other) > fabsf(best) || (fabsf(other) == fabsf(best) && other_at < at);
            best = take ? other : best;
            at = take ? other_at : at;
        }
        float d = __fdiv_rn(best, -8.0f);
        float id = d == 0.0f ? 0.0f : __fdiv_rn(1.0f, d);
        int q = (int)(signed char)(int)__fadd_rn(__fmul_rn(v, id), 8.5f);
        q = q > 15 ? 15 : q;
        int high = __shfl_down_sync(full, q, 16);
        if (lane < 16) t[2 + lane] = (uint8_t)((q & 0xff) | ((high & 0xff) << 4));
        if (lane == 0) *(__half*)t = __float2half_rn(d);
        return;
    }
    uint8_t* t = out + block * 20;
    float lo = v, hi = v;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(full, lo, off));
        hi = fmaxf(hi, __shfl_xor_sync(full, hi, off));
    }
    float d = __fdiv_rn(__fsub_rn(hi, lo), 15.0f);
    float id = d == 0.0f ? 0.0f : __fdiv_rn(1.0f, d);
    int q = (int)(signed char)(int)__fadd_rn(__fmul_rn(__fsub_rn(v, lo), id), 0.5f);
    q = q > 15 ? 15 : q;
    int high = __shfl_down_sync(full, q, 16);
    if (lane < 16) t[4 + lane] = (uint8_t)((q & 0xff) | ((high & 0xff) << 4));
    if (lane == 0) {
        ((__half*)t)[0] = __float2half_rn(d);
        ((__half*)t)[1] = __float2half_rn(lo);
    }
}

int launch_quantize_blocks(tsm_ctx* ctx, const float* x, int64_t count, int kind, uint8_t* out) {
    OpTimer timer(ctx, "Quantize", count);
    if (count % 32 != 0) return fail(ctx, TSM_ERR_ARG, std::to_string(count) + " values do not split into blocks of 32");
    if (kind < 0 || kind > 2) return fail(ctx, TSM_ERR_UNSUPPORTED, "not a block format");
    int64_t blocks = count / 32;
    if (blocks == 0) return TSM_OK;
    quantize_blocks_kernel<<<(unsigned)((blocks + 7) / 8), 256, 0, ctx->stream>>>(x, blocks, kind, out);
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

// Element j of a row of blocks (block_value, kernels.cu:1160-1168; Quant.dequantize_*, quant.cr:537-556).
__device__ __forceinline__ float block_element(const uint8_t* row, int kind, int j) {
    int b = j >> 5, at = j & 31;
    if (kind == TSM_Q8_0) {
        const uint8_t* blk = row + b * 34;
        float d = half_bits_to_float(blk[0] | (blk[1] << 8));
        return __fmul_rn((float)(signed char)blk[2 + at], d);
    }
    if (kind == TSM_Q4_0) {
        const uint8_t* blk = row + b * 18;
        float d = half_bits_to_float(blk[0] | (blk[1] << 8));
        unsigned packed = blk[2 + (at & 15)];
        int q = at < 16 ? (packed & 0x0f) : (packed >> 4);
        return __fmul_rn((float)(q - 8), d);
    }
    const uint8_t* blk = row + b * 20;
    float d = half_bits_to_float(blk[0] | (blk[1] << 8));
    float m = half_bits_to_float(blk[2] | (blk[3] << 8));
    unsigned packed = blk[4 + (at & 15)];
    int q = at < 16 ? (packed & 0x0f) : (packed >> 4);
    return __fadd_rn(__fmul_rn(d, (float)q), m);
}

__global__ void dequantize_blocks_kernel(const uint8_t* __restrict__ blocks, int64_t count, int kind, float* out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    int bb = kind == TSM_Q8_0 ? 34 : kind == TSM_Q4_0 ? 18 : 20;
    out[i] = block_element(blocks + (i >> 5) * bb, kind, (int)(i & 31));
}

int launch_dequantize_blocks(tsm_ctx* ctx, const uint8_t* blocks, int64_t count, int kind, float* out) {
    OpTimer timer(ctx, "Dequantize", count);
    if (count % 32 != 0) return fail(ctx, TSM_ERR_ARG, std::to_string(count) + " values do not split into blocks of 32");
    if (kind < 0 || kind > 2) return fail(ctx, TSM_ERR_UNSUPPORTED, "not a block format");
    if (count == 0) return TSM_OK;
    dequantize_blocks_kernel<<<(unsigned)((count + 255) / 256), 256, 0, ctx->stream>>>(blocks, count, kind, out);
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

// Embedding lookup (gather_blocks_f32, kernels.cu:1172-1185).  With a second table (GPT-2's positions,
// gpt2.cr:189-191) the two dequantised rows are added: wte[id] + wpe[position].
__global__ void gather_blocks_kernel(const uint8_t* __restrict__ table, int kind, int table_rows, int width,
                                     const int* __restrict__ ids, int64_t total, float* out, ErrorRecord* errors,
                                     const uint8_t* __restrict__ table2, const int* __restrict__ ids2, int ids2_stride) {
    chained_kernel_entry();
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    int token = (int)(i / width), col = (int)(i % width);
    int id = ids[token];
    if (id < 0 || id >= table_rows) {
        if (col == 0) report_bad_index(errors, id, table_rows);
        out[i] = 0.0f;
        return;
    }
    int bb = kind == TSM_Q8_0 ? 34 : kind == TSM_Q4_0 ? 18 : 20;
    int64_t row_bytes = (int64_t)(width >> 5) * bb;
    float v = block_element(table + (int64_t)id * row_bytes, kind, col);
    if (table2) v = __fadd_rn(v, block_element(table2 + (int64_t)ids2[(int64_t)token * ids2_stride] * row_bytes, kind, col));
    out[i] = v;
}

int launch_gather_blocks(tsm_ctx* ctx, const uint8_t* table, int kind, int table_rows, int width, const int* ids,
                         int count, float* out, const uint8_t* table2, const int* ids2, int ids2_stride) {
    OpTimer timer(ctx, "Gather blocks", count, width);
    if (width % 32 != 0) return fail(ctx, TSM_ERR_ARG, "rows of " + std::to_string(width) + " do not split into blocks of 32");
    if (kind < 0 || kind > 2) return fail(ctx, TSM_ERR_UNSUPPORTED, "not a block format");
    int64_t total = (int64_t)count * width;
    if (total == 0) return TSM_OK;
    TSM_CUDA(ctx, launch_chained(ctx, gather_blocks_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, table, kind, table_rows, width, ids,
                                 total, out, ctx->errors, table2, ids2, ids2_stride));
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

__global__ void gather_f32_kernel(const float* __restrict__ table, int table_rows, int width, const int* __restrict__ ids,
                                  int64_t total, float* out, ErrorRecord* errors, const float* __restrict__ table2,
                                  const int* __restrict__ ids2, int ids2_stride) {
    chained_kernel_entry();
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    int token = (int)(i / width), col = (int)(i % width);
    int id = ids[token];
    if (id < 0 || id >= table_rows) {
        if (col == 0) report_bad_index(errors, id, table_rows);
        out[i] = 0.0f;
        return;
    }
    float v = table[(int64_t)id * width + col];
    if (table2) v = __fadd_rn(v, table2[(int64_t)ids2[(int64_t)token * ids2_stride] * width + col]);
    out[i] = v;
}

int launch_gather_f32(tsm_ctx* ctx, const float* table, int table_rows, int width, const int* ids, int count, float* out,
                      const float* table2, const int* ids2, int ids2_stride) {
    OpTimer timer(ctx, "Gather", count, width);
    int64_t total = (int64_t)count * width;
    if (total == 0) return TSM_OK;
    TSM_CUDA(ctx, launch_chained(ctx, gather_f32_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, table, table_rows, width, ids, total, out,
                                 ctx->errors, table2, ids2, ids2_stride));
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

// ---- seeded fills -------------------------------------------------------------------------------

__device__ __forceinline__ uint64_t splitmix64(uint64_t z) {
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

// N(mean, stddev) by Box-Muller on a counter-based generator: element pair i depends only on (seed, i).
__global__ void normal_fill_kernel(float* out, int64_t count, float mean, float stddev, uint64_t seed) {
    int64_t pair = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (pair * 2 >= count) return;
    uint64_t bits = splitmix64(seed * 0x2545f4914f6cdd1dull + (uint64_t)pair);
    float u1 = ((float)(uint32_t)(bits >> 40) + 1.0f) * (1.0f / 16777217.0f);
    float u2 = (float)(uint32_t)((bits >> 8) & 0xffffff) * (1.0f / 16777216.0f);
    float radius = sqrtf(-2.0f * logf(u1));
    float s, c;
    sincospif(2.0f * u2, &s, &c);
    out[pair * 2] = mean + stddev * radius * c;
    if (pair * 2 + 1 < count) out[pair * 2 + 1] = mean + stddev * radius * s;
}

int launch_normal_fill(tsm_ctx* ctx, float* out, int64_t count, float mean, float stddev, uint64_t seed) {
    OpTimer timer(ctx, "Fill normal", count);
    if (count == 0) return TSM_OK;
    int64_t pairs = (count + 1) / 2;
    normal_fill_kernel<<<(unsigned)((pairs + 255) / 256), 256, 0, ctx->stream>>>(out, count, mean, stddev, seed);
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

__global__ void fill_kernel(float* out, int64_t count, float value) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) out[i] = value;
}

int launch_fill(tsm_ctx* ctx, float* out, int64_t count, float value) {
    if (count == 0) return TSM_OK;
    fill_kernel<<<(unsigned)((count + 255) / 256), 256, 0, ctx->stream>>>(out, count, value);
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

}  // namespace tsm
