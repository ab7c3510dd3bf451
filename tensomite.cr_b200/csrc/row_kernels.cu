// Row-wise and elementwise kernels of the decode step: RMSNorm, LayerNorm, RoPE, cache writes,
// SwiGLU, GELU, residual add, greedy argmax and top-k.  Norms and activations can also write their
// output already quantised for the product that follows (the quantiser of quant.cr:428-442), which
// removes the separate quantising launch the reference pays before every product.
#include "common.cuh"
#include "row_helpers.cuh"

namespace tsm {

struct QuantOut {
    float* scales;
    float* sums;
    int* totals;
    int8_t* qs;
};

static QuantOut quant_out(const QuantizedActs* q) {
    QuantOut o{nullptr, nullptr, nullptr, nullptr};
    if (q) o = QuantOut{(float*)q->scales, (float*)q->sums, (int*)q->totals, (int8_t*)q->qs};
    return o;
}

__device__ __forceinline__ float block_sum(float v, float* scratch) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.0f;
    for (int i = 0; i < warps; i++) total += scratch[i];
    return total;
}

// One CTA per row.  LAYER = false: x / sqrt(Σx²/n + eps) * w (rmsnorm_row, host.cr:391-403).
// LAYER = true: mean, centred, variance, c / std * w + b (host.cr:348-361).
template <bool LAYER>
__global__ void norm_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b, int n,
                            float eps, float* out, QuantOut q, int exact, int chunked_sum) {
    chained_kernel_entry();
    extern __shared__ __align__(16) float row[];  // [n], then the terms of the ordered sums, 16-byte aligned
    __shared__ float scratch[32];
    __shared__ SumScratch sum_scratch;
    float* terms = row + ((n + 3) & ~3);
    int r = blockIdx.x;
    const float* xr = x + (int64_t)r * n;
    // Rows of up to 8 values per thread: a thread keeps its values, and fetches their weights now, so that those loads are
    // in flight while one thread folds the ordered sums and nothing but arithmetic is left for afterwards.
    constexpr int kKeep = 8;
    const bool kept = n <= kKeep * (int)blockDim.x;
    float xv[kKeep], wv[kKeep], bv[kKeep];
    if (kept) {
#pragma unroll
        for (int i = 0; i < kKeep; i++) {
            int j = threadIdx.x + i * blockDim.x;
            bool in = j < n;
            xv[i] = in ? xr[j] : 0.0f;
            wv[i] = in && w ? w[j] : 1.0f;
            bv[i] = LAYER && in ? b[j] : 0.0f;
            if (in) row[j] = xv[i];
        }
    } else {
        for (int j = threadIdx.x; j < n; j += blockDim.x) row[j] = xr[j];
    }
    __syncthreads();
    float count = (float)n;
    float mean = 0.0f, denom;
    if (LAYER) {
        float total;
        if (exact) {
            total = ordered_sum<false>(row, terms, n, 0.0f, scratch);
        } else {
            float part = 0.0f;
            for (int j = threadIdx.x; j < n; j += blockDim.x) part += row[j];
            total = block_sum(part, scratch);
        }
        mean = __fdiv_rn(total, count);
    }
    float squares;
    if (exact) {
        squares = ordered_sum_squares(row, terms, n, mean, scratch, &sum_scratch, chunked_sum != 0);
    } else {
        float part = 0.0f;
        for (int j = threadIdx.x; j < n; j += blockDim.x) {
            float c = __fsub_rn(row[j], mean);
            part += c * c;
        }
        squares = block_sum(part, scratch);
    }
    denom = __fsqrt_rn(__fadd_rn(__fdiv_rn(squares, count), eps));
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    int blocks = (n + 31) >> 5;
    if (kept) {
        // the normed values go to shared memory (over the sums' terms, which are done with), then one thread per block
        // quantises them
        float* ybuf = terms;   // 36 floats per block of 32
#pragma unroll
        for (int i = 0; i < kKeep; i++) {
            int j = threadIdx.x + i * blockDim.x;
            if (j < n) {
                float c = LAYER ? __fsub_rn(xv[i], mean) : xv[i];
                float y = __fdiv_rn(c, denom);
                if (w) y = __fmul_rn(y, wv[i]);
                if (LAYER) y = __fadd_rn(y, bv[i]);
                if (out) out[(int64_t)r * n + j] = y;
                if (q.qs) ybuf[j + (j >> 5) * 4] = y;
            }
        }
        if (!q.qs) return;
        __syncthreads();
        const bool vector = (((uintptr_t)q.qs | (uintptr_t)n) & 15) == 0;
        for (int blk = threadIdx.x; blk < blocks; blk += blockDim.x) {
            int64_t at = (int64_t)r * (n >> 5) + blk;
            quantize_block_by_thread(ybuf + blk * 36, q.scales + at, q.sums + at, q.totals + at, q.qs + (int64_t)r * n + blk * 32, vector);
        }
        return;
    }
    for (int blk = warp; blk < blocks; blk += warps) {
        int j = blk * 32 + lane;
        float y = 0.0f;
        if (j < n) {
            float c = LAYER ? __fsub_rn(row[j], mean) : row[j];
            y = __fdiv_rn(c, denom);
            if (w) y = __fmul_rn(y, w[j]);
            if (LAYER) y = __fadd_rn(y, b[j]);
            if (out) out[(int64_t)r * n + j] = y;
        }
        if (q.qs) {
            int64_t at = (int64_t)r * (n >> 5) + blk;
            quantize_block_q8(y, lane, q.scales + at, q.sums + at, q.totals + at, q.qs + (int64_t)r * n + j);
        }
    }
}

static int launch_norm(tsm_ctx* ctx, bool layer, const float* x, const float* w, const float* b, int rows, int n, float eps,
                       float* out, const QuantizedActs* quantized) {
    OpTimer timer(ctx, layer ? "LayerNorm" : "RMSNorm", rows, n);
    if (rows == 0 || n == 0) return TSM_OK;
    if (quantized && n % 32 != 0) return fail(ctx, TSM_ERR_ARG, "rows of " + std::to_string(n) + " do not split into blocks of 32");
    if ((size_t)n * 4 > 100 * 1024) return fail(ctx, TSM_ERR_UNSUPPORTED, "norm rows over 25600 values");
    int threads = n >= 2048 ? 512 : n >= 512 ? 256 : 128;
    // the row, then the terms of its ordered sums or, after them, the normed values with 4 pad floats per block
    size_t smem = (size_t)(((n + 3) & ~3) + std::max((n + 15) & ~15, n + (n >> 5) * 4 + 4)) * 4;
    QuantOut q = quant_out(quantized);
    int exact = ctx->mode == TSM_EXACT;
    static const int chunked = getenv("TSM_PLAIN_ORDERED_SUM") ? 0 : 1;   // the term-by-term sum instead, for timing it
    if (layer) {
        if (smem > 48 * 1024) TSM_CUDA(ctx, cudaFuncSetAttribute(norm_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024));
        TSM_CUDA(ctx, launch_chained(ctx, norm_kernel<true>, dim3(rows), dim3(threads), smem, x, w, b, n, eps, out, q, exact, chunked));
    } else {
        if (smem > 48 * 1024) TSM_CUDA(ctx, cudaFuncSetAttribute(norm_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024));
        TSM_CUDA(ctx, launch_chained(ctx, norm_kernel<false>, dim3(rows), dim3(threads), smem, x, w, b, n, eps, out, q, exact, chunked));
    }
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

int launch_rmsnorm(tsm_ctx* ctx, const float* x, const float* w, int rows, int n, float eps, float* out,
                   const QuantizedActs* quantized) {
    return launch_norm(ctx, false, x, w, nullptr, rows, n, eps, out, quantized);
}

int launch_layernorm(tsm_ctx* ctx, const float* x, const float* w, const float* b, int rows, int n, float eps, float* out,
                     const QuantizedActs* quantized) {
    if (!w || !b) return fail(ctx, TSM_ERR_ARG, "layernorm needs a weight and a bias");
    return launch_norm(ctx, true, x, w, b, rows, n, eps, out, quantized);
}

// ---- RoPE (host.cr:448-466): x*cos + rotate_half(x)*sin, three roundings per element ------------

__global__ void rope_kernel(const float* __restrict__ x, int tokens, int heads, int width, int64_t x_stride,
                            const float* __restrict__ cos_table, const float* __restrict__ sin_table, int context,
                            const int* __restrict__ positions, float* out, ErrorRecord* errors) {
    int half = width >> 1;
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = (int64_t)tokens * heads * half;
    if (i >= total) return;
    int col = (int)(i % half);
    int head = (int)((i / half) % heads);
    int token = (int)(i / ((int64_t)half * heads));
    int pos = positions[token];
    float* o = out + ((int64_t)token * heads + head) * width;
    if (pos < 0 || pos >= context) {
        if (col == 0 && head == 0) report_bad_index(errors, pos, context);
        o[col] = 0.0f, o[col + half] = 0.0f;
        return;
    }
    const float* xr = x + (int64_t)token * x_stride + (int64_t)head * width;
    rotate_pair(xr[col], xr[col + half], cos_table + (int64_t)pos * width, sin_table + (int64_t)pos * width, col, half,
                &o[col], &o[col + half]);
}

int launch_rope(tsm_ctx* ctx, const float* x, int tokens, int heads, int width, int64_t x_stride, const float* cos_table,
                const float* sin_table, int context, const int* positions, float* out) {
    OpTimer timer(ctx, "Rope", tokens, heads, width);
    if (width % 2 != 0) return fail(ctx, TSM_ERR_ARG, "rotary embeddings need an even width, not " + std::to_string(width));
    int64_t total = (int64_t)tokens * heads * (width / 2);
    if (total == 0) return TSM_OK;
    rope_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(x, tokens, heads, width, x_stride, cos_table,
                                                                         sin_table, context, positions, out, ctx->errors);
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

// ---- cache writes (write_rows, host.cr:587-597) ---------------------------------------------------

__global__ void write_rows_kernel(float* cache, int rows, int heads, int capacity, int width, const float* __restrict__ values,
                                  int64_t v_stride, int64_t total, const int* __restrict__ slots, ErrorRecord* errors) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    int column = (int)(i % width);
    int head = (int)((i / width) % heads);
    int token = (int)(i / ((int64_t)width * heads));
    int slot = slots[token];
    if (slot < 0 || slot >= rows * capacity) {
        if (column == 0 && head == 0) report_bad_index(errors, slot, rows * capacity);
        return;
    }
    int row = slot / capacity, position = slot % capacity;
    cache[(((int64_t)row * heads + head) * capacity + position) * width + column] =
        values[(int64_t)token * v_stride + (int64_t)head * width + column];
}

int launch_write_rows(tsm_ctx* ctx, float* cache, int rows, int heads, int capacity, int width, const float* values,
                      int64_t v_stride, int tokens, const int* slots) {
    OpTimer timer(ctx, "WriteRows", tokens, heads, width);
    int64_t total = (int64_t)tokens * heads * width;
    if (total == 0) return TSM_OK;
    write_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(cache, rows, heads, capacity, width, values,
                                                                               v_stride, total, slots, ctx->errors);
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

// Op::Write (Tensor#write, tensor/structural.cr:64-74; copy_into_f32, kernels.cu:59-63) for a dense value written into a
// slice of a dense tensor along one axis: the region is `outer` runs of `chunk` consecutive floats, run o starting at
// dst[o * pitch + offset].
__global__ void write_region_kernel(float* dst, const float* __restrict__ src, int64_t total, int64_t pitch, int64_t chunk, int64_t offset) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    int64_t o = i / chunk, j = i % chunk;
    dst[o * pitch + offset + j] = src[i];
}

int launch_write_region(tsm_ctx* ctx, float* dst, const float* src, int64_t outer, int64_t pitch, int64_t chunk, int64_t offset) {
    OpTimer timer(ctx, "Write", outer, chunk);
    int64_t total = outer * chunk;
    if (total == 0) return TSM_OK;
    write_region_kernel<<<(unsigned)((total + 255) / 256), 256, 0, ctx->stream>>>(dst, src, total, pitch, chunk, offset);
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

// Rotates the q and k heads of each token's joined qkv row in place (Llama) and appends k and v to
// the token's cache row at its position: the RoPE x2 + WriteRows x2 of modules.cr:434-452 as one launch.
__global__ void rope_append_kernel(float* qkv, int tokens, int heads, int kv_heads, int width, const float* __restrict__ cos_table,
                                   const float* __restrict__ sin_table, int context, const int* __restrict__ table,
                                   float* keys, float* values, int rows, int capacity, ErrorRecord* errors) {
    chained_kernel_entry();
    int half = width >> 1;
    int all = heads + 2 * kv_heads;
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    int64_t total = (int64_t)tokens * all * half;
    if (i >= total) return;
    int col = (int)(i % half);
    int head = (int)((i / half) % all);
    int token = (int)(i / ((int64_t)half * all));
    int row = table[3 * token], pos = table[3 * token + 1];
    if (row < 0 || row >= rows || pos < 0 || pos >= capacity || (cos_table && pos >= context)) {
        if (col == 0 && head == 0) report_bad_index(errors, pos, capacity);
        return;
    }
    float* xr = qkv + (int64_t)token * all * width + (int64_t)head * width;
    float a = xr[col], b = xr[col + half];
    if (head < heads + kv_heads && cos_table) {
        float ra, rb;
        rotate_pair(a, b, cos_table + (int64_t)pos * width, sin_table + (int64_t)pos * width, col, half, &ra, &rb);
        a = ra, b = rb;
        xr[col] = a, xr[col + half] = b;
    }
    if (head >= heads) {
        bool is_key = head < heads + kv_heads;
        int kh = is_key ? head - heads : head - heads - kv_heads;
        float* dst = (is_key ? keys : values) + (((int64_t)row * kv_heads + kh) * capacity + pos) * width;
        dst[col] = a, dst[col + half] = b;
    }
}

// The same with four pairs per thread in 16-byte pieces (head widths that are multiples of 8, 16-byte aligned buffers): a
// thread's loads are all in flight at once, where one pair per thread left most of the launch waiting for its two.
__global__ void rope_append4_kernel(float* qkv, int tokens, int heads, int kv_heads, int width, const float* __restrict__ cos_table,
                                    const float* __restrict__ sin_table, int context, const int* __restrict__ table,
                                    float* keys, float* values, int rows, int capacity, ErrorRecord* errors) {
    chained_kernel_entry();
    const int half = width >> 1, quads = half >> 2;
    const int all = heads + 2 * kv_heads;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t total = (int64_t)tokens * all * quads;
    if (i >= total) return;
    const int col = (int)(i % quads) * 4;
    const int head = (int)((i / quads) % all);
    const int token = (int)(i / ((int64_t)quads * all));
    const int row = table[3 * token], pos = table[3 * token + 1];
    if (row < 0 || row >= rows || pos < 0 || pos >= capacity || (cos_table && pos >= context)) {
        if (col == 0 && head == 0) report_bad_index(errors, pos, capacity);
        return;
    }
    float* xr = qkv + (int64_t)token * all * width + (int64_t)head * width;
    float4 a = *(const float4*)(xr + col), b = *(const float4*)(xr + col + half);
    if (head < heads + kv_heads && cos_table) {
        const float* c = cos_table + (int64_t)pos * width;
        const float* sn = sin_table + (int64_t)pos * width;
        const float4 ca = *(const float4*)(c + col), cb = *(const float4*)(c + col + half);
        const float4 sa = *(const float4*)(sn + col), sb = *(const float4*)(sn + col + half);
        // rotate_pair, element by element: a' = a cos_i + (b * -1) sin_i, b' = b cos_(i+half) + a sin_(i+half)
        float4 ra, rb;
        ra.x = __fadd_rn(__fmul_rn(a.x, ca.x), __fmul_rn(__fmul_rn(b.x, -1.0f), sa.x)), rb.x = __fadd_rn(__fmul_rn(b.x, cb.x), __fmul_rn(a.x, sb.x));
        ra.y = __fadd_rn(__fmul_rn(a.y, ca.y), __fmul_rn(__fmul_rn(b.y, -1.0f), sa.y)), rb.y = __fadd_rn(__fmul_rn(b.y, cb.y), __fmul_rn(a.y, sb.y));
        ra.z = __fadd_rn(__fmul_rn(a.z, ca.z), __fmul_rn(__fmul_rn(b.z, -1.0f), sa.z)), rb.z = __fadd_rn(__fmul_rn(b.z, cb.z), __fmul_rn(a.z, sb.z));
        ra.w = __fadd_rn(__fmul_rn(a.w, ca.w), __fmul_rn(__fmul_rn(b.w, -1.0f), sa.w)), rb.w = __fadd_rn(__fmul_rn(b.w, cb.w), __fmul_rn(a.w, sb.w));
        a = ra, b = rb;
        *(float4*)(xr + col) = a, *(float4*)(xr + col + half) = b;
    }
    if (head >= heads) {
        const bool is_key = head < heads + kv_heads;
        const int kh = is_key ? head - heads : head - heads - kv_heads;
        float* dst = (is_key ? keys : values) + (((int64_t)row * kv_heads + kh) * capacity + pos) * width;
        *(float4*)(dst + col) = a, *(float4*)(dst + col + half) = b;
    }
}

int launch_rope_append(tsm_ctx* ctx, float* qkv, int tokens, int heads, int kv_heads, int width, const float* cos_table,
                       const float* sin_table, int context, const int* table, float* keys, float* values, int rows,
                       int capacity) {
    OpTimer timer(ctx, "Rope+WriteRows", tokens, heads + 2 * kv_heads, width);
    if (width % 2 != 0) return fail(ctx, TSM_ERR_ARG, "head width must be even, not " + std::to_string(width));
    int64_t total = (int64_t)tokens * (heads + 2 * kv_heads) * (width / 2);
    if (total == 0) return TSM_OK;
    const bool pieces = width % 8 == 0 && (((uintptr_t)qkv | (uintptr_t)keys | (uintptr_t)values | (uintptr_t)(cos_table ? cos_table : (const float*)qkv) |
                                            (uintptr_t)(sin_table ? sin_table : (const float*)qkv)) & 15) == 0;
    if (pieces) {
        TSM_CUDA(ctx, launch_chained(ctx, rope_append4_kernel, dim3((unsigned)((total / 4 + 255) / 256)), dim3(256), 0, qkv, tokens, heads, kv_heads,
                                     width, cos_table, sin_table, context, table, keys, values, rows, capacity, ctx->errors));
        count_launch(ctx);
        TSM_LAUNCH_CHECK(ctx);
        return TSM_OK;
    }
    TSM_CUDA(ctx, launch_chained(ctx, rope_append_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, qkv, tokens, heads, kv_heads, width,
                                 cos_table, sin_table, context, table, keys, values, rows, capacity, ctx->errors));
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

// ---- activations (kernels.cr:4,18 through the tape of kernel.cr:259-300) --------------------------

// One warp per 32 consecutive outputs of a row, so that the block quantiser can follow in registers.
template <bool GELU>
__global__ void activation_kernel(const float* __restrict__ a, const float* __restrict__ b, int rows, int n, int64_t in_stride,
                                  float* out, QuantOut q) {
    chained_kernel_entry();
    int lane = threadIdx.x & 31;
    int blocks = (n + 31) >> 5;
    int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (item >= (int64_t)rows * blocks) return;
    int r = (int)(item / blocks), blk = (int)(item % blocks);
    int j = blk * 32 + lane;
    float y = 0.0f;
    if (j < n) {
        y = GELU ? gelu_value(a[(int64_t)r * in_stride + j]) : swiglu_value(a[(int64_t)r * in_stride + j], b[(int64_t)r * in_stride + j]);
        if (out) out[(int64_t)r * n + j] = y;
    }
    if (q.qs) {
        int64_t at = (int64_t)r * (n >> 5) + blk;
        quantize_block_q8(y, lane, q.scales + at, q.sums + at, q.totals + at, q.qs + (int64_t)r * n + j);
    }
}

// The same for rows that go out quantised and can be read in 16-byte pieces: a CTA takes 32 consecutive blocks; every thread
// makes four consecutive values of one block (four independent chains of the exp polynomial), the values pass through
// shared memory, and one thread per block quantises them (quantize_block_by_thread).  12.6 -> about 7 us for 64 rows of
// 14336, where one warp per block went through load, exp and two chains of shuffles one after the other.
template <bool GELU>
__global__ void __launch_bounds__(256) activation_blocks_kernel(const float* __restrict__ a, const float* __restrict__ b, int64_t blocks,
                                                                int blocks_per_row, int64_t in_stride, float* out, QuantOut q) {
    chained_kernel_entry();
    __shared__ __align__(16) float ybuf[32 * 36];
    const int tid = threadIdx.x;
    const int64_t first = (int64_t)blockIdx.x * 32;
    {
        const int64_t B = first + (tid >> 3);
        if (B < blocks) {
            const int r = (int)(B / blocks_per_row), blk = (int)(B % blocks_per_row);
            const int j = blk * 32 + (tid & 7) * 4;
            const float4 g4 = *(const float4*)(a + (int64_t)r * in_stride + j);
            float4 y;
            if (GELU) {
                y.x = gelu_value(g4.x), y.y = gelu_value(g4.y), y.z = gelu_value(g4.z), y.w = gelu_value(g4.w);
            } else {
                const float4 u4 = *(const float4*)(b + (int64_t)r * in_stride + j);
                y.x = swiglu_value(g4.x, u4.x), y.y = swiglu_value(g4.y, u4.y), y.z = swiglu_value(g4.z, u4.z), y.w = swiglu_value(g4.w, u4.w);
            }
            if (out) *(float4*)(out + (int64_t)r * blocks_per_row * 32 + j) = y;
            *(float4*)(ybuf + (tid >> 3) * 36 + (tid & 7) * 4) = y;
        }
    }
    __syncthreads();
    if (tid < 32) {
        const int64_t B = first + tid;
        if (B < blocks) quantize_block_by_thread(ybuf + tid * 36, q.scales + B, q.sums + B, q.totals + B, q.qs + B * 32, true);
    }
}

static int launch_activation(tsm_ctx* ctx, bool gelu, const float* a, const float* b, int rows, int n, int64_t in_stride,
                             float* out, const QuantizedActs* quantized) {
    OpTimer timer(ctx, gelu ? "Kernel gelu" : "Kernel swiglu", rows, n);
    if (rows == 0 || n == 0) return TSM_OK;
    if (quantized && n % 32 != 0) return fail(ctx, TSM_ERR_ARG, "rows of " + std::to_string(n) + " do not split into blocks of 32");
    const bool pieces = quantized && in_stride % 4 == 0 &&
                        (((uintptr_t)a | (uintptr_t)(b ? b : a) | (uintptr_t)(out ? out : a) | (uintptr_t)quantized->qs) & 15) == 0;
    if (pieces) {
        QuantOut qb = quant_out(quantized);
        const int64_t blocks = (int64_t)rows * (n / 32);
        const unsigned ctas = (unsigned)((blocks + 31) / 32);
        if (gelu) TSM_CUDA(ctx, launch_chained(ctx, activation_blocks_kernel<true>, dim3(ctas), dim3(256), 0, a, b, blocks, n / 32, in_stride, out, qb));
        else TSM_CUDA(ctx, launch_chained(ctx, activation_blocks_kernel<false>, dim3(ctas), dim3(256), 0, a, b, blocks, n / 32, in_stride, out, qb));
        count_launch(ctx);
        TSM_LAUNCH_CHECK(ctx);
        return TSM_OK;
    }
    int64_t items = (int64_t)rows * ((n + 31) / 32);
    unsigned grid = (unsigned)((items + 7) / 8);
    QuantOut q = quant_out(quantized);
    if (gelu) TSM_CUDA(ctx, launch_chained(ctx, activation_kernel<true>, dim3(grid), dim3(256), 0, a, b, rows, n, in_stride, out, q));
    else TSM_CUDA(ctx, launch_chained(ctx, activation_kernel<false>, dim3(grid), dim3(256), 0, a, b, rows, n, in_stride, out, q));
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

int launch_swiglu(tsm_ctx* ctx, const float* gate, const float* up, int rows, int n, int64_t in_stride, float* out,
                  const QuantizedActs* quantized) {
    return launch_activation(ctx, false, gate, up, rows, n, in_stride, out, quantized);
}

int launch_gelu(tsm_ctx* ctx, const float* x, int rows, int n, float* out, const QuantizedActs* quantized) {
    return launch_activation(ctx, true, x, nullptr, rows, n, n, out, quantized);
}

// kernels.cr:15: x / (exp(-x) + 1), the tape's four steps each rounded on its own.
__global__ void silu_kernel(const float* __restrict__ x, int64_t count, float* out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float v = x[i];
    out[i] = __fdiv_rn(v, __fadd_rn(exact_exp(-v), 1.0f));
}

int launch_silu(tsm_ctx* ctx, const float* x, int64_t count, float* out) {
    OpTimer timer(ctx, "Kernel silu", count);
    if (count == 0) return TSM_OK;
    silu_kernel<<<(unsigned)((count + 255) / 256), 256, 0, ctx->stream>>>(x, count, out);
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

__global__ void add_kernel(const float* __restrict__ a, const float* __restrict__ b, int64_t count, float* out) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) out[i] = __fadd_rn(a[i], b[i]);
}

int launch_add(tsm_ctx* ctx, const float* a, const float* b, int64_t count, float* out) {
    OpTimer timer(ctx, "Add", count);
    if (count == 0) return TSM_OK;
    add_kernel<<<(unsigned)((count + 255) / 256), 256, 0, ctx->stream>>>(a, b, count, out);
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

// ---- sampling (sampler.cr:36, 77-96) -----------------------------------------------------------------

// Is (va, ia) ahead of (vb, ib) in the sampler's order: higher logit first, equal logits by lower index.
__device__ __forceinline__ bool ahead(float va, int ia, float vb, int ib) { return va > vb || (va == vb && ia < ib); }

// One CTA per row.  Round r picks the best candidate that comes after round r-1's pick, so no row
// is modified and ties keep index order.  count = 1 is the greedy pick.
__global__ void topk_kernel(const float* __restrict__ logits, int n, int count, int* out_ids, float* out_values) {
    chained_kernel_entry();
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    __shared__ float last_v;
    __shared__ int last_i;
    const float* row = logits + (int64_t)blockIdx.x * n;
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    for (int round = 0; round < count; round++) {
        float lv = last_v;
        int li = last_i;
        float v = 0.0f;
        int at = -1;
        // eight loads in flight per thread: one at a time, each would wait out a trip to L2
        for (int j0 = threadIdx.x; j0 < n; j0 += 8 * blockDim.x) {
            float xs[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                int j = j0 + u * blockDim.x;
                xs[u] = j < n ? row[j] : 0.0f;
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                int j = j0 + u * blockDim.x;
                if (j >= n) break;
                float x = xs[u];
                if (round > 0 && !ahead(lv, li, x, j)) continue;  // not after the last pick
                if (at < 0 || ahead(x, j, v, at)) v = x, at = j;
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            float ov = __shfl_xor_sync(0xffffffffu, v, off);
            int oi = __shfl_xor_sync(0xffffffffu, at, off);
            if (oi >= 0 && (at < 0 || ahead(ov, oi, v, at))) v = ov, at = oi;
        }
        if (lane == 0) best_v[warp] = v, best_i[warp] = at;
        __syncthreads();
        if (threadIdx.x == 0) {
            for (int w2 = 1; w2 < warps; w2++)
                if (best_i[w2] >= 0 && (at < 0 || ahead(best_v[w2], best_i[w2], v, at))) v = best_v[w2], at = best_i[w2];
            last_v = v, last_i = at;
            out_ids[(int64_t)blockIdx.x * count + round] = at;
            if (out_values) out_values[(int64_t)blockIdx.x * count + round] = v;
        }
        __syncthreads();
    }
}

int launch_topk(tsm_ctx* ctx, const float* logits, int rows, int n, int count, int* out_ids, float* out_values) {
    OpTimer timer(ctx, "TopK", rows, n, count);
    if (count < 1 || count > n) return fail(ctx, TSM_ERR_ARG, "top " + std::to_string(count) + " of " + std::to_string(n));
    if (rows == 0) return TSM_OK;
    TSM_CUDA(ctx, launch_chained(ctx, topk_kernel, dim3(rows), dim3(1024), 0, logits, n, count, out_ids, out_values));
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

int launch_argmax(tsm_ctx* ctx, const float* logits, int rows, int n, int* out) {
    OpTimer timer(ctx, "ArgMax", rows, n);
    if (n < 1) return fail(ctx, TSM_ERR_ARG, "argmax of an empty row");
    return launch_topk(ctx, logits, rows, n, 1, out, nullptr);
}

}  // namespace tsm
