// The unquantised product: out[row, col] = sum over k of x[row, k] * w[col, k], a Linear whose weight stayed F32.
//
// The host adds the k products of an output in index order, each product and each sum rounded on its own
// (devices/host.cr:700-721; the reference's CUDA matmul_f32, cuda/kernels.cu:357-375, does the same with one thread
// per output), then the bias (host.cr:725-734).  So an output is one chain of k dependent adds and no split of k keeps
// the bits.  What can be shared is the traffic: a CTA owns 128 weight rows (output columns) and up to 8 activation
// rows, stages 32 columns of k at a time in shared memory with coalesced loads, and every thread walks its own weight
// row's staged values once for all of its activation rows.  This is the path of models kept in F32 (the reference's
// F32 fixtures) and of an F32 token table used as the head; the quantised products are the fast path.
#include "common.cuh"

namespace tsm {

constexpr int kF32Cols = 128;  // weight rows (output columns) per CTA, one per thread
constexpr int kF32Rows = 8;    // activation rows per CTA
constexpr int kF32Step = 32;   // k values staged per pass

__global__ void __launch_bounds__(kF32Cols) matmul_f32_kernel(const float* __restrict__ x, const float* __restrict__ w, int rows, int n, int k,
                                                              const float* __restrict__ bias, const float* residual, float* out) {
    chained_kernel_entry();
    __shared__ float ws[kF32Cols][kF32Step + 1];  // +1: a thread's row starts one bank after its neighbour's
    __shared__ float xs[kF32Rows][kF32Step];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int col0 = blockIdx.x * kF32Cols, row0 = blockIdx.y * kF32Rows;
    const int my_rows = min(kF32Rows, rows - row0);
    float acc[kF32Rows];
#pragma unroll
    for (int r = 0; r < kF32Rows; r++) acc[r] = 0.0f;
    for (int k0 = 0; k0 < k; k0 += kF32Step) {
        const int width = min(kF32Step, k - k0);
        // a warp reads 32 consecutive k of one weight row per load
        for (int c = warp; c < kF32Cols; c += kF32Cols / 32) {
            int col = col0 + c;
            ws[c][lane] = (col < n && lane < width) ? w[(int64_t)col * k + k0 + lane] : 0.0f;
        }
        for (int r = warp; r < kF32Rows; r += kF32Cols / 32)
            xs[r][lane] = (r < my_rows && lane < width) ? x[(int64_t)(row0 + r) * k + k0 + lane] : 0.0f;
        __syncthreads();
        if (width == kF32Step) {
#pragma unroll
            for (int s = 0; s < kF32Step; s++) {
                float wv = ws[t][s];
#pragma unroll
                for (int r = 0; r < kF32Rows; r++) acc[r] = __fadd_rn(acc[r], __fmul_rn(xs[r][s], wv));
            }
        } else {
            for (int s = 0; s < width; s++) {
                float wv = ws[t][s];
#pragma unroll
                for (int r = 0; r < kF32Rows; r++) acc[r] = __fadd_rn(acc[r], __fmul_rn(xs[r][s], wv));
            }
        }
        __syncthreads();
    }
    const int col = col0 + t;
    if (col >= n) return;
#pragma unroll
    for (int r = 0; r < kF32Rows; r++) {
        if (r >= my_rows) break;
        float v = acc[r];
        if (bias) v = __fadd_rn(v, bias[col]);
        int64_t at = (int64_t)(row0 + r) * n + col;
        if (residual) v = __fadd_rn(residual[at], v);
        out[at] = v;
    }
}

int launch_matmul_f32(tsm_ctx* ctx, const float* x, int rows, int k, const float* w, int n, const float* bias, const float* residual,
                      float* out) {
    OpTimer timer(ctx, "MatMul", rows, k, n);
    if (rows < 0 || n < 0 || k < 0) return fail(ctx, TSM_ERR_ARG, "negative product shape");
    if (rows == 0 || n == 0) return TSM_OK;
    dim3 grid((unsigned)((n + kF32Cols - 1) / kF32Cols), (unsigned)((rows + kF32Rows - 1) / kF32Rows));
    if (grid.y > 65535) return fail(ctx, TSM_ERR_ARG, "more than 524280 rows in one F32 product");
    TSM_CUDA(ctx, launch_chained(ctx, matmul_f32_kernel, grid, dim3(kF32Cols), 0, x, w, rows, n, k, bias, residual, out));
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

}  // namespace tsm
