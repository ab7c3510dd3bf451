// tsm_block_matmul_static: the quantised product for callers that must not allocate device memory.
//
// Some hosts cannot let a call reach cudaMalloc: a server thread that holds a latency budget (cudaMalloc may
// take milliseconds and can synchronise the device), or a process whose device memory was carved up front and
// whose allocator is closed afterwards.  tsm_block_matmul grows a per-context scratch
// buffer on demand (for the 8-bit activations it quantises before the product), so it can allocate on any call.
// This entry point keeps that scratch in a file-scope device array of fixed size instead.  The array belongs to
// the loaded library image: every GPU that loads the library holds its 1.5 MB from then until the process ends.
#include "common.cuh"

namespace {

// Room for rows * k <= 1 Mi activations: their int8 values plus three 4-byte words per block of 32, each part
// rounded to 256 bytes as tsm::quant_scratch_layout lays them out.
constexpr int64_t kStaticActivations = 1 << 20;
constexpr int64_t kStaticBytes = ((kStaticActivations / 32) * 12 + 255) / 256 * 256 + kStaticActivations + 256;

static __device__ __align__(256) unsigned char static_scratch[kStaticBytes];

// The device address of the array, per device.  In host code `static_scratch` is only a handle for the symbol:
// passing it to a kernel would hand over a host address.  cudaGetSymbolAddress, called with the device current,
// gives the address kernels can use on that device.
std::mutex address_lock;
void* addresses[64] = {nullptr};

int scratch_address(tsm_ctx* ctx, void** out) {
    std::lock_guard<std::mutex> guard(address_lock);
    if (ctx->ordinal < 0 || ctx->ordinal >= 64) return tsm::fail(ctx, TSM_ERR_ARG, "device ordinal out of range");
    if (!addresses[ctx->ordinal]) {
        void* p = nullptr;
        cudaError_t err = cudaGetSymbolAddress(&p, static_scratch);  // the caller made ctx's device current
        if (err != cudaSuccess) return tsm::cuda_fail(ctx, err, "cudaGetSymbolAddress(static_scratch)");
        addresses[ctx->ordinal] = p;
    }
    *out = addresses[ctx->ordinal];
    return TSM_OK;
}

}  // namespace

extern "C" int tsm_block_matmul_static(tsm_ctx* ctx, tsm_dptr x, int rows, int k, int64_t x_stride, tsm_dptr w, int kind, int n,
                                       tsm_dptr bias, tsm_dptr out) {
    if (!ctx) return TSM_ERR_ARG;
    tsm::DeviceGuard device_guard(ctx->ordinal);
    if (k <= 0 || k % 32 != 0) return tsm::fail(ctx, TSM_ERR_ARG, "rows of " + std::to_string(k) + " do not split into blocks of 32");
    if (rows < 0 || n < 0) return tsm::fail(ctx, TSM_ERR_ARG, "negative size");
    if ((int64_t)rows * k > kStaticActivations)
        return tsm::fail(ctx, TSM_ERR_ARG,
                         std::to_string(rows) + " rows of " + std::to_string(k) + " activations exceed the " +
                             std::to_string(kStaticActivations) + " the static scratch holds; use tsm_block_matmul");
    if (rows == 0 || n == 0) return TSM_OK;
    void* base = nullptr;
    TSM_TRY(scratch_address(ctx, &base));
    // Nothing in the array has to start at zero: the quantiser writes every scale, sum, total and value that
    // the product then reads.
    tsm::QuantizedActs a = tsm::quant_scratch_layout(base, rows, k);
    TSM_TRY(tsm::launch_quantize_rows(ctx, (const float*)(uintptr_t)x, rows, k, x_stride, (float*)a.scales, (float*)a.sums,
                                      (int*)a.totals, (int8_t*)a.qs));
    return tsm::launch_block_matmul(ctx, a, rows, k, (const uint8_t*)(uintptr_t)w, kind, n, (const float*)(uintptr_t)bias, nullptr,
                                    (float*)(uintptr_t)out);
}
