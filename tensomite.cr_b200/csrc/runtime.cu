// The context (device, stream, buffer pool, error record, counters) and the operator-level C ABI.
#include <string.h>

#include <algorithm>

#include "common.cuh"

namespace tsm {

void set_message(tsm_ctx* ctx, const std::string& text) {
    if (!ctx) return;
    std::lock_guard<std::mutex> guard(ctx->message_lock);
    ctx->message = text;
}

int fail(tsm_ctx* ctx, int status, const std::string& text) {
    set_message(ctx, text);
    return status;
}

int cuda_fail(tsm_ctx* ctx, cudaError_t err, const char* what) {
    // "<call>: <NAME> (<string>)", as the reference words its DeviceError (cuda.cr:1070-1075)
    std::string text = std::string(what) + ": " + cudaGetErrorName(err) + " (" + cudaGetErrorString(err) + ")";
    set_message(ctx, text);
    return err == cudaErrorMemoryAllocation ? TSM_ERR_MEMORY : TSM_ERR_CUDA;
}

bool chained_launch_enabled() {
    static const bool on = !(getenv("TSM_CHAINED_LAUNCH") && getenv("TSM_CHAINED_LAUNCH")[0] == '0');
    return on;
}

int ensure_scratch(tsm_ctx* ctx, Scratch& s, int64_t bytes) {
    if (s.bytes >= bytes) return TSM_OK;
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(ctx->stream, &capturing);
    if (capturing != cudaStreamCaptureStatusNone)
        return fail(ctx, TSM_ERR_ARG, "scratch memory must be sized before a step is captured");
    if (s.ptr) {
        TSM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        TSM_CUDA(ctx, cudaFree(s.ptr));
        s.ptr = nullptr, s.bytes = 0;
    }
    int64_t rounded = (bytes + (1 << 20) - 1) / (1 << 20) * (1 << 20);
    TSM_CUDA(ctx, cudaMalloc(&s.ptr, (size_t)rounded));
    s.bytes = rounded;
    ctx->scratch_generation++;
    ctx->counters.allocs++;
    return TSM_OK;
}

int check_error_record(tsm_ctx* ctx) {
    ErrorRecord seen = *ctx->errors_host;
    if (seen.count == 0 && seen.timeout == 0) return TSM_OK;
    TSM_CUDA(ctx, cudaMemsetAsync(ctx->errors, 0, sizeof(ErrorRecord), ctx->stream));
    TSM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    ctx->errors_host->count = 0, ctx->errors_host->timeout = 0;
    if (seen.timeout != 0) return fail(ctx, TSM_ERR_TIMEOUT, "a device-side wait for an asynchronous copy ran out");
    return fail(ctx, TSM_ERR_EXECUTION,
                "index " + std::to_string(seen.first) + " out of range for " + std::to_string(seen.limit) + " rows" +
                    (seen.count > 1 ? " (and " + std::to_string(seen.count - 1) + " more)" : ""));
}

int pool_alloc(tsm_ctx* ctx, int64_t bytes, void** out) {
    if (bytes < 0) return fail(ctx, TSM_ERR_ARG, "alloc of " + std::to_string(bytes) + " bytes");
    if (bytes == 0) bytes = 1;
    {
        std::lock_guard<std::mutex> guard(ctx->pool.lock);
        auto found = ctx->pool.free_lists.find(bytes);
        if (found != ctx->pool.free_lists.end() && !found->second.empty()) {
            *out = found->second.back();
            found->second.pop_back();
            ctx->pool.held_bytes -= bytes;
            ctx->counters.pool_hits++;
            return TSM_OK;
        }
    }
    void* ptr = nullptr;
    cudaError_t err = cudaMalloc(&ptr, (size_t)bytes);
    if (err == cudaErrorMemoryAllocation) {
        // give the pooled memory back to the driver and try once more (cuda.cr:339-353)
        cudaGetLastError();
        std::vector<void*> drop;
        {
            std::lock_guard<std::mutex> guard(ctx->pool.lock);
            for (auto& entry : ctx->pool.free_lists) {
                for (void* p : entry.second) drop.push_back(p), ctx->pool.sizes.erase(p);
                entry.second.clear();
            }
            ctx->pool.held_bytes = 0;
        }
        cudaStreamSynchronize(ctx->stream);
        for (void* p : drop) cudaFree(p), ctx->counters.frees++;
        err = cudaMalloc(&ptr, (size_t)bytes);
    }
    if (err != cudaSuccess) return cuda_fail(ctx, err, "cudaMalloc");
    {
        std::lock_guard<std::mutex> guard(ctx->pool.lock);
        ctx->pool.sizes[ptr] = bytes;
    }
    ctx->counters.pool_misses++;
    ctx->counters.allocs++;
    *out = ptr;
    return TSM_OK;
}

void pool_release(tsm_ctx* ctx, void* p) {
    if (p) tsm_free(ctx, (tsm_dptr)(uintptr_t)p);
}

// ---- per-operator timing ------------------------------------------------------------------------

static cudaEvent_t profile_event(tsm_ctx* ctx) {
    Profile& pr = ctx->profile;
    if (!pr.spare.empty()) {
        cudaEvent_t e = pr.spare.back();
        pr.spare.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    if (cudaEventCreate(&e) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return e;
}

OpTimer::OpTimer(tsm_ctx* c, const char* name, int64_t a, int64_t b, int64_t d) : ctx(c) {
    Profile& pr = ctx->profile;
    if (!pr.on) return;
    if (pr.depth++ > 0) return;
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(ctx->stream, &capturing);
    if (capturing != cudaStreamCaptureStatusNone) return;
    start = profile_event(ctx);
    if (!start) return;
    label = name;
    if (pr.shapes && a >= 0) {
        label += " [" + std::to_string(a);
        if (b >= 0) label += "," + std::to_string(b);
        if (d >= 0) label += "," + std::to_string(d);
        label += "]";
    }
    cudaEventRecord(start, ctx->stream);
    active = true;
}

OpTimer::~OpTimer() {
    Profile& pr = ctx->profile;
    if (!pr.on && !active) return;
    if (pr.depth > 0) pr.depth--;
    if (!active) return;
    cudaEvent_t stop = dropped ? nullptr : profile_event(ctx);
    if (!stop) {
        pr.spare.push_back(start);
        return;
    }
    cudaEventRecord(stop, ctx->stream);
    pr.spans.push_back(ProfileSpan{label, start, stop});
}

// Waits for the stream, then moves every finished span into the totals.
static int profile_collect(tsm_ctx* ctx) {
    Profile& pr = ctx->profile;
    if (pr.spans.empty()) return TSM_OK;
    TSM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (ProfileSpan& span : pr.spans) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, span.start, span.stop) == cudaSuccess) {
            auto& slot = pr.totals[span.label];
            slot.first += 1, slot.second += (double)ms * 1e-3;
        } else {
            cudaGetLastError();
        }
        pr.spare.push_back(span.start), pr.spare.push_back(span.stop);
    }
    pr.spans.clear();
    return TSM_OK;
}

}  // namespace tsm

using namespace tsm;

#define CTX_GUARD(ctx)                         \
    if (!(ctx)) return TSM_ERR_ARG;            \
    tsm::DeviceGuard device_guard__((ctx)->ordinal)

extern "C" {

const char* tsm_status_name(int status) {
    switch (status) {
        case TSM_OK: return "TSM_OK";
        case TSM_ERR_CUDA: return "TSM_ERR_CUDA";
        case TSM_ERR_ARG: return "TSM_ERR_ARG";
        case TSM_ERR_EXECUTION: return "TSM_ERR_EXECUTION";
        case TSM_ERR_MEMORY: return "TSM_ERR_MEMORY";
        case TSM_ERR_IO: return "TSM_ERR_IO";
        case TSM_ERR_UNSUPPORTED: return "TSM_ERR_UNSUPPORTED";
        case TSM_ERR_TIMEOUT: return "TSM_ERR_TIMEOUT";
        case TSM_ERR_COMM: return "TSM_ERR_COMM";
    }
    return "TSM_ERR_UNKNOWN";
}

int tsm_device_count(int* count) {
    if (!count) return TSM_ERR_ARG;
    *count = 0;
    cudaError_t err = cudaGetDeviceCount(count);
    if (err != cudaSuccess) {
        cudaGetLastError();
        *count = 0;
        return TSM_ERR_CUDA;
    }
    return TSM_OK;
}

int tsm_ctx_create(int ordinal, tsm_ctx** out) {
    if (!out) return TSM_ERR_ARG;
    *out = nullptr;
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || ordinal < 0 || ordinal >= count) {
        cudaGetLastError();
        return TSM_ERR_CUDA;
    }
    tsm::DeviceGuard guard(ordinal);
    tsm_ctx* ctx = new tsm_ctx();
    ctx->ordinal = ordinal;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, ordinal) != cudaSuccess || cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaMalloc((void**)&ctx->errors, sizeof(ErrorRecord)) != cudaSuccess ||
        cudaMallocHost((void**)&ctx->errors_host, sizeof(ErrorRecord)) != cudaSuccess ||
        cudaMemset(ctx->errors, 0, sizeof(ErrorRecord)) != cudaSuccess) {
        cudaGetLastError();
        delete ctx;
        return TSM_ERR_CUDA;
    }
    ctx->sm_count = prop.multiProcessorCount;
    ctx->wait_hint = getenv("TSM_WAIT_HINT_NS") ? (unsigned)atoi(getenv("TSM_WAIT_HINT_NS")) : 0u;
    // what the pool may keep: max(1 GiB, a quarter of the device), as the reference's pool (cuda.cr:339-353)
    int64_t quarter = (int64_t)(prop.totalGlobalMem / 4);
    ctx->pool.limit_bytes = quarter > (1ll << 30) ? quarter : (1ll << 30);
    *out = ctx;
    return TSM_OK;
}

int tsm_ctx_destroy(tsm_ctx* ctx) {
    CTX_GUARD(ctx);
    cudaStreamSynchronize(ctx->stream);
    tsm::tp_release(ctx);
    for (auto& entry : ctx->pool.sizes) cudaFree(entry.first);
    if (ctx->quant.ptr) cudaFree(ctx->quant.ptr);
    if (ctx->attn.ptr) cudaFree(ctx->attn.ptr);
    if (ctx->order.ptr) cudaFree(ctx->order.ptr);
    for (auto& span : ctx->profile.spans) cudaEventDestroy(span.start), cudaEventDestroy(span.stop);
    for (cudaEvent_t e : ctx->profile.spare) cudaEventDestroy(e);
    cudaFree(ctx->errors);
    cudaFreeHost(ctx->errors_host);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return TSM_OK;
}

int tsm_last_error(tsm_ctx* ctx, char* buffer, int capacity) {
    if (!ctx || !buffer || capacity <= 0) return TSM_ERR_ARG;
    std::lock_guard<std::mutex> guard(ctx->message_lock);
    strncpy(buffer, ctx->message.c_str(), (size_t)capacity - 1);
    buffer[capacity - 1] = 0;
    return TSM_OK;
}

void* tsm_ctx_stream(tsm_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

int tsm_alloc(tsm_ctx* ctx, int64_t bytes, tsm_dptr* out) {
    CTX_GUARD(ctx);
    if (!out) return fail(ctx, TSM_ERR_ARG, "alloc needs somewhere to put the address");
    void* ptr = nullptr;
    TSM_TRY(pool_alloc(ctx, bytes, &ptr));
    *out = (tsm_dptr)(uintptr_t)ptr;
    return TSM_OK;
}

int tsm_free(tsm_ctx* ctx, tsm_dptr ptr) {
    if (!ctx || !ptr) return TSM_OK;
    void* p = (void*)(uintptr_t)ptr;
    std::lock_guard<std::mutex> guard(ctx->pool.lock);
    auto found = ctx->pool.sizes.find(p);
    if (found == ctx->pool.sizes.end()) return TSM_ERR_ARG;  // a buffer of another device (cuda.cr:456-458)
    int64_t bytes = found->second;
    // Kept for the next alloc of the same size; memory beyond the limit stays pooled too until an
    // allocation fails, because releasing it here would wait for the device, and this call never waits.
    ctx->pool.free_lists[bytes].push_back(p);
    ctx->pool.held_bytes += bytes;
    return TSM_OK;
}

int tsm_upload(tsm_ctx* ctx, tsm_dptr dst, const void* src, int64_t bytes) {
    CTX_GUARD(ctx);
    if (bytes < 0 || (bytes > 0 && (!dst || !src))) return fail(ctx, TSM_ERR_ARG, "upload of " + std::to_string(bytes) + " bytes");
    if (bytes == 0) return TSM_OK;
    TSM_CUDA(ctx, cudaMemcpyAsync((void*)(uintptr_t)dst, src, (size_t)bytes, cudaMemcpyHostToDevice, ctx->stream));
    TSM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    ctx->counters.uploads++;
    ctx->counters.upload_bytes += bytes;
    return TSM_OK;
}

int tsm_download(tsm_ctx* ctx, void* dst, tsm_dptr src, int64_t bytes) {
    CTX_GUARD(ctx);
    if (bytes < 0 || (bytes > 0 && (!dst || !src))) return fail(ctx, TSM_ERR_ARG, "download of " + std::to_string(bytes) + " bytes");
    if (bytes == 0) return TSM_OK;
    TSM_CUDA(ctx, cudaMemcpyAsync(dst, (const void*)(uintptr_t)src, (size_t)bytes, cudaMemcpyDeviceToHost, ctx->stream));
    TSM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    ctx->counters.downloads++;
    ctx->counters.download_bytes += bytes;
    return TSM_OK;
}

int tsm_sync(tsm_ctx* ctx) {
    CTX_GUARD(ctx);
    TSM_CUDA(ctx, cudaMemcpyAsync(ctx->errors_host, ctx->errors, sizeof(ErrorRecord), cudaMemcpyDeviceToHost, ctx->stream));
    TSM_TRY(tp_stream_wait(ctx));  // a plain stream wait on one GPU; bounded, with the communicator polled, in a group
    return check_error_record(ctx);
}

int tsm_counters_read(tsm_ctx* ctx, tsm_counters* out) {
    if (!ctx || !out) return TSM_ERR_ARG;
    *out = ctx->counters;
    std::lock_guard<std::mutex> guard(ctx->pool.lock);
    out->pool_held_bytes = ctx->pool.held_bytes;
    out->host_ops = 0;  // there is no host path to count
    return TSM_OK;
}

int tsm_counters_reset(tsm_ctx* ctx) {
    if (!ctx) return TSM_ERR_ARG;
    ctx->counters = tsm_counters{};
    return TSM_OK;
}

int tsm_profile_begin(tsm_ctx* ctx, int shapes) {
    CTX_GUARD(ctx);
    TSM_TRY(profile_collect(ctx));
    ctx->profile.totals.clear();
    ctx->profile.on = true, ctx->profile.shapes = shapes != 0, ctx->profile.depth = 0;
    return TSM_OK;
}

int tsm_profile_read(tsm_ctx* ctx, tsm_profile_entry* entries, int capacity, int* count) {
    CTX_GUARD(ctx);
    if (!count || capacity < 0 || (capacity > 0 && !entries)) return fail(ctx, TSM_ERR_ARG, "profile_read needs a place for its entries and their count");
    TSM_TRY(profile_collect(ctx));
    // longest total first, as the reference's report lists its operators (cuda/report.cr)
    std::vector<std::pair<std::string, std::pair<int64_t, double>>> rows(ctx->profile.totals.begin(), ctx->profile.totals.end());
    std::sort(rows.begin(), rows.end(), [](const auto& a, const auto& b) { return a.second.second > b.second.second; });
    *count = (int)rows.size();
    for (int i = 0; i < capacity && i < (int)rows.size(); i++) {
        memset(&entries[i], 0, sizeof(tsm_profile_entry));
        strncpy(entries[i].label, rows[i].first.c_str(), sizeof(entries[i].label) - 1);
        entries[i].count = rows[i].second.first;
        entries[i].seconds = rows[i].second.second;
    }
    return TSM_OK;
}

int tsm_profile_end(tsm_ctx* ctx) {
    CTX_GUARD(ctx);
    TSM_TRY(profile_collect(ctx));
    ctx->profile.on = false, ctx->profile.depth = 0;
    return TSM_OK;
}

int tsm_debug_wait_limit(tsm_ctx* ctx, unsigned spins, int starve_copies) {
    if (!ctx) return TSM_ERR_ARG;
    ctx->wait_spins = spins, ctx->starve_copies = starve_copies;
    return TSM_OK;
}

int tsm_set_mode(tsm_ctx* ctx, int mode) {
    if (!ctx || (mode != TSM_FAST && mode != TSM_EXACT)) return TSM_ERR_ARG;
    ctx->mode = mode;
    return TSM_OK;
}

// ---- operators ---------------------------------------------------------------------------------

#define PF(x) ((float*)(uintptr_t)(x))
#define PCF(x) ((const float*)(uintptr_t)(x))
#define PCI(x) ((const int*)(uintptr_t)(x))
#define PCB(x) ((const uint8_t*)(uintptr_t)(x))

int tsm_quantize_blocks(tsm_ctx* ctx, tsm_dptr x, int64_t count, int kind, tsm_dptr out) {
    CTX_GUARD(ctx);
    return launch_quantize_blocks(ctx, PCF(x), count, kind, (uint8_t*)(uintptr_t)out);
}

int tsm_dequantize_blocks(tsm_ctx* ctx, tsm_dptr blocks, int64_t count, int kind, tsm_dptr out) {
    CTX_GUARD(ctx);
    return launch_dequantize_blocks(ctx, PCB(blocks), count, kind, PF(out));
}

int tsm_quantize_rows_q8(tsm_ctx* ctx, tsm_dptr x, int rows, int k, int64_t x_stride, tsm_dptr scales, tsm_dptr sums,
                         tsm_dptr qs) {
    CTX_GUARD(ctx);
    if (k % 32 != 0) return fail(ctx, TSM_ERR_ARG, "rows of " + std::to_string(k) + " do not split into blocks of 32");
    // the per-block integer totals are internal: keep them in the context's scratch
    int64_t blocks = (int64_t)rows * (k / 32);
    TSM_TRY(ensure_scratch(ctx, ctx->quant, blocks * 4 + 256));
    return launch_quantize_rows(ctx, PCF(x), rows, k, x_stride, PF(scales), PF(sums), (int*)ctx->quant.ptr, (int8_t*)(uintptr_t)qs);
}

int tsm_block_matmul(tsm_ctx* ctx, tsm_dptr x, int rows, int k, int64_t x_stride, tsm_dptr w, int kind, int n, tsm_dptr bias,
                     tsm_dptr out) {
    CTX_GUARD(ctx);
    if (k <= 0 || k % 32 != 0) return fail(ctx, TSM_ERR_ARG, "rows of " + std::to_string(k) + " do not split into blocks of 32");
    if (rows < 0 || n < 0) return fail(ctx, TSM_ERR_ARG, "negative size");
    if (rows == 0 || n == 0) return TSM_OK;
    if (rows <= 4) {  // the streamed kernel quantises a few rows itself: one launch
        bool taken = false;
        TSM_TRY(launch_block_matvec_plain(ctx, PCF(x), x_stride, rows, k, PCB(w), kind, n, PCF(bias), nullptr, PF(out), &taken));
        if (taken) return TSM_OK;
    }
    TSM_TRY(ensure_scratch(ctx, ctx->quant, quant_scratch_bytes(rows, k)));
    QuantizedActs a = quant_scratch_layout(ctx->quant.ptr, rows, k);
    TSM_TRY(launch_quantize_rows(ctx, PCF(x), rows, k, x_stride, (float*)a.scales, (float*)a.sums, (int*)a.totals, (int8_t*)a.qs));
    return launch_block_matmul(ctx, a, rows, k, PCB(w), kind, n, PCF(bias), nullptr, PF(out));
}

int tsm_block_matmul_quantized(tsm_ctx* ctx, tsm_dptr scales, tsm_dptr sums, tsm_dptr qs, int rows, int k, tsm_dptr w, int kind,
                               int n, tsm_dptr bias, tsm_dptr out) {
    CTX_GUARD(ctx);
    if (k <= 0 || k % 32 != 0) return fail(ctx, TSM_ERR_ARG, "rows of " + std::to_string(k) + " do not split into blocks of 32");
    if (rows == 0 || n == 0) return TSM_OK;
    if ((qs & 3) != 0) return fail(ctx, TSM_ERR_ARG, "quantised activations must be 4-byte aligned");
    // the products take the blocks' integer sums from the quantised values themselves, so none are passed
    QuantizedActs a{PCF(scales), PCF(sums), nullptr, (const int8_t*)(uintptr_t)qs};
    return launch_block_matmul(ctx, a, rows, k, PCB(w), kind, n, PCF(bias), nullptr, PF(out));
}

int tsm_gather_blocks(tsm_ctx* ctx, tsm_dptr table, int kind, int table_rows, int width, tsm_dptr ids, int count, tsm_dptr out) {
    CTX_GUARD(ctx);
    return launch_gather_blocks(ctx, PCB(table), kind, table_rows, width, PCI(ids), count, PF(out), nullptr, nullptr, 0);
}

int tsm_gather_f32(tsm_ctx* ctx, tsm_dptr table, int table_rows, int width, tsm_dptr ids, int count, tsm_dptr out) {
    CTX_GUARD(ctx);
    return launch_gather_f32(ctx, PCF(table), table_rows, width, PCI(ids), count, PF(out));
}

int tsm_matmul_f32(tsm_ctx* ctx, tsm_dptr x, int rows, int k, tsm_dptr w, int n, tsm_dptr bias, tsm_dptr out) {
    CTX_GUARD(ctx);
    return launch_matmul_f32(ctx, PCF(x), rows, k, PCF(w), n, PCF(bias), nullptr, PF(out));
}

int tsm_rmsnorm(tsm_ctx* ctx, tsm_dptr x, tsm_dptr w, int rows, int n, float eps, tsm_dptr out) {
    CTX_GUARD(ctx);
    return launch_rmsnorm(ctx, PCF(x), PCF(w), rows, n, eps, PF(out), nullptr);
}

int tsm_layernorm(tsm_ctx* ctx, tsm_dptr x, tsm_dptr w, tsm_dptr b, int rows, int n, float eps, tsm_dptr out) {
    CTX_GUARD(ctx);
    return launch_layernorm(ctx, PCF(x), PCF(w), PCF(b), rows, n, eps, PF(out), nullptr);
}

int tsm_rope(tsm_ctx* ctx, tsm_dptr x, int tokens, int heads, int width, int64_t x_stride, tsm_dptr cos_table, tsm_dptr sin_table,
             int context, tsm_dptr positions, tsm_dptr out) {
    CTX_GUARD(ctx);
    return launch_rope(ctx, PCF(x), tokens, heads, width, x_stride, PCF(cos_table), PCF(sin_table), context, PCI(positions), PF(out));
}

int tsm_write_rows(tsm_ctx* ctx, tsm_dptr cache, int rows, int heads, int capacity, int width, tsm_dptr values, int64_t v_stride,
                   int tokens, tsm_dptr slots) {
    CTX_GUARD(ctx);
    return launch_write_rows(ctx, PF(cache), rows, heads, capacity, width, PCF(values), v_stride, tokens, PCI(slots));
}

int tsm_write(tsm_ctx* ctx, tsm_dptr dst, const int32_t* shape, int ndim, tsm_dptr value, int extent, int axis, int start) {
    CTX_GUARD(ctx);
    if (!shape || ndim < 1 || ndim > 8) return fail(ctx, TSM_ERR_ARG, "write takes tensors of 1 to 8 axes");
    if (axis < 0) axis += ndim;
    if (axis < 0 || axis >= ndim) return fail(ctx, TSM_ERR_ARG, "axis out of range");
    int64_t outer = 1, inner = 1;
    for (int i = 0; i < ndim; i++) {
        if (shape[i] < 0) return fail(ctx, TSM_ERR_ARG, "negative size");
        if (i < axis) outer *= shape[i];
        if (i > axis) inner *= shape[i];
    }
    if (extent < 0 || start < 0 || (int64_t)start + extent > shape[axis])
        return fail(ctx, TSM_ERR_ARG, "cannot write " + std::to_string(extent) + " at " + std::to_string(start) + " along an axis of " + std::to_string(shape[axis]));
    return launch_write_region(ctx, PF(dst), PCF(value), outer, (int64_t)shape[axis] * inner, (int64_t)extent * inner, (int64_t)start * inner);
}

int tsm_ragged_attention(tsm_ctx* ctx, tsm_dptr q, int64_t q_stride, int tokens, int heads, int width, tsm_dptr k, tsm_dptr v,
                         int rows, int kv_heads, int capacity, tsm_dptr table, float scale, tsm_dptr out) {
    CTX_GUARD(ctx);
    const int* order = nullptr;
    if (tokens > 1 && tokens <= 4096) {
        TSM_TRY(ensure_scratch(ctx, ctx->order, (int64_t)tokens * 4));
        TSM_TRY(launch_length_order(ctx, PCI(table), tokens, (int*)ctx->order.ptr));
        order = (const int*)ctx->order.ptr;
    }
    return launch_attention(ctx, PCF(q), q_stride, tokens, heads, width, PCF(k), PCF(v), rows, kv_heads, capacity, PCI(table), scale,
                            PF(out), nullptr, order);
}

int tsm_swiglu(tsm_ctx* ctx, tsm_dptr gate, tsm_dptr up, int rows, int n, int64_t in_stride, tsm_dptr out) {
    CTX_GUARD(ctx);
    return launch_swiglu(ctx, PCF(gate), PCF(up), rows, n, in_stride, PF(out), nullptr);
}

int tsm_silu(tsm_ctx* ctx, tsm_dptr x, int64_t count, tsm_dptr out) {
    CTX_GUARD(ctx);
    if (count < 0 || count > 0x7fffffff) return fail(ctx, TSM_ERR_ARG, "silu of more than 2^31 values");
    return launch_silu(ctx, PCF(x), count, PF(out));
}

int tsm_gelu(tsm_ctx* ctx, tsm_dptr x, int64_t count, tsm_dptr out) {
    CTX_GUARD(ctx);
    if (count > 0x7fffffff) return fail(ctx, TSM_ERR_ARG, "gelu of more than 2^31 values");
    return launch_gelu(ctx, PCF(x), 1, (int)count, PF(out), nullptr);
}

int tsm_add(tsm_ctx* ctx, tsm_dptr a, tsm_dptr b, int64_t count, tsm_dptr out) {
    CTX_GUARD(ctx);
    return launch_add(ctx, PCF(a), PCF(b), count, PF(out));
}

int tsm_fill_normal(tsm_ctx* ctx, tsm_dptr out, int64_t count, float mean, float stddev, uint64_t seed) {
    CTX_GUARD(ctx);
    return launch_normal_fill(ctx, PF(out), count, mean, stddev, seed);
}

int tsm_argmax(tsm_ctx* ctx, tsm_dptr logits, int rows, int n, tsm_dptr out) {
    CTX_GUARD(ctx);
    return launch_argmax(ctx, PCF(logits), rows, n, (int*)(uintptr_t)out);
}

int tsm_topk(tsm_ctx* ctx, tsm_dptr logits, int rows, int n, int count, tsm_dptr out_ids, tsm_dptr out_values) {
    CTX_GUARD(ctx);
    return launch_topk(ctx, PCF(logits), rows, n, count, (int*)(uintptr_t)out_ids, PF(out_values));
}

}  // extern "C"
