// Shared declarations of the library: the context, status plumbing and small device helpers.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <utility>
#include <vector>

#include "../../include/tsm_b200.h"

namespace tsm {

constexpr int kBlockBytes[3] = {34, 18, 20};  // Q8_0, Q4_0, Q4_1 (dtype.cr:38-45 of the reference)
inline int block_bytes(int kind) { return kBlockBytes[kind]; }

// The 3-int record kernels write for bad data (count, first id, limit), as the reference's
// kernels do (kernels.cu:178-183), plus a fourth word for bounded waits that ran out.
struct ErrorRecord {
    int count, first, limit, timeout;
};

// Exact-size free lists, as the reference's BufferPool keeps them (buffer_pool.cr:37-72).
struct Pool {
    std::mutex lock;
    std::unordered_map<int64_t, std::vector<void*>> free_lists;
    std::unordered_map<void*, int64_t> sizes;  // every live or pooled allocation
    int64_t held_bytes = 0, limit_bytes = 0;
};

struct Scratch {
    void* ptr = nullptr;
    int64_t bytes = 0;
};

// Per-operator GPU time, collected while tsm_profile_begin is in force: every launcher brackets its kernels with two
// events (OpTimer below); tsm_profile_read waits for the stream and adds the elapsed times up by label.
struct ProfileSpan {
    std::string label;
    cudaEvent_t start, stop;
};
struct Profile {
    bool on = false, shapes = false;
    std::vector<ProfileSpan> spans;          // recorded, not yet read
    std::vector<cudaEvent_t> spare;          // events ready for reuse
    std::map<std::string, std::pair<int64_t, double>> totals;  // label -> (count, seconds), from spans already read
    int depth = 0;                           // launchers nest (a product calls its quantiser): only the outermost is timed
};

}  // namespace tsm

struct tsm_ctx {
    int ordinal = 0;
    cudaStream_t stream = nullptr;
    int sm_count = 148;
    int mode = TSM_EXACT;
    tsm::Pool pool;
    tsm::ErrorRecord* errors = nullptr;       // device
    tsm::ErrorRecord* errors_host = nullptr;  // pinned
    tsm::Scratch quant;                       // activation quantiser output for tsm_block_matmul
    tsm::Scratch attn;                        // split-K partials
    tsm::Scratch order;                       // attention's longest-first token order (operator-level calls)
    uint64_t scratch_generation = 1;          // bumped whenever a scratch buffer moves
    int tp_rank = 0, tp_world = 1;            // this context's place in a tensor-parallel group
    bool chain_launches = false;              // the engine sets it around steps of a few rows (see launch_chained)
    const int* prefill_tiles = nullptr;       // set by the engine around a step that holds prompts: query tiles of 16 consecutive
    int prefill_tile_count = 0;               //   tokens of one stream (first token, count), longest first, in device memory
    void* comm = nullptr;                     // its NCCL communicator
    bool comm_failed = false;                 // an exchange failed or the group was aborted: every later one is refused
    int tp_variant = 0;                       // TSM_TP_GATHER or TSM_TP_REDUCE: how models built on this context are split
    std::mutex message_lock;
    std::string message;
    tsm_counters counters{};
    std::mutex counter_lock;
    tsm::Profile profile;
    unsigned wait_hint = 0;                   // TSM_WAIT_HINT_NS: nanoseconds a thread waiting on an mbarrier may sleep per poll
    unsigned wait_spins = 0;                  // tsm_debug_wait_limit: a shorter limit for the kernels' bounded waits (0: theirs)
    int starve_copies = 0;                    //                       and a stage the next product's producer leaves out
};

namespace tsm {

void set_message(tsm_ctx* ctx, const std::string& text);
int fail(tsm_ctx* ctx, int status, const std::string& text);
int cuda_fail(tsm_ctx* ctx, cudaError_t err, const char* what);
int ensure_scratch(tsm_ctx* ctx, Scratch& s, int64_t bytes);
int check_error_record(tsm_ctx* ctx);  // inspects the host copy of the record; clears the device's when set
int pool_alloc(tsm_ctx* ctx, int64_t bytes, void** out);
void pool_release(tsm_ctx* ctx, void* p);
inline void count_launch(tsm_ctx* ctx, int n = 1) { ctx->counters.launches += n; }

// Brackets the kernels a launcher queues with two events while the context's profile is on (and the stream is not being
// captured: a captured step cannot be timed node by node, so tsm_decode runs its step uncaptured under a profile).
// `label` is the operator's name; with shapes on, the sizes follow it, as the reference's per-kernel profile keys
// "MatMul [64,768]x[768,2304]" (cuda.cr:256-303, 463-477).
struct OpTimer {
    tsm_ctx* ctx;
    bool active = false;
    bool dropped = false;  // set by a launcher that queued nothing after all: the span is not recorded
    cudaEvent_t start = nullptr;
    std::string label;
    OpTimer(tsm_ctx* c, const char* name, int64_t a = -1, int64_t b = -1, int64_t d = -1);
    ~OpTimer();
};

// A launch that may begin while the kernel before it on the stream is still draining (programmatic dependent launch): the
// kernel's blocks are scheduled as soon as every block of its predecessor has started, run nothing but
// `chained_kernel_entry()` until the predecessor has finished and its writes are visible, and only then touch memory that a
// kernel writes (the streamed matvec starts the copies of its first weights before it waits: weights are written by no kernel
// of a step).  Every kernel launched through here calls chained_kernel_entry(), or its two halves, before anything else.
// The attribute is set only while the context's `chain_launches` is on, which the engine does for steps of at most 4 rows: measured, a batch-1 step of ~300
// very short kernels gains 5 %, while steps of 16 and 64 rows lose 9 % and 1 % (early blocks hold SM resources while they
// wait).  TSM_CHAINED_LAUNCH=0 turns it off everywhere.
bool chained_launch_enabled();
template <typename... Params, typename... Args>
inline cudaError_t launch_chained(tsm_ctx* ctx, void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid, config.blockDim = block, config.dynamicSmemBytes = smem, config.stream = ctx->stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = ctx->chain_launches && chained_launch_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&config, kernel, Params(std::forward<Args>(args))...);
}

#define TSM_CUDA(ctx, call)                                              \
    do {                                                                 \
        cudaError_t err__ = (call);                                      \
        if (err__ != cudaSuccess) return tsm::cuda_fail(ctx, err__, #call); \
    } while (0)

#define TSM_TRY(call)              \
    do {                           \
        int rc__ = (call);         \
        if (rc__ != TSM_OK) return rc__; \
    } while (0)

#define TSM_LAUNCH_CHECK(ctx) TSM_CUDA(ctx, cudaGetLastError())

struct DeviceGuard {
    int previous = -1;
    explicit DeviceGuard(int ordinal) {
        cudaGetDevice(&previous);
        if (previous != ordinal) cudaSetDevice(ordinal);
        else previous = -1;
    }
    ~DeviceGuard() {
        if (previous >= 0) cudaSetDevice(previous);
    }
};

// ---- launch declarations (each in its own .cu) -------------------------------------------------

struct QuantizedActs {
    const float* scales;  // [rows, k/32]  f32(f16(d))
    const float* sums;    // [rows, k/32]  f32(f16(total * d))
    const int* totals;    // [rows, k/32]  integer sum of the block's quantised values
    const int8_t* qs;     // [rows, k]
};

// Where a kernel that also quantises its output rows writes them (all null: it does not).
struct QuantSink {
    float* scales;
    float* sums;
    int* totals;
    int8_t* qs;
};
inline QuantSink quant_sink(const QuantizedActs* q) {
    QuantSink o{nullptr, nullptr, nullptr, nullptr};
    if (q) o = QuantSink{(float*)q->scales, (float*)q->sums, (int*)q->totals, (int8_t*)q->qs};
    return o;
}

int64_t quant_scratch_bytes(int rows, int k);
QuantizedActs quant_scratch_layout(void* base, int rows, int k);

int launch_quantize_rows(tsm_ctx* ctx, const float* x, int rows, int k, int64_t x_stride, float* scales, float* sums,
                         int* totals, int8_t* qs);
int launch_block_matmul(tsm_ctx* ctx, const QuantizedActs& a, int rows, int k, const uint8_t* w, int kind, int n,
                        const float* bias, const float* residual, float* out);
// A product of at most 4 F32 rows that quantises them itself, in every CTA of the streamed kernel (the quantiser's arithmetic,
// so the same bits): one launch instead of two.  `taken` false: the shape is not one the streamed kernel serves, nothing
// was launched.
int launch_block_matvec_plain(tsm_ctx* ctx, const float* x, int64_t x_stride, int rows, int k, const uint8_t* w, int kind, int n,
                              const float* bias, const float* residual, float* out, bool* taken);
bool mma_product_fits(const QuantizedActs& a, int rows, int k, const uint8_t* w, int kind, int n);
// Tensor-parallel exchanges (collective.cu).
int tp_all_gather(tsm_ctx* ctx, void* buffer, int64_t bytes);
int tp_all_reduce_sum(tsm_ctx* ctx, float* buffer, int64_t count);
int launch_interleave(tsm_ctx* ctx, const float* gathered, float* dst, int rows, int width, int parts, bool add);
void tp_release(tsm_ctx* ctx);
void tp_abort(tsm_ctx* ctx);
int tp_stream_wait(tsm_ctx* ctx);  // the stream wait of a group member: bounded, polls the communicator for failures
// A rank-2 tensor map over `rows` rows of `width` elements (row pitch in bytes), copied in boxes of box_w x box_h.
bool tensor_maps_available();
int make_tensor_map_2d(tsm_ctx* ctx, CUtensorMap* map, CUtensorMapDataType type, const void* base, uint64_t width, uint64_t rows,
                       uint64_t pitch_bytes, uint32_t box_w, uint32_t box_h, CUtensorMapSwizzle swizzle);
int64_t attention_stream_scratch_bytes(int tokens, int heads, int capacity);
bool attention_stream_fits(tsm_ctx* ctx, int tokens, int heads, int width, int kv_heads, const float* q, int64_t q_stride, const float* k,
                           const float* v);
int launch_attention_stream(tsm_ctx* ctx, const float* q, int64_t q_stride, int tokens, int heads, const float* k, const float* v,
                            int rows, int kv_heads, int capacity, const int* table, float scale, float* out, const int* order,
                            float* scratch, QuantSink sink);
int launch_attention_prefill(tsm_ctx* ctx, const float* q, int64_t q_stride, int tokens, int heads, const float* k, const float* v, int rows,
                             int kv_heads, int capacity, const int* table, float scale, float* out, float* scratch, QuantSink sink,
                             const int* qtiles, int tile_count);
bool pipe_product_fits(const QuantizedActs& a, int rows, int k, const uint8_t* w, int kind, int n);
int launch_block_matmul_pipe(tsm_ctx* ctx, const QuantizedActs& a, int rows, int k, const uint8_t* w, int kind, int n,
                             const float* bias, const float* residual, float* out);
bool umma_product_fits(const QuantizedActs& a, int rows, int k, const uint8_t* w, int kind, int n);
int launch_block_matmul_umma(tsm_ctx* ctx, const QuantizedActs& a, int rows, int k, const uint8_t* w, int kind, int n,
                             const float* bias, const float* residual, float* out);
int launch_block_matmul_mma(tsm_ctx* ctx, const QuantizedActs& a, int rows, int k, const uint8_t* w, int kind, int n,
                            const float* bias, const float* residual, float* out);
int launch_quantize_blocks(tsm_ctx* ctx, const float* x, int64_t count, int kind, uint8_t* out);
int launch_dequantize_blocks(tsm_ctx* ctx, const uint8_t* blocks, int64_t count, int kind, float* out);
int launch_gather_blocks(tsm_ctx* ctx, const uint8_t* table, int kind, int table_rows, int width, const int* ids,
                         int count, float* out, const uint8_t* table2, const int* ids2, int ids2_stride);
// With a second table (GPT-2's positions) the two rows are added: table[ids[t]] + table2[ids2[t * ids2_stride]].
int launch_gather_f32(tsm_ctx* ctx, const float* table, int table_rows, int width, const int* ids, int count, float* out,
                      const float* table2 = nullptr, const int* ids2 = nullptr, int ids2_stride = 0);
// The unquantised product x [rows, k] by w [n, k] -> out [rows, n], sums over k in index order; bias, residual may be null.
int launch_matmul_f32(tsm_ctx* ctx, const float* x, int rows, int k, const float* w, int n, const float* bias, const float* residual,
                      float* out);
int launch_rmsnorm(tsm_ctx* ctx, const float* x, const float* w, int rows, int n, float eps, float* out,
                   const QuantizedActs* quantized);
int launch_layernorm(tsm_ctx* ctx, const float* x, const float* w, const float* b, int rows, int n, float eps, float* out,
                     const QuantizedActs* quantized);
// Op::Write: `outer` runs of `chunk` floats of src, run o landing at dst[o * pitch + offset ...].
int launch_write_region(tsm_ctx* ctx, float* dst, const float* src, int64_t outer, int64_t pitch, int64_t chunk, int64_t offset);
int launch_rope(tsm_ctx* ctx, const float* x, int tokens, int heads, int width, int64_t x_stride, const float* cos_table,
                const float* sin_table, int context, const int* positions, float* out);
int launch_write_rows(tsm_ctx* ctx, float* cache, int rows, int heads, int capacity, int width, const float* values,
                      int64_t v_stride, int tokens, const int* slots);
// Rotates q and k in place inside qkv [tokens, (heads + 2 kv_heads) * width] (when cos_table is not null) and
// writes k and v to their cache slots (table[t] = row, position, ...): one launch per layer.
int launch_rope_append(tsm_ctx* ctx, float* qkv, int tokens, int heads, int kv_heads, int width, const float* cos_table,
                       const float* sin_table, int context, const int* table, float* keys, float* values, int rows,
                       int capacity);
// A decode step's rope + cache append done by the attention kernel itself (modules.cr:434-452 then 194-217): `q` is then the
// joined [q; k; v] row of each token, un-rotated; every CTA rotates its query heads and its kv head's new key as it loads
// them, the first CTA of a kv head writes key and value to the cache at the token's position, and every CTA uses its own
// copy of them for that position.  Only for steps in which each cache row receives ONE token (a token's CTAs never read what
// another token's CTAs write).  Kernels that do not serve it get the separate rope + append launch first.
struct FreshRows {
    const float* cos_table;  // null: no rotation (GPT-2)
    const float* sin_table;
    int context;             // positions the tables hold
};
int launch_attention(tsm_ctx* ctx, const float* q, int64_t q_stride, int tokens, int heads, int width, const float* k,
                     const float* v, int rows, int kv_heads, int capacity, const int* table, float scale, float* out,
                     const QuantizedActs* quantized, const int* order, const FreshRows* fresh = nullptr);
// order[r] = the token with the r-th most visible positions (ties by index), so that attention can start its
// longest tokens first; null means token order.
int launch_length_order(tsm_ctx* ctx, const int* table, int tokens, int* order);
int64_t attention_scratch_bytes(int tokens, int heads, int width, int capacity);
int launch_swiglu(tsm_ctx* ctx, const float* gate, const float* up, int rows, int n, int64_t in_stride, float* out,
                  const QuantizedActs* quantized);
int launch_gelu(tsm_ctx* ctx, const float* x, int rows, int n, float* out, const QuantizedActs* quantized);
int launch_silu(tsm_ctx* ctx, const float* x, int64_t count, float* out);
int launch_add(tsm_ctx* ctx, const float* a, const float* b, int64_t count, float* out);
int launch_argmax(tsm_ctx* ctx, const float* logits, int rows, int n, int* out);
int launch_topk(tsm_ctx* ctx, const float* logits, int rows, int n, int count, int* out_ids, float* out_values);
int launch_normal_fill(tsm_ctx* ctx, float* out, int64_t count, float mean, float stddev, uint64_t seed);
int launch_fill(tsm_ctx* ctx, float* out, int64_t count, float value);

}  // namespace tsm

// ---- device helpers ---------------------------------------------------------------------------
#ifdef __CUDACC__
namespace tsm {

// f32(f16(x)) with round-to-nearest-even, as the reference's F16.new(...).to_f32 (f16.cr:29-59).
__device__ __forceinline__ float round_to_half(float x) { return __half2float(__float2half_rn(x)); }
__device__ __forceinline__ float half_bits_to_float(unsigned int bits) {
    return __half2float(__ushort_as_half((unsigned short)bits));
}

// The reference's own exp (maths.cr:36-54), operation for operation; no contraction.
// First statement of every kernel launched with launch_chained: waits for the kernel before it (complete, writes visible),
// then lets the kernel after it be scheduled.  A no-op under an ordinary launch.  (Letting the successor in BEFORE the wait,
// so that several kernels' blocks queue up on the SMs, measured 8 % slower on a batch-1 step of 300 kernels.)
__device__ __forceinline__ void chained_kernel_entry() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
// The same with room before the wait for work that reads nothing a kernel writes (the streamed matvec starts the copies of
// its first weights there).
__device__ __forceinline__ void chained_kernel_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ float exact_exp(float x) {
    const float LOG2E = 1.44269504088896341f, LN2_HI = 0.693359375f, LN2_LO = -2.12194440e-4f;
    const float EXP_HI = 88.72283905f, EXP_LO = -87.3365447f, ROUNDER = 12582912.0f;
    float clamped = (x > EXP_HI || x < EXP_LO) ? 0.0f : x;
    float n = __fsub_rn(__fadd_rn(__fmul_rn(clamped, LOG2E), ROUNDER), ROUNDER);
    float r = __fsub_rn(__fsub_rn(clamped, __fmul_rn(n, LN2_HI)), __fmul_rn(n, LN2_LO));
    float z = __fmul_rn(r, r);
    float p = 1.9875691500e-4f;
    p = __fadd_rn(__fmul_rn(p, r), 1.3981999507e-3f);
    p = __fadd_rn(__fmul_rn(p, r), 8.3334519073e-3f);
    p = __fadd_rn(__fmul_rn(p, r), 4.1665795894e-2f);
    p = __fadd_rn(__fmul_rn(p, r), 1.6666665459e-1f);
    p = __fadd_rn(__fmul_rn(p, r), 5.0000001201e-1f);
    p = __fadd_rn(__fadd_rn(__fmul_rn(p, z), r), 1.0f);
    int whole = (int)n;
    int half = whole >> 1;
    float result = __fmul_rn(__fmul_rn(p, __int_as_float((half + 127) << 23)), __int_as_float((whole - half + 127) << 23));
    result = x > EXP_HI ? __int_as_float(0x7f800000) : result;
    result = x < EXP_LO ? 0.0f : result;
    return x != x ? x : result;
}

// The reference's own tanh (maths.cr:99-114).
__device__ __forceinline__ float exact_tanh(float x) {
    float a = fabsf(x);
    float z = __fmul_rn(x, x);
    float p = -5.70498872745e-3f;
    p = __fadd_rn(__fmul_rn(p, z), 2.06390887954e-2f);
    p = __fsub_rn(__fmul_rn(p, z), 5.37397155531e-2f);
    p = __fadd_rn(__fmul_rn(p, z), 1.33314422036e-1f);
    p = __fsub_rn(__fmul_rn(p, z), 3.33332819422e-1f);
    float near = __fadd_rn(__fmul_rn(__fmul_rn(p, z), x), x);
    float far = __fsub_rn(1.0f, __fdiv_rn(2.0f, __fadd_rn(exact_exp(__fadd_rn(a, a)), 1.0f)));
    far = a > 9.01f ? 1.0f : far;
    far = x < 0.0f ? -far : far;
    float result = a < 0.625f ? near : far;
    result = x == 0.0f ? x : result;
    return x != x ? x : result;
}

// One warp quantises one block of 32 activations, lane j holding element j, with the arithmetic of
// the reference's Quant.quantize_activations (quant.cr:428-442): d = amax / 127, id = 1 / d (IEEE
// division), q = round-half-away(x * id), scale = f32(f16(d)), sum = f32(f16(float(total) * d)).
__device__ __forceinline__ void quantize_block_q8(float x, int lane, float* scale, float* sum, int* total, int8_t* q_out) {
    float amax = fabsf(x);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
    float d = __fdiv_rn(amax, 127.0f);
    float id = d == 0.0f ? 0.0f : __fdiv_rn(1.0f, d);
    int q = (int)(signed char)(int)roundf(__fmul_rn(x, id));
    int t = q;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) t += __shfl_xor_sync(0xffffffffu, t, off);
    *q_out = (int8_t)q;
    if (lane == 0) {
        *scale = round_to_half(d);
        *sum = round_to_half(__fmul_rn((float)t, d));
        *total = t;
    }
}

__device__ __forceinline__ void report_bad_index(ErrorRecord* errors, int id, int limit) {
    if (atomicAdd(&errors->count, 1) == 0) {
        errors->first = id;
        errors->limit = limit;
    }
}

}  // namespace tsm
#endif
