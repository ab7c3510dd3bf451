/*
 * tsm_b200 — C ABI of the B200-native decode engine for tensomite's quantised token loop.
 *
 * Everything here is plain C: opaque handles, 64-bit device addresses, pointers and sizes.
 * Each entry point names the tensomite interface it stands in for (path within the
 * tensomite project : lines), so that a Crystal `lib` binding can replace the calls that
 * `Tensomite::CUDA` makes today (src/tensomite/cuda.cr, src/tensomite/cuda/lib.cr).
 *
 * Conventions
 *  - Every function returns a tsm_status (0 = ok).  The text of the last failure on a
 *    context is read with tsm_last_error, as CUDA.check builds its DeviceError message
 *    (cuda.cr:1070-1075).
 *  - Every function binds its context's device itself and keeps no thread-local state, so
 *    it may be called from any thread (Crystal fibers migrate: cuda.cr:1118-1125).
 *  - Kernels never trap on bad data.  An out-of-range row id is recorded in a 3-int error
 *    record (count, first id, limit) that tsm_sync reads and clears, returning
 *    TSM_ERR_EXECUTION (kernels.cu:178-183, cuda.cr:967-983).
 *  - All work of a context runs on one in-order stream, as the reference's CUDA device does
 *    (one stream per device, cuda.cr:200-253).
 *  - There is no CPU implementation behind any entry point: without a CUDA device every
 *    compute call fails with TSM_ERR_CUDA.
 */
#ifndef TSM_B200_H
#define TSM_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tsm_ctx tsm_ctx;     /* one device: context, stream, pool, scratch (cuda.cr:200-253) */
typedef struct tsm_model tsm_model; /* a Llama or GPT-2 with its weights resident (models/llama.cr, models/gpt2.cr) */
typedef struct tsm_cache tsm_cache; /* Generative::BatchCache (models/generative.cr:54-79) */
typedef uint64_t tsm_dptr;          /* a device address, as cuda/lib.cr passes CUdeviceptr (UInt64) */

typedef enum {
    TSM_OK = 0,
    TSM_ERR_CUDA = 1,        /* a CUDA call failed (DeviceError) */
    TSM_ERR_ARG = 2,         /* a shape, size or pointer the call cannot take (ShapeError / ArgumentError) */
    TSM_ERR_EXECUTION = 3,   /* a kernel met bad data, e.g. an index out of range (ExecutionError) */
    TSM_ERR_MEMORY = 4,      /* the device has no room */
    TSM_ERR_IO = 5,          /* a model file could not be read or is malformed (Tensomite::Error) */
    TSM_ERR_UNSUPPORTED = 6, /* a dtype or layout this build does not handle (DTypeError) */
    TSM_ERR_TIMEOUT = 7,     /* a bounded device-side wait ran out */
    TSM_ERR_COMM = 8         /* the tensor-parallel communicator failed */
} tsm_status;

/* Block formats, numbered as the reference's kernels number them (kernels.cu:1160-1168). */
typedef enum { TSM_Q8_0 = 0, TSM_Q4_0 = 1, TSM_Q4_1 = 2, TSM_F32 = -1 } tsm_kind;

/* ---- runtime: Device#alloc/upload/download/sync (device.cr:39-68; cuda.cr:339-428) ---------- */

int tsm_device_count(int* count);
int tsm_ctx_create(int ordinal, tsm_ctx** out);
int tsm_ctx_destroy(tsm_ctx* ctx);
const char* tsm_status_name(int status);
int tsm_last_error(tsm_ctx* ctx, char* buffer, int capacity);
void* tsm_ctx_stream(tsm_ctx* ctx); /* the context's cudaStream_t, for callers that share it */

/* Device#alloc: contents undefined; sizes are pooled by exact size (buffer_pool.cr:37-72). */
int tsm_alloc(tsm_ctx* ctx, int64_t bytes, tsm_dptr* out);
/* CUDABuffer#give_back -> retire (cuda.cr:439-454): callable from any thread, never waits or raises. */
int tsm_free(tsm_ctx* ctx, tsm_dptr ptr);
int tsm_upload(tsm_ctx* ctx, tsm_dptr dst, const void* src, int64_t bytes);   /* Device#upload */
int tsm_download(tsm_ctx* ctx, void* dst, tsm_dptr src, int64_t bytes);       /* Device#download */
int tsm_sync(tsm_ctx* ctx);                                                    /* Device#sync, cuda.cr:419-428 */

/* The counters of CUDA::Profile and BufferPool (cuda.cr:215-230, 256-303; buffer_pool.cr:13-34). */
typedef struct {
    int64_t launches, uploads, downloads, upload_bytes, download_bytes;
    int64_t allocs, pool_hits, pool_misses, pool_held_bytes, frees;
    int64_t host_ops;     /* always 0: no operator has a host fallback (fused_llama_spec.cr:82-90) */
    int64_t graph_replays;
    int64_t collectives;  /* exchanges queued between the GPUs of a tensor-parallel group (no counterpart in the reference) */
} tsm_counters;
int tsm_counters_read(tsm_ctx* ctx, tsm_counters* out);
int tsm_counters_reset(tsm_ctx* ctx);

/* CUDA::Profile with per_kernel (and shapes) set (cuda.cr:256-303, 463-477; cuda/report.cr): between tsm_profile_begin and
 * tsm_profile_end every operator's kernels are bracketed by two events on the context's stream; tsm_profile_read waits for
 * the stream and returns, longest total first, each operator's launches and GPU seconds, keyed by its name ("BlockMatMul
 * q4_0", "RaggedAttention", ...) and, with `shapes`, its sizes too ("BlockMatMul q4_0 [64,4096,28672]").  *count receives
 * how many labels there are; at most `capacity` are written.  While a profile is on, tsm_decode and tsm_decode_run launch
 * their steps kernel by kernel instead of replaying the captured graph, whose nodes cannot be timed one by one. */
typedef struct {
    char label[80];
    int64_t count;
    double seconds;
} tsm_profile_entry;
int tsm_profile_begin(tsm_ctx* ctx, int shapes);
int tsm_profile_read(tsm_ctx* ctx, tsm_profile_entry* entries, int capacity, int* count);
int tsm_profile_end(tsm_ctx* ctx);

/* For tests of the bounded device-side waits (no counterpart in the reference, whose kernels do not wait): `spins` replaces
 * the number of polls after which a kernel's wait for an asynchronous copy gives up (0: the built-in limit), and with
 * `starve_copies` = 1 the next batched products' copy threads leave out the last stage of their operands, so the warps
 * waiting for it run into that limit, set the record's timeout word, and return; tsm_sync then gives TSM_ERR_TIMEOUT.
 * Nothing traps and the context stays usable.  Call again with (0, 0) to restore. */
int tsm_debug_wait_limit(tsm_ctx* ctx, unsigned spins, int starve_copies);

/* How norms and attention add (both modes keep the block products bit-exact):
 *   TSM_EXACT  (default) the host's index-order sums and its own exp polynomial: the host's bits, so
 *              whole-model logits and greedy tokens equal the CPU device's;
 *   TSM_FAST   tree sums and split-K online softmax: each op within 1e-5 of the host, but a last-bit
 *              difference can flip an 8-bit activation, so logits follow the host only statistically
 *              (the reference's own GPU budget: 0.001 nats of KL per token). */
typedef enum { TSM_FAST = 0, TSM_EXACT = 1 } tsm_mode;
int tsm_set_mode(tsm_ctx* ctx, int mode);

/* ---- operators: one launcher per hot Op (node.cr:3-127; CUDA#launch, cuda.cr:486-502) ------- */

/* Tensor#quantize / Quant.quantize (quant.cr:77-90, 499-535): `count` F32 values -> ggml blocks. */
int tsm_quantize_blocks(tsm_ctx* ctx, tsm_dptr x, int64_t count, int kind, tsm_dptr out);
/* Tensor#dequantize / Quant.dequantize (quant.cr:93-105, 537-556). */
int tsm_dequantize_blocks(tsm_ctx* ctx, tsm_dptr blocks, int64_t count, int kind, tsm_dptr out);

/* quantize_rows_q8_f32 (kernels.cu:1190-1207; Quant.quantize_activations, quant.cr:428-442):
 * x [rows,k] F32 (row stride x_stride floats) -> scales, sums F32 [rows,k/32], qs I8 [rows,k]. */
int tsm_quantize_rows_q8(tsm_ctx* ctx, tsm_dptr x, int rows, int k, int64_t x_stride, tsm_dptr scales, tsm_dptr sums,
                         tsm_dptr qs);

/* Op::BlockMatMul (Tensor#linear, tensor/structural.cr:165-172; CUDA#launch_blocks, cuda.cr:736-769;
 * Quant.matmul_reference, quant.cr:122-142): out[rows,n] = x[rows,k] . w[n,k]^T (+ bias[n]) with the
 * host's bits.  w holds n rows of k/32 ggml blocks of `kind`, starting at an even address. */
int tsm_block_matmul(tsm_ctx* ctx, tsm_dptr x, int rows, int k, int64_t x_stride, tsm_dptr w, int kind, int n,
                     tsm_dptr bias, tsm_dptr out);
/* The product alone, on activations already quantised by tsm_quantize_rows_q8 (block_matmul_f32 /
 * block_matmul_lanes_f32, kernels.cu:1233-1328). */
int tsm_block_matmul_quantized(tsm_ctx* ctx, tsm_dptr scales, tsm_dptr sums, tsm_dptr qs, int rows, int k, tsm_dptr w,
                               int kind, int n, tsm_dptr bias, tsm_dptr out);
/* Op::MatMul of a Linear whose weight stayed F32 (Tensor#linear on an F32 leaf; host matmul, devices/host.cr:700-721;
 * matmul_f32, kernels.cu:357-375): out[rows,n] = x[rows,k] . w[n,k]^T (+ bias[n]); every output adds its k products in
 * index order, product and sum rounded separately, so the bits are the host's.  bias may be 0. */
int tsm_matmul_f32(tsm_ctx* ctx, tsm_dptr x, int rows, int k, tsm_dptr w, int n, tsm_dptr bias, tsm_dptr out);

/* tsm_block_matmul without any allocation (no counterpart in the reference, whose CUDA device allocates its
 * scratch from a pool on demand, cuda.cr:791-798).  For callers that cannot allocate device memory while they
 * run: latency-bound serving threads (cudaMalloc can take milliseconds and synchronise the device) and processes
 * whose device memory is handed out once at start-up.  The 8-bit activations are quantised into a fixed array inside the library
 * (1.5 MB per GPU that loads it, held until the process ends), so rows * k may be at most 1,048,576; larger
 * products are refused with TSM_ERR_ARG.  The first call on a device looks the array's address up, so make that
 * call before starting any stream capture.  Every call uses the same array, which keeps whatever the last call
 * left there: two calls whose kernels overlap on the GPU (different contexts or streams of one device) race. */
int tsm_block_matmul_static(tsm_ctx* ctx, tsm_dptr x, int rows, int k, int64_t x_stride, tsm_dptr w, int kind, int n,
                            tsm_dptr bias, tsm_dptr out);

/* Op::Gather on a block table (gather_blocks_f32, kernels.cu:1172-1185; Quant.gather, quant.cr:417-422):
 * out[count,width] = dequantised rows ids[i] of table[table_rows,width]; a bad id is recorded, its row zeroed. */
int tsm_gather_blocks(tsm_ctx* ctx, tsm_dptr table, int kind, int table_rows, int width, tsm_dptr ids, int count,
                      tsm_dptr out);
/* Op::Gather on an F32 table (gather_f32, kernels.cu:186-197). */
int tsm_gather_f32(tsm_ctx* ctx, tsm_dptr table, int table_rows, int width, tsm_dptr ids, int count, tsm_dptr out);

/* Op::RMSNorm (Tensor#rmsnorm, tensor/composite.cr:153-159; rmsnorm_f32, kernels.cu:930-956). w may be 0. */
int tsm_rmsnorm(tsm_ctx* ctx, tsm_dptr x, tsm_dptr w, int rows, int n, float eps, tsm_dptr out);
/* Op::LayerNorm (Tensor#layernorm, tensor/composite.cr:89-98; layernorm_f32, kernels.cu:904-923). */
int tsm_layernorm(tsm_ctx* ctx, tsm_dptr x, tsm_dptr w, tsm_dptr b, int rows, int n, float eps, tsm_dptr out);

/* Op::Rope (Tensor#rope, tensor/composite.cr:254-261; rope_f32, kernels.cu:1102-1112) in its packed form
 * (RotaryEmbedding#angles + #call, modules.cr:355-368): x [tokens,heads,width] with token stride x_stride,
 * rotated by rows positions[token] of the cos/sin tables [context,width]. out is dense [tokens,heads,width]. */
int tsm_rope(tsm_ctx* ctx, tsm_dptr x, int tokens, int heads, int width, int64_t x_stride, tsm_dptr cos_table,
             tsm_dptr sin_table, int context, tsm_dptr positions, tsm_dptr out);

/* Op::WriteRows (Tensor#write_rows, tensor/structural.cr:82-92; write_rows_f32, kernels.cu:68-76):
 * token t of values [tokens,heads,width] (token stride v_stride) -> cache[row,head,position,:],
 * slots[t] = row * capacity + position; cache is [rows,heads,capacity,width]. */
int tsm_write_rows(tsm_ctx* ctx, tsm_dptr cache, int rows, int heads, int capacity, int width, tsm_dptr values,
                   int64_t v_stride, int tokens, tsm_dptr slots);

/* Op::Write (Tensor#write, tensor/structural.cr:64-74; copy_into_f32, kernels.cu:59-63): `value`, dense, with dst's shape
 * except `extent` along `axis`, is written into dst (dense, `ndim` <= 8 axes of `shape`) at `start` along `axis`, in place:
 * what the single-stream CausalSelfAttention::Cache does for each step's keys and values (modules.cr:137-188). */
int tsm_write(tsm_ctx* ctx, tsm_dptr dst, const int32_t* shape, int ndim, tsm_dptr value, int extent, int axis, int start);

/* Op::RaggedAttention (Tensor.ragged_attention, tensor/composite.cr:210-227; attention_ragged_f32,
 * kernels.cu:1081-1097) and, with one row, Op::Attention (attention_f32, kernels.cu:1058-1073):
 * q [tokens,heads,width] (token stride q_stride); k, v [rows,kv_heads,capacity,width];
 * table I32 [tokens,3] = (row, last visible position, positions held); out dense [tokens,heads,width].
 * No limit on positions (the reference stops at 4096). */
int tsm_ragged_attention(tsm_ctx* ctx, tsm_dptr q, int64_t q_stride, int tokens, int heads, int width, tsm_dptr k,
                         tsm_dptr v, int rows, int kv_heads, int capacity, tsm_dptr table, float scale, tsm_dptr out);

/* Tensor#swiglu / #gelu (kernels.cr:4,18): elementwise over [rows,n]; strides in floats. */
int tsm_swiglu(tsm_ctx* ctx, tsm_dptr gate, tsm_dptr up, int rows, int n, int64_t in_stride, tsm_dptr out);
int tsm_gelu(tsm_ctx* ctx, tsm_dptr x, int64_t count, tsm_dptr out);
/* Tensor#silu (kernels.cr:15): x / (exp(-x) + 1) with the reference's own exp. */
int tsm_silu(tsm_ctx* ctx, tsm_dptr x, int64_t count, tsm_dptr out);
/* Op::Add (tensor/elementwise.cr:4-6). */
int tsm_add(tsm_ctx* ctx, tsm_dptr a, tsm_dptr b, int64_t count, tsm_dptr out);

/* Init.normal (module.cr; builder.cr:43-45): `count` F32 values drawn N(mean, stddev) on the device by a
 * counter-based generator, element i depending only on (seed, i). */
int tsm_fill_normal(tsm_ctx* ctx, tsm_dptr out, int64_t count, float mean, float stddev, uint64_t seed);

/* Sampler#pick, greedy (sampler.cr:36): first index of each row's maximum -> I32 [rows]. */
int tsm_argmax(tsm_ctx* ctx, tsm_dptr logits, int rows, int n, tsm_dptr out);
/* Sampler#top (sampler.cr:77-96): each row's `count` highest, highest first, ties to the lower index. */
int tsm_topk(tsm_ctx* ctx, tsm_dptr logits, int rows, int n, int count, tsm_dptr out_ids, tsm_dptr out_values);

/* ---- engine: the token loop (models/generative.cr, models/llama.cr, models/gpt2.cr) --------- */

typedef struct {
    int arch;                 /* 0 Llama, 1 GPT-2 */
    int layers, width, heads, kv_heads, head_width, hidden, vocab, context;
    float eps;
    double rope_theta;
    int tied;                 /* the head reuses the token table (llama.cr:294-303; always for GPT-2) */
} tsm_model_config;

/* Llama.load / GPT2.load of a .gguf file (llama.cr:165-206, gpt2.cr:75-89): reads the configuration
 * from the metadata, uploads every tensor, un-permutes q/k rows, joins [q;k;v] and [gate;up].  Matrices may be
 * Q8_0, Q4_0, Q4_1 or F32 (F16 / BF16 are widened to F32, gguf.cr:112-136); a Linear over an F32 matrix runs as
 * tsm_matmul_f32, and token tables may stay F32 beside quantised layers (Module#quantize without embeddings). */
int tsm_model_load_gguf(tsm_ctx* ctx, const char* path, tsm_model** out);
/* GGUF.open (gguf.cr:90-99, 297-325) alone: parses the header, the metadata and the tensor table and checks that every tensor
 * lies inside the file, without a device.  TSM_OK, or TSM_ERR_IO / TSM_ERR_UNSUPPORTED with the reason in `reason`
 * (a truncated file, an offset outside it, an empty axis, a token table that is not a matrix ...). */
int tsm_gguf_check(const char* path, char* reason, int capacity);
/* GPT2.load / Llama.load of Hugging Face safetensors weights (gpt2.cr:69-101, llama.cr:163-175, safetensors.cr), followed by
 * Module#quantize(kind, embeddings: true) (module.cr:262-274) on the device: F32 / F16 / BF16 matrices, GPT-2's Conv1D
 * weights transposed, every Linear and both embedding tables quantised to `kind`; with kind TSM_F32 nothing is quantised
 * and the model runs in F32 as loaded.  config->arch picks the family.  GPT-2
 * takes config->heads only; Llama takes heads, kv_heads, head_width (0: width / heads), eps, rope_theta and context
 * (what the model directory's config.json holds); all other sizes come from the tensor shapes. */
int tsm_model_load_safetensors(tsm_ctx* ctx, const char* path, const tsm_model_config* config, int kind, tsm_model** out);
/* Llama.new(config) / GPT2.new(config) with Init.normal(0.02) then Module#quantize(kind, embeddings: true)
 * (module.cr, builder.cr): weights drawn on the device from `seed`, quantised on the device. */
int tsm_model_random(tsm_ctx* ctx, const tsm_model_config* config, int kind, uint64_t seed, tsm_model** out);
/* Module#save("model.gguf") (module.cr:148-164; GGUF.write, gguf.cr:156-191): the model as the device holds it, block
 * formats byte for byte, written to a temporary beside `path` and renamed.  A Llama is written under llama.cpp's names with
 * llama.* metadata and q/k rows in llama.cpp's rotary order, a GPT-2 under tensomite's names with gpt2.heads, so the file
 * loads again through tsm_model_load_gguf and through the reference's Llama.load / GPT2.load.  One GPU only. */
int tsm_model_save_gguf(tsm_model* model, const char* path);
int tsm_model_config_get(tsm_model* model, tsm_model_config* out);
int tsm_model_free(tsm_model* model);
/* The weight behind a parameter ("embed", "head", "final_w", "final_b", "wpe", "<layer>.qkv", ".o", ".up",
 * ".down", ".norm1_w", ... and their "_b" biases): device address, kind, rows and columns. */
int tsm_model_tensor(tsm_model* model, const char* name, tsm_dptr* ptr, int* kind, int* n, int* k);

/* Generative#new_batch_cache (generative.cr:89-91): rows x capacity positions per layer, in place. */
int tsm_cache_create(tsm_model* model, int rows, int capacity, tsm_cache** out);
int tsm_cache_free(tsm_cache* cache);
int tsm_cache_length(tsm_cache* cache, int row, int* length);
int tsm_cache_reset(tsm_cache* cache, int row);                       /* BatchCache#reset */
/* Fills row `row` with `length` positions of seeded N(0,1) keys and values (a stand-in for a prefill
 * whose cost is out of reach; the bytes can be read back with tsm_cache_layer). */
int tsm_cache_fill(tsm_cache* cache, int row, int length, uint64_t seed);
int tsm_cache_layer(tsm_cache* cache, int layer, tsm_dptr* keys, tsm_dptr* values);

/* Generative#forward / #forward_last over a BatchCache (generative.cr:101-125): counts[row] new tokens
 * per row (0 = idle), ids packed row after row.  Writes logits of each row's last new token (last = 1)
 * or of every new token to the host array `logits` [outputs, vocab], and advances the cache. */
int tsm_forward(tsm_model* model, tsm_cache* cache, const int32_t* counts, const int32_t* ids, int last,
                float* logits);
/* One decode step for every row: ids[row] is the row's next token; picks each row's next token greedily
 * on the device (Sampler.greedy) and writes it to tokens[row].  The step is captured once as a CUDA
 * graph and replayed.  logits (may be NULL) receives [rows, vocab] on the host. */
int tsm_decode(tsm_model* model, tsm_cache* cache, const int32_t* ids, int32_t* tokens, float* logits);
/* `steps` greedy decode steps for every row without returning to the host in between: each row's pick
 * feeds its next step on the device (the loop of Generative#generate, generative.cr:181-188, for all rows
 * at once).  ids[row] is each row's first token; tokens receives [steps, rows] on the host. */
int tsm_decode_run(tsm_model* model, tsm_cache* cache, const int32_t* ids, int steps, int32_t* tokens);
/* ---- several GPUs -----------------------------------------------------------------------------------------
 * The reference runs a model on one device (src/tensomite/device.cr); these entry points have no counterpart there.
 * One process per GPU.  Independent streams need nothing here: every process loads the whole model and decodes its own
 * rows.  A model too large or too slow for one GPU is split by tensor parallelism: tsm_tp_init joins the context to a
 * group of `world` ranks (NCCL over NVLink; the 128-byte id comes from tsm_tp_unique_id on one rank and is carried
 * to the others by the host), and a model then loaded or drawn on that context holds only its rank's rows of every
 * projection (its heads of q, k and v, its slice of gate/up, o, down and the vocabulary head) and its own kv heads of
 * the cache.  Every rank calls tsm_forward / tsm_decode / tsm_decode_run / tsm_generate with the same arguments and
 * receives the same tokens and logits, bit for bit those of one GPU: projections are split by output rows only, so
 * no sum is reordered.  Heads, kv heads, width, hidden width and vocabulary must divide by `world`. */
int tsm_tp_unique_id(uint8_t* out /* [128] */);
int tsm_tp_init(tsm_ctx* ctx, int rank, int world, const uint8_t* id /* [128] */);
int tsm_tp_info(tsm_ctx* ctx, int* rank, int* world);
/* How models built on this context AFTER the call are split (set it between tsm_tp_init and the load):
 *   TSM_TP_GATHER (default) every projection by output rows, all-gathers between them: the bits of one GPU;
 *   TSM_TP_REDUCE           q/k/v, gate/up and the head by output rows, o and down by INPUT columns (each rank multiplies its
 *                           own heads' / hidden slice's columns) with an NCCL all-reduce of the partial sums after each: two
 *                           exchanges per layer instead of four and a shorter K loop per rank, but an output's blocks are then
 *                           summed in another order, so results agree with one GPU within the fast mode's budget (0.001 nats
 *                           KL per token), not bit for bit. */
typedef enum { TSM_TP_GATHER = 0, TSM_TP_REDUCE = 1 } tsm_tp_split;
int tsm_tp_variant(tsm_ctx* ctx, int variant);

/* Leaves the group without waiting for the other ranks (ncclCommAbort): what a rank does once the host has learnt that a
 * peer is gone.  Every later exchange on this context returns TSM_ERR_COMM.  An exchange that fails, and a wait during which
 * the communicator reports a failure of its own (ncclCommGetAsyncError is polled while the host waits for a step), return
 * TSM_ERR_COMM too; a step that makes no progress for TSM_TP_TIMEOUT_MS (default 60000) returns TSM_ERR_TIMEOUT. */
int tsm_tp_abort(tsm_ctx* ctx);

/* Generative#generate with Sampler.greedy (generative.cr:177-190): `count` tokens after `prompt`. */
int tsm_generate(tsm_model* model, const int32_t* prompt, int prompt_size, int count, int32_t* tokens);

/* Generative#generate(prompt, count, sampler, stop) (generative.cr:177-190) with the sampler's draw left to the host:
 * after each step the device keeps the `top_k` highest logits of the last position, highest first and equal logits by lower
 * index, as Sampler#top orders its candidates (sampler.cr:77-96), and hands their ids and values to `pick`, which returns the
 * chosen token (Sampler#pick_among, sampler.cr:57-72: the caller applies its temperature and makes its seeded draw).
 * top_k = 0 hands over the whole row of logits in index order (ids is then NULL and count the vocabulary).  pick = NULL is
 * Sampler.greedy on the device.  Generation ends after `count` tokens or after a token found in `stop` (which is the last
 * one returned); *produced receives how many tokens were written. */
typedef int32_t (*tsm_pick_fn)(void* user, int step, const int32_t* ids, const float* logits, int count);
int tsm_generate_sampled(tsm_model* model, const int32_t* prompt, int prompt_size, int count, const int32_t* stop, int stop_size,
                         int top_k, tsm_pick_fn pick, void* user, int32_t* tokens, int* produced);

#ifdef __cplusplus
}
#endif
#endif /* TSM_B200_H */
