// What the engine's files share: a model's resident weights, the buffers of one packed step, the batch cache, and the
// helpers that build a model whichever way its weights arrive (GGUF, safetensors, drawn on the device).
#pragma once
#include "common.cuh"

namespace tsm {

struct Linear {
    int kind = TSM_F32;
    int n = 0, k = 0;
    uint8_t* w = nullptr;
    float* bias = nullptr;
};

struct Layer {
    float *norm1_w = nullptr, *norm1_b = nullptr, *norm2_w = nullptr, *norm2_b = nullptr;
    Linear qkv, o, up, down;
};

struct Named {
    void* ptr;
    int kind, n, k;
};

// Buffers of one packed step over up to `tokens` new tokens.
struct Workspace {
    int tokens = 0;
    int* ids = nullptr;      // [T]
    int* table = nullptr;    // [T,3] row, position, positions held
    int* last = nullptr;     // [T] indices of the rows whose logits are wanted
    int* order = nullptr;    // [T] tokens by visible positions, most first (attention's launch order)
    int* qtiles = nullptr;   // [T, 2] query tiles of a step that holds prompts: first token, tokens (attention's prefill kernel)
    float* x = nullptr;      // [T, width]
    float* xl = nullptr;     // [T, width] gathered last rows
    float* qkv = nullptr;    // [T, (heads + 2 kv) * hw]
    float* att = nullptr;    // [T, heads * hw] (ordered attention writes F32 first)
    float* up = nullptr;     // [T, 2*hidden | hidden]
    float* h = nullptr;      // [T, max(width, hidden)] normed rows / activation output, when the next weight is F32
    float* logits = nullptr; // [T, vocab]
    int* picks = nullptr;    // [T]
    float* tp_parts = nullptr;   // tensor-parallel: [ranks][T, widest / ranks], the ranks' column slices as gathered
    float* tp_rows = nullptr;    //                  [T, widest], the same back in row order
    float* tp_best = nullptr;    //                  [ranks][T] best logit of each rank's vocabulary slice, then [ranks][T] its index
    void* qa = nullptr;      // quantised activations, K = width
    void* qb = nullptr;      // K = heads * hw
    void* qc = nullptr;      // K = hidden
    int32_t* host = nullptr; // pinned: ids [T] + table [3T] + picks [T] + query tiles [2T]
};

// The regions of the fused tensor-parallel exchange (tp_exchange.cu): this rank's and, mapped through CUDA IPC, the peers'.
struct Exchange {
    bool ready = false;
    void* local = nullptr;
    unsigned char* regions[8] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    int64_t bytes = 0, partial_at = 0, quant_at = 0;
    int rows = 0, width = 0;
};

// Rows [start, start + count) of a matrix.
struct RowRange {
    int64_t start, count;
};

}  // namespace tsm

namespace tsm { struct Stager; }

struct tsm_model {
    tsm_ctx* ctx = nullptr;
    tsm::Stager* stager = nullptr;    // the pinned staging buffers of a load in progress (model_gguf.cu)
    tsm_model_config cfg{};
    tsm::Linear embed, wpe, head;
    float *final_w = nullptr, *final_b = nullptr;
    std::vector<tsm::Layer> layers;
    float *rope_cos = nullptr, *rope_sin = nullptr;
    std::vector<void*> owned;
    std::map<std::string, tsm::Named> named;
    tsm::Workspace ws;
    uint64_t ws_generation = 1;
    bool one_token_per_row = false;   // the step being queued gives every cache row at most one token (a decode step)
    int tp = 1, tp_rank = 0;     // tensor-parallel group of the context the model was built on
    bool tp_reduce = false;      // o and down split by input columns and all-reduced (TSM_TP_REDUCE), not by output rows
    tsm::Linear head_local;           // this rank's rows of the vocabulary head (a view when the head is the embedding table)
    tsm::Exchange xchg;               // peer memory of the fused exchange (TSM_TP_REDUCE on GPUs that can map each other)
};

struct tsm_cache {
    tsm_model* model = nullptr;
    int rows = 0, capacity = 0;
    std::vector<float*> keys, values;
    std::vector<int> lengths;
    cudaGraphExec_t graph = nullptr;  // one decode step over all rows
    uint64_t graph_stamp = 0;         // what the captured step depends on (buffers, mode)
    cudaGraphExec_t run_graph = nullptr;  // one step of a device-resident run (tsm_decode_run)
    uint64_t run_stamp = 0;
    int* run_state = nullptr;         // device: [0] steps done, then tokens [steps, rows]
    int64_t run_capacity = 0;         // ints in run_state
    int graph_kernels = 0, run_kernels = 0;  // kernel nodes per replay, for the launch counter
    int graph_collectives = 0, run_collectives = 0;  // exchanges per replay
};

namespace tsm {

// Which rows of a projection a rank of a tensor-parallel group holds (shard_ranges); an empty list means all rows.
enum { SHARD_QKV, SHARD_WIDTH, SHARD_UP, SHARD_VOCAB };
std::vector<RowRange> shard_ranges(const tsm_model* m, int what);
int check_sharding(tsm_model* m);
int shard_inputs(tsm_model* m, Layer& l);
int shard_bias(tsm_model* m, float** bias, const std::vector<RowRange>& ranges);
// Device memory owned by the model and freed with it.
int dev_alloc(tsm_model* m, int64_t bytes, void** out);
int64_t weight_bytes(int kind, int64_t n, int64_t k);
int make_rope_tables(tsm_model* m);
int check_config(tsm_ctx* ctx, const tsm_model_config& c);
void register_names(tsm_model* m);
void set_head_local(tsm_model* m);
// The three ways a model is filled (model_gguf.cu, model_safetensors.cu, model.cu) and the way it is written out.
int load_gguf_model(tsm_model* m, const char* path);
int check_gguf_file(const char* path, std::string* why);
int save_gguf_model(tsm_model* m, const char* path);
int load_safetensors_model(tsm_model* m, const char* path, const tsm_model_config& config, int kind);
int build_random(tsm_model* m, int kind, uint64_t seed);
// The fused exchange of a TSM_TP_REDUCE step (tp_exchange.cu).
int xchg_setup(tsm_model* m);
void xchg_release(tsm_model* m);
bool xchg_takes(const tsm_model* m, int total);
float* xchg_partial(tsm_model* m);
void* xchg_quantized(tsm_model* m);
int launch_xchg_reduce_norm(tsm_model* m, int total, float* x, const float* bias, bool layer, const float* w, const float* b, float eps);

}  // namespace tsm
