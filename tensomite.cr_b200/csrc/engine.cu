// The token loop: models with resident weights, the batch cache, one packed forward step, its CUDA-graph
// replay for decoding, and the GGUF loader.  Host-side counterpart of the reference's
// models/{generative,llama,gpt2}.cr and modules.cr; the op order of one step is theirs.
#include <fcntl.h>
#include <math.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <memory>

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
    int32_t* host = nullptr; // pinned: ids [T] + table [3T] + picks [T]
};

}  // namespace tsm

using namespace tsm;

struct tsm_model {
    tsm_ctx* ctx = nullptr;
    tsm_model_config cfg{};
    Linear embed, wpe, head;
    float *final_w = nullptr, *final_b = nullptr;
    std::vector<Layer> layers;
    float *rope_cos = nullptr, *rope_sin = nullptr;
    std::vector<void*> owned;
    std::map<std::string, Named> named;
    Workspace ws;
    uint64_t ws_generation = 1;
    int tp = 1, tp_rank = 0;     // tensor-parallel group of the context the model was built on
    bool tp_reduce = false;      // o and down split by input columns and all-reduced (TSM_TP_REDUCE), not by output rows
    Linear head_local;           // this rank's rows of the vocabulary head (a view when the head is the embedding table)
};

// Rows [start, start + count) of a matrix.
struct RowRange {
    int64_t start, count;
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
};

namespace tsm {

static int dev_alloc(tsm_model* m, int64_t bytes, void** out);

// Which rows of a projection a rank of a tensor-parallel group holds.  Every projection is split by OUTPUT rows, so
// each output's sum over blocks stays on one GPU, whole and in block order: the sharded model's bits are the single
// GPU's.  Joined projections keep their parts: a rank takes its heads' rows of q, of k and of v (its slice of gate
// and of up).  An empty list means all rows.
enum { SHARD_QKV, SHARD_WIDTH, SHARD_UP, SHARD_VOCAB };
static std::vector<RowRange> shard_ranges(const tsm_model* m, int what) {
    std::vector<RowRange> ranges;
    if (m->tp <= 1) return ranges;
    const tsm_model_config& c = m->cfg;
    int64_t G = m->tp, r = m->tp_rank;
    int64_t qn = (int64_t)c.heads * c.head_width, kvn = (int64_t)c.kv_heads * c.head_width;
    switch (what) {
        case SHARD_QKV:
            ranges = {{r * qn / G, qn / G}, {qn + r * kvn / G, kvn / G}, {qn + kvn + r * kvn / G, kvn / G}};
            break;
        case SHARD_WIDTH:  // o and down: by output rows, unless they are split by input columns (shard_inputs)
            if (!m->tp_reduce) ranges = {{r * c.width / G, c.width / G}};
            break;
        case SHARD_UP:
            ranges = {{r * c.hidden / G, c.hidden / G}};
            if (c.arch == 0) ranges.push_back({c.hidden + r * c.hidden / G, c.hidden / G});
            break;
        case SHARD_VOCAB: ranges = {{r * c.vocab / G, c.vocab / G}}; break;
    }
    return ranges;
}

static int check_sharding(tsm_model* m) {
    if (m->tp <= 1) return TSM_OK;
    const tsm_model_config& c = m->cfg;
    int G = m->tp;
    if (c.heads % G || c.kv_heads % G || c.width % G || c.hidden % G || c.vocab % G)
        return fail(m->ctx, TSM_ERR_ARG, "heads, key/value heads, width, hidden width and vocabulary must all divide by the " + std::to_string(G) + " ranks");
    if (m->tp_reduce && ((c.heads / G * c.head_width) % 32 || (c.hidden / G) % 32))
        return fail(m->ctx, TSM_ERR_ARG, "a rank's share of the attention output and of the hidden width must be whole blocks of 32");
    return TSM_OK;
}

// Keeps block columns [first, first + blocks) of every row of a quantised matrix: a rank's share of the INPUT columns.
static int keep_block_columns(tsm_model* m, Linear* l, int64_t first, int64_t blocks) {
    int64_t B = block_bytes(l->kind), nb = l->k / 32;
    uint8_t* narrow = nullptr;
    TSM_TRY(dev_alloc(m, (int64_t)l->n * blocks * B, (void**)&narrow));
    TSM_CUDA(m->ctx, cudaMemcpy2DAsync(narrow, (size_t)(blocks * B), l->w + first * B, (size_t)(nb * B), (size_t)(blocks * B), (size_t)l->n,
                                       cudaMemcpyDeviceToDevice, m->ctx->stream));
    TSM_CUDA(m->ctx, cudaStreamSynchronize(m->ctx->stream));
    for (size_t i = 0; i < m->owned.size(); i++)
        if (m->owned[i] == (void*)l->w) {
            m->owned.erase(m->owned.begin() + (long)i);
            pool_release(m->ctx, l->w);
            break;
        }
    l->w = narrow, l->k = (int)(blocks * 32);
    return TSM_OK;
}

// TSM_TP_REDUCE: a layer's o and down keep all their rows but only this rank's input columns (its heads' attention
// outputs, its slice of the hidden width); their biases are added once, by rank 0.
static int shard_inputs(tsm_model* m, Layer& l) {
    if (!m->tp_reduce) return TSM_OK;
    const tsm_model_config& c = m->cfg;
    int64_t G = m->tp, r = m->tp_rank;
    int64_t o_blocks = (int64_t)c.heads * c.head_width / G / 32, down_blocks = (int64_t)c.hidden / G / 32;
    TSM_TRY(keep_block_columns(m, &l.o, r * o_blocks, o_blocks));
    TSM_TRY(keep_block_columns(m, &l.down, r * down_blocks, down_blocks));
    if (r != 0) l.o.bias = nullptr, l.down.bias = nullptr;
    return TSM_OK;
}

static int dev_alloc(tsm_model* m, int64_t bytes, void** out) {
    TSM_TRY(pool_alloc(m->ctx, bytes, out));
    m->owned.push_back(*out);
    return TSM_OK;
}

static void name_tensor(tsm_model* m, const std::string& name, void* ptr, int kind, int n, int k) {
    m->named[name] = Named{ptr, kind, n, k};
}

static void name_linear(tsm_model* m, const std::string& name, const Linear& l) {
    name_tensor(m, name, l.w, l.kind, l.n, l.k);
    if (l.bias) name_tensor(m, name + "_b", l.bias, TSM_F32, 1, l.n);
}

static int64_t weight_bytes(int kind, int64_t n, int64_t k) { return kind == TSM_F32 ? n * k * 4 : n * (k / 32) * block_bytes(kind); }

// cos/sin of every position, in F32 through the host's libm, as RotaryEmbedding computes them
// (modules.cr:343-351): freq_i = 1f / powf(theta_f32, f32(2i) / width).
static int make_rope_tables(tsm_model* m) {
    const tsm_model_config& c = m->cfg;
    int hw = c.head_width, half = hw / 2;
    std::vector<float> freq(half), cosv((size_t)c.context * hw), sinv((size_t)c.context * hw);
    for (int i = 0; i < half; i++) freq[i] = 1.0f / powf((float)c.rope_theta, (float)(2 * i) / (float)hw);
    for (int p = 0; p < c.context; p++)
        for (int i = 0; i < hw; i++) {
            float angle = (float)p * freq[i % half];
            cosv[(size_t)p * hw + i] = cosf(angle);
            sinv[(size_t)p * hw + i] = sinf(angle);
        }
    int64_t bytes = (int64_t)c.context * hw * 4;
    TSM_TRY(dev_alloc(m, bytes, (void**)&m->rope_cos));
    TSM_TRY(dev_alloc(m, bytes, (void**)&m->rope_sin));
    TSM_TRY(tsm_upload(m->ctx, (tsm_dptr)(uintptr_t)m->rope_cos, cosv.data(), bytes));
    TSM_TRY(tsm_upload(m->ctx, (tsm_dptr)(uintptr_t)m->rope_sin, sinv.data(), bytes));
    return TSM_OK;
}

static int check_config(tsm_ctx* ctx, const tsm_model_config& c) {
    if (c.arch != 0 && c.arch != 1) return fail(ctx, TSM_ERR_ARG, "unknown architecture");
    if (c.layers < 1 || c.width < 32 || c.heads < 1 || c.kv_heads < 1 || c.head_width < 2 || c.hidden < 32 || c.vocab < 1 || c.context < 1)
        return fail(ctx, TSM_ERR_ARG, "a model size is not positive");
    if (c.heads % c.kv_heads != 0)
        return fail(ctx, TSM_ERR_ARG, std::to_string(c.heads) + " query heads do not group into " + std::to_string(c.kv_heads) + " key and value heads");
    if (c.width % 32 != 0 || c.hidden % 32 != 0 || (c.heads * c.head_width) % 32 != 0)
        return fail(ctx, TSM_ERR_ARG, "quantised products need widths that split into blocks of 32");
    if (c.arch == 1 && (c.kv_heads != c.heads || c.heads * c.head_width != c.width))
        return fail(ctx, TSM_ERR_ARG, "width " + std::to_string(c.width) + " does not divide into " + std::to_string(c.heads) + " heads");
    return TSM_OK;
}

static void register_names(tsm_model* m) {
    name_linear(m, "embed", m->embed);
    if (m->wpe.w) name_linear(m, "wpe", m->wpe);
    name_linear(m, "head", m->head);
    name_tensor(m, "final_w", m->final_w, TSM_F32, 1, m->cfg.width);
    if (m->final_b) name_tensor(m, "final_b", m->final_b, TSM_F32, 1, m->cfg.width);
    for (size_t i = 0; i < m->layers.size(); i++) {
        std::string p = std::to_string(i) + ".";
        Layer& l = m->layers[i];
        name_tensor(m, p + "norm1_w", l.norm1_w, TSM_F32, 1, m->cfg.width);
        name_tensor(m, p + "norm2_w", l.norm2_w, TSM_F32, 1, m->cfg.width);
        if (l.norm1_b) name_tensor(m, p + "norm1_b", l.norm1_b, TSM_F32, 1, m->cfg.width);
        if (l.norm2_b) name_tensor(m, p + "norm2_b", l.norm2_b, TSM_F32, 1, m->cfg.width);
        name_linear(m, p + "qkv", l.qkv);
        name_linear(m, p + "o", l.o);
        name_linear(m, p + "up", l.up);
        name_linear(m, p + "down", l.down);
    }
}

// ---- GGUF (gguf.cr:297-381) ------------------------------------------------------------------------

struct GgufEntry {
    uint32_t kind;
    std::vector<int64_t> shape;  // outermost first
    int64_t offset;              // absolute
    int64_t bytes;
};

struct GgufFile {
    const uint8_t* data = nullptr;
    int64_t size = 0, pos = 0;
    bool bad = false;
    std::map<std::string, double> numbers;
    std::map<std::string, std::string> strings;
    std::map<std::string, GgufEntry> entries;
    std::vector<std::string> order;
    ~GgufFile() {
        if (data) munmap((void*)data, (size_t)size);
    }
    const uint8_t* take(int64_t n) {
        if (n < 0 || pos + n > size) {
            bad = true;
            static uint8_t zeros[16] = {0};
            return zeros;
        }
        const uint8_t* p = data + pos;
        pos += n;
        return p;
    }
    template <class T> T read() {
        T v;
        memcpy(&v, take(sizeof(T)), sizeof(T));
        return v;
    }
    std::string str() {
        uint64_t n = read<uint64_t>();
        if (n > (uint64_t)(size - pos)) {
            bad = true;
            return "";
        }
        return std::string((const char*)take((int64_t)n), (size_t)n);
    }
    // reads a value of GGUF type t; numbers and strings are kept under `key`, arrays skipped
    void value(uint32_t t, const std::string& key, int depth = 0) {
        switch (t) {
            case 0: numbers[key] = read<uint8_t>(); break;
            case 1: numbers[key] = read<int8_t>(); break;
            case 2: numbers[key] = read<uint16_t>(); break;
            case 3: numbers[key] = read<int16_t>(); break;
            case 4: numbers[key] = read<uint32_t>(); break;
            case 5: numbers[key] = read<int32_t>(); break;
            case 6: numbers[key] = read<float>(); break;
            case 7: numbers[key] = read<uint8_t>() != 0; break;
            case 8: strings[key] = str(); break;
            case 9: {
                uint32_t element = read<uint32_t>();
                uint64_t count = read<uint64_t>();
                for (uint64_t i = 0; i < count && !bad; i++) value(element, "", depth + 1);
                break;
            }
            case 10: numbers[key] = (double)read<uint64_t>(); break;
            case 11: numbers[key] = (double)read<int64_t>(); break;
            case 12: numbers[key] = read<double>(); break;
            default: bad = true;
        }
    }
};

static int64_t gguf_bytes(uint32_t kind, int64_t count) {
    switch (kind) {
        case 0: return count * 4;
        case 1: case 30: return count * 2;
        case 2: return count / 32 * 18;
        case 3: return count / 32 * 20;
        case 8: return count / 32 * 34;
    }
    return -1;
}

static int gguf_kind_to_tsm(uint32_t kind) { return kind == 8 ? TSM_Q8_0 : kind == 2 ? TSM_Q4_0 : kind == 3 ? TSM_Q4_1 : TSM_F32; }

static int gguf_open(tsm_ctx* ctx, const char* path, GgufFile& f) {
    int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(ctx, TSM_ERR_IO, std::string(path) + " cannot be opened");
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 24) {
        close(fd);
        return fail(ctx, TSM_ERR_IO, std::string(path) + " is not a GGUF file");
    }
    f.size = st.st_size;
    void* map = mmap(nullptr, (size_t)f.size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map == MAP_FAILED) return fail(ctx, TSM_ERR_IO, std::string(path) + " cannot be mapped");
    f.data = (const uint8_t*)map;
    if (f.read<uint32_t>() != 0x46554747u) return fail(ctx, TSM_ERR_IO, std::string(path) + " is not a GGUF file");
    uint32_t version = f.read<uint32_t>();
    if (version != 2 && version != 3) return fail(ctx, TSM_ERR_IO, std::string(path) + ": GGUF version " + std::to_string(version) + " is not supported");
    uint64_t tensors = f.read<uint64_t>(), keys = f.read<uint64_t>();
    for (uint64_t i = 0; i < keys && !f.bad; i++) {
        std::string key = f.str();
        f.value(f.read<uint32_t>(), key);
    }
    struct Info { std::string name; std::vector<int64_t> shape; uint32_t kind; int64_t offset; };
    std::vector<Info> infos;
    for (uint64_t i = 0; i < tensors && !f.bad; i++) {
        Info info;
        info.name = f.str();
        uint32_t nd = f.read<uint32_t>();
        if (nd > 8) { f.bad = true; break; }
        std::vector<int64_t> dims(nd);
        for (uint32_t d = 0; d < nd; d++) dims[d] = (int64_t)f.read<uint64_t>();
        info.shape.assign(dims.rbegin(), dims.rend());
        info.kind = f.read<uint32_t>();
        info.offset = (int64_t)f.read<uint64_t>();
        infos.push_back(info);
    }
    if (f.bad) return fail(ctx, TSM_ERR_IO, std::string(path) + " is malformed");
    int64_t alignment = f.numbers.count("general.alignment") ? (int64_t)f.numbers["general.alignment"] : 32;
    if (alignment < 1) alignment = 32;
    int64_t start = (f.pos + alignment - 1) / alignment * alignment;
    for (auto& info : infos) {
        int64_t count = 1;
        for (int64_t d : info.shape) count *= d;
        int64_t bytes = gguf_bytes(info.kind, count);
        if (bytes < 0) return fail(ctx, TSM_ERR_UNSUPPORTED, info.name + ": GGUF tensor type " + std::to_string(info.kind) + " is not supported yet");
        if ((info.kind == 2 || info.kind == 3 || info.kind == 8) && (info.shape.empty() || info.shape.back() % 32 != 0))
            return fail(ctx, TSM_ERR_IO, info.name + ": rows of " + std::to_string(info.shape.empty() ? 0 : info.shape.back()) + " do not split into blocks of 32");
        if (info.offset % alignment != 0 || start + info.offset + bytes > f.size)
            return fail(ctx, TSM_ERR_IO, info.name + ": " + std::to_string(bytes) + " bytes at " + std::to_string(info.offset) + " do not fit " + path);
        f.entries[info.name] = GgufEntry{info.kind, info.shape, start + info.offset, bytes};
        f.order.push_back(info.name);
    }
    return TSM_OK;
}

// F16 (GGUF type 1) or BF16 (type 30) values widened to F32, exactly (gguf.cr:112-136 widens them the same way).
static void widen_halves(const uint16_t* h, int64_t count, bool bf16, float* out) {
    for (int64_t i = 0; i < count; i++) {
        if (bf16) {
            uint32_t u = (uint32_t)h[i] << 16;
            memcpy(&out[i], &u, 4);
        } else {
            out[i] = __half2float(__ushort_as_half(h[i]));
        }
    }
}

// Uploads an F32 / F16 / BF16 vector or matrix as F32.
static int upload_f32(tsm_model* m, GgufFile& f, const std::string& name, int64_t expect, float** out) {
    auto found = f.entries.find(name);
    if (found == f.entries.end()) return fail(m->ctx, TSM_ERR_IO, "the file lacks " + name);
    const GgufEntry& e = found->second;
    int64_t count = 1;
    for (int64_t d : e.shape) count *= d;
    if (count != expect) return fail(m->ctx, TSM_ERR_ARG, name + ": the file holds " + std::to_string(count) + " values, the model " + std::to_string(expect));
    std::vector<float> wide;
    const void* src = f.data + e.offset;
    if (e.kind == 1 || e.kind == 30) {
        wide.resize((size_t)count);
        widen_halves((const uint16_t*)src, count, e.kind == 30, wide.data());
        src = wide.data();
    } else if (e.kind != 0) {
        return fail(m->ctx, TSM_ERR_UNSUPPORTED, name + " is a block format where F32 is expected");
    }
    TSM_TRY(dev_alloc(m, count * 4, (void**)out));
    return tsm_upload(m->ctx, (tsm_dptr)(uintptr_t)*out, src, count * 4);
}

struct RowSource {
    std::string name;
    int heads;  // > 0: undo llama.cpp's rotary row order for this many heads (llama.cr:226-235)
};

// Uploads one or several [n_i, k] block tensors as one row-joined weight (Linear.merge, modules.cr:36-54).
static int upload_rows(tsm_model* m, GgufFile& f, const std::vector<RowSource>& parts, int k, int expect_n, Linear* out,
                       const std::vector<RowRange>& ranges = {}) {
    int kind = -2;
    int64_t total_rows = 0;
    for (auto& part : parts) {
        auto found = f.entries.find(part.name);
        if (found == f.entries.end()) return fail(m->ctx, TSM_ERR_IO, "the file lacks " + part.name);
        const GgufEntry& e = found->second;
        if (e.shape.size() != 2 || e.shape[1] != k)
            return fail(m->ctx, TSM_ERR_ARG, part.name + ": the file's shape does not match the model's [" + std::to_string(expect_n) + ", " + std::to_string(k) + "]");
        int this_kind = gguf_kind_to_tsm(e.kind);
        if (kind != -2 && kind != this_kind) return fail(m->ctx, TSM_ERR_UNSUPPORTED, "joined projections must share a format");
        kind = this_kind;
        total_rows += e.shape[0];
    }
    if (total_rows != expect_n) return fail(m->ctx, TSM_ERR_ARG, parts[0].name + ": the file holds " + std::to_string(total_rows) + " rows, the model " + std::to_string(expect_n));
    int64_t row_bytes = weight_bytes(kind, 1, k);
    std::vector<uint8_t> staging((size_t)(total_rows * row_bytes));
    int64_t at = 0;
    for (auto& part : parts) {
        const GgufEntry& e = f.entries[part.name];
        const uint8_t* src = f.data + e.offset;
        int64_t rows = e.shape[0];
        std::vector<float> wide;
        if (e.kind == 1 || e.kind == 30) {  // F16 / BF16 matrices become F32 weights
            wide.resize((size_t)(rows * k));
            widen_halves((const uint16_t*)src, rows * k, e.kind == 30, wide.data());
            src = (const uint8_t*)wide.data();
        }
        if (part.heads > 0) {
            int64_t half = rows / part.heads / 2;
            int64_t dst_row = 0;
            for (int head = 0; head < part.heads; head++)
                for (int pair = 0; pair < 2; pair++)
                    for (int64_t i = 0; i < half; i++, dst_row++)
                        memcpy(&staging[(size_t)((at + dst_row) * row_bytes)], src + (head * 2 * half + 2 * i + pair) * row_bytes, (size_t)row_bytes);
        } else {
            memcpy(&staging[(size_t)(at * row_bytes)], src, (size_t)(rows * row_bytes));
        }
        at += rows;
    }
    if (!ranges.empty()) {  // a tensor-parallel rank keeps its rows only
        std::vector<uint8_t> kept;
        int64_t rows = 0;
        for (auto& range : ranges) {
            kept.insert(kept.end(), staging.begin() + (size_t)(range.start * row_bytes), staging.begin() + (size_t)((range.start + range.count) * row_bytes));
            rows += range.count;
        }
        staging.swap(kept);
        expect_n = (int)rows;
    }
    out->kind = kind, out->n = expect_n, out->k = k;
    TSM_TRY(dev_alloc(m, (int64_t)staging.size(), (void**)&out->w));
    return tsm_upload(m->ctx, (tsm_dptr)(uintptr_t)out->w, staging.data(), (int64_t)staging.size());
}

// Replaces a full bias vector by the entries of a rank's rows.
static int shard_bias(tsm_model* m, float** bias, const std::vector<RowRange>& ranges) {
    if (!*bias || ranges.empty()) return TSM_OK;
    int64_t rows = 0;
    for (auto& range : ranges) rows += range.count;
    float* local = nullptr;
    TSM_TRY(dev_alloc(m, rows * 4, (void**)&local));
    int64_t at = 0;
    for (auto& range : ranges) {
        TSM_CUDA(m->ctx, cudaMemcpyAsync(local + at, *bias + range.start, (size_t)range.count * 4, cudaMemcpyDeviceToDevice, m->ctx->stream));
        at += range.count;
    }
    *bias = local;  // the full vector stays owned by the model and is freed with it
    return TSM_OK;
}

static int load_llama(tsm_model* m, GgufFile& f) {
    auto num = [&](const std::string& key, double fallback, bool required, bool* missing) {
        auto found = f.numbers.find("llama." + key);
        if (found != f.numbers.end()) return found->second;
        if (required) *missing = true;
        return fallback;
    };
    bool missing = false;
    tsm_model_config& c = m->cfg;
    c.arch = 0;
    c.width = (int)num("embedding_length", 0, true, &missing);
    c.heads = (int)num("attention.head_count", 0, true, &missing);
    c.layers = (int)num("block_count", 0, true, &missing);
    c.hidden = (int)num("feed_forward_length", 0, true, &missing);
    c.context = (int)num("context_length", 0, true, &missing);
    c.eps = (float)num("attention.layer_norm_rms_epsilon", 0, true, &missing);
    if (missing) return fail(m->ctx, TSM_ERR_IO, "the file lacks a llama.* key the model needs");
    c.kv_heads = (int)num("attention.head_count_kv", c.heads, false, &missing);
    c.head_width = (int)num("rope.dimension_count", c.heads ? c.width / c.heads : 0, false, &missing);
    c.rope_theta = num("rope.freq_base", 10000.0, false, &missing);
    if (f.strings.count("llama.rope.scaling.type") && f.strings["llama.rope.scaling.type"] != "none")
        return fail(m->ctx, TSM_ERR_UNSUPPORTED, "rope scaling " + f.strings["llama.rope.scaling.type"] + " is not supported");
    if (!f.entries.count("token_embd.weight")) return fail(m->ctx, TSM_ERR_IO, "the file lacks token_embd.weight");
    c.vocab = (int)num("vocab_size", (double)f.entries["token_embd.weight"].shape[0], false, &missing);
    c.tied = f.entries.count("output.weight") ? 0 : 1;
    TSM_TRY(check_config(m->ctx, c));
    std::vector<std::string> used;
    auto use = [&](const std::string& name) { used.push_back(name); return name; };
    TSM_TRY(upload_rows(m, f, {{use("token_embd.weight"), 0}}, c.width, c.vocab, &m->embed));
    TSM_TRY(check_sharding(m));
    if (!c.tied) TSM_TRY(upload_rows(m, f, {{use("output.weight"), 0}}, c.width, c.vocab, &m->head, shard_ranges(m, SHARD_VOCAB)));
    else m->head = m->embed;
    TSM_TRY(upload_f32(m, f, use("output_norm.weight"), c.width, &m->final_w));
    int qn = c.heads * c.head_width, kvn = c.kv_heads * c.head_width;
    m->layers.resize(c.layers);
    for (int i = 0; i < c.layers; i++) {
        std::string p = "blk." + std::to_string(i) + ".";
        Layer& l = m->layers[i];
        TSM_TRY(upload_f32(m, f, use(p + "attn_norm.weight"), c.width, &l.norm1_w));
        TSM_TRY(upload_f32(m, f, use(p + "ffn_norm.weight"), c.width, &l.norm2_w));
        TSM_TRY(upload_rows(m, f, {{use(p + "attn_q.weight"), c.heads}, {use(p + "attn_k.weight"), c.kv_heads}, {use(p + "attn_v.weight"), 0}},
                            c.width, qn + 2 * kvn, &l.qkv, shard_ranges(m, SHARD_QKV)));
        TSM_TRY(upload_rows(m, f, {{use(p + "attn_output.weight"), 0}}, qn, c.width, &l.o, shard_ranges(m, SHARD_WIDTH)));
        TSM_TRY(upload_rows(m, f, {{use(p + "ffn_gate.weight"), 0}, {use(p + "ffn_up.weight"), 0}}, c.width, 2 * c.hidden, &l.up,
                            shard_ranges(m, SHARD_UP)));
        TSM_TRY(upload_rows(m, f, {{use(p + "ffn_down.weight"), 0}}, c.hidden, c.width, &l.down, shard_ranges(m, SHARD_WIDTH)));
        TSM_TRY(shard_inputs(m, l));
    }
    // any tensor left over is an error, as the reference's loader raises (llama.cr:202-203)
    for (auto& name : f.order) {
        bool seen = false;
        for (auto& u : used) seen = seen || u == name;
        if (!seen) return fail(m->ctx, TSM_ERR_IO, "the file has " + name + ", which the model lacks");
    }
    return make_rope_tables(m);
}

static int upload_bias(tsm_model* m, GgufFile& f, const std::string& name, int n, float** out) {
    if (!f.entries.count(name)) {
        *out = nullptr;
        return TSM_OK;
    }
    return upload_f32(m, f, name, n, out);
}

// GPT-2 in tensomite's own names (gpt2.cr:75-89; module.cr:200-213): wte, wpe, h.N.*, ln_f.
static int load_gpt2(tsm_model* m, GgufFile& f) {
    tsm_model_config& c = m->cfg;
    c.arch = 1;
    if (!f.strings.count("gpt2.heads")) return fail(m->ctx, TSM_ERR_IO, "the file lacks gpt2.heads");
    c.heads = atoi(f.strings["gpt2.heads"].c_str());
    if (!f.entries.count("wte.weight") || !f.entries.count("wpe.weight")) return fail(m->ctx, TSM_ERR_IO, "the file lacks wte.weight or wpe.weight");
    c.vocab = (int)f.entries["wte.weight"].shape[0];
    c.width = (int)f.entries["wte.weight"].shape[1];
    c.context = (int)f.entries["wpe.weight"].shape[0];
    c.layers = 0;
    while (f.entries.count("h." + std::to_string(c.layers) + ".ln_1.weight")) c.layers++;
    c.kv_heads = c.heads;
    c.head_width = c.heads > 0 ? c.width / c.heads : 0;
    c.hidden = 4 * c.width;
    c.eps = 1e-5f;
    c.rope_theta = 0;
    c.tied = 1;
    TSM_TRY(check_config(m->ctx, c));
    TSM_TRY(check_sharding(m));
    TSM_TRY(upload_rows(m, f, {{"wte.weight", 0}}, c.width, c.vocab, &m->embed));
    TSM_TRY(upload_rows(m, f, {{"wpe.weight", 0}}, c.width, c.context, &m->wpe));
    m->head = m->embed;
    TSM_TRY(upload_f32(m, f, "ln_f.weight", c.width, &m->final_w));
    TSM_TRY(upload_f32(m, f, "ln_f.bias", c.width, &m->final_b));
    m->layers.resize(c.layers);
    for (int i = 0; i < c.layers; i++) {
        std::string p = "h." + std::to_string(i) + ".";
        Layer& l = m->layers[i];
        TSM_TRY(upload_f32(m, f, p + "ln_1.weight", c.width, &l.norm1_w));
        TSM_TRY(upload_f32(m, f, p + "ln_1.bias", c.width, &l.norm1_b));
        TSM_TRY(upload_f32(m, f, p + "ln_2.weight", c.width, &l.norm2_w));
        TSM_TRY(upload_f32(m, f, p + "ln_2.bias", c.width, &l.norm2_b));
        TSM_TRY(upload_rows(m, f, {{p + "attn.c_attn.weight", 0}}, c.width, 3 * c.width, &l.qkv, shard_ranges(m, SHARD_QKV)));
        TSM_TRY(upload_bias(m, f, p + "attn.c_attn.bias", 3 * c.width, &l.qkv.bias));
        TSM_TRY(shard_bias(m, &l.qkv.bias, shard_ranges(m, SHARD_QKV)));
        TSM_TRY(upload_rows(m, f, {{p + "attn.c_proj.weight", 0}}, c.width, c.width, &l.o, shard_ranges(m, SHARD_WIDTH)));
        TSM_TRY(upload_bias(m, f, p + "attn.c_proj.bias", c.width, &l.o.bias));
        TSM_TRY(shard_bias(m, &l.o.bias, shard_ranges(m, SHARD_WIDTH)));
        TSM_TRY(upload_rows(m, f, {{p + "mlp.c_fc.weight", 0}}, c.width, c.hidden, &l.up, shard_ranges(m, SHARD_UP)));
        TSM_TRY(upload_bias(m, f, p + "mlp.c_fc.bias", c.hidden, &l.up.bias));
        TSM_TRY(shard_bias(m, &l.up.bias, shard_ranges(m, SHARD_UP)));
        TSM_TRY(upload_rows(m, f, {{p + "mlp.c_proj.weight", 0}}, c.hidden, c.width, &l.down, shard_ranges(m, SHARD_WIDTH)));
        TSM_TRY(upload_bias(m, f, p + "mlp.c_proj.bias", c.width, &l.down.bias));
        TSM_TRY(shard_bias(m, &l.down.bias, shard_ranges(m, SHARD_WIDTH)));
        TSM_TRY(shard_inputs(m, l));
    }
    return TSM_OK;
}

// ---- random models (Llama.new / GPT2.new with Init.normal(0.02), then Module#quantize) ---------------

// The whole matrix is drawn (so that a rank's rows are the rows of the one-GPU model), the rank's rows are kept.
static int random_linear(tsm_model* m, int kind, int n, int k, uint64_t seed, bool with_bias, float* scratch, Linear* out,
                         const std::vector<RowRange>& ranges = {}) {
    int64_t count = (int64_t)n * k;
    TSM_TRY(launch_normal_fill(m->ctx, scratch, count, 0.0f, 0.02f, seed));
    int64_t local = n;
    if (!ranges.empty()) {
        local = 0;
        for (auto& range : ranges) local += range.count;
    }
    out->kind = kind, out->n = (int)local, out->k = k;
    TSM_TRY(dev_alloc(m, weight_bytes(kind, local, k), (void**)&out->w));
    if (ranges.empty()) {
        TSM_TRY(launch_quantize_blocks(m->ctx, scratch, count, kind, out->w));
    } else {
        int64_t at = 0;
        for (auto& range : ranges) {
            TSM_TRY(launch_quantize_blocks(m->ctx, scratch + range.start * k, range.count * k, kind, out->w + weight_bytes(kind, at, k)));
            at += range.count;
        }
    }
    if (with_bias) {
        TSM_TRY(dev_alloc(m, local * 4, (void**)&out->bias));
        TSM_TRY(launch_fill(m->ctx, out->bias, local, 0.0f));
    }
    return TSM_OK;
}

// This rank's rows of the vocabulary head: the head itself on one GPU or when it was built sharded, else a view of the
// (replicated) embedding table it is tied to.
static void set_head_local(tsm_model* m) {
    m->head_local = m->head;
    if (m->tp > 1 && m->head.n == m->cfg.vocab) {
        int64_t rows = m->cfg.vocab / m->tp;
        m->head_local.n = (int)rows;
        m->head_local.w = m->head.w + weight_bytes(m->head.kind, rows * m->tp_rank, m->head.k);
    }
}

static int constant_vector(tsm_model* m, int n, float value, float** out) {
    TSM_TRY(dev_alloc(m, (int64_t)n * 4, (void**)out));
    return launch_fill(m->ctx, *out, n, value);
}

static int build_random(tsm_model* m, int kind, uint64_t seed) {
    const tsm_model_config& c = m->cfg;
    TSM_TRY(check_sharding(m));
    int qn = c.heads * c.head_width, kvn = c.kv_heads * c.head_width;
    int upn = c.arch == 0 ? 2 * c.hidden : c.hidden;
    int64_t biggest = (int64_t)c.vocab * c.width;
    int64_t others[] = {(int64_t)(qn + 2 * kvn) * c.width, (int64_t)upn * c.width, (int64_t)c.context * c.width};
    for (int64_t o : others) biggest = o > biggest ? o : biggest;
    float* scratch = nullptr;
    TSM_TRY(pool_alloc(m->ctx, biggest * 4, (void**)&scratch));
    bool gpt = c.arch == 1;
    uint64_t t = seed * 1000003ull;
    int rc = TSM_OK;
    do {
        if ((rc = random_linear(m, kind, c.vocab, c.width, t++, false, scratch, &m->embed))) break;
        if (gpt && (rc = random_linear(m, kind, c.context, c.width, t++, false, scratch, &m->wpe))) break;
        if (!c.tied) {
            if ((rc = random_linear(m, kind, c.vocab, c.width, t++, false, scratch, &m->head, shard_ranges(m, SHARD_VOCAB)))) break;
        } else {
            m->head = m->embed;
        }
        set_head_local(m);
        if ((rc = constant_vector(m, c.width, 1.0f, &m->final_w))) break;
        if (gpt && (rc = constant_vector(m, c.width, 0.0f, &m->final_b))) break;
        m->layers.resize(c.layers);
        for (int i = 0; i < c.layers && rc == TSM_OK; i++) {
            Layer& l = m->layers[i];
            if ((rc = constant_vector(m, c.width, 1.0f, &l.norm1_w))) break;
            if ((rc = constant_vector(m, c.width, 1.0f, &l.norm2_w))) break;
            if (gpt && ((rc = constant_vector(m, c.width, 0.0f, &l.norm1_b)) || (rc = constant_vector(m, c.width, 0.0f, &l.norm2_b)))) break;
            if ((rc = random_linear(m, kind, qn + 2 * kvn, c.width, t++, gpt, scratch, &l.qkv, shard_ranges(m, SHARD_QKV)))) break;
            if ((rc = random_linear(m, kind, c.width, qn, t++, gpt, scratch, &l.o, shard_ranges(m, SHARD_WIDTH)))) break;
            if ((rc = random_linear(m, kind, upn, c.width, t++, gpt, scratch, &l.up, shard_ranges(m, SHARD_UP)))) break;
            if ((rc = random_linear(m, kind, c.width, c.hidden, t++, gpt, scratch, &l.down, shard_ranges(m, SHARD_WIDTH)))) break;
            if ((rc = shard_inputs(m, l))) break;
        }
    } while (0);
    cudaStreamSynchronize(m->ctx->stream);
    pool_release(m->ctx, scratch);
    if (rc != TSM_OK) return rc;
    if (!gpt) TSM_TRY(make_rope_tables(m));
    return TSM_OK;
}

// ---- safetensors (safetensors.cr; GPT2.new(SafeTensors), gpt2.cr:93-101; Llama.load of a model directory, llama.cr:163-175) ----
// Hugging Face files hold F32 (or F16 / BF16) matrices; the model is quantised as Module#quantize(dtype, embeddings: true) does
// (module.cr:262-274): every Linear weight and both embedding tables, with the device's quantiser, whose bytes are ggml's.

struct StEntry {
    std::string dtype;
    std::vector<int64_t> shape;
    int64_t begin = 0, end = 0;  // within the payload
};

struct StFile {
    const uint8_t* data = nullptr;
    int64_t size = 0, payload = 0;
    std::map<std::string, StEntry> entries;
    ~StFile() {
        if (data) munmap((void*)data, (size_t)size);
    }
};

// The header is one JSON object: name -> {"dtype": "...", "shape": [...], "data_offsets": [b, e]}, plus "__metadata__".
struct StParser {
    const char* p;
    const char* end;
    bool bad = false;
    void space() {
        while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++;
    }
    bool take(char c) {
        space();
        if (p < end && *p == c) {
            p++;
            return true;
        }
        return false;
    }
    std::string text() {
        std::string out;
        space();
        if (p >= end || *p != '"') {
            bad = true;
            return out;
        }
        for (p++; p < end && *p != '"'; p++) {
            if (*p == '\\' && p + 1 < end) p++;
            out.push_back(*p);
        }
        if (p < end) p++;
        else bad = true;
        return out;
    }
    int64_t integer() {
        space();
        int64_t v = 0;
        bool any = false;
        while (p < end && *p >= '0' && *p <= '9') v = v * 10 + (*p++ - '0'), any = true;
        if (!any) bad = true;
        return v;
    }
    void skip() {  // any value
        space();
        if (p >= end) {
            bad = true;
        } else if (*p == '"') {
            text();
        } else if (*p == '{' || *p == '[') {
            char open = *p, close = open == '{' ? '}' : ']';
            p++;
            if (take(close)) return;
            do {
                if (open == '{') {
                    text();
                    if (!take(':')) bad = true;
                }
                skip();
            } while (!bad && take(','));
            if (!take(close)) bad = true;
        } else {
            while (p < end && *p != ',' && *p != '}' && *p != ']') p++;
        }
    }
};

static int st_open(tsm_ctx* ctx, const char* path, StFile& f) {
    int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(ctx, TSM_ERR_IO, std::string(path) + " cannot be opened");
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 10) {
        close(fd);
        return fail(ctx, TSM_ERR_IO, std::string(path) + " is not a safetensors file");
    }
    f.size = st.st_size;
    void* map = mmap(nullptr, (size_t)f.size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (map == MAP_FAILED) return fail(ctx, TSM_ERR_IO, std::string(path) + " cannot be mapped");
    f.data = (const uint8_t*)map;
    uint64_t header = 0;
    memcpy(&header, f.data, 8);
    if (header > (uint64_t)f.size - 8) return fail(ctx, TSM_ERR_IO, std::string(path) + " is not a safetensors file");
    f.payload = 8 + (int64_t)header;
    StParser js{(const char*)f.data + 8, (const char*)f.data + 8 + header};
    if (!js.take('{')) js.bad = true;
    if (!js.take('}')) {
        do {
            std::string name = js.text();
            if (!js.take(':')) js.bad = true;
            if (name == "__metadata__") {
                js.skip();
                continue;
            }
            StEntry e;
            if (!js.take('{')) js.bad = true;
            do {
                std::string key = js.text();
                if (!js.take(':')) js.bad = true;
                if (key == "dtype") {
                    e.dtype = js.text();
                } else if (key == "shape") {
                    if (!js.take('[')) js.bad = true;
                    if (!js.take(']')) {
                        do e.shape.push_back(js.integer());
                        while (!js.bad && js.take(','));
                        if (!js.take(']')) js.bad = true;
                    }
                } else if (key == "data_offsets") {
                    if (!js.take('[')) js.bad = true;
                    e.begin = js.integer();
                    if (!js.take(',')) js.bad = true;
                    e.end = js.integer();
                    if (!js.take(']')) js.bad = true;
                } else {
                    js.skip();
                }
            } while (!js.bad && js.take(','));
            if (!js.take('}')) js.bad = true;
            if (e.begin < 0 || e.end < e.begin || f.payload + e.end > f.size) js.bad = true;
            f.entries[name] = e;
        } while (!js.bad && js.take(','));
        if (!js.take('}')) js.bad = true;
    }
    if (js.bad) return fail(ctx, TSM_ERR_IO, std::string(path) + ": malformed safetensors header");
    return TSM_OK;
}

// The tensor `name` as F32 values (F16 and BF16 are widened, as llama.cr:163-164 says the reference does).
static int st_values(tsm_model* m, StFile& f, const std::string& name, std::vector<int64_t> shape, std::vector<float>& out) {
    auto found = f.entries.find(name);
    if (found == f.entries.end()) return fail(m->ctx, TSM_ERR_IO, "the file lacks " + name);
    const StEntry& e = found->second;
    if (e.shape != shape) return fail(m->ctx, TSM_ERR_ARG, name + ": the file's shape does not match the model's");
    int64_t count = 1;
    for (int64_t d : shape) count *= d;
    const uint8_t* src = f.data + f.payload + e.begin;
    out.resize((size_t)count);
    if (e.dtype == "F32" && e.end - e.begin == count * 4) {
        memcpy(out.data(), src, (size_t)count * 4);
    } else if ((e.dtype == "F16" || e.dtype == "BF16") && e.end - e.begin == count * 2) {
        const uint16_t* h = (const uint16_t*)src;
        for (int64_t i = 0; i < count; i++) {
            if (e.dtype == "BF16") {
                uint32_t u = (uint32_t)h[i] << 16;
                memcpy(&out[(size_t)i], &u, 4);
            } else {
                out[(size_t)i] = __half2float(__ushort_as_half(h[i]));
            }
        }
    } else {
        return fail(m->ctx, TSM_ERR_UNSUPPORTED, name + ": " + e.dtype + " tensors are not supported");
    }
    return TSM_OK;
}

static int st_vector(tsm_model* m, StFile& f, const std::string& name, int64_t n, float** out) {
    std::vector<float> values;
    TSM_TRY(st_values(m, f, name, {n}, values));
    TSM_TRY(dev_alloc(m, n * 4, (void**)out));
    return tsm_upload(m->ctx, (tsm_dptr)(uintptr_t)*out, values.data(), n * 4);
}

// Row-major [n, k] F32 values -> a quantised Linear holding the rows of `ranges` (all when empty).
static int linear_from_values(tsm_model* m, const std::vector<float>& values, int64_t n, int64_t k, int kind, Linear* out,
                              const std::vector<RowRange>& ranges = {}) {
    if (kind == TSM_F32) {  // kept as it is: Module#load without Module#quantize
        std::vector<RowRange> keep = ranges;
        if (keep.empty()) keep.push_back({0, n});
        int64_t local = 0;
        for (auto& range : keep) local += range.count;
        out->kind = kind, out->n = (int)local, out->k = (int)k;
        TSM_TRY(dev_alloc(m, weight_bytes(kind, local, k), (void**)&out->w));
        int64_t at = 0;
        for (auto& range : keep) {
            TSM_TRY(tsm_upload(m->ctx, (tsm_dptr)(uintptr_t)(out->w + weight_bytes(kind, at, k)), values.data() + range.start * k, range.count * k * 4));
            at += range.count;
        }
        return TSM_OK;
    }
    if (k % 32 != 0) return fail(m->ctx, TSM_ERR_ARG, "rows of " + std::to_string(k) + " do not split into blocks of 32");
    float* staged = nullptr;
    TSM_TRY(pool_alloc(m->ctx, n * k * 4, (void**)&staged));
    int rc = tsm_upload(m->ctx, (tsm_dptr)(uintptr_t)staged, values.data(), n * k * 4);
    std::vector<RowRange> keep = ranges;
    if (keep.empty()) keep.push_back({0, n});
    int64_t local = 0;
    for (auto& range : keep) local += range.count;
    out->kind = kind, out->n = (int)local, out->k = (int)k;
    if (rc == TSM_OK) rc = dev_alloc(m, weight_bytes(kind, local, k), (void**)&out->w);
    int64_t at = 0;
    for (auto& range : keep) {
        if (rc == TSM_OK) rc = launch_quantize_blocks(m->ctx, staged + range.start * k, range.count * k, kind, out->w + weight_bytes(kind, at, k));
        at += range.count;
    }
    cudaStreamSynchronize(m->ctx->stream);
    pool_release(m->ctx, staged);
    return rc;
}

// A Linear from one or more tensors stacked by rows; `transposed` tensors are stored [in, out] (GPT-2's Conv1D, gpt2.cr's TRANSPOSED).
static int st_linear(tsm_model* m, StFile& f, const std::vector<std::string>& names, int64_t k, bool transposed, int kind, Linear* out,
                     const std::vector<RowRange>& ranges = {}) {
    std::vector<float> all;
    int64_t n = 0;
    for (auto& name : names) {
        auto found = f.entries.find(name);
        if (found == f.entries.end()) return fail(m->ctx, TSM_ERR_IO, "the file lacks " + name);
        const std::vector<int64_t>& shape = found->second.shape;
        if (shape.size() != 2 || shape[transposed ? 0 : 1] != k) return fail(m->ctx, TSM_ERR_ARG, name + ": the file's shape does not match the model's");
        int64_t rows = shape[transposed ? 1 : 0];
        std::vector<float> part;
        TSM_TRY(st_values(m, f, name, shape, part));
        size_t base = all.size();
        all.resize(base + (size_t)(rows * k));
        if (transposed) {
            for (int64_t i = 0; i < k; i++)
                for (int64_t j = 0; j < rows; j++) all[base + (size_t)(j * k + i)] = part[(size_t)(i * rows + j)];
        } else {
            memcpy(&all[base], part.data(), (size_t)(rows * k) * 4);
        }
        n += rows;
    }
    return linear_from_values(m, all, n, k, kind, out, ranges);
}

static int load_gpt2_safetensors(tsm_model* m, StFile& f, int heads, int kind) {
    std::string p = f.entries.count("transformer.wte.weight") ? "transformer." : "";
    if (!f.entries.count(p + "wte.weight") || !f.entries.count(p + "wpe.weight")) return fail(m->ctx, TSM_ERR_IO, "the file lacks wte.weight or wpe.weight");
    tsm_model_config& c = m->cfg;
    c.arch = 1;
    c.vocab = (int)f.entries[p + "wte.weight"].shape[0];
    c.width = (int)f.entries[p + "wte.weight"].shape[1];
    c.context = (int)f.entries[p + "wpe.weight"].shape[0];
    c.layers = 0;
    while (f.entries.count(p + "h." + std::to_string(c.layers) + ".ln_1.weight")) c.layers++;
    c.heads = c.kv_heads = heads;
    c.head_width = heads > 0 ? c.width / heads : 0;
    c.hidden = 4 * c.width;
    c.eps = 1e-5f, c.rope_theta = 0, c.tied = 1;
    TSM_TRY(check_config(m->ctx, c));
    TSM_TRY(check_sharding(m));
    TSM_TRY(st_linear(m, f, {p + "wte.weight"}, c.width, false, kind, &m->embed));
    TSM_TRY(st_linear(m, f, {p + "wpe.weight"}, c.width, false, kind, &m->wpe));
    m->head = m->embed;
    TSM_TRY(st_vector(m, f, p + "ln_f.weight", c.width, &m->final_w));
    TSM_TRY(st_vector(m, f, p + "ln_f.bias", c.width, &m->final_b));
    m->layers.resize(c.layers);
    for (int i = 0; i < c.layers; i++) {
        std::string h = p + "h." + std::to_string(i) + ".";
        Layer& l = m->layers[i];
        TSM_TRY(st_vector(m, f, h + "ln_1.weight", c.width, &l.norm1_w));
        TSM_TRY(st_vector(m, f, h + "ln_1.bias", c.width, &l.norm1_b));
        TSM_TRY(st_vector(m, f, h + "ln_2.weight", c.width, &l.norm2_w));
        TSM_TRY(st_vector(m, f, h + "ln_2.bias", c.width, &l.norm2_b));
        TSM_TRY(st_linear(m, f, {h + "attn.c_attn.weight"}, c.width, true, kind, &l.qkv, shard_ranges(m, SHARD_QKV)));
        TSM_TRY(st_vector(m, f, h + "attn.c_attn.bias", 3 * c.width, &l.qkv.bias));
        TSM_TRY(shard_bias(m, &l.qkv.bias, shard_ranges(m, SHARD_QKV)));
        TSM_TRY(st_linear(m, f, {h + "attn.c_proj.weight"}, c.width, true, kind, &l.o, shard_ranges(m, SHARD_WIDTH)));
        TSM_TRY(st_vector(m, f, h + "attn.c_proj.bias", c.width, &l.o.bias));
        TSM_TRY(shard_bias(m, &l.o.bias, shard_ranges(m, SHARD_WIDTH)));
        TSM_TRY(st_linear(m, f, {h + "mlp.c_fc.weight"}, c.width, true, kind, &l.up, shard_ranges(m, SHARD_UP)));
        TSM_TRY(st_vector(m, f, h + "mlp.c_fc.bias", c.hidden, &l.up.bias));
        TSM_TRY(shard_bias(m, &l.up.bias, shard_ranges(m, SHARD_UP)));
        TSM_TRY(st_linear(m, f, {h + "mlp.c_proj.weight"}, c.hidden, true, kind, &l.down, shard_ranges(m, SHARD_WIDTH)));
        TSM_TRY(st_vector(m, f, h + "mlp.c_proj.bias", c.width, &l.down.bias));
        TSM_TRY(shard_bias(m, &l.down.bias, shard_ranges(m, SHARD_WIDTH)));
        TSM_TRY(shard_inputs(m, l));
    }
    return TSM_OK;
}

// Hugging Face Llama names; heads, kv heads, eps, theta and context come from the caller's config (the model
// directory's config.json, which the host reads: llama.cr:165-175); the other sizes from the shapes.
static int load_llama_safetensors(tsm_model* m, StFile& f, const tsm_model_config& given, int kind) {
    if (!f.entries.count("model.embed_tokens.weight")) return fail(m->ctx, TSM_ERR_IO, "the file lacks model.embed_tokens.weight");
    tsm_model_config& c = m->cfg;
    c = given;
    c.arch = 0;
    c.vocab = (int)f.entries["model.embed_tokens.weight"].shape[0];
    c.width = (int)f.entries["model.embed_tokens.weight"].shape[1];
    c.layers = 0;
    while (f.entries.count("model.layers." + std::to_string(c.layers) + ".input_layernorm.weight")) c.layers++;
    if (c.layers < 1) return fail(m->ctx, TSM_ERR_IO, "the file has no model.layers.0");
    if (c.head_width <= 0 && c.heads > 0) c.head_width = c.width / c.heads;
    if (c.kv_heads <= 0) c.kv_heads = c.heads;
    c.hidden = (int)f.entries["model.layers.0.mlp.gate_proj.weight"].shape[0];
    c.tied = f.entries.count("lm_head.weight") ? 0 : 1;
    TSM_TRY(check_config(m->ctx, c));
    TSM_TRY(check_sharding(m));
    int qn = c.heads * c.head_width;
    TSM_TRY(st_linear(m, f, {"model.embed_tokens.weight"}, c.width, false, kind, &m->embed));
    if (!c.tied) TSM_TRY(st_linear(m, f, {"lm_head.weight"}, c.width, false, kind, &m->head, shard_ranges(m, SHARD_VOCAB)));
    else m->head = m->embed;
    TSM_TRY(st_vector(m, f, "model.norm.weight", c.width, &m->final_w));
    m->layers.resize(c.layers);
    for (int i = 0; i < c.layers; i++) {
        std::string p = "model.layers." + std::to_string(i) + ".";
        Layer& l = m->layers[i];
        TSM_TRY(st_vector(m, f, p + "input_layernorm.weight", c.width, &l.norm1_w));
        TSM_TRY(st_vector(m, f, p + "post_attention_layernorm.weight", c.width, &l.norm2_w));
        TSM_TRY(st_linear(m, f, {p + "self_attn.q_proj.weight", p + "self_attn.k_proj.weight", p + "self_attn.v_proj.weight"}, c.width, false, kind,
                          &l.qkv, shard_ranges(m, SHARD_QKV)));
        if (l.qkv.n * m->tp != qn + 2 * c.kv_heads * c.head_width) return fail(m->ctx, TSM_ERR_ARG, "q, k and v projections do not match the heads given");
        TSM_TRY(st_linear(m, f, {p + "self_attn.o_proj.weight"}, qn, false, kind, &l.o, shard_ranges(m, SHARD_WIDTH)));
        TSM_TRY(st_linear(m, f, {p + "mlp.gate_proj.weight", p + "mlp.up_proj.weight"}, c.width, false, kind, &l.up, shard_ranges(m, SHARD_UP)));
        TSM_TRY(st_linear(m, f, {p + "mlp.down_proj.weight"}, c.hidden, false, kind, &l.down, shard_ranges(m, SHARD_WIDTH)));
        TSM_TRY(shard_inputs(m, l));
    }
    return make_rope_tables(m);
}

// ---- one packed step -----------------------------------------------------------------------------

// Whether any Linear of the model (the head included) kept an F32 weight.
static bool has_f32_matrix(const tsm_model* m) {
    if (m->head.kind == TSM_F32) return true;
    for (const Layer& l : m->layers)
        if (l.qkv.kind == TSM_F32 || l.o.kind == TSM_F32 || l.up.kind == TSM_F32 || l.down.kind == TSM_F32) return true;
    return false;
}

static void free_workspace(tsm_model* m) {
    Workspace& w = m->ws;
    void* bufs[] = {w.ids, w.table, w.last, w.order, w.x, w.xl, w.qkv, w.att, w.up, w.h, w.logits, w.picks, w.qa, w.qb, w.qc, w.tp_parts, w.tp_rows, w.tp_best};
    for (void* b : bufs) pool_release(m->ctx, b);
    if (w.host) cudaFreeHost(w.host);
    w = Workspace{};
}

static int ensure_workspace(tsm_model* m, int tokens) {
    if (m->ws.tokens >= tokens) return TSM_OK;
    cudaStreamSynchronize(m->ctx->stream);
    free_workspace(m);
    const tsm_model_config& c = m->cfg;
    Workspace& w = m->ws;
    int64_t T = tokens;
    int qn = c.heads * c.head_width, kvn = c.kv_heads * c.head_width;
    int upn = c.arch == 0 ? 2 * c.hidden : c.hidden;
    tsm_ctx* ctx = m->ctx;
    TSM_TRY(pool_alloc(ctx, T * 4, (void**)&w.ids));
    TSM_TRY(pool_alloc(ctx, T * 12, (void**)&w.table));
    TSM_TRY(pool_alloc(ctx, T * 4, (void**)&w.last));
    TSM_TRY(pool_alloc(ctx, T * 4, (void**)&w.order));
    TSM_TRY(pool_alloc(ctx, T * c.width * 4, (void**)&w.x));
    TSM_TRY(pool_alloc(ctx, T * c.width * 4, (void**)&w.xl));
    TSM_TRY(pool_alloc(ctx, T * (qn + 2 * kvn) * 4, (void**)&w.qkv));
    TSM_TRY(pool_alloc(ctx, T * qn * 4, (void**)&w.att));
    TSM_TRY(pool_alloc(ctx, T * upn * 4, (void**)&w.up));
    if (has_f32_matrix(m)) TSM_TRY(pool_alloc(ctx, T * std::max(c.width, c.hidden) * 4, (void**)&w.h));
    TSM_TRY(pool_alloc(ctx, T * c.vocab * 4, (void**)&w.logits));
    TSM_TRY(pool_alloc(ctx, T * 4, (void**)&w.picks));
    if (m->tp > 1) {
        int64_t widest = std::max<int64_t>(std::max<int64_t>(qn, c.width), std::max<int64_t>(c.hidden, c.vocab));
        TSM_TRY(pool_alloc(ctx, T * widest * 4, (void**)&w.tp_parts));
        TSM_TRY(pool_alloc(ctx, T * std::max<int64_t>(std::max<int64_t>(qn, c.width), c.hidden) * 4, (void**)&w.tp_rows));
        TSM_TRY(pool_alloc(ctx, (int64_t)m->tp * 2 * T * 4, (void**)&w.tp_best));
    }
    TSM_TRY(pool_alloc(ctx, quant_scratch_bytes(tokens, c.width), &w.qa));
    TSM_TRY(pool_alloc(ctx, quant_scratch_bytes(tokens, qn), &w.qb));
    TSM_TRY(pool_alloc(ctx, quant_scratch_bytes(tokens, c.hidden), &w.qc));
    TSM_CUDA(ctx, cudaMallocHost((void**)&w.host, (size_t)T * 5 * 4));
    w.tokens = tokens;
    m->ws_generation++;
    return TSM_OK;
}

// A Linear over `rows` rows.  A block weight reads the quantised rows `a`; a weight that stayed F32 reads the rows
// themselves, `plain`.  Whoever produces the rows asks feeds() which of the two this Linear wants.
static int product(tsm_model* m, const QuantizedActs& a, const float* plain, int rows, const Linear& l, const float* residual, float* out) {
    if (l.kind == TSM_F32) return launch_matmul_f32(m->ctx, plain, rows, l.k, (const float*)l.w, l.n, l.bias, residual, out);
    return launch_block_matmul(m->ctx, a, rows, l.k, l.w, l.kind, l.n, l.bias, residual, out);
}

// Where the producer of a Linear's input writes: F32 rows for an F32 weight, quantised blocks otherwise.
struct Feed {
    float* plain;
    const QuantizedActs* quantized;
};
static Feed feeds(const Linear& l, float* plain, const QuantizedActs* quantized) {
    return l.kind == TSM_F32 ? Feed{plain, nullptr} : Feed{nullptr, quantized};
}

// Tensor-parallel greedy pick: every rank holds, for each row, the best logit of its vocabulary slice and that logit's
// index within the slice ([ranks][2][rows] as gathered).  The highest wins; equal values go to the lower rank, whose
// slice holds the lower indices (Sampler.greedy keeps the first maximum).
__global__ void combine_picks_kernel(const float* __restrict__ best, int rows, int ranks, int slice, int* picks) {
    chained_kernel_entry();
    int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= rows) return;
    float top = best[t];
    int who = 0;
    for (int r = 1; r < ranks; r++) {
        float v = best[(int64_t)r * 2 * rows + t];
        if (v > top) top = v, who = r;
    }
    int index = ((const int*)best)[(int64_t)who * 2 * rows + rows + t];
    picks[t] = who * slice + index;
}

// One layer and the head of a tensor-parallel step.  Projections are split by output rows (shard_ranges), so a rank
// computes whole outputs in block order; what the next projection needs from the other ranks arrives by an in-place
// all-gather of column slices ([ranks][tokens, slice]) and is put back in row order by launch_interleave, which also
// performs the residual add where one follows.  Norms and quantisers run on full rows on every rank.  The bits are
// those of the one-GPU step.
static int launch_layer_sharded(tsm_model* m, tsm_cache* cache, int i, int total, const int* order, const QuantizedActs& qa,
                                const QuantizedActs& qb, const QuantizedActs& qc, bool ordered, float scale) {
    const tsm_model_config& c = m->cfg;
    tsm_ctx* ctx = m->ctx;
    Workspace& w = m->ws;
    Layer& l = m->layers[i];
    const int G = m->tp, r = m->tp_rank, hw = c.head_width;
    const int heads_l = c.heads / G, kv_l = c.kv_heads / G, qn = c.heads * hw, qn_l = heads_l * hw, qkvn_l = qn_l + 2 * kv_l * hw;
    const int hid_l = c.hidden / G, w_l = c.width / G;
    (void)ordered;
    if (c.arch == 0) TSM_TRY(launch_rmsnorm(ctx, w.x, l.norm1_w, total, c.width, c.eps, nullptr, &qa));
    else TSM_TRY(launch_layernorm(ctx, w.x, l.norm1_w, l.norm1_b, total, c.width, c.eps, nullptr, &qa));
    TSM_TRY(product(m, qa, nullptr, total, l.qkv, nullptr, w.qkv));
    TSM_TRY(launch_rope_append(ctx, w.qkv, total, heads_l, kv_l, hw, c.arch == 0 ? m->rope_cos : nullptr, c.arch == 0 ? m->rope_sin : nullptr,
                               c.context, w.table, cache->keys[i], cache->values[i], cache->rows, cache->capacity));
    TSM_TRY(launch_attention(ctx, w.qkv, qkvn_l, total, heads_l, hw, cache->keys[i], cache->values[i], cache->rows, kv_l, cache->capacity,
                             w.table, scale, w.tp_parts + (int64_t)r * total * qn_l, nullptr, order));
    TSM_TRY(tp_all_gather(ctx, w.tp_parts, (int64_t)total * qn_l * 4));
    TSM_TRY(launch_interleave(ctx, w.tp_parts, w.tp_rows, total, qn_l, G, false));
    TSM_TRY(launch_quantize_rows(ctx, w.tp_rows, total, qn, qn, (float*)qb.scales, (float*)qb.sums, (int*)qb.totals, (int8_t*)qb.qs));
    TSM_TRY(product(m, qb, nullptr, total, l.o, nullptr, w.tp_parts + (int64_t)r * total * w_l));
    TSM_TRY(tp_all_gather(ctx, w.tp_parts, (int64_t)total * w_l * 4));
    TSM_TRY(launch_interleave(ctx, w.tp_parts, w.x, total, w_l, G, true));
    if (c.arch == 0) TSM_TRY(launch_rmsnorm(ctx, w.x, l.norm2_w, total, c.width, c.eps, nullptr, &qa));
    else TSM_TRY(launch_layernorm(ctx, w.x, l.norm2_w, l.norm2_b, total, c.width, c.eps, nullptr, &qa));
    TSM_TRY(product(m, qa, nullptr, total, l.up, nullptr, w.up));
    float* hidden_part = w.tp_parts + (int64_t)r * total * hid_l;
    if (c.arch == 0) TSM_TRY(launch_swiglu(ctx, w.up, w.up + hid_l, total, hid_l, 2 * (int64_t)hid_l, hidden_part, nullptr));
    else TSM_TRY(launch_gelu(ctx, w.up, total, hid_l, hidden_part, nullptr));
    TSM_TRY(tp_all_gather(ctx, w.tp_parts, (int64_t)total * hid_l * 4));
    TSM_TRY(launch_interleave(ctx, w.tp_parts, w.tp_rows, total, hid_l, G, false));
    TSM_TRY(launch_quantize_rows(ctx, w.tp_rows, total, c.hidden, c.hidden, (float*)qc.scales, (float*)qc.sums, (int*)qc.totals, (int8_t*)qc.qs));
    TSM_TRY(product(m, qc, nullptr, total, l.down, nullptr, w.tp_parts + (int64_t)r * total * w_l));
    TSM_TRY(tp_all_gather(ctx, w.tp_parts, (int64_t)total * w_l * 4));
    TSM_TRY(launch_interleave(ctx, w.tp_parts, w.x, total, w_l, G, true));
    return TSM_OK;
}

// One layer of a TSM_TP_REDUCE step: q/k/v and gate/up by output rows as above, then o and down over this rank's own input
// columns (its heads' attention output, its slice of the hidden width, quantised where they are made) with an all-reduce of
// the partial sums; two exchanges per layer.  The partial sums are added in NCCL's order, not in block order.
static int launch_layer_reduced(tsm_model* m, tsm_cache* cache, int i, int total, const int* order, const QuantizedActs& qa, float scale) {
    const tsm_model_config& c = m->cfg;
    tsm_ctx* ctx = m->ctx;
    Workspace& w = m->ws;
    Layer& l = m->layers[i];
    const int G = m->tp, hw = c.head_width;
    const int heads_l = c.heads / G, kv_l = c.kv_heads / G, qn_l = heads_l * hw, qkvn_l = qn_l + 2 * kv_l * hw, hid_l = c.hidden / G;
    QuantizedActs qb = quant_scratch_layout(w.qb, total, qn_l);
    QuantizedActs qc = quant_scratch_layout(w.qc, total, hid_l);
    const int64_t count = (int64_t)total * c.width;
    if (c.arch == 0) TSM_TRY(launch_rmsnorm(ctx, w.x, l.norm1_w, total, c.width, c.eps, nullptr, &qa));
    else TSM_TRY(launch_layernorm(ctx, w.x, l.norm1_w, l.norm1_b, total, c.width, c.eps, nullptr, &qa));
    TSM_TRY(product(m, qa, nullptr, total, l.qkv, nullptr, w.qkv));
    TSM_TRY(launch_rope_append(ctx, w.qkv, total, heads_l, kv_l, hw, c.arch == 0 ? m->rope_cos : nullptr, c.arch == 0 ? m->rope_sin : nullptr,
                               c.context, w.table, cache->keys[i], cache->values[i], cache->rows, cache->capacity));
    TSM_TRY(launch_attention(ctx, w.qkv, qkvn_l, total, heads_l, hw, cache->keys[i], cache->values[i], cache->rows, kv_l, cache->capacity,
                             w.table, scale, w.att, &qb, order));
    TSM_TRY(product(m, qb, nullptr, total, l.o, nullptr, w.tp_rows));
    TSM_TRY(tp_all_reduce_sum(ctx, w.tp_rows, count));
    TSM_TRY(launch_add(ctx, w.x, w.tp_rows, count, w.x));
    if (c.arch == 0) TSM_TRY(launch_rmsnorm(ctx, w.x, l.norm2_w, total, c.width, c.eps, nullptr, &qa));
    else TSM_TRY(launch_layernorm(ctx, w.x, l.norm2_w, l.norm2_b, total, c.width, c.eps, nullptr, &qa));
    TSM_TRY(product(m, qa, nullptr, total, l.up, nullptr, w.up));
    if (c.arch == 0) TSM_TRY(launch_swiglu(ctx, w.up, w.up + hid_l, total, hid_l, 2 * (int64_t)hid_l, nullptr, &qc));
    else TSM_TRY(launch_gelu(ctx, w.up, total, hid_l, nullptr, &qc));
    TSM_TRY(product(m, qc, nullptr, total, l.down, nullptr, w.tp_rows));
    TSM_TRY(tp_all_reduce_sum(ctx, w.tp_rows, count));
    TSM_TRY(launch_add(ctx, w.x, w.tp_rows, count, w.x));
    return TSM_OK;
}

// The head of a tensor-parallel step: this rank's vocabulary slice, the greedy pick across ranks, and (when asked) the
// full logits in ws.logits.
static int launch_head_sharded(tsm_model* m, const QuantizedActs& qh, int outputs, bool pick, bool full_logits) {
    const tsm_model_config& c = m->cfg;
    tsm_ctx* ctx = m->ctx;
    Workspace& w = m->ws;
    const int G = m->tp, r = m->tp_rank, slice = c.vocab / G;
    Linear head = m->head_local;
    head.bias = nullptr;
    float* mine = w.tp_parts + (int64_t)r * outputs * slice;
    TSM_TRY(launch_block_matmul(ctx, qh, outputs, head.k, head.w, head.kind, head.n, nullptr, nullptr, mine));
    if (pick) {
        float* best = w.tp_best + (int64_t)r * 2 * outputs;
        TSM_TRY(launch_topk(ctx, mine, outputs, slice, 1, (int*)(best + outputs), best));
        TSM_TRY(tp_all_gather(ctx, w.tp_best, (int64_t)2 * outputs * 4));
        TSM_CUDA(ctx, launch_chained(ctx, combine_picks_kernel, dim3((outputs + 255) / 256), dim3(256), 0, w.tp_best, outputs, G, slice, w.picks));
        count_launch(ctx);
        TSM_LAUNCH_CHECK(ctx);
    }
    if (full_logits) {
        TSM_TRY(tp_all_gather(ctx, w.tp_parts, (int64_t)outputs * slice * 4));
        TSM_TRY(launch_interleave(ctx, w.tp_parts, w.logits, outputs, slice, G, false));
    }
    return TSM_OK;
}

// After a tensor-parallel step that only picked tokens: the ranks' logit slices, still in place, gathered into ws.logits.
static int gather_full_logits(tsm_model* m, int outputs) {
    int slice = m->cfg.vocab / m->tp;
    TSM_TRY(tp_all_gather(m->ctx, m->ws.tp_parts, (int64_t)outputs * slice * 4));
    return launch_interleave(m->ctx, m->ws.tp_parts, m->ws.logits, outputs, slice, m->tp, false);
}

// Launches one step over `total` packed tokens whose ids and table are already in the workspace.
// `outputs` rows (indices in ws.last when fewer than total) go through the final norm and the head.
static int launch_step_kernels(tsm_model* m, tsm_cache* cache, int total, int outputs, bool pick);

static int launch_step(tsm_model* m, tsm_cache* cache, int total, int outputs, bool pick) {
    m->ctx->chain_launches = total <= 4;  // a few rows: a chain of very short kernels, worth overlapping their launches
    int rc = launch_step_kernels(m, cache, total, outputs, pick);
    m->ctx->chain_launches = false;
    return rc;
}

static int launch_step_kernels(tsm_model* m, tsm_cache* cache, int total, int outputs, bool pick) {
    const tsm_model_config& c = m->cfg;
    tsm_ctx* ctx = m->ctx;
    Workspace& w = m->ws;
    int hw = c.head_width, qn = c.heads * hw, kvn = c.kv_heads * hw, qkvn = qn + 2 * kvn;
    QuantizedActs qa = quant_scratch_layout(w.qa, total, c.width);
    QuantizedActs qb = quant_scratch_layout(w.qb, total, qn);
    QuantizedActs qc = quant_scratch_layout(w.qc, total, c.hidden);
    float scale = (float)(1.0 / sqrt((double)hw));
    bool ordered = ctx->mode == TSM_EXACT || !(hw == 64 || hw == 128);

    if (m->tp > 1 && (has_f32_matrix(m) || m->embed.kind == TSM_F32))
        return fail(ctx, TSM_ERR_UNSUPPORTED, "tensor parallelism takes block-quantised weights only");
    if (c.arch == 1 && m->wpe.kind != m->embed.kind) return fail(ctx, TSM_ERR_UNSUPPORTED, "token and position tables must share a format");
    const int* positions = c.arch == 1 ? w.table + 1 : nullptr;  // gpt2.cr:189-191: wte(ids) + wpe(positions)
    if (m->embed.kind == TSM_F32) {
        TSM_TRY(launch_gather_f32(ctx, (const float*)m->embed.w, c.vocab, c.width, w.ids, total, w.x, c.arch == 1 ? (const float*)m->wpe.w : nullptr,
                                  positions, 3));
    } else {
        TSM_TRY(launch_gather_blocks(ctx, m->embed.w, m->embed.kind, c.vocab, c.width, w.ids, total, w.x, c.arch == 1 ? m->wpe.w : nullptr,
                                     positions, 3));
    }
    const int* order = nullptr;
    if (total > 1 && total <= 4096) {  // the same order serves every layer of the step
        TSM_TRY(launch_length_order(ctx, w.table, total, w.order));
        order = w.order;
    }
    for (int i = 0; i < c.layers; i++) {
        if (m->tp > 1) {
            if (m->tp_reduce) TSM_TRY(launch_layer_reduced(m, cache, i, total, order, qa, scale));
            else TSM_TRY(launch_layer_sharded(m, cache, i, total, order, qa, qb, qc, ordered, scale));
            continue;
        }
        Layer& l = m->layers[i];
        Feed f = feeds(l.qkv, w.h, &qa);
        if (c.arch == 0) TSM_TRY(launch_rmsnorm(ctx, w.x, l.norm1_w, total, c.width, c.eps, f.plain, f.quantized));
        else TSM_TRY(launch_layernorm(ctx, w.x, l.norm1_w, l.norm1_b, total, c.width, c.eps, f.plain, f.quantized));
        TSM_TRY(product(m, qa, w.h, total, l.qkv, nullptr, w.qkv));
        TSM_TRY(launch_rope_append(ctx, w.qkv, total, c.heads, c.kv_heads, hw, c.arch == 0 ? m->rope_cos : nullptr,
                                   c.arch == 0 ? m->rope_sin : nullptr, c.context, w.table, cache->keys[i], cache->values[i],
                                   cache->rows, cache->capacity));
        f = feeds(l.o, w.att, &qb);
        TSM_TRY(launch_attention(ctx, w.qkv, qkvn, total, c.heads, hw, cache->keys[i], cache->values[i], cache->rows, c.kv_heads,
                                 cache->capacity, w.table, scale, ordered || f.plain ? w.att : nullptr, f.quantized, order));
        TSM_TRY(product(m, qb, w.att, total, l.o, w.x, w.x));
        f = feeds(l.up, w.h, &qa);
        if (c.arch == 0) TSM_TRY(launch_rmsnorm(ctx, w.x, l.norm2_w, total, c.width, c.eps, f.plain, f.quantized));
        else TSM_TRY(launch_layernorm(ctx, w.x, l.norm2_w, l.norm2_b, total, c.width, c.eps, f.plain, f.quantized));
        TSM_TRY(product(m, qa, w.h, total, l.up, nullptr, w.up));
        f = feeds(l.down, w.h, &qc);
        if (c.arch == 0) TSM_TRY(launch_swiglu(ctx, w.up, w.up + c.hidden, total, c.hidden, 2 * (int64_t)c.hidden, f.plain, f.quantized));
        else TSM_TRY(launch_gelu(ctx, w.up, total, c.hidden, f.plain, f.quantized));
        TSM_TRY(product(m, qc, w.h, total, l.down, w.x, w.x));
    }
    const float* xl = w.x;
    if (outputs < total) {
        TSM_TRY(launch_gather_f32(ctx, w.x, total, c.width, w.last, outputs, w.xl));
        xl = w.xl;
    }
    QuantizedActs qh = quant_scratch_layout(w.qa, outputs, c.width);
    Feed f = feeds(m->head, w.h, &qh);
    if (c.arch == 0) TSM_TRY(launch_rmsnorm(ctx, xl, m->final_w, outputs, c.width, c.eps, f.plain, f.quantized));
    else TSM_TRY(launch_layernorm(ctx, xl, m->final_w, m->final_b, outputs, c.width, c.eps, f.plain, f.quantized));
    if (m->tp > 1) return launch_head_sharded(m, qh, outputs, pick, !pick);
    Linear head = m->head;
    head.bias = nullptr;
    TSM_TRY(product(m, qh, w.h, outputs, head, nullptr, w.logits));
    if (pick) TSM_TRY(launch_argmax(ctx, w.logits, outputs, c.vocab, w.picks));
    return TSM_OK;
}

static int prepare_scratch(tsm_model* m, tsm_cache* cache, int tokens) {
    const tsm_model_config& c = m->cfg;
    TSM_TRY(ensure_workspace(m, tokens));
    if (m->ctx->mode == TSM_FAST && (c.head_width == 64 || c.head_width == 128))
        TSM_TRY(ensure_scratch(m->ctx, m->ctx->attn, attention_scratch_bytes(tokens, c.heads, c.head_width, cache->capacity)));
    if (m->ctx->mode != TSM_FAST && c.head_width == 128 && c.kv_heads > 0 && (c.heads / c.kv_heads) % 4 == 0)
        TSM_TRY(ensure_scratch(m->ctx, m->ctx->attn, attention_stream_scratch_bytes(tokens, c.heads, cache->capacity)));
    return TSM_OK;
}

static void drop_graph(tsm_cache* cache) {
    if (cache->graph) cudaGraphExecDestroy(cache->graph);
    cache->graph = nullptr;
}

// Kernel nodes of a captured step: what one replay launches.
static int kernel_nodes(cudaGraph_t graph) {
    size_t count = 0;
    if (cudaGraphGetNodes(graph, nullptr, &count) != cudaSuccess || count == 0) return 0;
    std::vector<cudaGraphNode_t> nodes(count);
    if (cudaGraphGetNodes(graph, nodes.data(), &count) != cudaSuccess) return 0;
    int kernels = 0;
    for (size_t i = 0; i < count; i++) {
        cudaGraphNodeType type;
        if (cudaGraphNodeGetType(nodes[i], &type) == cudaSuccess && type == cudaGraphNodeTypeKernel) kernels++;
    }
    return kernels;
}

static void drop_run_graph(tsm_cache* cache) {
    if (cache->run_graph) cudaGraphExecDestroy(cache->run_graph);
    cache->run_graph = nullptr;
}

// Between the steps of a device-resident run: each row's pick becomes its next token and its
// position moves on, so that no step waits for the host.
__global__ void run_advance_kernel(int* ids, int* table, const int* picks, int rows, const int* state) {
    chained_kernel_entry();
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows || state[0] == 0) return;
    ids[r] = picks[r];
    table[3 * r + 1] += 1;
    table[3 * r + 2] += 1;
}

__global__ void run_record_kernel(const int* picks, int rows, int* state) {
    chained_kernel_entry();
    int r = blockIdx.x * blockDim.x + threadIdx.x;
    int step = state[0];
    if (r < rows) state[1 + (int64_t)step * rows + r] = picks[r];
    __syncthreads();
    if (r == 0) state[0] = step + 1;
}

}  // namespace tsm

#define MODEL_GUARD(m)                                \
    if (!(m) || !(m)->ctx) return TSM_ERR_ARG;        \
    tsm::DeviceGuard device_guard__((m)->ctx->ordinal)

// ---- Module#save to a .gguf file (module.cr:148-164; GGUF.write, gguf.cr:156-191) ---------------------------------
//
// Writes the model as it is held on the device: block formats keep their bytes, F32 stays F32.  A Llama goes out under
// llama.cpp's names with its llama.* metadata and with q and k rows back in llama.cpp's rotary order (the inverse of what
// the loader undoes, llama.cr:226-235), the joined projections cut back into their parts; a GPT-2 under tensomite's own
// names with gpt2.heads.  Either file loads again here and in the reference.

struct SavedTensor {
    std::string name;
    uint32_t kind;               // GGUF's type number
    std::vector<int64_t> shape;  // outermost first
    std::vector<uint8_t> bytes;
};

static uint32_t gguf_kind_of(int kind) { return kind == TSM_Q8_0 ? 8 : kind == TSM_Q4_0 ? 2 : kind == TSM_Q4_1 ? 3 : 0; }

// Rows [first, first + rows) of a weight, downloaded; heads > 0 puts them back into llama.cpp's rotary order.
static int saved_rows(tsm_model* m, const Linear& l, const std::string& name, int64_t first, int64_t rows, int heads, std::vector<SavedTensor>& out) {
    SavedTensor t;
    t.name = name, t.kind = gguf_kind_of(l.kind), t.shape = {rows, (int64_t)l.k};
    int64_t row_bytes = weight_bytes(l.kind, 1, l.k);
    t.bytes.resize((size_t)(rows * row_bytes));
    TSM_TRY(tsm_download(m->ctx, t.bytes.data(), (tsm_dptr)(uintptr_t)(l.w + first * row_bytes), rows * row_bytes));
    if (heads > 0) {
        std::vector<uint8_t> file((size_t)(rows * row_bytes));
        int64_t half = rows / heads / 2, held = 0;
        for (int head = 0; head < heads; head++)
            for (int pair = 0; pair < 2; pair++)
                for (int64_t i = 0; i < half; i++, held++)
                    memcpy(&file[(size_t)((head * 2 * half + 2 * i + pair) * row_bytes)], &t.bytes[(size_t)(held * row_bytes)], (size_t)row_bytes);
        t.bytes.swap(file);
    }
    out.push_back(std::move(t));
    return TSM_OK;
}

static int saved_vector(tsm_model* m, const float* values, const std::string& name, int64_t count, std::vector<SavedTensor>& out) {
    if (!values) return TSM_OK;
    SavedTensor t;
    t.name = name, t.kind = 0, t.shape = {count};
    t.bytes.resize((size_t)count * 4);
    TSM_TRY(tsm_download(m->ctx, t.bytes.data(), (tsm_dptr)(uintptr_t)values, count * 4));
    out.push_back(std::move(t));
    return TSM_OK;
}

struct GgufWriter {
    std::vector<uint8_t> bytes;
    template <typename T>
    void put(T v) {
        const uint8_t* p = (const uint8_t*)&v;
        bytes.insert(bytes.end(), p, p + sizeof(T));
    }
    void str(const std::string& s) {
        put<uint64_t>(s.size());
        bytes.insert(bytes.end(), s.begin(), s.end());
    }
    void u32(const std::string& key, uint32_t v) { str(key), put<uint32_t>(4), put<uint32_t>(v); }
    void f32(const std::string& key, float v) { str(key), put<uint32_t>(6), put<float>(v); }
    void text(const std::string& key, const std::string& v) { str(key), put<uint32_t>(8), str(v); }
};

extern "C" {

int tsm_model_free(tsm_model* model) {
    if (!model) return TSM_OK;
    MODEL_GUARD(model);
    cudaStreamSynchronize(model->ctx->stream);
    free_workspace(model);
    for (void* p : model->owned) pool_release(model->ctx, p);
    delete model;
    return TSM_OK;
}

int tsm_model_load_gguf(tsm_ctx* ctx, const char* path, tsm_model** out) {
    if (!ctx || !path || !out) return TSM_ERR_ARG;
    tsm::DeviceGuard guard(ctx->ordinal);
    *out = nullptr;
    GgufFile f;
    TSM_TRY(gguf_open(ctx, path, f));
    std::unique_ptr<tsm_model> m(new tsm_model());
    m->ctx = ctx;
    m->tp = ctx->tp_world, m->tp_rank = ctx->tp_rank, m->tp_reduce = ctx->tp_world > 1 && ctx->tp_variant == TSM_TP_REDUCE;
    std::string arch = f.strings.count("general.architecture") ? f.strings["general.architecture"] : "";
    int rc;
    if (arch == "llama") rc = load_llama(m.get(), f);
    else if (f.strings.count("gpt2.heads")) rc = load_gpt2(m.get(), f);
    else rc = fail(ctx, TSM_ERR_IO, std::string(path) + " holds a " + arch + " model, not a Llama or GPT-2");
    if (rc != TSM_OK) {
        tsm_model_free(m.release());
        return rc;
    }
    set_head_local(m.get());
    register_names(m.get());
    *out = m.release();
    return TSM_OK;
}

int tsm_model_load_safetensors(tsm_ctx* ctx, const char* path, const tsm_model_config* config, int kind, tsm_model** out) {
    if (!ctx || !path || !config || !out) return TSM_ERR_ARG;
    tsm::DeviceGuard guard(ctx->ordinal);
    *out = nullptr;
    if (kind < TSM_F32 || kind > 2) return fail(ctx, TSM_ERR_UNSUPPORTED, "not a weight format");
    StFile f;
    TSM_TRY(st_open(ctx, path, f));
    std::unique_ptr<tsm_model> m(new tsm_model());
    m->ctx = ctx;
    m->tp = ctx->tp_world, m->tp_rank = ctx->tp_rank, m->tp_reduce = ctx->tp_world > 1 && ctx->tp_variant == TSM_TP_REDUCE;
    int rc;
    if (config->arch == 1) rc = load_gpt2_safetensors(m.get(), f, config->heads, kind);
    else if (config->arch == 0) rc = load_llama_safetensors(m.get(), f, *config, kind);
    else rc = fail(ctx, TSM_ERR_ARG, "unknown architecture");
    if (rc != TSM_OK) {
        tsm_model_free(m.release());
        return rc;
    }
    set_head_local(m.get());
    register_names(m.get());
    *out = m.release();
    return TSM_OK;
}

int tsm_model_random(tsm_ctx* ctx, const tsm_model_config* config, int kind, uint64_t seed, tsm_model** out) {
    if (!ctx || !config || !out) return TSM_ERR_ARG;
    tsm::DeviceGuard guard(ctx->ordinal);
    *out = nullptr;
    if (kind < 0 || kind > 2) return fail(ctx, TSM_ERR_UNSUPPORTED, "not a block format");
    TSM_TRY(check_config(ctx, *config));
    std::unique_ptr<tsm_model> m(new tsm_model());
    m->ctx = ctx;
    m->tp = ctx->tp_world, m->tp_rank = ctx->tp_rank, m->tp_reduce = ctx->tp_world > 1 && ctx->tp_variant == TSM_TP_REDUCE;
    m->cfg = *config;
    if (m->cfg.arch == 1) m->cfg.tied = 1;
    int rc = build_random(m.get(), kind, seed);
    if (rc != TSM_OK) {
        tsm_model_free(m.release());
        return rc;
    }
    register_names(m.get());
    *out = m.release();
    return TSM_OK;
}

int tsm_model_save_gguf(tsm_model* m, const char* path) {
    if (!m || !path) return TSM_ERR_ARG;
    tsm_ctx* ctx = m->ctx;
    tsm::DeviceGuard guard(ctx->ordinal);
    if (m->tp > 1) return fail(ctx, TSM_ERR_UNSUPPORTED, "a tensor-parallel rank holds a part of the model; save from one GPU");
    const tsm_model_config& c = m->cfg;
    TSM_TRY(tsm_sync(ctx));
    std::vector<SavedTensor> tensors;
    GgufWriter head;
    uint64_t keys = 0;
    const int64_t qn = (int64_t)c.heads * c.head_width, kvn = (int64_t)c.kv_heads * c.head_width;
    if (c.arch == 0) {
        head.text("general.architecture", "llama"), keys++;
        head.u32("llama.block_count", (uint32_t)c.layers), keys++;
        head.u32("llama.context_length", (uint32_t)c.context), keys++;
        head.u32("llama.embedding_length", (uint32_t)c.width), keys++;
        head.u32("llama.feed_forward_length", (uint32_t)c.hidden), keys++;
        head.u32("llama.attention.head_count", (uint32_t)c.heads), keys++;
        head.u32("llama.attention.head_count_kv", (uint32_t)c.kv_heads), keys++;
        head.u32("llama.rope.dimension_count", (uint32_t)c.head_width), keys++;
        head.u32("llama.vocab_size", (uint32_t)c.vocab), keys++;
        head.f32("llama.rope.freq_base", (float)c.rope_theta), keys++;
        head.f32("llama.attention.layer_norm_rms_epsilon", c.eps), keys++;
        TSM_TRY(saved_rows(m, m->embed, "token_embd.weight", 0, c.vocab, 0, tensors));
        if (!c.tied) TSM_TRY(saved_rows(m, m->head, "output.weight", 0, c.vocab, 0, tensors));
        TSM_TRY(saved_vector(m, m->final_w, "output_norm.weight", c.width, tensors));
        for (int i = 0; i < c.layers; i++) {
            std::string p = "blk." + std::to_string(i) + ".";
            Layer& l = m->layers[i];
            TSM_TRY(saved_vector(m, l.norm1_w, p + "attn_norm.weight", c.width, tensors));
            TSM_TRY(saved_vector(m, l.norm2_w, p + "ffn_norm.weight", c.width, tensors));
            TSM_TRY(saved_rows(m, l.qkv, p + "attn_q.weight", 0, qn, c.heads, tensors));
            TSM_TRY(saved_rows(m, l.qkv, p + "attn_k.weight", qn, kvn, c.kv_heads, tensors));
            TSM_TRY(saved_rows(m, l.qkv, p + "attn_v.weight", qn + kvn, kvn, 0, tensors));
            TSM_TRY(saved_rows(m, l.o, p + "attn_output.weight", 0, c.width, 0, tensors));
            TSM_TRY(saved_rows(m, l.up, p + "ffn_gate.weight", 0, c.hidden, 0, tensors));
            TSM_TRY(saved_rows(m, l.up, p + "ffn_up.weight", c.hidden, c.hidden, 0, tensors));
            TSM_TRY(saved_rows(m, l.down, p + "ffn_down.weight", 0, c.width, 0, tensors));
        }
    } else {
        head.text("general.architecture", "gpt2"), keys++;
        head.text("gpt2.heads", std::to_string(c.heads)), keys++;
        TSM_TRY(saved_rows(m, m->embed, "wte.weight", 0, c.vocab, 0, tensors));
        TSM_TRY(saved_rows(m, m->wpe, "wpe.weight", 0, c.context, 0, tensors));
        TSM_TRY(saved_vector(m, m->final_w, "ln_f.weight", c.width, tensors));
        TSM_TRY(saved_vector(m, m->final_b, "ln_f.bias", c.width, tensors));
        for (int i = 0; i < c.layers; i++) {
            std::string p = "h." + std::to_string(i) + ".";
            Layer& l = m->layers[i];
            TSM_TRY(saved_vector(m, l.norm1_w, p + "ln_1.weight", c.width, tensors));
            TSM_TRY(saved_vector(m, l.norm1_b, p + "ln_1.bias", c.width, tensors));
            TSM_TRY(saved_vector(m, l.norm2_w, p + "ln_2.weight", c.width, tensors));
            TSM_TRY(saved_vector(m, l.norm2_b, p + "ln_2.bias", c.width, tensors));
            const std::pair<const Linear*, const char*> parts[] = {{&l.qkv, "attn.c_attn"}, {&l.o, "attn.c_proj"}, {&l.up, "mlp.c_fc"}, {&l.down, "mlp.c_proj"}};
            for (auto& part : parts) {
                TSM_TRY(saved_rows(m, *part.first, p + part.second + ".weight", 0, part.first->n, 0, tensors));
                TSM_TRY(saved_vector(m, part.first->bias, p + part.second + ".bias", part.first->n, tensors));
            }
        }
    }
    const int64_t alignment = 32;
    GgufWriter file;
    file.put<uint32_t>(0x46554747u);  // "GGUF"
    file.put<uint32_t>(3);
    file.put<uint64_t>(tensors.size());
    file.put<uint64_t>(keys);
    file.bytes.insert(file.bytes.end(), head.bytes.begin(), head.bytes.end());
    int64_t offset = 0;
    std::vector<int64_t> offsets;
    for (auto& t : tensors) {
        file.str(t.name);
        file.put<uint32_t>((uint32_t)t.shape.size());
        for (auto d = t.shape.rbegin(); d != t.shape.rend(); ++d) file.put<uint64_t>((uint64_t)*d);  // innermost first
        file.put<uint32_t>(t.kind);
        file.put<uint64_t>((uint64_t)offset);
        offsets.push_back(offset);
        offset = (offset + (int64_t)t.bytes.size() + alignment - 1) / alignment * alignment;
    }
    file.bytes.resize((file.bytes.size() + alignment - 1) / alignment * alignment, 0);
    // a temporary beside the target, renamed when whole, as GGUF.write does (gguf.cr:165-190)
    std::string temp = std::string(path) + "." + std::to_string((long)getpid()) + ".tmp";
    FILE* fp = fopen(temp.c_str(), "wb");
    if (!fp) return fail(ctx, TSM_ERR_IO, "cannot write " + temp);
    bool ok = fwrite(file.bytes.data(), 1, file.bytes.size(), fp) == file.bytes.size();
    static const uint8_t zeros[32] = {0};
    for (size_t i = 0; ok && i < tensors.size(); i++) {
        const SavedTensor& t = tensors[i];
        ok = fwrite(t.bytes.data(), 1, t.bytes.size(), fp) == t.bytes.size();
        size_t pad = (size_t)((alignment - (int64_t)t.bytes.size() % alignment) % alignment);
        if (ok && pad) ok = fwrite(zeros, 1, pad, fp) == pad;
    }
    ok = (fclose(fp) == 0) && ok;
    if (!ok || rename(temp.c_str(), path) != 0) {
        remove(temp.c_str());
        return fail(ctx, TSM_ERR_IO, std::string("cannot write ") + path);
    }
    return TSM_OK;
}

int tsm_model_config_get(tsm_model* model, tsm_model_config* out) {
    if (!model || !out) return TSM_ERR_ARG;
    *out = model->cfg;
    return TSM_OK;
}

int tsm_model_tensor(tsm_model* model, const char* name, tsm_dptr* ptr, int* kind, int* n, int* k) {
    if (!model || !name) return TSM_ERR_ARG;
    auto found = model->named.find(name);
    if (found == model->named.end()) return fail(model->ctx, TSM_ERR_ARG, std::string("the model has no parameter ") + name);
    if (ptr) *ptr = (tsm_dptr)(uintptr_t)found->second.ptr;
    if (kind) *kind = found->second.kind;
    if (n) *n = found->second.n;
    if (k) *k = found->second.k;
    return TSM_OK;
}

int tsm_cache_create(tsm_model* model, int rows, int capacity, tsm_cache** out) {
    MODEL_GUARD(model);
    if (!out) return TSM_ERR_ARG;
    *out = nullptr;
    if (rows < 1 || capacity < 1) return fail(model->ctx, TSM_ERR_ARG, "a cache needs rows and positions");
    const tsm_model_config& c = model->cfg;
    std::unique_ptr<tsm_cache> cache(new tsm_cache());
    cache->model = model, cache->rows = rows, cache->capacity = capacity;
    cache->lengths.assign(rows, 0);
    int64_t bytes = (int64_t)rows * (c.kv_heads / model->tp) * capacity * c.head_width * 4;  // a rank holds its own kv heads
    for (int i = 0; i < c.layers; i++) {
        void *kp = nullptr, *vp = nullptr;
        int rc = pool_alloc(model->ctx, bytes, &kp);
        if (rc == TSM_OK) cache->keys.push_back((float*)kp), rc = pool_alloc(model->ctx, bytes, &vp);
        if (rc == TSM_OK) cache->values.push_back((float*)vp);
        if (rc != TSM_OK) {
            tsm_cache_free(cache.release());
            return rc;
        }
    }
    *out = cache.release();
    return TSM_OK;
}

int tsm_cache_free(tsm_cache* cache) {
    if (!cache) return TSM_OK;
    MODEL_GUARD(cache->model);
    cudaStreamSynchronize(cache->model->ctx->stream);
    drop_graph(cache);
    drop_run_graph(cache);
    pool_release(cache->model->ctx, cache->run_state);
    for (float* p : cache->keys) pool_release(cache->model->ctx, p);
    for (float* p : cache->values) pool_release(cache->model->ctx, p);
    delete cache;
    return TSM_OK;
}

int tsm_cache_length(tsm_cache* cache, int row, int* length) {
    if (!cache || !length || row < 0 || row >= cache->rows) return TSM_ERR_ARG;
    *length = cache->lengths[row];
    return TSM_OK;
}

int tsm_cache_reset(tsm_cache* cache, int row) {
    if (!cache || row < 0 || row >= cache->rows) return TSM_ERR_ARG;
    cache->lengths[row] = 0;
    return TSM_OK;
}

int tsm_cache_layer(tsm_cache* cache, int layer, tsm_dptr* keys, tsm_dptr* values) {
    if (!cache || layer < 0 || layer >= (int)cache->keys.size()) return TSM_ERR_ARG;
    if (keys) *keys = (tsm_dptr)(uintptr_t)cache->keys[layer];
    if (values) *values = (tsm_dptr)(uintptr_t)cache->values[layer];
    return TSM_OK;
}

int tsm_cache_fill(tsm_cache* cache, int row, int length, uint64_t seed) {
    if (!cache) return TSM_ERR_ARG;
    MODEL_GUARD(cache->model);
    tsm_model* m = cache->model;
    if (row < 0 || row >= cache->rows || length < 0 || length > cache->capacity || length > m->cfg.context)
        return fail(m->ctx, TSM_ERR_ARG, std::to_string(length) + " positions exceed the " + std::to_string(cache->capacity) + " a row holds");
    const tsm_model_config& c = m->cfg;
    const int kv_local = c.kv_heads / m->tp;
    for (int i = 0; i < c.layers; i++)
        for (int local = 0; local < kv_local; local++) {
            int kh = m->tp_rank * kv_local + local;  // seeded by the head's place in the whole model: a shard's rows are the whole cache's
            int64_t at = ((int64_t)row * kv_local + local) * cache->capacity * c.head_width;
            uint64_t s = seed * 7919ull + (uint64_t)((i * c.kv_heads + kh) * 2 + 1) * 1000003ull + (uint64_t)row;
            TSM_TRY(launch_normal_fill(m->ctx, cache->keys[i] + at, (int64_t)length * c.head_width, 0.0f, 1.0f, s));
            TSM_TRY(launch_normal_fill(m->ctx, cache->values[i] + at, (int64_t)length * c.head_width, 0.0f, 1.0f, s + 1));
        }
    cache->lengths[row] = length;
    return TSM_OK;
}

// Generative#packed (generative.cr:112-125) with optional greedy picks of each output row.
static int forward_impl(tsm_model* model, tsm_cache* cache, const int32_t* counts, const int32_t* ids, int last, float* logits,
                        int32_t* picks) {
    if (!cache || cache->model != model || !counts || !ids || (!logits && !picks)) return fail(model->ctx, TSM_ERR_ARG, "forward needs a cache of this model, counts, ids and a place for logits");
    tsm_ctx* ctx = model->ctx;
    const tsm_model_config& c = model->cfg;
    int total = 0, active = 0;
    int limit = cache->capacity < c.context ? cache->capacity : c.context;
    for (int row = 0; row < cache->rows; row++) {
        if (counts[row] < 0) return fail(ctx, TSM_ERR_ARG, "a negative token count");
        if (counts[row] == 0) continue;
        if (cache->lengths[row] + counts[row] > limit)
            return fail(ctx, TSM_ERR_ARG, std::to_string(cache->lengths[row] + counts[row]) + " positions exceed the " + std::to_string(limit) + " a row holds");
        total += counts[row];
        active++;
    }
    if (total == 0) return fail(ctx, TSM_ERR_ARG, "forward of no tokens");
    TSM_TRY(prepare_scratch(model, cache, total));
    Workspace& w = model->ws;
    int32_t* h_ids = w.host;
    int32_t* h_table = w.host + w.tokens;
    int32_t* h_last = w.host + 4 * (int64_t)w.tokens;
    int t = 0, outputs = 0;
    for (int row = 0; row < cache->rows; row++) {
        int past = cache->lengths[row];
        for (int j = 0; j < counts[row]; j++, t++) {
            h_ids[t] = ids[t];
            h_table[3 * t] = row, h_table[3 * t + 1] = past + j, h_table[3 * t + 2] = past + counts[row];
            if (!last || j == counts[row] - 1) h_last[outputs++] = t;
        }
    }
    TSM_CUDA(ctx, cudaMemcpyAsync(w.ids, h_ids, (size_t)total * 4, cudaMemcpyHostToDevice, ctx->stream));
    TSM_CUDA(ctx, cudaMemcpyAsync(w.table, h_table, (size_t)total * 12, cudaMemcpyHostToDevice, ctx->stream));
    TSM_CUDA(ctx, cudaMemcpyAsync(w.last, h_last, (size_t)outputs * 4, cudaMemcpyHostToDevice, ctx->stream));
    ctx->counters.uploads += 3;
    ctx->counters.upload_bytes += (int64_t)total * 16 + (int64_t)outputs * 4;
    TSM_TRY(launch_step(model, cache, total, outputs, picks != nullptr));
    if (logits && picks && model->tp > 1) TSM_TRY(gather_full_logits(model, outputs));
    if (logits) {
        TSM_CUDA(ctx, cudaMemcpyAsync(logits, w.logits, (size_t)outputs * c.vocab * 4, cudaMemcpyDeviceToHost, ctx->stream));
        ctx->counters.downloads++;
        ctx->counters.download_bytes += (int64_t)outputs * c.vocab * 4;
    }
    if (picks) {
        TSM_CUDA(ctx, cudaMemcpyAsync(picks, w.picks, (size_t)outputs * 4, cudaMemcpyDeviceToHost, ctx->stream));
        ctx->counters.downloads++;
        ctx->counters.download_bytes += (int64_t)outputs * 4;
    }
    TSM_TRY(tsm_sync(ctx));
    for (int row = 0; row < cache->rows; row++) cache->lengths[row] += counts[row];
    return TSM_OK;
}

int tsm_forward(tsm_model* model, tsm_cache* cache, const int32_t* counts, const int32_t* ids, int last, float* logits) {
    MODEL_GUARD(model);
    if (!logits) return fail(model->ctx, TSM_ERR_ARG, "forward needs a place for logits");
    return forward_impl(model, cache, counts, ids, last, logits, nullptr);
}

int tsm_decode(tsm_model* model, tsm_cache* cache, const int32_t* ids, int32_t* tokens, float* logits) {
    MODEL_GUARD(model);
    if (!cache || cache->model != model || !ids || !tokens) return fail(model->ctx, TSM_ERR_ARG, "decode needs a cache of this model, ids and a place for tokens");
    tsm_ctx* ctx = model->ctx;
    const tsm_model_config& c = model->cfg;
    int rows = cache->rows;
    int limit = cache->capacity < c.context ? cache->capacity : c.context;
    for (int row = 0; row < rows; row++)
        if (cache->lengths[row] + 1 > limit)
            return fail(ctx, TSM_ERR_ARG, std::to_string(cache->lengths[row] + 1) + " positions exceed the " + std::to_string(limit) + " a row holds");
    TSM_TRY(prepare_scratch(model, cache, rows));
    // a captured step holds the addresses of the workspace and of the scratch memory, and the mode's kernels
    uint64_t stamp = model->ws_generation * 1000003ull + ctx->scratch_generation * 10ull + (uint64_t)ctx->mode;
    if (cache->graph && cache->graph_stamp != stamp) drop_graph(cache);
    cache->graph_stamp = stamp;
    Workspace& w = model->ws;
    int32_t* h_ids = w.host;
    int32_t* h_table = w.host + w.tokens;
    int32_t* h_picks = w.host + 4 * (int64_t)w.tokens;
    for (int row = 0; row < rows; row++) {
        h_ids[row] = ids[row];
        h_table[3 * row] = row, h_table[3 * row + 1] = cache->lengths[row], h_table[3 * row + 2] = cache->lengths[row] + 1;
    }
    if (!cache->graph) {
        // the step reads ids and positions from device memory, so one capture serves every later step
        cudaGraph_t graph = nullptr;
        TSM_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        int rc = TSM_OK;
        cudaError_t e1 = cudaMemcpyAsync(w.ids, h_ids, (size_t)rows * 4, cudaMemcpyHostToDevice, ctx->stream);
        cudaError_t e2 = cudaMemcpyAsync(w.table, h_table, (size_t)rows * 12, cudaMemcpyHostToDevice, ctx->stream);
        if (e1 != cudaSuccess || e2 != cudaSuccess) rc = cuda_fail(ctx, e1 != cudaSuccess ? e1 : e2, "cudaMemcpyAsync");
        if (rc == TSM_OK) rc = launch_step(model, cache, rows, rows, true);
        cudaError_t e3 = cudaMemcpyAsync(h_picks, w.picks, (size_t)rows * 4, cudaMemcpyDeviceToHost, ctx->stream);
        if (e3 == cudaSuccess) e3 = cudaMemcpyAsync(ctx->errors_host, ctx->errors, sizeof(ErrorRecord), cudaMemcpyDeviceToHost, ctx->stream);
        cudaError_t e4 = cudaStreamEndCapture(ctx->stream, &graph);
        if (rc == TSM_OK && (e3 != cudaSuccess || e4 != cudaSuccess)) rc = cuda_fail(ctx, e3 != cudaSuccess ? e3 : e4, "capture of a decode step");
        if (rc == TSM_OK) {
            cudaError_t e5 = cudaGraphInstantiate(&cache->graph, graph, 0);
            if (e5 != cudaSuccess) rc = cuda_fail(ctx, e5, "cudaGraphInstantiate");
            cache->graph_kernels = kernel_nodes(graph);
            ctx->counters.launches -= cache->graph_kernels;  // captured, not launched; replays count below
        }
        if (graph) cudaGraphDestroy(graph);
        if (rc != TSM_OK) {
            cudaGetLastError();
            return rc;
        }
    }
    TSM_CUDA(ctx, cudaGraphLaunch(cache->graph, ctx->stream));
    ctx->counters.graph_replays++;
    ctx->counters.launches += cache->graph_kernels;
    ctx->counters.uploads += 2, ctx->counters.upload_bytes += (int64_t)rows * 16;
    ctx->counters.downloads += 1, ctx->counters.download_bytes += (int64_t)rows * 4;
    if (logits) {
        if (model->tp > 1) TSM_TRY(gather_full_logits(model, rows));
        TSM_CUDA(ctx, cudaMemcpyAsync(logits, w.logits, (size_t)rows * c.vocab * 4, cudaMemcpyDeviceToHost, ctx->stream));
        ctx->counters.downloads++, ctx->counters.download_bytes += (int64_t)rows * c.vocab * 4;
    }
    TSM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    TSM_TRY(check_error_record(ctx));  // the replayed step copied the record to the host
    for (int row = 0; row < rows; row++) {
        tokens[row] = h_picks[row];
        cache->lengths[row] += 1;
    }
    return TSM_OK;
}

int tsm_decode_run(tsm_model* model, tsm_cache* cache, const int32_t* ids, int steps, int32_t* tokens) {
    MODEL_GUARD(model);
    if (!cache || cache->model != model || !ids || !tokens || steps < 1) return fail(model->ctx, TSM_ERR_ARG, "a run needs a cache of this model, ids, steps and a place for tokens");
    tsm_ctx* ctx = model->ctx;
    const tsm_model_config& c = model->cfg;
    int rows = cache->rows;
    if (rows > 1024) return fail(ctx, TSM_ERR_UNSUPPORTED, "a device-resident run takes at most 1024 rows");
    int limit = cache->capacity < c.context ? cache->capacity : c.context;
    for (int row = 0; row < rows; row++)
        if (cache->lengths[row] + steps > limit)
            return fail(ctx, TSM_ERR_ARG, std::to_string(cache->lengths[row] + steps) + " positions exceed the " + std::to_string(limit) + " a row holds");
    TSM_TRY(prepare_scratch(model, cache, rows));
    // room for at least 1024 steps: the captured step holds this buffer's address, so growing it means capturing again
    int64_t need = 1 + (int64_t)std::max(steps, 1024) * rows;
    if (cache->run_capacity < need) {
        TSM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        pool_release(ctx, cache->run_state);
        cache->run_state = nullptr, cache->run_capacity = 0;
        drop_run_graph(cache);
        TSM_TRY(pool_alloc(ctx, need * 4, (void**)&cache->run_state));
        cache->run_capacity = need;
    }
    uint64_t stamp = model->ws_generation * 1000003ull + ctx->scratch_generation * 10ull + (uint64_t)ctx->mode;
    if (cache->run_graph && cache->run_stamp != stamp) drop_run_graph(cache);
    cache->run_stamp = stamp;
    Workspace& w = model->ws;
    int32_t* h_ids = w.host;
    int32_t* h_table = w.host + w.tokens;
    for (int row = 0; row < rows; row++) {
        h_ids[row] = ids[row];
        h_table[3 * row] = row, h_table[3 * row + 1] = cache->lengths[row], h_table[3 * row + 2] = cache->lengths[row] + 1;
    }
    TSM_CUDA(ctx, cudaMemcpyAsync(w.ids, h_ids, (size_t)rows * 4, cudaMemcpyHostToDevice, ctx->stream));
    TSM_CUDA(ctx, cudaMemcpyAsync(w.table, h_table, (size_t)rows * 12, cudaMemcpyHostToDevice, ctx->stream));
    TSM_CUDA(ctx, cudaMemsetAsync(cache->run_state, 0, 4, ctx->stream));
    ctx->counters.uploads += 2, ctx->counters.upload_bytes += (int64_t)rows * 16;
    if (!cache->run_graph) {
        cudaGraph_t graph = nullptr;
        TSM_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        cudaError_t e0 = launch_chained(ctx, run_advance_kernel, dim3((rows + 255) / 256), dim3(256), 0, w.ids, w.table, w.picks, rows, cache->run_state);
        count_launch(ctx);
        int rc = launch_step(model, cache, rows, rows, true);
        if (e0 == cudaSuccess) e0 = launch_chained(ctx, run_record_kernel, dim3(1), dim3(1024), 0, w.picks, rows, cache->run_state);
        count_launch(ctx);
        cudaError_t e1 = e0 != cudaSuccess ? e0 : cudaGetLastError();
        cudaError_t e2 = cudaStreamEndCapture(ctx->stream, &graph);
        if (rc == TSM_OK && (e1 != cudaSuccess || e2 != cudaSuccess)) rc = cuda_fail(ctx, e1 != cudaSuccess ? e1 : e2, "capture of a decode step");
        if (rc == TSM_OK) {
            cudaError_t e3 = cudaGraphInstantiate(&cache->run_graph, graph, 0);
            if (e3 != cudaSuccess) rc = cuda_fail(ctx, e3, "cudaGraphInstantiate");
            cache->run_kernels = kernel_nodes(graph);
            ctx->counters.launches -= cache->run_kernels;
        }
        if (graph) cudaGraphDestroy(graph);
        if (rc != TSM_OK) {
            cudaGetLastError();
            return rc;
        }
    }
    for (int s = 0; s < steps; s++) {
        TSM_CUDA(ctx, cudaGraphLaunch(cache->run_graph, ctx->stream));
        // Measured with 2 to 8 ranks: replays holding NCCL all-gathers queued back to back ran at half the rate of replays
        // the host waits for one by one, so a tensor-parallel run pays one stream wait per step.
        if (model->tp > 1 && !getenv("TSM_TP_RUN_QUEUED")) TSM_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    ctx->counters.graph_replays += steps;
    ctx->counters.launches += (int64_t)steps * cache->run_kernels;
    TSM_CUDA(ctx, cudaMemcpyAsync(tokens, cache->run_state + 1, (size_t)steps * rows * 4, cudaMemcpyDeviceToHost, ctx->stream));
    ctx->counters.downloads++, ctx->counters.download_bytes += (int64_t)steps * rows * 4;
    TSM_TRY(tsm_sync(ctx));
    for (int row = 0; row < rows; row++) cache->lengths[row] += steps;
    return TSM_OK;
}

int tsm_generate(tsm_model* model, const int32_t* prompt, int prompt_size, int count, int32_t* tokens) {
    MODEL_GUARD(model);
    if (!prompt || prompt_size < 1 || count < 0 || (count > 0 && !tokens)) return fail(model->ctx, TSM_ERR_ARG, "generate needs a prompt and a place for tokens");
    const tsm_model_config& c = model->cfg;
    if (count == 0) return TSM_OK;
    int capacity = prompt_size + count < c.context ? prompt_size + count : c.context;
    tsm_cache* cache = nullptr;
    TSM_TRY(tsm_cache_create(model, 1, capacity, &cache));
    int32_t counts[1] = {prompt_size};
    // Sampler.greedy picks on the device: the first index of the maximum (sampler.cr:36)
    int rc = forward_impl(model, cache, counts, prompt, 1, nullptr, &tokens[0]);
    if (rc == TSM_OK && count > 1) rc = tsm_decode_run(model, cache, &tokens[0], count - 1, &tokens[1]);
    tsm_cache_free(cache);
    return rc;
}

}  // extern "C"
