// Hugging Face safetensors files (safetensors.cr; GPT2.new(SafeTensors), gpt2.cr:93-101; Llama.load of a model directory,
// llama.cr:163-175), quantised on the device as they load.
#include <fcntl.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include "model.cuh"

namespace tsm {

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
    if (f.entries[p + "wte.weight"].shape.size() != 2 || f.entries[p + "wpe.weight"].shape.size() != 2)
        return fail(m->ctx, TSM_ERR_IO, "wte.weight and wpe.weight must be matrices");
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
    if (f.entries["model.embed_tokens.weight"].shape.size() != 2) return fail(m->ctx, TSM_ERR_IO, "model.embed_tokens.weight must be a matrix");
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
    if (!f.entries.count("model.layers.0.mlp.gate_proj.weight") || f.entries["model.layers.0.mlp.gate_proj.weight"].shape.size() != 2)
        return fail(m->ctx, TSM_ERR_IO, "model.layers.0.mlp.gate_proj.weight is missing or not a matrix");
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

// GPT2.load / Llama.load of a safetensors file, then Module#quantize(kind, embeddings: true) unless kind is TSM_F32.
int load_safetensors_model(tsm_model* m, const char* path, const tsm_model_config& config, int kind) {
    StFile f;
    TSM_TRY(st_open(m->ctx, path, f));
    if (config.arch == 1) return load_gpt2_safetensors(m, f, config.heads, kind);
    if (config.arch == 0) return load_llama_safetensors(m, f, config, kind);
    return fail(m->ctx, TSM_ERR_ARG, "unknown architecture");
}

}  // namespace tsm
