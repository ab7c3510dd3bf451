// GGUF files: the reader (gguf.cr:297-381) with the Llama and GPT-2 name maps (llama.cr:57-101, 184-235; gpt2.cr:75-89),
// and the writer behind Module#save (module.cr:148-164; GGUF.write, gguf.cr:156-191).
#include <fcntl.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <thread>

#include "model.cuh"

namespace tsm {

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
    if (!path) return fail(ctx, TSM_ERR_ARG, "no path");
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
        for (uint32_t d = 0; d < nd; d++) {
            uint64_t extent = f.read<uint64_t>();
            if (extent == 0 || extent > (uint64_t)1 << 40) f.bad = true;  // no axis of a weight is empty or anywhere near 2^40 long
            dims[d] = (int64_t)extent;
        }
        info.shape.assign(dims.rbegin(), dims.rend());
        info.kind = f.read<uint32_t>();
        uint64_t offset = f.read<uint64_t>();
        if (offset > (uint64_t)f.size) f.bad = true;  // also what a negative offset looks like once it is unsigned
        info.offset = (int64_t)offset;
        infos.push_back(info);
    }
    if (f.bad) return fail(ctx, TSM_ERR_IO, std::string(path) + " is malformed");
    int64_t alignment = f.numbers.count("general.alignment") ? (int64_t)f.numbers["general.alignment"] : 32;
    if (alignment < 1) alignment = 32;
    int64_t start = (f.pos + alignment - 1) / alignment * alignment;
    for (auto& info : infos) {
        int64_t count = 1;
        for (int64_t d : info.shape) {
            if (count > ((int64_t)1 << 46) / d) return fail(ctx, TSM_ERR_IO, info.name + ": more values than any file holds");
            count *= d;
        }
        int64_t bytes = gguf_bytes(info.kind, count);
        if (bytes < 0) return fail(ctx, TSM_ERR_UNSUPPORTED, info.name + ": GGUF tensor type " + std::to_string(info.kind) + " is not supported yet");
        if ((info.kind == 2 || info.kind == 3 || info.kind == 8) && (info.shape.empty() || info.shape.back() % 32 != 0))
            return fail(ctx, TSM_ERR_IO, info.name + ": rows of " + std::to_string(info.shape.empty() ? 0 : info.shape.back()) + " do not split into blocks of 32");
        if (info.offset < 0 || info.offset % alignment != 0 || bytes > f.size || start + info.offset > f.size - bytes)
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

// Weights travel from the mapped file to the device through two pinned buffers: while one is being copied to the device
// (cudaMemcpyAsync on the context's stream), the host fills the other from the file, on a few threads.  The reference's
// loader hands each tensor to Device#upload as one pageable block (gguf.cr:112-136, cuda.cr:389-391); for files of
// several gigabytes the pageable copy and the wait after every tensor were most of the load time.
struct Stager {
    static constexpr size_t kBytes = 48u << 20;
    tsm_ctx* ctx = nullptr;
    uint8_t* buffer[2] = {nullptr, nullptr};
    cudaEvent_t sent[2] = {nullptr, nullptr};
    bool busy[2] = {false, false};
    int turn = 0;
    int64_t bytes_sent = 0;
    int begin(tsm_ctx* c) {
        ctx = c;
        for (int i = 0; i < 2; i++) {
            TSM_CUDA(ctx, cudaMallocHost((void**)&buffer[i], kBytes));
            TSM_CUDA(ctx, cudaEventCreateWithFlags(&sent[i], cudaEventDisableTiming));
        }
        return TSM_OK;
    }
    // a pinned buffer that no copy is reading any more
    int acquire(uint8_t** out) {
        if (busy[turn]) {
            TSM_CUDA(ctx, cudaEventSynchronize(sent[turn]));
            busy[turn] = false;
        }
        *out = buffer[turn];
        return TSM_OK;
    }
    int send(void* dst, size_t bytes) {
        TSM_CUDA(ctx, cudaMemcpyAsync(dst, buffer[turn], bytes, cudaMemcpyHostToDevice, ctx->stream));
        TSM_CUDA(ctx, cudaEventRecord(sent[turn], ctx->stream));
        busy[turn] = true, turn ^= 1, bytes_sent += (int64_t)bytes;
        ctx->counters.uploads++, ctx->counters.upload_bytes += (int64_t)bytes;
        return TSM_OK;
    }
    ~Stager() {
        if (!ctx) return;
        cudaStreamSynchronize(ctx->stream);
        for (int i = 0; i < 2; i++) {
            if (sent[i]) cudaEventDestroy(sent[i]);
            if (buffer[i]) cudaFreeHost(buffer[i]);
        }
    }
};

// Copies rows[first .. first + count) (row_bytes each) into dst back to back, on up to four threads.
static void gather_rows(uint8_t* dst, const std::vector<const uint8_t*>& rows, int64_t first, int64_t count, int64_t row_bytes) {
    const int workers = (int)std::min<int64_t>(4, std::max<int64_t>(1, count * row_bytes >> 22));
    auto part = [&](int w) {
        int64_t a = first + count * w / workers, b = first + count * (w + 1) / workers;
        for (int64_t r = a; r < b; r++) memcpy(dst + (r - first) * row_bytes, rows[(size_t)r], (size_t)row_bytes);
    };
    if (workers == 1) return part(0);
    std::vector<std::thread> pool;
    for (int w = 1; w < workers; w++) pool.emplace_back(part, w);
    part(0);
    for (auto& t : pool) t.join();
}

struct RowSource {
    std::string name;
    int heads;  // > 0: undo llama.cpp's rotary row order for this many heads (llama.cr:226-235)
    // A Linear under tensomite's own names: while it is unquantised the file holds it as the module does, [inputs, outputs]
    // (modules.cr:1-20; Module#load reverses the shape for block formats only, module.cr:217-228), so it is transposed on
    // the way in; a block format is [outputs, inputs] already.
    bool linear_of_module = false;
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
        const bool flip = part.linear_of_module && (e.kind == 0 || e.kind == 1 || e.kind == 30);
        if (e.shape.size() != 2 || e.shape[flip ? 0 : 1] != k)
            return fail(m->ctx, TSM_ERR_ARG, part.name + ": the file's shape does not match the model's " +
                                                 (flip ? "[" + std::to_string(k) + ", " + std::to_string(expect_n) + "]" : "[" + std::to_string(expect_n) + ", " + std::to_string(k) + "]"));
        int this_kind = gguf_kind_to_tsm(e.kind);
        if (kind != -2 && kind != this_kind) return fail(m->ctx, TSM_ERR_UNSUPPORTED, "joined projections must share a format");
        kind = this_kind;
        total_rows += e.shape[flip ? 1 : 0];
    }
    if (total_rows != expect_n) return fail(m->ctx, TSM_ERR_ARG, parts[0].name + ": the file holds " + std::to_string(total_rows) + " rows, the model " + std::to_string(expect_n));
    int64_t row_bytes = weight_bytes(kind, 1, k);
    // Rows that are in the file as the device wants them (block formats, F32): streamed through the pinned buffers, row
    // order (joined parts, rotary order undone, a rank's share) applied while the buffer is filled.
    bool as_stored = m->stager != nullptr;
    for (auto& part : parts) {
        const GgufEntry& e = f.entries[part.name];
        if (e.kind == 1 || e.kind == 30 || (part.linear_of_module && e.kind == 0)) as_stored = false;
    }
    if (as_stored) {
        std::vector<const uint8_t*> rows;
        rows.reserve((size_t)total_rows);
        for (auto& part : parts) {
            const GgufEntry& e = f.entries[part.name];
            const uint8_t* src = f.data + e.offset;
            int64_t count = e.shape[0];
            if (part.heads > 0) {
                int64_t half = count / part.heads / 2;
                for (int head = 0; head < part.heads; head++)
                    for (int pair = 0; pair < 2; pair++)
                        for (int64_t i = 0; i < half; i++) rows.push_back(src + (head * 2 * half + 2 * i + pair) * row_bytes);
            } else {
                for (int64_t r = 0; r < count; r++) rows.push_back(src + r * row_bytes);
            }
        }
        if (!ranges.empty()) {  // a tensor-parallel rank keeps its rows only
            std::vector<const uint8_t*> kept;
            for (auto& range : ranges) kept.insert(kept.end(), rows.begin() + range.start, rows.begin() + range.start + range.count);
            rows.swap(kept);
        }
        const int64_t held = (int64_t)rows.size();
        out->kind = kind, out->n = (int)held, out->k = k;
        TSM_TRY(dev_alloc(m, held * row_bytes, (void**)&out->w));
        const int64_t per_chunk = std::max<int64_t>(1, (int64_t)Stager::kBytes / row_bytes);
        for (int64_t first = 0; first < held; first += per_chunk) {
            int64_t count = std::min(per_chunk, held - first);
            uint8_t* pinned = nullptr;
            TSM_TRY(m->stager->acquire(&pinned));
            gather_rows(pinned, rows, first, count, row_bytes);
            TSM_TRY(m->stager->send(out->w + first * row_bytes, (size_t)(count * row_bytes)));
        }
        return TSM_OK;
    }
    std::vector<uint8_t> staging((size_t)(total_rows * row_bytes));
    int64_t at = 0;
    for (auto& part : parts) {
        const GgufEntry& e = f.entries[part.name];
        const uint8_t* src = f.data + e.offset;
        const bool flip = part.linear_of_module && (e.kind == 0 || e.kind == 1 || e.kind == 30);
        int64_t rows = e.shape[flip ? 1 : 0];
        std::vector<float> wide, turned;
        if (e.kind == 1 || e.kind == 30) {  // F16 / BF16 matrices become F32 weights
            wide.resize((size_t)(rows * k));
            widen_halves((const uint16_t*)src, rows * k, e.kind == 30, wide.data());
            src = (const uint8_t*)wide.data();
        }
        if (flip) {  // [k, rows] in the file -> the rows the products read
            const float* from = (const float*)src;
            turned.resize((size_t)(rows * k));
            for (int64_t i = 0; i < (int64_t)k; i++)
                for (int64_t r = 0; r < rows; r++) turned[(size_t)(r * k + i)] = from[i * rows + r];
            src = (const uint8_t*)turned.data();
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
    if (f.entries["token_embd.weight"].shape.size() != 2) return fail(m->ctx, TSM_ERR_IO, "token_embd.weight is not a matrix");
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
    if (f.entries["wte.weight"].shape.size() != 2 || f.entries["wpe.weight"].shape.size() != 2)
        return fail(m->ctx, TSM_ERR_IO, "wte.weight and wpe.weight must be matrices");
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
        TSM_TRY(upload_rows(m, f, {{p + "attn.c_attn.weight", 0, true}}, c.width, 3 * c.width, &l.qkv, shard_ranges(m, SHARD_QKV)));
        TSM_TRY(upload_bias(m, f, p + "attn.c_attn.bias", 3 * c.width, &l.qkv.bias));
        TSM_TRY(shard_bias(m, &l.qkv.bias, shard_ranges(m, SHARD_QKV)));
        TSM_TRY(upload_rows(m, f, {{p + "attn.c_proj.weight", 0, true}}, c.width, c.width, &l.o, shard_ranges(m, SHARD_WIDTH)));
        TSM_TRY(upload_bias(m, f, p + "attn.c_proj.bias", c.width, &l.o.bias));
        TSM_TRY(shard_bias(m, &l.o.bias, shard_ranges(m, SHARD_WIDTH)));
        TSM_TRY(upload_rows(m, f, {{p + "mlp.c_fc.weight", 0, true}}, c.width, c.hidden, &l.up, shard_ranges(m, SHARD_UP)));
        TSM_TRY(upload_bias(m, f, p + "mlp.c_fc.bias", c.hidden, &l.up.bias));
        TSM_TRY(shard_bias(m, &l.up.bias, shard_ranges(m, SHARD_UP)));
        TSM_TRY(upload_rows(m, f, {{p + "mlp.c_proj.weight", 0, true}}, c.hidden, c.width, &l.down, shard_ranges(m, SHARD_WIDTH)));
        TSM_TRY(upload_bias(m, f, p + "mlp.c_proj.bias", c.width, &l.down.bias));
        TSM_TRY(shard_bias(m, &l.down.bias, shard_ranges(m, SHARD_WIDTH)));
        TSM_TRY(shard_inputs(m, l));
    }
    return TSM_OK;
}

// Reads a file's header and tensor table the way the loaders do, without a device: TSM_OK, or TSM_ERR_IO / _UNSUPPORTED with
// the reason in `why`.
int check_gguf_file(const char* path, std::string* why) {
    tsm_ctx scratch;  // only its message slot is used
    GgufFile f;
    int rc = gguf_open(&scratch, path, f);
    if (rc == TSM_OK) {
        std::string arch = f.strings.count("general.architecture") ? f.strings["general.architecture"] : "";
        if (arch == "llama") {
            if (!f.entries.count("token_embd.weight") || f.entries["token_embd.weight"].shape.size() != 2)
                rc = fail(&scratch, TSM_ERR_IO, "token_embd.weight is missing or not a matrix");
        } else if (f.strings.count("gpt2.heads")) {
            for (const char* name : {"wte.weight", "wpe.weight"})
                if (!f.entries.count(name) || f.entries[name].shape.size() != 2) rc = fail(&scratch, TSM_ERR_IO, std::string(name) + " is missing or not a matrix");
        }
    }
    if (why) *why = scratch.message;
    return rc;
}

// Llama.load / GPT2.load of a .gguf file: the family is read from the metadata.
int load_gguf_model(tsm_model* m, const char* path) {
    GgufFile f;
    TSM_TRY(gguf_open(m->ctx, path, f));
    std::string arch = f.strings.count("general.architecture") ? f.strings["general.architecture"] : "";
    Stager stager;   // two pinned buffers for the length of the load; the destructor waits for the last copy
    static const bool pageable = getenv("TSM_LOAD_PAGEABLE") != nullptr;   // the one-block-per-tensor path, for timing it
    if (!pageable) {
        TSM_TRY(stager.begin(m->ctx));
        m->stager = &stager;
    }
    int rc;
    if (arch == "llama") rc = load_llama(m, f);
    else if (f.strings.count("gpt2.heads")) rc = load_gpt2(m, f);
    else rc = fail(m->ctx, TSM_ERR_IO, std::string(path) + " holds a " + arch + " model, not a Llama or GPT-2");
    m->stager = nullptr;
    if (rc == TSM_OK) rc = tsm_sync(m->ctx);   // every copy has landed before the file is unmapped
    return rc;
}

// ---- Module#save to a .gguf file (module.cr:148-164; GGUF.write, gguf.cr:156-191) ---------------------------------
//
// Writes the model as it is held on the device: block formats keep their bytes, F32 stays F32.  A Llama goes out under
// llama.cpp's names with its llama.* metadata and with q and k rows back in llama.cpp's rotary order (the inverse of what
// the loader undoes, llama.cr:226-235), the joined projections cut back into their parts; a GPT-2 under tensomite's own
// names with gpt2.heads.  Either file loads again here and in the reference.

// One tensor of the file to be written: where its bytes are on the device.  The bytes are fetched when the tensor's turn
// to be written comes, so the host never holds more than the largest tensor.
struct SavedTensor {
    std::string name;
    uint32_t kind;               // GGUF's type number
    std::vector<int64_t> shape;  // outermost first
    const uint8_t* source;       // device address
    int64_t size;                // bytes
    int64_t row_bytes;
    int heads;                   // > 0: rows go back into llama.cpp's rotary order for this many heads
    bool turned = false;         // an unquantised Linear under tensomite's names goes out [inputs, outputs]
};

static uint32_t gguf_kind_of(int kind) { return kind == TSM_Q8_0 ? 8 : kind == TSM_Q4_0 ? 2 : kind == TSM_Q4_1 ? 3 : 0; }

// Rows [first, first + rows) of a weight; heads > 0 puts them back into llama.cpp's rotary order.
static int saved_rows(tsm_model* m, const Linear& l, const std::string& name, int64_t first, int64_t rows, int heads, std::vector<SavedTensor>& out) {
    (void)m;
    int64_t row_bytes = weight_bytes(l.kind, 1, l.k);
    out.push_back(SavedTensor{name, gguf_kind_of(l.kind), {rows, (int64_t)l.k}, l.w + first * row_bytes, rows * row_bytes, row_bytes, heads});
    return TSM_OK;
}

static int saved_vector(tsm_model* m, const float* values, const std::string& name, int64_t count, std::vector<SavedTensor>& out) {
    (void)m;
    if (values) out.push_back(SavedTensor{name, 0, {count}, (const uint8_t*)values, count * 4, count * 4, 0});
    return TSM_OK;
}

// Downloads a tensor's bytes in the order the file holds them.
static int fetch_saved(tsm_model* m, const SavedTensor& t, std::vector<uint8_t>& bytes) {
    bytes.resize((size_t)t.size);
    TSM_TRY(tsm_download(m->ctx, bytes.data(), (tsm_dptr)(uintptr_t)t.source, t.size));
    if (t.turned) {  // held [n, k], written [k, n]
        const int64_t k = t.shape[0], n = t.shape[1];
        std::vector<uint8_t> file((size_t)t.size);
        const float* held = (const float*)bytes.data();
        float* out = (float*)file.data();
        for (int64_t r = 0; r < n; r++)
            for (int64_t i = 0; i < k; i++) out[i * n + r] = held[r * k + i];
        bytes.swap(file);
    }
    if (t.heads > 0) {
        std::vector<uint8_t> file((size_t)t.size);
        int64_t rows = t.size / t.row_bytes, half = rows / t.heads / 2, held = 0;
        for (int head = 0; head < t.heads; head++)
            for (int pair = 0; pair < 2; pair++)
                for (int64_t i = 0; i < half; i++, held++)
                    memcpy(&file[(size_t)((head * 2 * half + 2 * i + pair) * t.row_bytes)], &bytes[(size_t)(held * t.row_bytes)], (size_t)t.row_bytes);
        bytes.swap(file);
    }
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

int save_gguf_model(tsm_model* m, const char* path) {
    tsm_ctx* ctx = m->ctx;
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
                if (part.first->kind == TSM_F32) {  // as Module#save writes an unquantised Linear: [inputs, outputs]
                    tensors.back().turned = true;
                    tensors.back().shape = {(int64_t)part.first->k, (int64_t)part.first->n};
                }
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
    for (auto& t : tensors) {
        file.str(t.name);
        file.put<uint32_t>((uint32_t)t.shape.size());
        for (auto d = t.shape.rbegin(); d != t.shape.rend(); ++d) file.put<uint64_t>((uint64_t)*d);  // innermost first
        file.put<uint32_t>(t.kind);
        file.put<uint64_t>((uint64_t)offset);
        offset = (offset + t.size + alignment - 1) / alignment * alignment;
    }
    file.bytes.resize((file.bytes.size() + alignment - 1) / alignment * alignment, 0);
    // a temporary beside the target, renamed when whole, as GGUF.write does (gguf.cr:165-190)
    std::string temp = std::string(path) + "." + std::to_string((long)getpid()) + ".tmp";
    FILE* fp = fopen(temp.c_str(), "wb");
    if (!fp) return fail(ctx, TSM_ERR_IO, "cannot write " + temp);
    bool ok = fwrite(file.bytes.data(), 1, file.bytes.size(), fp) == file.bytes.size();
    static const uint8_t zeros[32] = {0};
    std::vector<uint8_t> bytes;
    int fetched = TSM_OK;
    for (size_t i = 0; ok && i < tensors.size(); i++) {
        const SavedTensor& t = tensors[i];
        if ((fetched = fetch_saved(m, t, bytes)) != TSM_OK) break;
        ok = fwrite(bytes.data(), 1, bytes.size(), fp) == bytes.size();
        size_t pad = (size_t)((alignment - t.size % alignment) % alignment);
        if (ok && pad) ok = fwrite(zeros, 1, pad, fp) == pad;
    }
    ok = (fclose(fp) == 0) && ok;
    if (fetched != TSM_OK) {
        remove(temp.c_str());
        return fetched;
    }
    if (!ok || rename(temp.c_str(), path) != 0) {
        remove(temp.c_str());
        return fail(ctx, TSM_ERR_IO, std::string("cannot write ") + path);
    }
    return TSM_OK;
}

}  // namespace tsm
