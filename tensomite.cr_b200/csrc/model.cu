// A model's resident weights: tensor-parallel sharding, names, rotary tables, configuration checks, and models drawn on
// the device (Llama.new / GPT2.new with Init.normal(0.02), then Module#quantize).
#include <math.h>

#include <algorithm>

#include "model.cuh"

namespace tsm {

// Which rows of a projection a rank of a tensor-parallel group holds.  Every projection is split by OUTPUT rows, so
// each output's sum over blocks stays on one GPU, whole and in block order: the sharded model's bits are the single
// GPU's.  Joined projections keep their parts: a rank takes its heads' rows of q, of k and of v (its slice of gate
// and of up).  An empty list means all rows.
std::vector<RowRange> shard_ranges(const tsm_model* m, int what) {
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

int check_sharding(tsm_model* m) {
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
int shard_inputs(tsm_model* m, Layer& l) {
    if (!m->tp_reduce) return TSM_OK;
    const tsm_model_config& c = m->cfg;
    int64_t G = m->tp, r = m->tp_rank;
    int64_t o_blocks = (int64_t)c.heads * c.head_width / G / 32, down_blocks = (int64_t)c.hidden / G / 32;
    TSM_TRY(keep_block_columns(m, &l.o, r * o_blocks, o_blocks));
    TSM_TRY(keep_block_columns(m, &l.down, r * down_blocks, down_blocks));
    if (r != 0) l.o.bias = nullptr, l.down.bias = nullptr;
    return TSM_OK;
}

int dev_alloc(tsm_model* m, int64_t bytes, void** out) {
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

int64_t weight_bytes(int kind, int64_t n, int64_t k) { return kind == TSM_F32 ? n * k * 4 : n * (k / 32) * block_bytes(kind); }

// cos/sin of every position, in F32 through the host's libm, as RotaryEmbedding computes them
// (modules.cr:343-351): freq_i = 1f / powf(theta_f32, f32(2i) / width).
int make_rope_tables(tsm_model* m) {
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

int check_config(tsm_ctx* ctx, const tsm_model_config& c) {
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

void register_names(tsm_model* m) {
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

// Replaces a full bias vector by the entries of a rank's rows.
int shard_bias(tsm_model* m, float** bias, const std::vector<RowRange>& ranges) {
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
void set_head_local(tsm_model* m) {
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

int build_random(tsm_model* m, int kind, uint64_t seed) {
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

}  // namespace tsm
