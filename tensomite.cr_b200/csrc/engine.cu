// The token loop: one packed forward step over a model's resident weights and the batch cache, its CUDA-graph replay for
// decoding, the device-resident run and the generate loop.  Host-side counterpart of the reference's
// models/{generative,llama,gpt2}.cr and modules.cr; the op order of one step is theirs.
#include <math.h>
#include <string.h>

#include <algorithm>
#include <memory>

#include "model.cuh"

using namespace tsm;

namespace tsm {

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
    void* bufs[] = {w.ids, w.table, w.last, w.order, w.qtiles, w.x, w.xl, w.qkv, w.att, w.up, w.h, w.logits, w.picks, w.qa, w.qb, w.qc, w.tp_parts, w.tp_rows, w.tp_best};
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
    TSM_TRY(pool_alloc(ctx, T * 8, (void**)&w.qtiles));
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
    TSM_CUDA(ctx, cudaMallocHost((void**)&w.host, (size_t)T * 7 * 4));
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

// One layer of a TSM_TP_REDUCE step through the fused exchange (tp_exchange.cu).  On entry the exchange's activation buffer
// holds the layer's first norm of every row, quantised; o and down write their partial products into the exchange region,
// and each exchange kernel sums them over the ranks, adds the residual on the rows this rank owns, norms them with the NEXT
// norm's weights and delivers the quantised rows to every rank.  Eight launches per layer, two of them exchanges.
static int launch_layer_fused(tsm_model* m, tsm_cache* cache, int i, int total, const int* order, float scale) {
    const tsm_model_config& c = m->cfg;
    tsm_ctx* ctx = m->ctx;
    Workspace& w = m->ws;
    Layer& l = m->layers[i];
    const int G = m->tp, hw = c.head_width;
    const int heads_l = c.heads / G, kv_l = c.kv_heads / G, qn_l = heads_l * hw, qkvn_l = qn_l + 2 * kv_l * hw, hid_l = c.hidden / G;
    const bool layer = c.arch == 1;
    QuantizedActs qx = quant_scratch_layout(xchg_quantized(m), total, c.width);
    QuantizedActs qb = quant_scratch_layout(w.qb, total, qn_l);
    QuantizedActs qc = quant_scratch_layout(w.qc, total, hid_l);
    TSM_TRY(product(m, qx, nullptr, total, l.qkv, nullptr, w.qkv));
    TSM_TRY(launch_rope_append(ctx, w.qkv, total, heads_l, kv_l, hw, c.arch == 0 ? m->rope_cos : nullptr, c.arch == 0 ? m->rope_sin : nullptr,
                               c.context, w.table, cache->keys[i], cache->values[i], cache->rows, cache->capacity));
    TSM_TRY(launch_attention(ctx, w.qkv, qkvn_l, total, heads_l, hw, cache->keys[i], cache->values[i], cache->rows, kv_l, cache->capacity,
                             w.table, scale, w.att, &qb, order));
    TSM_TRY(product(m, qb, nullptr, total, l.o, nullptr, xchg_partial(m)));
    TSM_TRY(launch_xchg_reduce_norm(m, total, w.x, nullptr, layer, l.norm2_w, l.norm2_b, c.eps));
    TSM_TRY(product(m, qx, nullptr, total, l.up, nullptr, w.up));
    if (c.arch == 0) TSM_TRY(launch_swiglu(ctx, w.up, w.up + hid_l, total, hid_l, 2 * (int64_t)hid_l, nullptr, &qc));
    else TSM_TRY(launch_gelu(ctx, w.up, total, hid_l, nullptr, &qc));
    TSM_TRY(product(m, qc, nullptr, total, l.down, nullptr, xchg_partial(m)));
    const bool last = i + 1 == c.layers;
    const float* next_w = last ? m->final_w : m->layers[i + 1].norm1_w;
    const float* next_b = last ? m->final_b : m->layers[i + 1].norm1_b;
    return launch_xchg_reduce_norm(m, total, w.x, nullptr, layer, next_w, next_b, c.eps);
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
    // TSM_TP_REDUCE with mapped peer memory, every token an output (a decode step): the fused exchange; the first norm of the
    // first layer is the only one computed on full rows
    const bool fused = m->tp > 1 && m->tp_reduce && outputs == total && xchg_takes(m, total);
    if (fused) {
        QuantizedActs qx = quant_scratch_layout(xchg_quantized(m), total, c.width);
        if (c.arch == 0) TSM_TRY(launch_rmsnorm(ctx, w.x, m->layers[0].norm1_w, total, c.width, c.eps, nullptr, &qx));
        else TSM_TRY(launch_layernorm(ctx, w.x, m->layers[0].norm1_w, m->layers[0].norm1_b, total, c.width, c.eps, nullptr, &qx));
    }
    for (int i = 0; i < c.layers; i++) {
        if (fused) {
            TSM_TRY(launch_layer_fused(m, cache, i, total, order, scale));
            continue;
        }
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
        // a decode step of a few rows: rope and the cache append happen inside the attention kernel
        const bool fresh_rows = total <= 4 && m->one_token_per_row;
        FreshRows fresh{c.arch == 0 ? m->rope_cos : nullptr, c.arch == 0 ? m->rope_sin : nullptr, c.context};
        if (!fresh_rows)
            TSM_TRY(launch_rope_append(ctx, w.qkv, total, c.heads, c.kv_heads, hw, c.arch == 0 ? m->rope_cos : nullptr,
                                       c.arch == 0 ? m->rope_sin : nullptr, c.context, w.table, cache->keys[i], cache->values[i],
                                       cache->rows, cache->capacity));
        f = feeds(l.o, w.att, &qb);
        TSM_TRY(launch_attention(ctx, w.qkv, qkvn, total, c.heads, hw, cache->keys[i], cache->values[i], cache->rows, c.kv_heads,
                                 cache->capacity, w.table, scale, ordered || f.plain ? w.att : nullptr, f.quantized, order,
                                 fresh_rows ? &fresh : nullptr));
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
    if (fused)   // the last exchange delivered the final norm of every row
        return launch_head_sharded(m, quant_scratch_layout(xchg_quantized(m), total, c.width), outputs, pick, !pick);
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

extern "C" {

int tsm_model_free(tsm_model* model) {
    if (!model) return TSM_OK;
    MODEL_GUARD(model);
    cudaStreamSynchronize(model->ctx->stream);
    free_workspace(model);
    xchg_release(model);
    for (void* p : model->owned) pool_release(model->ctx, p);
    delete model;
    return TSM_OK;
}

int tsm_model_load_gguf(tsm_ctx* ctx, const char* path, tsm_model** out) {
    if (!ctx || !path || !out) return TSM_ERR_ARG;
    tsm::DeviceGuard guard(ctx->ordinal);
    *out = nullptr;
    std::unique_ptr<tsm_model> m(new tsm_model());
    m->ctx = ctx;
    m->tp = ctx->tp_world, m->tp_rank = ctx->tp_rank, m->tp_reduce = ctx->tp_world > 1 && ctx->tp_variant == TSM_TP_REDUCE;
    int rc = load_gguf_model(m.get(), path);
    if (rc != TSM_OK) {
        tsm_model_free(m.release());
        return rc;
    }
    set_head_local(m.get());
    register_names(m.get());
    rc = xchg_setup(m.get());
    if (rc != TSM_OK) {
        tsm_model_free(m.release());
        return rc;
    }
    *out = m.release();
    return TSM_OK;
}

int tsm_gguf_check(const char* path, char* reason, int capacity) {
    std::string why;
    int rc = check_gguf_file(path, &why);
    if (reason && capacity > 0) {
        strncpy(reason, why.c_str(), (size_t)capacity - 1);
        reason[capacity - 1] = 0;
    }
    return rc;
}

int tsm_model_load_safetensors(tsm_ctx* ctx, const char* path, const tsm_model_config* config, int kind, tsm_model** out) {
    if (!ctx || !path || !config || !out) return TSM_ERR_ARG;
    tsm::DeviceGuard guard(ctx->ordinal);
    *out = nullptr;
    if (kind < TSM_F32 || kind > 2) return fail(ctx, TSM_ERR_UNSUPPORTED, "not a weight format");
    std::unique_ptr<tsm_model> m(new tsm_model());
    m->ctx = ctx;
    m->tp = ctx->tp_world, m->tp_rank = ctx->tp_rank, m->tp_reduce = ctx->tp_world > 1 && ctx->tp_variant == TSM_TP_REDUCE;
    int rc = load_safetensors_model(m.get(), path, *config, kind);
    if (rc != TSM_OK) {
        tsm_model_free(m.release());
        return rc;
    }
    set_head_local(m.get());
    register_names(m.get());
    rc = xchg_setup(m.get());
    if (rc != TSM_OK) {
        tsm_model_free(m.release());
        return rc;
    }
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
    rc = xchg_setup(m.get());
    if (rc != TSM_OK) {
        tsm_model_free(m.release());
        return rc;
    }
    *out = m.release();
    return TSM_OK;
}

int tsm_model_save_gguf(tsm_model* model, const char* path) {
    if (!model || !path) return TSM_ERR_ARG;
    MODEL_GUARD(model);
    return save_gguf_model(model, path);
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
                        int32_t* picks, bool keep_on_device = false) {
    if (!cache || cache->model != model || !counts || !ids || (!logits && !picks && !keep_on_device)) return fail(model->ctx, TSM_ERR_ARG, "forward needs a cache of this model, counts, ids and a place for logits");
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
    // A step that holds a prompt (a row with 8 new tokens or more): attention takes the tokens in tiles of 16 consecutive
    // tokens of one row, the tiles that see the most positions first.
    int longest = 0;
    for (int row = 0; row < cache->rows; row++) longest = std::max(longest, (int)counts[row]);
    ctx->prefill_tiles = nullptr, ctx->prefill_tile_count = 0;
    if (longest >= 8) {
        int32_t* h_tiles = w.host + 5 * (int64_t)w.tokens;
        std::vector<std::pair<int, std::pair<int, int>>> tiles;   // (last position, (first token, count))
        int first = 0;
        for (int row = 0; row < cache->rows; row++) {
            for (int j = 0; j < counts[row]; j += 16) {
                int n = std::min(16, (int)counts[row] - j);
                tiles.push_back({cache->lengths[row] + j + n - 1, {first + j, n}});
            }
            first += counts[row];
        }
        std::stable_sort(tiles.begin(), tiles.end(), [](const auto& a, const auto& b) { return a.first > b.first; });
        for (size_t i = 0; i < tiles.size(); i++) h_tiles[2 * i] = tiles[i].second.first, h_tiles[2 * i + 1] = tiles[i].second.second;
        TSM_CUDA(ctx, cudaMemcpyAsync(w.qtiles, h_tiles, tiles.size() * 8, cudaMemcpyHostToDevice, ctx->stream));
        ctx->prefill_tiles = w.qtiles, ctx->prefill_tile_count = (int)tiles.size();
    }
    model->one_token_per_row = longest <= 1;
    int step_rc = launch_step(model, cache, total, outputs, picks != nullptr);
    ctx->prefill_tiles = nullptr, ctx->prefill_tile_count = 0;
    TSM_TRY(step_rc);
    if (logits && picks && model->tp > 1) TSM_TRY(gather_full_logits(model, outputs));
    if (keep_on_device) {  // the caller reads ws.logits itself, after its own kernels
        for (int row = 0; row < cache->rows; row++) cache->lengths[row] += counts[row];
        return TSM_OK;
    }
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
    if (ctx->profile.on) {
        // a profile times operators one by one, which a replayed graph does not allow: the same step, launched directly
        std::vector<int32_t> ones(rows, 1);
        return forward_impl(model, cache, ones.data(), ids, 1, logits, tokens);
    }
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
        const int64_t exchanges_before = ctx->counters.collectives;
        TSM_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        int rc = TSM_OK;
        cudaError_t e1 = cudaMemcpyAsync(w.ids, h_ids, (size_t)rows * 4, cudaMemcpyHostToDevice, ctx->stream);
        cudaError_t e2 = cudaMemcpyAsync(w.table, h_table, (size_t)rows * 12, cudaMemcpyHostToDevice, ctx->stream);
        if (e1 != cudaSuccess || e2 != cudaSuccess) rc = cuda_fail(ctx, e1 != cudaSuccess ? e1 : e2, "cudaMemcpyAsync");
        model->one_token_per_row = true;
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
            cache->graph_collectives = (int)(ctx->counters.collectives - exchanges_before);
            ctx->counters.collectives = exchanges_before;
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
    ctx->counters.collectives += cache->graph_collectives;
    ctx->counters.uploads += 2, ctx->counters.upload_bytes += (int64_t)rows * 16;
    ctx->counters.downloads += 1, ctx->counters.download_bytes += (int64_t)rows * 4;
    if (logits) {
        if (model->tp > 1) TSM_TRY(gather_full_logits(model, rows));
        TSM_CUDA(ctx, cudaMemcpyAsync(logits, w.logits, (size_t)rows * c.vocab * 4, cudaMemcpyDeviceToHost, ctx->stream));
        ctx->counters.downloads++, ctx->counters.download_bytes += (int64_t)rows * c.vocab * 4;
    }
    TSM_TRY(tp_stream_wait(ctx));
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
    if (ctx->profile.on) {
        std::vector<int32_t> feed(ids, ids + rows);
        for (int s = 0; s < steps; s++) {
            TSM_TRY(tsm_decode(model, cache, feed.data(), tokens + (int64_t)s * rows, nullptr));
            feed.assign(tokens + (int64_t)s * rows, tokens + (int64_t)(s + 1) * rows);
        }
        return TSM_OK;
    }
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
        const int64_t exchanges_before = ctx->counters.collectives;
        TSM_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        cudaError_t e0 = launch_chained(ctx, run_advance_kernel, dim3((rows + 255) / 256), dim3(256), 0, w.ids, w.table, w.picks, rows, cache->run_state);
        count_launch(ctx);
        model->one_token_per_row = true;
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
            cache->run_collectives = (int)(ctx->counters.collectives - exchanges_before);
            ctx->counters.collectives = exchanges_before;
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
        if (model->tp > 1 && !getenv("TSM_TP_RUN_QUEUED")) TSM_TRY(tp_stream_wait(ctx));
    }
    ctx->counters.graph_replays += steps;
    ctx->counters.launches += (int64_t)steps * cache->run_kernels;
    ctx->counters.collectives += (int64_t)steps * cache->run_collectives;
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

int tsm_generate_sampled(tsm_model* model, const int32_t* prompt, int prompt_size, int count, const int32_t* stop, int stop_size,
                         int top_k, tsm_pick_fn pick, void* user, int32_t* tokens, int* produced) {
    MODEL_GUARD(model);
    tsm_ctx* ctx = model->ctx;
    if (produced) *produced = 0;
    if (!prompt || prompt_size < 1 || count < 0 || (count > 0 && !tokens) || stop_size < 0 || (stop_size > 0 && !stop) || top_k < 0)
        return fail(ctx, TSM_ERR_ARG, "generate needs a prompt, a place for tokens and a stop list that matches its size");
    const tsm_model_config& c = model->cfg;
    if (top_k >= c.vocab) top_k = 0;  // Sampler#pick: every token, in index order (sampler.cr:38)
    if (pick && top_k > 1024) return fail(ctx, TSM_ERR_UNSUPPORTED, "at most 1024 candidates are kept on the device");
    if (count == 0) return TSM_OK;
    int capacity = prompt_size + count < c.context ? prompt_size + count : c.context;
    tsm_cache* cache = nullptr;
    TSM_TRY(tsm_cache_create(model, 1, capacity, &cache));
    const int kept = pick ? (top_k > 0 ? top_k : c.vocab) : 0;
    std::vector<int32_t> cand_ids(top_k > 0 ? top_k : 0);
    std::vector<float> cand_values(kept);
    int* d_ids = nullptr;
    float* d_values = nullptr;
    int rc = TSM_OK;
    if (pick && top_k > 0) {
        rc = pool_alloc(ctx, (int64_t)top_k * 4, (void**)&d_ids);
        if (rc == TSM_OK) rc = pool_alloc(ctx, (int64_t)top_k * 4, (void**)&d_values);
    }
    int made = 0;
    int32_t counts[1] = {prompt_size};
    const int32_t* feed = prompt;
    int32_t last_token = 0;
    while (rc == TSM_OK && made < count) {
        int32_t token = 0;
        if (!pick) {
            rc = forward_impl(model, cache, counts, feed, 1, nullptr, &token);   // Sampler.greedy on the device (sampler.cr:36)
        } else if (top_k > 0) {
            rc = forward_impl(model, cache, counts, feed, 1, nullptr, nullptr, true);
            if (rc == TSM_OK) rc = launch_topk(ctx, model->ws.logits, 1, c.vocab, top_k, d_ids, d_values);
            if (rc == TSM_OK) {
                cudaError_t e = cudaMemcpyAsync(cand_ids.data(), d_ids, (size_t)top_k * 4, cudaMemcpyDeviceToHost, ctx->stream);
                if (e == cudaSuccess) e = cudaMemcpyAsync(cand_values.data(), d_values, (size_t)top_k * 4, cudaMemcpyDeviceToHost, ctx->stream);
                if (e != cudaSuccess) rc = cuda_fail(ctx, e, "cudaMemcpyAsync");
                ctx->counters.downloads += 2, ctx->counters.download_bytes += (int64_t)top_k * 8;
            }
            if (rc == TSM_OK) rc = tsm_sync(ctx);
            if (rc == TSM_OK) token = pick(user, made, cand_ids.data(), cand_values.data(), top_k);
        } else {
            rc = forward_impl(model, cache, counts, feed, 1, cand_values.data(), nullptr);
            if (rc == TSM_OK) token = pick(user, made, nullptr, cand_values.data(), c.vocab);
        }
        if (rc != TSM_OK) break;
        if (token < 0 || token >= c.vocab) {
            rc = fail(ctx, TSM_ERR_ARG, "the sampler returned token " + std::to_string(token) + " of a vocabulary of " + std::to_string(c.vocab));
            break;
        }
        tokens[made++] = token;
        bool stopped = false;
        for (int i = 0; i < stop_size; i++) stopped = stopped || stop[i] == token;
        if (stopped) break;
        last_token = token, feed = &last_token, counts[0] = 1;
    }
    pool_release(ctx, d_ids), pool_release(ctx, d_values);
    tsm_cache_free(cache);
    if (produced) *produced = made;
    return rc;
}

}  // extern "C"
