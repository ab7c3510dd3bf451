/*
 * CPU oracle for the quantised decode path of tensomite (TEST INFRASTRUCTURE).
 *
 * This file restates, in plain C, the arithmetic of tensomite's CPU device for
 * the token loop of its Llama and GPT-2 models over ggml Q8_0 / Q4_0 / Q4_1
 * weights.  It exists only to check the CUDA library against and to be timed
 * as the CPU baseline; the product never links, loads or calls it.
 *
 * Every function names the reference source it follows (path within the
 * tensomite project : lines).  Each `*`, `+`, `-`, `/` on floats below is a
 * separately rounded IEEE-754 binary32 operation; build with
 * `-ffp-contract=off` so that the compiler never fuses a multiply with an add.
 *
 * Parity pins: the block quantisers and dequantisers are checked byte for byte
 * against the reference's golden fixture (spec/fixtures/quant/expected.json);
 * the activation quantiser, the block products and the block gather are checked
 * bit for bit against the reference's own kernel sources compiled for the host
 * (Makefile target `ref`); the F32 model arithmetic is checked against the
 * reference's tiny_llama / tiny_gpt2 logits fixtures.
 */
#define _POSIX_C_SOURCE 200809L
#include <math.h>
#include <pthread.h>
#include <stdatomic.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

#define ORC_Q8_0 0
#define ORC_Q4_0 1
#define ORC_Q4_1 2

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* ---- F16 <-> F32 : src/tensomite/f16.cr:29-59 ---------------------------- */

/* f16.cr:29-41: nearest half, ties to even; overflow to infinity from 65520. */
uint16_t orc_f32_to_f16(float value) {
    uint32_t word = f2u(value);
    uint16_t sign = (uint16_t)((word >> 16) & 0x8000u);
    uint32_t magnitude = word & 0x7fffffffu;
    if (magnitude >= 0x7f800000u) return (uint16_t)(sign | (magnitude > 0x7f800000u ? 0x7e00u : 0x7c00u));
    if (magnitude >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);
    if (magnitude < 0x38800000u) return (uint16_t)(sign | (uint16_t)rintf(u2f(magnitude) * 16777216.0f));
    return (uint16_t)(sign | ((magnitude - 0x38000000u + 0xfffu + ((magnitude >> 13) & 1u)) >> 13));
}

/* f16.cr:44-59: exact widening. */
float orc_f16_to_f32(uint16_t bits) {
    uint32_t sign = ((uint32_t)bits & 0x8000u) << 16;
    uint32_t exponent = ((uint32_t)bits >> 10) & 0x1fu;
    uint32_t fraction = (uint32_t)bits & 0x3ffu;
    if (exponent == 0) {
        float magnitude = (float)fraction * 5.9604645e-8f;
        return sign == 0 ? magnitude : -magnitude;
    }
    if (exponent == 31) return u2f(sign | 0x7f800000u | (fraction << 13));
    return u2f(sign | ((exponent + 112u) << 23) | (fraction << 13));
}

static inline float half_at(const uint8_t* p) { return orc_f16_to_f32((uint16_t)(p[0] | (p[1] << 8))); }
static inline void put_half(uint8_t* p, float v) { uint16_t b = orc_f32_to_f16(v); p[0] = (uint8_t)(b & 0xff); p[1] = (uint8_t)(b >> 8); }
static inline float round_to_half(float v) { return orc_f16_to_f32(orc_f32_to_f16(v)); }

/* ---- own exp / tanh : src/tensomite/maths.cr:36-54, 99-114 ---------------- */

float orc_exp(float x) {
    const float LOG2E = 1.44269504088896341f, LN2_HI = 0.693359375f, LN2_LO = -2.12194440e-4f;
    const float EXP_HI = 88.72283905f, EXP_LO = -87.3365447f, ROUNDER = 12582912.0f;
    float clamped = (x > EXP_HI || x < EXP_LO) ? 0.0f : x;
    float n = (clamped * LOG2E + ROUNDER) - ROUNDER;
    float r = clamped - n * LN2_HI - n * LN2_LO;
    float z = r * r;
    float p = 1.9875691500e-4f;
    p = p * r + 1.3981999507e-3f;
    p = p * r + 8.3334519073e-3f;
    p = p * r + 4.1665795894e-2f;
    p = p * r + 1.6666665459e-1f;
    p = p * r + 5.0000001201e-1f;
    p = p * z + r + 1.0f;
    int32_t whole = (int32_t)n;
    int32_t half = whole >> 1;
    float result = p * u2f((uint32_t)(half + 127) << 23) * u2f((uint32_t)(whole - half + 127) << 23);
    if (x > EXP_HI) result = INFINITY;
    if (x < EXP_LO) result = 0.0f;
    return x != x ? x : result;
}

float orc_tanh(float x) {
    float a = fabsf(x);
    float z = x * x;
    float p = -5.70498872745e-3f;
    p = p * z + 2.06390887954e-2f;
    p = p * z - 5.37397155531e-2f;
    p = p * z + 1.33314422036e-1f;
    p = p * z - 3.33332819422e-1f;
    float near = p * z * x + x;
    float far = 1.0f - 2.0f / (orc_exp(a + a) + 1.0f);
    if (a > 9.01f) far = 1.0f;
    if (x < 0.0f) far = -far;
    float result = a < 0.625f ? near : far;
    if (x == 0.0f) result = x;
    return x != x ? x : result;
}

/* ---- block formats : src/tensomite/quant.cr:499-556 ----------------------- */

int orc_block_bytes(int kind) { return kind == ORC_Q8_0 ? 34 : kind == ORC_Q4_0 ? 18 : 20; }

/* Crystal's Float32#round(:ties_away) then to_i8! (wrapping narrow). */
static inline int8_t round_away_i8(float v) { return (int8_t)(int32_t)roundf(v); }
/* Crystal's Float32#to_i8! truncates toward zero and wraps. */
static inline int trunc_i8(float v) { return (int)(int8_t)(int32_t)v; }

/* quant.cr:499-505 */
static void quantize_q8_0(const float* x, uint8_t* t) {
    float amax = fabsf(x[0]);
    for (int j = 1; j < 32; j++) { float a = fabsf(x[j]); if (a > amax) amax = a; }
    float d = amax / 127.0f;
    float id = d == 0.0f ? 0.0f : 1.0f / d;
    put_half(t, d);
    for (int j = 0; j < 32; j++) t[2 + j] = (uint8_t)round_away_i8(x[j] * id);
}

/* quant.cr:509-520 */
static void quantize_q4_0(const float* x, uint8_t* t) {
    float max = x[0];
    for (int j = 0; j < 32; j++) if (fabsf(x[j]) > fabsf(max)) max = x[j];
    float d = max / -8.0f;
    float id = d == 0.0f ? 0.0f : 1.0f / d;
    put_half(t, d);
    for (int j = 0; j < 16; j++) {
        int low = trunc_i8(x[j] * id + 8.5f), high = trunc_i8(x[j + 16] * id + 8.5f);
        if (low > 15) low = 15;
        if (high > 15) high = 15;
        t[2 + j] = (uint8_t)((uint8_t)low | (uint8_t)((uint8_t)high << 4));
    }
}

/* quant.cr:524-535 */
static void quantize_q4_1(const float* x, uint8_t* t) {
    float min = x[0], max = x[0];
    for (int j = 1; j < 32; j++) { if (x[j] < min) min = x[j]; if (x[j] > max) max = x[j]; }
    float d = (max - min) / 15.0f;
    float id = d == 0.0f ? 0.0f : 1.0f / d;
    put_half(t, d);
    put_half(t + 2, min);
    for (int j = 0; j < 16; j++) {
        int low = trunc_i8((x[j] - min) * id + 0.5f), high = trunc_i8((x[j + 16] - min) * id + 0.5f);
        if (low > 15) low = 15;
        if (high > 15) high = 15;
        t[4 + j] = (uint8_t)((uint8_t)low | (uint8_t)((uint8_t)high << 4));
    }
}

/* quant.cr:77-90: `count` values (a whole number of blocks) -> block bytes. */
void orc_quantize(int kind, const float* x, int64_t count, uint8_t* out) {
    int bb = orc_block_bytes(kind);
    for (int64_t b = 0; b < count / 32; b++) {
        if (kind == ORC_Q8_0) quantize_q8_0(x + b * 32, out + b * bb);
        else if (kind == ORC_Q4_0) quantize_q4_0(x + b * 32, out + b * bb);
        else quantize_q4_1(x + b * 32, out + b * bb);
    }
}

/* quant.cr:537-556 */
static void dequantize_block(int kind, const uint8_t* b, float* x) {
    if (kind == ORC_Q8_0) {
        float d = half_at(b);
        for (int j = 0; j < 32; j++) x[j] = (float)(int8_t)b[2 + j] * d;
    } else if (kind == ORC_Q4_0) {
        float d = half_at(b);
        for (int j = 0; j < 16; j++) {
            x[j] = (float)((int)(b[2 + j] & 0x0f) - 8) * d;
            x[j + 16] = (float)((int)(b[2 + j] >> 4) - 8) * d;
        }
    } else {
        float d = half_at(b), m = half_at(b + 2);
        for (int j = 0; j < 16; j++) {
            x[j] = d * (float)(b[4 + j] & 0x0f) + m;
            x[j + 16] = d * (float)(b[4 + j] >> 4) + m;
        }
    }
}

/* quant.cr:93-105 */
void orc_dequantize(int kind, const uint8_t* bytes, int64_t count, float* x) {
    int bb = orc_block_bytes(kind);
    for (int64_t b = 0; b < count / 32; b++) dequantize_block(kind, bytes + b * bb, x + b * 32);
}

/* quant.cr:417-422 with devices/host.cr:648-658: returns the first id out of
 * range (and writes nothing for it) or -1... the host raises ExecutionError. */
int64_t orc_gather_blocks(int kind, const uint8_t* table, int64_t table_rows, int width, const int32_t* ids,
                          int64_t count, float* dst) {
    int64_t row_bytes = (int64_t)(width / 32) * orc_block_bytes(kind);
    for (int64_t i = 0; i < count; i++) {
        if (ids[i] < 0 || ids[i] >= table_rows) return i;
        orc_dequantize(kind, table + ids[i] * row_bytes, width, dst + i * width);
    }
    return -1;
}

/* ---- activation quantiser : quant.cr:428-442 ------------------------------ */

void orc_quantize_activations(const float* x, int k, float* scales, float* sums, int8_t* qs, int with_sums) {
    for (int block = 0; block < k / 32; block++) {
        const float* v = x + block * 32;
        float amax = fabsf(v[0]);
        for (int j = 1; j < 32; j++) { float a = fabsf(v[j]); if (a > amax) amax = a; }
        float d = amax / 127.0f;
        float id = d == 0.0f ? 0.0f : 1.0f / d;
        int total = 0;
        for (int j = 0; j < 32; j++) {
            int8_t q = round_away_i8(v[j] * id);
            qs[block * 32 + j] = q;
            total += q;
        }
        scales[block] = round_to_half(d);
        if (with_sums) sums[block] = round_to_half((float)total * d);
    }
}

/* ---- the oracle product : quant.cr:122-142, 446-491 ----------------------- */

static float dot_q8_0(const uint8_t* w, const float* scales, const int8_t* qs, int blocks) {
    float sum = 0.0f;
    for (int b = 0; b < blocks; b++) {
        const uint8_t* base = w + b * 34;
        const int8_t* qb = qs + b * 32;
        int total = 0;
        for (int j = 0; j < 32; j++) total += (int)(int8_t)base[2 + j] * qb[j];
        sum += (float)total * (half_at(base) * scales[b]);
    }
    return sum;
}

static float dot_q4_0(const uint8_t* w, const float* scales, const int8_t* qs, int blocks) {
    float sum = 0.0f;
    for (int b = 0; b < blocks; b++) {
        const uint8_t* base = w + b * 18;
        const int8_t* qb = qs + b * 32;
        int low = 0, high = 0;
        for (int j = 0; j < 16; j++) {
            uint8_t packed = base[2 + j];
            low += ((int)(packed & 0x0f) - 8) * qb[j];
            high += ((int)(packed >> 4) - 8) * qb[j + 16];
        }
        sum += (float)(low + high) * half_at(base) * scales[b];
    }
    return sum;
}

static float dot_q4_1(const uint8_t* w, const float* scales, const float* sums, const int8_t* qs, int blocks) {
    float sum = 0.0f;
    for (int b = 0; b < blocks; b++) {
        const uint8_t* base = w + b * 20;
        const int8_t* qb = qs + b * 32;
        int low = 0, high = 0;
        for (int j = 0; j < 16; j++) {
            uint8_t packed = base[4 + j];
            low += (int)(packed & 0x0f) * qb[j];
            high += (int)(packed >> 4) * qb[j + 16];
        }
        sum += (half_at(base) * scales[b]) * (float)(low + high) + half_at(base + 2) * sums[b];
    }
    return sum;
}

/* quant.cr:122-142. dst is [rows, n]; bias (may be NULL) is added after each
 * full sum as devices/host.cr:725-734 does. */
void orc_matmul_reference(int kind, const float* x, const uint8_t* w, int rows, int n, int k, const float* bias,
                          float* dst) {
    int blocks = k / 32;
    int64_t row_bytes = (int64_t)blocks * orc_block_bytes(kind);
    float* scales = (float*)malloc(sizeof(float) * (size_t)blocks);
    float* sums = (float*)malloc(sizeof(float) * (size_t)blocks);
    int8_t* qs = (int8_t*)malloc((size_t)k);
    for (int row = 0; row < rows; row++) {
        orc_quantize_activations(x + (int64_t)row * k, k, scales, sums, qs, kind == ORC_Q4_1);
        for (int col = 0; col < n; col++) {
            const uint8_t* weight = w + col * row_bytes;
            float v = kind == ORC_Q8_0   ? dot_q8_0(weight, scales, qs, blocks)
                      : kind == ORC_Q4_0 ? dot_q4_0(weight, scales, qs, blocks)
                                         : dot_q4_1(weight, scales, sums, qs, blocks);
            dst[(int64_t)row * n + col] = bias ? v + bias[col] : v;
        }
    }
    free(scales); free(sums); free(qs);
}

/* ---- the fast threaded product : quant.cr:155-211, 219-302, 318-413 ------- */

static float HALVES[65536];
static pthread_once_t halves_once = PTHREAD_ONCE_INIT;
static void build_halves(void) { for (int i = 0; i < 65536; i++) HALVES[i] = orc_f16_to_f32((uint16_t)i); }
static inline float fast_half(const uint8_t* p) { return HALVES[p[0] | (p[1] << 8)]; }

/* quant.cr:309-313 */
static inline int32_t round_away(float value) {
    int32_t whole = (int32_t)value;
    float fraction = value - (float)whole;
    return whole + (fraction >= 0.5f ? 1 : 0) - (fraction <= -0.5f ? 1 : 0);
}

/* quant.cr:318-334 */
static void fast_quantize(const float* x, int blocks, float* sp, float* mp, int32_t* tp, int8_t* qp, int with_sums) {
    for (int block = 0; block < blocks; block++) {
        const float* v = x + block * 32;
        float top = fabsf(v[0]);
        for (int j = 1; j < 32; j++) if (fabsf(v[j]) > top) top = fabsf(v[j]);
        float d = top / 127.0f;
        float id = d == 0.0f ? 0.0f : 1.0f / d;
        int8_t* qb = qp + block * 32;
        for (int j = 0; j < 32; j++) qb[j] = (int8_t)round_away(v[j] * id);
        int32_t total = 0;
        for (int j = 0; j < 32; j++) total += qb[j];
        tp[block] = total;
        sp[block] = round_to_half(d);
        if (with_sums) mp[block] = round_to_half((float)total * d);
    }
}

/* quant.cr:349-366: two weight rows share each load of the activations. */
static void fast_q8_0(const uint8_t* w0, const uint8_t* w1, const float* sp, const int8_t* qp, int blocks, float* o0,
                      float* o1) {
    float sum0 = 0.0f, sum1 = 0.0f;
    for (int b = 0; b < blocks; b++) {
        const uint8_t *base0 = w0 + b * 34, *base1 = w1 + b * 34;
        const int8_t *v0 = (const int8_t*)(base0 + 2), *v1 = (const int8_t*)(base1 + 2), *qb = qp + b * 32;
        int32_t t0 = 0, t1 = 0;
        for (int j = 0; j < 32; j++) { int32_t y = qb[j]; t0 += v0[j] * y; t1 += v1[j] * y; }
        sum0 += (float)t0 * (fast_half(base0) * sp[b]);
        sum1 += (float)t1 * (fast_half(base1) * sp[b]);
    }
    *o0 = sum0; *o1 = sum1;
}

/* quant.cr:373-386 */
static inline void nibble_dot(const uint8_t* p0, const uint8_t* p1, const int8_t* qb, int32_t* d0, int32_t* d1) {
    int32_t t0 = 0, t1 = 0;
    for (int j = 0; j < 16; j++) {
        int32_t y = qb[j];
        t0 += (int32_t)(int8_t)((int8_t)(p0[j] & 0x0f) - 8) * y;
        t1 += (int32_t)(int8_t)((int8_t)(p1[j] & 0x0f) - 8) * y;
    }
    for (int j = 0; j < 16; j++) {
        int32_t y = qb[j + 16];
        t0 += (int32_t)(int8_t)((int8_t)(p0[j] >> 4) - 8) * y;
        t1 += (int32_t)(int8_t)((int8_t)(p1[j] >> 4) - 8) * y;
    }
    *d0 = t0; *d1 = t1;
}

/* quant.cr:388-399 */
static void fast_q4_0(const uint8_t* w0, const uint8_t* w1, const float* sp, const int8_t* qp, int blocks, float* o0,
                      float* o1) {
    float sum0 = 0.0f, sum1 = 0.0f;
    for (int b = 0; b < blocks; b++) {
        const uint8_t *base0 = w0 + b * 18, *base1 = w1 + b * 18;
        int32_t t0, t1;
        nibble_dot(base0 + 2, base1 + 2, qp + b * 32, &t0, &t1);
        sum0 += (float)t0 * fast_half(base0) * sp[b];
        sum1 += (float)t1 * fast_half(base1) * sp[b];
    }
    *o0 = sum0; *o1 = sum1;
}

/* quant.cr:401-413 */
static void fast_q4_1(const uint8_t* w0, const uint8_t* w1, const float* sp, const float* mp, const int32_t* tp,
                      const int8_t* qp, int blocks, float* o0, float* o1) {
    float sum0 = 0.0f, sum1 = 0.0f;
    for (int b = 0; b < blocks; b++) {
        const uint8_t *base0 = w0 + b * 20, *base1 = w1 + b * 20;
        int32_t d0, d1;
        nibble_dot(base0 + 4, base1 + 4, qp + b * 32, &d0, &d1);
        int32_t shift = 8 * tp[b];
        sum0 += (fast_half(base0) * sp[b]) * (float)(d0 + shift) + fast_half(base0 + 2) * mp[b];
        sum1 += (fast_half(base1) * sp[b]) * (float)(d1 + shift) + fast_half(base1 + 2) * mp[b];
    }
    *o0 = sum0; *o1 = sum1;
}

/* One product's shared state for the span workers. */
typedef struct {
    int kind, n, blocks;
    int64_t row_bytes;
    const uint8_t* w;
    const float *sp, *mp;
    const int32_t* tp;
    const int8_t* qp;
    float* out;
} span_job;

static void run_span(const span_job* j, int first, int stop) {
    for (int col = first; col < stop; col += 2) {
        const uint8_t* w0 = j->w + col * j->row_bytes;
        const uint8_t* w1 = col + 1 < stop ? w0 + j->row_bytes : w0;
        float a, b;
        if (j->kind == ORC_Q8_0) fast_q8_0(w0, w1, j->sp, j->qp, j->blocks, &a, &b);
        else if (j->kind == ORC_Q4_0) fast_q4_0(w0, w1, j->sp, j->qp, j->blocks, &a, &b);
        else fast_q4_1(w0, w1, j->sp, j->mp, j->tp, j->qp, j->blocks, &a, &b);
        j->out[col] = a;
        if (col + 1 < stop) j->out[col + 1] = b;
    }
}

/* quant.cr:219-302: workers spin on one word: generation << 32 | spans << 16 |
 * next span; a span is claimed by compare-and-set on the whole word. */
#define ORC_MAX_THREADS 1024
static struct {
    _Atomic uint64_t claim;
    _Atomic int done;
    _Atomic int quit;
    int count;
    const span_job* job;
    int workers;
    pthread_t threads[ORC_MAX_THREADS];
} pool;

static void pool_help(uint64_t generation) {
    for (;;) {
        uint64_t claim = atomic_load(&pool.claim);
        if (claim >> 32 != generation) return;
        int spans = (int)((claim >> 16) & 0xffff), span = (int)(claim & 0xffff);
        if (span >= spans) return;
        if (!atomic_compare_exchange_weak(&pool.claim, &claim, claim + 1)) continue;
        int count = pool.count;
        run_span(pool.job, (int)((int64_t)count * span / spans), (int)((int64_t)count * (span + 1) / spans));
        atomic_fetch_add(&pool.done, 1);
    }
}

static void* pool_work(void* arg) {
    (void)arg;
    uint64_t seen = 0;
    for (;;) {
        int idle = 0;
        uint64_t current;
        while ((current = atomic_load(&pool.claim) >> 32) == seen) {
            if (atomic_load(&pool.quit)) return NULL;
            if (idle < 1000000) { idle++; __builtin_ia32_pause(); }
            else { struct timespec nap = {0, 100000}; nanosleep(&nap, NULL); }
        }
        seen = current;
        pool_help(current);
    }
}

static void pool_run(int threads, int spans, int count, const span_job* job) {
    while (pool.workers < threads - 1 && pool.workers < ORC_MAX_THREADS) {
        pthread_create(&pool.threads[pool.workers], NULL, pool_work, NULL);
        pool.workers++;
    }
    pool.job = job;
    pool.count = count;
    atomic_store(&pool.done, 0);
    uint64_t generation = ((atomic_load(&pool.claim) >> 32) + 1) & 0xffffffffull;
    atomic_store(&pool.claim, generation << 32 | (uint64_t)spans << 16);
    pool_help(generation);
    while (atomic_load(&pool.done) != spans) __builtin_ia32_pause();
}

/* Stops and joins the pool's workers (so a test process can exit cleanly). */
void orc_pool_shutdown(void) {
    atomic_store(&pool.quit, 1);
    for (int i = 0; i < pool.workers; i++) pthread_join(pool.threads[i], NULL);
    pool.workers = 0;
    atomic_store(&pool.quit, 0);
}

/* quant.cr:155-182 with in_parallel :204-211: spans = min(threads*4, n,
 * bytes / 64 KiB); one span on the caller when that is <= 1. */
void orc_matmul_fast(int kind, const float* x, const uint8_t* w, int rows, int n, int k, const float* bias, float* dst,
                     int threads) {
    pthread_once(&halves_once, build_halves);
    int blocks = k / 32;
    int64_t row_bytes = (int64_t)blocks * orc_block_bytes(kind);
    float* sp = (float*)malloc(sizeof(float) * (size_t)blocks);
    float* mp = (float*)malloc(sizeof(float) * (size_t)blocks);
    int32_t* tp = (int32_t*)malloc(sizeof(int32_t) * (size_t)blocks);
    int8_t* qp = (int8_t*)malloc((size_t)k);
    if (threads < 1) threads = 1;
    if (threads > ORC_MAX_THREADS) threads = ORC_MAX_THREADS;
    for (int row = 0; row < rows; row++) {
        fast_quantize(x + (int64_t)row * k, blocks, sp, mp, tp, qp, kind == ORC_Q4_1);
        span_job job = {kind, n, blocks, row_bytes, w, sp, mp, tp, qp, dst + (int64_t)row * n};
        int64_t by_bytes = (int64_t)n * row_bytes / (64 * 1024);
        int64_t spans = (int64_t)threads * 4;
        if (n < spans) spans = n;
        if (by_bytes < spans) spans = by_bytes;
        if (spans <= 1 || threads <= 1) run_span(&job, 0, n);
        else pool_run(threads, (int)spans, n, &job);
        if (bias) for (int col = 0; col < n; col++) dst[(int64_t)row * n + col] = dst[(int64_t)row * n + col] + bias[col];
    }
    free(sp); free(mp); free(tp); free(qp);
}

/* ---- host row ops : src/tensomite/devices/host.cr ------------------------- */

/* host.cr:391-403: squares folded from zero in index order. */
void orc_rmsnorm(const float* x, const float* w, int rows, int n, float eps, float* dst) {
    for (int r = 0; r < rows; r++) {
        const float* xr = x + (int64_t)r * n;
        float squares = 0.0f;
        for (int j = 0; j < n; j++) squares += xr[j] * xr[j];
        float root = sqrtf(squares / (float)n + eps);
        for (int j = 0; j < n; j++) dst[(int64_t)r * n + j] = w ? xr[j] / root * w[j] : xr[j] / root;
    }
}

/* host.cr:348-361 */
void orc_layernorm(const float* x, const float* w, const float* b, int rows, int n, float eps, float* dst) {
    for (int r = 0; r < rows; r++) {
        const float* xr = x + (int64_t)r * n;
        float* o = dst + (int64_t)r * n;
        float total = 0.0f;
        for (int j = 0; j < n; j++) total += xr[j];
        float mean = total / (float)n;
        float squares = 0.0f;
        for (int j = 0; j < n; j++) { float c = o[j] = xr[j] - mean; squares += c * c; }
        float std = sqrtf(squares / (float)n + eps);
        for (int j = 0; j < n; j++) o[j] = o[j] / std * w[j] + b[j];
    }
}

/* modules.cr:343-351: cos/sin tables [context, width] in F32 through libm. */
void orc_rope_tables(int width, int context, double theta, float* cos_out, float* sin_out) {
    int half = width / 2;
    float* freq = (float*)malloc(sizeof(float) * (size_t)half);
    for (int i = 0; i < half; i++) freq[i] = 1.0f / powf((float)theta, (float)(2 * i) / (float)width);
    for (int p = 0; p < context; p++)
        for (int i = 0; i < width; i++) {
            float angle = (float)p * freq[i % half];
            cos_out[(int64_t)p * width + i] = cosf(angle);
            sin_out[(int64_t)p * width + i] = sinf(angle);
        }
    free(freq);
}

/* host.cr:448-466: one row of `n` values rotated by its cos/sin row. */
void orc_rope_row(const float* x, const float* c, const float* s, int n, float* dst) {
    int half = n / 2;
    for (int col = 0; col < n; col++) {
        float partner = x[col < half ? col + half : col - half];
        float rotated = col < half ? partner * -1.0f : partner;
        dst[col] = x[col] * c[col] + rotated * s[col];
    }
}

/* kernels.cr:15 through kernel.cr:259-300: x / (exp(-x) + 1). */
void orc_silu(const float* x, int64_t count, float* dst) {
    for (int64_t i = 0; i < count; i++) {
        float t1 = orc_exp(-x[i]);
        float t2 = t1 + 1.0f;
        dst[i] = x[i] / t2;
    }
}

/* kernels.cr:18 through kernel.cr:259-300: gate / (exp(-gate) + 1) * up. */
void orc_swiglu(const float* gate, const float* up, int64_t count, float* dst) {
    for (int64_t i = 0; i < count; i++) {
        float t1 = orc_exp(-gate[i]);
        float t2 = t1 + 1.0f;
        float t3 = gate[i] / t2;
        dst[i] = t3 * up[i];
    }
}

/* kernels.cr:4: x * 0.5 * (tanh((x + x*x*x*0.044715) * sqrt(2/pi)) + 1), each
 * operation its own statement, constants narrowed to F32. */
void orc_gelu(const float* x, int64_t count, float* dst) {
    const float c = (float)sqrt(2.0 / 3.14159265358979323846);
    for (int64_t i = 0; i < count; i++) {
        float v = x[i];
        float t0 = v * 0.5f;
        float t1 = v * v;
        float t2 = t1 * v;
        float t3 = t2 * 0.044715f;
        float t4 = v + t3;
        float t5 = t4 * c;
        float t6 = orc_tanh(t5);
        float t7 = t6 + 1.0f;
        dst[i] = t0 * t7;
    }
}

/* The composite attention of one query row over positions 0...len of one
 * key/value head: matmul (host.cr:700-721), scaled softmax row (:368-387),
 * matmul again; every sum in index order from zero.  `stride` is the distance
 * in floats between consecutive positions of k and v. scores: len floats. */
void orc_attend(const float* q, const float* k, const float* v, int len, int width, int64_t stride, float scale,
                float* scores, float* out) {
    for (int p = 0; p < len; p++) {
        const float* kp = k + p * stride;
        float dot = 0.0f;
        for (int d = 0; d < width; d++) dot += q[d] * kp[d];
        scores[p] = dot * scale + 0.0f; /* visible positions carry a mask of 0 */
    }
    float top = scores[0];
    for (int p = 1; p < len; p++) if (scores[p] > top) top = scores[p];
    for (int p = 0; p < len; p++) scores[p] = orc_exp(scores[p] - top);
    float total = 0.0f;
    for (int p = 0; p < len; p++) total += scores[p];
    for (int p = 0; p < len; p++) scores[p] = scores[p] / total;
    for (int c = 0; c < width; c++) {
        float acc = 0.0f;
        for (int p = 0; p < len; p++) acc += scores[p] * v[p * stride + c];
        out[c] = acc;
    }
}

/* sampler.cr:36: the first index of the maximum. */
int orc_argmax_first(const float* logits, int n) {
    int best = 0;
    for (int i = 1; i < n; i++) if (logits[i] > logits[best]) best = i;
    return best;
}

/* sampler.cr:77-96: the `count` highest, highest first, ties by lower index. */
void orc_topk(const float* logits, int n, int count, int32_t* out) {
    /* selection by repeated scan: fine for the oracle's sizes */
    uint8_t* taken = (uint8_t*)calloc((size_t)n, 1);
    for (int r = 0; r < count && r < n; r++) {
        int best = -1;
        for (int i = 0; i < n; i++) {
            if (taken[i]) continue;
            if (best < 0 || logits[i] > logits[best]) best = i;
        }
        taken[best] = 1;
        out[r] = best;
    }
    free(taken);
}

/* ---- whole models : models/llama.cr:265-303, models/gpt2.cr:156-196,
 *      models/generative.cr:112-190, modules.cr (op order) ------------------- */

typedef struct {
    int kind;          /* ORC_Q8_0 / Q4_0 / Q4_1, or -1 for an F32 [n,k] row-major weight */
    int n, k;
    const uint8_t* w;  /* block bytes, rows of k/32 blocks ([n,k] floats when kind = -1) */
    const float* bias; /* or NULL */
} orc_linear;

typedef struct {
    const float *norm1_w, *norm1_b, *norm2_w, *norm2_b;
    orc_linear qkv, o, up, down; /* qkv: joined rows [q;k;v]; up: [gate;up] (Llama) or c_fc (GPT-2) */
} orc_layer;

typedef struct {
    int arch; /* 0 Llama, 1 GPT-2 */
    int layers, width, heads, kv_heads, head_width, hidden, vocab, context;
    float eps;
    double rope_theta;
    orc_linear embed;  /* token table as an [vocab,width] weight (kind -1: F32) */
    orc_linear wpe;    /* GPT-2 positions */
    orc_linear head;   /* the head's weight: the token table when tied */
    const float *final_w, *final_b;
    const orc_layer* blocks;
    const float *rope_cos, *rope_sin; /* [context, head_width] (Llama) */
    int threads;       /* for the fast product */
    int reference_products; /* 1: use orc_matmul_reference instead of the fast product */
} orc_model;

typedef struct {
    int rows, capacity;
    float** keys;   /* per layer: [rows, kv_heads, capacity, head_width] */
    float** values;
    int* lengths;
} orc_cache;

static void linear(const orc_model* m, const orc_linear* l, const float* x, int rows, float* dst) {
    if (l->kind < 0) {
        /* F32 weight [n,k]: devices/host.cr:700-721, sum over k in index order */
        const float* w = (const float*)l->w;
        for (int r = 0; r < rows; r++)
            for (int c = 0; c < l->n; c++) {
                float acc = 0.0f;
                for (int s = 0; s < l->k; s++) acc += x[(int64_t)r * l->k + s] * w[(int64_t)c * l->k + s];
                dst[(int64_t)r * l->n + c] = l->bias ? acc + l->bias[c] : acc;
            }
        return;
    }
    if (m->reference_products) orc_matmul_reference(l->kind, x, l->w, rows, l->n, l->k, l->bias, dst);
    else orc_matmul_fast(l->kind, x, l->w, rows, l->n, l->k, l->bias, dst, m->threads);
}

static void embed_rows(const orc_linear* t, const int32_t* ids, int count, float* dst) {
    if (t->kind < 0) {
        const float* w = (const float*)t->w;
        for (int i = 0; i < count; i++) memcpy(dst + (int64_t)i * t->k, w + (int64_t)ids[i] * t->k, sizeof(float) * (size_t)t->k);
    } else {
        orc_gather_blocks(t->kind, t->w, t->n, t->k, ids, count, dst);
    }
}

/* Runs `total` new tokens, packed row after row: token t belongs to cache row
 * rows[t] at position positions[t] and sees positions 0..positions[t]
 * (generative.cr:130-145).  Appends keys and values, then writes the logits of
 * the tokens flagged in `want` (in token order) to `logits`.  The caller
 * advances cache lengths.  Returns 0, or -1 for a bad token id. */
int orc_forward(const orc_model* m, orc_cache* cache, const int32_t* ids, const int32_t* rows, const int32_t* positions,
                int total, const uint8_t* want, float* logits) {
    int d = m->width, hw = m->head_width, H = m->heads, KV = m->kv_heads, F = m->hidden;
    int qn = H * hw, kvn = KV * hw, qkvn = qn + 2 * kvn;
    for (int t = 0; t < total; t++) if (ids[t] < 0 || ids[t] >= m->vocab) return -1;
    float* x = (float*)malloc(sizeof(float) * (size_t)total * d);
    float* h = (float*)malloc(sizeof(float) * (size_t)total * (d > qn ? d : qn));
    float* qkv = (float*)malloc(sizeof(float) * (size_t)total * qkvn);
    float* att = (float*)malloc(sizeof(float) * (size_t)total * qn);
    int upn = m->arch == 0 ? 2 * F : F;
    float* up = (float*)malloc(sizeof(float) * (size_t)total * upn);
    float* act = (float*)malloc(sizeof(float) * (size_t)total * F);
    float* tmp = (float*)malloc(sizeof(float) * (size_t)total * d);
    float* rot = (float*)malloc(sizeof(float) * (size_t)hw);
    int maxlen = 1;
    for (int t = 0; t < total; t++) if (positions[t] + 1 > maxlen) maxlen = positions[t] + 1;
    float* scores = (float*)malloc(sizeof(float) * (size_t)maxlen);
    float scale = (float)(1.0 / sqrt((double)hw));

    embed_rows(&m->embed, ids, total, x);
    if (m->arch == 1) { /* gpt2.cr:189-191: wte(ids) + wpe(positions) */
        embed_rows(&m->wpe, positions, total, tmp);
        for (int64_t i = 0; i < (int64_t)total * d; i++) x[i] = x[i] + tmp[i];
    }
    for (int l = 0; l < m->layers; l++) {
        const orc_layer* b = &m->blocks[l];
        if (m->arch == 0) orc_rmsnorm(x, b->norm1_w, total, d, m->eps, h);
        else orc_layernorm(x, b->norm1_w, b->norm1_b, total, d, m->eps, h);
        linear(m, &b->qkv, h, total, qkv);
        /* rotate (Llama), append, attend: modules.cr:434-473 */
        for (int t = 0; t < total; t++) {
            float* row = qkv + (int64_t)t * qkvn;
            int pos = positions[t];
            if (m->arch == 0) {
                const float* c = m->rope_cos + (int64_t)pos * hw;
                const float* s = m->rope_sin + (int64_t)pos * hw;
                for (int hd = 0; hd < H + KV; hd++) {
                    orc_rope_row(row + hd * hw, c, s, hw, rot);
                    memcpy(row + hd * hw, rot, sizeof(float) * (size_t)hw);
                }
            }
            for (int kh = 0; kh < KV; kh++) {
                int64_t slot = (((int64_t)rows[t] * KV + kh) * cache->capacity + pos) * hw;
                memcpy(cache->keys[l] + slot, row + qn + kh * hw, sizeof(float) * (size_t)hw);
                memcpy(cache->values[l] + slot, row + qn + kvn + kh * hw, sizeof(float) * (size_t)hw);
            }
        }
        for (int t = 0; t < total; t++) {
            const float* row = qkv + (int64_t)t * qkvn;
            for (int hq = 0; hq < H; hq++) {
                int kh = hq / (H / KV);
                int64_t base = ((int64_t)rows[t] * KV + kh) * cache->capacity * hw;
                orc_attend(row + hq * hw, cache->keys[l] + base, cache->values[l] + base, positions[t] + 1, hw, hw, scale,
                           scores, att + (int64_t)t * qn + hq * hw);
            }
        }
        linear(m, &b->o, att, total, tmp);
        for (int64_t i = 0; i < (int64_t)total * d; i++) x[i] = x[i] + tmp[i];
        if (m->arch == 0) orc_rmsnorm(x, b->norm2_w, total, d, m->eps, h);
        else orc_layernorm(x, b->norm2_w, b->norm2_b, total, d, m->eps, h);
        linear(m, &b->up, h, total, up);
        if (m->arch == 0) {
            for (int t = 0; t < total; t++)
                orc_swiglu(up + (int64_t)t * 2 * F, up + (int64_t)t * 2 * F + F, F, act + (int64_t)t * F);
        } else {
            orc_gelu(up, (int64_t)total * F, act);
        }
        linear(m, &b->down, act, total, tmp);
        for (int64_t i = 0; i < (int64_t)total * d; i++) x[i] = x[i] + tmp[i];
    }
    int out = 0;
    for (int t = 0; t < total; t++) {
        if (!want[t]) continue;
        if (m->arch == 0) orc_rmsnorm(x + (int64_t)t * d, m->final_w, 1, d, m->eps, h);
        else orc_layernorm(x + (int64_t)t * d, m->final_w, m->final_b, 1, d, m->eps, h);
        linear(m, &m->head, h, 1, logits + (int64_t)out * m->vocab);
        out++;
    }
    free(x); free(h); free(qkv); free(att); free(up); free(act); free(tmp); free(rot); free(scores);
    return 0;
}
