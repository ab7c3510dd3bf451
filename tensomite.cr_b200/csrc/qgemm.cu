// The quantised product for several rows of activations (batched decode, prefill), with the reference's
// bits (Quant.matmul_reference, quant.cr:122-142): out[m, n] = sum over blocks, in block order, of the
// block's contribution.
//
// A block is 32 elements, which is exactly the K of one int8 tensor-core instruction
// (mma.sync m16n8k32, s8 x s8 -> s32).  One instruction therefore gives the exact integer dot products
// of 16 weight rows with 8 activation rows for ONE block, into a fresh accumulator; the float work that
// must stay ordered (scale, scale, add to the running sum) then happens in the thread that holds each
// (weight row, activation row) pair, block after block, so the sum is folded in block order without
// any exchange between threads.  ggml's nibble layout (low nibble = element j, high = element j + 16)
// matches the instruction's fragment layout: one 32-bit word of packed nibbles yields both of a
// thread's A registers.  The accumulator is started at the bit pattern of 1.5 * 2^23, so the integer
// result read back as a float is 12582912 + dot and one subtraction converts it exactly.
//
// Weights stream through shared memory in chunks of 8 blocks per weight row.  Each row's chunk is one
// bulk asynchronous copy (cp.async.bulk) whose start is rounded down and end rounded up to 16 bytes,
// so rows of any even pitch (612-byte rows of 18 Q8_0 blocks included) are handled; the reader adds the
// row's shift back.  The quantised activations and their scales for the same 8 blocks are staged beside
// them with cp.async, so the inner loop reads shared memory only.  For Q4_0 the nibbles are turned into
// signed bytes (nibble - 8) before the multiply, which removes the -8 * sum(q) correction.
#include <stdlib.h>

#include "common.cuh"

namespace tsm {

namespace {

constexpr int kGemmStages = 3;
constexpr unsigned kGemmSpins = 4u << 20;

template <int KIND> struct GFmt;
template <> struct GFmt<TSM_Q8_0> { static constexpr int B = 34; };
template <> struct GFmt<TSM_Q4_0> { static constexpr int B = 18; };
template <> struct GFmt<TSM_Q4_1> { static constexpr int B = 20; };

struct GemmParams {
    const uint8_t* w;
    int n, nb, m;          // weight rows, blocks per row, activation rows
    QuantizedActs acts;
    const float* bias;
    const float* residual;
    float* out;            // [m, n]
    ErrorRecord* errors;
};

__device__ __forceinline__ unsigned g_smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void g_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(g_smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void g_mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(g_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool g_mbar_try_wait(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(g_smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool g_mbar_wait(uint64_t* bar, unsigned parity) {
    for (unsigned spin = 0; spin < kGemmSpins; spin++) {
        if (g_mbar_try_wait(bar, parity)) return true;
        if (spin > 4096) __nanosleep(64);
    }
    return false;
}
__device__ __forceinline__ void g_bulk_load(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(g_smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(g_smem_u32(bar))
                 : "memory");
}

// The 4 bytes at p (2-byte aligned, in shared memory) as a little-endian word.
__device__ __forceinline__ unsigned lds_u32_at2(const unsigned char* p) {
    // through the 32-bit shared address: a pointer rebuilt from an integer would be a generic one, and its loads generic loads
    const unsigned a = g_smem_u32(p);
    unsigned lo, hi;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(lo) : "r"(a & ~3u));
    asm volatile("ld.shared.u32 %0, [%1 + 4];" : "=r"(hi) : "r"(a & ~3u));
    return __funnelshift_r(lo, hi, (a & 3u) * 8);
}
__device__ __forceinline__ unsigned lds_u16_at2(const unsigned char* p) { return *(const unsigned short*)p; }

__device__ __forceinline__ void mma_s8(int (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1) {
    const int bias = 0x4b400000;  // 1.5 * 2^23 as a float: the result reads back as 12582912 + dot
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};\n"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "r"(bias));
}

__device__ __forceinline__ void g_cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(g_smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void g_cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(g_smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void g_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void g_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Nibbles 0..15 in the low half of each byte of x -> signed bytes nibble - 8, without touching neighbours:
// (b | 128) - 8 never borrows, and flipping bit 7 afterwards leaves b - 8 in two's complement.
__device__ __forceinline__ unsigned nibbles_minus_8(unsigned x) { return (((x & 0x0f0f0f0fu) | 0x80808080u) - 0x08080808u) ^ 0x80808080u; }

// Blocks of K per stage: 4 when a CTA takes 64 activation rows (their staging dominates shared memory), else 8.
__host__ __device__ constexpr int chunk_blocks(int cols) { return cols >= 64 ? 4 : 8; }

// A CTA of WR x WC warps takes 16 WR weight rows and 8 NT WC activation rows; warp (wr, wc) owns weight rows
// [16 wr, 16 wr + 16) and NT tiles of 8 activation rows from tile wc * NT; a weight fragment is prepared once
// per warp and block and used by NT multiplies.  Per
// stage of 4 or 8 blocks the weights arrive by one bulk copy per row and the quantised activations by 16-byte
// cp.async; scales are staged [block][activation row], so that a thread's two activation rows are one 8-byte load.
template <int KIND, int NT, int WR, int WC>
__global__ void __launch_bounds__(32 * WR * WC) matmul_mma_kernel(GemmParams p) {
    chained_kernel_entry();
    constexpr int B = GFmt<KIND>::B;
    constexpr int ROWS = 16 * WR, COLS = 8 * NT * WC, THREADS = 32 * WR * WC;
    constexpr int kChunkBlocks = chunk_blocks(COLS);
    constexpr int WP = (kChunkBlocks * B + 30 + 15) / 16 * 16;  // weight row pitch: a chunk plus the slack of rounding both ends, itself a multiple of 16 (a bulk copy's destination must be)
    constexpr int AP = kChunkBlocks * 32 + 16;  // activation row pitch: the 8 rows x 4 words of a B fragment fall in 32 distinct banks
    constexpr int STAGE = ROWS * WP + COLS * AP + 2 * COLS * kChunkBlocks * 4;
    extern __shared__ __align__(128) unsigned char smem[];
    uint64_t* full = (uint64_t*)smem;
    int* abort_flag = (int*)(smem + 64);
    unsigned char* stages = smem + 128;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int nb = p.nb;
    const int64_t rb = (int64_t)nb * B;
    const int row0 = blockIdx.x * ROWS;
    const int col0 = blockIdx.y * COLS;
    const int chunks = (nb + kChunkBlocks - 1) / kChunkBlocks;
    const int64_t k = (int64_t)nb * 32;

    auto issue = [&](int chunk) {  // every thread commits one cp.async group per call, so group c is chunk c
        if (chunk < chunks) {
            int s = chunk % kGemmStages;
            int count = min(kChunkBlocks, nb - chunk * kChunkBlocks);
            int len = count * B;
            unsigned char* base = stages + (size_t)s * STAGE;
            if (warp == 0) {
                // each lane sizes and issues its rows' copies; the lanes' bytes are summed for the barrier first
                unsigned mine = 0;
                for (int r = lane; r < ROWS && row0 + r < p.n; r += 32) {
                    int64_t o = (int64_t)(row0 + r) * rb + (int64_t)chunk * kChunkBlocks * B;
                    mine += (unsigned)(((o + len + 15) & ~(int64_t)15) - (o & ~(int64_t)15));
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, off);
                if (lane == 0) g_mbar_expect_tx(&full[s], mine);
                __syncwarp();
                for (int r = lane; r < ROWS && row0 + r < p.n; r += 32) {
                    int64_t o = (int64_t)(row0 + r) * rb + (int64_t)chunk * kChunkBlocks * B;
                    int64_t a0 = o & ~(int64_t)15;
                    g_bulk_load(base + (size_t)r * WP, p.w + a0, (unsigned)(((o + len + 15) & ~(int64_t)15) - a0), &full[s]);
                }
            }
            unsigned char* acts = base + ROWS * WP;
            float* sc = (float*)(acts + COLS * AP);
            float* aux = sc + COLS * kChunkBlocks;
            for (int i = tid; i < COLS * count * 2; i += THREADS) {
                int c = i / (count * 2), piece = i % (count * 2);
                int col = min(col0 + c, p.m - 1);
                g_cp_async16(acts + c * AP + piece * 16, p.acts.qs + (int64_t)col * k + (int64_t)chunk * kChunkBlocks * 32 + piece * 16);
            }
            for (int i = tid; i < COLS * count; i += THREADS) {
                int c = i / count, j = i % count;
                int col = min(col0 + c, p.m - 1);
                int64_t at = (int64_t)col * nb + chunk * kChunkBlocks + j;
                g_cp_async4(sc + j * COLS + c, p.acts.scales + at);
                if (KIND == TSM_Q4_1) g_cp_async4(aux + j * COLS + c, p.acts.sums + at);
            }
        }
        g_cp_async_commit();
    };

    if (tid == 0) {
        for (int s = 0; s < kGemmStages; s++) g_mbar_init(&full[s], 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
#pragma unroll
    for (int c = 0; c < kGemmStages - 1; c++) issue(c);

    const int wr = warp / WC, wc = warp % WC;
    const int lcol0 = wc * 8 * NT;               // first activation row of this warp within the CTA's slab
    const int ra = 16 * wr + g, rbw = ra + 8;    // this thread's two weight rows within the CTA's slab
    const int64_t start_a = (int64_t)(row0 + ra) * rb, start_b = (int64_t)(row0 + rbw) * rb;

    float acc[NT][4];  // [tile][(row a, col 2t), (row a, col 2t+1), (row b, col 2t), (row b, col 2t+1)]
#pragma unroll
    for (int i = 0; i < NT; i++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[i][e] = 0.0f;

    for (int chunk = 0; chunk < chunks; chunk++) {
        int s = chunk % kGemmStages;
        g_cp_async_wait<kGemmStages - 2>();
        bool arrived = g_mbar_wait(&full[s], (unsigned)((chunk / kGemmStages) & 1));
        if (!arrived) *abort_flag = 1;
        __syncthreads();  // chunk's data is visible, and every thread is done with the previous chunk's stage
        if (*abort_flag) break;
        issue(chunk + kGemmStages - 1);  // refills the stage the previous iteration read
        const unsigned char* base = stages + (size_t)s * STAGE;
        // a chunk of 4 blocks is not always a multiple of 16 bytes, so a row's shift inside its slot can vary by chunk
        int64_t off = (int64_t)chunk * kChunkBlocks * B;
        const unsigned char* slot_a = base + (size_t)ra * WP + (int)((start_a + off) & 15);
        const unsigned char* slot_b = base + (size_t)rbw * WP + (int)((start_b + off) & 15);
        const unsigned char* acts = base + ROWS * WP;
        const float* sc = (const float*)(acts + COLS * AP);
        const float* aux = sc + COLS * kChunkBlocks;
        int count = min(kChunkBlocks, nb - chunk * kChunkBlocks);
#pragma unroll
        for (int j = 0; j < kChunkBlocks; j++) {
            if (j < count) {
                const unsigned char* pa = slot_a + j * B;
                const unsigned char* pb = slot_b + j * B;
                unsigned a0, a1, a2, a3;
                float dwa = half_bits_to_float(lds_u16_at2(pa)), dwb = half_bits_to_float(lds_u16_at2(pb));
                float mwa = 0.0f, mwb = 0.0f;
                if (KIND == TSM_Q8_0) {
                    a0 = lds_u32_at2(pa + 2 + 4 * t), a2 = lds_u32_at2(pa + 18 + 4 * t);
                    a1 = lds_u32_at2(pb + 2 + 4 * t), a3 = lds_u32_at2(pb + 18 + 4 * t);
                } else if (KIND == TSM_Q4_0) {
                    unsigned na = lds_u32_at2(pa + 2 + 4 * t), nbw = lds_u32_at2(pb + 2 + 4 * t);
                    a0 = nibbles_minus_8(na), a2 = nibbles_minus_8(na >> 4);
                    a1 = nibbles_minus_8(nbw), a3 = nibbles_minus_8(nbw >> 4);
                } else {
                    unsigned na = lds_u32_at2(pa + 4 + 4 * t), nbw = lds_u32_at2(pb + 4 + 4 * t);
                    a0 = na & 0x0f0f0f0fu, a2 = (na >> 4) & 0x0f0f0f0fu;
                    a1 = nbw & 0x0f0f0f0fu, a3 = (nbw >> 4) & 0x0f0f0f0fu;
                    mwa = half_bits_to_float(lds_u16_at2(pa + 2)), mwb = half_bits_to_float(lds_u16_at2(pb + 2));
                }
#pragma unroll
                for (int i = 0; i < NT; i++) {
                    const unsigned* xq = (const unsigned*)(acts + (lcol0 + 8 * i + g) * AP + j * 32);
                    int d[4];
                    mma_s8(d, a0, a1, a2, a3, xq[t], xq[4 + t]);
                    int c = lcol0 + 8 * i + 2 * t;
                    float2 dx2 = *(const float2*)(sc + j * COLS + c);
                    float2 sx2 = make_float2(0.0f, 0.0f);
                    if (KIND == TSM_Q4_1) sx2 = *(const float2*)(aux + j * COLS + c);
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        float dx = e == 0 ? dx2.x : dx2.y;
                        float fa = __fsub_rn(__int_as_float(d[e]), 12582912.0f), fb = __fsub_rn(__int_as_float(d[2 + e]), 12582912.0f);
                        if (KIND == TSM_Q8_0) {
                            acc[i][e] = __fadd_rn(acc[i][e], __fmul_rn(fa, __fmul_rn(dwa, dx)));
                            acc[i][2 + e] = __fadd_rn(acc[i][2 + e], __fmul_rn(fb, __fmul_rn(dwb, dx)));
                        } else if (KIND == TSM_Q4_0) {
                            acc[i][e] = __fadd_rn(acc[i][e], __fmul_rn(__fmul_rn(fa, dwa), dx));
                            acc[i][2 + e] = __fadd_rn(acc[i][2 + e], __fmul_rn(__fmul_rn(fb, dwb), dx));
                        } else {
                            float sx = e == 0 ? sx2.x : sx2.y;
                            acc[i][e] = __fadd_rn(acc[i][e], __fadd_rn(__fmul_rn(__fmul_rn(dwa, dx), fa), __fmul_rn(mwa, sx)));
                            acc[i][2 + e] = __fadd_rn(acc[i][2 + e], __fadd_rn(__fmul_rn(__fmul_rn(dwb, dx), fb), __fmul_rn(mwb, sx)));
                        }
                    }
                }
            }
        }
    }
    if (*abort_flag) {
        g_cp_async_wait<0>();
        if (tid == 0) {
            atomicExch(&p.errors->timeout, 1);
            for (int s = 0; s < kGemmStages; s++) g_mbar_wait(&full[s], 0), g_mbar_wait(&full[s], 1);
        }
        return;
    }
    g_cp_async_wait<0>();
#pragma unroll
    for (int i = 0; i < NT; i++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            int row = row0 + (e < 2 ? ra : rbw);
            int col = col0 + lcol0 + 8 * i + 2 * t + (e & 1);
            if (row < p.n && col < p.m) {
                float v = acc[i][e];
                if (p.bias) v = __fadd_rn(v, p.bias[row]);
                if (p.residual) v = __fadd_rn(p.residual[(int64_t)col * p.n + row], v);
                p.out[(int64_t)col * p.n + row] = v;
            }
        }
}

template <int KIND, int NT, int WR, int WC>
int launch_shape(tsm_ctx* ctx, const GemmParams& p) {
    constexpr int B = GFmt<KIND>::B;
    constexpr int ROWS = 16 * WR, COLS = 8 * NT * WC, THREADS = 32 * WR * WC;
    constexpr int kChunkBlocks = chunk_blocks(COLS);
    constexpr int WP = (kChunkBlocks * B + 30 + 15) / 16 * 16, AP = kChunkBlocks * 32 + 16;
    size_t smem = 128 + (size_t)kGemmStages * (ROWS * WP + COLS * AP + 2 * COLS * kChunkBlocks * 4);
    auto kernel = matmul_mma_kernel<KIND, NT, WR, WC>;
    if (smem > 48 * 1024) {
        static std::mutex lock;
        static std::map<std::pair<int, const void*>, bool> done;
        std::lock_guard<std::mutex> guard(lock);
        auto key = std::make_pair(ctx->ordinal, (const void*)kernel);
        if (!done.count(key)) {
            TSM_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            done[key] = true;
        }
    }
    dim3 grid((p.n + ROWS - 1) / ROWS, (p.m + COLS - 1) / COLS);
    TSM_CUDA(ctx, launch_chained(ctx, kernel, grid, dim3(THREADS), smem, p));
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

// The shapes a CTA can take, as WR * 100 + WC * 10 + NT.
template <int KIND>
int launch_config(tsm_ctx* ctx, const GemmParams& p, int config) {
    switch (config) {
        case 418: return launch_shape<KIND, 8, 4, 1>(ctx, p);  // 64 rows x 64 activation rows, 4 warps
        case 818: return launch_shape<KIND, 8, 8, 1>(ctx, p);  // 128 x 64, 8 warps
        case 424: return launch_shape<KIND, 4, 4, 2>(ctx, p);  // 64 x 64, 8 warps
        case 242: return launch_shape<KIND, 2, 2, 4>(ctx, p);  // 32 x 64, 8 warps
        case 224: return launch_shape<KIND, 4, 2, 2>(ctx, p);  // 32 x 64, 4 warps
        case 142: return launch_shape<KIND, 2, 1, 4>(ctx, p);  // 16 x 64, 4 warps
        case 414: return launch_shape<KIND, 4, 4, 1>(ctx, p);  // 64 x 32
        case 422: return launch_shape<KIND, 2, 4, 2>(ctx, p);  // 64 x 32, 8 warps
        case 222: return launch_shape<KIND, 2, 2, 2>(ctx, p);  // 32 x 32
        case 412: return launch_shape<KIND, 2, 4, 1>(ctx, p);  // 64 x 16
        case 421: return launch_shape<KIND, 1, 4, 2>(ctx, p);  // 64 x 16, 8 warps
        case 221: return launch_shape<KIND, 1, 2, 2>(ctx, p);  // 32 x 16
        case 121: return launch_shape<KIND, 1, 1, 2>(ctx, p);  // 16 x 16
        case 411: return launch_shape<KIND, 1, 4, 1>(ctx, p);  // 64 x 8
        case 211: return launch_shape<KIND, 1, 2, 1>(ctx, p);  // 32 x 8
    }
    return fail(ctx, TSM_ERR_ARG, "unknown tensor-core product shape " + std::to_string(config));
}

template <int KIND>
int launch_kind(tsm_ctx* ctx, const GemmParams& p) {
    // TSM_GEMM_CONFIG picks a CTA shape for timing variants without rebuilding (as TENSOMITE_BLOCK_MATMUL does in
    // the reference, quant.cr:36-41)
    static const int forced = getenv("TSM_GEMM_CONFIG") ? atoi(getenv("TSM_GEMM_CONFIG")) : 0;
    if (forced) return launch_config<KIND>(ctx, p, forced);
    // Measured on B200: with many weight rows, tall CTAs (64 rows, one warp per 16 rows over all activation rows)
    // stage the activations least often; with few rows, small CTAs win because more of them hide each other's waits.
    if (p.m <= 8) return launch_config<KIND>(ctx, p, p.n >= 128 * ctx->sm_count ? 411 : 211);
    if (p.m <= 16) return launch_config<KIND>(ctx, p, p.n >= 32 * ctx->sm_count ? 221 : 121);
    if (p.m <= 32) return launch_config<KIND>(ctx, p, p.n >= 64 * ctx->sm_count ? 422 : 222);
    return launch_config<KIND>(ctx, p, p.n >= 128 * ctx->sm_count ? 418 : 142);
}

}  // namespace

// Whether the tensor-core kernel takes this product: 16-byte aligned weights whose total size is a
// multiple of 16 bytes (so that no rounded-up copy reads past the matrix), 4-byte aligned activations.
bool mma_product_fits(const QuantizedActs& a, int rows, int k, const uint8_t* w, int kind, int n) {
    int64_t total = (int64_t)n * (k / 32) * block_bytes(kind);
    return rows >= 1 && ((uintptr_t)w & 15) == 0 && total % 16 == 0 && ((uintptr_t)a.qs & 3) == 0;
}

int launch_block_matmul_mma(tsm_ctx* ctx, const QuantizedActs& a, int rows, int k, const uint8_t* w, int kind, int n,
                            const float* bias, const float* residual, float* out) {
    GemmParams p;
    p.w = w, p.n = n, p.nb = k / 32, p.m = rows, p.acts = a, p.bias = bias, p.residual = residual, p.out = out, p.errors = ctx->errors;
    switch (kind) {
        case TSM_Q8_0: return launch_kind<TSM_Q8_0>(ctx, p);
        case TSM_Q4_0: return launch_kind<TSM_Q4_0>(ctx, p);
        case TSM_Q4_1: return launch_kind<TSM_Q4_1>(ctx, p);
    }
    return fail(ctx, TSM_ERR_UNSUPPORTED, "not a block format");
}

}  // namespace tsm
