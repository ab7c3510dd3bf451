// The quantised product for several rows of activations, as a producer / consumer pipeline.
//
// Same arithmetic and same bits as matmul_mma_kernel (qgemm.cu): one int8 tensor-core instruction
// (mma.sync m16n8k32) gives the exact integer dot products of 16 weight rows with 8 activation rows for one
// 32-element block, and the thread that holds a (weight row, activation row) pair folds the block's float
// contribution into its running sum, block after block (Quant.matmul_reference, quant.cr:122-142).
//
// What differs is how the operands reach the multiply:
//   * one producer thread per CTA moves a whole stage (8 blocks of K) with four or five tiled tensor copies
//     (cp.async.bulk.tensor.2d through tensor maps): the CTA's weight rows as one box of the block matrix, the
//     quantised activations as two boxes of 128 bytes x 64 rows written with the 128-byte swizzle, their scales as
//     one box.  Copies complete on a "full" mbarrier per stage; consumer warps release a stage through an "empty"
//     mbarrier.  The main loop has no CTA-wide barrier and the consumer warps issue no copies.  (One copy per
//     weight row and chunk, as matmul_mma_kernel does, is bounded by the rate at which an SM issues small bulk
//     copies: about one per 30 ns measured.)
//   * a CTA takes ALL activation rows (up to 64) and as many groups of 16 weight rows as keep every SM equally
//     loaded, so a stage of activations is staged once per SM and used by every consumer warp;
//   * a consumer warp prepares the weight fragments of 4 blocks, then walks its tiles of 8 activation rows with
//     the 4 blocks innermost: the activation scales of a tile arrive as one 16-byte load per column, and the
//     int -> float conversion of the dot product is folded into the first multiply (Q4_0); activation fragments come
//     by ldmatrix, four 8 x 16-byte pieces per instruction.
// matmul_pipe_t_kernel is the same pipeline with the operands' roles exchanged (8 weight rows as the multiply's B
// operand, 16 activation rows as A), for matrices with too few rows to give every SM enough 16-row groups.
//
// Shapes this kernel does not take (blocks per row not a multiple of 8, unaligned operands) stay with
// matmul_mma_kernel.
#include <stdlib.h>

#include <type_traits>

#include "common.cuh"

namespace tsm {

namespace {

constexpr int kPipeStages = 4;
constexpr unsigned kPipeSpins = 4u << 20;
constexpr int kSub = 4;  // blocks whose weight fragments a warp holds at once

template <int KIND> struct PFmt;
template <> struct PFmt<TSM_Q8_0> { static constexpr int B = 34; };
template <> struct PFmt<TSM_Q4_0> { static constexpr int B = 18; };
template <> struct PFmt<TSM_Q4_1> { static constexpr int B = 20; };

struct PipeParams {
    const uint8_t* w;
    int n, nb, m;          // weight rows, blocks per row, activation rows
    int groups;            // ceil(n / 16)
    QuantizedActs acts;
    const float* bias;
    const float* residual;
    float* out;            // [m, n]
    ErrorRecord* errors;
    unsigned spins;        // polls after which a wait gives up
    int skip_chunks;       // stages the producer leaves out at the end (0 but for tsm_debug_wait_limit's test of the waits)
    unsigned wait_hint;    // nanoseconds a waiting thread may sleep per poll (0: plain polling)
};

__device__ __forceinline__ unsigned p_smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void p_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(p_smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void p_mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(p_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void p_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(p_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool p_mbar_try_wait(uint64_t* bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(p_smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded: gives up after `limit` polls (kPipeSpins unless a test lowered it), or as soon as another warp has raised the
// CTA's abort flag.
__device__ __forceinline__ bool p_mbar_try_wait_sleeping(uint64_t* bar, unsigned parity, unsigned hint_ns) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(p_smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
// abort_flag[2] holds the suspend hint in nanoseconds: with one, a poll may sleep until the phase completes, which leaves
// the waiting warp's issue slots to the warps that have work (0: plain polling).
__device__ __forceinline__ bool p_mbar_wait(uint64_t* bar, unsigned parity, volatile int* abort_flag, unsigned limit) {
    if (p_mbar_try_wait(bar, parity)) return true;
    const unsigned hint = (unsigned)abort_flag[2];
    for (unsigned spin = 0; spin < limit; spin++) {
        if (hint ? p_mbar_try_wait_sleeping(bar, parity, hint) : p_mbar_try_wait(bar, parity)) return true;
        if (hint || spin > 1024) {
            if (*abort_flag) return false;
            if (!hint) __nanosleep(64);
        }
    }
    return false;
}
__device__ __forceinline__ void p_tensor_load(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     p_smem_u32(dst)),
                 "l"(map), "r"(x), "r"(y), "r"(p_smem_u32(bar))
                 : "memory");
}

// The 4 bytes at p (2-byte aligned, in shared memory) as a little-endian word.
__device__ __forceinline__ unsigned p_lds_u32_at2(const unsigned char* p) {
    // through the 32-bit shared address: a pointer rebuilt from an integer would be a generic one, and its loads generic loads
    const unsigned a = p_smem_u32(p);
    unsigned lo, hi;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(lo) : "r"(a & ~3u));
    asm volatile("ld.shared.u32 %0, [%1 + 4];" : "=r"(hi) : "r"(a & ~3u));
    return __funnelshift_r(lo, hi, (a & 3u) * 8);
}
__device__ __forceinline__ unsigned p_lds_u16(const unsigned char* p) { return *(const unsigned short*)p; }

// Nibbles 0..15 in the low half of each byte of x -> signed bytes nibble - 8, without touching neighbours.
__device__ __forceinline__ unsigned p_nibbles_minus_8(unsigned x) { return (((x & 0x0f0f0f0fu) | 0x80808080u) - 0x08080808u) ^ 0x80808080u; }

constexpr float kMagic = 12582912.0f;  // 1.5 * 2^23: an int32 accumulator started at this float's bits reads back as kMagic + dot

// d = C + A * B with the accumulator input C given as four registers that the caller keeps alive across calls.
__device__ __forceinline__ void p_mma_s8(int (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1, const int (&c)[4]) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};\n"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}

// Four 8-row x 16-byte pieces of shared memory as tensor-core fragments: lane l gives the address of row l % 8 of piece
// l / 8 and receives, from each piece, the 4 bytes its place in the fragment holds.
__device__ __forceinline__ void p_ldmatrix4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}

constexpr int kCB = 8;  // blocks of K per stage

template <int KIND, int COLS>
struct PipeLayout {
    static constexpr int B = PFmt<KIND>::B;
    static constexpr int WP = kCB * B;                       // a weight row's chunk, dense: 144, 272 or 160 bytes
    static constexpr int ABOX = COLS * 128;                  // one swizzled box of activations: 4 blocks x COLS rows
    static constexpr int SP = kCB * 4;                       // scales of one activation row
    static constexpr int SCALE_BYTES = COLS * SP * (KIND == TSM_Q4_1 ? 2 : 1);
    __host__ __device__ static constexpr int weights_at() { return 2 * ABOX; }
    // `rows` = weight rows a CTA stages; the scale box wants a 256-byte boundary (its swizzle pattern's period)
    __host__ __device__ static constexpr int scales_at(int rows) { return (2 * ABOX + rows * WP + 255) / 256 * 256; }
    __host__ __device__ static constexpr int stage_bytes(int rows) { return (scales_at(rows) + SCALE_BYTES + 1023) / 1024 * 1024; }
};

struct PipeMaps {
    CUtensorMap weights;  // u16 [n, nb * B / 2], box (kCB * B / 2) x (16 * groups per CTA)
    CUtensorMap acts;     // u8 [m, k], box 128 x COLS, 128-byte swizzle
    CUtensorMap scales;   // f32 [m, nb], box kCB x COLS, 32-byte swizzle (a warp's 16-byte reads then fall in distinct banks)
    CUtensorMap sums;     // the same over the block sums (Q4_1)
};

// A consumer warp owns one group of 16 weight rows and NT tiles of 8 activation rows (from tile wc * NT); the
// CTA has `wr_max` groups x WC such warps plus one producer warp (the last).  CTA b takes the groups
// [b * groups / gridDim.x, (b + 1) * groups / gridDim.x): at most wr_max of them by the host's choice of grid.
template <int KIND, int NT, int WC>
__global__ void __launch_bounds__(512, 1) matmul_pipe_kernel(PipeParams p, int wr_max, const __grid_constant__ PipeMaps maps) {
    chained_kernel_entry();
    constexpr int COLS = 8 * NT * WC;
    using L = PipeLayout<KIND, COLS>;
    constexpr int B = L::B, WP = L::WP;
    extern __shared__ unsigned char smem_raw[];
    // the swizzled boxes need 1024-byte alignment: barriers sit in the first 128 bytes, stages start at the next 1024
    unsigned char* smem = smem_raw + ((1024u - (p_smem_u32(smem_raw) & 1023u)) & 1023u);  // an offset from the shared array: the address space stays known
    uint64_t* full = (uint64_t*)smem;                 // [kPipeStages]
    uint64_t* empty = full + kPipeStages;             // [kPipeStages]
    volatile int* abort_flag = (volatile int*)(smem + 96);
    unsigned char* stages = smem + 1024;
    const int stage_bytes = L::stage_bytes(wr_max * 16);
    const int scales_at = L::scales_at(wr_max * 16);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nb = p.nb;
    const int group0 = (int)((int64_t)blockIdx.x * p.groups / gridDim.x);
    const int group_count = (int)((int64_t)(blockIdx.x + 1) * p.groups / gridDim.x) - group0;
    const int col0 = blockIdx.y * COLS;
    const int valid = min(COLS, p.m - col0);          // activation rows this CTA really has
    const int active_wc = min(WC, (valid + 8 * NT - 1) / (8 * NT));
    const int chunks = nb / kCB;
    const int producer_warp = wr_max * WC;

    if (tid == 0) {
        for (int s = 0; s < kPipeStages; s++) {
            p_mbar_init(&full[s], 1);
            p_mbar_init(&empty[s], group_count * active_wc);
        }
        abort_flag[0] = 0, abort_flag[1] = 0, abort_flag[2] = (int)p.wait_hint, abort_flag[3] = 0;  // [1] stays 0: a wait that must not be cut short polls it
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == producer_warp) {
        // ---------------------------------------------------------------- producer: one thread
        if (lane != 0) return;
        // a box that reaches past the matrix is filled with zeros and still counts in full
        const unsigned tx = (unsigned)(2 * L::ABOX + wr_max * 16 * WP + L::SCALE_BYTES);
        int issued = 0;
        bool ok = true;
        for (int chunk = 0; chunk < chunks - p.skip_chunks; chunk++) {
            int s = chunk % kPipeStages;
            if (chunk >= kPipeStages) ok = p_mbar_wait(&empty[s], (unsigned)((chunk / kPipeStages - 1) & 1), abort_flag, p.spins);
            if (!ok) break;
            unsigned char* base = stages + (size_t)s * stage_bytes;
            p_mbar_expect_tx(&full[s], tx);
            p_tensor_load(base, &maps.acts, chunk * kCB * 32, col0, &full[s]);
            p_tensor_load(base + L::ABOX, &maps.acts, chunk * kCB * 32 + 128, col0, &full[s]);
            p_tensor_load(base + L::weights_at(), &maps.weights, chunk * (kCB * B / 2), group0 * 16, &full[s]);
            p_tensor_load(base + scales_at, &maps.scales, chunk * kCB, col0, &full[s]);
            if (KIND == TSM_Q4_1) p_tensor_load(base + scales_at + COLS * L::SP, &maps.sums, chunk * kCB, col0, &full[s]);
            issued = chunk + 1;
        }
        if (!ok) {
            // a consumer stopped arriving: say so, then see the copies already issued land before leaving
            *abort_flag = 1;
            atomicExch(&p.errors->timeout, 1);
            for (int chunk = max(0, issued - kPipeStages); chunk < issued; chunk++)
                p_mbar_wait(&full[chunk % kPipeStages], (unsigned)((chunk / kPipeStages) & 1), abort_flag + 1, p.spins);
        }
        return;
    }

    // -------------------------------------------------------------------- consumers
    const int wr = warp / WC, wc = warp % WC;
    if (wr >= group_count || wc >= active_wc) return;
    const int g = lane >> 2, t = lane & 3;
    const int lcol0 = wc * 8 * NT;
    const int my_tiles = min(NT, (valid - lcol0 + 7) / 8);
    const int row0 = (group0 + wr) * 16;
    const int ra = wr * 16 + g, rbw = ra + 8;         // this thread's two weight rows within the CTA's box
    // The activation fragments of two blocks of a tile are four 8 x 16-byte pieces: (block, low half), (block, high
    // half), (block + 1, low), (block + 1, high); lane l addresses row l % 8 of piece l / 8, whose 16 bytes (piece
    // 2 u + half of the row's 128) are stored at piece ^ (row & 7).
    unsigned frag_at[kSub / 2];
#pragma unroll
    for (int pair = 0; pair < kSub / 2; pair++)
        frag_at[pair] = (unsigned)((lcol0 + (lane & 7)) * 128 + (((4 * pair + (lane >> 3)) ^ (lane & 7)) << 4));

    int cq[4];  // the accumulator input of every multiply: four registers holding kMagic's bits, set once
#pragma unroll
    for (int e = 0; e < 4; e++) asm volatile("mov.b32 %0, 0x4b400000;" : "=r"(cq[e]));

    float acc[NT][4];  // [tile][(row a, col 2t), (row a, col 2t+1), (row b, col 2t), (row b, col 2t+1)]
#pragma unroll
    for (int i = 0; i < NT; i++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[i][e] = 0.0f;

    bool ok = true;
    for (int chunk = 0; chunk < chunks; chunk++) {
        int s = chunk % kPipeStages;
        ok = p_mbar_wait(&full[s], (unsigned)((chunk / kPipeStages) & 1), abort_flag, p.spins);
        if (!ok) break;
        const unsigned char* base = stages + (size_t)s * stage_bytes;
        const unsigned char* slot_a = base + L::weights_at() + (size_t)ra * WP;
        const unsigned char* slot_b = base + L::weights_at() + (size_t)rbw * WP;
        const float* sc = (const float*)(base + scales_at);
        const float* aux = sc + COLS * kCB;
#pragma unroll
        for (int sub = 0; sub < kCB / kSub; sub++) {
            const unsigned char* abox = base + sub * L::ABOX;
            unsigned a[kSub][4];
            float dwa[kSub], dwb[kSub], xa[kSub], xb[kSub];  // xa/xb: Q4_0 -kMagic * dw; Q4_1 the block minimum
            bool plain = true;
#pragma unroll
            for (int u = 0; u < kSub; u++) {
                const unsigned char* pa = slot_a + (sub * kSub + u) * B;
                const unsigned char* pb = slot_b + (sub * kSub + u) * B;
                dwa[u] = half_bits_to_float(p_lds_u16(pa)), dwb[u] = half_bits_to_float(p_lds_u16(pb));
                if (KIND == TSM_Q8_0) {
                    a[u][0] = p_lds_u32_at2(pa + 2 + 4 * t), a[u][2] = p_lds_u32_at2(pa + 18 + 4 * t);
                    a[u][1] = p_lds_u32_at2(pb + 2 + 4 * t), a[u][3] = p_lds_u32_at2(pb + 18 + 4 * t);
                    xa[u] = xb[u] = 0.0f;
                } else if (KIND == TSM_Q4_0) {
                    unsigned na = p_lds_u32_at2(pa + 2 + 4 * t), nbw = p_lds_u32_at2(pb + 2 + 4 * t);
                    a[u][0] = p_nibbles_minus_8(na), a[u][2] = p_nibbles_minus_8(na >> 4);
                    a[u][1] = p_nibbles_minus_8(nbw), a[u][3] = p_nibbles_minus_8(nbw >> 4);
                    xa[u] = __fmul_rn(-kMagic, dwa[u]), xb[u] = __fmul_rn(-kMagic, dwb[u]);
                    plain = plain && fabsf(dwa[u]) <= 65504.0f && fabsf(dwb[u]) <= 65504.0f;
                } else {
                    unsigned na = p_lds_u32_at2(pa + 4 + 4 * t), nbw = p_lds_u32_at2(pb + 4 + 4 * t);
                    a[u][0] = na & 0x0f0f0f0fu, a[u][2] = (na >> 4) & 0x0f0f0f0fu;
                    a[u][1] = nbw & 0x0f0f0f0fu, a[u][3] = (nbw >> 4) & 0x0f0f0f0fu;
                    xa[u] = half_bits_to_float(p_lds_u16(pa + 2)), xb[u] = half_bits_to_float(p_lds_u16(pb + 2));
                }
            }
            // Q4_0: (float(dot) * dw) * dx with float(dot) * dw taken as fma(kMagic + dot, dw, -kMagic * dw): both
            // products are exact (dw has 11 significant bits), so the one rounding is that of dot * dw.  With a
            // scale that is not finite the fused form would give NaN where the reference gives an infinity, so
            // such a group of blocks takes the subtract-then-multiply form instead.
            const bool all_plain = KIND == TSM_Q4_0 && __all_sync(0xffffffffu, plain);
            // the tile loop exists twice, behind a real branch: as one loop with the choice inside, both forms
            // were issued for every element and one of them predicated off
            auto tiles = [&](auto fused_tag) {
            constexpr bool fused = decltype(fused_tag)::value;
#pragma unroll
            for (int i = 0; i < NT; i++) {
                if (i < my_tiles) {
                    const int c = lcol0 + 8 * i + 2 * t;
                    // scales are stored with the 32-byte swizzle: the half (blocks 0-3 or 4-7) of column c sits at
                    // half ^ bit 2 of c, which for columns 8 i + 2 t (+ 1) is bit 1 of t
                    const int half = (sub ^ (t >> 1)) * kSub;
                    const float4 s0 = *(const float4*)(sc + c * kCB + half);
                    const float4 s1 = *(const float4*)(sc + (c + 1) * kCB + half);
                    float4 m0 = make_float4(0.f, 0.f, 0.f, 0.f), m1 = m0;
                    if (KIND == TSM_Q4_1) {
                        m0 = *(const float4*)(aux + c * kCB + half);
                        m1 = *(const float4*)(aux + (c + 1) * kCB + half);
                    }
                    const unsigned tile = p_smem_u32(abox) + i * 1024;
                    unsigned xq[kSub / 2][4];
#pragma unroll
                    for (int pair = 0; pair < kSub / 2; pair++) p_ldmatrix4(xq[pair], tile + frag_at[pair]);
#pragma unroll
                    for (int u = 0; u < kSub; u++) {
                        int d[4];
                        p_mma_s8(d, a[u], xq[u >> 1][2 * (u & 1)], xq[u >> 1][2 * (u & 1) + 1], cq);
                        const float dx0 = u == 0 ? s0.x : u == 1 ? s0.y : u == 2 ? s0.z : s0.w;
                        const float dx1 = u == 0 ? s1.x : u == 1 ? s1.y : u == 2 ? s1.z : s1.w;
#pragma unroll
                        for (int e = 0; e < 2; e++) {
                            const float dx = e == 0 ? dx0 : dx1;
                            const float fa_bits = __int_as_float(d[e]), fb_bits = __int_as_float(d[2 + e]);
                            if (KIND == TSM_Q8_0) {
                                float fa = __fsub_rn(fa_bits, kMagic), fb = __fsub_rn(fb_bits, kMagic);
                                acc[i][e] = __fadd_rn(acc[i][e], __fmul_rn(fa, __fmul_rn(dwa[u], dx)));
                                acc[i][2 + e] = __fadd_rn(acc[i][2 + e], __fmul_rn(fb, __fmul_rn(dwb[u], dx)));
                            } else if (KIND == TSM_Q4_0) {
                                float pa, pb;
                                if (fused) {
                                    pa = __fmaf_rn(fa_bits, dwa[u], xa[u]), pb = __fmaf_rn(fb_bits, dwb[u], xb[u]);
                                } else {
                                    pa = __fmul_rn(__fsub_rn(fa_bits, kMagic), dwa[u]), pb = __fmul_rn(__fsub_rn(fb_bits, kMagic), dwb[u]);
                                }
                                acc[i][e] = __fadd_rn(acc[i][e], __fmul_rn(pa, dx));
                                acc[i][2 + e] = __fadd_rn(acc[i][2 + e], __fmul_rn(pb, dx));
                            } else {
                                const float sx = e == 0 ? (u == 0 ? m0.x : u == 1 ? m0.y : u == 2 ? m0.z : m0.w)
                                                        : (u == 0 ? m1.x : u == 1 ? m1.y : u == 2 ? m1.z : m1.w);
                                float fa = __fsub_rn(fa_bits, kMagic), fb = __fsub_rn(fb_bits, kMagic);
                                acc[i][e] = __fadd_rn(acc[i][e], __fadd_rn(__fmul_rn(__fmul_rn(dwa[u], dx), fa), __fmul_rn(xa[u], sx)));
                                acc[i][2 + e] = __fadd_rn(acc[i][2 + e], __fadd_rn(__fmul_rn(__fmul_rn(dwb[u], dx), fb), __fmul_rn(xb[u], sx)));
                            }
                        }
                    }
                }
            }
            };
            if (all_plain) tiles(std::true_type{});
            else tiles(std::false_type{});
        }
        __syncwarp();
        if (lane == 0) p_mbar_arrive(&empty[s]);
    }
    if (!ok) {
        *abort_flag = 1;
        if (lane == 0) atomicExch(&p.errors->timeout, 1);
        return;
    }
#pragma unroll
    for (int i = 0; i < NT; i++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            int row = row0 + g + (e < 2 ? 0 : 8);
            int col = col0 + lcol0 + 8 * i + 2 * t + (e & 1);
            if (row < p.n && col < p.m) {
                float v = acc[i][e];
                if (p.bias) v = __fadd_rn(v, p.bias[row]);
                if (p.residual) v = __fadd_rn(p.residual[(int64_t)col * p.n + row], v);
                p.out[(int64_t)col * p.n + row] = v;
            }
        }
}


// The same pipeline with the operands' roles exchanged, for matrices with few rows: the multiply takes 16 ACTIVATION
// rows as its A operand and 8 WEIGHT rows as its B operand, so a warp's group is 8 weight rows (twice as many groups
// to spread over the SMs) and a weight fragment is one word per lane and block, prepared once and used for all the
// warp's MT tiles of 16 activation rows.  A thread then holds the outputs of activation rows g, g + 8 and weight rows
// 2t, 2t + 1 of each tile; every output's blocks are still folded in block order.
template <int KIND, int MT, int WC>
__global__ void __launch_bounds__(512, 1) matmul_pipe_t_kernel(PipeParams p, int wr_max, const __grid_constant__ PipeMaps maps) {
    chained_kernel_entry();
    constexpr int COLS = 16 * MT * WC;
    using L = PipeLayout<KIND, COLS>;
    constexpr int B = L::B, WP = L::WP;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (p_smem_u32(smem_raw) & 1023u)) & 1023u);  // an offset from the shared array: the address space stays known
    uint64_t* full = (uint64_t*)smem;
    uint64_t* empty = full + kPipeStages;
    volatile int* abort_flag = (volatile int*)(smem + 96);
    unsigned char* stages = smem + 1024;
    const int stage_bytes = L::stage_bytes(wr_max * 8);
    const int scales_at = L::scales_at(wr_max * 8);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nb = p.nb;
    const int groups = (p.n + 7) / 8;
    const int group0 = (int)((int64_t)blockIdx.x * groups / gridDim.x);
    const int group_count = (int)((int64_t)(blockIdx.x + 1) * groups / gridDim.x) - group0;
    const int col0 = blockIdx.y * COLS;
    const int valid = min(COLS, p.m - col0);
    const int active_wc = min(WC, (valid + 16 * MT - 1) / (16 * MT));
    const int chunks = nb / kCB;
    const int producer_warp = wr_max * WC;

    if (tid == 0) {
        for (int s = 0; s < kPipeStages; s++) {
            p_mbar_init(&full[s], 1);
            p_mbar_init(&empty[s], group_count * active_wc);
        }
        abort_flag[0] = 0, abort_flag[1] = 0, abort_flag[2] = (int)p.wait_hint, abort_flag[3] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == producer_warp) {
        if (lane != 0) return;
        const unsigned tx = (unsigned)(2 * L::ABOX + wr_max * 8 * WP + L::SCALE_BYTES);
        int issued = 0;
        bool ok = true;
        for (int chunk = 0; chunk < chunks - p.skip_chunks; chunk++) {
            int s = chunk % kPipeStages;
            if (chunk >= kPipeStages) ok = p_mbar_wait(&empty[s], (unsigned)((chunk / kPipeStages - 1) & 1), abort_flag, p.spins);
            if (!ok) break;
            unsigned char* base = stages + (size_t)s * stage_bytes;
            p_mbar_expect_tx(&full[s], tx);
            p_tensor_load(base, &maps.acts, chunk * kCB * 32, col0, &full[s]);
            p_tensor_load(base + L::ABOX, &maps.acts, chunk * kCB * 32 + 128, col0, &full[s]);
            p_tensor_load(base + L::weights_at(), &maps.weights, chunk * (kCB * B / 2), group0 * 8, &full[s]);
            p_tensor_load(base + scales_at, &maps.scales, chunk * kCB, col0, &full[s]);
            if (KIND == TSM_Q4_1) p_tensor_load(base + scales_at + COLS * L::SP, &maps.sums, chunk * kCB, col0, &full[s]);
            issued = chunk + 1;
        }
        if (!ok) {
            *abort_flag = 1;
            atomicExch(&p.errors->timeout, 1);
            for (int chunk = max(0, issued - kPipeStages); chunk < issued; chunk++)
                p_mbar_wait(&full[chunk % kPipeStages], (unsigned)((chunk / kPipeStages) & 1), abort_flag + 1, p.spins);
        }
        return;
    }

    const int wr = warp / WC, wc = warp % WC;
    if (wr >= group_count || wc >= active_wc) return;
    const int g = lane >> 2, t = lane & 3;
    const int lcol0 = wc * 16 * MT;
    const int my_tiles = min(MT, (valid - lcol0 + 15) / 16);
    const int row0 = (group0 + wr) * 8;
    // A block's activation fragment of a tile is four 8 x 16-byte pieces: (rows 0-7, low half), (rows 8-15, low), (rows
    // 0-7, high), (rows 8-15, high); lane l addresses row l % 8 of piece l / 8; the 16 bytes (piece 2 u + half of the
    // row's 128) are stored at piece ^ (row & 7).
    unsigned frag_at[kSub];
#pragma unroll
    for (int u = 0; u < kSub; u++)
        frag_at[u] = (unsigned)((lcol0 + (lane & 7) + 8 * ((lane >> 3) & 1)) * 128 + (((2 * u + (lane >> 4)) ^ (lane & 7)) << 4));
    const int scale_half = (g >> 2) & 1;  // the 32-byte swizzle of the scale box: bit 2 of the activation row

    int cq[4];
#pragma unroll
    for (int e = 0; e < 4; e++) asm volatile("mov.b32 %0, 0x4b400000;" : "=r"(cq[e]));

    float acc[MT][4];  // [tile][(act g, weight 2t), (act g, weight 2t+1), (act g+8, weight 2t), (act g+8, weight 2t+1)]
#pragma unroll
    for (int i = 0; i < MT; i++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[i][e] = 0.0f;

    bool ok = true;
    for (int chunk = 0; chunk < chunks; chunk++) {
        int s = chunk % kPipeStages;
        ok = p_mbar_wait(&full[s], (unsigned)((chunk / kPipeStages) & 1), abort_flag, p.spins);
        if (!ok) break;
        const unsigned char* base = stages + (size_t)s * stage_bytes;
        const unsigned char* wbase = base + L::weights_at() + (size_t)(wr * 8) * WP;
        const unsigned char* slot_q = wbase + (size_t)g * WP;            // the row whose quantised values this lane feeds
        const unsigned char* slot_0 = wbase + (size_t)(2 * t) * WP;      // the two rows whose outputs this lane holds
        const unsigned char* slot_1 = slot_0 + WP;
        const float* sc = (const float*)(base + scales_at);
        const float* aux = sc + COLS * kCB;
#pragma unroll
        for (int sub = 0; sub < kCB / kSub; sub++) {
            const unsigned char* abox = base + sub * L::ABOX;
            unsigned b[kSub][2];
            float dw0[kSub], dw1[kSub], x0[kSub], x1[kSub];  // x: Q4_0 -kMagic * dw; Q4_1 the block minimum
            bool plain = true;
#pragma unroll
            for (int u = 0; u < kSub; u++) {
                const int at = (sub * kSub + u) * B;
                dw0[u] = half_bits_to_float(p_lds_u16(slot_0 + at)), dw1[u] = half_bits_to_float(p_lds_u16(slot_1 + at));
                if (KIND == TSM_Q8_0) {
                    b[u][0] = p_lds_u32_at2(slot_q + at + 2 + 4 * t), b[u][1] = p_lds_u32_at2(slot_q + at + 18 + 4 * t);
                    x0[u] = x1[u] = 0.0f;
                } else if (KIND == TSM_Q4_0) {
                    unsigned nq = p_lds_u32_at2(slot_q + at + 2 + 4 * t);
                    b[u][0] = p_nibbles_minus_8(nq), b[u][1] = p_nibbles_minus_8(nq >> 4);
                    x0[u] = __fmul_rn(-kMagic, dw0[u]), x1[u] = __fmul_rn(-kMagic, dw1[u]);
                    plain = plain && fabsf(dw0[u]) <= 65504.0f && fabsf(dw1[u]) <= 65504.0f;
                } else {
                    unsigned nq = p_lds_u32_at2(slot_q + at + 4 + 4 * t);
                    b[u][0] = nq & 0x0f0f0f0fu, b[u][1] = (nq >> 4) & 0x0f0f0f0fu;
                    x0[u] = half_bits_to_float(p_lds_u16(slot_0 + at + 2)), x1[u] = half_bits_to_float(p_lds_u16(slot_1 + at + 2));
                }
            }
            const bool all_plain = KIND == TSM_Q4_0 && __all_sync(0xffffffffu, plain);
            auto tiles = [&](auto fused_tag) {
                constexpr bool fused = decltype(fused_tag)::value;
#pragma unroll
                for (int i = 0; i < MT; i++) {
                    if (i < my_tiles) {
                        const int r_lo = lcol0 + 16 * i + g;  // activation rows r_lo and r_lo + 8
                        const int half = (sub ^ scale_half) * kSub;
                        const float4 s_lo = *(const float4*)(sc + r_lo * kCB + half);
                        const float4 s_hi = *(const float4*)(sc + (r_lo + 8) * kCB + half);
                        float4 m_lo = make_float4(0.f, 0.f, 0.f, 0.f), m_hi = m_lo;
                        if (KIND == TSM_Q4_1) {
                            m_lo = *(const float4*)(aux + r_lo * kCB + half);
                            m_hi = *(const float4*)(aux + (r_lo + 8) * kCB + half);
                        }
                        const unsigned tile = p_smem_u32(abox) + i * 2048;
#pragma unroll
                        for (int u = 0; u < kSub; u++) {
                            unsigned a[4];
                            p_ldmatrix4(a, tile + frag_at[u]);
                            int d[4];
                            p_mma_s8(d, a, b[u][0], b[u][1], cq);
                            const float dx_lo = u == 0 ? s_lo.x : u == 1 ? s_lo.y : u == 2 ? s_lo.z : s_lo.w;
                            const float dx_hi = u == 0 ? s_hi.x : u == 1 ? s_hi.y : u == 2 ? s_hi.z : s_hi.w;
#pragma unroll
                            for (int e = 0; e < 4; e++) {
                                const float dx = e < 2 ? dx_lo : dx_hi;
                                const float dw = (e & 1) ? dw1[u] : dw0[u];
                                const float xw = (e & 1) ? x1[u] : x0[u];
                                const float bits = __int_as_float(d[e]);
                                if (KIND == TSM_Q8_0) {
                                    acc[i][e] = __fadd_rn(acc[i][e], __fmul_rn(__fsub_rn(bits, kMagic), __fmul_rn(dw, dx)));
                                } else if (KIND == TSM_Q4_0) {
                                    float scaled = fused ? __fmaf_rn(bits, dw, xw) : __fmul_rn(__fsub_rn(bits, kMagic), dw);
                                    acc[i][e] = __fadd_rn(acc[i][e], __fmul_rn(scaled, dx));
                                } else {
                                    const float4& mm = e < 2 ? m_lo : m_hi;
                                    const float sx = u == 0 ? mm.x : u == 1 ? mm.y : u == 2 ? mm.z : mm.w;
                                    acc[i][e] = __fadd_rn(acc[i][e], __fadd_rn(__fmul_rn(__fmul_rn(dw, dx), __fsub_rn(bits, kMagic)), __fmul_rn(xw, sx)));
                                }
                            }
                        }
                    }
                }
            };
            if (all_plain) tiles(std::true_type{});
            else tiles(std::false_type{});
        }
        __syncwarp();
        if (lane == 0) p_mbar_arrive(&empty[s]);
    }
    if (!ok) {
        *abort_flag = 1;
        if (lane == 0) atomicExch(&p.errors->timeout, 1);
        return;
    }
#pragma unroll
    for (int i = 0; i < MT; i++)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            int row = row0 + 2 * t + (e & 1);
            int col = col0 + lcol0 + 16 * i + g + (e < 2 ? 0 : 8);
            if (row < p.n && col < p.m) {
                float v = acc[i][e];
                if (p.bias) v = __fadd_rn(v, p.bias[row]);
                if (p.residual) v = __fadd_rn(p.residual[(int64_t)col * p.n + row], v);
                p.out[(int64_t)col * p.n + row] = v;
            }
        }
}

template <int KIND, int NT, int WC>
int launch_pipe_shape(tsm_ctx* ctx, PipeParams p, int ctas_per_sm_forced) {
    constexpr int COLS = 8 * NT * WC;
    using L = PipeLayout<KIND, COLS>;
    constexpr int B = L::B;
    constexpr size_t kSmemBudget = 224 * 1024;
    auto smem_for = [](int groups) { return (size_t)2048 + (size_t)kPipeStages * L::stage_bytes(groups * 16); };
    const int wr_cap = 15 / WC;  // 15 consumer warps and the producer: 512 threads
    int wr_max = 0, grid_x = 0;
    // the fewest CTAs per SM whose share of the weight-row groups fits a CTA; every SM then gets the same share
    for (int c = 1; c <= 4 && !wr_max; c++) {
        if (ctas_per_sm_forced && c != ctas_per_sm_forced) continue;
        int gx = std::min(p.groups, ctx->sm_count * c);
        int need = (p.groups + gx - 1) / gx;
        if (need <= wr_cap && smem_for(need) * c <= kSmemBudget && 32 * (need * WC + 1) * c <= 512) wr_max = need, grid_x = gx;
    }
    if (!wr_max) {
        wr_max = wr_cap;
        while (wr_max > 1 && smem_for(wr_max) > kSmemBudget) wr_max--;
        grid_x = (p.groups + wr_max - 1) / wr_max;
    }
    size_t smem = smem_for(wr_max);
    auto kernel = matmul_pipe_kernel<KIND, NT, WC>;
    {
        static std::mutex lock;
        static std::map<std::pair<int, const void*>, bool> done;
        std::lock_guard<std::mutex> guard(lock);
        auto key = std::make_pair(ctx->ordinal, (const void*)kernel);
        if (!done.count(key)) {
            TSM_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            done[key] = true;
        }
    }
    PipeMaps maps;
    const uint64_t nb = (uint64_t)p.nb;
    TSM_TRY(make_tensor_map_2d(ctx, &maps.weights, CU_TENSOR_MAP_DATA_TYPE_UINT16, p.w, nb * B / 2, (uint64_t)p.n, nb * B, kCB * B / 2, 16 * wr_max,
                     CU_TENSOR_MAP_SWIZZLE_NONE));
    TSM_TRY(make_tensor_map_2d(ctx, &maps.acts, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.acts.qs, nb * 32, (uint64_t)p.m, nb * 32, 128, COLS,
                     CU_TENSOR_MAP_SWIZZLE_128B));
    TSM_TRY(make_tensor_map_2d(ctx, &maps.scales, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p.acts.scales, nb, (uint64_t)p.m, nb * 4, kCB, COLS,
                     CU_TENSOR_MAP_SWIZZLE_32B));
    TSM_TRY(make_tensor_map_2d(ctx, &maps.sums, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, KIND == TSM_Q4_1 ? p.acts.sums : p.acts.scales, nb, (uint64_t)p.m, nb * 4,
                     kCB, COLS, CU_TENSOR_MAP_SWIZZLE_32B));
    dim3 grid(grid_x, (p.m + COLS - 1) / COLS);
    TSM_CUDA(ctx, launch_chained(ctx, kernel, grid, dim3(32 * (wr_max * WC + 1)), smem, p, wr_max, maps));
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

// The role-swapped kernel's launch: groups of 8 weight rows, tiles of 16 activation rows.
template <int KIND, int MT, int WC>
int launch_pipe_t_shape(tsm_ctx* ctx, PipeParams p, int ctas_per_sm_forced) {
    constexpr int COLS = 16 * MT * WC;
    using L = PipeLayout<KIND, COLS>;
    constexpr int B = L::B;
    constexpr size_t kSmemBudget = 224 * 1024;
    auto smem_for = [](int groups) { return (size_t)2048 + (size_t)kPipeStages * L::stage_bytes(groups * 8); };
    const int groups = (p.n + 7) / 8;
    const int wr_cap = 15 / WC;
    int wr_max = 0, grid_x = 0;
    for (int c = 1; c <= 4 && !wr_max; c++) {
        if (ctas_per_sm_forced && c != ctas_per_sm_forced) continue;
        int gx = std::min(groups, ctx->sm_count * c);
        int need = (groups + gx - 1) / gx;
        if (need <= wr_cap && smem_for(need) * c <= kSmemBudget && 32 * (need * WC + 1) * c <= 512) wr_max = need, grid_x = gx;
    }
    if (!wr_max) {
        wr_max = wr_cap;
        while (wr_max > 1 && smem_for(wr_max) > kSmemBudget) wr_max--;
        grid_x = (groups + wr_max - 1) / wr_max;
    }
    size_t smem = smem_for(wr_max);
    auto kernel = matmul_pipe_t_kernel<KIND, MT, WC>;
    {
        static std::mutex lock;
        static std::map<std::pair<int, const void*>, bool> done;
        std::lock_guard<std::mutex> guard(lock);
        auto key = std::make_pair(ctx->ordinal, (const void*)kernel);
        if (!done.count(key)) {
            TSM_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
            done[key] = true;
        }
    }
    PipeMaps maps;
    const uint64_t nb = (uint64_t)p.nb;
    TSM_TRY(make_tensor_map_2d(ctx, &maps.weights, CU_TENSOR_MAP_DATA_TYPE_UINT16, p.w, nb * B / 2, (uint64_t)p.n, nb * B, kCB * B / 2, 8 * wr_max,
                               CU_TENSOR_MAP_SWIZZLE_NONE));
    TSM_TRY(make_tensor_map_2d(ctx, &maps.acts, CU_TENSOR_MAP_DATA_TYPE_UINT8, p.acts.qs, nb * 32, (uint64_t)p.m, nb * 32, 128, COLS,
                               CU_TENSOR_MAP_SWIZZLE_128B));
    TSM_TRY(make_tensor_map_2d(ctx, &maps.scales, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, p.acts.scales, nb, (uint64_t)p.m, nb * 4, kCB, COLS,
                               CU_TENSOR_MAP_SWIZZLE_32B));
    TSM_TRY(make_tensor_map_2d(ctx, &maps.sums, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, KIND == TSM_Q4_1 ? p.acts.sums : p.acts.scales, nb, (uint64_t)p.m,
                               nb * 4, kCB, COLS, CU_TENSOR_MAP_SWIZZLE_32B));
    dim3 grid(grid_x, (p.m + COLS - 1) / COLS);
    TSM_CUDA(ctx, launch_chained(ctx, kernel, grid, dim3(32 * (wr_max * WC + 1)), smem, p, wr_max, maps));
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

template <int KIND>
int launch_pipe_kind(tsm_ctx* ctx, const PipeParams& p) {
    // TSM_PIPE_CONFIG = swapped * 100 + WC * 10 + CTAs per SM picks a shape for timing variants without rebuilding
    static const int forced = getenv("TSM_PIPE_CONFIG") ? atoi(getenv("TSM_PIPE_CONFIG")) : 0;
    const int c = forced % 10;
    const int rows = std::min(p.m, 64);
    // Many weight rows: 16-row groups, one warp per group over all activation rows (the weight fragments, which cost the
    // most to prepare, are then used 8 times).  Few: the role-swapped kernel, whose groups are 8 rows and whose weight
    // fragment is one word, with the activation rows split over 2 or 4 warps when the SMs would otherwise be short of warps.
    bool swapped = p.groups < 8 * ctx->sm_count;
    if (forced) swapped = forced / 100 != 0;
    if (!swapped) {
        const int tiles = (rows + 7) / 8;
        int wc = p.groups >= 8 * ctx->sm_count ? 1 : p.groups >= 4 * ctx->sm_count ? 2 : 4;
        if (forced) wc = forced / 10 % 10;
        if (tiles > 4) {
            if (wc >= 4) return launch_pipe_shape<KIND, 2, 4>(ctx, p, c);
            if (wc == 2) return launch_pipe_shape<KIND, 4, 2>(ctx, p, c);
            return launch_pipe_shape<KIND, 8, 1>(ctx, p, c);
        }
        if (tiles > 2) {
            if (wc >= 2) return launch_pipe_shape<KIND, 2, 2>(ctx, p, c);
            return launch_pipe_shape<KIND, 4, 1>(ctx, p, c);
        }
        if (tiles > 1) {
            if (wc >= 2) return launch_pipe_shape<KIND, 1, 2>(ctx, p, c);
            return launch_pipe_shape<KIND, 2, 1>(ctx, p, c);
        }
        return launch_pipe_shape<KIND, 1, 1>(ctx, p, c);
    }
    const int groups8 = (p.n + 7) / 8;
    const int tiles = (rows + 15) / 16;
    int wc = groups8 >= 6 * ctx->sm_count ? 1 : groups8 >= 3 * ctx->sm_count ? 2 : 4;
    if (forced) wc = forced / 10 % 10;
    if (tiles > 2) {
        if (wc >= 4) return launch_pipe_t_shape<KIND, 1, 4>(ctx, p, c);
        if (wc == 2) return launch_pipe_t_shape<KIND, 2, 2>(ctx, p, c);
        return launch_pipe_t_shape<KIND, 4, 1>(ctx, p, c);
    }
    if (tiles > 1) {
        if (wc >= 2) return launch_pipe_t_shape<KIND, 1, 2>(ctx, p, c);
        return launch_pipe_t_shape<KIND, 2, 1>(ctx, p, c);
    }
    return launch_pipe_t_shape<KIND, 1, 1>(ctx, p, c);
}

}  // namespace

// Whether the pipelined kernel takes this product: 16-byte aligned weights, quantised activations and scales, and a
// whole number of 8-block chunks per row (which also makes every row pitch a multiple of 16 bytes, as a tensor
// map requires).
bool pipe_product_fits(const QuantizedActs& a, int rows, int k, const uint8_t* w, int kind, int n) {
    if (getenv("TSM_NO_PIPE")) return false;
    int nb = k / 32;
    bool aligned = (((uintptr_t)w | (uintptr_t)a.qs | (uintptr_t)a.scales | (uintptr_t)(kind == TSM_Q4_1 ? a.sums : a.scales)) & 15) == 0;
    return rows >= 1 && nb >= kCB && nb % kCB == 0 && aligned && tensor_maps_available();
}

int launch_block_matmul_pipe(tsm_ctx* ctx, const QuantizedActs& a, int rows, int k, const uint8_t* w, int kind, int n,
                             const float* bias, const float* residual, float* out) {
    PipeParams p;
    p.w = w, p.n = n, p.nb = k / 32, p.m = rows, p.groups = (n + 15) / 16, p.acts = a, p.bias = bias, p.residual = residual, p.out = out;
    p.errors = ctx->errors;
    p.spins = ctx->wait_spins ? ctx->wait_spins : kPipeSpins;
    p.skip_chunks = ctx->starve_copies ? 1 : 0;
    p.wait_hint = ctx->wait_hint;
    switch (kind) {
        case TSM_Q8_0: return launch_pipe_kind<TSM_Q8_0>(ctx, p);
        case TSM_Q4_0: return launch_pipe_kind<TSM_Q4_0>(ctx, p);
        case TSM_Q4_1: return launch_pipe_kind<TSM_Q4_1>(ctx, p);
    }
    return fail(ctx, TSM_ERR_UNSUPPORTED, "not a block format");
}

}  // namespace tsm
