// The quantised product for several rows of activations on the fifth-generation tensor cores (tcgen05 + tensor memory).
//
// Same arithmetic and same bits as matmul_pipe_kernel (qgemm_pipe.cu) and Quant.matmul_reference (quant.cr:122-142): the
// integer dot product of one 32-element block is exact in any order, the float contributions of a row's blocks are added
// in block order, each product and sum rounded on its own.  One tcgen05.mma of kind::i8 with K = 32 is exactly one ggml
// block: 128 weight rows (the M of the instruction, one per lane of tensor memory) by up to 64 activation rows (its N, one
// per column), s32 results.  What changes against the mma.sync kernels is who does what:
//   * one thread issues the multiplies; its operands are read from shared memory by the tensor core itself and the results
//     land in tensor memory, so the warps that fold the sums issue no multiply, no ldmatrix and prepare no fragment;
//   * four "repack" warps (one thread per weight row) turn a stage of raw ggml blocks (one tiled tensor copy, as before)
//     into the K-major core-matrix layout the multiply reads: Q4_0 / Q4_1 nibbles become int8 (nibble - 8, or the nibble
//     itself), Q8_0's 34-byte blocks become 16-byte-aligned rows; the block scales go to a small table as floats;
//   * eight "fold" warps read each block's 128 x N tile back with tcgen05.ld in the accumulator-fragment shape (.16x256b:
//     a thread holds rows g, g + 8 and columns 2t, 2t + 1 of every 8-column group, like an mma.sync accumulator, so the two
//     scales of an output are per-thread values fetched with a few 16-byte loads instead of warp-wide broadcasts) and fold
//     `fma, mul, add` per output in block order.  A tile is started at the bits of 1.5 * 2^23 (written to tensor memory by
//     the fold warps, the multiply accumulates onto it), so its s32 entries read back as floats 12582912 + dot and the
//     conversion folds into the first multiply exactly as in the mma.sync kernels.
// Tensor memory holds a ring of eight tiles, so the multiplies run up to eight blocks ahead of the folds.  Every wait is
// bounded; on expiry the CTA's abort flag is raised, every role drains, tensor memory is freed and the kernel returns
// with the error record's timeout word set.  Tensor maps cover this GPU's memory only; no cluster, no multicast.
#include <stdlib.h>

#include <type_traits>

#include "common.cuh"

namespace tsm {

namespace {

constexpr int kUB = 8;                 // blocks of K per stage
constexpr int kUSlots = 8;             // tiles of tensor memory in the ring
constexpr unsigned kUSpins = 4u << 20;
constexpr float kUMagic = 12582912.0f;  // 1.5 * 2^23
constexpr int kFoldWarps = 8, kRepackWarps = 4;
constexpr int kUThreads = 32 * (kFoldWarps + kRepackWarps + 2);

template <int KIND> struct UFmt;
template <> struct UFmt<TSM_Q8_0> { static constexpr int B = 34; };
template <> struct UFmt<TSM_Q4_0> { static constexpr int B = 18; };
template <> struct UFmt<TSM_Q4_1> { static constexpr int B = 20; };

struct UmmaParams {
    const uint8_t* w;
    int n, nb, m;          // weight rows, blocks per row, activation rows
    const float* bias;
    const float* residual;
    float* out;            // [m, n]
    ErrorRecord* errors;
    unsigned spins;
    int skip_chunks;       // see tsm_debug_wait_limit
};

struct UmmaMaps {
    CUtensorMap weights;  // u16 [n, nb * B / 2], box (kUB * B / 2) x 128
    CUtensorMap acts;     // u8 [m, k], box 128 x NCOL, 128-byte swizzle
    CUtensorMap scales;   // f32 [m, nb], box kUB x NCOL, 32-byte swizzle
    CUtensorMap sums;     // the same over the block sums (Q4_1)
};

template <int KIND, int NCOL>
struct ULayout {
    static constexpr int B = UFmt<KIND>::B;
    static constexpr int WP = kUB * B;                 // a weight row's raw chunk: 144, 272 or 160 bytes
    static constexpr int ABOX = NCOL * 128;            // one swizzled box of activations: 4 blocks x NCOL rows
    static constexpr int ATILE = 128 * 32;             // one block of 128 weight rows, repacked
    static constexpr int acts_at = 0;
    static constexpr int a_at = 2 * ABOX;                                  // 1024-aligned (ABOX is a multiple of 2048)
    static constexpr int raw_at = a_at + kUB * ATILE;
    static constexpr int scales_at = (raw_at + 128 * WP + 255) / 256 * 256;
    static constexpr int SCALE_BYTES = NCOL * kUB * 4 * (KIND == TSM_Q4_1 ? 2 : 1);
    static constexpr int wscale_at = scales_at + SCALE_BYTES;              // [128 rows][kUB] floats (Q4_1: then the minima)
    static constexpr int WS_BYTES = 128 * kUB * 4 * (KIND == TSM_Q4_1 ? 2 : 1);
    static constexpr int stage_bytes = (wscale_at + WS_BYTES + 1023) / 1024 * 1024;
    static constexpr int stages = (220 * 1024) / stage_bytes >= 3 ? 3 : 2;
    static constexpr unsigned tx = 2 * ABOX + 128 * WP + SCALE_BYTES;
};

__device__ __forceinline__ unsigned u_smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void u_mbar_init(uint64_t* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(u_smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void u_mbar_expect_tx(uint64_t* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(u_smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void u_mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(u_smem_u32(bar)) : "memory");
}
// One poll that may sleep: the thread is suspended until the barrier's phase completes or about `hint_ns` have passed,
// whichever comes first, so a warp that waits does not spend the issue slots the folding warps need.
__device__ __forceinline__ bool u_mbar_try_wait(uint64_t* bar, unsigned parity, unsigned hint_ns) {
    unsigned ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(u_smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
// Bounded: gives up after `limit` polls (each may sleep up to two microseconds), or soon after another role has raised the
// CTA's abort flag.
__device__ __forceinline__ bool u_mbar_wait(uint64_t* bar, unsigned parity, volatile int* abort_flag, unsigned limit) {
    if (u_mbar_try_wait(bar, parity, 0u)) return true;
    for (unsigned spin = 0; spin < limit; spin++) {
        if (u_mbar_try_wait(bar, parity, 2000u)) return true;
        if (*abort_flag) return false;
    }
    return false;
}
__device__ __forceinline__ void u_tensor_load(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
                     u_smem_u32(dst)),
                 "l"(map), "r"(x), "r"(y), "r"(u_smem_u32(bar))
                 : "memory");
}

// Shared-memory matrix descriptor of the tensor core: start address >> 4 in bits 0-13, leading-dimension byte offset >> 4 in
// 16-29, stride-dimension byte offset >> 4 in 32-45, descriptor version 1 in 46-47, swizzle mode in 61-63 (0 none, 2 128-byte).
__device__ __forceinline__ uint64_t u_desc(unsigned saddr, unsigned lbo_bytes, unsigned sbo_bytes, unsigned layout) {
    return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16) | ((uint64_t)((sbo_bytes >> 4) & 0x3fff) << 32) |
           (1ull << 46) | ((uint64_t)layout << 61);
}
// Instruction descriptor, kind::i8: s32 result (2 at bit 4), s8 A (1 at bit 7), s8 B (1 at bit 10), both K-major, N >> 3 at bit 17,
// M >> 4 at bit 24.
__host__ __device__ constexpr unsigned u_idesc(int m, int n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}
__device__ __forceinline__ void u_mma(unsigned taddr, uint64_t adesc, uint64_t bdesc, unsigned idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, 1, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(taddr), "l"(adesc), "l"(bdesc), "r"(idesc)
        : "memory");
}
__device__ __forceinline__ void u_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(u_smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void u_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void u_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// J groups of 8 columns of 16 lanes in the accumulator-fragment shape: registers [4 j + e] = (lane g + 8 (e >> 1), column
// 8 j + 2 t + (e & 1)) for thread 4 g + t.  `load` only issues the read; `landed` waits for every read issued so far (the
// registers themselves are guarded by the hardware's scoreboard like those of any load; naming them as operands of the wait
// cost a register copy each).
template <int J> struct UTmem;
template <> struct UTmem<1> {
    static __device__ __forceinline__ void load(unsigned taddr, unsigned (&v)[4]) {
        asm volatile("tcgen05.ld.sync.aligned.16x256b.x1.b32 {%0,%1,%2,%3}, [%4];"
                     : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(taddr) : "memory");
    }
    static __device__ __forceinline__ void landed(unsigned (&v)[4]) {
        (void)v;
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    }
    static __device__ __forceinline__ void store(unsigned taddr, unsigned x) {
        asm volatile("tcgen05.st.sync.aligned.16x256b.x1.b32 [%0], {%1,%1,%1,%1};" ::"r"(taddr), "r"(x) : "memory");
    }
};
template <> struct UTmem<2> {
    static __device__ __forceinline__ void load(unsigned taddr, unsigned (&v)[8]) {
        asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                     : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "r"(taddr) : "memory");
    }
    static __device__ __forceinline__ void landed(unsigned (&v)[8]) {
        (void)v;
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    }
    static __device__ __forceinline__ void store(unsigned taddr, unsigned x) {
        asm volatile("tcgen05.st.sync.aligned.16x256b.x2.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1};" ::"r"(taddr), "r"(x) : "memory");
    }
};
template <> struct UTmem<4> {
    static __device__ __forceinline__ void load(unsigned taddr, unsigned (&v)[16]) {
        asm volatile(
            "tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]),
              "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(taddr) : "memory");
    }
    static __device__ __forceinline__ void landed(unsigned (&v)[16]) {
        (void)v;
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    }
    static __device__ __forceinline__ void store(unsigned taddr, unsigned x) {
        asm volatile("tcgen05.st.sync.aligned.16x256b.x4.b32 [%0], {%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1,%1};" ::"r"(taddr), "r"(x) : "memory");
    }
};

__device__ __forceinline__ unsigned u_nibbles_minus_8(unsigned x) { return (((x & 0x0f0f0f0fu) | 0x80808080u) - 0x08080808u) ^ 0x80808080u; }

// Word `index` (counted in 32-bit words from byte `byte0`, which is even) of a row chunk held in registers as 32-bit words.
template <int WORDS>
__device__ __forceinline__ unsigned u_word_at(const unsigned (&raw)[WORDS], int byte0, int index) {
    const int at = byte0 + 4 * index;
    return (at & 3) ? __funnelshift_r(raw[at >> 2], raw[(at >> 2) + 1 < WORDS ? (at >> 2) + 1 : at >> 2], 16) : raw[at >> 2];
}

// One block's fold of one half (16 lanes) of a fold warp's part of the tile: two weight rows by 2 J activation rows.  FUSED is
// a template argument so that the two forms of the Q4_0 product are two bodies behind one real branch: as one body with the
// choice inside, both forms were computed for every output and one of them dropped.
template <int KIND, int J, bool FUSED>
__device__ __forceinline__ void u_fold_half(float (&acc)[J][4], const unsigned (&d)[4 * J], const float (&dwv)[2], const float (&mv)[2],
                                            const float (&dxv)[J][2], const float (&sxv)[J][2]) {
#pragma unroll
    for (int hi = 0; hi < 2; hi++) {
        const float xw = __fmul_rn(-kUMagic, dwv[hi]);
#pragma unroll
        for (int j = 0; j < J; j++)
#pragma unroll
            for (int lo = 0; lo < 2; lo++) {
                const float bits = __uint_as_float(d[4 * j + 2 * hi + lo]);
                float& a = acc[j][2 * hi + lo];
                if (KIND == TSM_Q8_0) {
                    // float(dot) * (dw * dx), then the add
                    a = __fadd_rn(a, __fmul_rn(__fsub_rn(bits, kUMagic), __fmul_rn(dwv[hi], dxv[j][lo])));
                } else if (KIND == TSM_Q4_0) {
                    // (float(dot) * dw) * dx: fma(1.5 * 2^23 + dot, dw, -1.5 * 2^23 * dw) has exact products (dw has 11
                    // significant bits), so it rounds once, like float(dot) * dw; a scale that is not finite takes the
                    // subtract-then-multiply form, which gives the reference's infinities instead of NaN
                    float scaled = FUSED ? __fmaf_rn(bits, dwv[hi], xw) : __fmul_rn(__fsub_rn(bits, kUMagic), dwv[hi]);
                    a = __fadd_rn(a, __fmul_rn(scaled, dxv[j][lo]));
                } else {
                    a = __fadd_rn(a, __fadd_rn(__fmul_rn(__fmul_rn(dwv[hi], dxv[j][lo]), __fsub_rn(bits, kUMagic)), __fmul_rn(mv[hi], sxv[j][lo])));
                }
            }
    }
}

// Roles by warp: 0-7 fold (tensor-memory lanes 32 (warp & 3) .., columns of half warp >> 2), 8-11 repack, 12 copies, 13 multiplies.
template <int KIND, int NCOL>
__global__ void __launch_bounds__(kUThreads, 1) matmul_umma_kernel(UmmaParams p, const __grid_constant__ UmmaMaps maps) {
    chained_kernel_entry();
    using L = ULayout<KIND, NCOL>;
    constexpr int B = L::B, WP = L::WP, S = L::stages;
    constexpr int J = NCOL / 16;                       // 8-column groups per fold warp (each takes half the columns)
    constexpr int TCOLS = NCOL * kUSlots < 32 ? 32 : NCOL * kUSlots;
    extern __shared__ unsigned char smem_raw[];
    // aligned by an offset from the shared array itself, so that the compiler still knows these are shared-memory addresses
    unsigned char* smem = smem_raw + ((1024u - (u_smem_u32(smem_raw) & 1023u)) & 1023u);
    uint64_t* full = (uint64_t*)smem;                  // [S]      a stage's copies have landed
    uint64_t* empty = full + 4;                        // [S]      repack, fold and multiply are done with the stage
    uint64_t* a_ready = empty + 4;                     // [S]      the stage's blocks are repacked
    uint64_t* t_full = a_ready + 4;                    // [slots]  a block's tile is complete in tensor memory
    uint64_t* t_empty = t_full + kUSlots;              // [slots]  the tile has been folded and reset
    unsigned* tmem_slot = (unsigned*)(smem + 512);
    volatile int* abort_flag = (volatile int*)(smem + 520);   // [1] stays 0
    unsigned char* stages = smem + 1024;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nb = p.nb, chunks = nb / kUB;
    const int row0 = blockIdx.x * 128, col0 = blockIdx.y * NCOL;

    if (tid == 0) {
        for (int s = 0; s < S; s++) {
            u_mbar_init(&full[s], 1);
            u_mbar_init(&empty[s], kRepackWarps + kFoldWarps + 1);
            u_mbar_init(&a_ready[s], kRepackWarps);
        }
        for (int i = 0; i < kUSlots; i++) u_mbar_init(&t_full[i], 1), u_mbar_init(&t_empty[i], kFoldWarps);
        abort_flag[0] = 0, abort_flag[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(u_smem_u32(tmem_slot)), "n"(TCOLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    u_fence_before();
    __syncthreads();
    u_fence_after();
    const unsigned tmem = *tmem_slot;
    bool ok = true;

    if (warp == kFoldWarps + kRepackWarps) {
        // ---------------------------------------------------------------- copies: one thread
        if (lane == 0) {
            int issued = 0;
            for (int chunk = 0; chunk < chunks - p.skip_chunks; chunk++) {
                int s = chunk % S;
                if (chunk >= S) ok = u_mbar_wait(&empty[s], (unsigned)((chunk / S - 1) & 1), abort_flag, p.spins);
                if (!ok) break;
                unsigned char* base = stages + (size_t)s * L::stage_bytes;
                u_mbar_expect_tx(&full[s], L::tx);
                u_tensor_load(base + L::acts_at, &maps.acts, chunk * kUB * 32, col0, &full[s]);
                u_tensor_load(base + L::acts_at + L::ABOX, &maps.acts, chunk * kUB * 32 + 128, col0, &full[s]);
                u_tensor_load(base + L::raw_at, &maps.weights, chunk * (kUB * B / 2), row0, &full[s]);
                u_tensor_load(base + L::scales_at, &maps.scales, chunk * kUB, col0, &full[s]);
                if (KIND == TSM_Q4_1) u_tensor_load(base + L::scales_at + NCOL * kUB * 4, &maps.sums, chunk * kUB, col0, &full[s]);
                issued = chunk + 1;
            }
            if (!ok) {
                *abort_flag = 1;
                atomicExch(&p.errors->timeout, 1);
                // see the copies already issued land before the CTA's shared memory goes away
                for (int chunk = max(0, issued - S); chunk < issued; chunk++) u_mbar_wait(&full[chunk % S], (unsigned)((chunk / S) & 1), abort_flag + 1, p.spins);
            }
        }
    } else if (warp == kFoldWarps + kRepackWarps + 1) {
        // ---------------------------------------------------------------- multiplies: one thread
        if (lane == 0) {
            constexpr unsigned idesc = u_idesc(128, NCOL);
            for (int chunk = 0; chunk < chunks && ok; chunk++) {
                int s = chunk % S;
                const unsigned parity = (unsigned)((chunk / S) & 1);
                ok = u_mbar_wait(&full[s], parity, abort_flag, p.spins) && u_mbar_wait(&a_ready[s], parity, abort_flag, p.spins);
                if (!ok) break;
                u_fence_after();
                const unsigned base = u_smem_u32(stages + (size_t)s * L::stage_bytes);
#pragma unroll 1
                for (int u = 0; u < kUB; u++) {
                    const int block = chunk * kUB + u, slot = block % kUSlots;
                    ok = u_mbar_wait(&t_empty[slot], (unsigned)((block / kUSlots) & 1), abort_flag, p.spins);
                    if (!ok) break;
                    u_fence_after();
                    // A: block u of the repacked stage, unswizzled core matrices (8 rows x 16 bytes): the two 16-byte halves of
                    // K are 128 bytes apart, groups of 8 rows 256 bytes.  B: activation box u / 4, 128-byte swizzle, block
                    // u % 4 at 32 bytes inside the swizzle atom, groups of 8 rows 1024 bytes apart.
                    uint64_t adesc = u_desc(base + L::a_at + u * L::ATILE, 128, 256, 0);
                    uint64_t bdesc = u_desc(base + L::acts_at + (u >> 2) * L::ABOX + (u & 3) * 32, 16, 1024, 2);
                    u_mma(tmem + slot * NCOL, adesc, bdesc, idesc);
                    u_commit(&t_full[slot]);
                }
                if (ok) u_commit(&empty[s]);   // arrives once every multiply of the stage has read its operands
            }
            if (!ok) {
                *abort_flag = 1;
                atomicExch(&p.errors->timeout, 1);
            }
        }
    } else if (warp >= kFoldWarps) {
        // ---------------------------------------------------------------- repack: thread = weight row of the tile
        const int r = tid - 32 * kFoldWarps;
        const unsigned a_off = (unsigned)((r >> 3) * 256 + (r & 7) * 16);
        for (int chunk = 0; chunk < chunks; chunk++) {
            int s = chunk % S;
            ok = u_mbar_wait(&full[s], (unsigned)((chunk / S) & 1), abort_flag, p.spins);
            if (!ok) break;
            unsigned char* base = stages + (size_t)s * L::stage_bytes;
            unsigned raw[WP / 4];
            const uint4* src = (const uint4*)(base + L::raw_at + (size_t)r * WP);
#pragma unroll
            for (int i = 0; i < WP / 16; i++) {
                uint4 v = src[i];
                raw[4 * i] = v.x, raw[4 * i + 1] = v.y, raw[4 * i + 2] = v.z, raw[4 * i + 3] = v.w;
            }
            float* ws = (float*)(base + L::wscale_at) + r * kUB;
            float dws[kUB], mins[kUB];
#pragma unroll
            for (int u = 0; u < kUB; u++) {
                const int o = u * B;
                const unsigned head = raw[o >> 2] >> ((o & 3) * 8);
                dws[u] = half_bits_to_float(head & 0xffffu);
                uint4 lo, hi;
                if (KIND == TSM_Q8_0) {
                    lo = make_uint4(u_word_at(raw, o + 2, 0), u_word_at(raw, o + 2, 1), u_word_at(raw, o + 2, 2), u_word_at(raw, o + 2, 3));
                    hi = make_uint4(u_word_at(raw, o + 2, 4), u_word_at(raw, o + 2, 5), u_word_at(raw, o + 2, 6), u_word_at(raw, o + 2, 7));
                    mins[u] = 0.0f;
                } else if (KIND == TSM_Q4_0) {
                    unsigned n0 = u_word_at(raw, o + 2, 0), n1 = u_word_at(raw, o + 2, 1), n2 = u_word_at(raw, o + 2, 2), n3 = u_word_at(raw, o + 2, 3);
                    lo = make_uint4(u_nibbles_minus_8(n0), u_nibbles_minus_8(n1), u_nibbles_minus_8(n2), u_nibbles_minus_8(n3));
                    hi = make_uint4(u_nibbles_minus_8(n0 >> 4), u_nibbles_minus_8(n1 >> 4), u_nibbles_minus_8(n2 >> 4), u_nibbles_minus_8(n3 >> 4));
                    mins[u] = 0.0f;
                } else {
                    unsigned n0 = raw[(o >> 2) + 1], n1 = raw[(o >> 2) + 2], n2 = raw[(o >> 2) + 3], n3 = raw[(o >> 2) + 4];
                    lo = make_uint4(n0 & 0x0f0f0f0fu, n1 & 0x0f0f0f0fu, n2 & 0x0f0f0f0fu, n3 & 0x0f0f0f0fu);
                    hi = make_uint4((n0 >> 4) & 0x0f0f0f0fu, (n1 >> 4) & 0x0f0f0f0fu, (n2 >> 4) & 0x0f0f0f0fu, (n3 >> 4) & 0x0f0f0f0fu);
                    mins[u] = half_bits_to_float(head >> 16);
                }
                unsigned char* tile = base + L::a_at + u * L::ATILE + a_off;
                *(uint4*)tile = lo;           // elements 0..15 of the block
                *(uint4*)(tile + 128) = hi;   // elements 16..31
            }
            *(float4*)ws = make_float4(dws[0], dws[1], dws[2], dws[3]);
            *(float4*)(ws + 4) = make_float4(dws[4], dws[5], dws[6], dws[7]);
            if (KIND == TSM_Q4_1) {
                float* wm = ws + 128 * kUB;
                *(float4*)wm = make_float4(mins[0], mins[1], mins[2], mins[3]);
                *(float4*)(wm + 4) = make_float4(mins[4], mins[5], mins[6], mins[7]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the tensor core reads what these stores wrote
            __syncwarp();
            if (lane == 0) {
                u_mbar_arrive(&a_ready[s]);
                u_mbar_arrive(&empty[s]);   // the raw blocks have been read
            }
        }
        if (!ok) {
            *abort_flag = 1;
            if (lane == 0) atomicExch(&p.errors->timeout, 1);
        }
    } else {
        // ---------------------------------------------------------------- fold: the ordered sums
        const int quarter = warp & 3, chalf = warp >> 2;
        const int g = lane >> 2, t = lane & 3;
        const int cbase = chalf * (NCOL / 2);                       // this warp's first column within the tile
        const unsigned lane_addr = tmem + ((unsigned)(quarter * 32) << 16) + (unsigned)cbase;
        // every tile starts as the bits of 1.5 * 2^23 in this warp's part of it
#pragma unroll 1
        for (int slot = 0; slot < kUSlots; slot++) {
            UTmem<J>::store(lane_addr + slot * NCOL, 0x4b400000u);
            UTmem<J>::store(lane_addr + slot * NCOL + (16u << 16), 0x4b400000u);
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        u_fence_before();
        __syncwarp();
        if (lane == 0)
            for (int slot = 0; slot < kUSlots; slot++) u_mbar_arrive(&t_empty[slot]);

        float acc[2][J][4];
#pragma unroll
        for (int h = 0; h < 2; h++)
#pragma unroll
            for (int j = 0; j < J; j++)
#pragma unroll
                for (int e = 0; e < 4; e++) acc[h][j][e] = 0.0f;
        const int rloc = quarter * 32 + g;                         // rows rloc + 16 h + 8 hi of the tile
        // The tile of block b is read in two halves, and one read is always in flight: while the first half of a block is
        // folded the second is on its way, and while the second is folded the first half of the next block is.
        unsigned d0[4 * J], d1[4 * J];
        ok = u_mbar_wait(&t_full[0], 0u, abort_flag, p.spins);
        u_fence_after();
        UTmem<J>::load(lane_addr, d0);
        for (int chunk = 0; chunk < chunks; chunk++) {
            int s = chunk % S;
            const unsigned parity = (unsigned)((chunk / S) & 1);
            if (!u_mbar_wait(&full[s], parity, abort_flag, p.spins)) ok = false;      // the scale boxes have landed
            if (!u_mbar_wait(&a_ready[s], parity, abort_flag, p.spins)) ok = false;   // the block scales are in their table
            const unsigned char* base = stages + (size_t)s * L::stage_bytes;
            const float* sc = (const float*)(base + L::scales_at);
            const float* sm = sc + NCOL * kUB;
            const float* ws = (const float*)(base + L::wscale_at) + rloc * kUB;
            const float* wm = ws + 128 * kUB;
            const float* sc_mine = sc + (cbase + 2 * t) * kUB;
            const float* sm_mine = sm + (cbase + 2 * t) * kUB;
            const int flip = ((t >> 1) & 1) << 2;
#pragma unroll 1
            for (int u = 0; u < kUB; u++) {
                const int block = chunk * kUB + u, slot = block % kUSlots;
                const unsigned t0 = lane_addr + slot * NCOL, t1 = t0 + (16u << 16);
                // this block's scales: two weight rows per half, 2 J activation rows
                float dwv[2][2], mv[2][2], dxv[J][2], sxv[J][2];
#pragma unroll
                for (int h = 0; h < 2; h++)
#pragma unroll
                    for (int hi = 0; hi < 2; hi++) {
                        dwv[h][hi] = ws[(16 * h + 8 * hi) * kUB + u];
                        mv[h][hi] = KIND == TSM_Q4_1 ? wm[(16 * h + 8 * hi) * kUB + u] : 0.0f;
                    }
                // The scale box is written with the 32-byte swizzle: the 16-byte half (blocks 0-3 or 4-7) of column c sits at
                // half ^ bit 2 of c.  This thread's columns are cbase + 8 j + 2 t + lo, whose bit 2 is bit 1 of t for every
                // j and lo, so block u is found at index u ^ flip of each of its columns' eight floats.
                const float* su = sc_mine + (u ^ flip);
                const float* mu = sm_mine + (u ^ flip);
#pragma unroll
                for (int j = 0; j < J; j++)
#pragma unroll
                    for (int lo = 0; lo < 2; lo++) {
                        dxv[j][lo] = su[(8 * j + lo) * kUB];
                        sxv[j][lo] = KIND == TSM_Q4_1 ? mu[(8 * j + lo) * kUB] : 0.0f;
                    }
                bool plain = fabsf(dwv[0][0]) <= 65504.0f && fabsf(dwv[0][1]) <= 65504.0f && fabsf(dwv[1][0]) <= 65504.0f && fabsf(dwv[1][1]) <= 65504.0f;
                const bool fused = KIND != TSM_Q4_0 || __all_sync(0xffffffffu, plain);
                UTmem<J>::landed(d0);
                if (block > 0) {
                    // the block before this one: its tile was reset a whole fold ago, so this wait costs nothing by now
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                    u_fence_before();
                    __syncwarp();
                    if (lane == 0) u_mbar_arrive(&t_empty[(block - 1) % kUSlots]);
                }
                UTmem<J>::load(t1, d1);
                UTmem<J>::store(t0, 0x4b400000u);   // the tile goes back to 1.5 * 2^23 for the block that uses it next
                if (fused) u_fold_half<KIND, J, true>(acc[0], d0, dwv[0], mv[0], dxv, sxv);
                else u_fold_half<KIND, J, false>(acc[0], d0, dwv[0], mv[0], dxv, sxv);
                UTmem<J>::landed(d1);
                UTmem<J>::store(t1, 0x4b400000u);
                if (block + 1 < nb) {
                    const int next = (block + 1) % kUSlots;
                    if (!u_mbar_wait(&t_full[next], (unsigned)(((block + 1) / kUSlots) & 1), abort_flag, p.spins)) ok = false;
                    u_fence_after();
                    UTmem<J>::load(lane_addr + next * NCOL, d0);
                }
                if (fused) u_fold_half<KIND, J, true>(acc[1], d1, dwv[1], mv[1], dxv, sxv);
                else u_fold_half<KIND, J, false>(acc[1], d1, dwv[1], mv[1], dxv, sxv);
            }
            __syncwarp();
            if (lane == 0) u_mbar_arrive(&empty[s]);   // the stage's scales have been read
            if (!ok) break;
        }
        asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");   // the last block's tile
        u_fence_before();
        __syncwarp();
        if (lane == 0 && nb > 0) u_mbar_arrive(&t_empty[(nb - 1) % kUSlots]);
        if (!ok) {
            *abort_flag = 1;
            if (lane == 0) atomicExch(&p.errors->timeout, 1);
        } else {
#pragma unroll
            for (int h = 0; h < 2; h++)
#pragma unroll
                for (int j = 0; j < J; j++)
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const int row = row0 + rloc + 16 * h + 8 * (e >> 1);
                        const int col = col0 + cbase + 8 * j + 2 * t + (e & 1);
                        if (row < p.n && col < p.m) {
                            float v = acc[h][j][e];
                            if (p.bias) v = __fadd_rn(v, p.bias[row]);
                            if (p.residual) v = __fadd_rn(p.residual[(int64_t)col * p.n + row], v);
                            p.out[(int64_t)col * p.n + row] = v;
                        }
                    }
        }
    }
    // every role ends here, whether it finished or gave up: tensor memory is freed by the warp that took it
    u_fence_before();
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(TCOLS) : "memory");
}

template <int KIND, int NCOL>
int launch_umma_shape(tsm_ctx* ctx, const UmmaParams& p, const QuantizedActs& a) {
    using L = ULayout<KIND, NCOL>;
    constexpr int B = L::B;
    // never less than 120 KB: two CTAs must not share an SM, each would wait for the other's tensor memory
    const size_t smem = std::max<size_t>(120 * 1024, 2048 + (size_t)L::stages * L::stage_bytes);
    auto kernel = matmul_umma_kernel<KIND, NCOL>;
    {
        static std::mutex lock;
        static std::map<std::pair<int, const void*>, bool> done;
        std::lock_guard<std::mutex> guard(lock);
        auto key = std::make_pair(ctx->ordinal, (const void*)kernel);
        if (!done.count(key)) {
            TSM_CUDA(ctx, cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            done[key] = true;
        }
    }
    UmmaMaps maps;
    const uint64_t nb = (uint64_t)p.nb;
    TSM_TRY(make_tensor_map_2d(ctx, &maps.weights, CU_TENSOR_MAP_DATA_TYPE_UINT16, p.w, nb * B / 2, (uint64_t)p.n, nb * B, kUB * B / 2, 128,
                               CU_TENSOR_MAP_SWIZZLE_NONE));
    TSM_TRY(make_tensor_map_2d(ctx, &maps.acts, CU_TENSOR_MAP_DATA_TYPE_UINT8, a.qs, nb * 32, (uint64_t)p.m, nb * 32, 128, NCOL,
                               CU_TENSOR_MAP_SWIZZLE_128B));
    TSM_TRY(make_tensor_map_2d(ctx, &maps.scales, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, a.scales, nb, (uint64_t)p.m, nb * 4, kUB, NCOL,
                               CU_TENSOR_MAP_SWIZZLE_32B));
    TSM_TRY(make_tensor_map_2d(ctx, &maps.sums, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, KIND == TSM_Q4_1 ? a.sums : a.scales, nb, (uint64_t)p.m, nb * 4,
                               kUB, NCOL, CU_TENSOR_MAP_SWIZZLE_32B));
    dim3 grid((p.n + 127) / 128, (p.m + NCOL - 1) / NCOL);
    TSM_CUDA(ctx, launch_chained(ctx, kernel, grid, dim3(kUThreads), smem, p, maps));
    count_launch(ctx);
    TSM_LAUNCH_CHECK(ctx);
    return TSM_OK;
}

template <int KIND>
int launch_umma_kind(tsm_ctx* ctx, const UmmaParams& p, const QuantizedActs& a) {
    // Activation columns per CTA: all 64 when the 128-row tiles alone give every SM work, fewer (the weights are then repacked
    // by several CTAs) when the matrix has few rows.  TSM_UMMA_COLS forces a width, for timing.
    static const int forced = getenv("TSM_UMMA_COLS") ? atoi(getenv("TSM_UMMA_COLS")) : 0;
    const int tiles = (p.n + 127) / 128;
    const int rows = std::min(p.m, 64);
    // a CTA's time per block is about 35 instructions of repacking per row plus 3.6 per output; the launch lasts as many
    // rounds as its CTAs need on the SMs (one CTA per SM)
    int ncol = 64;
    double best = 0.0;
    for (int candidate : {64, 32, 16}) {
        if (candidate / 2 >= rows && candidate > 16) continue;   // twice as wide as the activations: only padding
        int64_t ctas = (int64_t)tiles * ((rows + candidate - 1) / candidate);
        int64_t rounds = (ctas + ctx->sm_count - 1) / ctx->sm_count;
        double cost = (double)rounds * (35.0 + 3.6 * candidate);
        if (best == 0.0 || cost < best) best = cost, ncol = candidate;
    }
    if (forced == 16 || forced == 32 || forced == 64) ncol = forced;
    if (ncol == 64) return launch_umma_shape<KIND, 64>(ctx, p, a);
    if (ncol == 32) return launch_umma_shape<KIND, 32>(ctx, p, a);
    return launch_umma_shape<KIND, 16>(ctx, p, a);
}

}  // namespace

// Whether the tensor-memory kernel takes this product: what the tensor-map pipeline needs (16-byte aligned operands, a whole
// number of 8-block chunks per row) and enough activation rows to be worth a 128-row tile.  TSM_NO_UMMA sends everything to
// the mma.sync pipeline instead.
bool umma_product_fits(const QuantizedActs& a, int rows, int k, const uint8_t* w, int kind, int n) {
    static const bool off = getenv("TSM_NO_UMMA") != nullptr || !(getenv("TSM_UMMA") && getenv("TSM_UMMA")[0] == '1');
    if (off) return false;
    return rows >= 5 && n >= 128 && pipe_product_fits(a, rows, k, w, kind, n);
}

int launch_block_matmul_umma(tsm_ctx* ctx, const QuantizedActs& a, int rows, int k, const uint8_t* w, int kind, int n, const float* bias,
                             const float* residual, float* out) {
    UmmaParams p;
    p.w = w, p.n = n, p.nb = k / 32, p.m = rows, p.bias = bias, p.residual = residual, p.out = out, p.errors = ctx->errors;
    p.spins = ctx->wait_spins ? ctx->wait_spins : kUSpins;
    p.skip_chunks = ctx->starve_copies ? 1 : 0;
    switch (kind) {
        case TSM_Q8_0: return launch_umma_kind<TSM_Q8_0>(ctx, p, a);
        case TSM_Q4_0: return launch_umma_kind<TSM_Q4_0>(ctx, p, a);
        case TSM_Q4_1: return launch_umma_kind<TSM_Q4_1>(ctx, p, a);
    }
    return fail(ctx, TSM_ERR_UNSUPPORTED, "not a block format");
}

}  // namespace tsm
