// Weight gradient of a linear layer straight from the compressed layer input, sm_100a:
//     dW[n, k] = sum_m dY[m, n] * X~[m, k],   X~[m, k] = bf16(code[m, k] * scale[g] + min[g])
// where X was saved by act_quant_pack as b-bit codes with one (scale, min) per group of G
// consecutive elements of the row-major [M, K] input (G divides K, so a group never leaves its
// row) and dY is bf16 [M, N].  The decoded values are exactly those act_dequant_unpack would
// write as bf16; they are produced inside the GEMM's operand pipeline instead of in HBM.
// Reference: the author's Triton attempt at the same fusion ran at 0.06-0.17x of
// dequantise + cuBLAS (Activation_Compression/test2.ipynb:14-19, 478-491).
//
// One CTA per (256 x 256 output tile, slice of M); 576 threads:
//   warp 0       TMA producer: 64 rows of dY x 256 columns per stage, as four 64 x 64 boxes with
//                the 128-byte swizzle.  dY is row-major [M, N], so the tile lands with the
//                output dimension n contiguous: the "MN-major" operand form of tcgen05.mma.
//   warp 1       MMA issuer: per stage 2 x 4 tcgen05.mma.kind::f16 (bf16, M = 128, N = 256,
//                K = 16), both operands MN-major, two 128 x 256 fp32 accumulators = all 512
//                columns of tensor memory.
//   warps 2..17  decoders (four per scheduler: with eight, 244 us instead of 208 on the ViT MLP
//                shapes): read the codes of 64 rows x 256 columns (2 bytes per 8 two-bit
//                codes), look the two bytes of every bf16 value up in the group's table of 2^b
//                outputs with a byte permute (the arithmetic of dequant_unpack_kernel), and
//                store 16-byte pieces into the same swizzled MN-major layout a bulk tensor copy
//                of a dense bf16 X would have produced; 8 lanes cover one 128-byte row, so the
//                stores are conflict-free.  After the last stage the same warps drain the
//                accumulators and add them to dW with vector reductions (red.global.add.v4.f32):
//                slices of M owned by different CTAs sum into the same fp32 tile, which the host
//                zeroes first.
// Every mbarrier wait is bounded; on a timeout the kernel records a reason and leaves.
// Bound: bf16 tensor throughput, flops = 2*M*N*K; the decoders need about 2.5 issue slots per
// element and an element is used by 256 output rows, which keeps them under the MMA time.
#include <cuda.h>

#include "act_common.cuh"

namespace act {
namespace dw {

constexpr int TM = 256;                   // output rows (n) per tile: two M = 128 accumulators
constexpr int TN = 256;                   // output columns (k) per tile
constexpr int KB = 64;                    // rows of the reduction dimension m per stage
constexpr int UMMA_K = 16;                // K of one tcgen05.mma for 16-bit operands
constexpr int STAGES = 3;
#ifndef ACT_DW_PREFETCH_BLOCKS
#define ACT_DW_PREFETCH_BLOCKS 8
#endif
constexpr int PREFETCH_BLOCKS = ACT_DW_PREFETCH_BLOCKS;   // distance of the L2 prefetch of dY, in 64-row blocks (0: off)
constexpr int A_STAGE = KB * TM * 2, B_STAGE = KB * TN * 2;      // 32 KB each
constexpr int CHUNK = KB * 128;           // one 64-column chunk of a stage: 64 rows x 128 bytes
#ifndef ACT_DW_DEC_WARPS
#define ACT_DW_DEC_WARPS 16
#endif
constexpr int DEC_WARPS = ACT_DW_DEC_WARPS;                // 8 or 16 (a multiple of four: the epilogue's TMEM lane quarters)
constexpr int PIECES = (KB * TN / 8) / (DEC_WARPS * 32);  // 16-byte pieces of a stage per decoder thread
constexpr int EPI_COLS = TN / (DEC_WARPS / 4);            // accumulator columns per warp in the epilogue
constexpr int THREADS = 64 + DEC_WARPS * 32;
static_assert(DEC_WARPS % 4 == 0 && PIECES >= 2 && PIECES % 2 == 0 && EPI_COLS % 32 == 0, "decoder split");
constexpr int TMEM_COLS = 512;
constexpr uint32_t SPIN_LIMIT = 1u << 24;

struct __align__(1024) Smem {
    uint8_t a[STAGES][A_STAGE];
    uint8_t b[STAGES][B_STAGE];
    uint64_t full_a[STAGES], full_b[STAGES], empty[STAGES], acc_full;
    uint32_t tmem_base;
    volatile uint32_t abort;
};
static_assert(sizeof(Smem) <= 227 * 1024, "shared memory of the dW kernel exceeds one SM");

__device__ unsigned int g_dw_error = 0;         // last abort reason (0 = none)

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, Smem* s, uint32_t code) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (s->abort) return false;
    }
    s->abort = 1;
    atomicExch(&g_dw_error, code);
    return false;
}
// warp-wide: lane 0 polls, everybody learns the outcome
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, Smem* s, uint32_t code) {
    uint32_t ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, s, code) ? 1u : 0u;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
// requests a tile into L2 only (no shared-memory destination, nothing to wait for)
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* map, int c0, int c1) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" :: "l"(map), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(dst_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void red_add_v4(float* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};"
                 :: "l"(p), "f"(__uint_as_float(a)), "f"(__uint_as_float(b)), "f"(__uint_as_float(c)), "f"(__uint_as_float(d)) : "memory");
}

// Shared-memory descriptor of an MN-major operand held as 64-element (128-byte) chunks of the
// MN dimension: inside a chunk, reduction row r sits at r * 128 bytes with its 16-byte pieces
// xor-swizzled by r & 7 (what a 128-byte-swizzled bulk tensor copy writes); groups of eight
// reduction rows are 1024 bytes apart (stride byte offset), chunks CHUNK bytes apart (leading
// byte offset).  Version 1, layout type 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t make_mn_major_desc(const void* start) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(start) & 0x3FFFF) >> 4);
    d |= (uint64_t)(CHUNK >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// fp32 accumulate, A and B bf16, both MN-major, N = 256, M = 128
__host__ __device__ constexpr uint32_t make_idesc() {
    return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) |
           ((uint32_t)(TN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}

// ---------------------------------------------------------------- decoding
// The 2^BITS possible bf16 outputs of a group, BITS <= 2: (code * scale + min) rounded once to
// fp32 and once to bf16, as dequant_unpack_kernel does.
template <int BITS>
__device__ __forceinline__ void group_table(float s, float m, uint32_t& t_lo, uint32_t& t_hi) {
    const f32x2 s2 = pack2(s, s), m2 = pack2(m, m);
    uint32_t f0, f1, f2, f3;
    unpack2u(fma2_rn(pack2(0.0f, 1.0f), s2, m2), f0, f1);
    { const __nv_bfloat162 t = __floats2bfloat162_rn(__uint_as_float(f0), __uint_as_float(f1)); t_lo = *reinterpret_cast<const uint32_t*>(&t); }
    t_hi = 0u;
    if (BITS == 2) {
        unpack2u(fma2_rn(pack2(2.0f, 3.0f), s2, m2), f2, f3);
        const __nv_bfloat162 t = __floats2bfloat162_rn(__uint_as_float(f2), __uint_as_float(f3)); t_hi = *reinterpret_cast<const uint32_t*>(&t);
    }
}
// eight 1- or 2-bit codes -> eight bf16 values picked out of the table, two bytes each, by byte permute
template <int BITS>
__device__ __forceinline__ uint4 decode8_table(uint32_t w32, uint32_t t_lo, uint32_t t_hi) {
    uint4 out;
    uint32_t* o = &out.x;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint32_t z;
        if (BITS == 2) {
            const uint32_t x = (w32 >> (8 * h)) & 0xFFu;
            const uint32_t y = (x * 4097u) & 0x000F000Fu;
            z = (y * 65u) & 0x03030303u;
        } else {
            const uint32_t x = (w32 >> (4 * h)) & 0xFu;
            z = (x * 0x00204081u) & 0x01010101u;
        }
        const uint32_t sel = z * 0x22u + 0x10101010u;
        o[2 * h] = __byte_perm(t_lo, t_hi, sel);
        o[2 * h + 1] = __byte_perm(t_lo, t_hi, sel >> 16);
    }
    return out;
}
// eight b-bit codes (the low 8*BITS bits of w) of one group -> eight bf16 values = one 16-byte piece
template <int BITS>
__device__ __forceinline__ uint4 decode8(uint64_t w, float s, float m) {
    if (BITS <= 2) {
        uint32_t t_lo, t_hi;
        group_table<BITS>(s, m, t_lo, t_hi);
        return decode8_table<BITS>((uint32_t)w, t_lo, t_hi);
    }
    const f32x2 s2 = pack2(s, s), m2 = pack2(m, m);
    uint4 out;
    uint32_t* o = &out.x;
    constexpr uint64_t MASK = (1ull << BITS) - 1ull;
#pragma unroll
    for (int p = 0; p < 4; ++p) {
        const float c0 = (float)(uint32_t)((w >> (2 * p * BITS)) & MASK);
        const float c1 = (float)(uint32_t)((w >> ((2 * p + 1) * BITS)) & MASK);
        uint32_t lo, hi;
        unpack2u(fma2_rn(pack2(c0, c1), s2, m2), lo, hi);
        const __nv_bfloat162 t = __floats2bfloat162_rn(__uint_as_float(lo), __uint_as_float(hi));
        o[p] = *reinterpret_cast<const uint32_t*>(&t);
    }
    return out;
}

template <int BITS> struct CodePiece;       // the BITS bytes that hold eight codes
template <> struct CodePiece<1> { static __device__ __forceinline__ uint64_t ld(const uint8_t* p) { return __ldg(p); } };
template <> struct CodePiece<2> { static __device__ __forceinline__ uint64_t ld(const uint8_t* p) { return __ldg(reinterpret_cast<const uint16_t*>(p)); } };
template <> struct CodePiece<4> { static __device__ __forceinline__ uint64_t ld(const uint8_t* p) { return __ldg(reinterpret_cast<const uint32_t*>(p)); } };
template <> struct CodePiece<8> { static __device__ __forceinline__ uint64_t ld(const uint8_t* p) { return __ldg(reinterpret_cast<const unsigned long long*>(p)); } };

// ------------------------------------------------------------------ the kernel
// Work item w = (tile, slice): tile = w / slices walks the output tiles row-major, slice =
// w % slices is a contiguous run of 64-row blocks of M.
template <int BITS>
__global__ void __launch_bounds__(THREADS, 1)
dw_gemm_kernel(const __grid_constant__ CUtensorMap map_dy, const uint8_t* __restrict__ packed,
               const float* __restrict__ scale, const float* __restrict__ mn, float* __restrict__ dw,
               int M, int N, int K, int log2_gs, int ld_dw, int slices)
{
    extern __shared__ __align__(1024) uint8_t smem_raw_dw[];
    Smem* s = reinterpret_cast<Smem*>(smem_raw_dw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_tiles = (N + TM - 1) / TM, k_tiles = (K + TN - 1) / TN;
    const int n_work = n_tiles * k_tiles * slices;
    const int m_blocks = (M + KB - 1) / KB;

    if (smem_u32(s) & 1023u) {                                // the swizzled tiles need this alignment
        if (threadIdx.x == 0) atomicExch(&g_dw_error, 5u);
        return;
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&s->full_a[i], 1); mbar_init(&s->full_b[i], DEC_WARPS); mbar_init(&s->empty[i], 1); }
        mbar_init(&s->acc_full, 1);
        s->abort = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(&s->tmem_base, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s->tmem_base;

    // blocks [b_lo, b_hi) of 64 rows belong to slice sl: as even a split as whole blocks allow
    auto slice_range = [&](int sl, int& b_lo, int& b_hi) {
        const int per = m_blocks / slices, extra = m_blocks % slices;
        b_lo = sl * per + (sl < extra ? sl : extra);
        b_hi = b_lo + per + (sl < extra ? 1 : 0);
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (dY)
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int w = blockIdx.x; ok && w < n_work; w += gridDim.x) {
                const int tile = w / slices, n0 = (tile / k_tiles) * TM;
                int b_lo, b_hi;
                slice_range(w % slices, b_lo, b_hi);
                for (int mb = b_lo; mb < b_hi; ++mb) {
                    if (!(ok = mbar_wait(&s->empty[stage], phase ^ 1, s, 1))) break;
                    mbar_expect_tx(&s->full_a[stage], A_STAGE);       // rows and columns past the edges arrive as zeros
#pragma unroll
                    for (int j = 0; j < TM / 64; ++j)
                        tma_load_2d(s->a[stage] + j * CHUNK, &map_dy, &s->full_a[stage], n0 + j * 64, mb * KB);
                    // dY streams out of HBM and the ring is only three blocks deep: ask for the block
                    // PREFETCH_BLOCKS ahead to be brought into L2 now
                    if (PREFETCH_BLOCKS > 0 && mb + PREFETCH_BLOCKS < b_hi) {
#pragma unroll
                        for (int j = 0; j < TM / 64; ++j)
                            tma_prefetch_l2_2d(&map_dy, n0 + j * 64, (mb + PREFETCH_BLOCKS) * KB);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc();
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int w = blockIdx.x; ok && w < n_work; w += gridDim.x) {
                int b_lo, b_hi;
                slice_range(w % slices, b_lo, b_hi);
                // A second work item overwrites the accumulators with its first MMA.  That MMA waits
                // for full_b of its stage, on which every decoder warp arrives only after it has read
                // the previous item's accumulators out of tensor memory (program order in the warp).
                for (int mb = b_lo; mb < b_hi; ++mb) {
                    if (!(ok = mbar_wait(&s->full_a[stage], phase, s, 3))) break;
                    if (!(ok = mbar_wait(&s->full_b[stage], phase, s, 4))) break;
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < KB / UMMA_K; ++k) {
                        const uint64_t bdesc = make_mn_major_desc(s->b[stage] + k * (UMMA_K * 128));
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint64_t adesc = make_mn_major_desc(s->a[stage] + h * 2 * CHUNK + k * (UMMA_K * 128));
                            umma_bf16(tmem_base + (uint32_t)(h * TN), adesc, bdesc, idesc, (mb > b_lo || k > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(&s->empty[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit(&s->acc_full);
            }
        }
    } else {
        // ------------------------------------------- decoders (X~ into shared memory), then epilogue
        const int dwarp = warp - 2;
        const int piece = lane & 7, rsub = lane >> 3;          // 8 lanes = one 128-byte row of a chunk; 4 rows per warp
        const int q = warp & 3;                                // TMEM lane quarter for the epilogue
        const int col_part = dwarp >> 2;                       // which EPI_COLS columns of a tile in the epilogue
        uint32_t stage = 0, phase = 0, acc_phase = 0;
        bool ok = true;
        for (int w = blockIdx.x; w < n_work; w += gridDim.x) {
            const int tile = w / slices;
            const int n0 = (tile / k_tiles) * TM, k0 = (tile % k_tiles) * TN;
            int b_lo, b_hi;
            slice_range(w % slices, b_lo, b_hi);
            // Per piece i of this thread (eight per stage: two row quads x four 64-column chunks): where
            // its codes and its group's scale and minimum lie for the first block, advanced by a constant
            // per block; where it goes in the stage (fixed).  Nothing in the stage loop multiplies.
            const uint8_t* pcode[PIECES];
            int gidx[PIECES];
            uint32_t soff[PIECES], rowi[PIECES];
            bool colok[PIECES];
#pragma unroll
            for (int i = 0; i < PIECES; ++i) {
                const int qd = dwarp * PIECES + i, chunk = qd & 3, row = (qd >> 2) * 4 + rsub;
                const int col = k0 + chunk * 64 + piece * 8;
                const int64_t e0 = ((int64_t)b_lo * KB + row) * K + col;
                pcode[i] = packed + (e0 >> 3) * BITS;
                gidx[i] = (int)(e0 >> log2_gs);
                soff[i] = (uint32_t)(chunk * CHUNK + row * 128 + ((piece ^ (row & 7)) << 4));
                rowi[i] = (uint32_t)row;
                colok[i] = col < K;
            }
            const int code_step = KB * (K >> 3) * BITS;            // bytes of codes per 64-row block
            const int group_step = (KB * K) >> log2_gs;            // groups per 64-row block (group_size divides K)
            // The codes, scales and minima of a block are fetched one block ahead of their use, into
            // two register sets that swap roles (the loop body is written out twice).
            uint64_t cd[2][PIECES];
            float sv[2][PIECES], mv[2][PIECES];
            auto fetch = [&](int mb, int set) {
                const uint32_t rows_left = mb < b_hi ? (uint32_t)(M - mb * KB) : 0u;   // > 63 except in the last block of M
#pragma unroll
                for (int i = 0; i < PIECES; ++i) {
                    cd[set][i] = 0; sv[set][i] = 0.0f; mv[set][i] = 0.0f;
                    if (colok[i] && rowi[i] < rows_left) {
                        cd[set][i] = CodePiece<BITS>::ld(pcode[i]);
                        sv[set][i] = __ldg(scale + gidx[i]);
                        mv[set][i] = __ldg(mn + gidx[i]);
                    }
                    pcode[i] += code_step;
                    gidx[i] += group_step;
                }
            };
            auto produce = [&](int mb, int set) {
                const uint32_t rows_left = (uint32_t)(M - mb * KB);
                uint8_t* base = s->b[stage];
                if (BITS <= 2 && log2_gs >= 7) {
                    // pieces 2j and 2j+1 lie in chunks 2c and 2c+1 of one row, i.e. in one group of
                    // 128 or more columns: one table serves both
#pragma unroll
                    for (int i = 0; i < PIECES; i += 2) {
                        uint32_t t_lo, t_hi;
                        group_table<BITS>(sv[set][i], mv[set][i], t_lo, t_hi);
                        const bool rows_ok = rowi[i] < rows_left;
                        uint4 v0 = make_uint4(0u, 0u, 0u, 0u), v1 = v0;
                        if (colok[i] && rows_ok) v0 = decode8_table<BITS>((uint32_t)cd[set][i], t_lo, t_hi);
                        if (colok[i + 1] && rows_ok) v1 = decode8_table<BITS>((uint32_t)cd[set][i + 1], t_lo, t_hi);
                        *reinterpret_cast<uint4*>(base + soff[i]) = v0;
                        *reinterpret_cast<uint4*>(base + soff[i + 1]) = v1;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < PIECES; ++i) {
                        uint4 v = make_uint4(0u, 0u, 0u, 0u);  // rows past M and columns past K contribute nothing
                        if (colok[i] && rowi[i] < rows_left) v = decode8<BITS>(cd[set][i], sv[set][i], mv[set][i]);
                        *reinterpret_cast<uint4*>(base + soff[i]) = v;
                    }
                }
                fence_proxy_async();                           // generic-proxy stores -> visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(&s->full_b[stage]);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            };
            fetch(b_lo, 0);
            for (int mb = b_lo; ok && mb < b_hi; mb += 2) {
                fetch(mb + 1, 1);
                if (ok) ok = mbar_wait_warp(&s->empty[stage], phase ^ 1, s, 2);
                if (!ok) break;
                produce(mb, 0);
                if (mb + 1 >= b_hi) break;
                fetch(mb + 2, 0);
                if (ok) ok = mbar_wait_warp(&s->empty[stage], phase ^ 1, s, 2);
                if (!ok) break;
                produce(mb + 1, 1);
            }
            // ---- epilogue of this work item: accumulators -> dW (fp32, summed over slices)
            if (ok) ok = mbar_wait_warp(&s->acc_full, acc_phase, s, 6);
            if (!ok) continue;
            acc_phase ^= 1;
            tc_fence_after();
#pragma unroll 1
            for (int h = 0; h < 2; ++h) {
                const int row = n0 + h * 128 + q * 32 + lane;
                const uint32_t t_base = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(h * TN + col_part * EPI_COLS);
#pragma unroll 1
                for (int c = 0; c < EPI_COLS / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld32(t_base + (uint32_t)(c * 32), r);
                    tmem_ld_wait();
                    const int col0 = k0 + col_part * EPI_COLS + c * 32;
                    if (row < N) {
                        float* dst = dw + (int64_t)row * ld_dw + col0;
#pragma unroll
                        for (int v = 0; v < 8; ++v)
                            if (col0 + v * 4 < K) red_add_v4(dst + v * 4, r[4 * v], r[4 * v + 1], r[4 * v + 2], r[4 * v + 3]);
                    }
                }
            }
            // the accumulators may be overwritten once every decoder warp is past this point: the
            // next item's first MMA waits for full_b of its first stage, on which each warp arrives
            // only after its reads above (tcgen05.wait::ld) and this fence
            tc_fence_before();
        }
    }

    // ---------------------------------------------------------------- teardown
    __syncwarp();
    if (s->abort) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace dw
}  // namespace act

// ------------------------------------------------------------------- host side
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

constexpr int kMaxDevices = 64;

template <int BITS>
int launch(const CUtensorMap& map, const uint8_t* packed, const float* scale, const float* mn, float* dw,
           int M, int N, int K, int log2_gs, int ld_dw, int slices, int grid, cudaStream_t st)
{
    using namespace act::dw;
    static bool attr_set[kMaxDevices];                       // the shared-memory opt-in is per device
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return ACT_ERR_DEVICE;
    if (!attr_set[dev]) {
        if (cudaFuncSetAttribute(dw_gemm_kernel<BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem)) != cudaSuccess)
            return ACT_ERR_DEVICE;
        attr_set[dev] = true;
    }
    dw_gemm_kernel<BITS><<<grid, THREADS, sizeof(Smem), st>>>(map, packed, scale, mn, dw, M, N, K, log2_gs, ld_dw, slices);
    return cudaGetLastError() == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
}

}  // namespace

extern "C" int act_dw_from_packed(const void* dy, const void* packed, const float* scale, const float* mn,
                                  int bits, int group_size, int M, int N, int K, int ld_dy,
                                  float* dw, int ld_dw, void* stream)
{
    using namespace act::dw;
    if (M < 0 || N < 0 || K < 0) return ACT_ERR_SIZE;
    if (bits != 1 && bits != 2 && bits != 4 && bits != 8) return ACT_ERR_BITS;
    if (group_size < 32 || group_size > 1024 || (group_size & (group_size - 1))) return ACT_ERR_GROUP;
    if (N == 0 || K == 0) return ACT_OK;
    if (!dw) return ACT_ERR_NULL;
    // whole groups per row; 16-byte rows of dY for the tensor map; 16-byte pieces of dW for the vector adds
    if ((K % group_size) || (N & 7) || (ld_dy & 7) || ld_dy < N || (ld_dw & 3) || ld_dw < K || (K & 7)) return ACT_ERR_SIZE;
    if ((uintptr_t)dw & 15) return ACT_ERR_ALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (cudaMemset2DAsync(dw, (size_t)ld_dw * 4, 0, (size_t)K * 4, (size_t)N, st) != cudaSuccess) return ACT_ERR_LAUNCH;
    if (M == 0) return ACT_OK;
    if (!dy || !packed || !scale || !mn) return ACT_ERR_NULL;
    if (((uintptr_t)dy & 15) || ((uintptr_t)packed & 7)) return ACT_ERR_ALIGN;

    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return ACT_ERR_DEVICE;
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)ld_dy * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)KB};
    const cuuint32_t estr[2] = {1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(dy), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) return ACT_ERR_DEVICE;

    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int tiles = ((N + TM - 1) / TM) * ((K + TN - 1) / TN);
    const int m_blocks = (M + KB - 1) / KB;
    // slices of M: enough work items to occupy every SM once, never more slices than blocks
    int slices = tiles >= sms ? 1 : sms / tiles;
    if (slices > m_blocks) slices = m_blocks;
    if (slices < 1) slices = 1;
    const int work = tiles * slices;
    const int grid = work < sms ? work : sms;
    int log2_gs = 0;
    while ((1 << log2_gs) < group_size) ++log2_gs;
    const uint8_t* pk = static_cast<const uint8_t*>(packed);
    switch (bits) {
        case 1: return launch<1>(map, pk, scale, mn, dw, M, N, K, log2_gs, ld_dw, slices, grid, st);
        case 2: return launch<2>(map, pk, scale, mn, dw, M, N, K, log2_gs, ld_dw, slices, grid, st);
        case 4: return launch<4>(map, pk, scale, mn, dw, M, N, K, log2_gs, ld_dw, slices, grid, st);
        default: return launch<8>(map, pk, scale, mn, dw, M, N, K, log2_gs, ld_dw, slices, grid, st);
    }
}

// Abort reason of the last weight-gradient GEMM on the current device (0 = none); synchronises.
extern "C" int act_dw_from_packed_status(unsigned int* out, int clear) {
    if (!out) return ACT_ERR_NULL;
    if (cudaMemcpyFromSymbol(out, act::dw::g_dw_error, sizeof(unsigned int)) != cudaSuccess) return ACT_ERR_DEVICE;
    if (clear) {
        const unsigned int zero = 0;
        if (cudaMemcpyToSymbol(act::dw::g_dw_error, &zero, sizeof(zero)) != cudaSuccess) return ACT_ERR_DEVICE;
    }
    return ACT_OK;
}
