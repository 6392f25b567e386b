// Weight gradient of a linear layer straight from the compressed layer input, sm_100a:
//     dW[n, k] = sum_m dY[m, n] * X~[m, k],   X~[m, k] = bf16(code[m, k] * scale[g] + min[g])
// where X was saved by act_quant_pack as b-bit codes with one (scale, min) per group of G
// consecutive elements of the row-major [M, K] input (G divides K, so a group never leaves its
// row) and dY is bf16 [M, N].  The decoded values are exactly those act_dequant_unpack would
// write as bf16; they are produced inside the GEMM's operand pipeline instead of in HBM.
// Reference: the author's Triton attempt at the same fusion ran at 0.06-0.17x of
// dequantise + cuBLAS (Activation_Compression/test2.ipynb:14-19, 478-491).
//
// One CTA pair (a cluster of two, tcgen05 cta_group::2) per (output tile, slice of M); 576 threads
// per CTA.  A tile is 256 columns of dW (k, the side that has to be decoded: 128 per CTA) by 256,
// 384 or 512 rows (n, the dY side, which TMA delivers).  The decoded operand is the M side of the
// MMA (M = 256 over the pair), dY the N side, so the accumulators hold the tile transposed
// (tensor-memory lane = k, column = n), and each CTA stages only its half of every dY block: the
// pair's tensor cores read both halves.  Against one CTA per 256 x 256 tile this halves the
// decoding per flop at the same dY traffic out of L2 (one CTA per 128 x 512 tile halves the
// decoding too, but doubles that traffic and then waits for L2: 238 us against 208).
//   warp 0       TMA producer (both CTAs): 96 rows of dY x this CTA's half of the tile's columns
//                per stage, as 64 x 96 boxes with the 128-byte swizzle, completion counted on the
//                leader's barrier.  dY is row-major [M, N], so a box lands with the output
//                dimension n contiguous: the "MN-major" operand form of tcgen05.mma.
//   warp 1       MMA issuer (leader CTA only): per stage and K step of 16 rows one
//                tcgen05.mma.cta_group::2.kind::f16 (bf16, M = 256, N = 256) and, for tiles wider
//                than 256, a second one (N = 128 or 256) on the next 256 columns of tensor memory;
//                both operands MN-major.  Its commits free the stage in both CTAs.
//   warps 2..17  (both CTAs) twelve of them decode, the four on the MMA issuer's warp scheduler
//                only drain: read the codes of 96 rows x 128 columns (2 bytes per 8 two-bit
//                codes), look the two bytes of every bf16 value up in the group's table of
//                2^b outputs with a byte permute (the arithmetic of dequant_unpack_kernel), and
//                store 16-byte pieces into the same swizzled MN-major layout a bulk tensor copy of
//                a dense bf16 X would have produced; 8 lanes cover one 128-byte row, so the stores
//                are conflict-free; then arrive on the leader's barrier.  After the last stage the
//                same warps drain their CTA's accumulators and add them to dW with
//                red.global.add.f32 (the 32 lanes of a warp hold 32 consecutive k of one row n:
//                one 128-byte line per instruction): slices of M owned by different pairs sum into
//                the same fp32 tile, which the host zeroes first.
// Every mbarrier wait is bounded; on a timeout the kernel records a reason, tells the other CTA of
// the pair, and leaves.  Bound: bf16 tensor throughput, flops = 2*M*N*K.
#include <cuda.h>

#include "act_common.cuh"

namespace act {
namespace dw {

constexpr int TK = 128;                   // output columns (k) per CTA: the decoded operand, half of the MMA's M = 256
constexpr int TN_MAX = 512;               // output rows (n) per tile at most: two MMAs of N = 256
constexpr int KB = 96;                    // rows of the reduction dimension m per stage
constexpr int UMMA_K = 16;                // K of one tcgen05.mma for 16-bit operands
constexpr int STAGES = 3;
#ifndef ACT_DW_PREFETCH_BLOCKS
#define ACT_DW_PREFETCH_BLOCKS 0
#endif
constexpr int PREFETCH_BLOCKS = ACT_DW_PREFETCH_BLOCKS;   // distance of the L2 prefetch of dY, in 96-row blocks (0: off)
constexpr int CHUNK = KB * 128;           // one 64-column chunk of a stage: KB rows x 128 bytes
constexpr int DY_STAGE = KB * (TN_MAX / 2) * 2;   // 32 KB: this CTA's half of the tile's columns
constexpr int X_STAGE = KB * TK * 2;      // 16 KB
// Warps 2..17 drain the accumulators; twelve of them decode.  The four whose index is 1 modulo 4
// sit on the warp scheduler of the MMA issuer (warp 1) and stay out of the main loop: with decoders
// on its scheduler the issuing thread needed 100 cycles per MMA instead of 70 and the tensor pipe
// ran dry (1250 cycles per 1024 of work).
constexpr int EPI_WARPS = 16;
constexpr int DEC_WARPS = 12;
constexpr int PIECES = (KB * TK / 8) / (DEC_WARPS * 32);  // 16-byte pieces of a stage per decoder thread
constexpr int THREADS = 64 + EPI_WARPS * 32;
static_assert((KB * TK / 8) % (DEC_WARPS * 32) == 0 && PIECES >= 2 && PIECES % 2 == 0, "decoder split");
#ifndef ACT_DW_DEPTH
#define ACT_DW_DEPTH 2
#endif
constexpr int DEPTH = ACT_DW_DEPTH;                       // register sets of fetched codes: blocks in flight + 1
constexpr int TMEM_COLS = 512;
constexpr uint32_t SPIN_LIMIT = 1u << 24;

struct __align__(1024) Smem {
    uint8_t dy[STAGES][DY_STAGE];            // B operand: dY boxes
    uint8_t x[STAGES][X_STAGE];              // A operand: decoded X~
    uint64_t full[STAGES], empty[STAGES], acc_full, acc_free;
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
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r;
}
__device__ __forceinline__ uint32_t cluster_id() {
    uint32_t r; asm volatile("mov.u32 %0, %%clusterid.x;" : "=r"(r)); return r;
}
__device__ __forceinline__ uint32_t n_clusters() {
    uint32_t r; asm volatile("mov.u32 %0, %%nclusterid.x;" : "=r"(r)); return r;
}
// address of the same shared-memory location in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank)); return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" :: "r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" :: "r"(cluster_addr), "r"(v) : "memory");
}
// A wait that runs out records why, raises this CTA's abort flag and the other CTA's (peer_abort:
// its cluster address), so that every role of the pair leaves.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, Smem* s, uint32_t code, uint32_t peer_abort) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (s->abort) return false;
    }
    s->abort = 1;
    st_cluster_u32(peer_abort, 1u);
    atomicExch(&g_dw_error, code);
    return false;
}
// warp-wide: lane 0 polls, everybody learns the outcome
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, Smem* s, uint32_t code, uint32_t peer_abort) {
    uint32_t ok = 1;
    if ((threadIdx.x & 31) == 0) ok = mbar_wait(bar, parity, s, code, peer_abort) ? 1u : 0u;
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// tile load whose completion bytes are counted on an mbarrier of the pair's leader
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t leader_bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(smem_u32(dst)), "l"(map), "r"(leader_bar), "r"(c0), "r"(c1) : "memory");
}
// requests a tile into L2 only (no shared-memory destination, nothing to wait for)
__device__ __forceinline__ void tma_prefetch_l2_2d(const CUtensorMap* map, int c0, int c1) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" :: "l"(map), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(dst_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_bf16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// the same with the accumulate predicate fixed to true (no predicate to compute per instruction)
__device__ __forceinline__ void umma_bf16_pair_acc(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.u32 p, 1, 1;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc) : "memory");
}
// arrives, once the pair's MMAs issued so far are done, on the barrier at this offset in both CTAs
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 :: "r"(smem_u32(bar)), "h"(both) : "memory");
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
__device__ __forceinline__ void red_add(float* p, uint32_t a) {
    asm volatile("red.global.add.f32 [%0], %1;" :: "l"(p), "f"(__uint_as_float(a)) : "memory");
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
// fp32 accumulate, A and B bf16, both MN-major, M = 256 (both CTAs together), N = n
__host__ __device__ constexpr uint32_t make_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) |
           ((uint32_t)(n >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
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
template <> struct CodePiece<1> { typedef uint32_t reg_t; static __device__ __forceinline__ reg_t ld(const uint8_t* p) { return __ldg(p); } };
template <> struct CodePiece<2> { typedef uint32_t reg_t; static __device__ __forceinline__ reg_t ld(const uint8_t* p) { return __ldg(reinterpret_cast<const uint16_t*>(p)); } };
template <> struct CodePiece<4> { typedef uint32_t reg_t; static __device__ __forceinline__ reg_t ld(const uint8_t* p) { return __ldg(reinterpret_cast<const uint32_t*>(p)); } };
template <> struct CodePiece<8> { typedef uint64_t reg_t; static __device__ __forceinline__ reg_t ld(const uint8_t* p) { return __ldg(reinterpret_cast<const unsigned long long*>(p)); } };

// ------------------------------------------------------------------ the kernel
// Work item w = (tile, slice), taken by pair w % pairs: tile = w / slices = nt * k_tiles + kt, so
// the pairs that run together share their columns of dY (L2 serves all but the first read of a
// block); slice = w % slices is a contiguous run of 96-row blocks of M.  nj = width of a tile in
// 128-row units of n; a tile is 256 columns of k wide, 128 per CTA.
template <int BITS>
__global__ void __launch_bounds__(THREADS, 1)
dw_gemm_kernel(const __grid_constant__ CUtensorMap map_dy, const uint8_t* __restrict__ packed,
               const float* __restrict__ scale, const float* __restrict__ mn, float* __restrict__ dw,
               int M, int N, int K, int log2_gs, int ld_dw, int slices, int nj)
{
    extern __shared__ __align__(1024) uint8_t smem_raw_dw[];
    Smem* s = reinterpret_cast<Smem*>(smem_raw_dw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile_n = 128 * nj;
    const int n_tiles = (N + tile_n - 1) / tile_n, k_tiles = (K + 2 * TK - 1) / (2 * TK);
    const int n_work = n_tiles * k_tiles * slices;
    const uint32_t rank = cluster_ctarank();                  // 0 = leader of the pair
    const int first = (int)cluster_id(), stride = (int)n_clusters();
    const uint32_t peer_abort = map_to_cta(smem_u32((const void*)&s->abort), rank ^ 1u);
    const int m_blocks = (M + KB - 1) / KB;

    if (smem_u32(s) & 1023u) {                                // the swizzled tiles need this alignment
        if (threadIdx.x == 0) atomicExch(&g_dw_error, 5u);
        return;
    }
    if (threadIdx.x == 0) {
        // `full` of the leader collects, per stage, the producer's arrival (with the byte count of both
        // CTAs' dY boxes) and the decoder warps of both CTAs: the MMA issuer then waits once per stage
        // (a wait that is already satisfied still costs it about 230 cycles)
        for (int i = 0; i < STAGES; ++i) { mbar_init(&s->full[i], 1 + 2 * DEC_WARPS); mbar_init(&s->empty[i], 1); }
        mbar_init(&s->acc_full, 1);
        mbar_init(&s->acc_free, 2 * EPI_WARPS);             // leader's: every draining warp of the pair has read its part
        s->abort = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc_pair(&s->tmem_base, TMEM_COLS);  // the same warp of both CTAs
    tc_fence_before();
    cluster_sync_all();                                       // barriers of both CTAs exist from here on
    tc_fence_after();
    const uint32_t tmem_base = s->tmem_base;

    // blocks [b_lo, b_hi) of 96 rows belong to slice sl: as even a split as whole blocks allow
    auto slice_range = [&](int sl, int& b_lo, int& b_hi) {
        const int per = m_blocks / slices, extra = m_blocks % slices;
        b_lo = sl * per + (sl < extra ? sl : extra);
        b_hi = b_lo + per + (sl < extra ? 1 : 0);
    };

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (dY, both CTAs)
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            // This CTA's columns of the tile: its half of the first 256 (two boxes of 64), and its
            // half of what lies beyond them (nj = 3: one box; nj = 4: two).
            const int boxes_hi = nj - 2;
            for (int w = first; ok && w < n_work; w += stride) {
                const int tile = w / slices, n0 = (tile / k_tiles) * tile_n;
                const int n_lo = n0 + (int)rank * 128, n_hi = n0 + 256 + (int)rank * 64 * boxes_hi;
                int b_lo, b_hi;
                slice_range(w % slices, b_lo, b_hi);
                for (int mb = b_lo; mb < b_hi; ++mb) {
                    if (!(ok = mbar_wait(&s->empty[stage], phase ^ 1, s, 1, peer_abort))) break;
                    // the leader's barrier counts the bytes of both CTAs' boxes (rows and columns past
                    // the edges arrive as zeros)
                    if (rank == 0) mbar_expect_tx(&s->full[stage], (uint32_t)(2 * nj * CHUNK));
                    const uint32_t bar = map_to_cta(smem_u32(&s->full[stage]), 0);
                    tma_load_2d_pair(s->dy[stage], &map_dy, bar, n_lo, mb * KB);
                    tma_load_2d_pair(s->dy[stage] + CHUNK, &map_dy, bar, n_lo + 64, mb * KB);
                    for (int j = 0; j < boxes_hi; ++j)
                        tma_load_2d_pair(s->dy[stage] + (2 + j) * CHUNK, &map_dy, bar, n_hi + j * 64, mb * KB);
                    // ask for the block PREFETCH_BLOCKS ahead to be brought into L2 now (off by default:
                    // with several pairs reading the same columns it only added requests)
                    if (PREFETCH_BLOCKS > 0 && mb + PREFETCH_BLOCKS < b_hi) {
                        tma_prefetch_l2_2d(&map_dy, n_lo, (mb + PREFETCH_BLOCKS) * KB);
                        tma_prefetch_l2_2d(&map_dy, n_lo + 64, (mb + PREFETCH_BLOCKS) * KB);
                        for (int j = 0; j < boxes_hi; ++j)
                            tma_prefetch_l2_2d(&map_dy, n_hi + j * 64, (mb + PREFETCH_BLOCKS) * KB);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            // tail: every slot handed out has come back, i.e. no arrival from the leader's commits
            // is still on its way to this CTA's barriers when the CTA leaves
            for (int i = 0; ok && i < STAGES; ++i) {
                ok = mbar_wait(&s->empty[stage], phase ^ 1, s, 7, peer_abort);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer (leader only)
        if (lane == 0 && rank == 0) {
            constexpr uint32_t idesc256 = make_idesc(256), idesc128 = make_idesc(128);
            const uint32_t idesc_hi = (nj == 4) ? idesc256 : idesc128;     // the MMA on columns 256.. of a tile wider than 256
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            const uint64_t adesc0 = make_mn_major_desc(s->x[0]), bdesc0 = make_mn_major_desc(s->dy[0]);
            int items_done = 0;
            for (int w = first; ok && w < n_work; w += stride) {
                int b_lo, b_hi;
                slice_range(w % slices, b_lo, b_hi);
                // A later work item overwrites the accumulators with its first MMA: every warp of the
                // pair that drains them has arrived on acc_free once it was done with the previous item.
                if (items_done > 0 && !(ok = mbar_wait(&s->acc_free, (uint32_t)((items_done - 1) & 1), s, 8, peer_abort))) break;
                ++items_done;
                // The issuing thread is the narrowest part of the kernel.  Measured with cycle stamps: an
                // MMA costs it about 70 cycles to issue (100 with decoder warps on its scheduler), a
                // wait that is already satisfied 250-300, a commit 80, against 128 cycles of tensor
                // work per MMA; the tensor pipe holds only two or three MMAs beyond the one it
                // executes.  Hence twelve MMAs per wait (96-row stages), the wait for the NEXT stage
                // between the two halves of this stage's MMAs, the commit after the second half, and
                // the stage's descriptors (start address field in 16-byte units) computed before the wait.
                bool have = false;                               // the current stage's wait is already done
                for (int mb = b_lo; mb < b_hi; ++mb) {
                    const uint64_t adesc = adesc0 + (uint64_t)(stage * (X_STAGE >> 4));
                    const uint64_t bdesc = bdesc0 + (uint64_t)(stage * (DY_STAGE >> 4));
                    const uint64_t bdesc_hi = bdesc + (uint64_t)((2 * CHUNK) >> 4);
                    const uint32_t acc0 = mb > b_lo ? 1u : 0u;
                    const uint32_t next_stage = stage + 1 == STAGES ? 0u : stage + 1;
                    const uint32_t next_phase = stage + 1 == STAGES ? phase ^ 1u : phase;
                    if (!have && !(ok = mbar_wait(&s->full[stage], phase, s, 3, peer_abort))) break;
                    tc_fence_after();
                    constexpr uint64_t KSTEP = (uint64_t)((UMMA_K * 128) >> 4);
                    constexpr int KS = KB / UMMA_K;
                    umma_bf16_pair(tmem_base, adesc, bdesc, idesc256, acc0);
                    if (nj > 2) umma_bf16_pair(tmem_base + 256u, adesc, bdesc_hi, idesc_hi, acc0);
#pragma unroll
                    for (int k = 1; k < KS / 2; ++k) {
                        umma_bf16_pair_acc(tmem_base, adesc + k * KSTEP, bdesc + k * KSTEP, idesc256);
                        if (nj > 2) umma_bf16_pair_acc(tmem_base + 256u, adesc + k * KSTEP, bdesc_hi + k * KSTEP, idesc_hi);
                    }
                    have = mb + 1 < b_hi;
                    if (have && !(ok = mbar_wait(&s->full[next_stage], next_phase, s, 4, peer_abort))) break;
                    tc_fence_after();
#pragma unroll
                    for (int k = KS / 2; k < KS; ++k) {
                        umma_bf16_pair_acc(tmem_base, adesc + k * KSTEP, bdesc + k * KSTEP, idesc256);
                        if (nj > 2) umma_bf16_pair_acc(tmem_base + 256u, adesc + k * KSTEP, bdesc_hi + k * KSTEP, idesc_hi);
                    }
                    umma_commit_pair(&s->empty[stage]);        // frees the slot in both CTAs
                    stage = next_stage; phase = next_phase;
                }
                if (!ok) break;
                umma_commit_pair(&s->acc_full);                // both CTAs' accumulators are complete
            }
        }
    } else {
        // ------------------------------------------- decoders (X~ into shared memory), then epilogue
        const int ew = warp - 2;                               // 0..15
        const bool decodes = (ew & 3) != 3;                    // warps 5, 9, 13, 17 only drain
        const int dwarp = (ew >> 2) * 3 + (ew & 3);            // 0..11 among the decoders
        const int piece = lane & 7, rsub = lane >> 3;          // 8 lanes = one 128-byte row of a chunk; 4 rows per warp
        const int q = warp & 3;                                // TMEM lane quarter for the epilogue
        const int col_part = ew >> 2;                          // which 32-column blocks of the accumulators in the epilogue
        uint32_t stage = 0, phase = 0, acc_phase = 0;
        bool ok = true;
        const uint32_t leader_full = map_to_cta(smem_u32(&s->full[0]), 0);
        for (int w = first; w < n_work; w += stride) {
            const int tile = w / slices;
            const int n0 = (tile / k_tiles) * tile_n, k0 = (tile % k_tiles) * (2 * TK) + (int)rank * TK;
            int b_lo, b_hi;
            slice_range(w % slices, b_lo, b_hi);
            // Per piece i of this thread (PIECES per stage, two neighbouring chunks of one row each pair): where its codes and its
            // group's scale and minimum lie for the first block, advanced by a constant per block;
            // where it goes in the stage (fixed).  Nothing in the stage loop multiplies.
            const uint8_t* pcode[PIECES];
            int gidx[PIECES];
            uint32_t soff[PIECES], rowi[PIECES];
            bool colok[PIECES];
#pragma unroll
            for (int i = 0; i < PIECES; ++i) {
                const int qd = dwarp * PIECES + i, chunk = qd & 1, row = (qd >> 1) * 4 + rsub;
                const int col = k0 + chunk * 64 + piece * 8;
                const int64_t e0 = ((int64_t)b_lo * KB + row) * K + col;
                pcode[i] = packed + (e0 >> 3) * BITS;
                gidx[i] = (int)(e0 >> log2_gs);
                soff[i] = (uint32_t)(chunk * CHUNK + row * 128 + ((piece ^ (row & 7)) << 4));
                rowi[i] = (uint32_t)row;
                colok[i] = col < K;
            }
            const int code_step = KB * (K >> 3) * BITS;            // bytes of codes per 96-row block
            const int group_step = (KB * K) >> log2_gs;            // groups per 96-row block (group_size divides K)
            // The codes, scales and minima of a block are fetched DEPTH - 1 blocks ahead of their use
            // (a block of 96 rows is 1536 cycles of MMA), into
            // register sets that take turns (the loop body is unrolled over them).
            typedef typename CodePiece<BITS>::reg_t code_t;       // 32 bits hold eight codes of up to four bits
            code_t cd[DEPTH][PIECES];
            float sv[DEPTH][PIECES], mv[DEPTH][PIECES];
            auto fetch = [&](int mb, int set) {
                const uint32_t rows_left = mb < b_hi ? (uint32_t)(M - mb * KB) : 0u;   // > 31 except in the last block of M
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
                uint8_t* base = s->x[stage];
                if (BITS <= 2 && log2_gs >= 7) {
                    // pieces 2j and 2j+1 lie in chunks 0 and 1 of one row, i.e. in one group of
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
                if (lane == 0) mbar_arrive_cluster(leader_full + stage * (uint32_t)sizeof(uint64_t));
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            };
            if (decodes) {
#pragma unroll
            for (int d = 0; d < DEPTH - 1; ++d) fetch(b_lo + d, d);
            for (int mb = b_lo; ok && mb < b_hi; mb += DEPTH) {
#pragma unroll
                for (int d = 0; d < DEPTH; ++d) {
                    if (!ok || mb + d >= b_hi) break;
                    fetch(mb + d + DEPTH - 1, (d + DEPTH - 1) % DEPTH);
                    ok = mbar_wait_warp(&s->empty[stage], phase ^ 1, s, 2, peer_abort);
                    if (ok) produce(mb + d, d);
                }
            }
            }
            // ---- epilogue of this work item: accumulators (lane = k, column = n) -> dW[n, k], fp32,
            // summed over slices.  A warp owns the 32 lanes of its quarter and every other 32-column
            // block; for one column its lanes add to 32 consecutive floats of one row of dW.
            if (ok) ok = mbar_wait_warp(&s->acc_full, acc_phase, s, 6, peer_abort);
            if (!ok) continue;
            acc_phase ^= 1;
            tc_fence_after();
            const int kk = k0 + q * 32 + lane;
#pragma unroll 1
            for (int cb = col_part; cb < 4 * nj; cb += EPI_WARPS / 4) {
                uint32_t r[32];
                tmem_ld32(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(cb * 32), r);
                tmem_ld_wait();
                const int nn = n0 + cb * 32;
                if (kk < K) {
                    float* dst = dw + (int64_t)nn * ld_dw + kk;
#pragma unroll
                    for (int v = 0; v < 32; ++v)
                        if (nn + v < N) red_add(dst + (int64_t)v * ld_dw, r[v]);
                }
            }
            // this warp is done with the item's accumulators (tcgen05.wait::ld above): tell the issuer
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&s->acc_free), 0));
        }
    }

    // ---------------------------------------------------------------- teardown
    __syncwarp();                                             // lanes that had no role wait for the one that had
    if (s->abort) {
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    cluster_sync_all();                                       // neither CTA's memory is needed by the other any more
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem_base, TMEM_COLS);
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

// Per-device state of one instantiation: the shared-memory opt-in (a per-device attribute of the
// kernel) and how many CTA pairs the device holds at once.
template <int BITS>
int pairs_resident(int* out) {
    using namespace act::dw;
    static int pairs[kMaxDevices];                           // 0: not yet set up on that device
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return ACT_ERR_DEVICE;
    if (!pairs[dev]) {
        int sms = 0;
        if (cudaFuncSetAttribute(dw_gemm_kernel<BITS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem)) != cudaSuccess)
            return ACT_ERR_DEVICE;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms < 2) return ACT_ERR_DEVICE;
        cudaLaunchConfig_t q = {};
        q.gridDim = dim3(2u * (unsigned)(sms / 2), 1, 1);
        q.blockDim = dim3(THREADS, 1, 1);
        q.dynamicSmemBytes = sizeof(Smem);
        cudaLaunchAttribute qa[1];
        qa[0].id = cudaLaunchAttributeClusterDimension;
        qa[0].val.clusterDim.x = 2; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
        q.attrs = qa; q.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, dw_gemm_kernel<BITS>, &q) != cudaSuccess || n <= 0) {
            (void)cudaGetLastError();
            n = sms / 2;
        }
        pairs[dev] = n < sms / 2 ? n : sms / 2;
    }
    *out = pairs[dev];
    return ACT_OK;
}

template <int BITS>
int launch(const CUtensorMap& map, const uint8_t* packed, const float* scale, const float* mn, float* dw,
           int M, int N, int K, int log2_gs, int ld_dw, int nj, cudaStream_t st)
{
    using namespace act::dw;
    int resident = 0;
    const int rc = pairs_resident<BITS>(&resident);
    if (rc != ACT_OK) return rc;
    const int tiles = ((N + 128 * nj - 1) / (128 * nj)) * ((K + 2 * TK - 1) / (2 * TK));
    const int m_blocks = (M + KB - 1) / KB;
    // slices of M: enough work items to occupy every pair once, never more slices than blocks
    int slices = tiles >= resident ? 1 : resident / tiles;
    if (slices > m_blocks) slices = m_blocks;
    if (slices < 1) slices = 1;
    const int work = tiles * slices;
    const int clusters = work < resident ? work : resident;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2u * (unsigned)clusters, 1, 1);
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = sizeof(Smem);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, dw_gemm_kernel<BITS>, map, packed, scale, mn, dw, M, N, K, log2_gs, ld_dw, slices, nj) != cudaSuccess) {
        (void)cudaGetLastError();
        return ACT_ERR_LAUNCH;
    }
    return ACT_OK;
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
    // whole groups per row; 16-byte rows of dY for the tensor map
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

    // width of a tile in 128-row units of n: the least padded of 512, 384 and 256, the widest on a tie
    int nj = 4;
    for (int c = 3; c >= 2; --c)
        if (((N + 128 * c - 1) / (128 * c)) * c < ((N + 128 * nj - 1) / (128 * nj)) * nj) nj = c;
    int log2_gs = 0;
    while ((1 << log2_gs) < group_size) ++log2_gs;
    const uint8_t* pk = static_cast<const uint8_t*>(packed);
    switch (bits) {
        case 1: return launch<1>(map, pk, scale, mn, dw, M, N, K, log2_gs, ld_dw, nj, st);
        case 2: return launch<2>(map, pk, scale, mn, dw, M, N, K, log2_gs, ld_dw, nj, st);
        case 4: return launch<4>(map, pk, scale, mn, dw, M, N, K, log2_gs, ld_dw, nj, st);
        default: return launch<8>(map, pk, scale, mn, dw, M, N, K, log2_gs, ld_dw, nj, st);
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
