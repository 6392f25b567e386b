// FP8 (e4m3) GEMM with per-row / per-column fp32 scales and bf16 output, sm_100a:
//     C[m,n] = bf16( (sum_k A[m,k] * B[k,n]) * sa[m] * sb[n] )
//
// Two kernels.  Problems with more than one 128-row block run on CTA pairs (namespace pair
// below: tcgen05.mma.cta_group::2 on 256 x 256 tiles); single-row-block problems, and callers
// that pass ACT_GEMM_SINGLE_CTA, run the kernel described here:
// one persistent CTA per SM, 320 threads in three roles:
//   warp 0      TMA producer: one lane issues cp.async.bulk.tensor loads of the
//               128x128 A tile and the 256x128 B^T tile of a k-block into a
//               4-stage shared-memory ring (128-byte swizzle), mbarrier-tracked;
//   warp 1      MMA issuer: one lane issues tcgen05.mma (kind::f8f6f4, M=128,
//               N=256, K=32) with both operands from shared memory and the fp32
//               accumulator in tensor memory; tcgen05.commit releases ring slots
//               and hands finished accumulators to the epilogue;
//   warps 2..9  epilogue: tcgen05.ld the accumulator (two 256-column buffers, so
//               the next tile's MMAs overlap this tile's epilogue; loads of the
//               next 32 columns overlap the arithmetic of the current ones),
//               apply the scales, convert to bf16, store 16-byte vectors.
// No TMA multicast is used anywhere.  Every mbarrier wait is bounded: after the
// limit the kernel raises an abort flag, records an error word, drains, frees
// its tensor memory and returns.
//
// B may be [N,K] (K contiguous, the layout of nn.Linear weights) or [K,N], the layout of
// the reference's Triton_Linear (Activation_Compression/triton_kernel/linear.py:43-95).
// The CTA-pair kernel reads either in place ([K,N] as an MN-major tensor-core operand);
// the lone-CTA kernel takes [N,K] and has a [K,N] operand transposed into the caller's
// workspace first.
//
// Bound: FP8 tensor throughput; flops = 2*M*N*K.
#include <cuda.h>

#include "act_common.cuh"

namespace act {
namespace gemm {

constexpr int BM = 128, BN = 256, BK = 128;     // CTA tile; BK bytes = one 128-byte swizzle row
constexpr int UMMA_K = 32;                      // K of one tcgen05.mma for 8-bit operands
constexpr int STAGES = 4;
constexpr int A_STAGE = BM * BK, B_STAGE = BN * BK;
constexpr int EPI_WARPS = 8;                    // two warps per TMEM lane quarter, 128 columns each
constexpr int THREADS = 64 + EPI_WARPS * 32;
constexpr int TMEM_COLS = 512;                  // two fp32 accumulators of 256 columns
constexpr uint32_t SPIN_LIMIT = 1u << 24;       // polls of one mbarrier before giving up

struct __align__(1024) Smem {
    uint8_t a[STAGES][A_STAGE];
    uint8_t b[STAGES][B_STAGE];
    float sb[2][BN];                            // column scales of the tile in each accumulator buffer
    uint8_t cstage[EPI_WARPS][32 * 64];         // per warp: 32 rows x 32 bf16, 16-byte pieces xor-swizzled
    uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
    uint32_t tmem_base;
    volatile uint32_t abort;
};

__device__ unsigned int g_gemm_error = 0;       // last abort reason (0 = none)

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
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
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (after raising the abort flag) when the barrier did
// not flip within the limit or another role has already aborted.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, Smem* s, uint32_t code) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (s->abort) return false;
    }
    s->abort = 1;
    atomicExch(&g_gemm_error, code);
    return false;
}
// Warp-wide bounded wait: lane 0 polls (with a short sleep between polls, so the 256
// epilogue threads do not flood the shared-memory pipe), the outcome is broadcast.
__device__ __forceinline__ bool mbar_wait_warp(uint64_t* bar, uint32_t parity, Smem* s, uint32_t code) {
    uint32_t ok = 1;
    if ((threadIdx.x & 31) == 0) {
        ok = 0;
        for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
            if (mbar_try_wait(bar, parity)) { ok = 1; break; }
            if (s->abort) break;
            __nanosleep(32);
        }
        if (!ok && !s->abort) { s->abort = 1; atomicExch(&g_gemm_error, code); }
    }
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
// bulk tensor store of a 2-D box from shared memory (async proxy); the box is clipped at
// the tensor's edges, so partial tiles need no guards
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
                 :: "l"(map), "r"(smem_u32(src)), "r"(c0), "r"(c1) : "memory");
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                 :: "r"(smem_u32(dst_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives on the mbarrier once all tcgen05.mma issued so far by this thread are done
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 :: "r"(smem_u32(bar)) : "memory");
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

// Shared-memory matrix descriptor of an operand tile stored as rows of 128 bytes with the
// 128-byte swizzle (what the TMA box writes): start address >> 4, stride between 8-row groups
// 1024 bytes, descriptor version 1, layout type 2 (128-byte swizzle).  For a K-major tile the
// rows are the M/N index and the leading-dimension offset is unused; the same bits describe an
// MN-major tile of one 128-byte chunk (rows = K index), which is how a [K,N] B tile is read.
__device__ __forceinline__ uint64_t make_kmajor_desc(const void* tile) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_u32(tile) & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;                         // leading byte offset (ignored), encoded 1
    d |= (uint64_t)(1024 >> 4) << 32;               // stride byte offset
    d |= (uint64_t)1 << 46;                         // descriptor version
    d |= (uint64_t)2 << 61;                         // SWIZZLE_128B
    return d;
}
// Instruction descriptor: fp32 accumulate, A and B e4m3, both K-major, N>>3, M>>4.
__host__ __device__ constexpr uint32_t make_idesc() {
    return (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (0u << 16) |
           ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// ------------------------------------------------------------------ the kernel
__global__ void __launch_bounds__(THREADS, 1)
fp8_gemm_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_bt,
                const __grid_constant__ CUtensorMap map_c,
                const float* __restrict__ sa, const float* __restrict__ sb, int M, int N, int K)
{
    extern __shared__ uint8_t smem_raw[];
    Smem* s = reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN;
    const int n_work = m_tiles * n_tiles;
    const int k_blocks = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&s->full[i], 1); mbar_init(&s->empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&s->acc_full[i], 1); mbar_init(&s->acc_empty[i], EPI_WARPS); }
        s->abort = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(&s->tmem_base, TMEM_COLS);      // whole warp, writes the base address to smem
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = s->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int w = blockIdx.x; ok && w < n_work; w += gridDim.x) {
                const int m0 = (w / n_tiles) * BM, n0 = (w % n_tiles) * BN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!(ok = mbar_wait(&s->empty[stage], phase ^ 1, s, 1))) break;
                    mbar_expect_tx(&s->full[stage], A_STAGE + B_STAGE);   // out-of-range parts arrive as zeros
                    tma_load_2d(s->a[stage], &map_a, &s->full[stage], kb * BK, m0);
                    tma_load_2d(s->b[stage], &map_bt, &s->full[stage], kb * BK, n0);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc();
            uint32_t stage = 0, phase = 0, acc_phase[2] = {0, 0};
            bool ok = true;
            int t = 0;
            for (int w = blockIdx.x; ok && w < n_work; w += gridDim.x, ++t) {
                const int buf = t & 1;
                if (!(ok = mbar_wait(&s->acc_empty[buf], acc_phase[buf] ^ 1, s, 2))) break;
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!(ok = mbar_wait(&s->full[stage], phase, s, 3))) break;
                    tc_fence_after();
                    const uint64_t adesc = make_kmajor_desc(s->a[stage]);
                    const uint64_t bdesc = make_kmajor_desc(s->b[stage]);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)      // +32 bytes along K = +2 in the address field
                        umma_f8(d, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) ? 1u : 0u);
                    umma_commit(&s->empty[stage]);             // slot is free once these MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit(&s->acc_full[buf]);                // accumulator complete
                acc_phase[buf] ^= 1;
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int q = warp & 3;                                // TMEM lane quarter this warp may read
        const int half = (warp - 2) >> 2;                      // which 128 columns of the tile
        const int etid = threadIdx.x - 64;                     // 0..255 among the epilogue threads
        uint32_t full_phase[2] = {0, 0};
        bool ok = true;
        int t = 0;
        // Every epilogue warp walks every tile even after an abort (skipping the work), so
        // that nobody is left waiting alone at the named barrier below.
        for (int w = blockIdx.x; w < n_work; w += gridDim.x, ++t) {
            const int buf = t & 1;
            const int m0 = (w / n_tiles) * BM, n0 = (w % n_tiles) * BN;
            // stage the tile's 256 column scales while the MMAs are still running
            s->sb[buf][etid] = (n0 + etid < N) ? __ldg(sb + n0 + etid) : 0.0f;
            asm volatile("bar.sync 1, %0;" :: "n"(EPI_WARPS * 32) : "memory");
            const int row = m0 + q * 32 + lane;
            const float sa_row = row < M ? __ldg(sa + row) : 0.0f;
            const f32x2 sa2 = pack2(sa_row, sa_row);
            if (ok) ok = mbar_wait_warp(&s->acc_full[buf], full_phase[buf], s, 4);
            if (!ok) continue;
            full_phase[buf] ^= 1;
            tc_fence_after();
            const uint32_t t_base = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + half * 128);
            const float* sb_s = s->sb[buf] + half * 128;
            uint32_t r[2][32];
            tmem_ld32(t_base, r[0]);
#pragma unroll
            for (int chunk = 0; chunk < 4; ++chunk) {
                tmem_ld_wait();
                if (chunk + 1 < 4) tmem_ld32(t_base + (uint32_t)((chunk + 1) * 32), r[(chunk + 1) & 1]);
                else {
                    // the accumulator now lives in registers: hand the buffer back early
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&s->acc_empty[buf]);
                }
                const uint32_t* rc = r[chunk & 1];
                const int col0 = n0 + half * 128 + chunk * 32;
                // scale, convert, and park the lane's 32 columns (64 bytes) in shared memory;
                // piece v of row l sits at slot v ^ ((l >> 1) & 3): conflict-free both ways
                uint8_t* my_stage = s->cstage[warp - 2];
                uint32_t o[4][4];
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    const float4 s0 = *reinterpret_cast<const float4*>(sb_s + chunk * 32 + v * 8);
                    const float4 s1 = *reinterpret_cast<const float4*>(sb_s + chunk * 32 + v * 8 + 4);
                    const f32x2 sc[4] = {pack2(s0.x, s0.y), pack2(s0.z, s0.w), pack2(s1.x, s1.y), pack2(s1.z, s1.w)};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        // (acc * sa) * sb, each product rounded to fp32, two columns per instruction
                        uint32_t lo, hi;
                        unpack2u(mul2_rn(mul2_rn(pack2u(rc[v * 8 + 2 * i], rc[v * 8 + 2 * i + 1]), sa2), sc[i]), lo, hi);
                        const __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(lo), __uint_as_float(hi));
                        o[v][i] = *reinterpret_cast<const uint32_t*>(&p);
                    }
                }
                // the previous chunk's bulk store must have read the stage before it is rewritten
                if (lane == 0) tma_store_wait_read();
                __syncwarp();
#pragma unroll
                for (int v = 0; v < 4; ++v)
                    *reinterpret_cast<uint4*>(my_stage + lane * 64 + ((v ^ ((lane >> 1) & 3)) << 4)) =
                        make_uint4(o[v][0], o[v][1], o[v][2], o[v][3]);
                // the 32 x 32 chunk leaves as one bulk tensor store (64-byte swizzle = the xor
                // pattern above); rows and columns past the edge of C are clipped by the copy
                fence_proxy_async();
                __syncwarp();
                if (lane == 0 && col0 < N && m0 + q * 32 < M) tma_store_2d(&map_c, my_stage, col0, m0 + q * 32);
            }
        }
        if (lane == 0) tma_store_wait_all();        // all of this warp's stores are complete before exit
    }

    // ---------------------------------------------------------------- teardown
    if (s->abort) {
        // give copies and MMAs still in flight time to land before the memory is released
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ===================================================================== CTA-pair kernel
// Two CTAs on the two SMs of one TPC (a cluster of two) compute one 256 x 256 tile with
// tcgen05.mma.cta_group::2: each CTA stages its own 128 rows of A and its own 128 rows of
// B^T (32 KB per k-block instead of the 48 KB a lone CTA needs for 128 x 256), the tensor
// cores of the pair exchange the B halves over the SM-to-SM link, and each CTA keeps the
// 128 x 256 accumulator of its own rows in its own tensor memory.  L2-to-SM traffic per
// flop drops by a third, which is what bounds the lone-CTA kernel on short-K shapes.
//
// Roles per CTA (320 threads): warp 0 = TMA producer (both CTAs load; the loads carry
// .cta_group::2 so that their bytes are counted on the leader's mbarrier; no multicast),
// warp 1 = MMA issuer (rank 0 of the pair only; its commits arrive on the barriers of both
// CTAs), warps 2..9 = epilogue (each CTA drains its own accumulator; 32 x 64 bf16 pieces go
// through a swizzled staging buffer per warp into bulk tensor stores of full 128-byte rows).
// Every wait is bounded as in the lone-CTA kernel.
namespace pair {

constexpr int BM_CTA = 128;                     // rows of A (and of B^T) staged per CTA
constexpr int BN = 256, BK = 128;
constexpr int TILE_M = 2 * BM_CTA;              // rows of C per pair
// Six ring slots of 32 KB and one 4 KB staging buffer per epilogue warp fill the SM's 227 KB.
// Measured on the three evaluation shapes: five slots with two staging buffers per warp ran
// 1-2 % slower (the ring hides L2 latency, the second staging buffer hid nothing), and handing
// each cluster one contiguous run of tiles instead of dealing them out round-robin 1-3 % slower.
constexpr int STAGES = 6;
constexpr int EPI_BUFS = 1;                     // staging buffers per epilogue warp
constexpr int A_STAGE = BM_CTA * BK, B_STAGE = BM_CTA * BK;
constexpr int PIECE_BYTES = 32 * 128;           // 32 rows x 64 bf16

struct __align__(1024) Smem {
    uint8_t a[STAGES][A_STAGE];
    uint8_t b[STAGES][B_STAGE];
    uint8_t cstage[EPI_WARPS][EPI_BUFS][PIECE_BYTES];   // 128-byte rows, 16-byte pieces xor-swizzled by row & 7
    float sb[2][BN];
    uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
    uint32_t tmem_base;
    volatile uint32_t abort;
};
static_assert(sizeof(Smem) <= 227 * 1024, "shared memory of the pair kernel exceeds one SM");

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
// Arrival on an mbarrier of (possibly) the other CTA of the pair.  It orders nothing but the
// tensor-memory loads before it, which tcgen05.wait::ld and the tcgen05 fence already did, so it
// carries the default CTA-scope release: a cluster-scope release made every accumulator hand-back
// wait about 3000 cycles for the thread's earlier stores.
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" :: "r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void st_cluster_u32(uint32_t cluster_addr, uint32_t v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" :: "r"(cluster_addr), "r"(v) : "memory");
}
// tile load whose completion bytes are counted on an mbarrier of the pair's leader
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, uint32_t leader_bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
                 " [%0], [%1, {%3, %4}], [%2];"
                 :: "r"(smem_u32(dst)), "l"(map), "r"(leader_bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void umma_f8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
                 :: "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// arrives, once the pair's MMAs issued so far are done, on the barrier at this offset in both CTAs
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 :: "r"(smem_u32(bar)), "h"(both) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;"
                 :: "r"(smem_u32(dst_smem)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" :: "r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tma_store_wait_read_keep(int keep) {
    if (keep == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
    else           asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
}
// fp32 accumulate, A and B e4m3, both K-major, N = 256, M = 256 (both CTAs together)
__host__ __device__ constexpr uint32_t make_idesc_pair() {
    return (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(TILE_M >> 4) << 24);
}

template <typename S>
__device__ __forceinline__ bool wait_bar(uint64_t* bar, uint32_t parity, S* s, uint32_t code, uint32_t peer_abort_addr) {
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (s->abort) return false;
    }
    s->abort = 1;
    st_cluster_u32(peer_abort_addr, 1u);            // the other CTA of the pair gives up too
    atomicExch(&g_gemm_error, code);
    return false;
}
template <typename S>
__device__ __forceinline__ bool wait_bar_warp(uint64_t* bar, uint32_t parity, S* s, uint32_t code, uint32_t peer_abort_addr) {
    uint32_t ok = 1;
    if ((threadIdx.x & 31) == 0) {
        ok = 0;
        for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
            if (mbar_try_wait(bar, parity)) { ok = 1; break; }
            if (s->abort) break;
            __nanosleep(32);
        }
        if (!ok && !s->abort) { s->abort = 1; st_cluster_u32(peer_abort_addr, 1u); atomicExch(&g_gemm_error, code); }
    }
    return __shfl_sync(0xffffffffu, ok, 0) != 0;
}

__global__ void __launch_bounds__(THREADS, 1)
fp8_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_bt,
                     const __grid_constant__ CUtensorMap map_c,
                     const float* __restrict__ sa, const float* __restrict__ sb, int M, int N, int K, int b_kn)
{
    extern __shared__ __align__(1024) uint8_t smem_raw_pair[];
    Smem* s = reinterpret_cast<Smem*>(smem_raw_pair);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();                  // 0 = leader of the pair
    const int m_tiles = (M + TILE_M - 1) / TILE_M, n_tiles = (N + BN - 1) / BN;
    const int n_work = m_tiles * n_tiles;
    const int k_blocks = (K + BK - 1) / BK;
    const int first = (int)cluster_id(), stride = (int)n_clusters();
    const uint32_t peer_abort = map_to_cta(smem_u32((const void*)&s->abort), rank ^ 1u);

    if (smem_u32(s) & 1023u) {                                // the swizzled tiles need this alignment
        if (threadIdx.x == 0) atomicExch(&g_gemm_error, 5u);
        return;                                               // uniform over the grid: nobody waits for anybody
    }
    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&s->full[i], 1); mbar_init(&s->empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&s->acc_full[i], 1); mbar_init(&s->acc_empty[i], 2 * EPI_WARPS); }
        s->abort = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc_pair(&s->tmem_base, TMEM_COLS);   // the same warp of both CTAs
    tc_fence_before();
    cluster_sync_all();                                       // barriers of both CTAs exist from here on
    tc_fence_after();
    const uint32_t tmem_base = s->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (int w = first; ok && w < n_work; w += stride) {
                const int m0 = (w / n_tiles) * TILE_M + (int)rank * BM_CTA;
                const int n0 = (w % n_tiles) * BN + (int)rank * BM_CTA;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!(ok = wait_bar(&s->empty[stage], phase ^ 1, s, 1, peer_abort))) break;
                    // the leader's barrier counts the bytes of all four loads of the pair
                    if (rank == 0) mbar_expect_tx(&s->full[stage], 2 * (A_STAGE + B_STAGE));
                    const uint32_t bar = map_to_cta(smem_u32(&s->full[stage]), 0);
                    tma_load_2d_pair(s->a[stage], &map_a, bar, kb * BK, m0);
                    // B as [N,K]: 128 rows of n, k contiguous.  B as [K,N]: 128 rows of k, n contiguous,
                    // the same 16 KB with the roles of rows and bytes exchanged (no transposed copy)
                    if (b_kn) tma_load_2d_pair(s->b[stage], &map_bt, bar, n0, kb * BK);
                    else      tma_load_2d_pair(s->b[stage], &map_bt, bar, kb * BK, n0);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
            // tail: every slot handed out has come back, i.e. no arrival from the leader's
            // commits is still on its way to this CTA's barriers when the CTA leaves
            for (int i = 0; ok && i < STAGES; ++i) {
                ok = wait_bar(&s->empty[stage], phase ^ 1, s, 6, peer_abort);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer (leader only)
        if (lane == 0 && rank == 0) {
            // a [K,N] tile is an "MN-major" operand: bit 16 of the instruction descriptor, and one
            // K step of 32 rows is 32 * 128 bytes further on instead of 32 bytes
            const uint32_t idesc = make_idesc_pair() | (b_kn ? (1u << 16) : 0u);
            const uint64_t b_step = b_kn ? (uint64_t)((UMMA_K * 128) >> 4) : 2ull;
            uint32_t stage = 0, phase = 0, acc_phase[2] = {0, 0};
            bool ok = true;
            int t = 0;
            for (int w = first; ok && w < n_work; w += stride, ++t) {
                const int buf = t & 1;
                if (!(ok = wait_bar(&s->acc_empty[buf], acc_phase[buf] ^ 1, s, 2, peer_abort))) break;
                tc_fence_after();
                const uint32_t d = tmem_base + (uint32_t)(buf * BN);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!(ok = wait_bar(&s->full[stage], phase, s, 3, peer_abort))) break;
                    tc_fence_after();
                    const uint64_t adesc = make_kmajor_desc(s->a[stage]);
                    const uint64_t bdesc = make_kmajor_desc(s->b[stage]);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_f8_pair(d, adesc + 2 * k, bdesc + b_step * k, idesc, (kb | k) ? 1u : 0u);
                    umma_commit_pair(&s->empty[stage]);        // frees the slot in both CTAs
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (!ok) break;
                umma_commit_pair(&s->acc_full[buf]);           // both CTAs' accumulators are complete
                acc_phase[buf] ^= 1;
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (both CTAs)
        const int q = warp & 3;                                // TMEM lane quarter this warp may read
        const int half = (warp - 2) >> 2;                      // which 128 columns of the tile
        const int etid = threadIdx.x - 64;
        uint8_t* my_stage = &s->cstage[warp - 2][0][0];
        uint32_t full_phase[2] = {0, 0};
        // a tile is two 32 x 64 pieces per warp, piece p staged in buffer p % EPI_BUFS
        uint32_t groups = 0, last_group[EPI_BUFS] = {};        // lane 0: store groups committed, and which one last read a buffer
        bool ok = true;
        int t = 0;
        for (int w = first; w < n_work; w += stride, ++t) {
            const int buf = t & 1;
            const int m0 = (w / n_tiles) * TILE_M + (int)rank * BM_CTA, n0 = (w % n_tiles) * BN;
            s->sb[buf][etid] = (n0 + etid < N) ? __ldg(sb + n0 + etid) : 0.0f;
            asm volatile("bar.sync 1, %0;" :: "n"(EPI_WARPS * 32) : "memory");
            const int row = m0 + q * 32 + lane;
            const float sa_row = row < M ? __ldg(sa + row) : 0.0f;
            const f32x2 sa2 = pack2(sa_row, sa_row);
            if (ok) ok = wait_bar_warp(&s->acc_full[buf], full_phase[buf], s, 4, peer_abort);
            if (!ok) continue;
            full_phase[buf] ^= 1;
            tc_fence_after();
            const uint32_t t_base = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + half * 128);
            const float* sb_s = s->sb[buf] + half * 128;
            uint32_t r[2][32];
            tmem_ld32(t_base, r[0]);
#pragma unroll
            for (int chunk = 0; chunk < 4; ++chunk) {
                tmem_ld_wait();
                if (chunk + 1 < 4) tmem_ld32(t_base + (uint32_t)((chunk + 1) * 32), r[(chunk + 1) & 1]);
                else {
                    // the accumulator now lives in registers: hand the buffer back to the leader
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&s->acc_empty[buf]), 0));
                }
                const uint32_t* rc = r[chunk & 1];
                constexpr int kBufOfPiece[2] = {0, 1 % EPI_BUFS};
                const int pb = kBufOfPiece[chunk >> 1];
                uint8_t* stage_buf = my_stage + pb * PIECE_BYTES;
                if ((chunk & 1) == 0) {
                    // the store that last read this staging buffer must be done with it: it is if at
                    // most (groups committed after it) groups are still reading (a skipped store, at a
                    // ragged edge, commits no group, so the count is kept rather than assumed)
                    if (lane == 0) tma_store_wait_read_keep(groups - last_group[pb] >= 1u ? 1 : 0);
                    __syncwarp();
                }
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    const float4 s0 = *reinterpret_cast<const float4*>(sb_s + chunk * 32 + v * 8);
                    const float4 s1 = *reinterpret_cast<const float4*>(sb_s + chunk * 32 + v * 8 + 4);
                    const f32x2 sc[4] = {pack2(s0.x, s0.y), pack2(s0.z, s0.w), pack2(s1.x, s1.y), pack2(s1.z, s1.w)};
                    uint32_t o[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        uint32_t lo, hi;
                        unpack2u(mul2_rn(mul2_rn(pack2u(rc[v * 8 + 2 * i], rc[v * 8 + 2 * i + 1]), sa2), sc[i]), lo, hi);
                        const __nv_bfloat162 p = __floats2bfloat162_rn(__uint_as_float(lo), __uint_as_float(hi));
                        o[i] = *reinterpret_cast<const uint32_t*>(&p);
                    }
                    // row `lane`, 16-byte piece (chunk & 1) * 4 + v of its 128 bytes, xor-swizzled by the row
                    const int pc = ((chunk & 1) * 4 + v) ^ (lane & 7);
                    *reinterpret_cast<uint4*>(stage_buf + lane * 128 + (pc << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                }
                if (chunk & 1) {
                    // 32 rows x 64 columns leave as one bulk tensor store of full 128-byte rows
                    fence_proxy_async();
                    __syncwarp();
                    const int col0 = n0 + half * 128 + (chunk >> 1) * 64;
                    if (lane == 0 && col0 < N && m0 + q * 32 < M) {
                        tma_store_2d(&map_c, stage_buf, col0, m0 + q * 32);
                        last_group[pb] = ++groups;
                    }
                }
            }
        }
        if (lane == 0) tma_store_wait_all();
    }

    __syncwarp();                                             // lanes that had no role wait for the one that had
    // ---------------------------------------------------------------- teardown
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

}  // namespace pair

// ---------------------------------------------------------- [K,N] -> [N,K] bytes
// 64x64 byte tiles through shared memory; both global sides move 4-byte words.
__global__ void __launch_bounds__(256)
transpose_u8_kernel(const uint8_t* __restrict__ in, uint8_t* __restrict__ out, int K, int N, int ld_in, int ld_out)
{
    __shared__ uint8_t tile[64][68];                 // [n][k], padded
    const int k0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;       // 16 x 16 threads, 4x4 bytes each
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int k = k0 + ty * 4 + i, n = n0 + tx * 4;
        uint32_t w = 0;
        if (k < K && n < N) w = *reinterpret_cast<const uint32_t*>(in + (size_t)k * ld_in + n);
#pragma unroll
        for (int j = 0; j < 4; ++j) tile[tx * 4 + j][ty * 4 + i] = (uint8_t)(w >> (8 * j));
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int n = n0 + ty * 4 + i, k = k0 + tx * 4;
        if (n < N && k < K)
            *reinterpret_cast<uint32_t*>(out + (size_t)n * ld_out + k) =
                *reinterpret_cast<const uint32_t*>(&tile[ty * 4 + i][tx * 4]);
    }
}

}  // namespace gemm
}  // namespace act

// ------------------------------------------------------------------- host side
namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry-point lookup, so the
// library carries no link-time dependency on libcuda.
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

// 2-D byte tensor [rows, cols] with row pitch ld, box = box_rows x 128 bytes, 128-byte swizzle
// C: bf16 [rows, cols], row pitch ld elements, box 32 x 32 elements, 64-byte swizzle
bool make_map_c(CUtensorMap* map, void* base, int rows, int cols, int ld) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {32, 32};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// C for the pair kernel: box 64 x 32 elements (full 128-byte rows), 128-byte swizzle
bool make_map_c_wide(CUtensorMap* map, void* base, int rows, int cols, int ld) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {64, 32};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool make_map(CUtensorMap* map, const void* base, int rows, int cols, int ld, int box_rows) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld};
    const cuuint32_t box[2] = {(cuuint32_t)act::gemm::BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, estr,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

int round_up(int v, int m) { return (v + m - 1) / m * m; }

constexpr int kMaxDevices = 64;                      // per-device host state below is indexed by ordinal
constexpr int kForceTranspose = 1 << 30;             // internal flag: always stage a [K,N] operand through the workspace

}  // namespace

extern "C" size_t act_fp8_gemm_workspace(int M, int N, int K, int flags) {
    if (flags & ACT_GEMM_B_IS_NK) return 0;
    if (N <= 0 || K <= 0) return 0;
    // more than one 128-row block: CTA pairs read a [K,N] operand in place, provided its pitch is a
    // multiple of 16 (assumed here: ldb = N) and its base 16-byte aligned
    if (M > act::gemm::BM && !(flags & ACT_GEMM_SINGLE_CTA) && (N & 15) == 0) return 0;
    return (size_t)N * (size_t)round_up(K, 16);
}

extern "C" int act_fp8_gemm(const void* A, const void* B, const float* sa, const float* sb, void* C,
                            int M, int N, int K, int lda, int ldb, int ldc, int flags,
                            void* workspace, size_t ws_bytes, void* stream)
{
    using namespace act::gemm;
    if (M < 0 || N < 0 || K < 0) return ACT_ERR_SIZE;
    if (M == 0 || N == 0) return ACT_OK;
    if (!A || !B || !sa || !sb || !C) return ACT_ERR_NULL;
    const bool b_is_nk = (flags & ACT_GEMM_B_IS_NK) != 0;
    // TMA needs 16-byte aligned bases and pitches; the epilogue stores 8 bf16 at a time
    if (K == 0 || (K & 15) || (lda & 15) || lda < K || (N & 7) || (ldc & 7) || ldc < N) return ACT_ERR_SIZE;
    if (b_is_nk ? ((ldb & 15) || ldb < K) : ((ldb & 3) || ldb < N || (N & 3))) return ACT_ERR_SIZE;
    if (((uintptr_t)A | (uintptr_t)C | (uintptr_t)sb) & 15) return ACT_ERR_ALIGN;
    if ((uintptr_t)B & (b_is_nk ? 15 : 3)) return ACT_ERR_ALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    const uint8_t* bt = static_cast<const uint8_t*>(B);
    int ldbt = ldb;
    // CTA pairs read a [K,N] operand in place when a tensor map can describe it (16-byte base and
    // pitch); otherwise, and for the lone-CTA kernel, it is transposed into the workspace first
    const bool pairs = !(flags & ACT_GEMM_SINGLE_CTA) && M > BM;
    const bool b_in_place = !b_is_nk && pairs && !(flags & kForceTranspose) && !(ldb & 15) && !((uintptr_t)B & 15);
    if (!b_is_nk && !b_in_place) {
        const size_t need = act_fp8_gemm_workspace(M, N, K, flags);
        if (!workspace || ws_bytes < need) return ACT_ERR_WORKSPACE;
        if ((uintptr_t)workspace & 15) return ACT_ERR_ALIGN;
        ldbt = round_up(K, 16);
        dim3 grid((N + 63) / 64, (K + 63) / 64);
        transpose_u8_kernel<<<grid, 256, 0, st>>>(static_cast<const uint8_t*>(B), static_cast<uint8_t*>(workspace),
                                                   K, N, ldb, ldbt);
        if (cudaGetLastError() != cudaSuccess) return ACT_ERR_LAUNCH;
        bt = static_cast<const uint8_t*>(workspace);
    }

    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return ACT_ERR_DEVICE;
    // Per-device state, set up on the first call on that device: the shared-memory opt-in is a
    // per-device attribute of each kernel, so a process driving several GPUs sets it on each.
    struct DeviceState { int sms; int clusters; };
    static DeviceState state[kMaxDevices];                  // sms == 0: not yet set up
    const int smem_one = (int)sizeof(Smem) + 1024;
    const int smem_pair = (int)sizeof(pair::Smem);
    DeviceState& ds = state[dev];
    if (!ds.sms) {
        int sms = 0;
        if (cudaFuncSetAttribute(fp8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_one) != cudaSuccess ||
            cudaFuncSetAttribute(pair::fp8_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_pair) != cudaSuccess)
            return ACT_ERR_DEVICE;
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) return ACT_ERR_DEVICE;
        // how many CTA pairs the device holds at once (one CTA per SM, both SMs of a TPC)
        cudaLaunchConfig_t q = {};
        q.gridDim = dim3(2u * (unsigned)sms, 1, 1);
        q.blockDim = dim3(THREADS, 1, 1);
        q.dynamicSmemBytes = (size_t)smem_pair;
        cudaLaunchAttribute qa[1];
        qa[0].id = cudaLaunchAttributeClusterDimension;
        qa[0].val.clusterDim.x = 2; qa[0].val.clusterDim.y = 1; qa[0].val.clusterDim.z = 1;
        q.attrs = qa; q.numAttrs = 1;
        int clusters = 0;
        if (cudaOccupancyMaxActiveClusters(&clusters, pair::fp8_gemm_pair_kernel, &q) != cudaSuccess || clusters <= 0) {
            (void)cudaGetLastError();
            clusters = sms / 2;
        }
        ds.clusters = clusters < sms / 2 ? clusters : sms / 2;
        ds.sms = sms;
    }

    CUtensorMap map_a, map_bt, map_c;
    // A lone CTA per 128 x 256 tile when asked for, or when the problem has a single row block
    // (the second CTA of a pair would stage rows that do not exist); otherwise CTA pairs.
    if (!pairs) {
        if (!make_map(&map_a, A, M, K, lda, BM) || !make_map(&map_bt, bt, N, K, ldbt, BN) ||
            !make_map_c(&map_c, C, M, N, ldc)) return ACT_ERR_DEVICE;
        const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
        const int grid = tiles < ds.sms ? tiles : ds.sms;
        fp8_gemm_kernel<<<grid, THREADS, smem_one, st>>>(map_a, map_bt, map_c, sa, sb, M, N, K);
        return cudaGetLastError() == cudaSuccess ? ACT_OK : ACT_ERR_LAUNCH;
    }
    if (!make_map(&map_a, A, M, K, lda, pair::BM_CTA) ||
        !(b_in_place ? make_map(&map_bt, B, K, N, ldb, pair::BK) : make_map(&map_bt, bt, N, K, ldbt, pair::BM_CTA)) ||
        !make_map_c_wide(&map_c, C, M, N, ldc)) return ACT_ERR_DEVICE;
    const int work = ((M + pair::TILE_M - 1) / pair::TILE_M) * ((N + pair::BN - 1) / pair::BN);
    const int clusters = work < ds.clusters ? work : ds.clusters;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2u * (unsigned)clusters, 1, 1);
    cfg.blockDim = dim3(THREADS, 1, 1);
    cfg.dynamicSmemBytes = (size_t)smem_pair;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, pair::fp8_gemm_pair_kernel, map_a, map_bt, map_c, sa, sb, M, N, K,
                           b_in_place ? 1 : 0) != cudaSuccess) {
        (void)cudaGetLastError();
        return ACT_ERR_LAUNCH;
    }
    return ACT_OK;
}

// Reads (and optionally clears) the abort reason of the last GEMM on the current
// device: 0 = none, 1..4 = which wait ran out (slot free, accumulator free, data
// ready, accumulator ready).  Synchronises the device; for diagnostics only.
extern "C" int act_fp8_gemm_status(unsigned int* out, int clear) {
    if (!out) return ACT_ERR_NULL;
    if (cudaMemcpyFromSymbol(out, act::gemm::g_gemm_error, sizeof(unsigned int)) != cudaSuccess) return ACT_ERR_DEVICE;
    if (clear) {
        const unsigned int zero = 0;
        if (cudaMemcpyToSymbol(act::gemm::g_gemm_error, &zero, sizeof(zero)) != cudaSuccess) return ACT_ERR_DEVICE;
    }
    return ACT_OK;
}

// ------------------------------------------------- entry point that allocates nothing
// Some callers of this library run where device memory cannot be requested at call
// time: a plugin invoked from inside another framework's memory plan (all device
// memory already handed out), a real-time loop whose rules forbid allocator calls
// because their latency is unbounded.  For them the [K,N] -> [N,K] staging
// buffer of the GEMM lives in the library image itself.  The array below is part of
// every device's copy of the module from load until exit (4 MiB per GPU).
constexpr size_t kStaticScratchBytes = 4u << 20;
static __device__ __align__(256) uint8_t g_static_bt_scratch[kStaticScratchBytes];

// Device address of the array on each device, looked up on first use.  In host code
// the array's name is only a handle for this lookup, never a pointer to pass along.
static uint8_t* g_static_scratch_ptr[kMaxDevices];

extern "C" size_t act_fp8_gemm_static_limit(void) { return kStaticScratchBytes; }

extern "C" int act_fp8_gemm_static(const void* A, const void* B, const float* sa, const float* sb, void* C,
                                   int M, int N, int K, int lda, int ldb, int ldc, void* stream)
{
    if (M < 0 || N < 0 || K < 0) return ACT_ERR_SIZE;
    if ((size_t)N * (size_t)round_up(K > 0 ? K : 1, 16) > kStaticScratchBytes) return ACT_ERR_STATIC_LIMIT;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return ACT_ERR_DEVICE;
    uint8_t* scratch = g_static_scratch_ptr[dev];
    if (!scratch) {
        // once per device, with that device current (it is: cudaGetDevice just said so)
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_static_bt_scratch) != cudaSuccess || !p) return ACT_ERR_DEVICE;
        scratch = static_cast<uint8_t*>(p);
        g_static_scratch_ptr[dev] = scratch;
    }
    // B in the [K,N] layout, always staged through the transposed copy (this entry point exists
    // for that copy's buffer); the shared array is the workspace of the ordinary entry point
    return act_fp8_gemm(A, B, sa, sb, C, M, N, K, lda, ldb, ldc, kForceTranspose, scratch, kStaticScratchBytes, stream);
}
