// twm_gemm_tc.cuh — the tcgen05 / TMEM W4A16 kernel (FP16 activations).
//
// The contraction C[m][n] = sum_k A[m][k] * w[k][n] runs on the 5th-generation
// tensor cores with the roles swapped: the 128 weight columns of a CTA are the
// MMA's M dimension (one TMEM lane per column), the activation rows are its N
// dimension (padded to NB), and K advances 16 at a time.  There is no
// counterpart in the reference: its only batched W4A16 kernel is a 32x32 SIMT
// tile kernel on another layout (crates/kernels/src/quantize.rs:186-246), and
// its TW-Marlin kernel is M=1 only (quantize.rs:1186-1298).  Same result
// definition as those: w = f32(scale) * (nibble - 8), FP32 accumulation.
//
// Data path per CTA (128 columns x a K slice):
//   warp 0       streams packed rows into a shared-memory ring with 1-D bulk
//                copies (TMA unit, mbarrier completion; no multicast).
//   warps 4-7    "dequant": each thread owns one column = one TMEM lane.  It
//                reads its 16-byte block (one 128-bit shared load, conflict
//                free) and turns the four u32 words into sixteen half2
//                registers with five integer ops per word, no conversion and
//                no floating-point op: a nibble left in place in a 16-bit half,
//                `v & 0x000F000F` or `v & 0x00F000F0`, IS the FP16 subnormal
//                q * 2^-24 (resp. q * 2^-20) exactly.  tcgen05.st puts the
//                registers into TMEM as the MMA's A operand.  The weights never
//                go back to shared memory.
//   warps 2-3    stage the activations of the slice into shared memory as the
//                MMA's B operand (K-major core matrices, no swizzle), in the K
//                order the nibble extraction produces, and compute the block
//                sums of A that fold the "-8" of every nibble.
//   warp 1       one thread issues tcgen05.mma (A from TMEM, B from shared
//                memory, D in TMEM): two per 32-block, one for the 2^-24
//                nibbles and one for the 2^-20 nibbles, each into the block's
//                own accumulator (no accumulate chains).  One tcgen05.commit
//                per block tells the dequant warps that the slot's A operand is
//                consumed and the epilogue that its accumulators are complete.
//   warps 8-11   epilogue: read each block's two accumulators (tcgen05.ld),
//                combine them into the scale group's sum, and at every group
//                boundary subtract 8*sum(A), multiply by the group's FP32 scale
//                and add to the running total in registers.  Products are exact
//                (4-bit x 11-bit) and the scale is applied in FP32, as in the
//                reference's kernel.
// Split-K finish and the programmatic-dependent-launch rules are the same as
// in the streaming kernel (twm_gemv_simt.cuh).
#pragma once

#include "twm_common.cuh"

namespace twm {
namespace tc {

constexpr int NT = 128;               // columns per CTA = MMA M = TMEM lanes
constexpr int WSTAGE_BLOCKS = 4;      // 32-blocks per ring stage (8 KB)
constexpr int WSTAGES = 8;            // ring depth: 64 KB in flight per CTA
constexpr int SLOTS = 5;              // TMEM slots: one 32-block's A operand + its two accumulators each
constexpr int THREADS = 12 * 32;
constexpr int ASUM_CAP = 2048;        // floats: (blocks in the K slice) * MV must fit
constexpr int B_BUF_BYTES = 16384;    // one staged activation chunk
constexpr int EPI_THREADS = 128;
constexpr int STAGER_THREADS = 64;

template <int NB>
struct Cfg {
    static constexpr int SLICE_BYTES = NB * 32;                     // NB rows x 16 K-slots x 2 B
    static constexpr int BLOCK_B_BYTES = 2 * SLICE_BYTES;           // "lo" and "hi" slices of a 32-block
    static constexpr int CHUNK_BLOCKS = B_BUF_BYTES / BLOCK_B_BYTES;   // 32-blocks per staged chunk
    static constexpr int A_COL0 = 0;                                // A slot s: columns [16 s, 16 s + 16)
    static constexpr int D_COL0 = SLOTS * 16;                       // D slot s: lo at D_COL0 + 2 NB s, hi NB further
    static constexpr int USED_COLS = SLOTS * (16 + 2 * NB);
    static constexpr int TMEM_COLS = USED_COLS <= 256 ? 256 : 512;
    static_assert(USED_COLS <= 512, "tensor memory holds 512 columns");
};

struct Smem {
    alignas(128) uint8_t packed[WSTAGES][WSTAGE_BLOCKS * NT * kBlockBytes];
    alignas(128) uint8_t b[2][B_BUF_BYTES];
    alignas(16) float asum8[ASUM_CAP]; // [block in slice][MV]: -8 * sum of the block's activations
    alignas(8) uint64_t w_full[WSTAGES];
    alignas(8) uint64_t w_empty[WSTAGES];
    alignas(8) uint64_t a_full[SLOTS];     // dequant -> MMA: the slot's A operand is in tensor memory
    alignas(8) uint64_t mma_done[SLOTS];   // MMA (commit) -> dequant and epilogue: A is consumed, D is complete
    alignas(8) uint64_t d_empty[SLOTS];    // epilogue -> MMA: the slot's accumulators are read out
    alignas(8) uint64_t b_full[2];
    alignas(8) uint64_t b_empty[2];
    uint32_t tmem_base;
    int abort_flag;
    int is_last;
};

// ------------------------------------------------------------ tcgen05 PTX --
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// D[128 x N] (+)= A[128 x 16] (TMEM) * B[N x 16]^T (shared memory descriptor)
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

template <int N>
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&v)[N]);
template <>
__device__ __forceinline__ void tmem_ld<1>(uint32_t taddr, uint32_t (&v)[1]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(v[0]) : "r"(taddr));
}
template <>
__device__ __forceinline__ void tmem_ld<2>(uint32_t taddr, uint32_t (&v)[2]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x2.b32 {%0,%1}, [%2];" : "=r"(v[0]), "=r"(v[1]) : "r"(taddr));
}
template <>
__device__ __forceinline__ void tmem_ld<4>(uint32_t taddr, uint32_t (&v)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(taddr));
}
template <>
__device__ __forceinline__ void tmem_ld<8>(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]) : "r"(taddr));
}
template <>
__device__ __forceinline__ void tmem_ld<16>(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr));
}

// Shared-memory matrix descriptor, K-major, no swizzle: core matrices are 8 rows
// x 16 bytes stored as 128 contiguous bytes; the next core matrix along K lies
// 128 bytes further (leading offset), the next 8 rows 256 bytes further (stride
// offset).  Descriptor version 1 = sm_100.
__device__ __forceinline__ uint64_t make_b_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(128u >> 4) << 16;
    d |= (uint64_t)(256u >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

// warp-uniform bounded wait
__device__ __forceinline__ bool wait_uniform(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    const bool got = mbar_wait_bounded(bar, parity, abort_flag);
    return __all_sync(0xffffffffu, got);
}

// NB = MMA N (activation rows padded), MV = rows the epilogue carries (power of two >= M, <= NB)
template <int NB, int MV>
__global__ void __launch_bounds__(THREADS, (Cfg<NB>::TMEM_COLS <= 256) ? 2 : 1)
gemm_kernel(const GemmParams p)
{
    using C = Cfg<NB>;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>(smem_raw);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int n0 = blockIdx.x * NT;
    const int cols = min(NT, p.N - n0);
    const int b0 = blockIdx.y * p.blocks_per_split;
    const int b1 = min(p.nkb, b0 + p.blocks_per_split);
    const int total_blocks = b1 - b0;
    const int gmask = p.group / kBlockK - 1;                 // 32-blocks per scale group (1 or 4), minus one
    const int gshift = (p.group == 128) ? 2 : 0;

    if (tid == 0) {
        for (int s = 0; s < WSTAGES; ++s) { mbar_init(&sm.w_full[s], 1); mbar_init(&sm.w_empty[s], 4); }
        for (int s = 0; s < SLOTS; ++s) {
            mbar_init(&sm.a_full[s], 4); mbar_init(&sm.mma_done[s], 1); mbar_init(&sm.d_empty[s], 4);
        }
        for (int s = 0; s < 2; ++s) { mbar_init(&sm.b_full[s], STAGER_THREADS / 32); mbar_init(&sm.b_empty[s], 1); }
        sm.abort_flag = 0;
        sm.is_last = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    volatile int* abort_flag = &sm.abort_flag;

    // TMA producer state (warp 0).  The first ring-full of stages is issued
    // before the TMEM allocation below, so that weights are already streaming
    // while an earlier kernel's CTA may still hold this SM's tensor memory.
    const uint8_t* packed = p.packed;
    const int n_wstages = (total_blocks + WSTAGE_BLOCKS - 1) / WSTAGE_BLOCKS;
    auto issue_stage = [&](int st) {
        const int slot = st % WSTAGES;
        const int bstart = b0 + st * WSTAGE_BLOCKS;
        const int nb = min(WSTAGE_BLOCKS, b1 - bstart);
        mbar_arrive_expect_tx(&sm.w_full[slot], (uint32_t)nb * cols * kBlockBytes);
        for (int r = 0; r < nb; ++r)
            bulk_g2s(&sm.packed[slot][r * NT * kBlockBytes],
                     packed + ((size_t)(bstart + r) * p.N + n0) * kBlockBytes,
                     (uint32_t)cols * kBlockBytes, &sm.w_full[slot]);
    };
    if (warp == 0) {
        if (p.packed_offsets != nullptr) {
            pdl_wait_prior_grids();                  // the offset table may come from the kernel before
            packed += p.packed_offsets[p.expert_idx];
        }
        if (lane == 0)
            for (int st = 0; st < min(n_wstages, WSTAGES); ++st) issue_stage(st);
        __syncwarp();
    } else if (warp == 1) {
        tmem_alloc(&sm.tmem_base, C::TMEM_COLS);
        tc_fence_before();
    }
    // every role needs the TMEM base address
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sm.tmem_base;

    if (warp == 0) {
        // ---------------------------------------------- TMA producer (packed) --
        PROF_DECL;
        for (int st = WSTAGES; st < n_wstages; ++st) {
            const int slot = st % WSTAGES;
            PROF_BEGIN(t0);
            if (!wait_uniform(&sm.w_empty[slot], ((st / WSTAGES) - 1) & 1, abort_flag)) break;
            PROF_END(t0, 0);
            if (lane == 0) issue_stage(st);
            __syncwarp();
        }
        PROF_FLUSH(0);
    } else if (warp == 1) {
        // ------------------------------------------------------- MMA issuer --
        // Every 32-block gets its own pair of accumulators (no accumulate
        // chain: back-to-back MMAs into one accumulator would each wait out the
        // tensor pipe's latency); the epilogue adds them up.
        if (lane == 0) {
            uint32_t idesc = 0;
            idesc |= 1u << 4;                         // D format f32
            idesc |= (uint32_t)(NB >> 3) << 17;       // N
            idesc |= (uint32_t)(128 >> 4) << 24;      // M
            const uint64_t desc0[2] = {make_b_desc(smem_u32(&sm.b[0][0])), make_b_desc(smem_u32(&sm.b[1][0]))};
            PROF_DECL;
            int slot = 0, use = 0, bi = 0, chunk = 0;
            for (int i = 0; i < total_blocks; ++i) {
                PROF_BEGIN(t0);
                if (bi == 0 && !mbar_wait_bounded(&sm.b_full[chunk & 1], (chunk >> 1) & 1, abort_flag)) break;
                PROF_END(t0, 0);
                PROF_BEGIN(t1);
                if (use > 0 && !mbar_wait_bounded(&sm.d_empty[slot], (use - 1) & 1, abort_flag)) break;
                PROF_END(t1, 1);
                PROF_BEGIN(t2);
                if (!mbar_wait_bounded(&sm.a_full[slot], use & 1, abort_flag)) break;
                PROF_END(t2, 2);
                PROF_BEGIN(t3);
                tc_fence_after();
                const uint32_t a_addr = tmem_base + C::A_COL0 + slot * 16;
                const uint32_t d_addr = tmem_base + C::D_COL0 + slot * 2 * NB;
                // descriptor start-address field counts 16-byte units
                const uint64_t bd = desc0[chunk & 1] + (uint64_t)((bi * C::BLOCK_B_BYTES) >> 4);
                tc_mma_ts(d_addr, a_addr, bd, idesc, 0u);
                tc_mma_ts(d_addr + NB, a_addr + 8, bd + (uint64_t)(C::SLICE_BYTES >> 4), idesc, 0u);
                PROF_END(t3, 3);
                PROF_BEGIN(t4);
                tc_commit(&sm.mma_done[slot]);
                const bool chunk_end = (bi == C::CHUNK_BLOCKS - 1) || (i == total_blocks - 1);
                if (chunk_end) tc_commit(&sm.b_empty[chunk & 1]);
                PROF_END(t4, 4);
                if (++slot == SLOTS) { slot = 0; ++use; }
                if (chunk_end) { bi = 0; ++chunk; } else { ++bi; }
            }
            PROF_FLUSH(1);
        }
        __syncwarp();
    } else if (warp == 2 || warp == 3) {
        // ---------------------------------------------- activation stagers --
        // One item = 8 consecutive K of one row (one 16-byte load).  The loads of
        // a chunk are issued before the wait for its buffer, so their latency
        // hides behind the MMAs that still read the buffer's previous contents.
        pdl_wait_prior_grids();
        const int st_tid = tid - 64;
        const __half* A = reinterpret_cast<const __half*>(p.a);
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(A) & 15) == 0) && ((p.lda & 7) == 0);
        const int n_chunks = (total_blocks + C::CHUNK_BLOCKS - 1) / C::CHUNK_BLOCKS;
        constexpr int PF = 8;                                            // items in flight per thread
        PROF_DECL;
        bool ok = true;
        for (int chunk = 0; chunk < n_chunks && ok; ++chunk) {
            const int buf = chunk & 1;
            const int use = chunk >> 1;
            const int cb0 = chunk * C::CHUNK_BLOCKS;
            const int cb = min(C::CHUNK_BLOCKS, total_blocks - cb0);
            const int items = p.M * cb * 4;
            bool waited = false;
            for (int base = 0; base < items; base += STAGER_THREADS * PF) {
                uint4 x[PF];
                PROF_BEGIN(t1);
#pragma unroll
                for (int u = 0; u < PF; ++u) {
                    const int it = base + u * STAGER_THREADS + st_tid;
                    x[u] = make_uint4(0, 0, 0, 0);
                    if (it < items) {
                        const int m = it / (cb * 4);
                        const int rem = it - m * (cb * 4);
                        const size_t off = (size_t)m * p.lda + (size_t)(b0 + cb0 + (rem >> 2)) * kBlockK + (rem & 3) * 8;
                        if (vec_ok) {
                            x[u] = *reinterpret_cast<const uint4*>(A + off);
                        } else {
                            const uint16_t* a16 = reinterpret_cast<const uint16_t*>(A) + off;
                            x[u].x = a16[0] | ((uint32_t)a16[1] << 16); x[u].y = a16[2] | ((uint32_t)a16[3] << 16);
                            x[u].z = a16[4] | ((uint32_t)a16[5] << 16); x[u].w = a16[6] | ((uint32_t)a16[7] << 16);
                        }
                    }
                }
                PROF_END(t1, 1);
                if (!waited) {
                    PROF_BEGIN(t0);
                    if (use > 0 && !wait_uniform(&sm.b_empty[buf], (use - 1) & 1, abort_flag)) { ok = false; break; }
                    PROF_END(t0, 0);
                    waited = true;
                }
                PROF_BEGIN(t2);
#pragma unroll
                for (int u = 0; u < PF; ++u) {
                    const int it = base + u * STAGER_THREADS + st_tid;
                    float s = 0.0f;
                    int m = 0, bi = 0;
                    if (it < items) {
                        m = it / (cb * 4);
                        const int rem = it - m * (cb * 4);
                        bi = rem >> 2;
                        const int w = rem & 3;
                        // K order of the "lo" slice: k0,k4,k2,k6 ; of the "hi" slice: k1,k5,k3,k7
                        uint2 lo, hi;
                        lo.x = __byte_perm(x[u].x, x[u].z, 0x5410); lo.y = __byte_perm(x[u].y, x[u].w, 0x5410);
                        hi.x = __byte_perm(x[u].x, x[u].z, 0x7632); hi.y = __byte_perm(x[u].y, x[u].w, 0x7632);
                        uint8_t* dst = &sm.b[buf][bi * C::BLOCK_B_BYTES + (m >> 3) * 256 + (w >> 1) * 128 + (m & 7) * 16 + (w & 1) * 8];
                        *reinterpret_cast<uint2*>(dst) = lo;
                        *reinterpret_cast<uint2*>(dst + C::SLICE_BYTES) = hi;
                        const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&x[u].x));
                        const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&x[u].y));
                        const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&x[u].z));
                        const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&x[u].w));
                        s = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
                    }
                    // four consecutive items (lanes) are the four words of one block
                    s += __shfl_xor_sync(0xffffffffu, s, 1);
                    s += __shfl_xor_sync(0xffffffffu, s, 2);
                    if (it < items && (it & 3) == 0) sm.asum8[(cb0 + bi) * MV + m] = -8.0f * s;
                }
                PROF_END(t2, 2);
            }
            if (!ok) break;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> MMA's async reads
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.b_full[buf]);
        }
        PROF_FLUSH(2);
    } else if (warp >= 4 && warp < 8) {
        // ------------------------------------------------------- dequant --
        const int quarter = warp & 3;
        const int col = quarter * 32 + lane;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + C::A_COL0;
        PROF_DECL;
        int slot = 0, use = 0;
        for (int i = 0; i < total_blocks; ++i) {
            const int st = i / WSTAGE_BLOCKS;
            const int r = i - st * WSTAGE_BLOCKS;
            const int wslot = st % WSTAGES;
            PROF_BEGIN(t0);
            if (r == 0 && !wait_uniform(&sm.w_full[wslot], (st / WSTAGES) & 1, abort_flag)) break;
            PROF_END(t0, 0);
            PROF_BEGIN(t1);
            const uint4 v = lds128(&sm.packed[wslot][(r * NT + col) * kBlockBytes]);
            const uint32_t words[4] = {v.x, v.y, v.z, v.w};
            uint32_t regs[16];
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const uint32_t x = words[w];
                const uint32_t x8 = x >> 8;
                regs[2 * w] = x & 0x000F000Fu;          // (k0, k4) * 2^-24
                regs[2 * w + 1] = x8 & 0x000F000Fu;     // (k2, k6) * 2^-24
                regs[8 + 2 * w] = x & 0x00F000F0u;      // (k1, k5) * 2^-20
                regs[8 + 2 * w + 1] = x8 & 0x00F000F0u; // (k3, k7) * 2^-20
            }
            if (r == WSTAGE_BLOCKS - 1 || i == total_blocks - 1) {
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm.w_empty[wslot]);      // ring stage read out
            }
            PROF_END(t1, 1);
            PROF_BEGIN(t2);
            if (use > 0 && !wait_uniform(&sm.mma_done[slot], (use - 1) & 1, abort_flag)) break;
            PROF_END(t2, 2);
            PROF_BEGIN(t3);
            tc_fence_after();
            tmem_st16(lane_base + slot * 16, regs);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.a_full[slot]);
            PROF_END(t3, 3);
            if (++slot == SLOTS) { slot = 0; ++use; }
        }
        PROF_FLUSH(3);
    } else if (warp >= 8) {
        // ------------------------------------------------------- epilogue --
        pdl_wait_prior_grids();
        const int quarter = warp & 3;
        const int col = quarter * 32 + lane;
        const int n = n0 + col;
        const bool owner = n < p.N;
        const uint16_t* scales = p.scales;
        if (p.scales_offsets != nullptr) scales += p.scales_offsets[p.expert_idx];
        const uint32_t lane_d = tmem_base + ((uint32_t)(quarter * 32) << 16) + C::D_COL0;
        float tot[MV], gsum[MV], a8[MV];
#pragma unroll
        for (int m = 0; m < MV; ++m) { tot[m] = 0.0f; gsum[m] = 0.0f; a8[m] = 0.0f; }
        PROF_DECL;
        uint16_t s_bits = owner ? scales[(size_t)(b0 >> gshift) * p.N + n] : (uint16_t)0;
        uint16_t s_next = s_bits;
        int slot = 0, use = 0;
        for (int i = 0; i < total_blocks; ++i) {
            const int b = b0 + i;
            const bool first_in_group = (i == 0) || ((b & gmask) == 0);
            const bool last_in_group = (i == total_blocks - 1) || (((b + 1) & gmask) == 0);
            if (first_in_group) {
                s_bits = s_next;
                const int g_next = (b >> gshift) + 1;
                if (owner && (g_next << gshift) < b1) s_next = scales[(size_t)g_next * p.N + n];   // prefetch
            }
            PROF_BEGIN(t0);
            if (!wait_uniform(&sm.mma_done[slot], use & 1, abort_flag)) break;
            PROF_END(t0, 0);
            PROF_BEGIN(t1);
            tc_fence_after();
            uint32_t lo[MV], hi[MV];
            tmem_ld<MV>(lane_d + slot * 2 * NB, lo);
            tmem_ld<MV>(lane_d + slot * 2 * NB + NB, hi);
            tmem_wait_ld();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.d_empty[slot]);
            PROF_END(t1, 1);
            PROF_BEGIN(t2);
            // lo holds sum(a*q) * 2^-24, hi holds sum(a*q) * 2^-20
#pragma unroll
            for (int m = 0; m < MV; ++m) {
                gsum[m] += fmaf(__uint_as_float(lo[m]), 16.0f, __uint_as_float(hi[m]));
                a8[m] += sm.asum8[i * MV + m];
            }
            if (last_in_group) {
                const float s = f16_bits_to_f32(s_bits);
                const float s20 = s * 1048576.0f;             // 2^20
#pragma unroll
                for (int m = 0; m < MV; ++m) {
                    tot[m] = fmaf(s20, gsum[m], tot[m]);
                    tot[m] = fmaf(s, a8[m], tot[m]);
                    gsum[m] = 0.0f;
                    a8[m] = 0.0f;
                }
            }
            PROF_END(t2, 2);
            if (++slot == SLOTS) { slot = 0; ++use; }
        }
        PROF_FLUSH(4);

        // --------------------------------------------- store / split-K finish --
        named_bar_sync(2, EPI_THREADS);
        const bool aborted = (*abort_flag != 0);
        auto store_c = [&](int m, float v) {
            const size_t off = (size_t)m * p.ldc + n;
            if (p.c_is_f16) {
                __half* cp = reinterpret_cast<__half*>(p.c);
                if (p.accumulate) v += __half2float(cp[off]);
                cp[off] = __float2half_rn(v);
            } else {
                float* cp = reinterpret_cast<float*>(p.c);
                if (p.accumulate) v += cp[off];
                cp[off] = v;
            }
        };
        if (!aborted) {
            if (p.splits == 1) {
                if (owner) {
#pragma unroll
                    for (int m = 0; m < MV; ++m)
                        if (m < p.M) store_c(m, tot[m]);
                }
            } else {
                if (owner) {
#pragma unroll
                    for (int m = 0; m < MV; ++m)
                        if (m < p.M) p.ws_partials[((size_t)blockIdx.y * p.M + m) * p.N + n] = tot[m];
                }
                __threadfence();
                named_bar_sync(2, EPI_THREADS);
                if (tid == 8 * 32) {
                    const unsigned prev = atomicAdd(&p.ws_counters[blockIdx.x], 1u);
                    sm.is_last = (prev == (unsigned)(p.splits - 1));
                }
                named_bar_sync(2, EPI_THREADS);
                if (sm.is_last) {
                    __threadfence();
                    if (owner) {
#pragma unroll
                        for (int m = 0; m < MV; ++m) {
                            if (m < p.M) {
                                float s = 0.0f;
                                for (int sp = 0; sp < p.splits; ++sp)
                                    s += ld_cg_f32(&p.ws_partials[((size_t)sp * p.M + m) * p.N + n]);
                                store_c(m, s);
                            }
                        }
                    }
                    if (tid == 8 * 32) atomicExch(&p.ws_counters[blockIdx.x], 0u);
                }
            }
        }
    }

    // ------------------------------------------------------------ teardown --
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

}  // namespace tc
}  // namespace twm
