// twm_gemm_tc.cuh — the tcgen05 / TMEM W4A16 kernel (FP16 activations, M >= 9).
//
// The contraction C[m][n] = sum_k A[m][k] * w[k][n] runs on the 5th-generation
// tensor cores with the roles swapped: the 128 weight columns of a CTA are the
// MMA's M dimension (one TMEM lane per column), the activation rows are its N
// dimension (padded to NB = 16, 32 or 64), and K advances 16 at a time.  There
// is no counterpart in the reference: its only batched W4A16 kernel is a 32x32
// SIMT tile kernel on another layout (crates/kernels/src/quantize.rs:186-246),
// and its TW-Marlin kernel is M=1 only (quantize.rs:1186-1298).  The MMA's
// weight operand is fp16_rn(f32(scale) * (nibble - 8)), i.e. exactly what the
// reference's dequant_q4_to_f16 produces (quantize.rs:534-571); accumulation
// is FP32 in tensor memory over the whole K slice.
//
// Data path per CTA (128 columns x a K slice):
//   warp 0       streams packed rows into a shared-memory ring: one tiled TMA
//                load per stage of four 32-blocks (no multicast), 1-D bulk
//                copies row by row for ragged stages.
//   warps 4-11   "dequant", two sets of four warps taking alternate blocks;
//                each thread owns one column = one TMEM lane.  It reads its
//                16-byte block (one conflict-free 128-bit shared load); per u32
//                word one shift and four LOP3 `(v & mask) | 0x64006400` give the
//                FP16 pairs (1024 + q) resp. (1024 + 16 q); one HSUB2 / HFMA2
//                makes them q - 8 exactly and one HMUL2 applies the group's
//                scale.  tcgen05.st writes the sixteen registers into tensor
//                memory as the MMA's A operand: the weights never go back to
//                shared memory.
//   (pre-pass)   permute_activations_kernel rewrites the launch's activation rows
//                once into [K/8][rows][8] FP16 with the K order the nibble
//                extraction produces inside every 8 (k0,k4,k1,k5,k2,k6,k3,k7), so
//                that warp 0 can bring the MMA's B operand for a stage (K-major
//                8x16-byte core matrices, no swizzle) with one tiled TMA load.
//   warp 1       one thread issues tcgen05.mma.cta_group::1.kind::f16 (A from
//                TMEM, B from shared memory, D in TMEM), two per 32-block, all
//                accumulating into the CTA's one [128 x NB] FP32 accumulator;
//                tcgen05.commit frees the A slot and, at the end, releases D.
//   warps 4-7    after their last block: epilogue, tcgen05.ld of D, FP16/FP32
//                store or split-K partial.
// Split-K finish and the programmatic-dependent-launch rules are the same as
// in the streaming kernels.
#pragma once

#include "twm_common.cuh"

namespace twm {
namespace tc {

constexpr int NT = 128;               // columns per CTA = MMA M = TMEM lanes
constexpr int WSTAGE_BLOCKS = 4;      // 32-blocks per ring stage (8 KB)
constexpr int WSTAGES = 6;            // packed ring depth: 48 KB in flight per CTA
constexpr int BSTAGES = 3;            // activation ring depth (one stage = the same four 32-blocks)
constexpr int ASLOTS = 3;             // TMEM slots holding one dequantised ring stage (4 blocks x 16 columns) each
constexpr int THREADS = 12 * 32;
constexpr int EPI_THREADS = 128;
constexpr int B_STAGE_KCORES = WSTAGE_BLOCKS * 4;     // 8-wide K cores per activation stage
constexpr int DEQ_SETS = 2;           // dequant warp sets, alternate blocks

template <int NB>
struct Cfg {
    static constexpr int KCORE_BYTES = NB * 16;                     // one K core: NB rows x 8 K x 2 B
    static constexpr int B_STAGE_BYTES = B_STAGE_KCORES * KCORE_BYTES;
    static constexpr int A_SLOT_COLS = WSTAGE_BLOCKS * 16;          // A slot s: columns [64 s, 64 s + 64)
    static constexpr int A_COL0 = 0;
    static constexpr int D_COL0 = ASLOTS * A_SLOT_COLS;             // the accumulator: NB columns
    static constexpr int USED_COLS = ASLOTS * A_SLOT_COLS + NB;
    static constexpr int TMEM_COLS = USED_COLS <= 256 ? 256 : 512;
    static_assert(USED_COLS <= 512, "tensor memory holds 512 columns");
};

template <int NB>
struct Smem {
    alignas(128) uint8_t packed[WSTAGES][WSTAGE_BLOCKS * NT * kBlockBytes];
    alignas(128) uint8_t b[BSTAGES][Cfg<NB>::B_STAGE_BYTES];     // [K core][row][8 K]
    alignas(8) uint64_t w_full[WSTAGES];
    alignas(8) uint64_t w_empty[WSTAGES];
    alignas(8) uint64_t a_full[ASLOTS];      // dequant -> MMA: a stage's A operands are in tensor memory
    alignas(8) uint64_t a_empty[ASLOTS];     // MMA (commit) -> dequant: the stage's A operands are consumed
    alignas(8) uint64_t b_full[BSTAGES];
    alignas(8) uint64_t b_empty[BSTAGES];
    alignas(8) uint64_t d_full;            // MMA (commit) -> epilogue: the accumulator is complete
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
// x 16 bytes stored as 128 contiguous bytes; `lbo_bytes` is the distance to the
// next core matrix along K (leading offset), `sbo_bytes` to the next 8 rows
// (stride offset).  Descriptor version 1 = sm_100.
__device__ __forceinline__ uint64_t make_b_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(lbo_bytes >> 4) << 16;
    d |= (uint64_t)(sbo_bytes >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

// warp-uniform bounded wait
__device__ __forceinline__ bool wait_uniform(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
    const bool got = mbar_wait_bounded(bar, parity, abort_flag);
    return __all_sync(0xffffffffu, got);
}

// NB = MMA N (activation rows padded to 16, 32 or 64)
template <int NB>
__global__ void __launch_bounds__(THREADS, (Cfg<NB>::TMEM_COLS <= 256) ? 2 : 1)
gemm_kernel(const __grid_constant__ GemmParams p)
{
    using C = Cfg<NB>;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Smem<NB>& sm = *reinterpret_cast<Smem<NB>*>(smem_raw);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int n0 = blockIdx.x * NT;
    const int cols = min(NT, p.N - n0);
    const int b0 = blockIdx.y * p.blocks_per_split;
    const int b1 = min(p.nkb, b0 + p.blocks_per_split);
    const int total_blocks = b1 - b0;
    const int gshift = (p.group == 128) ? 2 : 0;

    if (tid == 0) {
        for (int s = 0; s < WSTAGES; ++s) { mbar_init(&sm.w_full[s], 1); mbar_init(&sm.w_empty[s], 4 * DEQ_SETS); }
        for (int s = 0; s < ASLOTS; ++s) { mbar_init(&sm.a_full[s], 4 * DEQ_SETS); mbar_init(&sm.a_empty[s], 1); }
        for (int s = 0; s < BSTAGES; ++s) { mbar_init(&sm.b_full[s], 1); mbar_init(&sm.b_empty[s], 1); }
        mbar_init(&sm.d_full, 1);
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
    auto issue_stage = [&](int st) {                       // executed by the whole warp
        const int slot = st % WSTAGES;
        const int bstart = b0 + st * WSTAGE_BLOCKS;
        const int nb = min(WSTAGE_BLOCKS, b1 - bstart);
        const bool tiled = (p.map_rows == WSTAGE_BLOCKS) && (nb == WSTAGE_BLOCKS) && (p.packed_offsets == nullptr);
        if (lane == 0) {
            mbar_arrive_expect_tx(&sm.w_full[slot], tiled ? (uint32_t)WSTAGE_BLOCKS * NT * kBlockBytes
                                                          : (uint32_t)nb * cols * kBlockBytes);
            if (tiled) tma_load_2d(&sm.packed[slot][0], &p.packed_map, n0 * 2, bstart, &sm.w_full[slot]);
        }
        __syncwarp();
        if (!tiled && lane < nb)
            bulk_g2s(&sm.packed[slot][lane * NT * kBlockBytes],
                     packed + ((size_t)(bstart + lane) * p.N + n0) * kBlockBytes,
                     (uint32_t)cols * kBlockBytes, &sm.w_full[slot]);
        __syncwarp();
    };
    if (warp == 0) {
        if (p.packed_offsets != nullptr) {
            pdl_wait_prior_grids();                  // the offset table may come from the kernel before
            packed += p.packed_offsets[p.expert_idx];
        }
        for (int st = 0; st < min(n_wstages, WSTAGES); ++st) issue_stage(st);
    } else if (warp == 1) {
        tmem_alloc(&sm.tmem_base, C::TMEM_COLS);
        tc_fence_before();
    }
    // every role needs the TMEM base address
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sm.tmem_base;

    if (warp == 0) {
        // ------------------------------ TMA producer (packed, then activations) --
        // Weight stages WSTAGES.. and all activation stages.  Activations come from the
        // pre-pass kernel, so they wait for the preceding grid; weights never do.
        PROF_DECL;
        pdl_wait_prior_grids();
        auto issue_b = [&](int st) {
            if (lane == 0) {
                const int bs = st % BSTAGES;
                mbar_arrive_expect_tx(&sm.b_full[bs], (uint32_t)C::B_STAGE_BYTES);
                tma_load_2d(&sm.b[bs][0], &p.act_map, 0, (b0 + st * WSTAGE_BLOCKS) * 4, &sm.b_full[bs]);
            }
            __syncwarp();
        };
        // Two independent streams, each as far ahead as its ring allows: activation stages
        // (BSTAGES deep) and weight stages (WSTAGES deep).  Single polls, so neither ring
        // waits for the other; the idle counter bounds the loop.
        int bst = 0, wst = min(n_wstages, WSTAGES);
        uint32_t idle = 0;
        while ((bst < n_wstages || wst < n_wstages) && idle < (1u << 22)) {
            bool progress = false;
            if (bst < n_wstages) {
                bool free_b = bst < BSTAGES;
                if (!free_b) free_b = mbar_try_wait(&sm.b_empty[bst % BSTAGES], ((bst / BSTAGES) - 1) & 1);
                if (__all_sync(0xffffffffu, free_b)) { issue_b(bst); ++bst; progress = true; }
            }
            if (wst < n_wstages) {
                const bool free_w = mbar_try_wait(&sm.w_empty[wst % WSTAGES], ((wst / WSTAGES) - 1) & 1);
                if (__all_sync(0xffffffffu, free_w)) { issue_stage(wst); ++wst; progress = true; }
            }
            if (progress) { idle = 0; } else { ++idle; if (idle > 64) __nanosleep(64); if (*abort_flag) break; }
        }
        if (bst < n_wstages || wst < n_wstages) { *abort_flag = 1; atomicOr(&g_error_word, 1u); }
        PROF_FLUSH(0);
    } else if (warp == 1) {
        // ------------------------------------------------------- MMA issuer --
        if (lane == 0) {
            uint32_t idesc = 0;
            idesc |= 1u << 4;                         // D format f32
            idesc |= (uint32_t)(NB >> 3) << 17;       // N
            idesc |= (uint32_t)(128 >> 4) << 24;      // M
            const uint32_t d_addr = tmem_base + C::D_COL0;
            // One pass per ring stage (four 32-blocks): two waits, eight MMAs back to back, two
            // commits.  The issuing thread's own instruction stream is the scarce resource here
            // (about 46 clk per tcgen05.mma, as much again per commit or barrier poll).
            const uint64_t kcore_step = (uint64_t)(C::KCORE_BYTES >> 4);           // descriptor address units
            PROF_DECL;
            bool ok = true;
            for (int st = 0; st < n_wstages; ++st) {
                const int aslot = st % ASLOTS;
                const int bs = st % BSTAGES;
                const int nb = min(WSTAGE_BLOCKS, total_blocks - st * WSTAGE_BLOCKS);
                PROF_BEGIN(t0);
                if (!mbar_wait_bounded(&sm.b_full[bs], (st / BSTAGES) & 1, abort_flag)) { ok = false; break; }
                PROF_END(t0, 0);
                PROF_BEGIN(t2);
                if (!mbar_wait_bounded(&sm.a_full[aslot], (st / ASLOTS) & 1, abort_flag)) { ok = false; break; }
                PROF_END(t2, 2);
                PROF_BEGIN(t3);
                tc_fence_after();
                uint32_t a_addr = tmem_base + C::A_COL0 + aslot * C::A_SLOT_COLS;
                // a block's four K cores sit C::KCORE_BYTES apart; 8-row groups 128 bytes apart
                uint64_t bd = make_b_desc(smem_u32(&sm.b[bs][0]), C::KCORE_BYTES, 128);
#pragma unroll
                for (int bi = 0; bi < WSTAGE_BLOCKS; ++bi) {
                    if (bi < nb) {
                        tc_mma_ts(d_addr, a_addr, bd, idesc, (st == 0 && bi == 0) ? 0u : 1u);
                        tc_mma_ts(d_addr, a_addr + 8, bd + 2 * kcore_step, idesc, 1u);
                    }
                    a_addr += 16;
                    bd += 4 * kcore_step;
                }
                PROF_END(t3, 3);
                PROF_BEGIN(t4);
                tc_commit(&sm.a_empty[aslot]);
                tc_commit(&sm.b_empty[bs]);
                PROF_END(t4, 4);
            }
            if (ok) tc_commit(&sm.d_full);
            PROF_FLUSH(1);
        }
        __syncwarp();
    } else if (warp == 2 || warp == 3) {
        // spare warps (the dequant warps must start at a multiple of four: TMEM lane quarters)
    } else {
        // ------------------------------------------------------- dequant --
        const int set = (warp - 4) >> 2;                       // 0: even blocks, 1: odd blocks
        const int quarter = warp & 3;
        const int col = quarter * 32 + lane;
        const int n = n0 + col;
        const bool owner = n < p.N;
        const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16) + C::A_COL0;
        const uint16_t* scales = p.scales;
        if (p.scales_offsets != nullptr) {
            pdl_wait_prior_grids();                  // the offset table may come from the kernel before
            scales += p.scales_offsets[p.expert_idx];
        }
        PROF_DECL;
        bool ok = true;
        // FP16 scale of this column for each of this set's two blocks of a stage, requested one
        // stage ahead so that the L2 round trip is never waited for
        auto load_scale = [&](int st, int rr) -> uint16_t {
            const int i = st * WSTAGE_BLOCKS + set + rr * DEQ_SETS;
            if (!owner || i >= total_blocks) return (uint16_t)0;
            return __ldg(scales + (size_t)((b0 + i) >> gshift) * p.N + n);
        };
        uint16_t s_next[WSTAGE_BLOCKS / DEQ_SETS];
#pragma unroll
        for (int rr = 0; rr < WSTAGE_BLOCKS / DEQ_SETS; ++rr) s_next[rr] = load_scale(0, rr);
        const __half2 k1032 = __float2half2_rn(1032.0f), k16th = __float2half2_rn(0.0625f), k72 = __float2half2_rn(-72.0f);
        for (int st = 0; st < n_wstages; ++st) {
            const int wslot = st % WSTAGES;
            const int aslot = st % ASLOTS;
            const int nb = min(WSTAGE_BLOCKS, total_blocks - st * WSTAGE_BLOCKS);
            PROF_BEGIN(t0);
            if (!wait_uniform(&sm.w_full[wslot], (st / WSTAGES) & 1, abort_flag)) { ok = false; break; }
            PROF_END(t0, 0);
            bool slot_free = (st < ASLOTS);
            uint16_t s_cur[WSTAGE_BLOCKS / DEQ_SETS];
#pragma unroll
            for (int rr = 0; rr < WSTAGE_BLOCKS / DEQ_SETS; ++rr) {
                s_cur[rr] = s_next[rr];
                s_next[rr] = load_scale(st + 1, rr);
            }
#pragma unroll
            for (int rr = 0; rr < WSTAGE_BLOCKS / DEQ_SETS; ++rr) {
                const int r = set + rr * DEQ_SETS;                 // this set's blocks of the stage: set, set + 2
                if (r < nb) {                                      // warp-uniform
                    const __half2 s2 = __half2half2(__ushort_as_half(s_cur[rr]));
                    PROF_BEGIN(t1);
                    const uint4 v = lds128(&sm.packed[wslot][(r * NT + col) * kBlockBytes]);
                    const uint32_t words[4] = {v.x, v.y, v.z, v.w};
                    uint32_t regs[16];
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        const uint32_t x = words[w];
                        const uint32_t x8 = x >> 8;
                        uint32_t t0b = (x & 0x000F000Fu) | 0x64006400u;      // 1024 + (k0, k4)
                        uint32_t t1b = (x & 0x00F000F0u) | 0x64006400u;      // 1024 + 16 (k1, k5)
                        uint32_t t2b = (x8 & 0x000F000Fu) | 0x64006400u;     // 1024 + (k2, k6)
                        uint32_t t3b = (x8 & 0x00F000F0u) | 0x64006400u;     // 1024 + 16 (k3, k7)
                        const __half2 q0 = __hsub2(*reinterpret_cast<__half2*>(&t0b), k1032);          // q - 8, exact
                        const __half2 q1 = __hfma2(*reinterpret_cast<__half2*>(&t1b), k16th, k72);
                        const __half2 q2 = __hsub2(*reinterpret_cast<__half2*>(&t2b), k1032);
                        const __half2 q3 = __hfma2(*reinterpret_cast<__half2*>(&t3b), k16th, k72);
                        const __half2 w0 = __hmul2(q0, s2), w1 = __hmul2(q1, s2), w2 = __hmul2(q2, s2), w3 = __hmul2(q3, s2);
                        regs[4 * w + 0] = *reinterpret_cast<const uint32_t*>(&w0);
                        regs[4 * w + 1] = *reinterpret_cast<const uint32_t*>(&w1);
                        regs[4 * w + 2] = *reinterpret_cast<const uint32_t*>(&w2);
                        regs[4 * w + 3] = *reinterpret_cast<const uint32_t*>(&w3);
                    }
                    PROF_END(t1, 1);
                    if (!slot_free) {                              // the MMAs that read this slot's previous contents are done
                        PROF_BEGIN(t2);
                        if (!wait_uniform(&sm.a_empty[aslot], ((st / ASLOTS) - 1) & 1, abort_flag)) { ok = false; break; }
                        PROF_END(t2, 2);
                        tc_fence_after();
                        slot_free = true;
                    }
                    PROF_BEGIN(t3);
                    tmem_st16(lane_base + aslot * C::A_SLOT_COLS + r * 16, regs);
                    PROF_END(t3, 3);
                }
            }
            if (!ok) break;
            if (!slot_free) {      // a warp without a block in this (ragged) stage still keeps the slot's phases in step
                if (!wait_uniform(&sm.a_empty[aslot], ((st / ASLOTS) - 1) & 1, abort_flag)) { ok = false; break; }
            }
            PROF_BEGIN(t4);
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(&sm.a_full[aslot]);            // this warp's share of the stage is in tensor memory
                mbar_arrive(&sm.w_empty[wslot]);           // and read out of the ring
            }
            PROF_END(t4, 4);
        }
        PROF_FLUSH(3);

        if (set == 0) {
            // --------------------------------------------------- epilogue --
            // (a K slice with a single block leaves set 1 idle; stages whose odd block is missing are
            //  released by set 0 alone: see the w_empty arrival count below)
            pdl_wait_prior_grids();
            bool have = ok && wait_uniform(&sm.d_full, 0, abort_flag);
            named_bar_sync(2, EPI_THREADS);
            have = have && (*abort_flag == 0);
            const uint32_t lane_d = tmem_base + ((uint32_t)(quarter * 32) << 16) + C::D_COL0;
            auto store_c = [&](int m, float vv) {
                const size_t off = (size_t)m * p.ldc + n;
                if (p.c_is_f16) {
                    __half* cp = reinterpret_cast<__half*>(p.c);
                    if (p.accumulate) vv += __half2float(cp[off]);
                    cp[off] = __float2half_rn(vv);
                } else {
                    float* cp = reinterpret_cast<float*>(p.c);
                    if (p.accumulate) vv += cp[off];
                    cp[off] = vv;
                }
            };
            if (have) {
                tc_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < NB; c0 += 16) {
                    if (c0 < p.M) {                                        // warp-uniform
                        uint32_t d[16];
                        tmem_ld<16>(lane_d + c0, d);
                        tmem_wait_ld();
                        if (owner) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                const int m = c0 + j;
                                if (m < p.M) {
                                    if (p.splits == 1) store_c(m, __uint_as_float(d[j]));
                                    else p.ws_partials[((size_t)blockIdx.y * p.M + m) * p.N + n] = __uint_as_float(d[j]);
                                }
                            }
                        }
                    }
                }
                tc_fence_before();
                if (p.splits > 1) {
                    __threadfence();
                    named_bar_sync(2, EPI_THREADS);
                    if (tid == 4 * 32) {
                        const unsigned prev = atomicAdd(&p.ws_counters[blockIdx.x], 1u);
                        sm.is_last = (prev == (unsigned)(p.splits - 1));
                    }
                    named_bar_sync(2, EPI_THREADS);
                    if (sm.is_last) {
                        __threadfence();
                        if (owner) {
                            for (int m = 0; m < p.M; ++m) {
                                float acc = 0.0f;
                                for (int sp = 0; sp < p.splits; ++sp)
                                    acc += ld_cg_f32(&p.ws_partials[((size_t)sp * p.M + m) * p.N + n]);
                                store_c(m, acc);
                            }
                        }
                        if (tid == 4 * 32) atomicExch(&p.ws_counters[blockIdx.x], 0u);
                    }
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

// Pre-pass of the tcgen05 kernel: rows [0, rows) of the activations, f16 [rows][lda], rewritten as
// [K/8][rows][8] with the eight K of a core in the order k0,k4,k1,k5,k2,k6,k3,k7 (the order in which
// the dequant warps lay nibbles into tensor memory).  One thread per (K core, row).
__global__ void __launch_bounds__(256)
permute_activations_kernel(__half* __restrict__ out, const __half* __restrict__ a, long lda, int rows, int kcores)
{
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * kcores) return;
    const int kc = idx / rows, m = idx - kc * rows;
    const __half* src = a + (size_t)m * lda + (size_t)kc * 8;
    uint4 x;
    if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
        x = *reinterpret_cast<const uint4*>(src);
    } else {
        const uint16_t* s16 = reinterpret_cast<const uint16_t*>(src);
        x.x = s16[0] | ((uint32_t)s16[1] << 16); x.y = s16[2] | ((uint32_t)s16[3] << 16);
        x.z = s16[4] | ((uint32_t)s16[5] << 16); x.w = s16[6] | ((uint32_t)s16[7] << 16);
    }
    uint4 o;
    o.x = __byte_perm(x.x, x.z, 0x5410);      // k0,k4
    o.y = __byte_perm(x.x, x.z, 0x7632);      // k1,k5
    o.z = __byte_perm(x.y, x.w, 0x5410);      // k2,k6
    o.w = __byte_perm(x.y, x.w, 0x7632);      // k3,k7
    reinterpret_cast<uint4*>(out)[idx] = o;
}

}  // namespace tc
}  // namespace twm
