// twm_gemm_tc.cuh — the tcgen05 / TMEM W4A16 kernel (FP16 activations, M >= 9).
//
// The contraction C[m][n] = sum_k A[m][k] * w[k][n] runs on the 5th-generation
// tensor cores with the roles swapped: the 128 weight columns of a CTA are the
// MMA's M dimension (one TMEM lane per column), the activation rows are its N
// dimension (padded to NB = 16 or 32), and K advances 16 at a time.  There
// is no counterpart in the reference: its only batched W4A16 kernel is a 32x32
// SIMT tile kernel on another layout (crates/kernels/src/quantize.rs:186-246),
// and its TW-Marlin kernel is M=1 only (quantize.rs:1186-1298).  Result
// definition as in the streaming kernels: w = f32(scale) * (nibble - 8), exact
// products, FP32 accumulation, the FP32 scale applied per group.
//
// The weight operand is never converted.  A nibble left in place in its 16-bit
// half IS an FP16 subnormal: `v & 0x000F000F` = (q0, q4) * 2^-24, `v & 0x00F000F0`
// = (q1, q5) * 2^-20, the same on `v >> 8` for (q2, q6), (q3, q7): five integer
// instructions per eight nibbles; one FP16 add (or fused multiply-add by 2^-4) per
// pair then makes them the signed weights (q - 8) * 2^-24, exactly (signed_low /
// signed_high below), and the sixteen registers of a 32-block go into tensor memory
// with one tcgen05.st as the MMA's A operand.  The activations enter as they are (the pre-pass only reorders them), so
// every product is exact whatever their magnitude; the scale meets the accumulator
// when a group's sum is read back.
//
// Data path per CTA (128 columns x a K slice of whole scale groups):
//   warp 12      streams packed rows (one tiled TMA load per stage of four
//                32-blocks, 6 deep) and the pre-permuted activations (one tiled
//                TMA load per stage, K-major 8x16-byte core matrices, no swizzle).
//   warps 0-7    unpack: two sets of four warps; each thread owns one column =
//                one TMEM lane; per stage a set unpacks two of the four blocks
//                into the stage's A slot in tensor memory.
//   warps 8-11   read-back: each thread owns one column; for every finished scale
//                group it reads the accumulator (tcgen05.ld), multiplies by its
//                column's scale and adds into registers; at the end it stores C.
//   warp 13      one thread issues tcgen05.mma.cta_group::1.kind::f16 (A from
//                TMEM, B from shared memory, D in TMEM), two per 32-block; every
//                scale group starts a fresh accumulator (two, used in turn);
//                tcgen05.commit hands the accumulator to the readers and frees
//                the A slot and activation stage.
// Tensor memory: ASLOTS x 64 columns of A operands + 2 x NB accumulator columns
// <= 256, so two CTAs share an SM.
// Split-K finish and the programmatic-dependent-launch rules are the same as
// in the streaming kernels.
#pragma once

#include "twm_common.cuh"

namespace twm {
namespace tc {

constexpr int NT = 128;               // columns per CTA = MMA M = TMEM lanes
constexpr int WSTAGE_BLOCKS = 4;      // 32-blocks per ring stage (8 KB)
constexpr int WSTAGES = 6;            // packed ring depth: 48 KB in flight per CTA
constexpr int DEQ_SETS = 2;           // unpack warp sets, alternate blocks
constexpr int DEQ_THREADS = DEQ_SETS * 128;
constexpr int WARP_READ0 = 8;         // first read-back warp
constexpr int B_STAGE_KCORES = WSTAGE_BLOCKS * 4;     // 8-wide K cores per activation stage

// Two nibbles left in place in their 16-bit halves are the FP16 subnormals n * 2^-24 (bits 0-3) or
// (n << 4) * 2^-24 (bits 4-7).  One FP16 instruction turns either pair into the signed weights
// (n - 8) * 2^-24: every value involved is a multiple of 2^-24 below 2^-14, so the results are exact
// (no flush to zero: the intrinsics compile to add/fma without .ftz), and the FP16 pipe is otherwise idle
// in the unpack warps.  With the "-8" inside the operand nothing has to be added to an accumulator later.
__device__ __forceinline__ uint32_t signed_low(uint32_t pair)
{
    const uint32_t minus8 = 0x80088008u;                 // two times -8 * 2^-24 = -2^-21 as FP16 subnormals
    const __half2 r = __hadd2(*reinterpret_cast<const __half2*>(&pair), *reinterpret_cast<const __half2*>(&minus8));
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t signed_high(uint32_t pair)
{
    const uint32_t minus8 = 0x80088008u;
    const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&pair), __float2half2_rn(0.0625f),
                              *reinterpret_cast<const __half2*>(&minus8));
    return *reinterpret_cast<const uint32_t*>(&r);
}

template <int NB>
struct Cfg {
    static constexpr int ASLOTS = (NB == 64) ? 2 : 3;               // stages of A operands (and of activations) in flight
    static constexpr int KCORE_BYTES = NB * 16;                     // one K core: NB rows x 8 K x 2 B
    static constexpr int B_STAGE_BYTES = B_STAGE_KCORES * KCORE_BYTES;
    static constexpr int A_SLOT_COLS = WSTAGE_BLOCKS * 16;          // A slot s: columns [64 s, 64 s + 64)
    static constexpr int D_COL0 = ASLOTS * A_SLOT_COLS;             // two accumulators of NB columns
    // 256 tensor-memory columns, two CTAs per SM; four read-back warps per 32 accumulator columns
    // (64 rows: two A slots instead of three, eight read-back warps).
    static constexpr int TMEM_COLS = (D_COL0 + 2 * NB <= 256) ? 256 : 512;
    static constexpr int READ_SETS = (NB + 31) / 32;
    static constexpr int READ_COLS = NB / READ_SETS;                // accumulator columns per read-back warp
    static constexpr int EPI_THREADS = READ_SETS * 128;
    static constexpr int WARP_TMA = WARP_READ0 + 4 * READ_SETS;
    static constexpr int WARP_MMA = WARP_TMA + 1;
    static constexpr int THREADS = (WARP_MMA + 1) * 32;
    static constexpr int CTAS_PER_SM = (TMEM_COLS == 256) ? 2 : 1;
    static_assert(D_COL0 + 2 * NB <= TMEM_COLS, "tensor memory budget of a CTA");
};

template <int NB>
struct Smem {
    alignas(128) uint8_t packed[WSTAGES][WSTAGE_BLOCKS * NT * kBlockBytes];
    alignas(128) uint8_t b[Cfg<NB>::ASLOTS][Cfg<NB>::B_STAGE_BYTES];          // [K core][row][8 K]
    alignas(8) uint64_t w_full[WSTAGES];
    alignas(8) uint64_t w_empty[WSTAGES];
    alignas(8) uint64_t a_full[Cfg<NB>::ASLOTS];     // unpack -> MMA: a stage's A operands are in tensor memory
    alignas(8) uint64_t ab_empty[Cfg<NB>::ASLOTS];   // MMA (commit) -> unpack and TMA: A slot and activation stage are consumed
    alignas(8) uint64_t b_full[Cfg<NB>::ASLOTS];
    alignas(8) uint64_t d_full[2];                   // MMA (commit) -> readers: a scale group's accumulator is complete
    alignas(8) uint64_t d_empty[2];                  // readers -> MMA: the accumulator has been read
    // group-128 path (a stage is one scale group): everything the MMA thread waits for before a
    // stage arrives on ONE barrier (8 unpack warps + the activation stage's bytes + the 4 readers
    // that freed the accumulator two stages ago), and one commit per stage tells everybody that
    // the stage's MMAs are done (accumulator complete, A slot and activation stage free)
    alignas(8) uint64_t ready[Cfg<NB>::ASLOTS];
    alignas(8) uint64_t done[4];
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
// NB = MMA N (activation rows padded to 16 or 32)
template <int NB>
__global__ void __launch_bounds__(Cfg<NB>::THREADS, Cfg<NB>::CTAS_PER_SM)
gemm_kernel(const __grid_constant__ GemmParams p)
{
    using C = Cfg<NB>;
    constexpr int ASLOTS = C::ASLOTS;
    constexpr int TMEM_COLS = C::TMEM_COLS;
    constexpr int EPI_THREADS = C::EPI_THREADS;
    constexpr int WARP_TMA = C::WARP_TMA;
    constexpr int WARP_MMA = C::WARP_MMA;
    constexpr int RC = C::READ_COLS;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Smem<NB>& sm = *reinterpret_cast<Smem<NB>*>(smem_raw);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int n0 = blockIdx.x * NT;
    const int cols = min(NT, p.N - n0);
    const int b0 = blockIdx.y * p.blocks_per_split;          // a multiple of the group's blocks (host plan)
    const int b1 = min(p.nkb, b0 + p.blocks_per_split);
    const int total_blocks = b1 - b0;
    const int gshift = (p.group == 128) ? 2 : 0;
    const int n_wstages = (total_blocks + WSTAGE_BLOCKS - 1) / WSTAGE_BLOCKS;
    const bool lean = (gshift == 2);         // one scale group per stage

    if (tid == 0) {
        for (int s = 0; s < WSTAGES; ++s) { mbar_init(&sm.w_full[s], 1); mbar_init(&sm.w_empty[s], 4 * DEQ_SETS); }
        for (int s = 0; s < ASLOTS; ++s) {
            mbar_init(&sm.a_full[s], 4 * DEQ_SETS); mbar_init(&sm.ab_empty[s], 1); mbar_init(&sm.b_full[s], 1);
        }
        for (int s = 0; s < 2; ++s) { mbar_init(&sm.d_full[s], 1); mbar_init(&sm.d_empty[s], EPI_THREADS / 32); }
        for (int s = 0; s < ASLOTS; ++s) mbar_init(&sm.ready[s], 4 * DEQ_SETS + 1 + EPI_THREADS / 32);
        for (int s = 0; s < 4; ++s) mbar_init(&sm.done[s], 1);
        // the first two stages find their accumulators free: the readers' arrivals are made here
        for (int s = 0; s < 2; ++s)
            for (int i = 0; i < EPI_THREADS / 32; ++i) mbar_arrive(&sm.ready[s]);
        sm.abort_flag = 0;
        sm.is_last = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    volatile int* abort_flag = &sm.abort_flag;

    // TMA producer state (warp 12).  The first ring-full of stages is issued before the TMEM
    // allocation below, so that weights are already streaming while an earlier kernel's CTA may
    // still hold this SM's tensor memory.
    const uint8_t* packed = p.packed;
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
    if (warp == WARP_TMA) {
        if (p.packed_offsets != nullptr) {
            pdl_wait_prior_grids();                  // the offset table may come from the kernel before
            packed += p.packed_offsets[p.expert_idx];
        }
        for (int st = 0; st < min(n_wstages, WSTAGES); ++st) issue_stage(st);
    } else if (warp == WARP_MMA) {
        tmem_alloc(&sm.tmem_base, TMEM_COLS);
        tc_fence_before();
    }
    // every role needs the TMEM base address
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sm.tmem_base;

    if (warp == WARP_TMA) {
        // ------------------------------ TMA producer (packed, then activations) --
        // Weight stages WSTAGES.. and all activation stages.  Activations come from the
        // pre-pass kernel, so they wait for the preceding grid; weights never do.
        pdl_wait_prior_grids();
        auto issue_b = [&](int st) {
            if (lane == 0) {
                const int bs = st % ASLOTS;
                uint64_t* bar = lean ? &sm.ready[bs] : &sm.b_full[bs];
                mbar_arrive_expect_tx(bar, (uint32_t)C::B_STAGE_BYTES);
                tma_load_2d(&sm.b[bs][0], &p.act_map, 0, (b0 + st * WSTAGE_BLOCKS) * 4, bar);
            }
            __syncwarp();
        };
        // Two independent streams, each as far ahead as its ring allows.  Single polls, so
        // neither ring waits for the other; the idle counter bounds the loop.
        int bst = 0, wst = min(n_wstages, WSTAGES);
        uint32_t idle = 0;
        while ((bst < n_wstages || wst < n_wstages) && idle < (1u << 22)) {
            bool progress = false;
            if (bst < n_wstages) {
                bool free_b = bst < ASLOTS;
                if (!free_b)
                    free_b = lean ? mbar_try_wait(&sm.done[(bst - ASLOTS) & 3], ((bst - ASLOTS) >> 2) & 1)
                                  : mbar_try_wait(&sm.ab_empty[bst % ASLOTS], ((bst / ASLOTS) - 1) & 1);
                if (__all_sync(0xffffffffu, free_b)) { issue_b(bst); ++bst; progress = true; }
            }
            if (wst < n_wstages) {
                const bool free_w = mbar_try_wait(&sm.w_empty[wst % WSTAGES], ((wst / WSTAGES) - 1) & 1);
                if (__all_sync(0xffffffffu, free_w)) { issue_stage(wst); ++wst; progress = true; }
            }
            if (progress) { idle = 0; } else { ++idle; if (idle > 64) __nanosleep(64); if (*abort_flag) break; }
        }
        if (bst < n_wstages || wst < n_wstages) { *abort_flag = 1; atomicOr(&g_error_word, 1u); }
    } else if (warp == WARP_MMA) {
        // ------------------------------------------------------- MMA issuer --
        if (lane == 0) {
            uint32_t idesc = 0;
            idesc |= 1u << 4;                         // D format f32
            idesc |= (uint32_t)(NB >> 3) << 17;       // N
            idesc |= (uint32_t)(128 >> 4) << 24;      // M
            const uint64_t kcore_step = (uint64_t)(C::KCORE_BYTES >> 4);           // descriptor address units
            int gq = 0;                               // scale groups started so far: accumulator gq & 1
            bool ok = true;
            // accumulator for group gq: wait until the readers have taken its previous contents
            auto open_group = [&]() -> uint32_t {
                const int db = gq & 1;
                if (gq >= 2 && !mbar_wait_bounded(&sm.d_empty[db], ((gq >> 1) - 1) & 1, abort_flag)) ok = false;
                tc_fence_after();
                return tmem_base + C::D_COL0 + db * NB;
            };
            if (lean) {
                // per stage: one wait, eight MMAs into accumulator st & 1, one commit
                for (int st = 0; st < n_wstages; ++st) {
                    const int aslot = st % ASLOTS;
                    if (!mbar_wait_bounded(&sm.ready[aslot], (st / ASLOTS) & 1, abort_flag)) break;
                    tc_fence_after();
                    const uint32_t d_addr = tmem_base + C::D_COL0 + (st & 1) * NB;
                    uint32_t a_addr = tmem_base + aslot * C::A_SLOT_COLS;
                    uint64_t bd = make_b_desc(smem_u32(&sm.b[aslot][0]), C::KCORE_BYTES, 128);
#pragma unroll
                    for (int bi = 0; bi < WSTAGE_BLOCKS; ++bi) {
                        tc_mma_ts(d_addr, a_addr, bd, idesc, bi == 0 ? 0u : 1u);
                        tc_mma_ts(d_addr, a_addr + 8, bd + 2 * kcore_step, idesc, 1u);
                        a_addr += 16;
                        bd += 4 * kcore_step;
                    }
                    tc_commit(&sm.done[st & 3]);
                }
            } else
            for (int st = 0; st < n_wstages && ok; ++st) {
                const int aslot = st % ASLOTS;
                const int nb = min(WSTAGE_BLOCKS, total_blocks - st * WSTAGE_BLOCKS);
                if (!mbar_wait_bounded(&sm.b_full[aslot], (st / ASLOTS) & 1, abort_flag)) { ok = false; break; }
                if (!mbar_wait_bounded(&sm.a_full[aslot], (st / ASLOTS) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after();
                uint32_t a_addr = tmem_base + aslot * C::A_SLOT_COLS;
                // a block's four K cores sit C::KCORE_BYTES apart; 8-row groups 128 bytes apart
                uint64_t bd = make_b_desc(smem_u32(&sm.b[aslot][0]), C::KCORE_BYTES, 128);
                if (gshift == 2) {
                    // the stage is one scale group: eight MMAs into one fresh accumulator
                    const uint32_t d_addr = open_group();
                    if (!ok) break;
#pragma unroll
                    for (int bi = 0; bi < WSTAGE_BLOCKS; ++bi) {
                        if (bi < nb) {
                            tc_mma_ts(d_addr, a_addr, bd, idesc, bi == 0 ? 0u : 1u);
                            tc_mma_ts(d_addr, a_addr + 8, bd + 2 * kcore_step, idesc, 1u);
                        }
                        a_addr += 16;
                        bd += 4 * kcore_step;
                    }
                    tc_commit(&sm.d_full[gq & 1]);
                    ++gq;
                } else {
                    // every 32-block is a scale group
                    for (int bi = 0; bi < nb && ok; ++bi) {
                        const uint32_t d_addr = open_group();
                        if (!ok) break;
                        tc_mma_ts(d_addr, a_addr, bd, idesc, 0u);
                        tc_mma_ts(d_addr, a_addr + 8, bd + 2 * kcore_step, idesc, 1u);
                        tc_commit(&sm.d_full[gq & 1]);
                        ++gq;
                        a_addr += 16;
                        bd += 4 * kcore_step;
                    }
                }
                tc_commit(&sm.ab_empty[aslot]);
            }
        }
        __syncwarp();
    } else if (warp < WARP_READ0) {
        // ------------------------------------------------------------ unpack --
        const int set = warp >> 2;                             // 0: even blocks, 1: odd blocks
        const int quarter = warp & 3;
        const int col = quarter * 32 + lane;
        const uint32_t lane_tmem = tmem_base + ((uint32_t)(quarter * 32) << 16);
        for (int st = 0; st < n_wstages; ++st) {
            const int wslot = st % WSTAGES;
            const int aslot = st % ASLOTS;
            const int nb = min(WSTAGE_BLOCKS, total_blocks - st * WSTAGE_BLOCKS);
            if (!wait_uniform(&sm.w_full[wslot], (st / WSTAGES) & 1, abort_flag)) break;
            if (st >= ASLOTS) {        // the MMAs that read this slot's previous contents are done
                uint64_t* bar = lean ? &sm.done[(st - ASLOTS) & 3] : &sm.ab_empty[aslot];
                const uint32_t par = lean ? (((st - ASLOTS) >> 2) & 1) : (((st / ASLOTS) - 1) & 1);
                if (!wait_uniform(bar, par, abort_flag)) break;
                tc_fence_after();
            }
#pragma unroll
            for (int rr = 0; rr < WSTAGE_BLOCKS / DEQ_SETS; ++rr) {
                const int r = set + rr * DEQ_SETS;                 // this set's blocks of the stage: set, set + 2
                if (r < nb) {                                      // warp-uniform
                    const uint4 v = lds128(&sm.packed[wslot][(r * NT + col) * kBlockBytes]);
                    const uint32_t words[4] = {v.x, v.y, v.z, v.w};
                    uint32_t regs[16];
#pragma unroll
                    for (int w = 0; w < 4; ++w) {
                        const uint32_t x = words[w];
                        const uint32_t x8 = x >> 8;
                        regs[4 * w + 0] = signed_low(x & 0x000F000Fu);          // (k0, k4): (n - 8) * 2^-24
                        regs[4 * w + 1] = signed_high(x & 0x00F000F0u);         // (k1, k5)
                        regs[4 * w + 2] = signed_low(x8 & 0x000F000Fu);         // (k2, k6)
                        regs[4 * w + 3] = signed_high(x8 & 0x00F000F0u);        // (k3, k7)
                    }
                    tmem_st16(lane_tmem + aslot * C::A_SLOT_COLS + r * 16, regs);
                }
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(lean ? &sm.ready[aslot] : &sm.a_full[aslot]);   // this warp's share of the stage is in tensor memory
                mbar_arrive(&sm.w_empty[wslot]);                             // and read out of the ring
            }
        }
    } else if (warp < WARP_TMA) {
        // ------------------------------------- per-group read-back and epilogue --
        const int quarter = warp & 3;
        const int rset = (warp - WARP_READ0) >> 2;            // which RC accumulator columns (activation rows) this warp takes
        const int row0 = rset * RC;
        const int col = quarter * 32 + lane;
        const int n = n0 + col;
        const bool owner = n < p.N;
        const uint32_t lane_tmem = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint16_t* scales = p.scales;
        pdl_wait_prior_grids();          // C may be read by the kernel before
        if (p.scales_offsets != nullptr) scales += p.scales_offsets[p.expert_idx];
        float acc[RC];
#pragma unroll
        for (int j = 0; j < RC; ++j) acc[j] = 0.0f;
        bool ok = true;
        const int n_groups = (gshift == 2) ? n_wstages : total_blocks;
        const int grow0 = b0 >> gshift;
        auto load_scale = [&](int gq) -> uint16_t {
            return (owner && gq < n_groups) ? __ldg(scales + (size_t)(grow0 + gq) * p.N + n) : (uint16_t)0;
        };
        uint16_t s_next = load_scale(0);
        for (int gq = 0; gq < n_groups; ++gq) {
            // accumulator of scale group gq: acc += (s * 2^24) * D
            const int db = gq & 1;
            const float sg = f16_bits_to_f32(s_next) * 16777216.0f;
            s_next = load_scale(gq + 1);
            {
                uint64_t* bar = lean ? &sm.done[gq & 3] : &sm.d_full[db];
                const uint32_t par = lean ? ((gq >> 2) & 1) : ((gq >> 1) & 1);
                if (!wait_uniform(bar, par, abort_flag)) { ok = false; break; }
            }
            tc_fence_after();
#pragma unroll
            for (int c0 = 0; c0 < RC; c0 += 8) {
                if (row0 + c0 < p.M) {                                 // warp-uniform
                    uint32_t d[8];
                    tmem_ld<8>(lane_tmem + C::D_COL0 + db * NB + row0 + c0, d);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[c0 + j] = fmaf(sg, __uint_as_float(d[j]), acc[c0 + j]);
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(lean ? &sm.ready[(gq + 2) % ASLOTS] : &sm.d_empty[db]);   // the accumulator is free again
        }
        ok = ok && (*abort_flag == 0);

        // tensor-parallel row shard: the FP32 result goes to every peer's receive slot instead of C
        const unsigned int comm_seq = p.n_peers ? ld_volatile_u32(p.comm_state) : 0u;
        auto store_at = [&](int m, int nn, float vv) {
            const size_t off = (size_t)m * p.ldc + nn;
            if (p.n_peers) { comm_store(p, comm_seq, off, vv); return; }
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
        auto store_c = [&](int m, float vv) { store_at(m, n, vv); };
        if (ok && owner) {
#pragma unroll
            for (int j = 0; j < RC; ++j) {
                const int m = row0 + j;
                if (m < p.M) {
                    const float v = acc[j];
                    if (p.splits == 1) store_c(m, v);
                    else p.ws_partials[((size_t)blockIdx.y * p.M + m) * p.N + n] = v;
                }
            }
        }
        if (p.splits > 1) {
            __threadfence();
            named_bar_sync(3, EPI_THREADS);
            if (tid == WARP_READ0 * 32) {
                const unsigned prev = atomicAdd(&p.ws_counters[blockIdx.x], 1u);
                sm.is_last = (prev == (unsigned)(p.splits - 1));
            }
            named_bar_sync(3, EPI_THREADS);
            if (sm.is_last) {
                __threadfence();
                if (*abort_flag == 0) {
                    // Slices in slice order.  The tile is walked four columns per thread, a warp along a row
                    // (coalesced), by all read-back threads, the slices' loads issued together: a thread that
                    // summed its own column row by row waited a round trip to L2 per row and slice (45 us of a
                    // 49 us launch at 32 rows in 7 slices).
                    const bool vec = (p.N & 3) == 0;
                    const int e = tid - WARP_READ0 * 32;
                    for (int idx = e; idx < p.M * 32; idx += EPI_THREADS) {
                        const int m = idx >> 5, c = n0 + (idx & 31) * 4;
                        if (c >= p.N) continue;
                        float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                        if (vec) {
#pragma unroll 4
                            for (int sp = 0; sp < p.splits; ++sp) {
                                const float4 t4 = __ldcg(reinterpret_cast<const float4*>(&p.ws_partials[((size_t)sp * p.M + m) * p.N + c]));
                                v[0] += t4.x; v[1] += t4.y; v[2] += t4.z; v[3] += t4.w;
                            }
                        } else {
                            for (int sp = 0; sp < p.splits; ++sp)
                                for (int j = 0; j < 4; ++j)
                                    if (c + j < p.N) v[j] += ld_cg_f32(&p.ws_partials[((size_t)sp * p.M + m) * p.N + c + j]);
                        }
                        for (int j = 0; j < 4; ++j)
                            if (c + j < p.N) store_at(m, c + j, v[j]);
                    }
                }
                if (tid == WARP_READ0 * 32) atomicExch(&p.ws_counters[blockIdx.x], 0u);
            }
        }
        // the CTAs that stored a tile (every CTA without K slices, the last arriver of each tile with them)
        // count themselves; the last of them raises the peers' flags (also after an expired wait, so that
        // the peers' consumers do not wait for this rank in vain: the error word says the step is void)
        if (p.n_peers && (p.splits == 1 || sm.is_last)) {
            named_bar_sync(3, EPI_THREADS);
            if (tid == WARP_READ0 * 32) comm_cta_done(p, comm_seq, gridDim.x);
        }
    }

    // ------------------------------------------------------------ teardown --
    tc_fence_before();
    __syncthreads();
    if (warp == WARP_MMA) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// Pre-pass of the tcgen05 kernels, one launch per GEMM launch: rows [0, rows) of the activations,
// f16 [rows][lda], rewritten as [K/8][rows][8] with the eight K of a core in the order
// k0,k4,k1,k5,k2,k6,k3,k7 (the order in which the unpack lays nibbles into the operand).  The values
// themselves are not touched, so any FP16 activation, subnormals included, enters the products
// exactly.  One thread per (K core, row).
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
    o.x = __byte_perm(x.x, x.z, 0x5410);              // k0,k4
    o.y = __byte_perm(x.x, x.z, 0x7632);              // k1,k5
    o.z = __byte_perm(x.y, x.w, 0x5410);              // k2,k6
    o.w = __byte_perm(x.y, x.w, 0x7632);              // k3,k7
    reinterpret_cast<uint4*>(out)[idx] = o;
}

}  // namespace tc
}  // namespace twm
