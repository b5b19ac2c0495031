// twm_gemm_tcr.cuh — the tcgen05 / TMEM W4A16 kernel for many activation rows and wide matrices
// (65 ... 128 rows per launch, scale group 128, N of at least a wave of 256-column tiles).
//
// twm_gemm_tcw.cuh keeps the weights exact: the MMA multiplies (q - 8) * 2^-24 and the FP32 scale
// meets the accumulator once per 128-group, which costs a read-back of the accumulator per group,
// 64 running sums in registers per read-back thread (hence 128-column tiles), and leaves the
// kernel bound by shared-memory traffic: every MMA of 128 x 128 x 16 reads 8 KB of operands.
// This kernel takes the reference's own route for more than one row instead: the weights enter the
// tensor core as FP16, w16 = f16_rn(f32(scale) * (q - 8)), which is what dequant_q4_to_f16 stores
// before the reference's batched GEMM (crates/kernels/src/quantize.rs:534-571): one rounding per
// weight (relative 2^-11), exact products, FP32 accumulation over the whole K in ONE accumulator.
// No read-back per group, no running sums in registers: the tile is 128 rows x 256 columns, one
// tcgen05.mma does 128 x 256 x 16 and reads the activation operand once for 256 columns, and the
// accumulator is read out once, at the end, by the warps that unpacked.
//
// Stage = 64 K (two 32-blocks).  Warps 0-15: unpack (thread = one column of one of the stage's two
// blocks: masks leave the nibbles as
// 1024 + q or 1024 + 16 q in FP16, one FP16 subtract or fused multiply-add makes q - 8 exactly, one
// FP16 multiply by the column's scale rounds once), then, after the last stage, read-back and store
// (thread = activation row, 64 columns).  Warp 16: TMA producer.  Warp 17: MMA issuer.  K order inside an
// 8-wide core is k0,k4,k1,k5,k2,k6,k3,k7 as in the other tcgen05 kernels (the pre-pass writes the
// activations that way).  One CTA per SM (about 180 KB of shared memory), 256 TMEM columns.
#pragma once

#include "twm_common.cuh"
#include "twm_gemm_tc.cuh"
#include "twm_gemm_tcw.cuh"

namespace twm {
namespace tcr {

constexpr int NT = 256;                 // weight columns per CTA = MMA N
constexpr int MB = 128;                 // activation rows per MMA (rows past M are zero)
constexpr int SB = 2;                   // 32-blocks per stage: 64 K
constexpr int SSTAGES = 4;              // scale rows of the tile (one per 128-group, 512 B)
constexpr int KCORES = SB * 4;          // 8-wide K cores per stage
constexpr int A_BLOCK_BYTES = KCORES * MB * 16;        // one block of 128 rows: [K core][row][16 bytes]
constexpr int B_STAGE_BYTES = KCORES * NT * 16;        // [K core][column][16 bytes]
constexpr int P_HALF_BYTES = SB * 128 * kBlockBytes;   // one tensor-map box: [block][128 columns][16 bytes]
constexpr int P_STAGE_BYTES = 2 * P_HALF_BYTES;
constexpr int UNPACK_WARPS = 16;        // two sets of eight: set s unpacks block s of every stage
constexpr int WARP_TMA = UNPACK_WARPS, WARP_MMA = WARP_TMA + 1;
constexpr int THREADS = (WARP_MMA + 1) * 32;

// RB = blocks of 128 activation rows per launch (1: up to 128 rows, 2: up to 256).  With two blocks
// every unpacked stage feeds two MMAs per K step (one per row block, one accumulator each), so
// the unpack and the weight traffic are paid once for 256 rows.
template <int RB>
struct Cfg {
    static constexpr int PSTAGES = RB == 1 ? 6 : 5;            // packed ring, 8 KB stages
    static constexpr int ASTAGES = RB == 1 ? 4 : 3;            // activation stages of RB x 16 KB
    static constexpr int BSTAGES = RB == 1 ? 3 : 2;            // unpacked FP16 weights, 32 KB stages
    static constexpr int A_STAGE_BYTES = RB * A_BLOCK_BYTES;
    static constexpr int TMEM_COLS = RB * NT;                  // one accumulator of 256 columns per row block
};

template <int RB>
struct Smem {
    alignas(128) uint8_t packed[Cfg<RB>::PSTAGES][P_STAGE_BYTES];     // [half of the tile][block][column of the half][16 bytes]
    alignas(128) uint8_t bw[Cfg<RB>::BSTAGES][B_STAGE_BYTES];
    alignas(128) uint8_t a[Cfg<RB>::ASTAGES][Cfg<RB>::A_STAGE_BYTES]; // [row block][K core][row][16 bytes]
    alignas(16) uint16_t sc[SSTAGES][NT];
    alignas(8) uint64_t p_full[Cfg<RB>::PSTAGES];
    alignas(8) uint64_t p_empty[Cfg<RB>::PSTAGES];       // unpack warps
    alignas(8) uint64_t b_full[Cfg<RB>::BSTAGES];        // unpack warps
    alignas(8) uint64_t b_empty[Cfg<RB>::BSTAGES];       // MMA commit
    alignas(8) uint64_t a_full[Cfg<RB>::ASTAGES];
    alignas(8) uint64_t a_empty[Cfg<RB>::ASTAGES];       // MMA commit
    alignas(8) uint64_t d_full;                          // MMA commit: the tile's accumulators are complete
    uint32_t tmem_base;
    int abort_flag;
};

template <int RB>
__global__ void __launch_bounds__(THREADS, 1)
gemm_kernel(const __grid_constant__ GemmParams p)
{
    using C = Cfg<RB>;
    constexpr int PSTAGES = C::PSTAGES, ASTAGES = C::ASTAGES, BSTAGES = C::BSTAGES, TMEM_COLS = C::TMEM_COLS;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Smem<RB>& sm = *reinterpret_cast<Smem<RB>*>(smem_raw);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int n0 = blockIdx.x * NT;
    const int n_stages = p.nkb / SB;                         // the whole K: this kernel does not split it

    if (tid == 0) {
        for (int s = 0; s < PSTAGES; ++s) { mbar_init(&sm.p_full[s], 1); mbar_init(&sm.p_empty[s], UNPACK_WARPS); }
        for (int s = 0; s < BSTAGES; ++s) { mbar_init(&sm.b_full[s], UNPACK_WARPS); mbar_init(&sm.b_empty[s], 1); }
        for (int s = 0; s < ASTAGES; ++s) { mbar_init(&sm.a_full[s], 1); mbar_init(&sm.a_empty[s], 1); }
        mbar_init(&sm.d_full, 1);
        sm.abort_flag = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    volatile int* abort_flag = &sm.abort_flag;

    // A whole tile inside N with 16-byte aligned scale rows: the group's 256 scales (512 bytes) ride along with
    // the group's first packed stage; otherwise the unpack threads read them from global memory.
    const bool scale_bulk = (n0 + NT <= p.N) && ((p.N & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.scales) & 15) == 0);
    const bool second_half = n0 + 128 < p.N;                 // a ragged last tile may hold one half only
    auto issue_p = [&](int st) {                             // lane 0 of the TMA warp
        const int slot = st % PSTAGES;
        const bool with_scales = scale_bulk && (st & 1) == 0;
        mbar_arrive_expect_tx(&sm.p_full[slot], (uint32_t)(second_half ? P_STAGE_BYTES : P_HALF_BYTES) + (with_scales ? (uint32_t)NT * 2 : 0u));
        tma_load_2d(&sm.packed[slot][0], &p.packed_map, n0 * 2, st * SB, &sm.p_full[slot]);
        if (second_half) tma_load_2d(&sm.packed[slot][P_HALF_BYTES], &p.packed_map, (n0 + 128) * 2, st * SB, &sm.p_full[slot]);
        if (with_scales)
            bulk_g2s(&sm.sc[(st >> 1) % SSTAGES][0], p.scales + (size_t)(st >> 1) * p.N + n0, (uint32_t)NT * 2, &sm.p_full[slot]);
    };
    if (warp == WARP_TMA) {
        // weights are constants: the first ring-full streams before the preceding kernel has finished
        if (lane == 0)
            for (int st = 0; st < min(n_stages, PSTAGES); ++st) issue_p(st);
    } else if (warp == WARP_MMA) {
        tc::tmem_alloc(&sm.tmem_base, TMEM_COLS);
        tc::tc_fence_before();
    }
    __syncthreads();
    tc::tc_fence_after();
    const uint32_t tmem_base = sm.tmem_base;

    if (warp == WARP_TMA) {
        // ---------------------------------------------- TMA producer (one thread) --
        pdl_wait_prior_grids();                              // the activations come from the pre-pass
        if (lane == 0) {
            int ast = 0, pst = min(n_stages, PSTAGES);
            uint32_t idle = 0;
            while ((ast < n_stages || pst < n_stages) && idle < (1u << 22)) {
                bool progress = false;
                if (ast < n_stages) {
                    const int as = ast % ASTAGES;
                    if (ast < ASTAGES || mbar_try_wait(&sm.a_empty[as], ((ast / ASTAGES) - 1) & 1)) {
                        mbar_arrive_expect_tx(&sm.a_full[as], (uint32_t)C::A_STAGE_BYTES);
#pragma unroll
                        for (int rb = 0; rb < RB; ++rb)         // rows 128 rb ...: 256 64-bit words further along a K core's row run
                            tma_load_2d(&sm.a[as][rb * A_BLOCK_BYTES], &p.act_map, rb * MB * 2, ast * KCORES, &sm.a_full[as]);
                        ++ast; progress = true;
                    }
                }
                if (pst < n_stages) {
                    // the scale row's slot is free as well: its group was consumed before this packed slot's previous stage
                    if (mbar_try_wait(&sm.p_empty[pst % PSTAGES], ((pst / PSTAGES) - 1) & 1)) { issue_p(pst); ++pst; progress = true; }
                }
                if (progress) { idle = 0; } else { ++idle; if (idle > 64) __nanosleep(64); if (*abort_flag) break; }
            }
            if (ast < n_stages || pst < n_stages) { *abort_flag = 1; atomicOr(&g_error_word, 1u); }
        }
        __syncwarp();
    } else if (warp == WARP_MMA) {
        // -------------------------------------------------- MMA issuer (one thread) --
        if (lane == 0) {
            uint32_t idesc = 0;
            idesc |= 1u << 4;                          // D format f32 (A and B: f16, both K-major)
            idesc |= (uint32_t)(NT >> 3) << 17;        // N
            idesc |= (uint32_t)(MB >> 4) << 24;        // M
            bool ok = true;
            for (int st = 0; st < n_stages; ++st) {
                const int as = st % ASTAGES, bs = st % BSTAGES;
                if (!mbar_wait_bounded(&sm.a_full[as], (st / ASTAGES) & 1, abort_flag)) { ok = false; break; }
                if (!mbar_wait_bounded(&sm.b_full[bs], (st / BSTAGES) & 1, abort_flag)) { ok = false; break; }
                tc::tc_fence_after();
                // A: [K core][row][16 B]: next K core MB*16 bytes on, next 8 rows 128 bytes on.
                // B: [K core][column][16 B]: next K core NT*16 bytes on, next 8 columns 128 bytes on.
                constexpr uint64_t a_step = (uint64_t)((2 * MB * 16) >> 4), b_step = (uint64_t)((2 * NT * 16) >> 4);   // two K cores, in descriptor units
#pragma unroll
                for (int rb = 0; rb < RB; ++rb) {                           // one accumulator per block of 128 rows
                    uint64_t ad = tc::make_b_desc(smem_u32(&sm.a[as][rb * A_BLOCK_BYTES]), MB * 16, 128);
                    uint64_t bd = tc::make_b_desc(smem_u32(&sm.bw[bs][0]), NT * 16, 128);
#pragma unroll
                    for (int h = 0; h < 2 * SB; ++h) {                      // four MMAs of K = 16
                        tcw::mma_ss(tmem_base + rb * NT, ad, bd, idesc, (st == 0 && h == 0) ? 0u : 1u);
                        ad += a_step;
                        bd += b_step;
                    }
                }
                tc::tc_commit(&sm.b_empty[bs]);
                tc::tc_commit(&sm.a_empty[as]);
            }
            if (ok) tc::tc_commit(&sm.d_full);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ unpack --
        const int col = tid & 255;                             // 0 .. 255
        const int set = tid >> 8;                              // which of the stage's two blocks this thread unpacks
        const int half = col >> 7, hc = col & 127;
        const bool col_ok = n0 + col < p.N;
        __half2 s2 = __float2half2_rn(0.0f);
        bool ok = true;
        for (int st = 0; st < n_stages; ++st) {
            const int slot = st % PSTAGES, bs = st % BSTAGES;
            if (!tc::wait_uniform(&sm.p_full[slot], (st / PSTAGES) & 1, abort_flag)) { ok = false; break; }
            if (st >= BSTAGES && !tc::wait_uniform(&sm.b_empty[bs], ((st / BSTAGES) - 1) & 1, abort_flag)) { ok = false; break; }
            if ((st & 1) == 0) {                               // a new 128-group: this column's scale, both halves of a register
                uint16_t h = 0;
                if (scale_bulk) h = sm.sc[(st >> 1) % SSTAGES][col];
                else if (col_ok) h = __ldg(p.scales + (size_t)(st >> 1) * p.N + n0 + col);
                const uint32_t hh = (uint32_t)h | ((uint32_t)h << 16);
                s2 = *reinterpret_cast<const __half2*>(&hh);
            }
            const __half2 c1032 = __float2half2_rn(1032.0f), sixteenth = __float2half2_rn(0.0625f), c72 = __float2half2_rn(-72.0f);
            auto low = [&](uint32_t bits) -> uint32_t {        // 1024 + q  ->  f16(scale * (q - 8))
                const uint32_t v = bits | 0x64006400u;
                const __half2 r = __hmul2(__hsub2(*reinterpret_cast<const __half2*>(&v), c1032), s2);
                return *reinterpret_cast<const uint32_t*>(&r);
            };
            auto high = [&](uint32_t bits) -> uint32_t {       // 1024 + 16 q  ->  f16(scale * (q - 8))
                const uint32_t v = bits | 0x64006400u;
                const __half2 r = __hmul2(__hfma2(*reinterpret_cast<const __half2*>(&v), sixteenth, c72), s2);
                return *reinterpret_cast<const uint32_t*>(&r);
            };
            {
                const int bi = set;
                uint4 v = make_uint4(0x88888888u, 0x88888888u, 0x88888888u, 0x88888888u);      // q = 8: weight zero
                if (half == 0 || second_half) v = lds128(&sm.packed[slot][half * P_HALF_BYTES + (bi * 128 + hc) * kBlockBytes]);
                const uint32_t words[4] = {v.x, v.y, v.z, v.w};
                uint8_t* dst = &sm.bw[bs][(bi * 4) * (NT * 16) + col * 16];
#pragma unroll
                for (int w = 0; w < 4; ++w) {                               // word w = K core w of the block
                    const uint32_t x = words[w];
                    const uint32_t x8 = x >> 8;
                    uint4 o;
                    o.x = low(x & 0x000F000Fu);             // (k0, k4)
                    o.y = high(x & 0x00F000F0u);            // (k1, k5)
                    o.z = low(x8 & 0x000F000Fu);            // (k2, k6)
                    o.w = high(x8 & 0x00F000F0u);           // (k3, k7)
                    *reinterpret_cast<uint4*>(dst + w * (NT * 16)) = o;
                }
            }
            // written through the generic proxy, read by the tensor core through the async proxy
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) { mbar_arrive(&sm.b_full[bs]); mbar_arrive(&sm.p_empty[slot]); }
        }
        // ------------------------------------------------- read-back and store --
        // thread = activation row (its TMEM lane); warp w takes lanes 32 (w & 3) ... and columns 64 (w >> 2) ...
        constexpr int RCOLS = NT / (UNPACK_WARPS / 4);
        const int quarter = warp & 3, cpart = warp >> 2;
        ok = ok && tc::wait_uniform(&sm.d_full, 0, abort_flag);
        tc::tc_fence_after();
        pdl_wait_prior_grids();                                // C may be read (or, with the accumulate flag, was written) by a kernel before
        ok = ok && (*abort_flag == 0);
        const int nb = n0 + cpart * RCOLS;
#pragma unroll 1
        for (int rb = 0; rb < RB && ok; ++rb) {
            const int m = rb * MB + quarter * 32 + lane;
            const uint32_t lane_tmem = tmem_base + ((uint32_t)(quarter * 32) << 16) + rb * NT + cpart * RCOLS;
            const bool row_ok = m < p.M;
            const size_t row_off = (size_t)m * p.ldc + nb;
#pragma unroll 1
            for (int c0 = 0; c0 < RCOLS; c0 += 16) {
                uint32_t d[16];
                tc::tmem_ld<16>(lane_tmem + c0, d);
                tc::tmem_wait_ld();
                if (!row_ok || nb + c0 >= p.N) continue;
                const bool full = nb + c0 + 16 <= p.N;
                if (p.c_is_f16) {
                    __half* cp = reinterpret_cast<__half*>(p.c) + row_off + c0;
                    if (full && !p.accumulate && ((reinterpret_cast<uintptr_t>(cp) & 15) == 0)) {
#pragma unroll
                        for (int j = 0; j < 16; j += 8) {
                            const __half2 h0 = __floats2half2_rn(__uint_as_float(d[j]), __uint_as_float(d[j + 1]));
                            const __half2 h1 = __floats2half2_rn(__uint_as_float(d[j + 2]), __uint_as_float(d[j + 3]));
                            const __half2 h2 = __floats2half2_rn(__uint_as_float(d[j + 4]), __uint_as_float(d[j + 5]));
                            const __half2 h3 = __floats2half2_rn(__uint_as_float(d[j + 6]), __uint_as_float(d[j + 7]));
                            uint4 o;
                            o.x = *reinterpret_cast<const uint32_t*>(&h0); o.y = *reinterpret_cast<const uint32_t*>(&h1);
                            o.z = *reinterpret_cast<const uint32_t*>(&h2); o.w = *reinterpret_cast<const uint32_t*>(&h3);
                            *reinterpret_cast<uint4*>(cp + j) = o;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (nb + c0 + j < p.N) {
                                float vv = __uint_as_float(d[j]);
                                if (p.accumulate) vv += __half2float(cp[j]);
                                cp[j] = __float2half_rn(vv);
                            }
                        }
                    }
                } else {
                    float* cp = reinterpret_cast<float*>(p.c) + row_off + c0;
                    if (full && !p.accumulate && ((reinterpret_cast<uintptr_t>(cp) & 15) == 0)) {
#pragma unroll
                        for (int j = 0; j < 16; j += 4)
                            *reinterpret_cast<float4*>(cp + j) = make_float4(__uint_as_float(d[j]), __uint_as_float(d[j + 1]),
                                                                             __uint_as_float(d[j + 2]), __uint_as_float(d[j + 3]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            if (nb + c0 + j < p.N) {
                                float vv = __uint_as_float(d[j]);
                                if (p.accumulate) vv += cp[j];
                                cp[j] = vv;
                            }
                        }
                    }
                }
            }
        }
    }

    // ------------------------------------------------------------ teardown --
    tc::tc_fence_before();
    __syncthreads();
    if (warp == WARP_MMA) {
        tc::tc_fence_after();
        tc::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

}  // namespace tcr
}  // namespace twm
