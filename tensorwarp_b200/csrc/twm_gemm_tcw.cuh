// twm_gemm_tcw.cuh — the tcgen05 / TMEM W4A16 kernel for many activation rows (65 ... 128 per
// launch, scale group 128).
//
// twm_gemm_tc.cuh puts the CTA's 128 weight columns on the MMA's M dimension and the (few)
// activation rows on N = 16 ... 64: right while the weight stream is the bound, but an MMA of
// 128 x 16 x 16 costs the tensor core as many issue cycles as one of 128 x 128 x 16, so with many
// rows most of the tensor pipe idles.  Here the roles are the other way round: the 128
// activation rows are the MMA's M dimension (one TMEM lane per row), the CTA's 128 weight columns
// are N, and one tcgen05.mma does 128 x 128 x 16.  There is no counterpart in the reference: its
// only batched W4A16 kernel is a 32x32 SIMT tile kernel (crates/kernels/src/quantize.rs:186-246).
//
// Same result definition as every other kernel of the library: w = f32(scale) * (nibble - 8),
// exact products, FP32 accumulation, the scale applied in FP32 per 128-group.  The weight operand
// is never converted: `v & 0x000F000F` etc. leave each nibble as an FP16 subnormal, one FP16 add or
// fused multiply-add per pair makes it the signed weight (q - 8) * 2^-24, exactly (nine instructions
// per eight nibbles); the unpack warps write those bit patterns into shared memory as
// the MMA's B operand (K-major 8x16-byte core matrices, no swizzle).  The activations come from
// the same pre-pass as in twm_gemm_tc.cuh (K order k0,k4,k1,k5,...) and are the A operand, loaded
// by tiled TMA.  Every scale group accumulates into a fresh accumulator (two, used in turn); the
// read-back warps take a finished group out of tensor memory, multiply by their column's FP32
// scale and add into registers: thread = one activation row, 128 column sums.
//
// Warp roles: 0-7 read-back and store (TMEM lane quarter = warp & 3, column half = warp >> 2),
// 8-11 unpack (thread = column), 12 TMA producer, 13 MMA issuer.  One CTA per SM (about 195 KB of
// shared memory, all 512 TMEM columns: four accumulators).
#pragma once

#include "twm_common.cuh"
#include "twm_gemm_tc.cuh"

namespace twm {
namespace tcw {

constexpr int NT = 128;                 // weight columns per CTA = MMA N
constexpr int MB = 128;                 // activation rows per launch = MMA M (rows past M are zero)
constexpr int GROUP_BLOCKS = 4;         // 32-blocks per ring stage = one scale group of 128
constexpr int WSTAGES = 3;              // packed ring: 3 x 16 KB
constexpr int BSTAGES = 2;              // unpacked weights, one scale group (four 32-blocks) per stage: 2 x 32 KB
constexpr int ASTAGES = 3;              // activation stages, one scale group each: 3 x 32 KB
constexpr int SSTAGES = 8;              // scale rows (one per group, 256 B) stay until the read-back warps have used them
constexpr int ACCS = 4;                 // accumulators in tensor memory (128 columns each), used in turn
constexpr int A_KCORES = GROUP_BLOCKS * 4;              // 8-wide K cores per activation stage
constexpr int A_STAGE_BYTES = A_KCORES * MB * 16;       // [K core][row][16 bytes]
constexpr int B_BLOCK_BYTES = 4 * NT * 16;              // [K core of the block][column][16 bytes]
constexpr int B_STAGE_BYTES = GROUP_BLOCKS * B_BLOCK_BYTES;
constexpr int W_STAGE_BYTES = GROUP_BLOCKS * NT * kBlockBytes;
constexpr int EPI_WARPS = 8;            // read-back: warp w takes TMEM lane quarter w & 3, columns 64 * (w >> 2) ...
constexpr int EPI_THREADS = EPI_WARPS * 32;
constexpr int EPI_COLS = NT / (EPI_WARPS / 4);
constexpr int WARP_UNPACK0 = EPI_WARPS, UNPACK_WARPS = 4;
constexpr int WARP_TMA = WARP_UNPACK0 + UNPACK_WARPS, WARP_MMA = WARP_TMA + 1;
constexpr int THREADS = (WARP_MMA + 1) * 32;
constexpr int TMEM_COLS = ACCS * NT;    // 512: the whole tensor memory of the SM (one CTA per SM)

struct Smem {
    alignas(128) uint8_t packed[WSTAGES][W_STAGE_BYTES];
    alignas(128) uint8_t bw[BSTAGES][B_STAGE_BYTES];
    alignas(128) uint8_t a[ASTAGES][A_STAGE_BYTES];
    alignas(16) uint16_t sc[SSTAGES][NT];        // the group's scale row of this tile, arrives with the packed stage
    alignas(16) float scf[2][NT];                // the same as FP32, converted once per group by the read-back warps
    alignas(8) uint64_t s_empty[SSTAGES];        // read-back warps
    alignas(8) uint64_t w_full[WSTAGES];
    alignas(8) uint64_t w_empty[WSTAGES];        // unpack warps
    alignas(8) uint64_t b_full[BSTAGES];         // unpack warps
    alignas(8) uint64_t b_empty[BSTAGES];        // MMA commit
    alignas(8) uint64_t a_full[ASTAGES];
    alignas(8) uint64_t a_empty[ASTAGES];        // MMA commit
    alignas(8) uint64_t d_full[ACCS];            // MMA commit
    alignas(8) uint64_t d_empty[ACCS];           // read-back warps
    uint32_t tmem_base;
    int abort_flag;
    int is_last;
};

// D[128 x N] (+)= A[128 x 16] (shared memory) * B[N x 16]^T (shared memory)
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

__global__ void __launch_bounds__(THREADS, 1)
gemm_kernel(const __grid_constant__ GemmParams p)
{
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>(smem_raw);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int n0 = blockIdx.x * NT;
    const int b0 = blockIdx.y * p.blocks_per_split;          // a multiple of four (whole 128-groups, host plan)
    const int b1 = min(p.nkb, b0 + p.blocks_per_split);
    const int n_stages = (b1 - b0) / GROUP_BLOCKS;           // scale groups of this K slice

    if (tid == 0) {
        for (int s = 0; s < WSTAGES; ++s) { mbar_init(&sm.w_full[s], 1); mbar_init(&sm.w_empty[s], UNPACK_WARPS); }
        for (int s = 0; s < BSTAGES; ++s) { mbar_init(&sm.b_full[s], UNPACK_WARPS); mbar_init(&sm.b_empty[s], 1); }
        for (int s = 0; s < ASTAGES; ++s) { mbar_init(&sm.a_full[s], 1); mbar_init(&sm.a_empty[s], 1); }
        for (int s = 0; s < ACCS; ++s) { mbar_init(&sm.d_full[s], 1); mbar_init(&sm.d_empty[s], EPI_WARPS); }
        for (int s = 0; s < SSTAGES; ++s) mbar_init(&sm.s_empty[s], EPI_WARPS);
        sm.abort_flag = 0;
        sm.is_last = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    volatile int* abort_flag = &sm.abort_flag;

    // A whole tile inside N with 16-byte aligned scale rows: the group's 128 scales (256 bytes) ride along
    // with the packed stage as one bulk copy; a ragged last tile reads them from global memory instead.
    const bool scale_bulk = (n0 + NT <= p.N) && ((p.N & 7) == 0) && ((reinterpret_cast<uintptr_t>(p.scales) & 15) == 0);
    auto issue_w = [&](int st) {                             // lane 0 of the TMA warp
        const int slot = st % WSTAGES;
        mbar_arrive_expect_tx(&sm.w_full[slot], (uint32_t)W_STAGE_BYTES + (scale_bulk ? (uint32_t)NT * 2 : 0u));
        tma_load_2d(&sm.packed[slot][0], &p.packed_map, n0 * 2, b0 + st * GROUP_BLOCKS, &sm.w_full[slot]);
        if (scale_bulk)
            bulk_g2s(&sm.sc[st % SSTAGES][0], p.scales + (size_t)(b0 / GROUP_BLOCKS + st) * p.N + n0, (uint32_t)NT * 2,
                     &sm.w_full[slot]);
    };
    if (warp == WARP_TMA) {
        // weights are constants: the first ring-full streams before the preceding kernel has finished
        if (lane == 0)
            for (int st = 0; st < min(n_stages, WSTAGES); ++st) issue_w(st);
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
            int ast = 0, wst = min(n_stages, WSTAGES);
            uint32_t idle = 0;
            while ((ast < n_stages || wst < n_stages) && idle < (1u << 22)) {
                bool progress = false;
                if (ast < n_stages) {
                    const int as = ast % ASTAGES;
                    if (ast < ASTAGES || mbar_try_wait(&sm.a_empty[as], ((ast / ASTAGES) - 1) & 1)) {
                        mbar_arrive_expect_tx(&sm.a_full[as], (uint32_t)A_STAGE_BYTES);
                        tma_load_2d(&sm.a[as][0], &p.act_map, 0, (b0 + ast * GROUP_BLOCKS) * 4, &sm.a_full[as]);
                        ++ast; progress = true;
                    }
                }
                if (wst < n_stages) {
                    // the packed slot is free, and so is the scale row's slot (the read-back of eight groups ago is done)
                    if (mbar_try_wait(&sm.w_empty[wst % WSTAGES], ((wst / WSTAGES) - 1) & 1) &&
                        (wst < SSTAGES || mbar_try_wait(&sm.s_empty[wst % SSTAGES], ((wst / SSTAGES) - 1) & 1))) {
                        issue_w(wst); ++wst; progress = true;
                    }
                }
                if (progress) { idle = 0; } else { ++idle; if (idle > 64) __nanosleep(64); if (*abort_flag) break; }
            }
            if (ast < n_stages || wst < n_stages) { *abort_flag = 1; atomicOr(&g_error_word, 1u); }
        }
        __syncwarp();
    } else if (warp == WARP_MMA) {
        // -------------------------------------------------- MMA issuer (one thread) --
        if (lane == 0) {
            uint32_t idesc = 0;
            idesc |= 1u << 4;                          // D format f32 (A and B: f16, both K-major)
            idesc |= (uint32_t)(NT >> 3) << 17;        // N
            idesc |= (uint32_t)(MB >> 4) << 24;        // M
            for (int st = 0; st < n_stages; ++st) {
                const int as = st % ASTAGES, bs = st % BSTAGES, acc = st % ACCS;
                if (!mbar_wait_bounded(&sm.a_full[as], (st / ASTAGES) & 1, abort_flag)) break;
                if (st >= ACCS && !mbar_wait_bounded(&sm.d_empty[acc], ((st / ACCS) - 1) & 1, abort_flag)) break;
                if (!mbar_wait_bounded(&sm.b_full[bs], (st / BSTAGES) & 1, abort_flag)) break;
                tc::tc_fence_after();
                const uint32_t d_addr = tmem_base + acc * NT;
                // A: [K core][row][16 B]: next K core MB*16 bytes on, next 8 rows 128 bytes on.
                // B: [K core][column][16 B]: next K core NT*16 bytes on, next 8 columns 128 bytes on.
                uint64_t ad = tc::make_b_desc(smem_u32(&sm.a[as][0]), MB * 16, 128);
                uint64_t bd = tc::make_b_desc(smem_u32(&sm.bw[bs][0]), NT * 16, 128);
                constexpr uint64_t a_step = (uint64_t)((2 * MB * 16) >> 4), b_step = (uint64_t)((2 * NT * 16) >> 4);   // two K cores, in descriptor units
#pragma unroll
                for (int h = 0; h < 2 * GROUP_BLOCKS; ++h) {                // eight MMAs of K = 16: the group's 128 K
                    mma_ss(d_addr, ad, bd, idesc, h == 0 ? 0u : 1u);
                    ad += a_step;
                    bd += b_step;
                }
                tc::tc_commit(&sm.b_empty[bs]);                             // the unpacked stage is free once these have run
                tc::tc_commit(&sm.d_full[acc]);                             // the group's accumulator is complete
                tc::tc_commit(&sm.a_empty[as]);
            }
        }
        __syncwarp();
    } else if (warp >= WARP_UNPACK0) {
        // ------------------------------------------------------------------ unpack --
        const int col = (warp - WARP_UNPACK0) * 32 + lane;
        for (int st = 0; st < n_stages; ++st) {
            const int wslot = st % WSTAGES, bs = st % BSTAGES;
            if (!tc::wait_uniform(&sm.w_full[wslot], (st / WSTAGES) & 1, abort_flag)) break;
            if (st >= BSTAGES && !tc::wait_uniform(&sm.b_empty[bs], ((st / BSTAGES) - 1) & 1, abort_flag)) break;
#pragma unroll
            for (int bi = 0; bi < GROUP_BLOCKS; ++bi) {
                const uint4 v = lds128(&sm.packed[wslot][(bi * NT + col) * kBlockBytes]);
                const uint32_t words[4] = {v.x, v.y, v.z, v.w};
                uint8_t* dst = &sm.bw[bs][bi * B_BLOCK_BYTES + col * 16];
#pragma unroll
                for (int w = 0; w < 4; ++w) {                               // word w = K core w of the block
                    const uint32_t x = words[w];
                    const uint32_t x8 = x >> 8;
                    uint4 o;
                    o.x = tc::signed_low(x & 0x000F000Fu);           // (k0, k4): (n - 8) * 2^-24
                    o.y = tc::signed_high(x & 0x00F000F0u);          // (k1, k5)
                    o.z = tc::signed_low(x8 & 0x000F000Fu);          // (k2, k6)
                    o.w = tc::signed_high(x8 & 0x00F000F0u);         // (k3, k7)
                    *reinterpret_cast<uint4*>(dst + w * (NT * 16)) = o;
                }
            }
            // written through the generic proxy, read by the tensor core through the async proxy
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) { mbar_arrive(&sm.b_full[bs]); mbar_arrive(&sm.w_empty[wslot]); }
        }
    } else {
        // ------------------------------------------------- read-back and store --
        const int quarter = warp & 3, half = warp >> 2;
        const int m = quarter * 32 + lane;                   // this thread's activation row = its TMEM lane
        const int cbase = half * EPI_COLS;                   // its first column inside the tile
        const uint32_t lane_tmem = tmem_base + ((uint32_t)(quarter * 32) << 16) + cbase;
        pdl_wait_prior_grids();                              // C may be read by the kernel before
        float acc[EPI_COLS];
#pragma unroll
        for (int j = 0; j < EPI_COLS; ++j) acc[j] = 0.0f;
        const int grow0 = b0 / GROUP_BLOCKS;
        bool ok = true;
        for (int st = 0; st < n_stages; ++st) {
            const int db = st % ACCS, sb = st & 1;
            if (!tc::wait_uniform(&sm.d_full[db], (st / ACCS) & 1, abort_flag)) { ok = false; break; }
            tc::tc_fence_after();
            // Every thread needs its columns' scales as FP32: thread j < 128 converts scale j once (the
            // f16 -> f32 conversion unit is narrow), all read them back as broadcast 128-bit loads.  Two
            // buffers, used in turn: the barrier of the group in between keeps a writer behind every reader.
            if (tid < NT) {
                const int n = n0 + tid;
                uint16_t h = 0;
                if (scale_bulk) h = sm.sc[st % SSTAGES][tid];
                else if (n < p.N) h = __ldg(p.scales + (size_t)(grow0 + st) * p.N + n);
                sm.scf[sb][tid] = f16_bits_to_f32(h) * 16777216.0f;      // the operand's 2^-24 comes out here
            }
            named_bar_sync(2, EPI_THREADS);
            const float* scf = &sm.scf[sb][cbase];
#pragma unroll
            for (int c0 = 0; c0 < EPI_COLS; c0 += 16) {
                uint32_t d[16];
                tc::tmem_ld<16>(lane_tmem + db * NT + c0, d);
                float sc[16];
#pragma unroll
                for (int j = 0; j < 16; j += 4) {
                    const float4 t4 = *reinterpret_cast<const float4*>(scf + c0 + j);
                    sc[j] = t4.x; sc[j + 1] = t4.y; sc[j + 2] = t4.z; sc[j + 3] = t4.w;
                }
                tc::tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    acc[c0 + j] = fmaf(sc[j], __uint_as_float(d[j]), acc[c0 + j]);
            }
            tc::tc_fence_before();
            __syncwarp();
            if (lane == 0) { mbar_arrive(&sm.d_empty[db]); mbar_arrive(&sm.s_empty[st % SSTAGES]); }
        }
        ok = ok && (*abort_flag == 0);
        const bool row_ok = m < p.M;
        const int nb = n0 + cbase;                                        // this thread's first column
        // this thread's 64 results are one contiguous run of its C row: 16-byte stores where the row allows
        const size_t row_off = (size_t)m * p.ldc + nb;
        const bool full = nb + EPI_COLS <= p.N;
        if (ok && row_ok) {
            if (p.splits == 1) {
                if (p.c_is_f16) {
                    __half* cp = reinterpret_cast<__half*>(p.c) + row_off;
                    if (full && !p.accumulate && ((reinterpret_cast<uintptr_t>(cp) & 15) == 0)) {
#pragma unroll
                        for (int j = 0; j < EPI_COLS; j += 8) {
                            const __half2 h0 = __floats2half2_rn(acc[j], acc[j + 1]), h1 = __floats2half2_rn(acc[j + 2], acc[j + 3]);
                            const __half2 h2 = __floats2half2_rn(acc[j + 4], acc[j + 5]), h3 = __floats2half2_rn(acc[j + 6], acc[j + 7]);
                            uint4 o;
                            o.x = *reinterpret_cast<const uint32_t*>(&h0); o.y = *reinterpret_cast<const uint32_t*>(&h1);
                            o.z = *reinterpret_cast<const uint32_t*>(&h2); o.w = *reinterpret_cast<const uint32_t*>(&h3);
                            *reinterpret_cast<uint4*>(cp + j) = o;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < EPI_COLS; ++j) {
                            if (nb + j < p.N) {
                                float vv = acc[j];
                                if (p.accumulate) vv += __half2float(cp[j]);
                                cp[j] = __float2half_rn(vv);
                            }
                        }
                    }
                } else {
                    float* cp = reinterpret_cast<float*>(p.c) + row_off;
                    if (full && !p.accumulate && ((reinterpret_cast<uintptr_t>(cp) & 15) == 0)) {
#pragma unroll
                        for (int j = 0; j < EPI_COLS; j += 4)
                            *reinterpret_cast<float4*>(cp + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < EPI_COLS; ++j) {
                            if (nb + j < p.N) {
                                float vv = acc[j];
                                if (p.accumulate) vv += cp[j];
                                cp[j] = vv;
                            }
                        }
                    }
                }
            } else {
                // (N is a multiple of 4 whenever a tile is full, and the partials start 16-byte aligned)
                float* part = p.ws_partials + ((size_t)blockIdx.y * p.M + m) * p.N + nb;
                if (full && (p.N & 3) == 0) {
#pragma unroll
                    for (int j = 0; j < EPI_COLS; j += 4)
                        *reinterpret_cast<float4*>(part + j) = make_float4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
                } else {
#pragma unroll
                    for (int j = 0; j < EPI_COLS; ++j)
                        if (nb + j < p.N) part[j] = acc[j];
                }
            }
        }
        if (p.splits > 1) {
            __threadfence();
            named_bar_sync(3, EPI_THREADS);
            if (tid == 0) {
                const unsigned prev = atomicAdd(&p.ws_counters[blockIdx.x], 1u);
                sm.is_last = (prev == (unsigned)(p.splits - 1));
            }
            named_bar_sync(3, EPI_THREADS);
            if (sm.is_last) {
                __threadfence();
                // the last arriver adds the slices in slice order.  The tile is walked four columns per thread,
                // a warp along a row (coalesced), the slices' loads issued together
                if (*abort_flag == 0) {
                    const bool vec = (p.N & 3) == 0;
                    for (int idx = tid; idx < MB * (NT / 4); idx += EPI_THREADS) {
                        const int r = idx / (NT / 4), c = n0 + (idx % (NT / 4)) * 4;
                        if (r >= p.M || c >= p.N) continue;
                        float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                        if (vec) {
#pragma unroll 4
                            for (int sp = 0; sp < p.splits; ++sp) {
                                const float4 t4 = __ldcg(reinterpret_cast<const float4*>(&p.ws_partials[((size_t)sp * p.M + r) * p.N + c]));
                                v[0] += t4.x; v[1] += t4.y; v[2] += t4.z; v[3] += t4.w;
                            }
                        } else {
                            for (int sp = 0; sp < p.splits; ++sp)
                                for (int j = 0; j < 4; ++j)
                                    if (c + j < p.N) v[j] += ld_cg_f32(&p.ws_partials[((size_t)sp * p.M + r) * p.N + c + j]);
                        }
                        const size_t off = (size_t)r * p.ldc + c;
                        for (int j = 0; j < 4; ++j) {
                            if (c + j >= p.N) break;
                            if (p.c_is_f16) {
                                __half* cp = reinterpret_cast<__half*>(p.c);
                                float sv = v[j];
                                if (p.accumulate) sv += __half2float(cp[off + j]);
                                cp[off + j] = __float2half_rn(sv);
                            } else {
                                float* cp = reinterpret_cast<float*>(p.c);
                                float sv = v[j];
                                if (p.accumulate) sv += cp[off + j];
                                cp[off + j] = sv;
                            }
                        }
                    }
                }
                if (tid == 0) atomicExch(&p.ws_counters[blockIdx.x], 0u);
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

}  // namespace tcw
}  // namespace twm
