// twm_gemv_simt.cuh — the memory-bound W4A16 kernel for M <= 8.
//
// Replaces warp_gemm_tw_marlin_m1 / _m1_direct
// (crates/kernels/src/quantize.rs:1186-1298) and the launcher's split-K
// (quantize.rs:1314-1357).  Same result definition: for every column n,
//   C[m][n] = sum_g f32(scale[g][n]) * sum_j A[m][32g+j] * (nibble_j - 8),
// FP32 products and FP32 accumulation.
//
// Shape of the work.  A CTA owns 128 columns and a contiguous range of
// 32-blocks of K.  One producer warp streams the packed rows
// (`packed[g][n0..n0+128]` is one contiguous 2 KB run) and the scale rows into a
// five-deep shared-memory ring with 1-D bulk copies (TMA unit) tracked by
// mbarriers, eight 32-blocks per stage.  Eight consumer warps each take one
// block of a stage and all 128 columns of it, four columns per lane, so the
// 16-byte block of a column is one conflict-free 128-bit shared load.
//
// Nibble unpack without conversions.  A nibble left in place inside its u32,
// `v & (0xF << 4j)`, read as an FP32 bit pattern, is the number
// q * 2^(4j-149) exactly (FP32 subnormals and the first normal binade are one
// linear ramp below 2^24).  The activation that multiplies it is pre-scaled by
// the inverse power of two when it is staged into shared memory, so one AND
// and one FMA per weight give A*q exactly as the reference's
// shift-mask-convert does; the "-8" of every nibble is folded into one term
// -8 * sum(A over the block), computed once per block with a warp shuffle
// reduction.  Nibbles 6 and 7 of a word reach into the exponent field, so
// they are taken from `v >> 8`.
//
// Split-K.  Slices write FP32 partials to the caller's workspace; the CTA that
// arrives last on the tile's counter adds the slices in slice order (so the
// result does not depend on arrival order), stores C and puts the counter back
// to zero.  No memset launch, no atomics on C.
//
// Programmatic dependent launch.  The producer starts streaming weights before
// the preceding kernel in the stream has finished (weights are constants);
// activations, workspace and C are only touched after griddepcontrol.wait.
#pragma once

#include "twm_common.cuh"

namespace twm {
namespace simt {

constexpr int NT = 128;          // columns per CTA
constexpr int SB = 8;            // 32-blocks per stage = consumer warps
constexpr int STAGES = 5;
constexpr int CONSUMERS = SB * 32;
constexpr int THREADS = CONSUMERS + 32;
constexpr int ACAP = 4096;       // staged activations (floats) per chunk, all rows together
constexpr int PRESCALE_EXP = 88; // activations are staged as a * 2^(88 - bit position)

constexpr int STAGE_PACKED_BYTES = SB * NT * kBlockBytes;  // 16 KB
constexpr int STAGE_SCALE_BYTES = SB * NT * 2;             // 2 KB (8 rows at G=32; 3 used at G=128)

struct Smem {
    alignas(128) uint8_t packed[STAGES][STAGE_PACKED_BYTES];
    alignas(128) uint16_t scales[STAGES][SB][NT];
    alignas(16) float a[ACAP];
    float asum8[ACAP / kBlockK];   // -8 * sum of the raw activations of a block
    alignas(8) uint64_t full[STAGES];
    alignas(8) uint64_t empty[STAGES];
    int abort_flag;
    int is_last;
};

__device__ __forceinline__ float as_f32(uint32_t u) { return __uint_as_float(u); }

template <int MMAX>
__global__ void __launch_bounds__(THREADS, (MMAX <= 4) ? 2 : 1)
gemv_kernel(const GemmParams p)
{
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
    const int n_stages = (total_blocks + SB - 1) / SB;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], SB);
        }
        sm.abort_flag = 0;
        sm.is_last = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    volatile int* abort_flag = &sm.abort_flag;

    if (warp == SB) {
        // ------------------------------------------------------- producer --
        const uint8_t* packed = p.packed;
        const uint16_t* scales = p.scales;
        if (p.packed_offsets != nullptr) {
            // the offset table may come from the kernel before this one
            pdl_wait_prior_grids();
            packed += p.packed_offsets[p.expert_idx];
            scales += p.scales_offsets[p.expert_idx];
        }
        const bool scale_bulk_ok = ((cols & 7) == 0) && ((p.N & 7) == 0) &&
                                   ((reinterpret_cast<uintptr_t>(scales + n0) & 15) == 0);
        for (int it = 0; it < n_stages; ++it) {
            const int slot = it % STAGES;
            const int use = it / STAGES;
            if (use > 0) {
                const bool got = mbar_wait_bounded(&sm.empty[slot], (use - 1) & 1, abort_flag);
                if (!__all_sync(0xffffffffu, got)) break;   // same decision in every lane
            }
            const int bstart = b0 + it * SB;
            const int nb = min(SB, b1 - bstart);
            const int srow_first = (bstart * kBlockK) / p.group;
            const int srow_last = ((bstart + nb - 1) * kBlockK) / p.group;
            const int nrows = srow_last - srow_first + 1;
            uint32_t tx = (uint32_t)nb * cols * kBlockBytes;
            if (scale_bulk_ok) {
                tx += (uint32_t)nrows * cols * 2;
            } else {
                // ragged or unaligned scale rows: plain loads by the whole warp
                for (int r = 0; r < nrows; ++r) {
                    const uint16_t* src = scales + (size_t)(srow_first + r) * p.N + n0;
                    for (int cidx = lane; cidx < cols; cidx += 32) sm.scales[slot][r][cidx] = src[cidx];
                }
                __syncwarp();
            }
            if (lane == 0) {
                mbar_arrive_expect_tx(&sm.full[slot], tx);
                for (int r = 0; r < nb; ++r) {
                    bulk_g2s(&sm.packed[slot][r * NT * kBlockBytes],
                             packed + ((size_t)(bstart + r) * p.N + n0) * kBlockBytes,
                             (uint32_t)cols * kBlockBytes, &sm.full[slot]);
                }
                if (scale_bulk_ok) {
                    for (int r = 0; r < nrows; ++r) {
                        bulk_g2s(&sm.scales[slot][r][0], scales + (size_t)(srow_first + r) * p.N + n0,
                                 (uint32_t)cols * 2, &sm.full[slot]);
                    }
                }
            }
            __syncwarp();
        }
        return;
    }

    // ---------------------------------------------------------- consumers --
    pdl_wait_prior_grids();

    float acc[4][MMAX];
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int m = 0; m < MMAX; ++m) acc[c][m] = 0.0f;

    constexpr int CHUNK_BLOCKS = ACAP / (kBlockK * MMAX);  // multiple of SB
    static_assert(CHUNK_BLOCKS % SB == 0, "chunk must hold whole stages");
    bool ok = true;

    // After an expired wait (`ok` false) every warp still walks the same barrier
    // sequence, without computing, so that no named barrier is left short.
    for (int chunk0 = 0; chunk0 < total_blocks; chunk0 += CHUNK_BLOCKS) {
        const int cb = min(CHUNK_BLOCKS, total_blocks - chunk0);
        const int chunk_k = cb * kBlockK;
        if (chunk0 > 0) named_bar_sync(1, CONSUMERS);  // previous chunk fully consumed
        // Stage activations: a'[m][k] = a[m][k] * 2^(PRESCALE_EXP - bitpos(k % 8)).
        {
            const size_t kbase = (size_t)(b0 + chunk0) * kBlockK;
            const int limit = MMAX * chunk_k;
            for (int idx = tid; idx < limit; idx += CONSUMERS) {
                const int m = idx / chunk_k;
                const int kk = idx - m * chunk_k;
                float v = 0.0f;
                if (m < p.M) {
                    const size_t off = (size_t)m * p.lda + kbase + kk;
                    v = p.a_is_f16 ? __half2float(reinterpret_cast<const __half*>(p.a)[off])
                                   : reinterpret_cast<const float*>(p.a)[off];
                }
                const int j = kk & 7;
                const int bitpos = (j < 6) ? 4 * j : 4 * j - 8;
                sm.a[idx] = v * as_f32((uint32_t)(127 + PRESCALE_EXP - bitpos) << 23);
                float s = v;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (lane == 0) sm.asum8[idx >> 5] = -8.0f * s;
            }
        }
        named_bar_sync(1, CONSUMERS);

        const int it_begin = chunk0 / SB;
        const int it_end = (chunk0 + cb + SB - 1) / SB;
        for (int it = it_begin; it < it_end; ++it) {
            const int slot = it % STAGES;
            if (!ok) continue;
            const bool got = mbar_wait_bounded(&sm.full[slot], (it / STAGES) & 1, abort_flag);
            if (!__all_sync(0xffffffffu, got)) { ok = false; continue; }   // same decision in every lane
            const int bstart = b0 + it * SB;
            const int nb = min(SB, b1 - bstart);
            if (warp < nb) {
                const int b = bstart + warp;
                const int srow = (b * kBlockK) / p.group - (bstart * kBlockK) / p.group;
                const int blk_local = (b - b0) - chunk0;       // block index inside the chunk
                uint4 w[4];
                float sc[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int col = c * 32 + lane;
                    w[c] = lds128(&sm.packed[slot][(warp * NT + col) * kBlockBytes]);
                    sc[c] = f16_bits_to_f32(sm.scales[slot][srow][col]);
                }
                float gd[4][MMAX];
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int m = 0; m < MMAX; ++m) gd[c][m] = 0.0f;

#pragma unroll
                for (int word = 0; word < 4; ++word) {
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        float4 av[MMAX];
#pragma unroll
                        for (int m = 0; m < MMAX; ++m) {
                            const uint4 t = lds128(&sm.a[m * chunk_k + blk_local * kBlockK + word * 8 + half * 4]);
                            av[m] = make_float4(as_f32(t.x), as_f32(t.y), as_f32(t.z), as_f32(t.w));
                        }
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const uint32_t v = (word == 0) ? w[c].x : (word == 1) ? w[c].y
                                             : (word == 2) ? w[c].z : w[c].w;
                            uint32_t t0, t1, t2, t3;
                            if (half == 0) {
                                t0 = v & 0x0000000Fu; t1 = v & 0x000000F0u;
                                t2 = v & 0x00000F00u; t3 = v & 0x0000F000u;
                            } else {
                                const uint32_t v8 = v >> 8;
                                t0 = v & 0x000F0000u; t1 = v & 0x00F00000u;
                                t2 = v8 & 0x000F0000u; t3 = v8 & 0x00F00000u;
                            }
#pragma unroll
                            for (int m = 0; m < MMAX; ++m) {
                                gd[c][m] = fmaf(av[m].x, as_f32(t0), gd[c][m]);
                                gd[c][m] = fmaf(av[m].y, as_f32(t1), gd[c][m]);
                                gd[c][m] = fmaf(av[m].z, as_f32(t2), gd[c][m]);
                                gd[c][m] = fmaf(av[m].w, as_f32(t3), gd[c][m]);
                            }
                        }
                    }
                }
                // undo the pre-scale (2^(149-88) = 2^61), fold in -8*sum(a), apply the group scale
                const float unscale = as_f32((uint32_t)(127 + 149 - PRESCALE_EXP) << 23);
#pragma unroll
                for (int m = 0; m < MMAX; ++m) {
                    const float a8 = sm.asum8[m * cb + blk_local];
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        acc[c][m] = fmaf(fmaf(gd[c][m], unscale, a8), sc[c], acc[c][m]);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.empty[slot]);
        }
    }

    // ------------------------------------------- reduce the eight warps --
    named_bar_sync(1, CONSUMERS);
    if (*abort_flag) return;   // a wait expired: leave C untouched, the error word is set
    float* red = reinterpret_cast<float*>(&sm.packed[0][0]);   // [SB][MMAX][NT], ring is idle now
#pragma unroll
    for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int m = 0; m < MMAX; ++m) red[(warp * MMAX + m) * NT + c * 32 + lane] = acc[c][m];
    named_bar_sync(1, CONSUMERS);

    const int n = n0 + tid;
    const bool owner = (tid < NT) && (n < p.N);
    float part[MMAX];
    if (owner) {
#pragma unroll
        for (int m = 0; m < MMAX; ++m) {
            float s = 0.0f;
#pragma unroll
            for (int w8 = 0; w8 < SB; ++w8) s += red[(w8 * MMAX + m) * NT + tid];
            part[m] = s;
        }
    }

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

    if (p.splits == 1) {
        if (owner) {
#pragma unroll
            for (int m = 0; m < MMAX; ++m)
                if (m < p.M) store_c(m, part[m]);
        }
        return;
    }

    // --------------------------------------------------- split-K finish --
    if (owner) {
#pragma unroll
        for (int m = 0; m < MMAX; ++m)
            if (m < p.M) p.ws_partials[((size_t)blockIdx.y * p.M + m) * p.N + n] = part[m];
    }
    __threadfence();
    named_bar_sync(1, CONSUMERS);
    if (tid == 0) {
        const unsigned prev = atomicAdd(&p.ws_counters[blockIdx.x], 1u);
        sm.is_last = (prev == (unsigned)(p.splits - 1));
    }
    named_bar_sync(1, CONSUMERS);
    if (!sm.is_last) return;
    __threadfence();
    if (owner) {
#pragma unroll
        for (int m = 0; m < MMAX; ++m) {
            if (m < p.M) {
                float s = 0.0f;
                for (int sp = 0; sp < p.splits; ++sp)
                    s += ld_cg_f32(&p.ws_partials[((size_t)sp * p.M + m) * p.N + n]);
                store_c(m, s);
            }
        }
    }
    if (tid == 0) atomicExch(&p.ws_counters[blockIdx.x], 0u);
}

}  // namespace simt
}  // namespace twm
