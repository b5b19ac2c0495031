// twm_gemv_strip.cuh — the memory-bound W4A16 kernel for M <= 8, FP16 activations, laid out so
// that consecutive GEMMs of a decode step overlap on the GPU.
//
// Replaces warp_gemm_tw_marlin_m1 / _m1_direct (crates/kernels/src/quantize.rs:1186-1298) and the
// launcher's split-K (quantize.rs:1314-1357).  Same result definition: w = f32(scale)*(nibble-8),
// exact products, FP32 accumulation, the scale applied in FP32 per group.
//
// Why another shape of the same arithmetic.  A decode step is a chain of dependent GEMMs, each a
// few microseconds of weight streaming.  A kernel that fills every CTA slot of every SM leaves
// HBM idle while it ramps up, reduces its K slices and drains, and the next one cannot start
// before it has gone.  Here one launch takes at most ONE CTA per SM and at most half of an SM's
// shared memory, registers and threads, so the next GEMM of the chain (launched programmatically
// early) is resident beside it and fills its own ring with weights while this one computes; when
// its activations arrive the first 64-96 KB per SM are already on chip.
//
// Shape of the work.  A CTA owns strips of 32 columns over the WHOLE K range, one after another
// (strip = blockIdx.x, + gridDim.x, ...), so there is no reduction between CTAs, no workspace
// and no cluster.  Inside the CTA the eight consumer warps are 2 column units (16 columns, the
// MMA's M) x 4 K phases: of each ring stage (32 K-blocks x 32 columns, one tiled TMA load of
// 16 KB plus one of the scale rows) a warp takes 8 consecutive K-blocks of its unit.  At the end
// of a strip the four K phases add up through shared memory in phase order (fixed, so the result
// does not depend on timing).  The ring runs on across strips.  The activations (all rows, whole
// K) are put into shared memory ONCE per CTA, in MMA fragment order with the per-group sums that
// fold the "-8", by the consumer warps together; shapes whose activations do not fit run on the
// split-K kernel instead.  Unpack and MMA are those of twm_gemv_mma.cuh (FP16 subnormal
// operands, five integer instructions per eight nibbles).
//
// Measured on B200 (7B decode shapes, M = 1, CUDA graph, programmatic dependent launch): the
// overlap works as designed (the next kernel's CTAs are resident and loaded when its activations
// arrive) but one CTA per SM unpacks only about 30 GB/s per SM, because the integer unpack plus
// warp-level MMA mix saturates at roughly the HBM rate when the WHOLE SM works on it; the layer
// chain takes 52.9 us against 38.2 us for the split-K kernel, whose two CTAs per SM are both
// active.  The heuristic therefore never picks this kernel; it runs when named
// (TWM_KERNEL_STRIP), needs no workspace for any M <= 8, and is the one to revisit if the
// unpack gets cheaper.
#pragma once

#include "twm_common.cuh"
#include "twm_gemv_mma.cuh"

namespace twm {
namespace strip {

constexpr int NT = 32;                        // columns per strip
constexpr int UNITS = NT / 16;                // 16-column MMA units per strip
constexpr int KPH = 4;                        // K phases (warps per unit)
constexpr int WB = 32 / KPH;                  // K-blocks per warp per stage
constexpr int SBLK = KPH * WB;                // K-blocks per ring stage
constexpr int CONSUMER_WARPS = UNITS * KPH;
constexpr int CONSUMERS = CONSUMER_WARPS * 32;
constexpr int THREADS = CONSUMERS + 32;       // + producer warp
constexpr int STAGE_BYTES = SBLK * NT * kBlockBytes;      // 16 KB
constexpr int SMEM_BUDGET = 112 * 1024;       // two CTAs per SM
constexpr int MAX_STAGES = 6;
constexpr int RED_BUFS = 4;                   // strips whose K-phase partials can be pending at once
constexpr int MIN_STAGES = 3;

// Dynamic shared memory, carved identically by the host (size, eligibility) and the kernel.
struct Layout {
    uint32_t packed, scales, afrag, asum, red, bars, total;
    int stages;
};
__host__ __device__ inline int asum_floats(int mp) { return mp < 2 ? 2 : mp; }
__host__ __device__ inline Layout make_layout(int nkb, int group, int mp, int stages)
{
    const int srows = SBLK / (group / 32);
    Layout l;
    l.stages = stages;
    l.packed = 0;
    l.scales = l.packed + (uint32_t)stages * STAGE_BYTES;
    l.afrag = l.scales + (uint32_t)stages * srows * NT * 2;
    l.asum = l.afrag + (((uint32_t)nkb * 64 * mp + 127) & ~127u);
    l.red = l.asum + (((uint32_t)(nkb / (group / 32)) * asum_floats(mp) * 4 + 127) & ~127u);
    l.bars = l.red + (uint32_t)RED_BUFS * KPH * mp * NT * 4;
    l.total = l.bars + 2u * MAX_STAGES * 8 + 16 + RED_BUFS * 4;
    return l;
}
// the deepest ring that fits beside the activations; 0 = this shape does not fit
__host__ inline int pick_stages(int nkb, int group, int mp)
{
    for (int st = MAX_STAGES; st >= MIN_STAGES; --st)
        if (make_layout(nkb, group, mp, st).total <= (uint32_t)SMEM_BUDGET) return st;
    return 0;
}

using mma::lds128_at;
using mma::lds16_at;
using mma::lds32_at;
using mma::lds64f_at;
using mma::mma_m16n8k16;

// MP = activation rows staged (power of two >= M, <= 8); GSHIFT = log2(32-blocks per scale group)
template <int MP, int GSHIFT>
__global__ void __launch_bounds__(THREADS, 2)
gemv_kernel(const __grid_constant__ GemmParams p)
{
    constexpr int GB = 1 << GSHIFT;
    constexpr int gmask = GB - 1;
    constexpr int SROWS = SBLK >> GSHIFT;                        // scale rows per stage
    constexpr int MPA = MP < 2 ? 2 : MP;                         // floats per group in the -8*sum table
    extern __shared__ __align__(128) uint8_t smem_raw[];
    const int STAGES = p.strip_stages;
    const Layout L = make_layout(p.nkb, p.group, MP, STAGES);
    uint64_t* full = reinterpret_cast<uint64_t*>(smem_raw + L.bars);
    uint64_t* empty = full + MAX_STAGES;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_raw + L.bars + 2 * MAX_STAGES * 8);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    TL_MARK(p.launch_id, 0);
    const int n_strips = (p.N + NT - 1) / NT;
    const int stages_per_strip = (p.nkb + SBLK - 1) / SBLK;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], CONSUMER_WARPS); }
        *abort_flag = 0;
        for (int i = 0; i < RED_BUFS; ++i)
            reinterpret_cast<volatile unsigned int*>(smem_raw + L.bars + 2 * MAX_STAGES * 8 + 16)[i] = 0u;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();

    if (warp == CONSUMER_WARPS) {
        // ------------------------------------------- producer: packed + scales --
        // Weights do not depend on the kernels before: the ring fills at once.
        int slot = 0;
        uint32_t use = 0;                 // how many times the ring has wrapped
        bool ok = true;
        for (int strip = blockIdx.x; strip < n_strips && ok; strip += gridDim.x) {
            const int n0 = strip * NT;
            for (int it = 0; it < stages_per_strip; ++it) {
                if (use > 0) {
                    const bool got = mbar_wait_bounded(&empty[slot], (use - 1) & 1, abort_flag);
                    if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
                }
                if (lane == 0) {
                    // rows past K and columns past N are zero-filled and still counted
                    mbar_arrive_expect_tx(&full[slot], (uint32_t)STAGE_BYTES + (uint32_t)SROWS * NT * 2);
                    tma_load_2d(smem_raw + L.packed + slot * STAGE_BYTES, &p.packed_map, n0 * 2, it * SBLK, &full[slot]);
                    tma_load_2d(smem_raw + L.scales + slot * (SROWS * NT * 2), &p.scale_map, n0, (it * SBLK) >> GSHIFT,
                                &full[slot]);
                }
                __syncwarp();
                if (++slot == STAGES) { slot = 0; ++use; }
            }
        }
        return;
    }

    // -------------------------------------------------------------- consumers --
    const int g = lane >> 2;
    const int t = lane & 3;
    const int unit = warp & (UNITS - 1);
    const int ph = warp / UNITS;

    // ---- activations, once: after the kernels before have completed ----
    // One item = 8 consecutive K of one row, stored as the 16 bytes
    // {k0,k4 | k2,k6 | k1,k5 | k3,k7}: the B fragments of the block's two MMAs.  Items are
    // numbered so that the 4 << GSHIFT lanes that hold one (scale group, row) are consecutive:
    // the group's sum of activations is a fixed-order warp-shuffle reduction.
    pdl_wait_prior_grids();
    TL_MARK(p.launch_id, 4);
    {
        const __half* A = reinterpret_cast<const __half*>(p.a);
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(A) & 15) == 0) && ((p.lda & 7) == 0);
        constexpr int PF = 10;                                // K = 18944 at one row: a single pass
        const int items = p.nkb * MP * 4;                     // item = (((gi * MP) + m) << GSHIFT | bj) * 4 + t
        uint8_t* afrag = smem_raw + L.afrag;
        float* asum = reinterpret_cast<float*>(smem_raw + L.asum);
        for (int base = 0; base < items; base += CONSUMERS * PF) {
            uint4 x[PF];
#pragma unroll
            for (int u = 0; u < PF; ++u) {
                const int it = base + u * CONSUMERS + tid;
                x[u] = make_uint4(0, 0, 0, 0);
                if (it < items) {
                    const int tt = it & 3;
                    const int bj = (it >> 2) & gmask;
                    const int rest = it >> (2 + GSHIFT);
                    const int m = rest % MP;
                    const int bi = ((rest / MP) << GSHIFT) + bj;
                    if (m < p.M) {
                        const size_t off = (size_t)m * p.lda + (size_t)bi * kBlockK + tt * 8;
                        if (vec_ok) {
                            x[u] = *reinterpret_cast<const uint4*>(A + off);
                        } else {
                            const uint16_t* a16 = reinterpret_cast<const uint16_t*>(A) + off;
                            x[u].x = a16[0] | ((uint32_t)a16[1] << 16); x[u].y = a16[2] | ((uint32_t)a16[3] << 16);
                            x[u].z = a16[4] | ((uint32_t)a16[5] << 16); x[u].w = a16[6] | ((uint32_t)a16[7] << 16);
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < PF; ++u) {
                const int it = base + u * CONSUMERS + tid;
                if (base + u * CONSUMERS + warp * 32 >= items) break;      // nothing left for this warp (warp-uniform)
                const int tt = it & 3;
                const int bj = (it >> 2) & gmask;
                const int rest = it >> (2 + GSHIFT);
                const int m = rest % MP;
                const int gi = rest / MP;
                float s = 0.0f;
                if (it < items) {
                    const int bi = (gi << GSHIFT) + bj;
                    uint4 o;
                    o.x = __byte_perm(x[u].x, x[u].z, 0x5410); o.y = __byte_perm(x[u].y, x[u].w, 0x5410);
                    o.z = __byte_perm(x[u].x, x[u].z, 0x7632); o.w = __byte_perm(x[u].y, x[u].w, 0x7632);
                    *reinterpret_cast<uint4*>(afrag + ((bi * MP + m) * 4 + tt) * 16) = o;
                    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&x[u].x));
                    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&x[u].y));
                    const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&x[u].z));
                    const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&x[u].w));
                    s = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
                }
                s += __shfl_xor_sync(0xffffffffu, s, 1);
                s += __shfl_xor_sync(0xffffffffu, s, 2);
                if (GSHIFT != 0) {                              // four blocks of a 128-group
                    s += __shfl_xor_sync(0xffffffffu, s, 4);
                    s += __shfl_xor_sync(0xffffffffu, s, 8);
                }
                if (it < items && (it & ((4 << GSHIFT) - 1)) == 0) asum[gi * MPA + m] = -8.0f * s;
            }
        }
        if (MP == 1) {      // row 1 of the table is read (and its result dropped): keep it finite
            const int ngroups = p.nkb >> GSHIFT;
            for (int gi = tid; gi < ngroups; gi += CONSUMERS) asum[gi * MPA + 1] = 0.0f;
        }
    }
    named_bar_sync(2, CONSUMERS);

    if (warp == 0) { TL_MARK(p.launch_id, 1); }
    const float zero4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const uint32_t w_base = smem_u32(smem_raw + L.packed) + ((ph * WB) * NT + unit * 16) * kBlockBytes + lane * 4;
    const uint32_t s_base = smem_u32(smem_raw + L.scales) + ((((ph * WB) >> GSHIFT) * NT) + unit * 16 + g) * 2;
    // lanes whose activation row does not exist (g >= MP) read row 0: their MMA output columns are never stored
    const uint32_t b_base = smem_u32(smem_raw + L.afrag) + (((g < MP) ? g : 0) * 4 + t) * 16 + (ph * WB) * (MP * 64);
    // rows 2t, 2t+1 of the group's -8*sum; lanes whose rows do not exist read rows 0, 1
    const uint32_t a8_base = smem_u32(smem_raw + L.asum) + ((2 * t + 1 < MPA) ? t * 8 : 0) + ((ph * WB) >> GSHIFT) * (MPA * 4);
    float* red = reinterpret_cast<float*>(smem_raw + L.red);       // [RED_BUFS][KPH][MP][NT]
    volatile unsigned int* red_cnt = reinterpret_cast<volatile unsigned int*>(smem_raw + L.bars + 2 * MAX_STAGES * 8 + 16);
    // tensor-parallel push: this launch's sequence number and buffer set (stable for the whole
    // launch: only the consumer kernel that follows advances it)
    const unsigned int comm_seq = p.n_peers ? ld_volatile_u32(p.comm_state) : 0u;
    bool ok = true;
    int sidx = 0;

    // One scale group of this warp's blocks: GB blocks x 16 columns, two MMA accumulator chains,
    // then value = 2^24*lo + 2^20*hi - 8*sum(a), times the FP32 scale.
    auto do_group = [&](float (&tot)[4], int r0, uint32_t w_st, uint32_t s_st, uint32_t b_st, uint32_t a8_st) {
        float lo[4], hi[4];
#pragma unroll
        for (int j = 0; j < GB; ++j) {
            const int r = r0 + j;
            const uint32_t v0 = lds32_at(w_st + r * (NT * kBlockBytes));          // column g, word t
            const uint32_t v1 = lds32_at(w_st + r * (NT * kBlockBytes) + 128);    // column g + 8, word t
            const uint4 xb = lds128_at(b_st + r * (MP * 64));
            const uint32_t v0s = v0 >> 8, v1s = v1 >> 8;
            // lo: nibbles (0,4),(2,6) scaled 2^-24 ; hi: nibbles (1,5),(3,7) scaled 2^-20
            if (j == 0) {
                mma_m16n8k16(lo, v0 & 0x000F000Fu, v1 & 0x000F000Fu, v0s & 0x000F000Fu, v1s & 0x000F000Fu, xb.x, xb.y, zero4);
                mma_m16n8k16(hi, v0 & 0x00F000F0u, v1 & 0x00F000F0u, v0s & 0x00F000F0u, v1s & 0x00F000F0u, xb.z, xb.w, zero4);
            } else {
                mma_m16n8k16(lo, v0 & 0x000F000Fu, v1 & 0x000F000Fu, v0s & 0x000F000Fu, v1s & 0x000F000Fu, xb.x, xb.y, lo);
                mma_m16n8k16(hi, v0 & 0x00F000F0u, v1 & 0x00F000F0u, v0s & 0x00F000F0u, v1s & 0x00F000F0u, xb.z, xb.w, hi);
            }
        }
        const float s0 = f16_bits_to_f32(lds16_at(s_st + (r0 >> GSHIFT) * (NT * 2)));
        const float s1 = f16_bits_to_f32(lds16_at(s_st + (r0 >> GSHIFT) * (NT * 2) + 16));
        const float2 a8 = lds64f_at(a8_st + (r0 >> GSHIFT) * (MPA * 4));
        const float k20 = 1048576.0f;                     // 2^20
        tot[0] = fmaf(s0, fmaf(fmaf(lo[0], 16.0f, hi[0]), k20, a8.x), tot[0]);
        tot[1] = fmaf(s0, fmaf(fmaf(lo[1], 16.0f, hi[1]), k20, a8.y), tot[1]);
        tot[2] = fmaf(s1, fmaf(fmaf(lo[2], 16.0f, hi[2]), k20, a8.x), tot[2]);
        tot[3] = fmaf(s1, fmaf(fmaf(lo[3], 16.0f, hi[3]), k20, a8.y), tot[3]);
    };

    int slot = 0;
    uint32_t ring_phase = 0;
    for (int strip = blockIdx.x; strip < n_strips; strip += gridDim.x, ++sidx) {
        const int n0 = strip * NT;
        float tot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int it = 0; it < stages_per_strip; ++it) {
            const int nb = min(SBLK, p.nkb - it * SBLK);
            if (ok) {
                const bool got = mbar_wait_bounded(&full[slot], ring_phase, abort_flag);
                if (!__all_sync(0xffffffffu, got)) ok = false;
            }
            if (ok) {
                const uint32_t w_st = w_base + slot * STAGE_BYTES;
                const uint32_t s_st = s_base + slot * (SROWS * NT * 2);
                const uint32_t b_st = b_base + (it * SBLK) * (MP * 64);
                const uint32_t a8_st = a8_base + ((it * SBLK) >> GSHIFT) * (MPA * 4);
                if (nb == SBLK) {
                    // the usual case, branch-free: the groups' MMA chains interleave
#pragma unroll
                    for (int r0 = 0; r0 < WB; r0 += GB) do_group(tot, r0, w_st, s_st, b_st, a8_st);
                } else {
                    // last stage of a strip when K is not a multiple of the stage: its whole groups
                    // are dealt evenly to the K phases, so that no warp idles through it
                    const int wb = ((((nb >> GSHIFT) + KPH - 1) / KPH) << GSHIFT);
                    const int first = ph * wb;
                    const int nbw = min(nb - first, wb);                   // may be <= 0
                    const int db = first - ph * WB;                        // blocks from the usual first block
                    const int dg = (first >> GSHIFT) - ((ph * WB) >> GSHIFT);
                    const uint32_t w2 = w_st + db * (NT * kBlockBytes), s2 = s_st + dg * (NT * 2);
                    const uint32_t b2 = b_st + db * (MP * 64), a82 = a8_st + dg * (MPA * 4);
#pragma unroll
                    for (int r0 = 0; r0 < WB; r0 += GB)
                        if (r0 < nbw) do_group(tot, r0, w2, s2, b2, a82);
                }
            }
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(&empty[slot]);
            if (++slot == STAGES) { slot = 0; ring_phase ^= 1u; }
        }
        TL_MARK(p.launch_id, 2);

        // ---- strip done.  No barrier: every warp leaves its partial in one of RED_BUFS buffers
        // and goes on; the warp that arrives last adds the K phases in phase order (the same
        // bits whoever is last) and stores the 32 columns.  A buffer's counter runs through
        // CONSUMER_WARPS arrivals and one release per use; a warp about to reuse a buffer waits
        // (bounded) for the release of its previous use.
        if (ok) {
            const int rbuf = sidx & (RED_BUFS - 1);
            const unsigned int base_cnt = (unsigned int)(sidx / RED_BUFS) * (CONSUMER_WARPS + 1);
            volatile unsigned int* cnt = red_cnt + rbuf;
            float* rb = red + rbuf * (KPH * MP * NT);
            {
                bool free_now = false;
                for (unsigned int i = 0; i < (1u << 22) && !free_now; ++i) {
                    free_now = *cnt >= base_cnt;
                    if (!free_now && i > 64) { __nanosleep(64); if (*abort_flag) break; }
                }
                if (!free_now) { *abort_flag = 1; atomicOr(&g_error_word, 1u); ok = false; }
            }
            if (ok) {
                // lane (g, t) holds C[m = 2t, 2t+1][column unit*16 + g] and the same rows for column + 8
                const int cA = unit * 16 + g, cB = cA + 8;
                if (2 * t < MP) { rb[(ph * MP + 2 * t) * NT + cA] = tot[0]; rb[(ph * MP + 2 * t) * NT + cB] = tot[2]; }
                if (2 * t + 1 < MP) { rb[(ph * MP + 2 * t + 1) * NT + cA] = tot[1]; rb[(ph * MP + 2 * t + 1) * NT + cB] = tot[3]; }
                __syncwarp();
                unsigned int old = 0;
                if (lane == 0) { __threadfence_block(); old = atomicAdd(const_cast<unsigned int*>(cnt), 1u); }
                old = __shfl_sync(0xffffffffu, old, 0);
                if (old == base_cnt + CONSUMER_WARPS - 1) {
                    __threadfence_block();
                    const int n = n0 + lane;
#pragma unroll
                    for (int m = 0; m < MP; ++m) {
                        if (m < p.M && n < p.N) {
                            float v = rb[m * NT + lane];
#pragma unroll
                            for (int k = 1; k < KPH; ++k) v += rb[(k * MP + m) * NT + lane];
                            const size_t off = (size_t)m * p.ldc + n;
                            if (p.n_peers) {
                                // plain stores into every peer's receive slot (its own GPU's memory), this rank's own included
                                const size_t at = ((size_t)(comm_seq & 1u) * p.n_peers + p.peer_rank) * p.peer_slot_elems + off;
                                for (int s = 0; s < p.n_peers; ++s) p.peer_data[s][at] = v;
                            } else if (p.c_is_f16) {
                                __half* cp = reinterpret_cast<__half*>(p.c);
                                if (p.accumulate) v += __half2float(cp[off]);
                                cp[off] = __float2half_rn(v);
                            } else {
                                float* cp = reinterpret_cast<float*>(p.c);
                                if (p.accumulate) v += cp[off];
                                cp[off] = v;
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) { __threadfence_block(); atomicAdd(const_cast<unsigned int*>(cnt), 1u); }   // release
                }
            }
        }
    }

    if (p.n_peers) {
        // After the CTA's stores: one thread's system-scope fence is cumulative over them (the
        // barrier orders them before it); the last CTA of the grid tells every peer that this
        // rank's partial for operation comm_seq is complete.
        named_bar_sync(3, CONSUMERS);
        if (tid == 0) {
            __threadfence_system();
            if (atomicAdd(&p.comm_state[1], 1u) == gridDim.x - 1) {
                atomicExch(&p.comm_state[1], 0u);
                for (int s = 0; s < p.n_peers; ++s)
                    st_release_sys_u32(p.peer_flags[s] + ((comm_seq & 1u) * p.n_peers + p.peer_rank) * 8, comm_seq + 1u);
            }
        }
    }
    if (warp == 0) { TL_MARK(p.launch_id, 3); }
}

}  // namespace strip
}  // namespace twm
