// twm_gemv_mma.cuh — the streaming W4A16 kernels on warp-level MMA, FP16 activations: gemv_kernel for up to
// eight rows (the decode kernel, memory-bound), gemm_rows_kernel + stage_rows_kernel for up to 32 (second half of
// the file).
//
// Replaces warp_gemm_tw_marlin_m1 / _m1_direct
// (crates/kernels/src/quantize.rs:1186-1298) and the launcher's split-K
// (quantize.rs:1314-1357) on B200, where one SM has to unpack about 46 nibbles
// per clock to keep up with HBM3e: more than FP32 FMAs (one per nibble plus the
// unpack) can issue.  Same result definition: w = f32(scale) * (nibble - 8),
// exact products, FP32 accumulation, the scale applied in FP32 per group.
//
// Shape of the work.  A CTA owns 128 columns and a contiguous range of
// 32-blocks of K.  One producer warp streams packed rows (2 KB contiguous per
// block) and scale rows into a five-deep shared-memory ring with 1-D bulk
// copies (TMA unit, mbarrier completion, no multicast).  One to four stager
// warps put the slice's activations into shared memory in the order the
// tensor-core fragments want them, with the per-group sums that fold the "-8".  Eight
// consumer warps own 16 columns each for the whole K range, so there is no
// cross-warp reduction.
//
// Register-level unpack.  Lane (g, t) reads u32 word t of column g's and
// column g+8's 16-byte block (the warp's two loads are each one contiguous
// 128-byte run).  `v & 0x000F000F` is, as two FP16 bit patterns, the pair of
// subnormals (q0, q4) * 2^-24; `v & 0x00F000F0` is (q1, q5) * 2^-20; the same
// on `v >> 8` gives (q2, q6) and (q3, q7).  Five integer instructions turn
// eight nibbles into four operand registers; no conversion, no floating-point
// instruction.  The four registers of the two columns are exactly the A
// fragments of two m16n8k16 MMAs (one per power of two), whose B fragment is
// the activation of the same K positions.  The accumulators of a scale group
// are combined as 2^24*lo + 2^20*hi, the group's -8*sum(A) is added, and the
// FP32 scale multiplies the sum, as the reference's kernel does per block.
//
// Split-K finish and the programmatic-dependent-launch rules are those of the
// FP32 streaming kernel (twm_gemv_simt.cuh).
#pragma once

#include "twm_common.cuh"

namespace twm {
namespace mma {

constexpr int NT = 128;          // columns per CTA
#ifndef TWM_MMA_SB
#define TWM_MMA_SB 8
#endif
#ifndef TWM_MMA_STAGES
#define TWM_MMA_STAGES 5
#endif
constexpr int SB = TWM_MMA_SB;            // 32-blocks per ring stage
constexpr int STAGES = TWM_MMA_STAGES;
constexpr int CONSUMER_WARPS = 8;
constexpr int CONSUMERS = CONSUMER_WARPS * 32;
// + producer warp + stager warps: one stager keeps up with one or two activation rows, four rows take three and
// eight take four (a stager's round is a global load, a permute and a group sum per lane, and every CTA stages
// all rows of its K range).  Measured on K=3584, N=37888: four rows 20.7 us with one stager, 17.0 with two, 16.3
// with three; eight rows 34.5 / 22.4 (three) / 19.0 (four), no gain from six or seven.
#ifndef TWM_MMA_SW4
#define TWM_MMA_SW4 3
#endif
#ifndef TWM_MMA_SW8
#define TWM_MMA_SW8 4
#endif
__host__ __device__ constexpr int stager_warps(int mp) { return mp >= 8 ? TWM_MMA_SW8 : (mp >= 4 ? TWM_MMA_SW4 : 1); }
__host__ __device__ constexpr int threads_for(int mp) { return CONSUMERS + 32 + 32 * stager_warps(mp); }
constexpr int THREADS = threads_for(1);
constexpr int B_BUF_BYTES = 4096;            // staged activations per chunk buffer
constexpr int ASUM_GROUPS = 64;              // scale groups per chunk, at most
#ifndef TWM_MMA_MAX_CLUSTER
#define TWM_MMA_MAX_CLUSTER 16
#endif
#ifndef TWM_MMA_MIN_CTAS
#define TWM_MMA_MIN_CTAS 2
#endif
constexpr int MAX_CLUSTER = TWM_MMA_MAX_CLUSTER;   // K slices that can add up through distributed shared memory
constexpr int CLUSTER_ROWS = 2;              // ... for up to this many activation rows (K slices x rows <= MAX_CLUSTER)

struct Smem {
    alignas(128) uint8_t packed[STAGES][SB * NT * kBlockBytes];
    alignas(128) uint16_t scales[STAGES][SB][NT];
    alignas(128) uint8_t b[2][B_BUF_BYTES];           // [block in chunk][row m < MP][t] x 16 bytes
    alignas(16) float asum8[2][ASUM_GROUPS][8];       // -8 * sum of a group's activations, per row
    alignas(16) float red[MAX_CLUSTER][NT];           // cluster leader only: row (slice * M + m) = one K slice's sums of activation row m
    alignas(8) uint64_t full[STAGES];
    alignas(8) uint64_t empty[STAGES];
    alignas(8) uint64_t b_full[2];
    alignas(8) uint64_t b_empty[2];
    int abort_flag;
    int is_last;
};

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], const uint32_t a0, const uint32_t a1, const uint32_t a2,
                                             const uint32_t a3, const uint32_t b0, const uint32_t b1, const float (&c)[4]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                 : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(c[0]), "f"(c[1]), "f"(c[2]), "f"(c[3]));
}

// loads from 32-bit shared-window addresses (base registers computed once per thread)
__device__ __forceinline__ uint32_t lds32_at(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128_at(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ float2 lds64f_at(uint32_t addr) {
    float2 v;
    asm volatile("ld.shared.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint16_t lds16_at(uint32_t addr) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
    return v;
}

// Eight consecutive K of one activation row as eight f16.  kind 0: the row holds them; kind 1 / 2:
// the row is a fused [gate | up] GEMM output (up at column K) and the GEMM reads
// silu(gate) * up (crates/kernels/src/ops.rs:966-977) or tanh-gelu(gate) * up
// (crates/kernels/src/moe_batched_marlin.rs:138-152), computed in FP32 and rounded to f16.
__device__ __forceinline__ uint4 load_act8(const __half* p8, int up_offset, int kind, bool vec_ok) {
    auto ld8 = [&](const __half* q8) -> uint4 {
        if (vec_ok) return *reinterpret_cast<const uint4*>(q8);
        const uint16_t* a16 = reinterpret_cast<const uint16_t*>(q8);
        uint4 x;
        x.x = a16[0] | ((uint32_t)a16[1] << 16); x.y = a16[2] | ((uint32_t)a16[3] << 16);
        x.z = a16[4] | ((uint32_t)a16[5] << 16); x.w = a16[6] | ((uint32_t)a16[7] << 16);
        return x;
    };
    const uint4 gt = ld8(p8);
    if (kind == 0) return gt;
    const uint4 up = ld8(p8 + up_offset);
    const __half2* gh = reinterpret_cast<const __half2*>(&gt);
    const __half2* uh = reinterpret_cast<const __half2*>(&up);
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 gf = __half22float2(gh[j]), uf = __half22float2(uh[j]);
        float r0, r1;
        if (kind == 1) {
            r0 = gf.x / (1.0f + expf(-gf.x)) * uf.x;
            r1 = gf.y / (1.0f + expf(-gf.y)) * uf.y;
        } else {
            r0 = 0.5f * gf.x * (1.0f + tanhf(0.7978845608f * (gf.x + 0.044715f * gf.x * gf.x * gf.x))) * uf.x;
            r1 = 0.5f * gf.y * (1.0f + tanhf(0.7978845608f * (gf.y + 0.044715f * gf.y * gf.y * gf.y))) * uf.y;
        }
        const __half2 r = __floats2half2_rn(r0, r1);
        ow[j] = *reinterpret_cast<const uint32_t*>(&r);
    }
    return o;
}

// MP = activation rows staged (power of two >= M, <= 8); GSHIFT = log2(32-blocks per scale group);
// AKIND = what the activation rows hold (0: f16 values; 1 / 2: [gate | up], see load_act8)
template <int MP, int GSHIFT, int AKIND = 0>
__global__ void __launch_bounds__(threads_for(MP), TWM_MMA_MIN_CTAS)
gemv_kernel(const __grid_constant__ GemmParams p)
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
    constexpr int gshift = GSHIFT;                           // 32-blocks per scale group = 1 << gshift
    constexpr int gmask = (1 << gshift) - 1;
    constexpr int CHUNK_BLOCKS = B_BUF_BYTES / (64 * MP);    // 64, 32, 16, 8: multiples of SB and of a group
    static_assert(CHUNK_BLOCKS % SB == 0 && CHUNK_BLOCKS <= ASUM_GROUPS, "chunk geometry");
    const int n_chunks = (total_blocks + CHUNK_BLOCKS - 1) / CHUNK_BLOCKS;
    const int slot = p.n_experts ? (int)blockIdx.z : 0;      // top-k slot of a batched expert GEMV
    const __half* A_base = reinterpret_cast<const __half*>(p.a) + (size_t)slot * p.a_expert_stride;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], CONSUMER_WARPS); }
        // a chunk of activations is full once every stager warp has arrived
        for (int s = 0; s < 2; ++s) { mbar_init(&sm.b_full[s], stager_warps(MP)); mbar_init(&sm.b_empty[s], CONSUMER_WARPS); }
        sm.abort_flag = 0;
        sm.is_last = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    // Cluster launches: a CTA may store into the leader's shared memory only once the leader has
    // started.  Everybody arrives here, and waits just before the first such store.
    if (p.cluster_reduce) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    volatile int* abort_flag = &sm.abort_flag;

    float tot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const int g = lane >> 2;
    const int t = lane & 3;
    const int wcol = warp * 16;                       // a consumer warp's 16 columns inside the tile
    if (warp == CONSUMER_WARPS) {
        // ------------------------------------------- producer: packed + scales --
        const uint8_t* packed = p.packed;
        const uint16_t* scales = p.scales;
        if (p.packed_offsets != nullptr) {
            pdl_wait_prior_grids();                       // the offset table may come from the kernel before
            packed += p.packed_offsets[p.expert_idx];
            scales += p.scales_offsets[p.expert_idx];
        }
        if (p.n_experts) {
            pdl_wait_prior_grids();                       // the router's choice comes from the kernel before
            const size_t eid = (size_t)(int)p.expert_ids[slot];
            packed += eid * p.packed_expert_stride;
            scales += eid * p.scales_expert_stride;
        }
        const bool scale_bulk_ok = ((cols & 7) == 0) && ((p.N & 7) == 0) &&
                                   ((reinterpret_cast<uintptr_t>(scales + n0) & 15) == 0);
        for (int it = 0; it < n_stages; ++it) {
            const int slot = it % STAGES;
            const int use = it / STAGES;
            if (use > 0) {
                const bool got = mbar_wait_bounded(&sm.empty[slot], (use - 1) & 1, abort_flag);
                if (!__all_sync(0xffffffffu, got)) break;
            }
            const int bstart = b0 + it * SB;
            const int nb = min(SB, b1 - bstart);
            const int srow_first = bstart >> gshift;
            const int nrows = ((bstart + nb - 1) >> gshift) - srow_first + 1;
            uint32_t tx = (uint32_t)nb * cols * kBlockBytes;
            if (scale_bulk_ok) {
                tx += (uint32_t)nrows * cols * 2;
            } else {
                for (int r = 0; r < nrows; ++r) {
                    const uint16_t* src = scales + (size_t)(srow_first + r) * p.N + n0;
                    for (int cidx = lane; cidx < cols; cidx += 32) sm.scales[slot][r][cidx] = src[cidx];
                }
                __syncwarp();
            }
            // A full stage of packed rows is one tiled TMA load (128 columns x SB blocks; columns
            // past N are zero-filled and still counted).  A ragged last stage, or a launch
            // without a tensor map, copies row by row, one 1-D bulk copy per lane.
            const bool tiled = (p.map_rows == SB) && (nb == SB) && (p.packed_offsets == nullptr);
            if (tiled) tx = (uint32_t)SB * NT * kBlockBytes + (scale_bulk_ok ? (uint32_t)nrows * cols * 2 : 0u);
            if (lane == 0) {
                mbar_arrive_expect_tx(&sm.full[slot], tx);
                if (tiled) tma_load_2d(&sm.packed[slot][0], &p.packed_map, n0 * 2, bstart, &sm.full[slot]);
            }
            __syncwarp();
            if (!tiled && lane < nb) {
                bulk_g2s(&sm.packed[slot][lane * NT * kBlockBytes],
                         packed + ((size_t)(bstart + lane) * p.N + n0) * kBlockBytes,
                         (uint32_t)cols * kBlockBytes, &sm.full[slot]);
            } else if (scale_bulk_ok && lane >= 16 && lane - 16 < nrows) {
                const int r = lane - 16;
                bulk_g2s(&sm.scales[slot][r][0], scales + (size_t)(srow_first + r) * p.N + n0,
                         (uint32_t)cols * 2, &sm.full[slot]);
            }
            __syncwarp();
        }
        // every load of this CTA is on its way: now the head of the next GEMM's weights, so that memory
        // stays busy while this grid drains and the next one starts up, and the next one starts from L2
        prefetch_next_head(p.next, blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z),
                           gridDim.x * gridDim.y * gridDim.z, lane);
        // A launch that does not wait for its predecessor must still not END before it: the kernel
        // after this one waits for this one only.  This warp has nothing left to do.
        if (p.no_wait) pdl_wait_prior_grids();
    } else if (warp > CONSUMER_WARPS) {
        // ----------------------------------------------- activation stagers --
        // One item = 8 consecutive K of one row, stored as the 16 bytes
        // {k0,k4 | k2,k6 | k1,k5 | k3,k7}: the B fragments of the block's two MMAs.
        // Items are numbered so that the 4 << gshift lanes that hold one (scale
        // group, row) are consecutive: the group's sum of activations is then a
        // fixed-order warp-shuffle reduction.  K slices start and end on group
        // boundaries (the host plan sees to that).
        if (!p.no_wait) pdl_wait_prior_grids();
        const __half* A = A_base;
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(A) & 15) == 0) && ((p.lda & 7) == 0) &&
                            ((p.a_expert_stride & 7) == 0);
        constexpr int SW = stager_warps(MP);
        // rounds of 32 items a warp has in flight; a chunk has eight.  (Four with one stager warp: the eight
        // 16-byte loads of a full chunk in flight made this kernel's 77 registers; with four it takes 64 and
        // each of the four decode GEMMs got 0.1-0.3 us faster.)
        constexpr int PF = SW == 1 ? 4 : 8 / SW + (8 % SW ? 1 : 0);
        const int sw = warp - CONSUMER_WARPS - 1;            // stager warp sw takes rounds sw, sw + SW, ...
        for (int chunk = 1; chunk < n_chunks; ++chunk) {     // chunk 0 is staged by the consumer warps (below)
            const int buf = chunk & 1;
            const int use = chunk >> 1;
            const int cb0 = chunk * CHUNK_BLOCKS;
            const int cb = min(CHUNK_BLOCKS, total_blocks - cb0);
            const int items = cb * MP * 4;                    // item = (((gi * MP) + m) << gshift | bj) * 4 + t
            bool waited = false, ok = true;
            for (int base = sw * 32; base < items && ok; base += 32 * SW * PF) {
                const int live = min(PF, (items - base + 32 * SW - 1) / (32 * SW));     // rounds of 32 items that hold anything (warp-uniform)
                uint4 x[PF];
#pragma unroll
                for (int u = 0; u < PF; ++u) {
                    const int it = base + u * 32 * SW + lane;
                    x[u] = make_uint4(0, 0, 0, 0);
                    if (u < live && it < items) {
                        const int tt = it & 3;
                        const int bj = (it >> 2) & gmask;
                        const int rest = it >> (2 + gshift);
                        const int m = rest % MP;
                        const int bi = ((rest / MP) << gshift) + bj;
                        if (m < p.M) {
                            const size_t off = (size_t)m * p.lda + (size_t)(b0 + cb0 + bi) * kBlockK + tt * 8;
                            x[u] = load_act8(A + off, p.K, AKIND, vec_ok);
                        }
                    }
                }
                if (!waited) {
                    if (use > 0) {
                        const bool got = mbar_wait_bounded(&sm.b_empty[buf], (use - 1) & 1, abort_flag);
                        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
                    }
                    waited = true;
                }
#pragma unroll
                for (int u = 0; u < PF; ++u) {
                    if (u >= live) break;                            // nothing in the later rounds: skip their shuffles too
                    const int it = base + u * 32 * SW + lane;
                    const int tt = it & 3;
                    const int bj = (it >> 2) & gmask;
                    const int rest = it >> (2 + gshift);
                    const int m = rest % MP;
                    const int gi = rest / MP;
                    float s = 0.0f;
                    if (it < items) {
                        const int bi = (gi << gshift) + bj;
                        uint4 o;
                        o.x = __byte_perm(x[u].x, x[u].z, 0x5410); o.y = __byte_perm(x[u].y, x[u].w, 0x5410);
                        o.z = __byte_perm(x[u].x, x[u].z, 0x7632); o.w = __byte_perm(x[u].y, x[u].w, 0x7632);
                        *reinterpret_cast<uint4*>(&sm.b[buf][((bi * MP + m) * 4 + tt) * 16]) = o;
                        const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&x[u].x));
                        const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&x[u].y));
                        const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&x[u].z));
                        const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&x[u].w));
                        s = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
                    }
                    s += __shfl_xor_sync(0xffffffffu, s, 1);
                    s += __shfl_xor_sync(0xffffffffu, s, 2);
                    if (gshift != 0) {                              // four blocks of a 128-group
                        s += __shfl_xor_sync(0xffffffffu, s, 4);
                        s += __shfl_xor_sync(0xffffffffu, s, 8);
                    }
                    if (it < items && (it & ((4 << gshift) - 1)) == 0) sm.asum8[buf][gi][m] = -8.0f * s;
                }
            }
            if (ok && !waited && use > 0) {
                // a warp with no item in a ragged last chunk still waits for the buffer's turn: its arrival
                // must not be counted into the phase of the chunk that used the buffer before
                const bool got = mbar_wait_bounded(&sm.b_empty[buf], (use - 1) & 1, abort_flag);
                if (!__all_sync(0xffffffffu, got)) ok = false;
            }
            if (!ok) break;
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.b_full[buf]);
        }
    } else {
    // ---------------------------------------------------------- consumers --
    // K slices hold whole scale groups and a ring stage holds whole groups, so
    // the per-stage work unrolls into straight-line code: per 32-block two
    // 32-bit loads, one 128-bit load, ten integer ops and two MMAs.
    constexpr int GB = 1 << GSHIFT;
    {
        // The first chunk of activations (at most 256 items) is staged by the 256 consumer threads,
        // one item each, in the stager's layout and summation order: the launch's first multiply
        // then waits for one round of loads instead of the stager warp's eight.
        if (!p.no_wait) pdl_wait_prior_grids();
        const __half* A = A_base;
        const bool vec_ok = ((reinterpret_cast<uintptr_t>(A) & 15) == 0) && ((p.lda & 7) == 0) &&
                            ((p.a_expert_stride & 7) == 0);
        const int items = min(CHUNK_BLOCKS, total_blocks) * MP * 4;
        const int it = tid;
        const int tt = it & 3;
        const int bj = (it >> 2) & gmask;
        const int rest = it >> (2 + gshift);
        const int m = rest % MP;
        const int gi = rest / MP;
        const int bi = (gi << gshift) + bj;
        uint4 x = make_uint4(0, 0, 0, 0);
        if (it < items && m < p.M) {
            const size_t off = (size_t)m * p.lda + (size_t)(b0 + bi) * kBlockK + tt * 8;
            x = load_act8(A + off, p.K, AKIND, vec_ok);
        }
        float s = 0.0f;
        if (it < items) {
            uint4 o;
            o.x = __byte_perm(x.x, x.z, 0x5410); o.y = __byte_perm(x.y, x.w, 0x5410);
            o.z = __byte_perm(x.x, x.z, 0x7632); o.w = __byte_perm(x.y, x.w, 0x7632);
            *reinterpret_cast<uint4*>(&sm.b[0][((bi * MP + m) * 4 + tt) * 16]) = o;
            const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&x.x));
            const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&x.y));
            const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&x.z));
            const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&x.w));
            s = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        if (gshift != 0) {
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            s += __shfl_xor_sync(0xffffffffu, s, 8);
        }
        if (it < items && (it & ((4 << gshift) - 1)) == 0) sm.asum8[0][gi][m] = -8.0f * s;
        named_bar_sync(1, CONSUMERS);
        if (tid == 0)
            for (int i = 0; i < stager_warps(MP); ++i) mbar_arrive(&sm.b_full[0]);      // the consumers stand in for every stager warp
    }
    const float zero4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const uint32_t w_base = smem_u32(&sm.packed[0][0]) + wcol * kBlockBytes + lane * 4;
    const uint32_t s_base = smem_u32(&sm.scales[0][0][0]) + (wcol + g) * 2;
    const uint32_t b_base = smem_u32(&sm.b[0][0]) + (g * 4 + t) * 16;
    const uint32_t a8_base = smem_u32(&sm.asum8[0][0][0]) + t * 8;
    bool ok = true;

    for (int it = 0; it < n_stages; ++it) {
        const int slot = it % STAGES;
        const int nb = min(SB, b1 - (b0 + it * SB));
        const int rel0 = it * SB;                                     // first block of the stage, relative to b0
        const int chunk = rel0 / CHUNK_BLOCKS;
        const int buf = chunk & 1;
        const int bi0 = rel0 - chunk * CHUNK_BLOCKS;                  // first block of the stage inside the chunk
        if (ok && bi0 == 0) {
            const bool got = mbar_wait_bounded(&sm.b_full[buf], (chunk >> 1) & 1, abort_flag);
            if (!__all_sync(0xffffffffu, got)) ok = false;
        }
        if (ok) {
            const bool got = mbar_wait_bounded(&sm.full[slot], (it / STAGES) & 1, abort_flag);
            if (!__all_sync(0xffffffffu, got)) ok = false;
        }
        if (ok) {
            const uint32_t w_st = w_base + slot * (SB * NT * kBlockBytes);
            const uint32_t s_st = s_base + slot * (SB * NT * 2);
            const uint32_t b_st = b_base + buf * B_BUF_BYTES + bi0 * (MP * 64);
            const uint32_t a8_st = a8_base + (buf * ASUM_GROUPS + (bi0 >> GSHIFT)) * 32;
#pragma unroll
            for (int r0 = 0; r0 < SB; r0 += GB) {
                if (r0 < nb) {
                    float lo[4], hi[4];
#pragma unroll
                    for (int j = 0; j < GB; ++j) {
                        const int r = r0 + j;
                        const uint32_t v0 = lds32_at(w_st + r * (NT * kBlockBytes));          // column g, word t
                        const uint32_t v1 = lds32_at(w_st + r * (NT * kBlockBytes) + 128);    // column g + 8, word t
                        uint4 xb = make_uint4(0, 0, 0, 0);
                        if (MP == 8 || g < MP) xb = lds128_at(b_st + r * (MP * 64));
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
                    // group done: value = 2^24*lo + 2^20*hi - 8*sum(a), times the FP32 scale
                    const float s0 = f16_bits_to_f32(lds16_at(s_st + (r0 >> GSHIFT) * (NT * 2)));
                    const float s1 = f16_bits_to_f32(lds16_at(s_st + (r0 >> GSHIFT) * (NT * 2) + 16));
                    const float2 a8 = lds64f_at(a8_st + (r0 >> GSHIFT) * 32);
                    const float k20 = 1048576.0f;                     // 2^20
                    tot[0] = fmaf(s0, fmaf(fmaf(lo[0], 16.0f, hi[0]), k20, a8.x), tot[0]);
                    tot[1] = fmaf(s0, fmaf(fmaf(lo[1], 16.0f, hi[1]), k20, a8.y), tot[1]);
                    tot[2] = fmaf(s1, fmaf(fmaf(lo[2], 16.0f, hi[2]), k20, a8.x), tot[2]);
                    tot[3] = fmaf(s1, fmaf(fmaf(lo[3], 16.0f, hi[3]), k20, a8.y), tot[3]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) {
            if (ok) mbar_arrive(&sm.empty[slot]);
            const bool chunk_end = ((rel0 + SB) % CHUNK_BLOCKS == 0) || (it == n_stages - 1);
            if (ok && chunk_end) mbar_arrive(&sm.b_empty[buf]);
        }
    }

    }   // consumers

    // ----------------------------------------------------- store / split-K --
    // lane (g, t) of a consumer warp holds C[m = 2t, 2t+1][n = n0 + wcol + g] and the same rows for column + 8
    const bool consumer = warp < CONSUMER_WARPS;
    const int nA = n0 + wcol + g, nB = nA + 8;
    const int mA = 2 * t, mB = 2 * t + 1;
    // tensor-parallel push: this launch's sequence number and buffer set (stable for the whole
    // launch: only the consumer kernel that follows advances it)
    const unsigned int comm_seq = p.n_peers ? ld_volatile_u32(p.comm_state) : 0u;
    if (p.expert_weights != nullptr && consumer) {
        // weighted sum over the slots: every slice carries its slot's router weight into the reduction
        const float wgt = __ldg(p.expert_weights + slot);
        tot[0] *= wgt; tot[1] *= wgt; tot[2] *= wgt; tot[3] *= wgt;
    }
    const size_t c_slot_off = (p.n_experts && p.expert_weights == nullptr) ? (size_t)slot * p.c_expert_stride : 0;
    auto store_c = [&](int m, int n, float v) {
        if (m >= p.M || n >= p.N) return;
        const size_t off = (size_t)m * p.ldc + n + c_slot_off;
        if (p.n_peers) {
            comm_store(p, comm_seq, off, v);
            return;
        }
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

    if (p.cluster_reduce) {
        // The K slices of this tile are the CTAs of one cluster.  Each writes its partial tile
        // into the leader's shared memory (distributed shared memory store), one cluster
        // barrier, and the leader adds the slices in slice order: no workspace, no atomics,
        // the same bits whatever order the slices finish in.  Every thread of every CTA
        // reaches the barrier (all loops above are bounded).
        const uint32_t rank = cluster_ctarank();
        asm volatile("barrier.cluster.wait.aligned;" ::: "memory");      // pairs with the arrive at the top: every CTA of the cluster runs
        if (consumer && t == 0 && *abort_flag == 0) {
            const uint32_t base = mapa_shared(smem_u32(&sm.red[rank * p.M][0]), 0);
            st_cluster_f32(base + (wcol + g) * 4, tot[0]);
            st_cluster_f32(base + (wcol + g + 8) * 4, tot[2]);
            if (p.M > 1) {
                st_cluster_f32(base + (NT + wcol + g) * 4, tot[1]);
                st_cluster_f32(base + (NT + wcol + g + 8) * 4, tot[3]);
            }
        }
        cluster_sync_all();
        if (rank == 0 && tid < p.M * NT && *abort_flag == 0) {
            const int m = tid / NT, col = tid - m * NT;
            float s = 0.0f;
            for (int sp = 0; sp < p.reduce_slices; ++sp) s += sm.red[sp * p.M + m][col];      // slices in (slot, K slice) order
            store_c(m, n0 + col, s);
        }
        if (p.n_peers && rank == 0) {       // only the cluster leaders store
            __syncthreads();
            if (tid == 0) comm_cta_done(p, comm_seq, gridDim.x);
        }
        return;
    }

    if (!consumer) return;
    named_bar_sync(1, CONSUMERS);
    if (*abort_flag && !p.n_peers) return;    // a wait expired: leave C untouched, the error word is set
    if (p.reduce_slices == 1) {
        if (*abort_flag == 0) {
            store_c(mA, nA, tot[0]); store_c(mB, nA, tot[1]); store_c(mA, nB, tot[2]); store_c(mB, nB, tot[3]);
        }
        if (p.n_peers) {
            named_bar_sync(1, CONSUMERS);
            if (tid == 0) comm_cta_done(p, comm_seq, gridDim.x * gridDim.y);
        }
        return;
    }
    auto ws_at = [&](int sp, int m, int n) -> float* { return &p.ws_partials[((size_t)sp * p.M + m) * p.N + n]; };
    const int my_slice = slot * p.splits + blockIdx.y;                 // (slot, K slice) order
    if (mA < p.M && nA < p.N) *ws_at(my_slice, mA, nA) = tot[0];
    if (mB < p.M && nA < p.N) *ws_at(my_slice, mB, nA) = tot[1];
    if (mA < p.M && nB < p.N) *ws_at(my_slice, mA, nB) = tot[2];
    if (mB < p.M && nB < p.N) *ws_at(my_slice, mB, nB) = tot[3];
    __threadfence();
    named_bar_sync(1, CONSUMERS);
    if (tid == 0) {
        const unsigned prev = atomicAdd(&p.ws_counters[blockIdx.x], 1u);
        sm.is_last = (prev == (unsigned)(p.reduce_slices - 1));
    }
    named_bar_sync(1, CONSUMERS);
    if (!sm.is_last) return;
    __threadfence();
    // The last arriver adds the slices in slice order, four slices' loads of all four outputs in flight together
    // (one load per slice in turn costs a round trip to L2 per slice and output).
    const int ms[4] = {mA, mB, mA, mB}, ns[4] = {nA, nA, nB, nB};
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int sp0 = 0; sp0 < p.reduce_slices; sp0 += 4) {
        float v[4][4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                v[u][e] = (sp0 + u < p.reduce_slices && ms[e] < p.M && ns[e] < p.N) ? ld_cg_f32(ws_at(sp0 + u, ms[e], ns[e])) : 0.0f;
#pragma unroll
        for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                if (sp0 + u < p.reduce_slices) acc[e] += v[u][e];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) store_c(ms[e], ns[e], acc[e]);
    if (tid == 0) atomicExch(&p.ws_counters[blockIdx.x], 0u);
}


// ------------------------------------------------------------ 9 to 32 rows --
// The same multiply with two or four MMA N-tiles of eight rows per block.  Here every CTA staging every
// row itself would cost more than the multiply (16 rows of K = 3584 are 114 KB per CTA), so a pre-pass
// (stage_rows_kernel) writes the B fragments and the group sums once, in the stagers' layout, to the
// workspace, and one lane per CTA copies a ring stage's share of them with bulk copies, next to the
// producer warp's weights.  Arithmetic and summation order are those of gemv_kernel.

constexpr int rows_stages(int mp) { return mp <= 8 ? 5 : (mp <= 16 ? 4 : 3); }    // ring depth that leaves two CTAs per SM

template <int MP>
struct RowsSmem {
    static constexpr int ST = rows_stages(MP);
    alignas(128) uint8_t packed[ST][SB * NT * kBlockBytes];
    alignas(128) uint16_t scales[ST][SB][NT];
    alignas(128) uint8_t b[ST][SB * MP * 64];            // [block in stage][row m < MP][t] x 16 bytes
    alignas(16) float asum8[ST][SB * MP];                // [group in stage][row]: -8 * sum of the group's activations
    alignas(8) uint64_t full[ST];
    alignas(8) uint64_t empty[ST];
    alignas(8) uint64_t b_full[ST];
    int abort_flag;
    int is_last;
};

// One thread per item (8 consecutive K of one row), numbered as the stager warps number them, so that the
// lanes of one (scale group, row) are consecutive and the group sum is the same fixed-order shuffle tree.
// bq: [K/32][MP][4][16 B]; asum: [K/group][MP].  Rows M..MP-1 are written as zeros.
template <int GSHIFT, int AKIND>
__global__ void __launch_bounds__(256)
stage_rows_kernel(uint8_t* __restrict__ bq, float* __restrict__ asum, const __half* __restrict__ A, long lda, int M, int MP,
                  int K, int nkb)
{
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    constexpr int gshift = GSHIFT;
    constexpr int gmask = (1 << gshift) - 1;
    const int it = blockIdx.x * blockDim.x + threadIdx.x;
    const int items = nkb * MP * 4;                          // a multiple of 32: whole warps are in or out
    if (it >= items) return;
    const int tt = it & 3;
    const int bj = (it >> 2) & gmask;
    const int rest = it >> (2 + gshift);
    const int m = rest % MP;
    const int gi = rest / MP;
    const int bi = (gi << gshift) + bj;
    const bool vec_ok = ((reinterpret_cast<uintptr_t>(A) & 15) == 0) && ((lda & 7) == 0);
    uint4 x = make_uint4(0, 0, 0, 0);
    if (m < M) x = load_act8(A + (size_t)m * lda + (size_t)bi * kBlockK + tt * 8, K, AKIND, vec_ok);
    uint4 o;
    o.x = __byte_perm(x.x, x.z, 0x5410); o.y = __byte_perm(x.y, x.w, 0x5410);
    o.z = __byte_perm(x.x, x.z, 0x7632); o.w = __byte_perm(x.y, x.w, 0x7632);
    *reinterpret_cast<uint4*>(bq + ((size_t)(bi * MP + m) * 4 + tt) * 16) = o;
    const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&x.x));
    const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&x.y));
    const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&x.z));
    const float2 f3 = __half22float2(*reinterpret_cast<const __half2*>(&x.w));
    float s = ((f0.x + f0.y) + (f1.x + f1.y)) + ((f2.x + f2.y) + (f3.x + f3.y));
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if (gshift != 0) {
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        s += __shfl_xor_sync(0xffffffffu, s, 8);
    }
    if ((it & ((4 << gshift) - 1)) == 0) asum[(size_t)gi * MP + m] = -8.0f * s;
}

// MP = 8, 16, 24 or 32 rows staged (whole MMA N-tiles of eight); GSHIFT as above.  p.rows_b / p.rows_asum: the pre-pass's output.
template <int MP, int GSHIFT>
__global__ void __launch_bounds__(THREADS, TWM_MMA_MIN_CTAS)
gemm_rows_kernel(const __grid_constant__ GemmParams p)
{
    extern __shared__ __align__(128) uint8_t smem_raw[];
    using Sm = RowsSmem<MP>;
    Sm& sm = *reinterpret_cast<Sm*>(smem_raw);
    constexpr int ST = Sm::ST;
    constexpr int NTL = MP / 8;                              // MMA N-tiles of eight rows
    constexpr int GB = 1 << GSHIFT;

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
        for (int s = 0; s < ST; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], CONSUMER_WARPS); mbar_init(&sm.b_full[s], 1); }
        sm.abort_flag = 0;
        sm.is_last = 0;
        mbar_fence_init();
    }
    __syncthreads();
    pdl_launch_dependents();
    volatile int* abort_flag = &sm.abort_flag;

    float tot[NTL][4];
#pragma unroll
    for (int nt = 0; nt < NTL; ++nt) { tot[nt][0] = tot[nt][1] = tot[nt][2] = tot[nt][3] = 0.0f; }
    const int g = lane >> 2;
    const int t = lane & 3;
    const int wcol = warp * 16;
    if (warp == CONSUMER_WARPS) {
        // -------------------------- producer: packed + scales (weights are constants: no wait) --
        const uint8_t* packed = p.packed;
        const uint16_t* scales = p.scales;
        const bool scale_bulk_ok = ((cols & 7) == 0) && ((p.N & 7) == 0) &&
                                   ((reinterpret_cast<uintptr_t>(scales + n0) & 15) == 0);
        for (int it = 0; it < n_stages; ++it) {
            const int slot = it % ST;
            const int use = it / ST;
            if (use > 0) {
                const bool got = mbar_wait_bounded(&sm.empty[slot], (use - 1) & 1, abort_flag);
                if (!__all_sync(0xffffffffu, got)) break;
            }
            const int bstart = b0 + it * SB;
            const int nb = min(SB, b1 - bstart);
            const int srow_first = bstart >> GSHIFT;
            const int nrows = ((bstart + nb - 1) >> GSHIFT) - srow_first + 1;
            uint32_t tx = (uint32_t)nb * cols * kBlockBytes;
            if (scale_bulk_ok) {
                tx += (uint32_t)nrows * cols * 2;
            } else {
                for (int r = 0; r < nrows; ++r) {
                    const uint16_t* src = scales + (size_t)(srow_first + r) * p.N + n0;
                    for (int cidx = lane; cidx < cols; cidx += 32) sm.scales[slot][r][cidx] = src[cidx];
                }
                __syncwarp();
            }
            const bool tiled = (p.map_rows == SB) && (nb == SB);
            if (tiled) tx = (uint32_t)SB * NT * kBlockBytes + (scale_bulk_ok ? (uint32_t)nrows * cols * 2 : 0u);
            if (lane == 0) {
                mbar_arrive_expect_tx(&sm.full[slot], tx);
                if (tiled) tma_load_2d(&sm.packed[slot][0], &p.packed_map, n0 * 2, bstart, &sm.full[slot]);
            }
            __syncwarp();
            if (!tiled && lane < nb) {
                bulk_g2s(&sm.packed[slot][lane * NT * kBlockBytes],
                         packed + ((size_t)(bstart + lane) * p.N + n0) * kBlockBytes,
                         (uint32_t)cols * kBlockBytes, &sm.full[slot]);
            } else if (scale_bulk_ok && lane >= 16 && lane - 16 < nrows) {
                const int r = lane - 16;
                bulk_g2s(&sm.scales[slot][r][0], scales + (size_t)(srow_first + r) * p.N + n0,
                         (uint32_t)cols * 2, &sm.full[slot]);
            }
            __syncwarp();
        }
        prefetch_next_head(p.next, blockIdx.x + gridDim.x * blockIdx.y, gridDim.x * gridDim.y, lane);
    } else if (warp == CONSUMER_WARPS + 1) {
        // ------------- staged activations: one lane, two bulk copies per ring stage, after the pre-pass --
        pdl_wait_prior_grids();
        if (lane == 0) {
            for (int it = 0; it < n_stages; ++it) {
                const int slot = it % ST;
                const int use = it / ST;
                if (use > 0 && !mbar_wait_bounded(&sm.empty[slot], (use - 1) & 1, abort_flag)) break;
                const int bstart = b0 + it * SB;
                const int nb = min(SB, b1 - bstart);
                const int ngroups = (nb + GB - 1) >> GSHIFT;
                const uint32_t b_bytes = (uint32_t)nb * MP * 64, s_bytes = (uint32_t)ngroups * MP * 4;
                mbar_arrive_expect_tx(&sm.b_full[slot], b_bytes + s_bytes);
                bulk_g2s(&sm.b[slot][0], p.rows_b + (size_t)bstart * MP * 64, b_bytes, &sm.b_full[slot]);
                bulk_g2s(&sm.asum8[slot][0], p.rows_asum + (size_t)(bstart >> GSHIFT) * MP, s_bytes, &sm.b_full[slot]);
            }
        }
    } else {
    // ---------------------------------------------------------- consumers --
    pdl_wait_prior_grids();          // their stores and workspace traffic come after the launch before
    const float zero4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    const uint32_t w_base = smem_u32(&sm.packed[0][0]) + wcol * kBlockBytes + lane * 4;
    const uint32_t s_base = smem_u32(&sm.scales[0][0][0]) + (wcol + g) * 2;
    const uint32_t b_base = smem_u32(&sm.b[0][0]) + (g * 4 + t) * 16;
    const uint32_t a8_base = smem_u32(&sm.asum8[0][0]) + t * 8;
    bool ok = true;
    for (int it = 0; it < n_stages; ++it) {
        const int slot = it % ST;
        const int nb = min(SB, b1 - (b0 + it * SB));
        if (ok) {
            const bool got = mbar_wait_bounded(&sm.b_full[slot], (it / ST) & 1, abort_flag);
            if (!__all_sync(0xffffffffu, got)) ok = false;
        }
        if (ok) {
            const bool got = mbar_wait_bounded(&sm.full[slot], (it / ST) & 1, abort_flag);
            if (!__all_sync(0xffffffffu, got)) ok = false;
        }
        if (ok) {
            const uint32_t w_st = w_base + slot * (SB * NT * kBlockBytes);
            const uint32_t s_st = s_base + slot * (SB * NT * 2);
            const uint32_t b_st = b_base + slot * (SB * MP * 64);
            const uint32_t a8_st = a8_base + slot * (SB * MP * 4);
#pragma unroll
            for (int r0 = 0; r0 < SB; r0 += GB) {
                if (r0 < nb) {
                    float lo[NTL][4], hi[NTL][4];
#pragma unroll
                    for (int j = 0; j < GB; ++j) {
                        const int r = r0 + j;
                        const uint32_t v0 = lds32_at(w_st + r * (NT * kBlockBytes));          // column g, word t
                        const uint32_t v1 = lds32_at(w_st + r * (NT * kBlockBytes) + 128);    // column g + 8, word t
                        const uint32_t v0s = v0 >> 8, v1s = v1 >> 8;
                        const uint32_t l0 = v0 & 0x000F000Fu, l1 = v1 & 0x000F000Fu, l2 = v0s & 0x000F000Fu, l3 = v1s & 0x000F000Fu;
                        const uint32_t h0 = v0 & 0x00F000F0u, h1 = v1 & 0x00F000F0u, h2 = v0s & 0x00F000F0u, h3 = v1s & 0x00F000F0u;
#pragma unroll
                        for (int nt = 0; nt < NTL; ++nt) {
                            const uint4 xb = lds128_at(b_st + r * (MP * 64) + nt * 512);      // rows 8 nt + g
                            if (j == 0) {
                                mma_m16n8k16(lo[nt], l0, l1, l2, l3, xb.x, xb.y, zero4);
                                mma_m16n8k16(hi[nt], h0, h1, h2, h3, xb.z, xb.w, zero4);
                            } else {
                                mma_m16n8k16(lo[nt], l0, l1, l2, l3, xb.x, xb.y, lo[nt]);
                                mma_m16n8k16(hi[nt], h0, h1, h2, h3, xb.z, xb.w, hi[nt]);
                            }
                        }
                    }
                    // group done: value = 2^24*lo + 2^20*hi - 8*sum(a), times the FP32 scale
                    const float s0 = f16_bits_to_f32(lds16_at(s_st + (r0 >> GSHIFT) * (NT * 2)));
                    const float s1 = f16_bits_to_f32(lds16_at(s_st + (r0 >> GSHIFT) * (NT * 2) + 16));
                    const float k20 = 1048576.0f;                     // 2^20
#pragma unroll
                    for (int nt = 0; nt < NTL; ++nt) {
                        const float2 a8 = lds64f_at(a8_st + (r0 >> GSHIFT) * (MP * 4) + nt * 32);
                        tot[nt][0] = fmaf(s0, fmaf(fmaf(lo[nt][0], 16.0f, hi[nt][0]), k20, a8.x), tot[nt][0]);
                        tot[nt][1] = fmaf(s0, fmaf(fmaf(lo[nt][1], 16.0f, hi[nt][1]), k20, a8.y), tot[nt][1]);
                        tot[nt][2] = fmaf(s1, fmaf(fmaf(lo[nt][2], 16.0f, hi[nt][2]), k20, a8.x), tot[nt][2]);
                        tot[nt][3] = fmaf(s1, fmaf(fmaf(lo[nt][3], 16.0f, hi[nt][3]), k20, a8.y), tot[nt][3]);
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0 && ok) mbar_arrive(&sm.empty[slot]);
    }
    }   // consumers

    // ----------------------------------------------------- store / split-K --
    // lane (g, t): C[m = 8 nt + 2t, + 1][n = n0 + wcol + g] and the same rows for column + 8
    if (warp >= CONSUMER_WARPS) return;
    const int nA = n0 + wcol + g, nB = nA + 8;
    // tensor-parallel push: this launch's sequence number and buffer set (only the consumer kernel advances it)
    const unsigned int comm_seq = p.n_peers ? ld_volatile_u32(p.comm_state) : 0u;
    auto store_c = [&](int m, int n, float v) {
        if (m >= p.M || n >= p.N) return;
        const size_t off = (size_t)m * p.ldc + n;
        if (p.n_peers) { comm_store(p, comm_seq, off, v); return; }
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
    named_bar_sync(1, CONSUMERS);
    // a wait expired: leave C untouched, the error word is set; with peers the CTA still counts itself, so that
    // their consumers do not wait for this rank in vain
    if (*abort_flag && !p.n_peers) return;
    if (p.reduce_slices == 1) {
        if (*abort_flag == 0) {
#pragma unroll
            for (int nt = 0; nt < NTL; ++nt) {
                const int mA = nt * 8 + 2 * t, mB = mA + 1;
                store_c(mA, nA, tot[nt][0]); store_c(mB, nA, tot[nt][1]); store_c(mA, nB, tot[nt][2]); store_c(mB, nB, tot[nt][3]);
            }
        }
        if (p.n_peers) {
            named_bar_sync(1, CONSUMERS);
            if (tid == 0) comm_cta_done(p, comm_seq, gridDim.x * gridDim.y);
        }
        return;
    }
    auto ws_at = [&](int sp, int m, int n) -> float* { return &p.ws_partials[((size_t)sp * p.M + m) * p.N + n]; };
    const int my_slice = blockIdx.y;
#pragma unroll
    for (int nt = 0; nt < NTL; ++nt) {
        const int mA = nt * 8 + 2 * t, mB = mA + 1;
        if (mA < p.M && nA < p.N) *ws_at(my_slice, mA, nA) = tot[nt][0];
        if (mB < p.M && nA < p.N) *ws_at(my_slice, mB, nA) = tot[nt][1];
        if (mA < p.M && nB < p.N) *ws_at(my_slice, mA, nB) = tot[nt][2];
        if (mB < p.M && nB < p.N) *ws_at(my_slice, mB, nB) = tot[nt][3];
    }
    __threadfence();
    named_bar_sync(1, CONSUMERS);
    if (tid == 0) {
        const unsigned prev = atomicAdd(&p.ws_counters[blockIdx.x], 1u);
        sm.is_last = (prev == (unsigned)(p.reduce_slices - 1));
    }
    named_bar_sync(1, CONSUMERS);
    if (!sm.is_last) return;
    __threadfence();
    // the last arriver adds the slices in slice order, one N-tile's four outputs over four slices in flight together
#pragma unroll
    for (int nt = 0; nt < NTL; ++nt) {
        const int mA = nt * 8 + 2 * t, mB = mA + 1;
        const int ms[4] = {mA, mB, mA, mB}, ns[4] = {nA, nA, nB, nB};
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (int sp0 = 0; sp0 < p.reduce_slices; sp0 += 4) {
            float v[4][4];
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    v[u][e] = (sp0 + u < p.reduce_slices && ms[e] < p.M && ns[e] < p.N) ? ld_cg_f32(ws_at(sp0 + u, ms[e], ns[e])) : 0.0f;
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (sp0 + u < p.reduce_slices) acc[e] += v[u][e];
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) store_c(ms[e], ns[e], acc[e]);
    }
    if (tid == 0) atomicExch(&p.ws_counters[blockIdx.x], 0u);
    if (p.n_peers) {                   // one storing CTA per tile
        named_bar_sync(1, CONSUMERS);
        if (tid == 0) comm_cta_done(p, comm_seq, gridDim.x);
    }
}

}  // namespace mma
}  // namespace twm
