// twm_chain.cuh — a sequence of dependent W4A16 GEMMs (M <= 8, FP16 activations) as ONE
// persistent launch.
//
// The reference enqueues one kernel per GEMM (gemm_tw_marlin_m1,
// crates/kernels/src/quantize.rs:1301-1360; four per layer in
// forward_decode_tw_marlin_graph, crates/kernels/src/generate.rs:2149-2206).  On B200 a
// decode-size GEMM streams its weights in 1-11 us, and a launch that has to wait for the one
// before costs about 3.6 us on top of that whatever its size: the previous grid drains, the new
// one fills its pipeline from empty.  Here every CTA of one cooperative grid walks the whole
// list of GEMMs.  The weight stream never stops at a GEMM boundary: the producer warp keeps
// filling the shared-memory ring with the NEXT GEMM's packed rows while the consumer warps
// finish the current one, and only the activation stager waits (bounded) on a completion
// counter in global memory for the GEMM whose output it reads.
//
// Arithmetic, fragment layout and per-stage code are those of twm::mma::gemv_kernel
// (twm_gemv_mma.cuh); the result definition is the same: w = f32(scale) * (nibble - 8), exact
// products, FP32 accumulation, the scale applied per group.
//
// Work split.  A GEMM is n_tiles x units_per_tile units (128 columns x 4 consecutive 32-blocks
// of K).  The units, numbered tile-major, are dealt to the CTAs in contiguous runs of nearly
// equal length ("stream-K"), so a CTA's run is a list of pieces (tile, K range).  A tile that
// is cut into several pieces is summed through FP32 partials in the chain's scratch by the
// CTA that arrives last on the tile's counter, in piece order: the result does not depend on
// arrival order.  Every finished tile adds one to the GEMM's completion counter.
#pragma once

#include "twm_common.cuh"
#include "twm_gemv_mma.cuh"

namespace twm {
namespace chain {

constexpr int NT = 128;                 // columns per tile
constexpr int SB = 8;                   // 32-blocks per full ring stage
constexpr int UNIT = 4;                 // 32-blocks per work unit (one 128-group)
constexpr int STAGES = 5;               // 5 x 16 KB of packed rows in flight per CTA, two CTAs per SM
constexpr int CONSUMER_WARPS = 8;
constexpr int CONSUMERS = CONSUMER_WARPS * 32;
constexpr int THREADS = CONSUMERS + 96; // + producer warp + stager warp + epilogue warp
constexpr int B_BUF_BYTES = 4096;
constexpr int ASUM_GROUPS = 64;
constexpr int CTAS_PER_SM = 2;

enum { A_F16 = 0, A_SILU_MUL = 1 };

// One GEMM of the list, device-resident, written once by the host when the chain is created.
struct alignas(128) Op {
    CUtensorMap map8;            // packed as u64 [K/32][2N], box 256 x 8 rows: one full ring stage
    CUtensorMap map4;            // the same with a 4-row box: the half stage that ends a piece
    const uint8_t* packed;
    const uint16_t* scales;
    const void* a;               // A_F16: f16 [M][lda];  A_SILU_MUL: f16 [M][lda] holding [gate | up], up at +K
    void* c;
    float* partials;             // [n_tiles][max_pieces][M][NT] f32
    unsigned int* tile_counters; // [n_tiles], zero between launches
    long lda, ldc;
    int M, N, K, nkb;
    int gshift;                  // log2(32-blocks per scale group): 0 or 2
    int n_tiles;
    int units_per_tile;
    int total_units;
    int ranks;                   // CTAs that take part: min(grid, total_units)
    int rot;                     // CTA c plays rank (c + rot) % grid
    int max_pieces;
    int a_kind;
    int c_is_f16;
    int accumulate;
    int wait_from;               // GEMMs [wait_from, own index) must be complete before `a` is read
    int use_maps;
};

// Global state of one chain.
struct State {
    unsigned int exit_count;     // CTAs that have left the kernel; the last one resets the counters
    unsigned int abort;          // some wait ran out: everybody stops waiting
    unsigned int n_tile_counters;
    unsigned int pad;
    unsigned int* all_tile_counters;
    unsigned int pad2[58];
};
static_assert(sizeof(State) == 256, "State is a 256-byte header");

// ---- the deal: pure integer arithmetic shared by host (planning, tests) and device ----
// rank r of `ranks` owns units [r * U / ranks, (r + 1) * U / ranks): never empty since ranks <= U.
__host__ __device__ inline long long rank_first_unit(int r, int total_units, int ranks) {
    return (long long)r * total_units / ranks;
}
// the rank that owns unit x
__host__ __device__ inline int rank_of_unit(long long x, int total_units, int ranks) {
    return (int)(((x + 1) * ranks + total_units - 1) / total_units) - 1;
}

struct Piece {
    int tile;
    int blk0, blk1;      // 32-blocks of K
    int slot;            // index of this piece among the pieces of its tile, in K order
    int n_pieces;        // pieces of the tile
};

// Walks the pieces of one rank for one GEMM.
struct Walker {
    long long u, u1;
    int upt, nkb, total_units, ranks, rank;
    __host__ __device__ void start(int rank_, int total_units_, int ranks_, int units_per_tile, int nkb_) {
        rank = rank_; total_units = total_units_; ranks = ranks_; upt = units_per_tile; nkb = nkb_;
        if (rank >= ranks) { u = u1 = 0; return; }
        u = rank_first_unit(rank, total_units, ranks);
        u1 = rank_first_unit(rank + 1, total_units, ranks);
    }
    __host__ __device__ bool next(Piece& p) {
        if (u >= u1) return false;
        const int tile = (int)(u / upt);
        const int ku0 = (int)(u - (long long)tile * upt);
        const long long left = u1 - u;
        const int ku1 = (left < (long long)(upt - ku0)) ? ku0 + (int)left : upt;
        p.tile = tile;
        p.blk0 = ku0 * UNIT;
        p.blk1 = (ku1 * UNIT < nkb) ? ku1 * UNIT : nkb;
        const int first = rank_of_unit((long long)tile * upt, total_units, ranks);
        const int last = rank_of_unit((long long)(tile + 1) * upt - 1, total_units, ranks);
        p.slot = rank - first;
        p.n_pieces = last - first + 1;
        u += ku1 - ku0;
        return true;
    }
};

constexpr int OUT_BUFS = 2;

struct Smem {
    alignas(128) uint8_t packed[STAGES][SB * NT * kBlockBytes];
    alignas(128) uint16_t scales[STAGES][SB][NT];
    alignas(128) uint8_t b[2][B_BUF_BYTES];           // [block in chunk][row m < MP][t] x 16 bytes
    alignas(16) float asum8[2][ASUM_GROUPS][8];       // -8 * sum of a group's activations, per row
    alignas(16) float out[OUT_BUFS][8][NT];           // a finished piece's sums, consumers -> epilogue warp
    alignas(8) uint64_t full[STAGES];
    alignas(8) uint64_t empty[STAGES];
    alignas(8) uint64_t b_full[2];
    alignas(8) uint64_t b_empty[2];
    alignas(8) uint64_t out_full[OUT_BUFS];
    alignas(8) uint64_t out_empty[OUT_BUFS];
    int abort_flag;
    int last_cta;
};

__device__ __forceinline__ unsigned int ld_acquire_gpu_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Release / acquire read-modify-writes at GPU scope.  A release by one lane after __syncwarp()
// (or a CTA barrier) publishes the stores of every thread that synchronised with it; these
// replace __threadfence() + atomicAdd, whose sequentially-consistent fence took microseconds
// while the weight stream was saturating the memory system.
__device__ __forceinline__ void red_release_gpu_add(unsigned int* p, unsigned int v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int atom_acq_rel_gpu_add(unsigned int* p, unsigned int v) {
    unsigned int old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ void prefetch_l2(const void* p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// One ring stage of `nb` 32-blocks (whole scale groups), the straight-line code of
// twm::mma::gemv_kernel: per 32-block two 32-bit loads, one 128-bit load, ten integer
// operations, two MMAs; per scale group one scale per column and the -8 * sum(a) term.
template <int MP, int GSHIFT>
__device__ __forceinline__ void consume_stage(float (&tot)[4], uint32_t w_st, uint32_t s_st, uint32_t b_st, uint32_t a8_st,
                                              int nb, int g)
{
    constexpr int GB = 1 << GSHIFT;
    const float zero4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int r0 = 0; r0 < SB; r0 += GB) {
        if (r0 < nb) {
            float lo[4], hi[4];
#pragma unroll
            for (int j = 0; j < GB; ++j) {
                const int r = r0 + j;
                const uint32_t v0 = mma::lds32_at(w_st + r * (NT * kBlockBytes));          // column g, word t
                const uint32_t v1 = mma::lds32_at(w_st + r * (NT * kBlockBytes) + 128);    // column g + 8, word t
                uint4 xb = make_uint4(0, 0, 0, 0);
                if (MP == 8 || g < MP) xb = mma::lds128_at(b_st + r * (MP * 64));
                const uint32_t v0s = v0 >> 8, v1s = v1 >> 8;
                if (j == 0) {
                    mma::mma_m16n8k16(lo, v0 & 0x000F000Fu, v1 & 0x000F000Fu, v0s & 0x000F000Fu, v1s & 0x000F000Fu, xb.x, xb.y, zero4);
                    mma::mma_m16n8k16(hi, v0 & 0x00F000F0u, v1 & 0x00F000F0u, v0s & 0x00F000F0u, v1s & 0x00F000F0u, xb.z, xb.w, zero4);
                } else {
                    mma::mma_m16n8k16(lo, v0 & 0x000F000Fu, v1 & 0x000F000Fu, v0s & 0x000F000Fu, v1s & 0x000F000Fu, xb.x, xb.y, lo);
                    mma::mma_m16n8k16(hi, v0 & 0x00F000F0u, v1 & 0x00F000F0u, v0s & 0x00F000F0u, v1s & 0x00F000F0u, xb.z, xb.w, hi);
                }
            }
            const float s0 = f16_bits_to_f32(mma::lds16_at(s_st + (r0 >> GSHIFT) * (NT * 2)));
            const float s1 = f16_bits_to_f32(mma::lds16_at(s_st + (r0 >> GSHIFT) * (NT * 2) + 16));
            const float2 a8 = mma::lds64f_at(a8_st + (r0 >> GSHIFT) * 32);
            const float k20 = 1048576.0f;                     // 2^20
            tot[0] = fmaf(s0, fmaf(fmaf(lo[0], 16.0f, hi[0]), k20, a8.x), tot[0]);
            tot[1] = fmaf(s0, fmaf(fmaf(lo[1], 16.0f, hi[1]), k20, a8.y), tot[1]);
            tot[2] = fmaf(s1, fmaf(fmaf(lo[2], 16.0f, hi[2]), k20, a8.x), tot[2]);
            tot[3] = fmaf(s1, fmaf(fmaf(lo[3], 16.0f, hi[3]), k20, a8.y), tot[3]);
        }
    }
}

// Eight consecutive K of one activation row as eight f16 (the stager's unit of work).
// A_SILU_MUL computes silu(gate) * up exactly as the separate SwiGLU kernel does
// (g / (1 + expf(-g)) * u, rounded to f16; crates/kernels/src/ops.rs:966-977).
__device__ __forceinline__ uint4 combine_silu(const uint4 gt, const uint4 up) {
    const __half2* gh = reinterpret_cast<const __half2*>(&gt);
    const __half2* uh = reinterpret_cast<const __half2*>(&up);
    uint4 o;
    uint32_t* ow = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 gf = __half22float2(gh[j]), uf = __half22float2(uh[j]);
        const __half2 r = __floats2half2_rn(gf.x / (1.0f + expf(-gf.x)) * uf.x, gf.y / (1.0f + expf(-gf.y)) * uf.y);
        ow[j] = *reinterpret_cast<const uint32_t*>(&r);
    }
    return o;
}

__device__ __forceinline__ uint4 ldcg_u4(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint4 ldcg_8xf16(const __half* p, bool vec_ok) {
    if (vec_ok) return ldcg_u4(p);
    const unsigned short* a16 = reinterpret_cast<const unsigned short*>(p);
    uint4 x;
    x.x = __ldcg(a16 + 0) | ((uint32_t)__ldcg(a16 + 1) << 16); x.y = __ldcg(a16 + 2) | ((uint32_t)__ldcg(a16 + 3) << 16);
    x.z = __ldcg(a16 + 4) | ((uint32_t)__ldcg(a16 + 5) << 16); x.w = __ldcg(a16 + 6) | ((uint32_t)__ldcg(a16 + 7) << 16);
    return x;
}

// MP = activation rows staged (power of two >= the largest M of the chain, <= 8)
//
// Warp roles: 0-7 consumers (16 columns each, MMA), 8 producer (packed rows and scales by TMA),
// 9 stager (activations into fragment order, waits for the GEMM it depends on), 10 epilogue
// (takes a finished piece from shared memory: store / partial + tile counter / tile sum /
// completion counter).  The consumers never touch global memory and never wait for it.
template <int MP>
__global__ void __launch_bounds__(THREADS, CTAS_PER_SM)
chain_kernel(const Op* __restrict__ ops, int n_ops, State* __restrict__ st, unsigned int* __restrict__ done /* [n_ops] finished tiles per GEMM */)
{
    extern __shared__ __align__(128) uint8_t smem_raw[];
    Smem& sm = *reinterpret_cast<Smem*>(smem_raw);

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int P = gridDim.x;
    const int cta = blockIdx.x;
    constexpr int CHUNK_BLOCKS = B_BUF_BYTES / (64 * MP);    // 64, 32, 16, 8: multiples of SB and of a group
    static_assert(CHUNK_BLOCKS % SB == 0 && CHUNK_BLOCKS <= ASUM_GROUPS, "chunk geometry");

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], CONSUMER_WARPS); }
        for (int s = 0; s < 2; ++s) { mbar_init(&sm.b_full[s], 1); mbar_init(&sm.b_empty[s], CONSUMER_WARPS); }
        for (int s = 0; s < OUT_BUFS; ++s) { mbar_init(&sm.out_full[s], CONSUMER_WARPS); mbar_init(&sm.out_empty[s], 1); }
        sm.abort_flag = 0;
        sm.last_cta = 0;
        mbar_fence_init();
    }
    __syncthreads();
    volatile int* abort_flag = &sm.abort_flag;

    auto my_rank = [&](int rot) { int r = cta + rot; return r >= P ? r - P : r; };
    // bring the descriptor of a later GEMM towards the SM while the current one is being worked on
    auto prefetch_op = [&](int oi) {
        if (oi < n_ops && lane < (int)(sizeof(Op) / 128)) prefetch_l2(reinterpret_cast<const char*>(&ops[oi]) + lane * 128);
    };

    if (warp == CONSUMER_WARPS) {
        // --------------------------------------------- producer: packed rows + scale rows --
        // Runs ahead of the consumers through the whole list: it needs no result of any GEMM.
        uint32_t it = 0;
        bool ok = true;
        prefetch_op(1);
        for (int oi = 0; oi < n_ops && ok; ++oi) {
            prefetch_op(oi + 2);
            const Op& op = ops[oi];
            const int N = op.N, gshift = op.gshift;
            const uint8_t* packed = op.packed;
            const uint16_t* scales = op.scales;
            const bool use_maps = op.use_maps != 0;
            Walker w;
            w.start(my_rank(op.rot), op.total_units, op.ranks, op.units_per_tile, op.nkb);
            Piece pc;
            while (ok && w.next(pc)) {
                const int n0 = pc.tile * NT;
                const int cols = min(NT, N - n0);
                const bool scale_bulk_ok = ((cols & 7) == 0) && ((N & 7) == 0) &&
                                           ((reinterpret_cast<uintptr_t>(scales + n0) & 15) == 0);
                for (int bstart = pc.blk0; bstart < pc.blk1; bstart += SB, ++it) {
                    const int slot = it % STAGES;
                    const uint32_t use = it / STAGES;
                    if (use > 0) {
                        const bool got = mbar_wait_bounded(&sm.empty[slot], (use - 1) & 1, abort_flag);
                        if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
                    }
                    const int nb = min(SB, pc.blk1 - bstart);
                    const int srow_first = bstart >> gshift;
                    const int nrows = ((bstart + nb - 1) >> gshift) - srow_first + 1;
                    if (!scale_bulk_ok) {
                        for (int r = 0; r < nrows; ++r) {
                            const uint16_t* src = scales + (size_t)(srow_first + r) * N + n0;
                            for (int cidx = lane; cidx < cols; cidx += 32) sm.scales[slot][r][cidx] = src[cidx];
                        }
                        __syncwarp();
                    }
                    // a stage of 8 or 4 blocks is one tiled TMA load (128 columns; columns past N are
                    // zero-filled and still counted); anything else is copied row by row
                    const bool tiled = use_maps && (nb == SB || nb == UNIT);
                    uint32_t tx = tiled ? (uint32_t)nb * NT * kBlockBytes : (uint32_t)nb * cols * kBlockBytes;
                    if (scale_bulk_ok) tx += (uint32_t)nrows * cols * 2;
                    if (lane == 0) {
                        mbar_arrive_expect_tx(&sm.full[slot], tx);
                        if (tiled) tma_load_2d(&sm.packed[slot][0], nb == SB ? &op.map8 : &op.map4, n0 * 2, bstart, &sm.full[slot]);
                    }
                    __syncwarp();
                    if (!tiled && lane < nb) {
                        bulk_g2s(&sm.packed[slot][lane * NT * kBlockBytes],
                                 packed + ((size_t)(bstart + lane) * N + n0) * kBlockBytes,
                                 (uint32_t)cols * kBlockBytes, &sm.full[slot]);
                    } else if (scale_bulk_ok && lane >= 16 && lane - 16 < nrows) {
                        const int r = lane - 16;
                        bulk_g2s(&sm.scales[slot][r][0], scales + (size_t)(srow_first + r) * N + n0,
                                 (uint32_t)cols * 2, &sm.full[slot]);
                    }
                    __syncwarp();
                }
            }
        }
    } else if (warp == CONSUMER_WARPS + 1) {
        // ----------------------------------------------------------- activation stager --
        // Item = 8 consecutive K of one row, stored as the 16 bytes {k0,k4 | k2,k6 | k1,k5 | k3,k7}
        // (the B fragments of a block's two MMAs); the 4 << gshift lanes that hold one (scale
        // group, row) are consecutive, so the group's sum is a fixed-order shuffle reduction.
        uint32_t cs = 0;                       // chunks staged so far (buffer = cs & 1)
        bool ok = true;
        for (int oi = 0; oi < n_ops && ok; ++oi) {
            const Op& op = ops[oi];
            Walker w;
            w.start(my_rank(op.rot), op.total_units, op.ranks, op.units_per_tile, op.nkb);
            if (w.u >= w.u1) continue;         // nothing to do for this GEMM: nothing to wait for either
            const int gshift = op.gshift;
            const int gmask = (1 << gshift) - 1;
            const int M = op.M, K = op.K;
            const long lda = op.lda;
            const int a_kind = op.a_kind;
            const __half* A = reinterpret_cast<const __half*>(op.a);
            const bool vec_ok = ((reinterpret_cast<uintptr_t>(A) & 15) == 0) && ((lda & 7) == 0) && ((K & 7) == 0);
            {
                // Ask L2 for this CTA's activation ranges before waiting: harmless if the GEMM before
                // is still writing them (L2 is where its stores land), a saved DRAM trip if they
                // have been sitting in memory.
                Walker wp = w;
                Piece pp;
                while (wp.next(pp)) {
                    const int lines = ((pp.blk1 - pp.blk0) * kBlockK * 2 + 127) / 128;
                    for (int m = 0; m < M; ++m) {
                        const char* base = reinterpret_cast<const char*>(A + (size_t)m * lda + (size_t)pp.blk0 * kBlockK);
                        for (int l = lane; l < lines; l += 32) {
                            prefetch_l2(base + l * 128);
                            if (a_kind == A_SILU_MUL) prefetch_l2(base + (size_t)K * 2 + l * 128);
                        }
                    }
                }
            }
            // wait (bounded) until the GEMMs whose output this one reads have finished every tile
            for (int dj = op.wait_from; dj < oi && ok; ++dj) {
                const unsigned int want = (unsigned int)ops[dj].n_tiles;
                bool got = false;
                if (lane == 0) {
                    for (uint32_t i = 0; i < (1u << 22); ++i) {
                        if (ld_acquire_gpu_u32(&done[dj]) >= want) { got = true; break; }
                        if (i > 16) {
                            __nanosleep(32);
                            if ((i & 63) == 0 && (*abort_flag || ld_volatile_u32(&st->abort))) break;
                        }
                    }
                    if (!got) { *abort_flag = 1; atomicOr(&g_error_word, 2u); atomicExch(&st->abort, 1u); }
                }
                got = __shfl_sync(0xffffffffu, got ? 1 : 0, 0) != 0;
                if (!got) ok = false;
            }
            if (!ok) break;
            Piece pc;
            while (ok && w.next(pc)) {
                const int total_blocks = pc.blk1 - pc.blk0;
                const int n_chunks = (total_blocks + CHUNK_BLOCKS - 1) / CHUNK_BLOCKS;
                for (int chunk = 0; chunk < n_chunks && ok; ++chunk, ++cs) {
                    const int buf = cs & 1;
                    const uint32_t use = cs >> 1;
                    const int cb0 = chunk * CHUNK_BLOCKS;
                    const int cb = min(CHUNK_BLOCKS, total_blocks - cb0);
                    const int items = cb * MP * 4;                    // item = (((gi * MP) + m) << gshift | bj) * 4 + t
                    bool waited = false;
                    constexpr int PF = 8;
                    for (int base = 0; base < items && ok; base += 32 * PF) {
                        const int live = min(PF, (items - base + 31) >> 5);     // rounds of 32 items that hold anything (warp-uniform)
                        uint4 x[PF];
                        if (a_kind == A_SILU_MUL) {
#pragma unroll
                            for (int h = 0; h < 2; ++h) {             // two halves of PF / 2: gate and up of each item in flight together
                                uint4 gt[PF / 2], up[PF / 2];
#pragma unroll
                                for (int u = 0; u < PF / 2; ++u) {
                                    const int itx = base + (h * (PF / 2) + u) * 32 + lane;
                                    gt[u] = make_uint4(0, 0, 0, 0); up[u] = make_uint4(0, 0, 0, 0);
                                    if (h * (PF / 2) + u < live && itx < items) {
                                        const int tt = itx & 3, bj = (itx >> 2) & gmask, rest = itx >> (2 + gshift);
                                        const int m = rest % MP, bi = ((rest / MP) << gshift) + bj;
                                        if (m < M) {
                                            const size_t off = (size_t)m * lda + (size_t)(pc.blk0 + cb0 + bi) * kBlockK + tt * 8;
                                            gt[u] = ldcg_8xf16(A + off, vec_ok);
                                            up[u] = ldcg_8xf16(A + off + K, vec_ok);
                                        }
                                    }
                                }
#pragma unroll
                                for (int u = 0; u < PF / 2; ++u)
                                    if (h * (PF / 2) + u < live) x[h * (PF / 2) + u] = combine_silu(gt[u], up[u]);
                            }
                        } else {
#pragma unroll
                            for (int u = 0; u < PF; ++u) {
                                const int itx = base + u * 32 + lane;
                                x[u] = make_uint4(0, 0, 0, 0);
                                if (itx < items) {
                                    const int tt = itx & 3, bj = (itx >> 2) & gmask, rest = itx >> (2 + gshift);
                                    const int m = rest % MP, bi = ((rest / MP) << gshift) + bj;
                                    if (m < M) {
                                        const size_t off = (size_t)m * lda + (size_t)(pc.blk0 + cb0 + bi) * kBlockK + tt * 8;
                                        x[u] = ldcg_8xf16(A + off, vec_ok);
                                    }
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
                            const int itx = base + u * 32 + lane;
                            const int tt = itx & 3, bj = (itx >> 2) & gmask, rest = itx >> (2 + gshift);
                            const int m = rest % MP, gi = rest / MP;
                            float s = 0.0f;
                            if (itx < items) {
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
                            if (itx < items && (itx & ((4 << gshift) - 1)) == 0) sm.asum8[buf][gi][m] = -8.0f * s;
                        }
                    }
                    if (!ok) break;
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sm.b_full[buf]);
                }
            }
        }
    } else if (warp == CONSUMER_WARPS + 2) {
        // ------------------------------------------------------------------ epilogue --
        // Takes the finished pieces in schedule order.  Lane l owns columns 4l .. 4l+3 of the tile.
        uint32_t pcount = 0;
        bool ok = true;
        for (int oi = 0; oi < n_ops && ok; ++oi) {
            const Op& op = ops[oi];
            Walker w;
            w.start(my_rank(op.rot), op.total_units, op.ranks, op.units_per_tile, op.nkb);
            const int M = op.M, N = op.N;
            const long ldc = op.ldc;
            const bool c_is_f16 = op.c_is_f16 != 0, accumulate = op.accumulate != 0;
            Piece pc;
            while (ok && w.next(pc)) {
                const int ob = pcount % OUT_BUFS;
                const uint32_t use = pcount / OUT_BUFS;
                ++pcount;
                {
                    const bool got = mbar_wait_bounded(&sm.out_full[ob], use & 1, abort_flag);
                    if (!__all_sync(0xffffffffu, got)) { ok = false; break; }
                }
                float4 v[MP];
#pragma unroll
                for (int m = 0; m < MP; ++m) v[m] = *reinterpret_cast<const float4*>(&sm.out[ob][m][lane * 4]);
                __syncwarp();
                if (lane == 0) mbar_arrive(&sm.out_empty[ob]);       // the values are in registers: the consumers may reuse the buffer
                const int n0 = pc.tile * NT;
                const int ncol = n0 + lane * 4;
                auto store4 = [&](int m, const float4 val) {
                    const float e[4] = {val.x, val.y, val.z, val.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (ncol + j < N) {
                            const size_t off = (size_t)m * ldc + ncol + j;
                            float r = e[j];
                            if (c_is_f16) {
                                __half* cp = reinterpret_cast<__half*>(op.c);
                                if (accumulate) r += __half2float(__ushort_as_half(__ldcg(reinterpret_cast<const unsigned short*>(cp + off))));
                                cp[off] = __float2half_rn(r);
                            } else {
                                float* cp = reinterpret_cast<float*>(op.c);
                                if (accumulate) r += __ldcg(cp + off);
                                cp[off] = r;
                            }
                        }
                    }
                };
                bool finish = true;                                    // this CTA writes the tile to C
                if (pc.n_pieces > 1) {
                    float* part = op.partials + ((size_t)pc.tile * op.max_pieces) * (size_t)M * NT;
                    float* mine = part + (size_t)pc.slot * M * NT;
#pragma unroll
                    for (int m = 0; m < MP; ++m)
                        if (m < M) *reinterpret_cast<float4*>(mine + m * NT + lane * 4) = v[m];
                    __syncwarp();
                    unsigned int prev = 0;
                    if (lane == 0) prev = atom_acq_rel_gpu_add(&op.tile_counters[pc.tile], 1u);
                    prev = __shfl_sync(0xffffffffu, prev, 0);
                    finish = (prev == (unsigned)(pc.n_pieces - 1));
                    if (finish) {
                        // last to arrive: add the pieces in piece order, four loads in flight per row
#pragma unroll
                        for (int m = 0; m < MP; ++m) {
                            if (m < M) {
                                float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
                                const float4* src = reinterpret_cast<const float4*>(part + m * NT + lane * 4);
                                const size_t stride4 = (size_t)M * NT / 4;
                                int sp = 0;
                                for (; sp + 4 <= pc.n_pieces; sp += 4) {
                                    const float4 t0 = __ldcg(src + (size_t)(sp + 0) * stride4), t1 = __ldcg(src + (size_t)(sp + 1) * stride4);
                                    const float4 t2 = __ldcg(src + (size_t)(sp + 2) * stride4), t3 = __ldcg(src + (size_t)(sp + 3) * stride4);
                                    acc.x += t0.x; acc.y += t0.y; acc.z += t0.z; acc.w += t0.w;
                                    acc.x += t1.x; acc.y += t1.y; acc.z += t1.z; acc.w += t1.w;
                                    acc.x += t2.x; acc.y += t2.y; acc.z += t2.z; acc.w += t2.w;
                                    acc.x += t3.x; acc.y += t3.y; acc.z += t3.z; acc.w += t3.w;
                                }
                                for (; sp < pc.n_pieces; ++sp) {
                                    const float4 t0 = __ldcg(src + (size_t)sp * stride4);
                                    acc.x += t0.x; acc.y += t0.y; acc.z += t0.z; acc.w += t0.w;
                                }
                                v[m] = acc;
                            }
                        }
                    }
                }
                if (finish) {
#pragma unroll
                    for (int m = 0; m < MP; ++m)
                        if (m < M) store4(m, v[m]);
                    __syncwarp();
                    if (lane == 0) {
                        if (pc.n_pieces > 1) op.tile_counters[pc.tile] = 0u;     // nobody touches it again in this launch
                        red_release_gpu_add(&done[oi], 1u);                      // one more tile of this GEMM is in memory
                    }
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ consumers --
        const int g = lane >> 2;
        const int t = lane & 3;
        const int wcol = warp * 16;                       // a consumer warp's 16 columns inside the tile
        const uint32_t w_base = smem_u32(&sm.packed[0][0]) + wcol * kBlockBytes + lane * 4;
        const uint32_t s_base = smem_u32(&sm.scales[0][0][0]) + (wcol + g) * 2;
        const uint32_t b_base = smem_u32(&sm.b[0][0]) + (g * 4 + t) * 16;
        const uint32_t a8_base = smem_u32(&sm.asum8[0][0][0]) + t * 8;
        uint32_t it = 0, cs = 0, pcount = 0;
        bool ok = true;
        for (int oi = 0; oi < n_ops; ++oi) {
            const Op& op = ops[oi];
            Walker w;
            w.start(my_rank(op.rot), op.total_units, op.ranks, op.units_per_tile, op.nkb);
            const int gshift = op.gshift;
            Piece pc;
            while (w.next(pc)) {
                float tot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                const int total_blocks = pc.blk1 - pc.blk0;
                const int n_stages = (total_blocks + SB - 1) / SB;
                const int n_chunks = (total_blocks + CHUNK_BLOCKS - 1) / CHUNK_BLOCKS;
                for (int si = 0; si < n_stages; ++si, ++it) {
                    const int slot = it % STAGES;
                    const int rel0 = si * SB;
                    const int nb = min(SB, total_blocks - rel0);
                    const int chunk = rel0 / CHUNK_BLOCKS;
                    const uint32_t ccs = cs + chunk;
                    const int buf = ccs & 1;
                    const int bi0 = rel0 - chunk * CHUNK_BLOCKS;
                    if (ok && bi0 == 0) {
                        const bool got = mbar_wait_bounded(&sm.b_full[buf], (ccs >> 1) & 1, abort_flag);
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
                        const uint32_t a8_st = a8_base + (buf * ASUM_GROUPS + (bi0 >> gshift)) * 32;
                        if (gshift == 2) consume_stage<MP, 2>(tot, w_st, s_st, b_st, a8_st, nb, g);
                        else consume_stage<MP, 0>(tot, w_st, s_st, b_st, a8_st, nb, g);
                    }
                    __syncwarp();
                    if (lane == 0 && ok) {
                        mbar_arrive(&sm.empty[slot]);
                        const bool chunk_end = ((rel0 + SB) % CHUNK_BLOCKS == 0) || (si == n_stages - 1);
                        if (chunk_end) mbar_arrive(&sm.b_empty[buf]);
                    }
                }
                cs += n_chunks;
                // ---- the piece is done: leave its sums in shared memory for the epilogue warp ----
                // lane (g, t) holds C[m = 2t, 2t+1][column wcol + g] and the same rows for column + 8
                const int ob = pcount % OUT_BUFS;
                const uint32_t use = pcount / OUT_BUFS;
                ++pcount;
                if (ok && use > 0) {
                    const bool got = mbar_wait_bounded(&sm.out_empty[ob], (use - 1) & 1, abort_flag);
                    if (!__all_sync(0xffffffffu, got)) ok = false;
                }
                if (ok) {
                    const int cA = wcol + g, mA = 2 * t, mB = 2 * t + 1;
                    if (mA < MP) { sm.out[ob][mA][cA] = tot[0]; sm.out[ob][mA][cA + 8] = tot[2]; }
                    if (mB < MP) { sm.out[ob][mB][cA] = tot[1]; sm.out[ob][mB][cA + 8] = tot[3]; }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sm.out_full[ob]);
                }
            }
        }
    }

    // ------------------------------------------------------------------------ exit --
    // The last CTA to leave puts the completion counters back to zero for the next launch (and,
    // after an expired wait, the tile counters too: they may have been left mid-count).
    __syncthreads();
    if (tid == 0) {
        if (sm.abort_flag) atomicExch(&st->abort, 1u);
        const unsigned prev = atom_acq_rel_gpu_add(&st->exit_count, 1u);
        sm.last_cta = (prev == (unsigned)(P - 1)) ? 1 : 0;
    }
    __syncthreads();
    if (sm.last_cta) {
        for (int i = tid; i < n_ops; i += THREADS) done[i] = 0u;
        if (ld_volatile_u32(&st->abort)) {
            const unsigned int ntc = st->n_tile_counters;
            for (unsigned int i = tid; i < ntc; i += THREADS) st->all_tile_counters[i] = 0u;
        }
        __syncthreads();
        if (tid == 0) { st->abort = 0u; st->exit_count = 0u; }
    }
}

}  // namespace chain
}  // namespace twm
