// twm_common.cuh — PTX wrappers and shared definitions for the sm_100a kernels.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/twmarlin.h"

namespace twm {

constexpr int kBlockK = 32;        // K values per packed 16-byte block
constexpr int kBlockBytes = 16;

// Device-side error word: bit 0 = an mbarrier wait ran out, bit 1 = a split-K
// arrival wait ran out, bit 2 = a peer-flag wait ran out.  Sticky until read.
// The library is one translation unit, so this definition is the only one.
__device__ unsigned int g_error_word = 0;

// ---------------------------------------------------------------- mbarrier --
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
    // make the initialised barriers visible to the async proxy (TMA unit)
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when the limit ran out; the caller must then
// stop using the data that barrier guards.  `abort_flag` (shared memory) lets
// one expired wait shorten every later wait in the CTA.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity,
                                                  volatile int* abort_flag) {
    // ~2^22 polls with back-off: of the order of a second, far beyond any real
    // memory latency, short enough that a broken pipeline ends by itself.
    for (uint32_t i = 0; i < (1u << 22); ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) {
            __nanosleep(i > 4096 ? 256 : 32);
            if (*abort_flag) break;
        }
    }
    *abort_flag = 1;
    atomicOr(&g_error_word, 1u);
    return false;
}

// ------------------------------------------------------------ bulk copies --
// 1-D bulk copy global -> shared of this CTA, completion counted on `bar`.
// Source, destination and size must be multiples of 16 bytes.  No multicast.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes,
                                         uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(smem_dst)), "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Ask the memory system to bring [src, src + bytes) into L2 (bytes a multiple of 16, src 16-byte aligned).
// Nothing waits for it and nothing depends on it.
__device__ __forceinline__ void l2_prefetch_bulk(const void* src, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// The weights the NEXT GEMM on the stream starts with (twm_gemm_args.next): `regions` runs of `bytes`
// bytes, `stride` apart, of its packed array and of its scale rows.  The CTAs of this launch share them
// out in 4 KB pieces; the producer warp asks for its pieces once its own last load is on its way.
struct NextHead {
    const uint8_t* packed;       // null = none
    const uint16_t* scales;
    unsigned long long packed_stride, scales_stride;   // bytes
    unsigned int packed_bytes, scales_bytes;           // per region, multiples of 16
    unsigned int regions;
};

__device__ __forceinline__ void prefetch_next_head(const NextHead& nh, unsigned cta, unsigned n_ctas, int lane) {
    if (nh.packed == nullptr) return;
    constexpr unsigned PIECE = 4096;
    auto run = [&](const uint8_t* base, unsigned long long stride, unsigned bytes) {
        const unsigned per = (bytes + PIECE - 1) / PIECE;
        const unsigned total = per * nh.regions;
        for (unsigned i = cta + (unsigned)lane * n_ctas; i < total; i += 32u * n_ctas) {
            const unsigned r = i / per, o = (i - r * per) * PIECE;
            l2_prefetch_bulk(base + (size_t)r * stride + o, min(PIECE, bytes - o));
        }
    };
    run(nh.packed, nh.packed_stride, nh.packed_bytes);
    if (nh.scales != nullptr && nh.scales_bytes != 0)
        run(reinterpret_cast<const uint8_t*>(nh.scales), nh.scales_stride, nh.scales_bytes);
}

// 2-D tiled TMA load (tensor map in kernel-parameter space), completion counted on `bar`.
// x is the innermost coordinate in elements of the map's data type; x * element size must
// be a multiple of 16 bytes.  No multicast.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}

// ------------------------------------------- programmatic dependent launch --
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait_prior_grids() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ------------------------------------------------- thread-block clusters --
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// address of the same shared-memory location in another CTA of the cluster
__device__ __forceinline__ uint32_t mapa_shared(uint32_t local_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void st_cluster_f32(uint32_t cluster_addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}
// hardware barrier over every thread of every CTA of the cluster (like __syncthreads, not a spin)
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// --------------------------------------------- system-scope flags (peers) --
__device__ __forceinline__ void st_release_sys_u32(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_u32(unsigned int* p, unsigned int v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
__device__ __forceinline__ unsigned int ld_acquire_sys_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned int ld_volatile_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// ----------------------------------------------------------- named barrier --
__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// ---------------------------------------------------------------- helpers --
__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) {
    float f;
    asm("cvt.f32.f16 %0, %1;" : "=f"(f) : "h"(h));
    return f;
}

__device__ __forceinline__ uint4 lds128(const void* p) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(smem_u32(p)));
    return v;
}

__device__ __forceinline__ float ld_cg_f32(const float* p) {
    float v;
    asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

// Launch parameters shared by the GEMM kernels.
struct GemmParams {
    int M, N, K, group;          // group = scale group size (32 or 128)
    int nkb;                     // K / 32
    int a_is_f16, c_is_f16;
    const void* a;
    long lda;
    const uint8_t* packed;
    const uint16_t* scales;
    void* c;
    long ldc;
    float* ws_partials;          // [splits][M][N] fp32, split-K only
    unsigned int* ws_counters;   // [n_tiles], zero between launches
    int splits;
    int blocks_per_split;
    int cluster_reduce;          // 1: the K slices of a tile form a thread-block cluster and add up in its leader's shared memory
    int accumulate;
    int no_wait;                 // the caller vouches that nothing this launch touches depends on the launch before it
    const uint32_t* packed_offsets;
    const uint32_t* scales_offsets;
    int expert_idx;
    // Batched expert GEMVs (mixture of experts): n_experts > 0 makes grid z the top-k slot.  Slot z
    // multiplies the weights of expert (int)expert_ids[z] (read on the device) with its own input
    // row (a + z * a_expert_stride; stride 0 = one shared row).  Without expert_weights every slot
    // stores its own output row (c + z * c_expert_stride); with them the slots' results are
    // multiplied by expert_weights[z] and added up, in slot order, into the one output row.
    int n_experts;
    int reduce_slices;           // K slices x slots that add up into one output tile (1 = none)
    int a_kind;                  // 0: a is f16; 1: SwiGLU, 2: tanh-GEGLU of a row [gate | up] (up at column K)
    NextHead next;               // what to pull into L2 for the GEMM after this one
    const float* expert_ids;
    const float* expert_weights;
    size_t packed_expert_stride; // bytes
    size_t scales_expert_stride; // elements
    long a_expert_stride, c_expert_stride;   // elements
    // Row-parallel output pushed straight to every tensor-parallel peer (one-shot all-reduce,
    // first half).  n_peers = 0: normal store to c.  Otherwise every stored value goes, as FP32,
    // to slot `peer_rank` of the current buffer set in each peer's receive buffer
    // (peer_data[s] + ((set * n_peers + peer_rank) * peer_slot_elems) + m * ldc + n), and the last
    // CTA of the grid publishes the peers' flags.  The state words live in this rank's memory.
    int n_peers;
    int peer_rank;
    long peer_slot_elems;
    float* peer_data[8];
    unsigned int* peer_flags[8];     // [set][source rank] words, 8 words apart
    unsigned int* comm_state;        // [0] operation sequence number, [1] CTAs done, [2] consumer CTAs done
    // Tensor map over `packed` seen as u64 [K/32][2N]: one TMA instruction brings a whole
    // ring stage (box = 256 u64 x map_rows rows = 128 columns x map_rows 32-blocks).
    int map_rows;                // 0 = no map (1-D bulk copies per row instead)
    alignas(64) CUtensorMap packed_map;
    // tcgen05 kernel: tensor map over the launch's permuted activations, f16 [K/8][rows][8]
    alignas(64) CUtensorMap act_map;
    // streaming kernel from nine rows on: the pre-pass's B fragments [K/32][rows16][4][16 B] and group sums [K/group][rows16]
    const uint8_t* rows_b;
    const float* rows_asum;
};

// ---- row-parallel output pushed to the tensor-parallel peers (GemmParams::n_peers != 0) ----
// One value of the FP32 result, element `off` of the [M, ldc] output: a plain store into every
// peer's receive slot for operation `seq` (each peer's own memory; this rank's own slot included).
__device__ __forceinline__ void comm_store(const GemmParams& p, unsigned int seq, size_t off, float v)
{
    const size_t slot = ((size_t)(seq & 1u) * p.n_peers + p.peer_rank) * p.peer_slot_elems + off;
    for (int s = 0; s < p.n_peers; ++s) p.peer_data[s][slot] = v;
}

// After a CTA's stores (if any): hand them to the grid's last storing CTA and, there, tell every
// peer that this rank's partial for operation `seq` is complete.  Called by ONE thread of each
// storing CTA after a CTA-wide barrier: the barrier orders the CTA's stores before this thread and
// its fence is cumulative over them (a fence by every thread would cost a link round trip each).
// The CTAs hand over at GPU scope (fence + relaxed atomic on this GPU's counter; relaxed atomic +
// fence on the other side); the last CTA's fence, at system scope, is also the release for its
// flag stores, which then go out back to back: a st.release per peer would wait for the previous
// flag's acknowledgement each time, one link round trip per peer.
__device__ __forceinline__ void comm_cta_done(const GemmParams& p, unsigned int seq, unsigned int total)
{
    fence_acq_rel_gpu();
    if (atomicAdd(&p.comm_state[1], 1u) == total - 1) {
        fence_acq_rel_sys();
        atomicExch(&p.comm_state[1], 0u);
        for (int s = 0; s < p.n_peers; ++s)
            st_relaxed_sys_u32(p.peer_flags[s] + ((seq & 1u) * p.n_peers + p.peer_rank) * 8, seq + 1u);
    }
}

}  // namespace twm
