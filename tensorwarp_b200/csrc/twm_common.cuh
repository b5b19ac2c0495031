// twm_common.cuh — PTX wrappers and shared definitions for the sm_100a kernels.
#pragma once

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

// ------------------------------------------- programmatic dependent launch --
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void pdl_wait_prior_grids() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
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
    int accumulate;
    const uint32_t* packed_offsets;
    const uint32_t* scales_offsets;
    int expert_idx;
};

}  // namespace twm
