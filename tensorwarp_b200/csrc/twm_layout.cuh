// twm_layout.cuh — load-time kernels on the TW-Marlin tensors: quantise + pack,
// dequantise.  Integer/byte results are bit-identical to the reference's CPU
// quantiser (crates/loader/src/gemma_moe_q4.rs:218-254) and decode
// (crates/kernels/src/quantize.rs:3642-3659).
#pragma once

#include "twm_common.cuh"

namespace twm {
namespace layout {

// One thread per (scale group, column).  [K,N] input: consecutive threads read
// consecutive columns, so every k step is one coalesced row segment.  [N,K]
// input: a thread walks its own contiguous run of `GROUP` floats with 128-bit
// loads.  The arithmetic is written exactly as the reference writes it:
// amax -> scale = amax/7 -> inv = 7/amax -> q = clamp(roundf(v*inv)+8, 0, 15);
// the stored scale is the f16 rounding of the f32 scale that quantised.
template <int GROUP>
__global__ void __launch_bounds__(128)
quantize_pack_kernel(const float* __restrict__ w, int w_is_nk, int K, int N,
                     uint8_t* __restrict__ packed, uint16_t* __restrict__ scales)
{
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int g = blockIdx.y;
    if (n >= N) return;
    float vals[GROUP];
    const size_t k0 = (size_t)g * GROUP;
    if (w_is_nk) {
        const float* src = w + (size_t)n * K + k0;
        if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
#pragma unroll
            for (int i = 0; i < GROUP; i += 4) {
                const float4 t = *reinterpret_cast<const float4*>(src + i);
                vals[i] = t.x; vals[i + 1] = t.y; vals[i + 2] = t.z; vals[i + 3] = t.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < GROUP; ++i) vals[i] = src[i];
        }
    } else {
#pragma unroll
        for (int i = 0; i < GROUP; ++i) vals[i] = w[(k0 + i) * (size_t)N + n];
    }
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < GROUP; ++i) {
        const float a = fabsf(vals[i]);
        if (a > amax) amax = a;
    }
    const float scale = __fdiv_rn(amax, 7.0f);
    const float inv = (scale != 0.0f) ? __fdiv_rn(7.0f, amax) : 0.0f;
    scales[(size_t)g * N + n] = __half_as_ushort(__float2half_rn(scale));
#pragma unroll
    for (int b = 0; b < GROUP / 32; ++b) {
        uint32_t words[4];
#pragma unroll
        for (int wd = 0; wd < 4; ++wd) {
            uint32_t word = 0;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                int q = (int)roundf(__fmul_rn(vals[b * 32 + wd * 8 + j], inv)) + 8;
                q = q < 0 ? 0 : (q > 15 ? 15 : q);
                word |= (uint32_t)q << (4 * j);
            }
            words[wd] = word;
        }
        const size_t blk = (size_t)g * (GROUP / 32) + b;
        *reinterpret_cast<uint4*>(packed + (blk * N + n) * kBlockBytes) =
            make_uint4(words[0], words[1], words[2], words[3]);
    }
}

// One thread per (32-block, column); 32 outputs each, coalesced along N.
template <typename OutT>
__global__ void __launch_bounds__(128)
dequant_kernel(const uint8_t* __restrict__ packed, const uint16_t* __restrict__ scales,
               OutT* __restrict__ out, int K, int N, int group)
{
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int b = blockIdx.y;
    if (n >= N) return;
    const uint4 v = *reinterpret_cast<const uint4*>(packed + ((size_t)b * N + n) * kBlockBytes);
    const float s = f16_bits_to_f32(scales[(size_t)((b * kBlockK) / group) * N + n]);
    const uint32_t words[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int wd = 0; wd < 4; ++wd) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int q = (int)((words[wd] >> (4 * j)) & 0xFu) - 8;
            const float val = __fmul_rn(s, (float)q);
            const size_t off = ((size_t)b * kBlockK + wd * 8 + j) * N + n;
            if constexpr (sizeof(OutT) == 2) out[off] = __float2half_rn(val);
            else out[off] = val;
        }
    }
}

// Column-major 20-byte Q4_0 blocks ([f32 scale][16 nibble bytes], block (col, g) at byte
// (col * nkb + g) * 20) -> TW-Marlin packed [g][col][16] and f16 scales [g][col]; replaces the host
// loop of reorder_to_tw_marlin (crates/kernels/src/quantize.rs:912-956: download, permute on the
// CPU, upload).  A 32 x 32 tile of blocks goes through shared memory so that the reads run along
// g (contiguous in the source) and the writes along col (contiguous in the destination).
__global__ void __launch_bounds__(1024)
reorder_q4_0_kernel(const uint32_t* __restrict__ src /* 5 words per block */, int nkb, int N,
                    uint8_t* __restrict__ packed, uint16_t* __restrict__ scales)
{
    __shared__ uint32_t tile[32][32][5 + 1];        // [col][g][word], padded against bank conflicts
    const int g0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
    {
        const int g = g0 + threadIdx.x, col = c0 + threadIdx.y;
        if (g < nkb && col < N) {
            const uint32_t* blk = src + ((size_t)col * nkb + g) * 5;
#pragma unroll
            for (int w = 0; w < 5; ++w) tile[threadIdx.y][threadIdx.x][w] = blk[w];
        }
    }
    __syncthreads();
    {
        const int col = c0 + threadIdx.x, g = g0 + threadIdx.y;
        if (g < nkb && col < N) {
            const uint32_t* t = tile[threadIdx.x][threadIdx.y];
            scales[(size_t)g * N + col] = __half_as_ushort(__float2half_rn(__uint_as_float(t[0])));
            *reinterpret_cast<uint4*>(packed + ((size_t)g * N + col) * kBlockBytes) = make_uint4(t[1], t[2], t[3], t[4]);
        }
    }
}

}  // namespace layout
}  // namespace twm
