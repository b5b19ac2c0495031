// Host launchers for the reference's own CUDA kernels (test infrastructure only).
//
// build_ref.py pulls the kernel source strings out of the reference tree at
// build time, unchanged, into a scratch file that this translation unit
// includes as REF_KERNELS_INC.  Nothing of the reference is stored in this
// repository: only the compiled library lands in oracle/_ref/.
//
// The launch geometry below follows the reference's Rust launchers:
//   gemm_tw_marlin_m1     crates/kernels/src/quantize.rs:1311-1357
//   quantize_q4_0         crates/kernels/src/quantize.rs:103-146 (one thread per 32-block, 256/CTA)
//   dequantize_q4_0       crates/kernels/src/quantize.rs:150-175
//   gemm_q4_0             crates/kernels/src/quantize.rs:1840-1844 (32x32 tiles)
//   dequant_q4_to_f16     crates/kernels/src/quantize.rs:600-606 (one thread per element)
//   batched_marlin_*      crates/kernels/src/moe_batched_marlin.rs:155-233 (256 threads, grid (ceil(n/256), top_k))
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include REF_KERNELS_INC

#define REF_CHECK() do { cudaError_t e_ = cudaGetLastError(); if (e_ != cudaSuccess) return (int)e_; } while (0)

extern "C" int twmref_gemm_tw_marlin_m1(float* c, const float* a, const unsigned char* packed,
                                        const unsigned short* scales, unsigned n, unsigned k,
                                        int force_splits, int* splits_used, void* stream_)
{
    cudaStream_t stream = (cudaStream_t)stream_;
    if (k % 32u) return -1;
    unsigned num_k_groups = k / 32u;
    unsigned threads = 256u;
    unsigned n_blocks = (n + threads - 1u) / threads;
    unsigned splits;
    if (force_splits > 0) {
        splits = (unsigned)force_splits;
    } else if (k < 2048u || n_blocks >= 128u) {
        splits = 1u;
    } else {
        unsigned max_splits = num_k_groups / 8u; if (max_splits < 1u) max_splits = 1u;
        splits = (256u + n_blocks - 1u) / n_blocks;
        if (splits < 1u) splits = 1u;
        if (splits > max_splits) splits = max_splits;
    }
    unsigned kbps = (num_k_groups + splits - 1u) / splits;
    if (splits_used) *splits_used = (int)splits;
    dim3 grid(n_blocks, splits, 1), block(threads, 1, 1);
    if (splits == 1u) {
        warp_gemm_tw_marlin_m1_direct<<<grid, block, 0, stream>>>(c, a, packed, scales, (int)k, (int)n,
                                                                 (int)num_k_groups, (int)kbps);
    } else {
        cudaError_t e = cudaMemsetAsync(c, 0, sizeof(float) * n, stream);
        if (e != cudaSuccess) return (int)e;
        warp_gemm_tw_marlin_m1<<<grid, block, 0, stream>>>(c, a, packed, scales, (int)k, (int)n,
                                                          (int)num_k_groups, (int)kbps);
    }
    REF_CHECK();
    return 0;
}

extern "C" int twmref_quantize_q4_0(unsigned char* out, const float* in, unsigned n, void* stream_)
{
    unsigned num_blocks = n / 32u;
    unsigned grid = (num_blocks + 255u) / 256u;
    warp_quantize_q4_0<<<grid, 256, 0, (cudaStream_t)stream_>>>(out, in, n, num_blocks);
    REF_CHECK();
    return 0;
}

extern "C" int twmref_dequantize_q4_0(float* out, const unsigned char* in, unsigned n, void* stream_)
{
    unsigned num_blocks = n / 32u;
    unsigned grid = (num_blocks + 255u) / 256u;
    warp_dequantize_q4_0<<<grid, 256, 0, (cudaStream_t)stream_>>>(out, in, n, num_blocks);
    REF_CHECK();
    return 0;
}

extern "C" int twmref_gemm_q4_0(float* c, const float* a, const unsigned char* b_quant, unsigned m,
                                unsigned n, unsigned k, void* stream_)
{
    dim3 grid((n + 31u) / 32u, (m + 31u) / 32u, 1), block(32, 32, 1);
    warp_gemm_q4_0<<<grid, block, 0, (cudaStream_t)stream_>>>(c, a, b_quant, m, n, k, k / 32u);
    REF_CHECK();
    return 0;
}

extern "C" int twmref_dequant_q4_to_f16(void* out, const unsigned char* b_quant, unsigned k,
                                        unsigned n, void* stream_)
{
    unsigned total = k * n;
    warp_dequant_q4_to_f16<<<(total + 255u) / 256u, 256, 0, (cudaStream_t)stream_>>>(
        (__half*)out, b_quant, k, n, k / 32u);
    REF_CHECK();
    return 0;
}

extern "C" int twmref_batched_marlin_gate_up(float* c, const float* a, const unsigned char* packed_base,
                                             const unsigned short* scales_base, const float* topk_ids,
                                             unsigned packed_bytes_per_expert, unsigned scales_per_expert, unsigned n,
                                             unsigned k, unsigned top_k, void* stream_)
{
    if (k % 32u) return -1;
    dim3 grid((n + 255u) / 256u, top_k, 1), block(256, 1, 1);
    batched_marlin_gate_up<<<grid, block, 0, (cudaStream_t)stream_>>>(c, a, packed_base, scales_base, topk_ids,
                                                                      packed_bytes_per_expert, scales_per_expert, (int)k,
                                                                      (int)n, (int)(k / 32u));
    REF_CHECK();
    return 0;
}

extern "C" int twmref_batched_marlin_down_axpy(float* acc, const float* a_all, const unsigned char* packed_base,
                                               const unsigned short* scales_base, const float* topk_ids,
                                               const float* topk_weights, unsigned packed_bytes_per_expert,
                                               unsigned scales_per_expert, unsigned n, unsigned k, unsigned top_k,
                                               void* stream_)
{
    if (k % 32u) return -1;
    dim3 grid((n + 255u) / 256u, top_k, 1), block(256, 1, 1);
    batched_marlin_down_axpy<<<grid, block, 0, (cudaStream_t)stream_>>>(acc, a_all, packed_base, scales_base, topk_ids,
                                                                        topk_weights, packed_bytes_per_expert,
                                                                        scales_per_expert, (int)k, (int)n, (int)(k / 32u),
                                                                        (int)k);
    REF_CHECK();
    return 0;
}

extern "C" int twmref_batched_marlin_split_geglu(float* out, const float* gate_up, unsigned moe_dim, unsigned top_k,
                                                 void* stream_)
{
    dim3 grid((moe_dim + 255u) / 256u, top_k, 1), block(256, 1, 1);
    batched_marlin_split_geglu<<<grid, block, 0, (cudaStream_t)stream_>>>(out, gate_up, (int)moe_dim);
    REF_CHECK();
    return 0;
}
