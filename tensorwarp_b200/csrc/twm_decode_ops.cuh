// twm_decode_ops.cuh — the small kernels either side of the W4A16 GEMMs in one decode step:
// embedding row, RMSNorm, bias + RoPE + KV append, split-KV decode attention, SwiGLU,
// FP16 LM head, arg-max.  They exist so that a whole decode step can be captured in one CUDA
// graph with device-side position/length buffers; the arithmetic follows the reference's
// kernels of the same role (cited at each kernel), with FP16 storage where the benchmark
// configuration states FP16 (KV cache, LM head, GEMM inputs) and FP32 for the residual stream.
//
// All kernels take part in programmatic dependent launch: they let their dependents start
// early and wait for the preceding kernel before touching memory.
#pragma once

#include "twm_common.cuh"

namespace twm {
namespace ops {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// x[row][h] (f32) = table[token[row]][h] (f16).  Reference: warp_embedding,
// crates/kernels/src/sampling.rs:16-32 (f32 table there).
__global__ void __launch_bounds__(256)
embed_kernel(float* __restrict__ x, const __half* __restrict__ table, const int* __restrict__ tokens, int hidden)
{
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const int row = blockIdx.y;
    const size_t tok = (size_t)tokens[row];
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < hidden; i += gridDim.x * blockDim.x)
        x[(size_t)row * hidden + i] = __half2float(table[tok * hidden + i]);
}

// Sum of squares of a row in ONE fixed order that every kernel below follows, so that a row
// normalised by the one-CTA kernel and the same row normalised by the multi-CTA all-reduce kernel
// come out with the same bits: the row is cut into segments of 256 float4; inside a segment
// thread t takes vector t with a four-term fused chain, the 32 lanes of a warp add up by an
// xor tree, the eight warps are added in warp order; the segments are added in segment order.
constexpr int RMS_SEG_VECS = 256;     // float4 per segment = threads per CTA
__device__ __forceinline__ float sumsq4(const float4 v) {
    return fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w)));
}

// y = f16(x * rsqrt(mean(x^2) + eps) * gamma), one CTA per row.  Reference: warp_rmsnorm,
// crates/kernels/src/ops.rs:302-336 (one warp per row there; here 256 threads and the fixed-order
// segment sum above).  With `add` the kernel first does x += add (and stops there when y is null).
constexpr int RMS_MAX_VEC = 8;        // float4 per thread held in registers: rows up to 8192 floats
__global__ void __launch_bounds__(256)
rmsnorm_kernel(__half* __restrict__ y, float* __restrict__ x, const float* __restrict__ add,
               const float* __restrict__ gamma, int hidden, float eps)
{
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    constexpr int RMS_MAX_SEGS = 16;                  // rows up to 16384 floats in the fixed order; longer rows: plain pass
    __shared__ float partial[RMS_MAX_SEGS][8];
    const int row = blockIdx.x;
    float* xr = x + (size_t)row * hidden;
    const float* ar = add ? add + (size_t)row * hidden : nullptr;
    const bool vec = ((hidden & 3) == 0) && (hidden <= 256 * 4 * RMS_MAX_SEGS) &&
                     ((reinterpret_cast<uintptr_t>(xr) & 15) == 0) && (!ar || (reinterpret_cast<uintptr_t>(ar) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(gamma) & 15) == 0);
    if (vec) {
        // the whole row sits in registers: every load is issued before the first use
        const int nvec = hidden >> 2;
        const int nseg = (nvec + RMS_SEG_VECS - 1) / RMS_SEG_VECS;
        float4 v[RMS_MAX_VEC];
#pragma unroll
        for (int j = 0; j < RMS_MAX_VEC; ++j) {
            const int i = threadIdx.x + j * 256;
            v[j] = (i < nvec) ? reinterpret_cast<const float4*>(xr)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (ar) {
#pragma unroll
            for (int j = 0; j < RMS_MAX_VEC; ++j) {
                const int i = threadIdx.x + j * 256;
                if (i < nvec) {
                    const float4 a = reinterpret_cast<const float4*>(ar)[i];
                    v[j].x += a.x; v[j].y += a.y; v[j].z += a.z; v[j].w += a.w;
                    reinterpret_cast<float4*>(xr)[i] = v[j];
                }
            }
            for (int j = RMS_MAX_VEC; j < nseg; ++j) {        // segments past the registers
                const int i = threadIdx.x + j * 256;
                if (i < nvec) {
                    float4 t = reinterpret_cast<const float4*>(xr)[i];
                    const float4 a = reinterpret_cast<const float4*>(ar)[i];
                    t.x += a.x; t.y += a.y; t.z += a.z; t.w += a.w;
                    reinterpret_cast<float4*>(xr)[i] = t;
                }
            }
            if (y == nullptr) return;
        }
#pragma unroll
        for (int j = 0; j < RMS_MAX_VEC; ++j) {
            if (j < nseg) {                                   // CTA-uniform
                const float ss = warp_sum(sumsq4(v[j]));
                if ((threadIdx.x & 31) == 0) partial[j][threadIdx.x >> 5] = ss;
            }
        }
        for (int j = RMS_MAX_VEC; j < nseg; ++j) {
            const int i = threadIdx.x + j * 256;              // each thread re-reads what it wrote itself
            const float4 t = (i < nvec) ? reinterpret_cast<const float4*>(xr)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            const float ss = warp_sum(sumsq4(t));
            if ((threadIdx.x & 31) == 0) partial[j][threadIdx.x >> 5] = ss;
        }
        __syncthreads();
        float tot = 0.0f;
        for (int j = 0; j < nseg; ++j) {
            float sj = 0.0f;
#pragma unroll
            for (int w = 0; w < 8; ++w) sj += partial[j][w];
            tot += sj;
        }
        const float rms = rsqrtf(tot / (float)hidden + eps);
        __half* yr = y + (size_t)row * hidden;
#pragma unroll
        for (int j = 0; j < RMS_MAX_VEC; ++j) {
            const int i = threadIdx.x + j * 256;
            if (i < nvec) {
                const float4 gm = reinterpret_cast<const float4*>(gamma)[i];
                const __half2 lo = __floats2half2_rn(v[j].x * rms * gm.x, v[j].y * rms * gm.y);
                const __half2 hi = __floats2half2_rn(v[j].z * rms * gm.z, v[j].w * rms * gm.w);
                uint2 o;
                o.x = *reinterpret_cast<const uint32_t*>(&lo);
                o.y = *reinterpret_cast<const uint32_t*>(&hi);
                reinterpret_cast<uint2*>(yr)[i] = o;
            }
        }
        for (int j = RMS_MAX_VEC; j < nseg; ++j) {
            const int i = threadIdx.x + j * 256;
            if (i < nvec) {
                const float4 t = reinterpret_cast<const float4*>(xr)[i];
                const float4 gm = reinterpret_cast<const float4*>(gamma)[i];
                const __half2 lo = __floats2half2_rn(t.x * rms * gm.x, t.y * rms * gm.y);
                const __half2 hi = __floats2half2_rn(t.z * rms * gm.z, t.w * rms * gm.w);
                uint2 o;
                o.x = *reinterpret_cast<const uint32_t*>(&lo);
                o.y = *reinterpret_cast<const uint32_t*>(&hi);
                reinterpret_cast<uint2*>(yr)[i] = o;
            }
        }
        return;
    }
    // rows longer than 16384 floats, or not 16-byte aligned: a plain strided pass
    float ss = 0.0f;
    if (ar != nullptr) {
        // x += add first (fused_residual_rmsnorm, ops.rs:928-962): the all-reduced output of a
        // row-parallel GEMM joins the residual stream here
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) { const float t = xr[i] + ar[i]; xr[i] = t; ss = fmaf(t, t, ss); }
        if (y == nullptr) return;
    } else {
        for (int i = threadIdx.x; i < hidden; i += blockDim.x) { const float t = xr[i]; ss = fmaf(t, t, ss); }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) partial[0][threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += partial[0][w];
    const float rms = rsqrtf(tot / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
        y[(size_t)row * hidden + i] = __float2half_rn(xr[i] * rms * gamma[i]);
}

// One-shot all-reduce, second half, fused with the residual add and the RMSNorm that follow a
// row-parallel GEMM: wait (bounded) until every rank's partial for the current operation has
// arrived in THIS GPU's receive buffer (the GEMM epilogues of all ranks stored them there over
// NVLink), add the slots in rank order (every rank gets the same bits), x += sum, y = norm(x).
// A row is shared by the CTAs of one thread-block cluster (grid x), one 256-vector segment per
// CTA and pass; the segments' sums of squares meet in every CTA's shared memory (distributed
// shared memory stores, one cluster barrier) and are added in segment order, which is the order
// rmsnorm_kernel uses.  The last CTA of the grid advances the operation sequence number.
// The reference sums partial outputs on the host (crates/kernels/src/multi_gpu.rs:329-366).
constexpr int ARN_THREADS = 256;
constexpr int ARN_MAX_SEGS = 16;        // rows up to 16384 floats
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__global__ void __launch_bounds__(ARN_THREADS)
allreduce_add_rmsnorm_kernel(__half* __restrict__ y, float* __restrict__ x, const float* __restrict__ recv,
                             const unsigned int* __restrict__ flags, unsigned int* __restrict__ state,
                             const float* __restrict__ gamma, int hidden, float eps, int n_ranks, long slot_elems,
                             unsigned long long wait_ns)
{
    pdl_launch_dependents();
    // every CTA of the cluster has started once it has arrived here: only then may the others
    // store into its shared memory
    asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");
    pdl_wait_prior_grids();
    __shared__ float partial[8];
    __shared__ float segtot[ARN_MAX_SEGS];
    __shared__ int s_ok;
    const int row = blockIdx.y;
    const int ncta = gridDim.x;                      // = cluster size
    const int crank = (int)cluster_ctarank();
    const unsigned int seq = ld_volatile_u32(state);
    const unsigned int set = seq & 1u;
    if (threadIdx.x == 0) s_ok = 1;
    __syncthreads();
    if (threadIdx.x < n_ranks) {
        // bounded by the wall clock (wait_ns) and, should the clock misbehave, by a poll count;
        // then the error word is set and the step's result is void
        const unsigned int* f = flags + (set * n_ranks + threadIdx.x) * 8;
        const unsigned long long t0 = globaltimer_ns();
        bool got = false;
        for (unsigned int i = 0; i < (1u << 26) && !got; ++i) {
            got = ld_acquire_sys_u32(f) == seq + 1u;
            if (!got && i > 64) {
                __nanosleep(128);
                if ((i & 15) == 0 && globaltimer_ns() - t0 > wait_ns) break;
            }
        }
        if (!got) { s_ok = 0; atomicOr(&g_error_word, 4u); }
    }
    __syncthreads();
    const bool okk = s_ok != 0;
    float* xr = x + (size_t)row * hidden;
    const float* base = recv + (size_t)set * n_ranks * slot_elems + (size_t)row * hidden;
    const int nvec = hidden >> 2;                    // hidden is a multiple of 4 (checked by the host)
    const int nseg = (nvec + RMS_SEG_VECS - 1) / RMS_SEG_VECS;
    constexpr int KEEP = 2;                          // segments per CTA (the host launches nseg CTAs up to 8, then 8)
    float4 keep[KEEP];
    asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
#pragma unroll
    for (int kept = 0; kept < KEEP; ++kept) {
        const int seg = crank + kept * ncta;
        if (seg >= nseg) break;                      // CTA-uniform
        const int i = seg * RMS_SEG_VECS + threadIdx.x;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (okk && i < nvec) {
            float4 acc = __ldcg(reinterpret_cast<const float4*>(base) + i);
            for (int r = 1; r < n_ranks; ++r) {
                const float4 t = __ldcg(reinterpret_cast<const float4*>(base + (size_t)r * slot_elems) + i);
                acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
            }
            v = reinterpret_cast<float4*>(xr)[i];
            v.x += acc.x; v.y += acc.y; v.z += acc.z; v.w += acc.w;
            reinterpret_cast<float4*>(xr)[i] = v;
        }
        keep[kept] = v;
        if (y != nullptr) {
            const float ss = warp_sum(sumsq4(v));
            if ((threadIdx.x & 31) == 0) partial[threadIdx.x >> 5] = ss;
            __syncthreads();
            if (threadIdx.x < ncta) {
                // this segment's sum, in warp order, into every CTA of the cluster
                float sj = 0.0f;
#pragma unroll
                for (int w = 0; w < 8; ++w) sj += partial[w];
                st_cluster_f32(mapa_shared(smem_u32(&segtot[seg]), threadIdx.x), sj);
            }
            __syncthreads();
        }
    }
    cluster_sync_all();                              // also: nobody leaves while its shared memory may still be written
    if (y != nullptr && okk) {
        float tot = 0.0f;
        for (int sg = 0; sg < nseg; ++sg) tot += segtot[sg];
        const float rms = rsqrtf(tot / (float)hidden + eps);
        __half* yr = y + (size_t)row * hidden;
#pragma unroll
        for (int kept = 0; kept < KEEP; ++kept) {
            const int seg = crank + kept * ncta;
            const int i = seg * RMS_SEG_VECS + threadIdx.x;
            if (seg < nseg && i < nvec) {
                const float4 v = keep[kept];
                const float4 g = __ldg(reinterpret_cast<const float4*>(gamma) + i);
                const __half2 h0 = __floats2half2_rn(v.x * rms * g.x, v.y * rms * g.y);
                const __half2 h1 = __floats2half2_rn(v.z * rms * g.z, v.w * rms * g.w);
                uint2 o;
                o.x = *reinterpret_cast<const unsigned int*>(&h0);
                o.y = *reinterpret_cast<const unsigned int*>(&h1);
                reinterpret_cast<uint2*>(yr)[i] = o;
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&state[2], 1u) == gridDim.x * gridDim.y - 1) {      // every CTA has read its slots
            atomicExch(&state[2], 0u);
            __threadfence();
            atomicAdd(&state[0], 1u);                         // next operation, other buffer set
        }
    }
}

// cos and sin of the rotation of pair `pair` at position `pos` (freq = 1/powf(base, 2*pair/head_dim),
// theta = pos*freq: crates/kernels/src/ops.rs:2601-2650), and the rotated value of one element of
// the pair (x0 = first half, x1 = second half).  Written without contraction so that every kernel
// that rotates gives the same bits.
__device__ __forceinline__ void rope_cos_sin(int pos, int pair, int head_dim, float rope_base, float* c, float* s)
{
    const float freq = 1.0f / powf(rope_base, 2.0f * (float)pair / (float)head_dim);
    const float theta = __fmul_rn((float)pos, freq);
    *c = cosf(theta);
    *s = sinf(theta);
}
__device__ __forceinline__ float rope_rotate(float x0, float x1, float c, float s, bool first_half)
{
    return first_half ? __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)) : __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
}

// The table of one position: cos [head_dim/2] then sin [head_dim/2], once per decode step, for the
// attention kernel that rotates q and k itself (attn_chunk_kernel<.., true>).
__global__ void __launch_bounds__(256)
rope_table_kernel(float* __restrict__ table, const int* __restrict__ pos_buf, int head_dim, float rope_base)
{
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const int half_d = head_dim / 2;
    const int pair = blockIdx.x * blockDim.x + threadIdx.x;
    if (pair < half_d) rope_cos_sin(pos_buf[0], pair, head_dim, rope_base, &table[pair], &table[half_d + pair]);
}

// q/k bias + rotate-half RoPE, v bias, append k and v at position pos_buf[0].  Reference:
// warp_fused_bias_rope_append_dp, crates/kernels/src/ops.rs:2601-2650 (same formulas: freq =
// 1/powf(base, 2*pair/head_dim), theta = pos*freq).  qkv is the fused GEMM output
// [q | k | v] (so no separate split_qkv pass, ops.rs:2255-2298); caches are f16
// [max_seq][kv_dim].
__global__ void __launch_bounds__(256)
rope_append_kernel(__half* __restrict__ q_out, __half* __restrict__ k_cache, __half* __restrict__ v_cache,
                   const __half* __restrict__ qkv, const float* __restrict__ bias /* [q|k|v] or null */,
                   int num_heads, int num_kv_heads, int head_dim, const int* __restrict__ pos_buf, int max_seq,
                   float rope_base)
{
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const int pos = pos_buf[0];
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    const int q_total = num_heads * head_dim;
    const int kv_dim = num_kv_heads * head_dim;
    const int half_d = head_dim / 2;
    // one sequence per grid row: its own q, its own cache, the shared position
    const size_t row = blockIdx.y;
    qkv += row * (size_t)(q_total + 2 * kv_dim);
    q_out += row * (size_t)q_total;
    k_cache += row * (size_t)max_seq * kv_dim;
    v_cache += row * (size_t)max_seq * kv_dim;
    if (idx < q_total + kv_dim) {
        const bool is_q = idx < q_total;
        const int local = is_q ? idx : idx - q_total;          // index inside q or inside k
        const int head = local / head_dim;
        const int d = local - head * head_dim;
        const int pair = d % half_d;
        float cos_t, sin_t;
        rope_cos_sin(pos, pair, head_dim, rope_base, &cos_t, &sin_t);
        const int src0 = (is_q ? 0 : q_total) + head * head_dim + pair;
        float x0 = __half2float(qkv[src0]), x1 = __half2float(qkv[src0 + half_d]);
        if (bias) { x0 += bias[src0]; x1 += bias[src0 + half_d]; }
        const float r = rope_rotate(x0, x1, cos_t, sin_t, d < half_d);
        if (is_q) q_out[local] = __float2half_rn(r);
        else if (pos < max_seq) k_cache[(size_t)pos * kv_dim + local] = __float2half_rn(r);
    }
    if (idx < kv_dim) {
        const int src = q_total + kv_dim + idx;
        float v = __half2float(qkv[src]);
        if (bias) v += bias[src];
        if (pos < max_seq) v_cache[(size_t)pos * kv_dim + idx] = __float2half_rn(v);
    }
}

// Split-KV decode attention, pass 1.  CTA = (chunk of ATT_CHUNK = 32 tokens, kv head); warp h of the
// CTA takes q head h of the group.  The CTA first copies the chunk's K and V rows (8 KB each) to
// shared memory with coalesced 16-byte loads, every load issued before the first store, so the
// rows leave L2 once per CTA however many q heads share the kv head.  Then per warp:
//   scores: one token per LANE, no cross-lane reduction per score: the lane walks its token's K
//           row (rows padded by 16 bytes: the 128-bit reads of a quarter warp hit 32 distinct banks)
//           against q_h, also in shared memory (broadcast reads);
//   soft-max statistics: one warp max and one warp sum for the 32 tokens;
//   P.V: lanes own 4 of the 128 dims; the 32 probabilities go round by shuffle.
// About 28 warp instructions per (token, head), staging included (1.64 M per call at 2049 tokens x
// 28 heads); the earlier one-token-per-warp loop with a shuffle reduction per score needed 87
// (5.0 M) and 123 registers.  Writes (max, sum, unnormalised o[128]) per (q head, chunk).  The
// sequence length is read from the device (len_buf[0]), the grid covers max_seq.  With many
// sequences in lock step the grid would be tens of waves of these small CTAs; the host then gives
// each CTA `span` consecutive chunks, which it walks with a running (max, sum, o) and with the next
// chunk's loads in flight during the arithmetic, and writes one partial per span (span = 1 gives
// the single-chunk result bit for bit).  Reference:
// warp_flash_decode_chunk_dl, crates/kernels/src/kv_cache.rs:951-1076.
constexpr int ATT_CHUNK = 32;       // tokens per CTA = lanes of a warp
constexpr int ATT_MAX_GROUP = 8;      // q heads per kv head, at most

//
// ROPE = true: the kernel takes the fused QKV GEMM output instead of a rotated q.  Every warp
// rotates its own q head on the way in (bias, rotate-half with the step's cos/sin table, rounding
// to f16 as rope_append_kernel stores q), and the one CTA per kv head whose chunk holds position
// pos_buf[0] rotates the new k row, adds the bias to the new v row, appends both to the caches
// (it is their only writer) and uses them from shared memory: the separate RoPE/append pass
// (fused_bias_rope_append_device_pos, ops.rs:2601-2680) disappears, same bits.
template <int HEAD_DIM, bool ROPE>
__global__ void __launch_bounds__(ATT_MAX_GROUP * 32)
attn_chunk_kernel(float* __restrict__ part /* [heads][parts][HEAD_DIM + 2] */, const __half* __restrict__ q,
                  __half* k_cache, __half* v_cache, int num_heads, int num_kv_heads, const int* __restrict__ len_buf,
                  int max_parts, int span, int max_seq, const float* __restrict__ bias, const float* __restrict__ rope,
                  const int* __restrict__ pos_buf)
{
    static_assert(HEAD_DIM == 128, "lane owns 4 of 128 dims");
    constexpr int ROW_BYTES = HEAD_DIM * 2;                 // one token's K (or V) row of this kv head
    constexpr int KROW = ROW_BYTES + 16;                    // padded K row in shared memory
    constexpr int PIECES = ATT_CHUNK * ROW_BYTES / 16;      // 16-byte pieces of the chunk's K (or V): 512
    constexpr int PER_ROW = ROW_BYTES / 16;                 // 16
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const int kvh = blockIdx.y;
    {   // one sequence per grid z: its own q (or fused q|k|v row), cache and partials
        const size_t row = blockIdx.z;
        q += row * (size_t)(ROPE ? (num_heads + 2 * num_kv_heads) : num_heads) * HEAD_DIM;
        k_cache += row * (size_t)max_seq * num_kv_heads * HEAD_DIM;
        v_cache += row * (size_t)max_seq * num_kv_heads * HEAD_DIM;
        part += row * (size_t)num_heads * max_parts * (HEAD_DIM + 2);
    }
    const int len = min(len_buf[0], max_seq);            // never past the cache
    const int chunk0 = blockIdx.x * span;                // this CTA's chunks: chunk0 .. chunk0 + span - 1
    const int group = num_heads / num_kv_heads;          // = warps of this CTA (the host launches group x 32 threads)
    const int kv_dim = num_kv_heads * HEAD_DIM;
    const int h = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* dst = part + ((size_t)(kvh * group + h) * max_parts + blockIdx.x) * (HEAD_DIM + 2);
    // four dims of one head, rotated: lane l holds dims 4l .. 4l+3, its partner lane l ^ 16 the other half of the pairs
    auto rope4 = [&](int elem0, bool rotate) -> uint2 {
        const uint2 raw = *reinterpret_cast<const uint2*>(q + elem0 + lane * 4);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
        float f[4] = {a.x, a.y, b.x, b.y};
        if (bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 4; ++j) f[j] += bias[elem0 + lane * 4 + j];
        }
        float r[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float other = __shfl_xor_sync(0xffffffffu, f[j], 16);
            const int pair = (lane & 15) * 4 + j;
            const bool first = lane < 16;
            r[j] = rotate ? rope_rotate(first ? f[j] : other, first ? other : f[j], rope[pair], rope[HEAD_DIM / 2 + pair], first)
                          : f[j];
        }
        const __half2 h0 = __floats2half2_rn(r[0], r[1]), h1 = __floats2half2_rn(r[2], r[3]);
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t*>(&h0);
        o.y = *reinterpret_cast<const uint32_t*>(&h1);
        return o;
    };
    const int q_total = num_heads * HEAD_DIM;
    const int pos = ROPE ? pos_buf[0] : -1;
    // the new token's row, if one of this CTA's chunks holds it (CTA-uniform)
    const bool has_new = ROPE && pos >= chunk0 * ATT_CHUNK && pos < (chunk0 + span) * ATT_CHUNK && pos < max_seq;
    uint2 k_new = make_uint2(0, 0), v_new = make_uint2(0, 0);
    if (has_new && h == 0) {                             // the new k and v rows of this kv head: into the caches
        k_new = rope4(q_total + kvh * HEAD_DIM, true);
        v_new = rope4(q_total + kv_dim + kvh * HEAD_DIM, false);
        *reinterpret_cast<uint2*>(k_cache + (size_t)pos * kv_dim + kvh * HEAD_DIM + lane * 4) = k_new;
        *reinterpret_cast<uint2*>(v_cache + (size_t)pos * kv_dim + kvh * HEAD_DIM + lane * 4) = v_new;
    }
    if (chunk0 * ATT_CHUNK >= len) {
        // nothing to attend to: mark the partial as empty so the merge ignores it
        if (lane == 0) { dst[HEAD_DIM] = -INFINITY; dst[HEAD_DIM + 1] = 0.0f; }
        return;
    }
    __shared__ __align__(16) unsigned char k_s[ATT_CHUNK * KROW];
    __shared__ __align__(16) unsigned char v_s[ATT_CHUNK * ROW_BYTES];
    __shared__ __align__(16) float q_s[ATT_MAX_GROUP][HEAD_DIM];
    {
        const uint2 qr = ROPE ? rope4((kvh * group + h) * HEAD_DIM, true)
                              : *reinterpret_cast<const uint2*>(q + (size_t)(kvh * group + h) * HEAD_DIM + lane * 4);
        const float scale = rsqrtf((float)HEAD_DIM);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&qr.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&qr.y));
        *reinterpret_cast<float4*>(&q_s[h][lane * 4]) = make_float4(a.x * scale, a.y * scale, b.x * scale, b.y * scale);
    }
    const size_t row_stride = (size_t)kv_dim * 2;
    constexpr int BATCH = 3;                             // 3 x 224 threads cover the 512 pieces of a 7-head group at once
    // With at least 171 threads one round of loads holds a whole chunk in registers: the next chunk's
    // loads are then issued before this chunk's arithmetic (CTAs that walk several chunks).
    const bool one_round = BATCH * (int)blockDim.x >= PIECES;
    uint4 kk[BATCH], vv[BATCH];
    // K and V of chunk c: piece i is bytes [16 i, 16 i + 16) of the chunk's rows laid end to end; rows past
    // the sequence end are zero (their probability is 0, and 0 x garbage could be NaN); the new token's
    // row is not in the cache yet
    auto load_round = [&](int c, int i0) {
        const int t0 = c * ATT_CHUNK;
        const int nt = min(ATT_CHUNK, len - t0);
        const unsigned char* kg = reinterpret_cast<const unsigned char*>(k_cache + (size_t)t0 * kv_dim + kvh * HEAD_DIM);
        const unsigned char* vg = reinterpret_cast<const unsigned char*>(v_cache + (size_t)t0 * kv_dim + kvh * HEAD_DIM);
#pragma unroll
        for (int b = 0; b < BATCH; ++b) {
            const int i = i0 + b * blockDim.x;
            const int tok = i / PER_ROW, piece = i % PER_ROW;
            const bool in = (i < PIECES) && (tok < nt) && !(has_new && t0 + tok == pos);
            kk[b] = in ? *reinterpret_cast<const uint4*>(kg + tok * row_stride + piece * 16) : make_uint4(0, 0, 0, 0);
            vv[b] = in ? *reinterpret_cast<const uint4*>(vg + tok * row_stride + piece * 16) : make_uint4(0, 0, 0, 0);
        }
    };
    auto store_round = [&](int c, int i0) {
        const int t0 = c * ATT_CHUNK;
#pragma unroll
        for (int b = 0; b < BATCH; ++b) {
            const int i = i0 + b * blockDim.x;
            if (i < PIECES) {
                const int tok = i / PER_ROW, piece = i % PER_ROW;
                if (has_new && t0 + tok == pos) continue;               // written by warp 0
                *reinterpret_cast<uint4*>(k_s + tok * KROW + piece * 16) = kk[b];
                *reinterpret_cast<uint4*>(v_s + i * 16) = vv[b];
            }
        }
    };
    float m_run = -INFINITY, l_run = 0.0f, o0 = 0.0f, o1 = 0.0f, o2 = 0.0f, o3 = 0.0f;
    if (one_round) load_round(chunk0, threadIdx.x);
    for (int sc = 0; sc < span; ++sc) {
        const int c = chunk0 + sc;
        const int t0 = c * ATT_CHUNK;
        if (t0 >= len) break;                              // CTA-uniform
        const int nt = min(ATT_CHUNK, len - t0);           // tokens of this chunk
        if (one_round) {
            store_round(c, threadIdx.x);
        } else {
            for (int i0 = threadIdx.x; i0 < PIECES; i0 += BATCH * blockDim.x) { load_round(c, i0); store_round(c, i0); }
        }
        if (has_new && h == 0 && pos >= t0 && pos < t0 + ATT_CHUNK) {
            *reinterpret_cast<uint2*>(k_s + (pos - t0) * KROW + lane * 8) = k_new;
            *reinterpret_cast<uint2*>(v_s + (pos - t0) * ROW_BYTES + lane * 8) = v_new;
        }
        __syncthreads();
        if (one_round && sc + 1 < span && (c + 1) * ATT_CHUNK < len) load_round(c + 1, threadIdx.x);
        // ---- score of this lane's token ----
        const bool valid = lane < nt;
        float s_tok = 0.0f;
        {
            const uint4* krow = reinterpret_cast<const uint4*>(k_s + lane * KROW);
#pragma unroll
            for (int dc = 0; dc < HEAD_DIM / 8; ++dc) {
                const uint4 kr = krow[dc];
                const float2 k0 = __half22float2(*reinterpret_cast<const __half2*>(&kr.x));
                const float2 k1 = __half22float2(*reinterpret_cast<const __half2*>(&kr.y));
                const float2 k2 = __half22float2(*reinterpret_cast<const __half2*>(&kr.z));
                const float2 k3 = __half22float2(*reinterpret_cast<const __half2*>(&kr.w));
                const float4 qa = *reinterpret_cast<const float4*>(&q_s[h][dc * 8]);
                const float4 qb = *reinterpret_cast<const float4*>(&q_s[h][dc * 8 + 4]);
                s_tok = fmaf(k0.x, qa.x, fmaf(k0.y, qa.y, fmaf(k1.x, qa.z, fmaf(k1.y, qa.w,
                        fmaf(k2.x, qb.x, fmaf(k2.y, qb.y, fmaf(k3.x, qb.z, fmaf(k3.y, qb.w, s_tok))))))));
            }
        }
        // ---- soft-max statistics of the chunk ----
        const float sv = valid ? s_tok : -INFINITY;
        const float mw = warp_max(sv);
        const float pr = valid ? __expf(sv - mw) : 0.0f;
        const float lw = warp_sum(pr);
        // ---- o[dims of this lane] = sum_t p[t] * v_t ----
        float c0 = 0.0f, c1 = 0.0f, c2 = 0.0f, c3 = 0.0f;
        const uint2* vcol = reinterpret_cast<const uint2*>(v_s) + lane;
#pragma unroll
        for (int j = 0; j < ATT_CHUNK; ++j) {
            const float pt = __shfl_sync(0xffffffffu, pr, j);              // 0 for tokens past the end
            const uint2 vr = vcol[j * (ROW_BYTES / 8)];
            const float2 v0 = __half22float2(*reinterpret_cast<const __half2*>(&vr.x));
            const float2 v1 = __half22float2(*reinterpret_cast<const __half2*>(&vr.y));
            c0 = fmaf(pt, v0.x, c0); c1 = fmaf(pt, v0.y, c1); c2 = fmaf(pt, v1.x, c2); c3 = fmaf(pt, v1.y, c3);
        }
        if (sc == 0) {
            m_run = mw; l_run = lw; o0 = c0; o1 = c1; o2 = c2; o3 = c3;
        } else {                                           // fold this chunk into the running (max, sum, o)
            const float m_new = fmaxf(m_run, mw);
            const float wa = __expf(m_run - m_new), wb = __expf(mw - m_new);
            l_run = fmaf(l_run, wa, lw * wb);
            o0 = fmaf(o0, wa, c0 * wb); o1 = fmaf(o1, wa, c1 * wb); o2 = fmaf(o2, wa, c2 * wb); o3 = fmaf(o3, wa, c3 * wb);
            m_run = m_new;
        }
        if (sc + 1 < span) __syncthreads();                // the next chunk overwrites the staged rows
    }
    // a partial is HEAD_DIM + 2 floats long, so its start is 8-byte aligned only: two float2 stores
    *reinterpret_cast<float2*>(dst + lane * 4) = make_float2(o0, o1);
    *reinterpret_cast<float2*>(dst + lane * 4 + 2) = make_float2(o2, o3);
    if (lane == 0) { dst[HEAD_DIM] = m_run; dst[HEAD_DIM + 1] = l_run; }
}

// ---- the same pass on the tensor cores, for launches whose CTAs walk several chunks ----
// With many sequences in lock step the lane-per-token kernel above is bound by instruction issue
// (28 warp instructions per token and q head).  Here the q heads of a kv head are the M dimension of
// warp-level MMAs (up to 8 heads, padded to 16 rows): per 32-token chunk each of the CTA's four warps
// takes 8 tokens, S = Q K^T as 8 x m16n8k16 (K rows are the B fragments as they lie in shared
// memory), an online soft-max of its own (the warp keeps its own running max, sum and O over "its"
// tokens of every chunk, so the warps never synchronise inside a chunk), and O += P V as 16 x m16n8k8
// with P rounded to f16 and V fragments fetched with ldmatrix.trans.  At the end the four warps'
// (max, sum, O) are merged through shared memory into one partial per q head, in the format of
// the kernel above.  About 130 warp instructions per warp and chunk instead of 896.
__device__ __forceinline__ void att_mma_16816(float (&d)[4], uint32_t a0, uint32_t a2, uint32_t b0, uint32_t b1)
{
    // rows 8..15 of A (a1, a3) are padding: zero
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void att_mma_1688(float& d0, float& d1, uint32_t a0, uint32_t b0)
{
    float z2 = 0.0f, z3 = 0.0f;                  // rows 8..15: padding, results dropped
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
                 : "+f"(d0), "+f"(d1), "+f"(z2), "+f"(z3)
                 : "r"(a0), "r"(0u), "r"(b0));
}
__device__ __forceinline__ void att_ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr));
}

constexpr int ATT_MMA_WARPS = 4;
constexpr int ATT_MMA_STAGES = 3;                             // chunks of K and V in shared memory: one in use, two on their way
constexpr int ATT_MMA_STAGE_BYTES = 2 * ATT_CHUNK * (128 * 2 + 16);
constexpr int ATT_MMA_SMEM_BYTES = ATT_MMA_STAGES * ATT_MMA_STAGE_BYTES;   // dynamic shared memory of attn_span_mma_kernel<128, .>
// 16 bytes global -> shared without passing through registers; src_bytes = 0 writes zeros and reads nothing
__device__ __forceinline__ void att_cp_async16(uint32_t smem_dst, const void* gsrc, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void att_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void att_cp_async_wait_all_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }
template <int HEAD_DIM, bool ROPE>
__global__ void __launch_bounds__(ATT_MMA_WARPS * 32)
attn_span_mma_kernel(float* __restrict__ part /* [heads][parts][HEAD_DIM + 2] */, const __half* __restrict__ q,
                     __half* k_cache, __half* v_cache, int num_heads, int num_kv_heads, const int* __restrict__ len_buf,
                     int max_parts, int span, int max_seq, const float* __restrict__ bias, const float* __restrict__ rope,
                     const int* __restrict__ pos_buf)
{
    static_assert(HEAD_DIM == 128, "lane owns 4 of 128 dims when staging");
    constexpr int ROW_BYTES = HEAD_DIM * 2;
    constexpr int KROW = ROW_BYTES + 16;                    // padded K and V rows: conflict-free fragment loads
    constexpr int PIECES = ATT_CHUNK * ROW_BYTES / 16;      // 512 16-byte pieces of a chunk's K (or V)
    constexpr int PER_ROW = ROW_BYTES / 16;
    constexpr int THREADS = ATT_MMA_WARPS * 32;
    constexpr int BATCH = PIECES / THREADS;                 // 4: one round of loads holds a whole chunk
    constexpr int STRIDE = HEAD_DIM + 2;
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const int kvh = blockIdx.y;
    {
        const size_t row = blockIdx.z;
        q += row * (size_t)(ROPE ? (num_heads + 2 * num_kv_heads) : num_heads) * HEAD_DIM;
        k_cache += row * (size_t)max_seq * num_kv_heads * HEAD_DIM;
        v_cache += row * (size_t)max_seq * num_kv_heads * HEAD_DIM;
        part += row * (size_t)num_heads * max_parts * STRIDE;
    }
    const int len = min(len_buf[0], max_seq);
    const int chunk0 = blockIdx.x * span;
    const int group = num_heads / num_kv_heads;          // q heads of this kv head, at most 8
    const int kv_dim = num_kv_heads * HEAD_DIM;
    const int w = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    float* dst0 = part + ((size_t)(kvh * group) * max_parts + blockIdx.x) * STRIDE;      // head h: + h * max_parts * STRIDE
    // four dims of one head (the whole warp: one head), biased and rotated, as f16
    auto rope4 = [&](int elem0, bool rotate) -> uint2 {
        const uint2 raw = *reinterpret_cast<const uint2*>(q + elem0 + lane * 4);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&raw.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&raw.y));
        float f[4] = {a.x, a.y, b.x, b.y};
        if (bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 4; ++j) f[j] += bias[elem0 + lane * 4 + j];
        }
        float r[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float other = __shfl_xor_sync(0xffffffffu, f[j], 16);
            const int pair = (lane & 15) * 4 + j;
            const bool first = lane < 16;
            r[j] = rotate ? rope_rotate(first ? f[j] : other, first ? other : f[j], rope[pair], rope[HEAD_DIM / 2 + pair], first)
                          : f[j];
        }
        const __half2 h0 = __floats2half2_rn(r[0], r[1]), h1 = __floats2half2_rn(r[2], r[3]);
        uint2 o;
        o.x = *reinterpret_cast<const uint32_t*>(&h0);
        o.y = *reinterpret_cast<const uint32_t*>(&h1);
        return o;
    };
    const int q_total = num_heads * HEAD_DIM;
    const int pos = ROPE ? pos_buf[0] : -1;
    const bool has_new = ROPE && pos >= chunk0 * ATT_CHUNK && pos < (chunk0 + span) * ATT_CHUNK && pos < max_seq;
    uint2 k_new = make_uint2(0, 0), v_new = make_uint2(0, 0);
    if (has_new && w == 0) {
        k_new = rope4(q_total + kvh * HEAD_DIM, true);
        v_new = rope4(q_total + kv_dim + kvh * HEAD_DIM, false);
        *reinterpret_cast<uint2*>(k_cache + (size_t)pos * kv_dim + kvh * HEAD_DIM + lane * 4) = k_new;
        *reinterpret_cast<uint2*>(v_cache + (size_t)pos * kv_dim + kvh * HEAD_DIM + lane * 4) = v_new;
    }
    if (chunk0 * ATT_CHUNK >= len) {
        for (int h = threadIdx.x; h < group; h += THREADS) {
            float* d = dst0 + (size_t)h * max_parts * STRIDE;
            d[HEAD_DIM] = -INFINITY; d[HEAD_DIM + 1] = 0.0f;
        }
        return;
    }
    // K and V of three chunks in turn (asynchronous copies, two chunks ahead of the arithmetic: with one chunk
    // ahead and the copy staged through registers the pass reached 54 % of the HBM rate at 32 sequences x 4096
    // tokens); after the last chunk the same bytes hold the four warps' results
    extern __shared__ __align__(16) unsigned char kv_s[];
    __shared__ __align__(16) __half q_s[ATT_MAX_GROUP][HEAD_DIM];
    constexpr int STAGE_BYTES = 2 * ATT_CHUNK * KROW;
    static_assert(STAGE_BYTES == ATT_MMA_STAGE_BYTES, "host and device agree on the stage size");
    static_assert(STAGE_BYTES >= ATT_MMA_WARPS * ATT_MAX_GROUP * STRIDE * 4, "merge buffer fits the staging bytes");
    for (int hh = w; hh < ATT_MAX_GROUP; hh += ATT_MMA_WARPS) {
        uint2 qr = make_uint2(0, 0);                     // heads past the group: zero rows
        if (hh < group)
            qr = ROPE ? rope4((kvh * group + hh) * HEAD_DIM, true)
                      : *reinterpret_cast<const uint2*>(q + (size_t)(kvh * group + hh) * HEAD_DIM + lane * 4);
        *reinterpret_cast<uint2*>(&q_s[hh][lane * 4]) = qr;
    }
    __syncthreads();
    uint32_t qa0[HEAD_DIM / 16], qa2[HEAD_DIM / 16];     // A fragments of Q, row g (rows 8..15 are zero)
#pragma unroll
    for (int ks = 0; ks < HEAD_DIM / 16; ++ks) {
        qa0[ks] = *reinterpret_cast<const uint32_t*>(&q_s[g][ks * 16 + 2 * t]);
        qa2[ks] = *reinterpret_cast<const uint32_t*>(&q_s[g][ks * 16 + 8 + 2 * t]);
    }
    const size_t row_stride = (size_t)kv_dim * 2;
    const uint32_t kv_base = smem_u32(kv_s);
    // chunk c into ring stage st: every thread copies four 16-byte pieces of K and of V; rows past the end
    // are zero-filled, the new row (not in the cache yet) is left to warp 0.  Always one commit, also for
    // a chunk that does not exist, so that "all but the latest group" means the same in every iteration.
    auto issue_chunk = [&](int c, int st) {
        const int t0 = c * ATT_CHUNK;
        if (t0 < len && c < chunk0 + span) {
            const int nt = min(ATT_CHUNK, len - t0);
            const unsigned char* kg = reinterpret_cast<const unsigned char*>(k_cache + (size_t)t0 * kv_dim + kvh * HEAD_DIM);
            const unsigned char* vg = reinterpret_cast<const unsigned char*>(v_cache + (size_t)t0 * kv_dim + kvh * HEAD_DIM);
            const uint32_t ks = kv_base + st * STAGE_BYTES, vs = ks + ATT_CHUNK * KROW;
#pragma unroll
            for (int b = 0; b < BATCH; ++b) {
                const int i = threadIdx.x + b * THREADS;
                const int tok = i / PER_ROW, piece = i % PER_ROW;
                if (has_new && t0 + tok == pos) continue;                      // written by warp 0
                const int bytes = (tok < nt) ? 16 : 0;
                const size_t goff = (tok < nt) ? (size_t)tok * row_stride + piece * 16 : 0;
                att_cp_async16(ks + tok * KROW + piece * 16, kg + goff, bytes);
                att_cp_async16(vs + tok * KROW + piece * 16, vg + goff, bytes);
            }
        }
        att_cp_async_commit();
    };
    const float scale = rsqrtf((float)HEAD_DIM);
    float m_run = -INFINITY, l_run = 0.0f;
    float o[HEAD_DIM / 8][2];                            // head g: dims 8 j + 2 t, + 1
#pragma unroll
    for (int j = 0; j < HEAD_DIM / 8; ++j) { o[j][0] = 0.0f; o[j][1] = 0.0f; }
    issue_chunk(chunk0, 0);
    issue_chunk(chunk0 + 1, 1);
    for (int sc = 0; sc < span; ++sc) {
        const int c = chunk0 + sc;
        const int t0 = c * ATT_CHUNK;
        if (t0 >= len) break;                              // CTA-uniform
        const int nt = min(ATT_CHUNK, len - t0);
        const int st = sc % ATT_MMA_STAGES;
        unsigned char* k_s = kv_s + st * STAGE_BYTES;
        unsigned char* v_s = k_s + ATT_CHUNK * KROW;
        att_cp_async_wait_all_but_one();                   // this thread's pieces of chunk c have landed
        if (has_new && w == 0 && pos >= t0 && pos < t0 + ATT_CHUNK) {
            *reinterpret_cast<uint2*>(k_s + (pos - t0) * KROW + lane * 8) = k_new;
            *reinterpret_cast<uint2*>(v_s + (pos - t0) * KROW + lane * 8) = v_new;
        }
        __syncthreads();                                   // everybody's pieces; and everybody is done with chunk c - 1,
        issue_chunk(c + 2, (sc + 2) % ATT_MMA_STAGES);     // whose stage the chunk after next now takes
        // ---- S[head g][tokens 8 w + 2 t, + 1] ----
        float s4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        {
            const unsigned char* krow = k_s + (8 * w + g) * KROW + 4 * t;
#pragma unroll
            for (int ks = 0; ks < HEAD_DIM / 16; ++ks) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + ks * 32);
                const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + ks * 32 + 16);
                att_mma_16816(s4, qa0[ks], qa2[ks], b0, b1);
            }
        }
        // ---- this warp's online soft-max over its 8 tokens ----
        const int tk = 8 * w + 2 * t;
        const float s0 = (tk < nt) ? s4[0] * scale : -INFINITY;
        const float s1 = (tk + 1 < nt) ? s4[1] * scale : -INFINITY;
        float mx = fmaxf(s0, s1);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const bool any = m_new != -INFINITY;               // the same for the four lanes of a head
        const float corr = (m_run == -INFINITY) ? 0.0f : __expf(m_run - m_new);
        const float p0 = (any && tk < nt) ? __expf(s0 - m_new) : 0.0f;
        const float p1 = (any && tk + 1 < nt) ? __expf(s1 - m_new) : 0.0f;
        float ps = p0 + p1;
        ps += __shfl_xor_sync(0xffffffffu, ps, 1);
        ps += __shfl_xor_sync(0xffffffffu, ps, 2);
        l_run = fmaf(l_run, corr, ps);
        m_run = m_new;
        const __half2 ph = __floats2half2_rn(p0, p1);
        const uint32_t pa = *reinterpret_cast<const uint32_t*>(&ph);
        // ---- O[head g][:] = O * corr + P V over the warp's 8 tokens ----
        const uint32_t v_base = smem_u32(v_s + (8 * w + (lane & 7)) * KROW + (lane >> 3) * 16);
#pragma unroll
        for (int j4 = 0; j4 < HEAD_DIM / 32; ++j4) {
            uint32_t vb[4];
            att_ldmatrix_x4_trans(vb, v_base + j4 * 64);     // dims 32 j4 .. 32 j4 + 31: four 8-dim tiles
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
                float& d0 = o[j4 * 4 + jj][0];
                float& d1 = o[j4 * 4 + jj][1];
                d0 *= corr; d1 *= corr;
                att_mma_1688(d0, d1, pa, vb[jj]);
            }
        }
    }
    // ---- merge the four warps' results per q head ----
    asm volatile("cp.async.wait_all;" ::: "memory");       // (only empty groups can be left)
    __syncthreads();                                       // everybody is done with the staged rows
    float* mb = reinterpret_cast<float*>(kv_s);            // [warp][head][STRIDE]
    if (g < group) {
        float* mine = mb + ((size_t)w * ATT_MAX_GROUP + g) * STRIDE;
#pragma unroll
        for (int j = 0; j < HEAD_DIM / 8; ++j) *reinterpret_cast<float2*>(mine + 8 * j + 2 * t) = make_float2(o[j][0], o[j][1]);
        if (t == 0) { mine[HEAD_DIM] = m_run; mine[HEAD_DIM + 1] = l_run; }
    }
    __syncthreads();
    const int d = threadIdx.x;                             // 128 threads = 128 dims
    for (int h = 0; h < group; ++h) {
        float mw[ATT_MMA_WARPS], mm = -INFINITY;
#pragma unroll
        for (int ww = 0; ww < ATT_MMA_WARPS; ++ww) {
            mw[ww] = mb[((size_t)ww * ATT_MAX_GROUP + h) * STRIDE + HEAD_DIM];
            mm = fmaxf(mm, mw[ww]);
        }
        float ov = 0.0f, lv = 0.0f;
#pragma unroll
        for (int ww = 0; ww < ATT_MMA_WARPS; ++ww) {
            const float wgt = (mw[ww] == -INFINITY) ? 0.0f : __expf(mw[ww] - mm);
            ov = fmaf(mb[((size_t)ww * ATT_MAX_GROUP + h) * STRIDE + d], wgt, ov);
            lv = fmaf(mb[((size_t)ww * ATT_MAX_GROUP + h) * STRIDE + HEAD_DIM + 1], wgt, lv);
        }
        float* dsth = dst0 + (size_t)h * max_parts * STRIDE;
        dsth[d] = ov;
        if (d == 0) { dsth[HEAD_DIM] = mm; dsth[HEAD_DIM + 1] = lv; }
    }
}

// Pass 2: merge the chunks of one q head (log-sum-exp weights), write f16.  CTA = q head, 4 x 128
// threads: thread (part, d) sums dimension d over every fourth chunk, eight loads in flight.
// Reference: warp_flash_decode_reduce, crates/kernels/src/kv_cache.rs:790-841.
constexpr int ATT_MERGE_PARTS = 4;
template <int HEAD_DIM>
__global__ void __launch_bounds__(HEAD_DIM * ATT_MERGE_PARTS)
attn_merge_kernel(__half* __restrict__ out, const float* __restrict__ part, const int* __restrict__ len_buf,
                  int max_chunks /* partials per head */, int span /* chunks per partial */)
{
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    constexpr int MAXC = 1024;                       // chunk weights kept in shared memory
    constexpr int THREADS = HEAD_DIM * ATT_MERGE_PARTS, WARPS = THREADS / 32, STRIDE = HEAD_DIM + 2;
    __shared__ float s_w[MAXC];
    __shared__ float s_l[MAXC];
    __shared__ float s_max[WARPS], s_sum[WARPS];
    __shared__ float s_o[ATT_MERGE_PARTS][HEAD_DIM];
    const int head = blockIdx.x, tid = threadIdx.x, d = tid % HEAD_DIM, prt = tid / HEAD_DIM;
    out += (size_t)blockIdx.y * gridDim.x * HEAD_DIM;
    part += (size_t)blockIdx.y * gridDim.x * max_chunks * STRIDE;
    const int chunks = min(min(max_chunks, MAXC), ((len_buf[0] + ATT_CHUNK - 1) / ATT_CHUNK + span - 1) / span);
    const float* base = part + (size_t)head * max_chunks * STRIDE;
    // every chunk's (max, sum) in one round of loads, one chunk per thread
    float mloc = -INFINITY;
    for (int c = tid; c < chunks; c += THREADS) {
        const float2 ml = *reinterpret_cast<const float2*>(base + (size_t)c * STRIDE + HEAD_DIM);
        s_w[c] = ml.x;
        s_l[c] = ml.y;
        mloc = fmaxf(mloc, ml.x);
    }
    mloc = warp_max(mloc);
    if ((tid & 31) == 0) s_max[tid >> 5] = mloc;
    __syncthreads();
    float mm = s_max[0];
#pragma unroll
    for (int w = 1; w < WARPS; ++w) mm = fmaxf(mm, s_max[w]);
    float lloc = 0.0f;
    for (int c = tid; c < chunks; c += THREADS) {
        const float mc = s_w[c];
        const float w = (mc == -INFINITY) ? 0.0f : __expf(mc - mm);
        s_w[c] = w;
        lloc += s_l[c] * w;
    }
    lloc = warp_sum(lloc);
    if ((tid & 31) == 0) s_sum[tid >> 5] = lloc;
    __syncthreads();
    float oo = 0.0f;
    for (int c0 = prt; c0 < chunks; c0 += ATT_MERGE_PARTS * 8) {
        float v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = c0 + j * ATT_MERGE_PARTS;
            v[j] = (c < chunks) ? base[(size_t)c * STRIDE + d] : 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int c = c0 + j * ATT_MERGE_PARTS;
            oo = fmaf(v[j], (c < chunks) ? s_w[c] : 0.0f, oo);
        }
    }
    s_o[prt][d] = oo;
    __syncthreads();
    if (prt == 0) {
        float ll = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) ll += s_sum[w];
        float tot = s_o[0][d];
#pragma unroll
        for (int p = 1; p < ATT_MERGE_PARTS; ++p) tot += s_o[p][d];
        out[(size_t)head * HEAD_DIM + d] = __float2half_rn(ll > 0.0f ? tot / ll : 0.0f);
    }
}

// act = silu(gate) * up on the fused gate+up GEMM output [gate | up] (no split_gate_up pass).
// Reference: warp_fused_silu_mul, crates/kernels/src/ops.rs:966-977 (g / (1 + expf(-g)) * up).
__global__ void __launch_bounds__(256)
silu_mul_kernel(__half* __restrict__ act, const __half* __restrict__ gate_up, int ffn, int rows)
{
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < ffn * rows) {
        const int r = i / ffn, c = i - r * ffn;
        const float g = __half2float(gate_up[(size_t)r * 2 * ffn + c]);
        const float u = __half2float(gate_up[(size_t)r * 2 * ffn + ffn + c]);
        act[i] = __float2half_rn(g / (1.0f + expf(-g)) * u);
    }
}

// FP16 LM head: logits[v] = sum_h x[h] * W[v][h], W row-major f16 [vocab][hidden], FP32
// accumulate.  One warp per vocabulary row (a row is one contiguous run), 128-bit loads, x in
// shared memory.  Reference: the LM head is a cuBLAS SGEMM outside the graph
// (crates/kernels/src/generate.rs:1727-1735); warp_hgemm_m1 (quantize.rs:3682-3716) is the
// in-tree FP16 GEMV of the same shape.
__global__ void __launch_bounds__(256)
lm_head_kernel(float* __restrict__ logits, const __half* __restrict__ x, const __half* __restrict__ w, int hidden,
               int vocab)
{
    pdl_launch_dependents();
    extern __shared__ __align__(16) uint8_t lm_smem[];
    __half* xs = reinterpret_cast<__half*>(lm_smem);
    pdl_wait_prior_grids();
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) xs[i] = x[i];
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int warps_total = gridDim.x * (blockDim.x >> 5);
    for (int v = blockIdx.x * (blockDim.x >> 5) + warp; v < vocab; v += warps_total) {
        const uint4* wr = reinterpret_cast<const uint4*>(w + (size_t)v * hidden);
        const uint4* xr = reinterpret_cast<const uint4*>(xs);
        float acc = 0.0f;
        for (int i = lane; i < hidden / 8; i += 32) {
            const uint4 a = __ldg(wr + i);
            const uint4 b = xr[i];
            const __half2* ah = reinterpret_cast<const __half2*>(&a);
            const __half2* bh = reinterpret_cast<const __half2*>(&b);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 fa = __half22float2(ah[j]), fb = __half22float2(bh[j]);
                acc = fmaf(fa.x, fb.x, acc);
                acc = fmaf(fa.y, fb.y, acc);
            }
        }
        acc = warp_sum(acc);
        if (lane == 0) logits[v] = acc;
    }
}

// arg-max with ties to the smallest index, two passes.  Reference: CPU sampling over the full
// logits after a D2H copy (crates/kernels/src/generate.rs:68-169, 2531-2534); here it stays on
// the device so the next token never leaves the GPU.
__global__ void __launch_bounds__(256)
argmax_partial_kernel(float* __restrict__ pval, int* __restrict__ pidx, const float* __restrict__ logits, int n)
{
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const float v = logits[i];
        if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
    __shared__ float sv[256];
    __shared__ int si[256];
    sv[threadIdx.x] = best; si[threadIdx.x] = bi;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            const float v = sv[threadIdx.x + s]; const int i = si[threadIdx.x + s];
            if (v > sv[threadIdx.x] || (v == sv[threadIdx.x] && i < si[threadIdx.x])) { sv[threadIdx.x] = v; si[threadIdx.x] = i; }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) { pval[blockIdx.x] = sv[0]; pidx[blockIdx.x] = si[0]; }
}

// Final pass; also advances the device-side position / length buffers for the next step and
// appends the token to the output list, so a replayed graph needs no host input at all.
__global__ void __launch_bounds__(256)
argmax_final_kernel(int* __restrict__ token_out, int* __restrict__ history, int history_capacity,
                    int* __restrict__ pos_buf, int* __restrict__ len_buf, int* __restrict__ step_buf,
                    const float* __restrict__ pval, const int* __restrict__ pidx, int nparts, int n)
{
    pdl_launch_dependents();
    pdl_wait_prior_grids();
    __shared__ float sv[256];
    __shared__ int si[256];
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < nparts; i += blockDim.x) {
        const float v = pval[i]; const int ix = pidx[i];
        if (v > best || (v == best && ix < bi)) { best = v; bi = ix; }
    }
    sv[threadIdx.x] = best; si[threadIdx.x] = bi;
    __syncthreads();
    for (int s = 128; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            const float v = sv[threadIdx.x + s]; const int i = si[threadIdx.x + s];
            if (v > sv[threadIdx.x] || (v == sv[threadIdx.x] && i < si[threadIdx.x])) { sv[threadIdx.x] = v; si[threadIdx.x] = i; }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        // every logit NaN or -inf leaves the index at its start value: token 0 then, never an index
        // past the vocabulary (the next step's embedding lookup uses it as a row number)
        const int tok = (si[0] >= 0 && si[0] < n) ? si[0] : 0;
        token_out[0] = tok;
        const int step = step_buf[0];
        if (history && step >= 0 && step < history_capacity) history[step] = tok;     // a full list is not overrun
        step_buf[0] += 1;
        pos_buf[0] += 1;
        len_buf[0] += 1;
    }
}

}  // namespace ops
}  // namespace twm
