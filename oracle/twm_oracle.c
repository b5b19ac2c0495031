/*
 * twm_oracle.c — CPU restatement of the TW-Marlin W4A16 Q4 arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the parity checker and the timed
 * CPU baseline.  Nothing in the product library links, loads or calls it.
 *
 * Each function names the reference source it restates (paths are relative to
 * the reference project root).  Arithmetic is plain scalar C; no vector
 * intrinsics, so that the order of floating-point operations is the one that
 * is written down.  Compile with -ffp-contract=off: every fused multiply-add
 * that must be fused is written as fmaf().
 *
 * Pinning status: the reference holds no test and no golden vector for any
 * TW-Marlin function.  What pins this restatement is (1) the closed-form
 * known-answer inputs of the reference's nearest tests
 * (crates/kernels/src/quantize.rs:3002-3042 and :3608-3664) and (2) outputs of
 * the reference's own CUDA kernels, compiled unchanged from the reference tree
 * and run on a B200, stored as fixtures under tests/golden/.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define TWMO_BLOCK 32 /* nibble block along K; crates/kernels/src/quantize.rs:25 */

/* ---------------------------------------------------------------- fp16 -- */

/* f32 -> f16, IEEE round-to-nearest-even, with subnormals, overflow to inf.
 * Same result as half::f16::from_f32 (crate half 2.7.1, named in the
 * reference's Cargo.lock:488-489) and as CUDA __float2half_rn. */
uint16_t twmo_f32_to_f16(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t exp = (x >> 23) & 0xFFu;
    uint32_t man = x & 0x7FFFFFu;
    if (exp == 0xFFu) /* inf / nan */
        return (uint16_t)(sign | 0x7C00u | (man ? (0x0200u | (man >> 13)) : 0u));
    int32_t e = (int32_t)exp - 127 + 15;
    if (e >= 0x1F)
        return (uint16_t)(sign | 0x7C00u);
    if (e <= 0) {
        if (e < -10)
            return (uint16_t)sign; /* below half of the smallest subnormal */
        man |= 0x800000u;
        uint32_t shift = (uint32_t)(14 - e); /* 14..24 */
        uint32_t half_man = man >> shift;
        uint32_t rem = man & ((1u << shift) - 1u);
        uint32_t halfway = 1u << (shift - 1);
        if (rem > halfway || (rem == halfway && (half_man & 1u)))
            half_man++;
        return (uint16_t)(sign | half_man);
    }
    uint32_t out = sign | ((uint32_t)e << 10) | (man >> 13);
    uint32_t rem = man & 0x1FFFu;
    if (rem > 0x1000u || (rem == 0x1000u && (out & 1u)))
        out++; /* carry may roll into the exponent, which is the right answer */
    return (uint16_t)out;
}

/* f16 bits -> f32, exact (what PTX cvt.f32.f16 does;
 * crates/kernels/src/quantize.rs:1223). */
float twmo_f16_to_f32(uint16_t h)
{
    uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t x;
    if (exp == 0) {
        if (man == 0) {
            x = sign;
        } else {
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while (!(man & 0x400u));
            x = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FFu) << 13);
        }
    } else if (exp == 0x1F) {
        x = sign | 0x7F800000u | (man << 13);
    } else {
        x = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &x, 4);
    return f;
}

void twmo_f32_to_f16_array(const float *src, uint16_t *dst, long n)
{
    for (long i = 0; i < n; i++)
        dst[i] = twmo_f32_to_f16(src[i]);
}

void twmo_f16_to_f32_array(const uint16_t *src, float *dst, long n)
{
    for (long i = 0; i < n; i++)
        dst[i] = twmo_f16_to_f32(src[i]);
}

/* ------------------------------------------------------ quantise + pack -- */

/* One scale group of `group` consecutive K values of one column.
 * crates/loader/src/gemma_moe_q4.rs:235-250 (and the GPU twin
 * crates/kernels/src/quantize.rs:119-144): amax, scale = amax/7,
 * inv = 7/amax (0 when the scale is 0), q = clamp(round_half_away(v*inv)+8, 0, 15).
 * The quantiser uses the f32 scale; the stored scale is its f16 rounding. */
static void quantise_group(const float *vals, int group, uint8_t *q_out, uint16_t *scale_out)
{
    float amax = 0.0f;
    for (int i = 0; i < group; i++) {
        float a = fabsf(vals[i]);
        if (a > amax) /* f32::max fold; NaN inputs are outside the contract */
            amax = a;
    }
    float scale = amax / 7.0f;
    float inv = (scale != 0.0f) ? 7.0f / amax : 0.0f;
    *scale_out = twmo_f32_to_f16(scale);
    for (int i = 0; i < group; i++) {
        int q = (int)roundf(vals[i] * inv) + 8; /* roundf: ties away from zero, as Rust f32::round */
        if (q < 0)
            q = 0;
        if (q > 15)
            q = 15;
        q_out[i] = (uint8_t)q;
    }
}

/* Quantise a weight matrix to the TW-Marlin tensors.
 *   w        : f32, [N,K] row-major when w_is_nk != 0 (the layout
 *              cpu_quantize_tw_marlin takes, gemma_moe_q4.rs:214,232),
 *              else [K,N] row-major (the layout quantize_f32_to_tw_marlin
 *              takes, quantize.rs:1171-1177).
 *   packed   : u8  [K/32][N][16]; byte i of a block holds k=2i in the low
 *              nibble and k=2i+1 in the high nibble (gemma_moe_q4.rs:241-249).
 *   scales   : f16 bits [K/group][N].
 * group = 32 is the reference bit for bit; group = 128 takes amax over four
 * consecutive 32-blocks and stores one scale for them. */
int twmo_quantize_pack(const float *w, int w_is_nk, int K, int N, int group,
                       uint8_t *packed, uint16_t *scales)
{
    if (K <= 0 || N <= 0 || (group != 32 && group != 128) || K % group != 0)
        return -1;
    float vals[128];
    uint8_t q[128];
    int blocks_per_group = group / TWMO_BLOCK;
    for (int col = 0; col < N; col++) {
        for (int g = 0; g < K / group; g++) {
            for (int i = 0; i < group; i++) {
                long k = (long)g * group + i;
                vals[i] = w_is_nk ? w[(long)col * K + k] : w[k * (long)N + col];
            }
            uint16_t s;
            quantise_group(vals, group, q, &s);
            scales[(long)g * N + col] = s;
            for (int b = 0; b < blocks_per_group; b++) {
                long blk = (long)g * blocks_per_group + b;
                uint8_t *dst = packed + (blk * N + col) * 16;
                for (int i = 0; i < 16; i++)
                    dst[i] = (uint8_t)(q[b * 32 + 2 * i] | (q[b * 32 + 2 * i + 1] << 4));
            }
        }
    }
    return 0;
}

/* Quantise-then-dequantise of a flat array in 32-blocks with the f32 scale
 * (the Q4_0 round trip the reference tests: cpu_q4_0_roundtrip,
 * crates/kernels/src/quantize.rs:2938-2954). */
void twmo_q4_0_roundtrip(const float *in, float *out, long n)
{
    for (long blk = 0; blk < n / 32; blk++) {
        const float *src = in + blk * 32;
        float amax = 0.0f;
        for (int i = 0; i < 32; i++) {
            float a = fabsf(src[i]);
            if (a > amax)
                amax = a;
        }
        float scale = amax / 7.0f;
        float inv = (scale != 0.0f) ? 7.0f / amax : 0.0f;
        for (int i = 0; i < 32; i++) {
            int q = (int)roundf(src[i] * inv) + 8;
            q = q < 0 ? 0 : (q > 15 ? 15 : q);
            out[blk * 32 + i] = scale * (float)(q - 8);
        }
    }
}

/* ---------------------------------------------------------------- decode -- */

/* Nibble of K index k in column n.  The kernel reads the 16 bytes as four
 * little-endian u32 and takes bits 4*(j%8) of word j/8
 * (crates/kernels/src/quantize.rs:1207-1217,1226-1236), which is byte j/2,
 * low nibble for even j. */
static inline int nibble_at(const uint8_t *packed, long N, long k, long n)
{
    const uint8_t *blk = packed + ((k / 32) * N + n) * 16;
    int j = (int)(k % 32);
    uint8_t byte = blk[j / 2];
    return (j & 1) ? (byte >> 4) : (byte & 0x0F);
}

/* Dequantise to f32 [K,N] row-major: w = f32(scale_f16) * (nibble - 8).
 * crates/kernels/src/quantize.rs:3642-3659 (scale * q), with the separated
 * fp16 scale of quantize.rs:1221-1223.  Exact in f32 (11-bit x 4-bit). */
int twmo_dequant_f32(const uint8_t *packed, const uint16_t *scales, int K, int N, int group,
                     float *out)
{
    if ((group != 32 && group != 128) || K % group != 0)
        return -1;
    for (long k = 0; k < K; k++) {
        const uint16_t *srow = scales + (k / group) * (long)N;
        for (long n = 0; n < N; n++)
            out[k * N + n] = twmo_f16_to_f32(srow[n]) * (float)(nibble_at(packed, N, k, n) - 8);
    }
    return 0;
}

/* Dequantise to f16 bits [K,N]: fp16_rn(f32(scale) * (nibble - 8)).
 * crates/kernels/src/quantize.rs:568 (__float2half of scale * q). */
int twmo_dequant_f16(const uint8_t *packed, const uint16_t *scales, int K, int N, int group,
                     uint16_t *out)
{
    if ((group != 32 && group != 128) || K % group != 0)
        return -1;
    for (long k = 0; k < K; k++) {
        const uint16_t *srow = scales + (k / group) * (long)N;
        for (long n = 0; n < N; n++)
            out[k * N + n] = twmo_f32_to_f16(twmo_f16_to_f32(srow[n]) *
                                             (float)(nibble_at(packed, N, k, n) - 8));
    }
    return 0;
}

/* ---------------------------------------------------------------- matmul -- */

/* Naive f32 GEMM, loops i -> j -> p, f32 accumulate, separate multiply and add.
 * crates/kernels/src/gemm.rs:162-173. */
void twmo_gemm_f32(const float *a, const float *b, float *c, int M, int N, int K)
{
    for (long i = 0; i < M; i++)
        for (long j = 0; j < N; j++) {
            float sum = 0.0f;
            for (long p = 0; p < K; p++)
                sum += a[i * K + p] * b[p * N + j];
            c[i * N + j] = sum;
        }
}

/* Same contraction with f64 accumulate: the adjudicator when two f32
 * summation orders disagree on a near-zero output. */
void twmo_gemm_f64acc(const float *a, const float *b, double *c, int M, int N, int K)
{
    for (long i = 0; i < M; i++)
        for (long j = 0; j < N; j++) {
            double sum = 0.0;
            for (long p = 0; p < K; p++)
                sum += (double)a[i * K + p] * (double)b[p * N + j];
            c[i * N + j] = sum;
        }
}

/* The reference's CPU route for one W4A16 GEMM, assembled literally:
 * dequantise the whole matrix (quantize.rs:3642-3659), then the naive GEMM
 * (gemm.rs:162-173).  `scratch` holds K*N floats.  Single thread. */
int twmo_w4a16_literal(const float *a, const uint8_t *packed, const uint16_t *scales, float *c,
                       int M, int N, int K, int group, float *scratch)
{
    if (twmo_dequant_f32(packed, scales, K, N, group, scratch))
        return -1;
    twmo_gemm_f32(a, scratch, c, M, N, K);
    return 0;
}

/* Same arithmetic per output element (dequantise, multiply, f32 accumulate in
 * increasing k, separate multiply and add), but without materialising the
 * matrix and with the columns spread over the host threads.  Each output is
 * bit-identical to twmo_w4a16_literal.  Returns the number of threads used. */
int twmo_w4a16_threaded(const float *a, const uint8_t *packed, const uint16_t *scales, float *c,
                        int M, int N, int K, int group)
{
    int used = 1;
#ifdef _OPENMP
    used = omp_get_max_threads();
#pragma omp parallel for schedule(static)
#endif
    for (long n = 0; n < N; n++) {
        float acc[256];
        int m_done = 0;
        while (m_done < M) {
            int mc = M - m_done < 256 ? M - m_done : 256;
            for (int m = 0; m < mc; m++)
                acc[m] = 0.0f;
            for (long k = 0; k < K; k++) {
                float w = twmo_f16_to_f32(scales[(k / group) * (long)N + n]) *
                          (float)(nibble_at(packed, N, k, n) - 8);
                for (int m = 0; m < mc; m++)
                    acc[m] += a[(long)(m_done + m) * K + k] * w;
            }
            for (int m = 0; m < mc; m++)
                c[(long)(m_done + m) * N + n] = acc[m];
            m_done += mc;
        }
    }
    return used;
}

/* f64-accumulate W4A16 result (adjudicator), threaded. */
void twmo_w4a16_f64acc(const float *a, const uint8_t *packed, const uint16_t *scales, double *c,
                       int M, int N, int K, int group)
{
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
    for (long n = 0; n < N; n++)
        for (long m = 0; m < M; m++) {
            double sum = 0.0;
            for (long k = 0; k < K; k++) {
                double w = (double)twmo_f16_to_f32(scales[(k / group) * (long)N + n]) *
                           (double)(nibble_at(packed, N, k, n) - 8);
                sum += (double)a[m * K + k] * w;
            }
            c[m * N + n] = sum;
        }
}

/* f64-accumulate result with the weights first rounded to f16, fp16_rn(f32(scale) * (nibble - 8)):
 * the operand a tensor-core path feeds its MMA (what dequant_q4_to_f16 produces,
 * crates/kernels/src/quantize.rs:534-571).  Adjudicator for such a path. */
void twmo_w4a16_f64acc_w16(const float *a, const uint8_t *packed, const uint16_t *scales, double *c,
                           int M, int N, int K, int group)
{
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
    for (long n = 0; n < N; n++)
        for (long m = 0; m < M; m++) {
            double sum = 0.0;
            for (long k = 0; k < K; k++) {
                float w32 = twmo_f16_to_f32(scales[(k / group) * (long)N + n]) *
                            (float)(nibble_at(packed, N, k, n) - 8);
                double w = (double)twmo_f16_to_f32(twmo_f32_to_f16(w32));
                sum += (double)a[m * K + k] * w;
            }
            c[m * N + n] = sum;
        }
}

/* The reference's M=1 CUDA kernel restated operation for operation for a K
 * range of 32-blocks [g0,g1): per block gdot = sum_j fma(A[32g+j], nib_j-8, gdot)
 * in increasing j, then dot = fma(gdot, scale, dot)
 * (crates/kernels/src/quantize.rs:1219-1239 and :1274-1292; nvcc contracts
 * `x += a*b` into one fused multiply-add, hence fmaf here).  With g0=0,
 * g1=K/32 this is the value the direct kernel stores (quantize.rs:1296).
 * The scale of block g is scales[(g*32/group)*N + n]; group=32 is the
 * reference's own indexing (quantize.rs:1221). */
void twmo_m1_kernel_order(const float *a, const uint8_t *packed, const uint16_t *scales, float *c,
                          int N, int group, int g0, int g1)
{
#ifdef _OPENMP
#pragma omp parallel for schedule(static)
#endif
    for (long n = 0; n < N; n++) {
        float dot = 0.0f;
        for (long g = g0; g < g1; g++) {
            float scale = twmo_f16_to_f32(scales[(g * 32 / group) * (long)N + n]);
            const uint8_t *blk = packed + (g * N + n) * 16;
            const float *ab = a + g * 32;
            float gdot = 0.0f;
            for (int j = 0; j < 32; j++) {
                int nib = (j & 1) ? (blk[j / 2] >> 4) : (blk[j / 2] & 0x0F);
                gdot = fmaf(ab[j], (float)(nib - 8), gdot);
            }
            dot = fmaf(gdot, scale, dot);
        }
        c[n] = dot;
    }
}

/* ------------------------------------------------------------- host logic -- */

/* The reference's adaptive split-K choice for the M=1 kernel
 * (crates/kernels/src/quantize.rs:1314-1325). */
void twmo_splitk_plan_ref(unsigned n, unsigned k, unsigned *n_blocks_out, unsigned *splits_out,
                          unsigned *k_blocks_per_split_out)
{
    unsigned num_k_groups = k / 32u;
    unsigned threads = 256u;
    unsigned n_blocks = (n + threads - 1u) / threads;
    unsigned splits;
    if (k < 2048u || n_blocks >= 128u) {
        splits = 1u;
    } else {
        unsigned target = 256u;
        unsigned max_splits = num_k_groups / 8u;
        if (max_splits < 1u)
            max_splits = 1u;
        splits = (target + n_blocks - 1u) / n_blocks;
        if (splits < 1u)
            splits = 1u;
        if (splits > max_splits)
            splits = max_splits;
    }
    *n_blocks_out = n_blocks;
    *splits_out = splits;
    *k_blocks_per_split_out = (num_k_groups + splits - 1u) / splits;
}

/* Concatenate TW-Marlin matrices along N, row of blocks by row of blocks
 * (crates/kernels/src/quantize.rs:1038-1055).  `rows` is K/32 for the packed
 * tensor (elem_bytes 16) and K/group for the scales (elem_bytes 2). */
void twmo_fuse_n(const uint8_t *const *srcs, const int *ns, int count, int rows, int elem_bytes,
                 uint8_t *dst)
{
    long total_n = 0;
    for (int i = 0; i < count; i++)
        total_n += ns[i];
    for (long g = 0; g < rows; g++) {
        long col_offset = 0;
        for (int i = 0; i < count; i++) {
            memcpy(dst + (g * total_n + col_offset) * elem_bytes,
                   srcs[i] + g * (long)ns[i] * elem_bytes, (size_t)ns[i] * elem_bytes);
            col_offset += ns[i];
        }
    }
}

/* ------------------------------------------- Q4_0 column blocks -> TW-Marlin -- */

/* reorder_to_tw_marlin, crates/kernels/src/quantize.rs:912-956.  src holds the 20-byte Q4_0
 * blocks [f32 scale][16 bytes of nibbles] of column `col`, 32-block `g` at byte
 * (col * nkb + g) * 20 (the layout every consumer in the reference reads: quantize.rs:217, 554,
 * 726, 932).  The nibble bytes are copied as they are; the scale is rounded to f16
 * (half::f16::from_f32 = round to nearest even).  Scale group 32 only: a Q4_0 block carries
 * one scale per 32 values. */
int twmo_reorder_to_tw_marlin(const uint8_t *src, int K, int N, uint8_t *packed, uint16_t *scales)
{
    if (K < 32 || (K % 32) || N < 1)
        return -1;
    const long nkb = K / 32;
    for (long col = 0; col < N; col++) {
        for (long g = 0; g < nkb; g++) {
            const uint8_t *blk = src + (col * nkb + g) * 20;
            float scale;
            memcpy(&scale, blk, 4);
            scales[g * N + col] = twmo_f32_to_f16(scale);
            memcpy(packed + (g * N + col) * 16, blk + 4, 16);
        }
    }
    return 0;
}

/* The inverse direction of the layout only (not in the reference; used by tests to build
 * column-block inputs from TW-Marlin tensors): scale widened back to f32. */
int twmo_tw_marlin_to_q4_0_blocks(const uint8_t *packed, const uint16_t *scales, int K, int N, uint8_t *dst)
{
    if (K < 32 || (K % 32) || N < 1)
        return -1;
    const long nkb = K / 32;
    for (long col = 0; col < N; col++) {
        for (long g = 0; g < nkb; g++) {
            uint8_t *blk = dst + (col * nkb + g) * 20;
            float scale = twmo_f16_to_f32(scales[g * N + col]);
            memcpy(blk, &scale, 4);
            memcpy(blk + 4, packed + (g * N + col) * 16, 16);
        }
    }
    return 0;
}

/* ------------------------------------------------- batched expert GEMVs (MoE) -- */

/* One expert's M=1 product in the operation order of the reference's batched kernels
 * (crates/kernels/src/moe_batched_marlin.rs:53-69 and 111-127): per 32-block a running sum
 * `gdot += a * (float)(nibble - 8)` over the 32 values in K order, then `dot += gdot * scale`.
 * These are separate multiplies and adds in the source; nvcc contracts them into fused
 * multiply-adds, which is what runs, so fmaf is used here (as in twmo_m1_kernel_order).
 * `group` generalises the scale lookup (32 = the reference). */
static float moe_expert_dot(const float *a, const uint8_t *packed, const uint16_t *scales, int K, int N, int group, long n)
{
    const int nkb = K / 32;
    float dot = 0.0f;
    for (int g = 0; g < nkb; g++) {
        const float scale = twmo_f16_to_f32(scales[(long)((g * 32) / group) * N + n]);
        const uint8_t *blk = packed + ((long)g * N + n) * 16;
        float gdot = 0.0f;
        for (int j = 0; j < 32; j++) {
            const int q = (j & 1) ? (blk[j >> 1] >> 4) : (blk[j >> 1] & 0x0F);
            gdot = fmaf(a[g * 32 + j], (float)(q - 8), gdot);
        }
        dot = fmaf(gdot, scale, dot);
    }
    return dot;
}

/* batched_marlin_gate_up (moe_batched_marlin.rs:21-74): out[e][n] for the top_k experts named
 * (as floats) in topk_ids; one shared input row. */
void twmo_moe_gate_up(const float *a, const uint8_t *packed_base, const uint16_t *scales_base, const float *topk_ids,
                      long packed_bytes_per_expert, long scales_per_expert, int top_k, int K, int N, int group, float *out)
{
    for (int e = 0; e < top_k; e++) {
        const int eid = (int)topk_ids[e];
        const uint8_t *packed = packed_base + (long)eid * packed_bytes_per_expert;
        const uint16_t *scales = scales_base + (long)eid * scales_per_expert;
#pragma omp parallel for schedule(static)
        for (long n = 0; n < N; n++)
            out[(long)e * N + n] = moe_expert_dot(a, packed, scales, K, N, group, n);
    }
}

/* batched_marlin_split_geglu (moe_batched_marlin.rs:138-152): out[e][i] = gelu_tanh(gate) * up. */
void twmo_moe_split_geglu(const float *gate_up, int top_k, int moe_dim, float *out)
{
    for (int e = 0; e < top_k; e++) {
        const float *gu = gate_up + (long)e * 2 * moe_dim;
        for (int i = 0; i < moe_dim; i++) {
            const float g = gu[i], u = gu[moe_dim + i];
            const float gelu_g = 0.5f * g * (1.0f + tanhf(0.7978845608f * (g + 0.044715f * g * g * g)));
            out[(long)e * moe_dim + i] = gelu_g * u;
        }
    }
}

/* batched_marlin_down_axpy (moe_batched_marlin.rs:78-134): acc[n] += weight[e] * dot_e[n].  The
 * reference adds with atomicAdd, in whatever order the experts' CTAs arrive; this restatement
 * adds in slot order e = 0 .. top_k-1 (double accumulation in *acc64 when given, for adjudication). */
void twmo_moe_down_axpy(const float *a_all, long a_stride, const uint8_t *packed_base, const uint16_t *scales_base,
                        const float *topk_ids, const float *topk_weights, long packed_bytes_per_expert,
                        long scales_per_expert, int top_k, int K, int N, int group, float *acc, double *acc64)
{
#pragma omp parallel for schedule(static)
    for (long n = 0; n < N; n++) {
        float s = acc[n];
        double s64 = acc64 ? acc64[n] : 0.0;
        for (int e = 0; e < top_k; e++) {
            const int eid = (int)topk_ids[e];
            const float d = moe_expert_dot(a_all + (long)e * a_stride, packed_base + (long)eid * packed_bytes_per_expert,
                                           scales_base + (long)eid * scales_per_expert, K, N, group, n);
            s += topk_weights[e] * d;
            s64 += (double)topk_weights[e] * (double)d;
        }
        acc[n] = s;
        if (acc64)
            acc64[n] = s64;
    }
}


/* Host threads the threaded routines use from now on (a launcher such as torchrun sets
 * OMP_NUM_THREADS=1 in the environment; the benchmark's CPU arm overrides that with the cores
 * the process may actually run on). */
void twmo_set_num_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int twmo_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
