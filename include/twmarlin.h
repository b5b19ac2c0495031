/*
 * twmarlin.h — C ABI of libtwmarlin: the TW-Marlin W4A16 Q4 GEMM family for
 * NVIDIA B200 (sm_100a), compiled ahead of time.  No JIT, no CPU fallback.
 *
 * Data contract (identical to the reference engine's tensors):
 *   packed : u8  [K/32][N][16]  byte i of a 16-byte block holds the nibble of
 *            k = 32*g + 2*i in its low half and k = 32*g + 2*i + 1 in its high
 *            half (crates/loader/src/gemma_moe_q4.rs:239-249,
 *            crates/kernels/src/quantize.rs:1207-1217,1226).
 *   scales : f16 [K/G][N]       one scale per G consecutive K of a column.
 *            G = 32 is the reference's layout (quantize.rs:1221); G = 128
 *            shares one scale between four consecutive 32-blocks.
 *   weight : w[k][n] = f32(scales[k/G][n]) * (nibble(k,n) - 8).
 *
 * Conventions, as on the reference's Rust entry points
 * (crates/kernels/src/quantize.rs:1301-1360): every pointer is a device
 * pointer owned by the caller; calls only enqueue work on the given stream and
 * never synchronise or allocate, so they are legal during stream capture; the
 * status is returned, nothing aborts.  `stream` is a CUstream / cudaStream_t
 * passed as void* (NULL = legacy default stream).
 */
#ifndef TWMARLIN_H
#define TWMARLIN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum twm_status {
    TWM_OK = 0,
    TWM_EINVAL = -1,     /* bad shape, dtype, null pointer (the reference panics: quantize.rs:1311) */
    TWM_EALIGN = -2,     /* packed not 16-byte aligned, a/c not aligned to their vector width */
    TWM_EWORKSPACE = -3, /* split-K needs more workspace than was passed */
    TWM_ELAUNCH = -4,    /* CUDA reported a launch error (DeviceError::Launch in the reference) */
    TWM_EARCH = -5,      /* the device is not sm_100 */
    TWM_ETIMEOUT = -6    /* a bounded device-side wait expired (reported by twm_device_error) */
} twm_status;

typedef enum twm_dtype { TWM_F32 = 0, TWM_F16 = 1 } twm_dtype;

/* Kernel families twm_plan can choose. */
enum {
    TWM_KERNEL_AUTO = 0,
    TWM_KERNEL_SIMT = 1, /* streaming kernel, FP32 FMA; the only one that takes FP32 activations */
    TWM_KERNEL_TC = 2,   /* tcgen05 kernel: weights dequantised into tensor memory, FP32 accumulate in TMEM */
    TWM_KERNEL_TCW = 4,  /* tcgen05 kernel for many rows (65 .. 128 per launch, group 128, N >= 128): the activation rows
                            are the MMA's M dimension, the unpacked weights its N = 128 */
    TWM_KERNEL_TCR = 5,  /* tcgen05 kernel for many rows and wide matrices (65 .. 256 rows per launch, group 128, no K
                            slices; chosen when N holds at least half a wave of 256-column tiles): the weights enter
                            the tensor core as f16_rn(scale * (q - 8)), the rounding of the reference's own batched
                            route (dequant_q4_to_f16, quantize.rs:534-571), and one FP32 accumulator per 128 rows runs
                            over the whole K.  Every other kernel multiplies exact weights; ask for TWM_KERNEL_TCW to
                            keep them exact at these shapes too. */
    TWM_KERNEL_MMA = 3   /* streaming kernel for up to 32 rows per launch, FP16 activations, warp-level MMA on unpacked
                            registers, 128-column tiles with split-K (inside a thread-block cluster for M <= 2).  Up to
                            eight rows its CTAs stage the activations themselves; from nine rows (and from three on
                            matrices of 2^26 weights or more when the workspace has room) a pre-pass stages them once
                            in the workspace (twm_plan's workspace_bytes says how much) */
};

/* Flags of twm_gemm_args.flags. */
enum {
    /* Launch with programmatic stream serialisation: the kernel may start
     * streaming packed/scales while the kernel before it in the stream is still
     * running, and waits for that kernel only before it reads `a`, the
     * workspace or `c`.  Set it when the weights are constants (the decode
     * loop); leave it clear when the preceding kernel writes packed/scales. */
    TWM_FLAG_PDL = 1,
    TWM_FLAG_ACCUMULATE = 2, /* c += result instead of c = result (residual add fused in the epilogue) */
    /* With TWM_FLAG_PDL: the caller asserts that the kernel launched before this one on the stream
     * neither writes this call's a nor reads or writes its c.  The launch then does not wait for that
     * kernel at all, and the two overlap CTA by CTA.  Honoured by the streaming MMA kernel when its
     * plan needs no workspace (M <= 2); ignored (the launch waits) otherwise.  A decode step has no
     * such pair of GEMMs; the flag exists to measure what the dependency between launches costs.
     * The launch still ends after the kernel ahead of it (one warp waits for that kernel before the
     * CTA exits), so a later kernel that waits for this one has waited for everything before it. */
    TWM_FLAG_INDEPENDENT = 4
};

/* Receive buffers of a tensor-parallel group for the one-shot all-reduce that is fused into
 * the row-parallel GEMM (no counterpart in the reference, whose multi-GPU helper sums on the host,
 * crates/kernels/src/multi_gpu.rs:329-366).  Every rank owns one buffer of twm_comm_bytes() in its
 * own GPU's memory, zeroed once, and knows every rank's buffer address (CUDA IPC between
 * processes: twm_ipc_*).  data[s] / flags[s] / state are produced by twm_comm_layout(). */
typedef struct twm_comm {
    int n_ranks, rank;
    long slot_elems;          /* floats per (set, source rank) slot: >= M * ldc of the GEMMs that use it */
    float* data[8];           /* rank s's slots, as addressable from this rank */
    unsigned int* flags[8];   /* rank s's arrival flags */
    unsigned int* state;      /* this rank's own state words */
    unsigned long long wait_ns; /* how long twm_allreduce_add_rmsnorm waits for the peers' partials before it gives
                                 up, sets the device error word and leaves x untouched; 0 = two seconds */
} twm_comm;

/* One GEMM  C[M,N] = A[M,K] x dequant(packed, scales).
 * Replaces gemm_tw_marlin_m1 (quantize.rs:1301-1360) for M = 1 with f32 A/C,
 * gemm_tw_marlin_m1_from_buffer (quantize.rs:1731-1782; pass offset pointers)
 * and gemm_tw_marlin_m1_indirect (quantize_indirect.rs:228-253; fill the
 * *_offsets fields), and is the M > 1 TW-Marlin GEMM the reference lacks
 * (its stand-in is gemm_q4_0, quantize.rs:1825-1858). */
/* What the activation rows of a GEMM hold (twm_gemm_args.a_prologue, twm_moe_args.a_prologue). */
enum {
    TWM_A_PLAIN = 0,     /* a is f16 (or f32) [M][lda] */
    TWM_A_SILU_MUL = 1,  /* a is f16 [M][lda] holding [gate | up] (up at column K): the GEMM reads
                            silu(gate) * up, rounded to f16 as twm_silu_mul would have stored it
                            (fused_silu_mul, crates/kernels/src/ops.rs:966-977) */
    TWM_A_GEGLU = 2      /* the same with tanh-gelu(gate) * up (batched_marlin_split_geglu,
                            crates/kernels/src/moe_batched_marlin.rs:138-152); not in GEMM chains */
};

typedef struct twm_gemm_args {
    int M, N, K;
    int group_size;          /* 32 or 128; K % group_size == 0 */
    int a_dtype, c_dtype;    /* twm_dtype */
    const void* a;           /* [M, lda] row-major, lda >= K elements */
    long lda;
    const uint8_t* packed;   /* [K/32][N][16], 16-byte aligned */
    const uint16_t* scales;  /* [K/G][N] fp16 bits */
    void* c;                 /* [M, ldc] row-major; every element of [M,N] is written */
    long ldc;
    void* workspace;         /* split-K scratch from twm_workspace_bytes(); may be NULL when 0 bytes are needed.
                                Zero it once after allocation; the kernels leave its counters at zero.
                                One workspace serves one stream at a time.  Without one (or with too small
                                a one) the streaming kernels run a plan that does not split K (slower on
                                small N); TWM_EWORKSPACE is returned only where scratch is indispensable:
                                the tcgen05 kernel, or a split count the caller asked for. */
    size_t workspace_bytes;
    int splits_override;     /* 0 = heuristic */
    int kernel_override;     /* TWM_KERNEL_* ; 0 = heuristic */
    int flags;               /* TWM_FLAG_* */
    /* Device-side expert indirection (quantize_indirect.rs:185-200).  When
     * packed_offsets != NULL the kernel reads packed + packed_offsets[expert_idx]
     * (bytes, multiple of 16) and scales + scales_offsets[expert_idx] (elements). */
    const uint32_t* packed_offsets;
    const uint32_t* scales_offsets;
    int expert_idx;
    /* Tensor-parallel row shard: when comm != NULL the FP32 result is not stored to `c` but pushed
     * into every rank's receive buffer (plain stores over NVLink into the peer's own memory, tile
     * by tile as the tiles finish), and the grid's last storing CTA raises the arrival flags.  The
     * sum is taken by twm_allreduce_add_rmsnorm on each rank.  FP16 activations, M <= 64: one or two
     * rows run on the streaming MMA kernel (one K slice per tile or a cluster reduce), three to 32
     * on its staged-rows form and more rows on the narrow tcgen05 kernel (workspace required for both). */
    const twm_comm* comm;
    /* What the activation rows hold: TWM_A_PLAIN (0) the activations; TWM_A_SILU_MUL / TWM_A_GEGLU: the
     * fused [gate | up] output of the preceding GEMM (2K f16 per row, up at column K, lda >= 2K), and the
     * GEMM multiplies act(gate) * up, computed in FP32 and rounded to f16 exactly as twm_silu_mul would
     * have stored it, so the separate pass and its buffer go away.  M <= 32, FP16 activations, streaming
     * MMA kernel only (TWM_EINVAL otherwise); from two rows on the prologue is applied by that kernel's
     * staging pre-pass, so the workspace must hold the staged rows (twm_workspace_bytes covers it). */
    int a_prologue;
    /* Optional: the GEMM that will be enqueued after this one (on this stream, other kernels may come
     * between).  Read during this call only.  While this GEMM's grid drains, its CTAs ask the memory
     * system to pull the first K blocks of that GEMM's weights (up to 16 MB, the part its CTAs start
     * with under its own plan) into L2, so HBM keeps streaming across the launch boundary and the next
     * GEMM starts from L2.  A hint: results never depend on it.  Streaming MMA kernel only. */
    const struct twm_gemm_args* next;
} twm_gemm_args;

/* What the heuristic decided for a shape; pure host arithmetic. */
typedef struct twm_plan_t {
    int kernel;          /* the TWM_KERNEL_* that will run */
    int n_tile;          /* columns per CTA */
    int splits;          /* K slices; 1 = no workspace traffic */
    int blocks_per_split;/* 32-blocks of K per slice (last slice may be shorter) */
    int grid_x, grid_y;  /* n tiles, splits */
    size_t workspace_bytes;
    int cluster_reduce;  /* 1: the K slices of a tile run as one thread-block cluster and add up in
                            distributed shared memory; no workspace is touched */
} twm_plan_t;

/* Replaces the adaptive split-K arithmetic of quantize.rs:1314-1325, re-derived
 * for 148 SMs.  sm_count <= 0 means 148.  Deterministic: the same arguments
 * always give the same plan, so a plan made before graph capture stays valid. */
twm_status twm_plan(int M, int N, int K, int group_size, int sm_count, int splits_override,
                    int kernel_override, twm_plan_t* out);

/* Workspace twm_gemm_w4a16 needs for this shape with the heuristic's own split
 * count on a 148-SM device (0 when it does not split).  With splits_override
 * ask twm_plan for the exact figure. */
size_t twm_workspace_bytes(int M, int N, int K, int group_size);

/* Enqueue one GEMM.  See twm_gemm_args. */
twm_status twm_gemm_w4a16(const twm_gemm_args* args, void* stream);

/* Bytes of one rank's receive buffer, and the addresses inside a buffer that starts at `base`
 * (`base` may be a peer's buffer as mapped into this process). */
size_t twm_comm_bytes(int n_ranks, long slot_elems);
twm_status twm_comm_layout(void* base, int n_ranks, long slot_elems, float** data, unsigned int** flags,
                           unsigned int** state);

/* Second half of the one-shot all-reduce, fused with the residual add and RMSNorm that follow a
 * row-parallel GEMM (fused_residual_rmsnorm, crates/kernels/src/ops.rs:928-962): waits, with a
 * bound, for every rank's partial, x += sum over ranks in rank order, y = rmsnorm(x) (y_f16 may be
 * NULL).  Every rank must enqueue the same sequence of comm GEMMs and of these calls. */
twm_status twm_allreduce_add_rmsnorm(void* y_f16, float* x, const twm_comm* comm, const float* gamma, int rows,
                                     int hidden, float eps, int flags, void* stream);

/* Device memory that other processes on the same box can map (CUDA IPC): allocation (zeroed),
 * 64-byte handle, mapping a peer's handle, and their inverses.  Set-up calls: they allocate and
 * synchronise. */
twm_status twm_ipc_alloc(size_t bytes, void** ptr);
twm_status twm_ipc_free(void* ptr);
twm_status twm_ipc_get_handle(void* ptr, unsigned char handle[64]);
twm_status twm_ipc_open(const unsigned char handle[64], void** ptr);
twm_status twm_ipc_close(void* ptr);

/* ---- A list of GEMMs as one persistent launch ------------------------------------------------
 * The reference's decode step enqueues its GEMMs one kernel at a time
 * (forward_decode_tw_marlin_graph, crates/kernels/src/generate.rs:2149-2206, each through
 * gemm_tw_marlin_m1, quantize.rs:1301-1360).  A chain takes the same list of GEMMs and runs it as
 * ONE cooperative kernel: GEMM i sees everything GEMMs 0..i-1 wrote, exactly as if they had been
 * enqueued one after another on the stream, but the packed weights of GEMM i+1 are already
 * streaming into shared memory while GEMM i finishes; only the reader of a GEMM's activations
 * waits (bounded, on a counter in device memory) for the GEMM that produces them.
 * Restrictions: M <= 8, FP16 activations, no expert indirection, no peer push.
 *
 * twm_chain_create is a set-up call: it allocates the chain's device memory (GEMM table, split
 * partials, counters; twm_chain_info reports the size) and synchronises.  twm_chain_launch only
 * enqueues and is legal during stream capture.  One chain runs on one stream at a time. */
typedef struct twm_chain_op {
    twm_gemm_args gemm;  /* workspace, *_override, *_offsets and comm must be zero; a_prologue TWM_A_PLAIN or
                            TWM_A_SILU_MUL (here with M up to 8); flags: TWM_FLAG_ACCUMULATE, and
                            TWM_FLAG_INDEPENDENT = this GEMM reads nothing an earlier GEMM of the chain
                            writes (it does not wait; a later dependent GEMM still waits for it and for
                            everything before it) */
} twm_chain_op;

typedef struct twm_chain twm_chain;      /* opaque */

typedef struct twm_chain_info_t {
    int count;           /* GEMMs */
    int grid;            /* CTAs of the launch (resident CTAs per SM x SMs) */
    int rows;            /* activation rows staged per GEMM (power of two >= the largest M) */
    size_t device_bytes; /* device memory the chain holds */
    int split_tiles;     /* tiles that are summed through partials, over the whole chain */
    int max_pieces;      /* most pieces any tile is cut into */
} twm_chain_info_t;

twm_status twm_chain_create(const twm_chain_op* ops, int count, twm_chain** out);
twm_status twm_chain_launch(twm_chain* chain, void* stream);
twm_status twm_chain_info(const twm_chain* chain, twm_chain_info_t* out);
twm_status twm_chain_destroy(twm_chain* chain);

/* How a chain deals one GEMM to its CTAs (pure host arithmetic, the same code the kernel runs):
 * the pieces (tile, first and last+1 32-block of K, index of the piece within its tile, pieces of
 * that tile) of `rank` out of `grid` for a GEMM of n_tiles x nkb 32-blocks.  Writes at most
 * `max_out` entries of five ints each and returns the count in *n_out. */
twm_status twm_chain_partition(int n_tiles, int nkb, int grid, int rank, int max_out, int* out5, int* n_out);

/* ---- Batched expert GEMVs of a mixture-of-experts layer, M = 1 --------------------------------
 * Replace batched_marlin_gate_up, batched_marlin_split_geglu and batched_marlin_down_axpy
 * (crates/kernels/src/moe_batched_marlin.rs:21-233): all top_k chosen experts in one launch, the
 * choice read on the device (topk_ids holds expert numbers as floats, as the reference's router
 * writes them), so no host round trip.  All experts' TW-Marlin tensors lie in two buffers,
 * expert e at packed_base + e * packed_bytes_per_expert and scales_base + e * scales_per_expert.
 * Differences from the reference: activations and gate+up outputs are FP16 (as everywhere in
 * this library); the gated activation is computed by the down GEMV as it reads [gate | up], so
 * there is no separate split/GEGLU pass; the weighted sum over experts is added in slot order
 * (inside a thread-block cluster, or through the workspace when K slices x top_k exceeds a
 * cluster), never with atomics, so it gives the same bits every run. */
typedef struct twm_moe_args {
    int top_k;                   /* experts chosen for this token */
    int N, K, group_size;        /* every expert's matrix is [K, N] */
    const void* a;               /* f16.  a_slot_stride = 0: one row shared by all slots (gate+up);
                                    otherwise slot s reads a + s * a_slot_stride.  With a_prologue
                                    SILU_MUL / GEGLU a row is [gate | up] of 2K values. */
    long a_slot_stride;
    int a_prologue;              /* TWM_A_* */
    const uint8_t* packed_base;
    const uint16_t* scales_base;
    size_t packed_bytes_per_expert;   /* multiple of 16 */
    size_t scales_per_expert;         /* elements */
    const float* topk_ids;       /* device, [top_k] */
    const float* topk_weights;   /* device, [top_k]: twm_moe_down_axpy only (NULL for twm_moe_gate_up) */
    void* c;                     /* gate_up: slot s writes c + s * c_slot_stride ([N] values);
                                    down_axpy: one row [N] = sum over slots of weight * product
                                    (added to what c holds with TWM_FLAG_ACCUMULATE) */
    int c_dtype;
    long c_slot_stride;
    void* workspace;             /* twm_moe_workspace_bytes(); zeroed once; may be NULL when that is 0 */
    size_t workspace_bytes;
    int flags;                   /* TWM_FLAG_PDL, TWM_FLAG_ACCUMULATE */
} twm_moe_args;

size_t twm_moe_workspace_bytes(int top_k, int N, int K, int group_size);
twm_status twm_moe_gate_up(const twm_moe_args* args, void* stream);
twm_status twm_moe_down_axpy(const twm_moe_args* args, void* stream);

/* The same GEMM for hosts that cannot give this library any device memory of its own:
 * an engine that carves the whole GPU into weights and KV cache at start-up and has no
 * allocator left to ask, or a plugin slot whose contract forbids allocation calls once
 * serving has begun.  Such a caller cannot create the split-K workspace twm_gemm_w4a16
 * wants, so this entry point brings its own: a fixed 8 MiB array (twm_static_ws_capacity())
 * inside the library's device image, present on every GPU that loads the library for as
 * long as the process lives.  It has no counterpart in the reference, whose split-K adds
 * into C with atomics and needs no scratch.
 *
 * args->workspace and args->workspace_bytes are ignored; inputs and outputs are the
 * caller's as before.  The call allocates and frees nothing (no cudaMalloc, no pool).
 * A shape whose split-K plan needs more than the array holds returns TWM_EWORKSPACE with
 * the two sizes in twm_last_error().  The first call on each device looks the array's
 * address up (one cudaGetSymbolAddress with that device current); make that first call
 * before starting any stream capture.  All calls on a device share the one array and it
 * keeps the previous call's contents: the counters are cleared on the stream before every
 * launch, and two calls that can overlap on the GPU (different streams) race on it, so
 * serialise them. */
twm_status twm_gemm_w4a16_static_ws(const twm_gemm_args* args, void* stream);

/* Bytes of the built-in scratch array used by twm_gemm_w4a16_static_ws. */
size_t twm_static_ws_capacity(void);

/* Dequantise to a dense [K,N] row-major matrix, f32 (exact) or f16 (round to
 * nearest even of the f32 product).  Replaces warp_dequantize_q4_0 /
 * dequant_q4_to_f16 (quantize.rs:150-175, 534-618) on the TW-Marlin tensors. */
twm_status twm_dequant(const uint8_t* packed, const uint16_t* scales, void* out, int out_dtype,
                       int K, int N, int group_size, void* stream);

/* Quantise + pack on the device.  w is f32, [K,N] row-major when w_is_nk == 0
 * (quantize_f32_to_tw_marlin, quantize.rs:1171-1180) or [N,K] row-major when
 * w_is_nk != 0 (cpu_quantize_tw_marlin, gemma_moe_q4.rs:218-254).  Same bytes
 * as the reference's CPU quantiser for group_size 32. */
twm_status twm_quantize_pack(const float* w, int w_is_nk, int K, int N, int group_size,
                             uint8_t* packed, uint16_t* scales, void* stream);

/* Column-major Q4_0 blocks -> TW-Marlin, on the device.  col_major_q4 holds the 20-byte blocks
 * [f32 scale][16 nibble bytes] of column c, 32-block g at byte (c * K/32 + g) * 20, the layout every
 * consumer in the reference reads (quantize.rs:217, 554, 726, 932).  Writes packed [K/32][N][16]
 * and f16 scales [K/32][N] (scale group 32: a Q4_0 block has one scale per 32 values).  Replaces
 * reorder_to_tw_marlin (quantize.rs:912-956), which copies to the host, permutes and uploads. */
twm_status twm_reorder_to_tw_marlin(const uint8_t* col_major_q4, int K, int N, uint8_t* packed, uint16_t* scales,
                                    void* stream);

/* Concatenate `count` TW-Marlin matrices along N (fuse_tw_marlin_n,
 * quantize.rs:1018-1063).  packed_srcs/scales_srcs/ns are HOST arrays of
 * device pointers / widths; dst tensors hold sum(ns) columns. */
twm_status twm_fuse_n(const uint8_t* const* packed_srcs, const uint16_t* const* scales_srcs,
                      const int* ns, int count, int K, int group_size, uint8_t* packed_dst,
                      uint16_t* scales_dst, void* stream);

/* Column slice [n0, n0+n_len) of a TW-Marlin matrix (tensor-parallel column
 * shard; the inverse of twm_fuse_n). */
twm_status twm_slice_n(const uint8_t* packed_src, const uint16_t* scales_src, int K, int N,
                       int group_size, int n0, int n_len, uint8_t* packed_dst,
                       uint16_t* scales_dst, void* stream);

/* Row slice [k0, k0+k_len) of a TW-Marlin matrix (tensor-parallel row shard);
 * k0 and k_len are multiples of group_size.  The slice is contiguous, so this
 * only returns the byte/element offsets. */
twm_status twm_slice_k_offsets(int K, int N, int group_size, int k0, int k_len,
                               size_t* packed_byte_offset, size_t* scales_elem_offset);

const char* twm_status_string(twm_status s);

/* Read and clear the device-side error word.  SYNCHRONISES the stream, so it
 * is a diagnostic for after a step, not for inside a capture.  *word: bit 0 an
 * mbarrier wait ran out, bit 1 a split-K wait, bit 2 a peer-flag wait.
 * Returns TWM_ETIMEOUT when the word was non-zero. */
twm_status twm_device_error(void* stream, unsigned int* word);

/* Text of the last CUDA error this thread saw inside libtwmarlin ("" if none). */
const char* twm_last_error(void);

/* Library build tag, e.g. "twmarlin sm_100a". */
const char* twm_version(void);

#ifdef __cplusplus
}
#endif
#endif /* TWMARLIN_H */
