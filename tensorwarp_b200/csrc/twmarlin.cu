// twmarlin.cu — the C ABI of libtwmarlin (see include/twmarlin.h) and the host
// logic behind it: argument checks, the tile / split-K plan, launches.
//
// Host-side counterpart of the reference's launcher gemm_tw_marlin_m1
// (crates/kernels/src/quantize.rs:1301-1360) and of its layout helpers
// (quantize.rs:1018-1063, 1171-1180).  One translation unit: every kernel
// header is included here so that no relocatable device code is needed.
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "twm_common.cuh"
#include "twm_gemv_simt.cuh"
#include "twm_gemm_tc.cuh"
#include "twm_gemm_tcw.cuh"
#include "twm_gemm_tcr.cuh"
#include "twm_gemv_mma.cuh"
#include "twm_chain.cuh"
#include "twm_layout.cuh"
#include "twm_decode_ops.cuh"
#include "../../include/twm_decode.h"

namespace {

thread_local char t_last_error[256] = "";

void set_error(const char* where, cudaError_t e)
{
    snprintf(t_last_error, sizeof(t_last_error), "%s: %s", where, cudaGetErrorString(e));
}

constexpr int kMaxDevices = 64;
constexpr int kDefaultSms = 148;
constexpr int kMaxSplits = 64;
constexpr size_t kCounterBytes = 16384;   // 4096 tile counters at the head of the workspace

// Dynamic shared memory of a tcgen05 launch.  Each CTA allocates 256 of the SM's 512 tensor-memory
// columns, so at most two fit; asking for at least 80 KB keeps a third CTA off the SM (it would
// sit in tcgen05.alloc until another CTA ends, and the SMs would finish unevenly).
size_t tc_smem_bytes(int rows)
{
    const size_t need = rows <= 16 ? sizeof(twm::tc::Smem<16>) : (rows <= 32 ? sizeof(twm::tc::Smem<32>) : sizeof(twm::tc::Smem<64>));
    return std::max(need, (size_t)80 * 1024);
}

struct DeviceState {
    bool ready = false;
    twm_status status = TWM_OK;
    int sm_count = kDefaultSms;
};
DeviceState g_dev[kMaxDevices];
std::mutex g_dev_mutex;

// Once per device: check the architecture and raise the dynamic shared memory
// limit of every kernel that needs more than 48 KB.
twm_status ensure_device(int* sm_count_out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { set_error("cudaGetDevice", e); return TWM_ELAUNCH; }
    if (dev < 0 || dev >= kMaxDevices) return TWM_EINVAL;
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceState& st = g_dev[dev];
    if (!st.ready) {
        int major = 0, sms = 0;
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        st.sm_count = sms > 0 ? sms : kDefaultSms;
        if (major != 10) {
            snprintf(t_last_error, sizeof(t_last_error), "device %d is sm_%d*, libtwmarlin holds sm_100a code only", dev, major);
            st.status = TWM_EARCH;
        } else {
            const int smem = (int)sizeof(twm::simt::Smem);
            cudaError_t r = cudaSuccess;
            auto raise = [&](const void* fn) {
                if (r == cudaSuccess) r = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
            };
            raise((const void*)twm::simt::gemv_kernel<1>);
            raise((const void*)twm::simt::gemv_kernel<2>);
            raise((const void*)twm::simt::gemv_kernel<4>);
            raise((const void*)twm::simt::gemv_kernel<8>);
            auto raise_tc = [&](const void* fn, size_t bytes) {
                if (r == cudaSuccess)
                    r = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
            };
            raise_tc((const void*)twm::tc::gemm_kernel<16>, tc_smem_bytes(16));
            raise_tc((const void*)twm::tc::gemm_kernel<32>, tc_smem_bytes(32));
            raise_tc((const void*)twm::tc::gemm_kernel<64>, tc_smem_bytes(64));
            raise_tc((const void*)twm::tcw::gemm_kernel, sizeof(twm::tcw::Smem));
            raise_tc((const void*)twm::tcr::gemm_kernel<1>, sizeof(twm::tcr::Smem<1>));
            raise_tc((const void*)twm::tcr::gemm_kernel<2>, sizeof(twm::tcr::Smem<2>));
            auto raise_mma = [&](const void* fn) {
                if (r == cudaSuccess)
                    r = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(twm::mma::Smem));
                if (r == cudaSuccess)      // clusters of up to 16 K slices
                    r = cudaFuncSetAttribute(fn, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            };
            raise_mma((const void*)twm::mma::gemv_kernel<1, 0>);
            raise_mma((const void*)twm::mma::gemv_kernel<2, 0>);
            raise_mma((const void*)twm::mma::gemv_kernel<4, 0>);
            raise_mma((const void*)twm::mma::gemv_kernel<8, 0>);
            raise_mma((const void*)twm::mma::gemv_kernel<1, 2>);
            raise_mma((const void*)twm::mma::gemv_kernel<2, 2>);
            raise_mma((const void*)twm::mma::gemv_kernel<4, 2>);
            raise_mma((const void*)twm::mma::gemv_kernel<8, 2>);
            raise_mma((const void*)twm::mma::gemv_kernel<1, 0, 1>);      // expert GEMVs reading [gate | up]
            raise_mma((const void*)twm::mma::gemv_kernel<1, 0, 2>);
            raise_mma((const void*)twm::mma::gemv_kernel<1, 2, 1>);
            raise_mma((const void*)twm::mma::gemv_kernel<1, 2, 2>);
            auto raise_rows = [&](const void* fn, size_t bytes) {
                if (r == cudaSuccess) r = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
            };
            raise_rows((const void*)twm::mma::gemm_rows_kernel<8, 0>, sizeof(twm::mma::RowsSmem<8>));
            raise_rows((const void*)twm::mma::gemm_rows_kernel<8, 2>, sizeof(twm::mma::RowsSmem<8>));
            raise_rows((const void*)twm::mma::gemm_rows_kernel<16, 0>, sizeof(twm::mma::RowsSmem<16>));
            raise_rows((const void*)twm::mma::gemm_rows_kernel<16, 2>, sizeof(twm::mma::RowsSmem<16>));
            raise_rows((const void*)twm::mma::gemm_rows_kernel<24, 0>, sizeof(twm::mma::RowsSmem<24>));
            raise_rows((const void*)twm::mma::gemm_rows_kernel<24, 2>, sizeof(twm::mma::RowsSmem<24>));
            raise_rows((const void*)twm::mma::gemm_rows_kernel<32, 0>, sizeof(twm::mma::RowsSmem<32>));
            raise_rows((const void*)twm::mma::gemm_rows_kernel<32, 2>, sizeof(twm::mma::RowsSmem<32>));
            raise_rows((const void*)twm::ops::attn_span_mma_kernel<128, true>, twm::ops::ATT_MMA_SMEM_BYTES);
            raise_rows((const void*)twm::ops::attn_span_mma_kernel<128, false>, twm::ops::ATT_MMA_SMEM_BYTES);
            auto raise_chain = [&](const void* fn) {
                if (r == cudaSuccess)
                    r = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(twm::chain::Smem));
            };
            raise_chain((const void*)twm::chain::chain_kernel<1>);
            raise_chain((const void*)twm::chain::chain_kernel<2>);
            raise_chain((const void*)twm::chain::chain_kernel<4>);
            raise_chain((const void*)twm::chain::chain_kernel<8>);
            if (r != cudaSuccess) { set_error("cudaFuncSetAttribute", r); st.status = TWM_ELAUNCH; }
        }
        st.ready = true;
    }
    if (sm_count_out) *sm_count_out = st.sm_count;
    return st.status;
}

// cuTensorMapEncodeTiled, fetched from the driver once (the library links the runtime only).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_tiled()
{
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

// Tensor map over packed viewed as u64 [K/32 rows][2N]: box = 2 * `cols` u64 x `rows`.
// Returns false when the map cannot be made (the kernels then copy row by row).
bool make_packed_map(CUtensorMap* map, const uint8_t* packed, int N, int nkb, int rows, int cols = 128)
{
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) return false;
    const cuuint64_t gdim[2] = {(cuuint64_t)N * 2, (cuuint64_t)nkb};
    const cuuint64_t gstride[1] = {(cuuint64_t)N * 16};
    const cuuint32_t box[2] = {(cuuint32_t)cols * 2, (cuuint32_t)rows};
    const cuuint32_t estride[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<uint8_t*>(packed), gdim, gstride, box, estride,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Tensor map over the permuted activations of one tcgen05 launch, f16 [K/8][rows][8], seen as
// 32-bit words [K/8][rows * 4]: a box of nb_rows * 4 words x 16 K cores is one ring stage (four
// 32-blocks) landing as [K core][row][16 bytes]; words past rows * 4 read as zero.
bool make_act_map(CUtensorMap* map, const void* xp, int rows, int K, int nb_rows)
{
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) return false;
    const cuuint64_t gdim[2] = {(cuuint64_t)rows * 4, (cuuint64_t)K / 8};
    const cuuint64_t gstride[1] = {(cuuint64_t)rows * 16};
    const cuuint32_t box[2] = {(cuuint32_t)nb_rows * 4, (cuuint32_t)twm::tc::B_STAGE_KCORES};
    const cuuint32_t estride[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(xp), gdim, gstride, box, estride,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Tensor map over the permuted activations of one wide tcgen05 launch, f16 [K/8][rows][8], seen as
// 64-bit words [K/8][rows * 2]: a box of 256 words x 16 K cores is one scale group of 128 K for
// 128 rows, landing as [K core][row][16 bytes]; rows past `rows` read as zero.
bool make_act_map_wide(CUtensorMap* map, const void* xp, int rows, int K, int kcores = twm::tcw::A_KCORES)
{
    EncodeTiledFn enc = get_encode_tiled();
    if (!enc) return false;
    const cuuint64_t gdim[2] = {(cuuint64_t)rows * 2, (cuuint64_t)K / 8};
    const cuuint64_t gstride[1] = {(cuuint64_t)rows * 16};
    const cuuint32_t box[2] = {(cuuint32_t)twm::tcw::MB * 2, (cuuint32_t)kcores};
    const cuuint32_t estride[2] = {1, 1};
    return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT64, 2, const_cast<void*>(xp), gdim, gstride, box, estride,
               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool shape_ok(int M, int N, int K, int G)
{
    return M >= 1 && N >= 1 && K >= 32 && (G == 32 || G == 128) && (K % G) == 0 && (K % 32) == 0 &&
           (long long)((N + twm::simt::NT - 1) / twm::simt::NT) <= (long long)(kCounterBytes / 4);
}

// Choose the number of K slices for the streaming kernel.  Costs are counted in
// units of one 32-block of one tile (2 KB of packed weights): a CTA pays a
// fixed start-up (barrier init, activation staging, warp reduce) worth about
// 16 such blocks, and a split tile pays the last-arriver's pass over the
// partials.  `slots` = CTAs that can be resident at once.
// `cluster` = the slices of a tile will be launched as one thread-block cluster.  A cluster
// lives inside one GPC (8 GPCs share the SMs), so a slice count that does not pack into a
// GPC's CTA slots costs a second wave: that is counted here.
void choose_splits(int n_tiles, int nkb, int slots, int sm_count, int max_bps, int align, int max_splits, bool cluster,
                   int* splits, int* bps)
{
    double best = 1e30;
    int best_s = 1, best_bps = nkb;
    const int smax = std::min(max_splits, nkb);
    for (int s = 1; s <= smax; ++s) {
        int b = (nkb + s - 1) / s;
        b = (b + align - 1) / align * align;     // slices of whole scale groups where the kernel wants them
        if (b > max_bps && s < smax) continue;   // the kernel's per-slice staging capacity
        const int s_eff = (nkb + b - 1) / b;
        if (s_eff != s) continue;   // same slicing as a smaller s
        const long ctas = (long)n_tiles * s_eff;
        long waves = (ctas + slots - 1) / slots;
        if (cluster && s_eff > 1) {
            // Measured on B200: the CTAs of a cluster land on s distinct SMs of one GPC, one CTA
            // slot "layer" at a time, so a GPC of 18 SMs with two slots per SM holds
            // 2 * floor(18 / s) clusters (4 of size 7, not 5).
            const int sms_per_gpc = sm_count / 8;
            const long resident_clusters = 8L * (slots / sm_count) * (sms_per_gpc / s_eff);
            if (resident_clusters == 0) continue;
            waves = std::max(waves, ((long)n_tiles + resident_clusters - 1) / resident_clusters);
        }
        // Every wave after the first starts from empty rings on SMs that have just been vacated (no weights
        // streamed in ahead of it): measured, about 40 blocks' worth.  K=28672 N=8192, one row: 9 slices (two
        // waves of clusters) 33.3 us, 4 slices (one wave) 27.5; K=8192 N=57344: 3 slices 59.3 us, none 57.6.
        double cost = (double)waves * (b + 16.0) + (double)(waves - 1) * 40.0;
        if (s_eff > 1) cost += 10.0 + 0.25 * s_eff;
        if (cost < best - 1e-9) { best = cost; best_s = s_eff; best_bps = b; }
    }
    *splits = best_s;
    *bps = best_bps;
}

int mmax_for(int M) { return M <= 1 ? 1 : (M <= 2 ? 2 : (M <= 4 ? 4 : 8)); }
// activation rows one launch of the streaming MMA kernel carries: up to eight staged by the CTAs themselves,
// 16, 24 or 32 through the staging pre-pass
int mma_rows_for(int M) { return M <= 8 ? 8 : (M <= 16 ? 16 : (M <= 24 ? 24 : 32)); }
// Whether a launch of `rows` rows goes through the staging pre-pass.  From nine rows it must (the CTAs' own stager
// warps stop at eight).  For three to eight rows both work: measured (us per GEMM, pre-pass / stager warps) on
// K=3584 N=37888: 15.0 / 16.2 at 3 rows, 15.3 / 19.6 at 8; K=18944 N=3584: 15.3 / 15.4 and 15.8 / 17.0; but
// K=3584 N=4608: 9.1 / 8.5 and 9.7 / 8.9 (the extra launch costs 0.6-0.8 us), hence the size threshold.
bool mma_prepass(int rows, long K, long N) { return rows >= 9 || (rows >= 3 && K * N >= (1L << 26)); }
// bytes of the staging pre-pass's output for `rows` rows: B fragments, then group sums
size_t mma_rows_b_bytes(int rows, int K) { return (size_t)(K / 32) * mma_rows_for(rows) * 64; }
size_t mma_rows_stage_bytes(int rows, int K, int group) { return mma_rows_b_bytes(rows, K) + (size_t)(K / group) * mma_rows_for(rows) * 4; }

// Measured (us per launch in a dependent chain, streaming MMA kernel / narrow tcgen05 kernel): 7B gate+up shape
// 15.3 / 24.5 at 8 rows, 19.2 / 25.5 at 16, 30.7 / 31.2 at 32; K=3584 N=4608: 8.9 / 18.2, 13.3 / 27.5 and
// 18.0 / 48.7 (the latter before its K-slice sum was pipelined); K=18944 N=3584: 17.0 / 27.2, 20.4 / 37.9, 31.9 / 62.6.
constexpr int kTcFromRows = 33;
// Measured on the 7B gate+up shape: 64 rows 51.6 us on the weight-stationary kernel against 58.0 on the wide one,
// 96 rows 76 against 59, 128 rows 79 (as two launches of 64; one launch with a 128-row accumulator was no faster) against 60.
constexpr int kTcwFromRows = 65;
int auto_kernel(int M, int N, int K, int G, bool a_is_f16, bool indirect, int splits_override)
{
    if (!a_is_f16) return TWM_KERNEL_SIMT;
    (void)K;
    // many rows: rows on the MMA's M dimension; group 128 and full 128-column tiles.  Wide matrices (at least half
    // a wave of 256-column tiles, no K slices asked for) take the 256-column kernel, whose weights enter the tensor
    // core rounded to FP16 as in the reference's batched route; the others the exact-weight kernel, which can split K.
    if (M >= kTcwFromRows && G == 128 && N >= 128 && !indirect) {
        // Measured on K=3584 (us, 128 / 256 rows): N=37888: tcr 43 / 60, tcw 56 / 111; N=28416: 44 / 60 against 56 / 112;
        // N=18944: 44 / 59 against 32 / 60; N=9472: 42 / 56 against 30 / 60; N=4608: 41 / 55 against 29 / 59.  And K=18944,
        // N=3584: tcr 182 (14 tiles, no K slices), tcw 64 in five slices.  So: more than one wave of 128-column
        // tiles, or more than 128 rows, goes to the 256-column kernel unless K is long and the tiles are few.
        const int tiles_w = (N + twm::tcw::NT - 1) / twm::tcw::NT, tiles_r = (N + twm::tcr::NT - 1) / twm::tcr::NT;
        const bool long_k_few_tiles = K >= 8192 && 4 * tiles_r <= kDefaultSms;
        const bool wide = (tiles_w > kDefaultSms || M > twm::tcw::MB) && !long_k_few_tiles && splits_override <= 1;
        return wide ? TWM_KERNEL_TCR : TWM_KERNEL_TCW;
    }
    // the streaming kernel reads per-expert offset tables only with its own stager warps (up to eight rows)
    return (M >= kTcFromRows || (M > 8 && indirect)) ? TWM_KERNEL_TC : TWM_KERNEL_MMA;
}

int resolve_kernel(const twm_gemm_args* a)
{
    if (a->kernel_override != TWM_KERNEL_AUTO) return a->kernel_override;
    int kernel = auto_kernel(a->M, a->N, a->K, a->group_size, a->a_dtype == TWM_F16, a->packed_offsets != nullptr,
                             a->splits_override);
    // pushing to tensor-parallel peers: the streaming kernel's cluster leaders push one or two rows, its
    // pre-pass form three to 32, the narrow tcgen05 kernel's read-back warps up to 64
    if (a->comm && a->a_dtype == TWM_F16) return a->M < kTcFromRows ? TWM_KERNEL_MMA : TWM_KERNEL_TC;
    return kernel;
}

constexpr int kTcRows = 64;      // activation rows one tcgen05 launch carries
constexpr int kTcwRows = twm::tcw::MB;   // ... and one wide tcgen05 launch
constexpr int kTcrRows = 2 * twm::tcr::MB;   // ... and one 256-column tcgen05 launch (two blocks of 128 rows)

twm_status launch_tcw(const twm::GemmParams& p, dim3 grid, bool pdl, cudaStream_t stream)
{
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = dim3(twm::tcw::THREADS, 1, 1);
    cfg.dynamicSmemBytes = sizeof(twm::tcw::Smem);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, twm::tcw::gemm_kernel, p);
    if (e != cudaSuccess) { set_error("launch tcw::gemm_kernel", e); return TWM_ELAUNCH; }
    return TWM_OK;
}

twm_status launch_tcr(const twm::GemmParams& p, int rows, dim3 grid, bool pdl, cudaStream_t stream)
{
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = dim3(twm::tcr::THREADS, 1, 1);
    cfg.dynamicSmemBytes = rows > twm::tcr::MB ? sizeof(twm::tcr::Smem<2>) : sizeof(twm::tcr::Smem<1>);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e = rows > twm::tcr::MB ? cudaLaunchKernelEx(&cfg, twm::tcr::gemm_kernel<2>, p)
                                        : cudaLaunchKernelEx(&cfg, twm::tcr::gemm_kernel<1>, p);
    if (e != cudaSuccess) { set_error("launch tcr::gemm_kernel", e); return TWM_ELAUNCH; }
    return TWM_OK;
}

twm_status launch_tc(const twm::GemmParams& p, int rows, dim3 grid, bool pdl, cudaStream_t stream)
{
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = dim3(rows <= 32 ? twm::tc::Cfg<32>::THREADS : twm::tc::Cfg<64>::THREADS, 1, 1);
    cfg.dynamicSmemBytes = tc_smem_bytes(rows);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e;
    if (rows <= 16) e = cudaLaunchKernelEx(&cfg, twm::tc::gemm_kernel<16>, p);
    else if (rows <= 32) e = cudaLaunchKernelEx(&cfg, twm::tc::gemm_kernel<32>, p);
    else e = cudaLaunchKernelEx(&cfg, twm::tc::gemm_kernel<64>, p);
    if (e != cudaSuccess) { set_error("launch tc::gemm_kernel", e); return TWM_ELAUNCH; }
    return TWM_OK;
}

twm_status launch_mma(const twm::GemmParams& p, int mp, dim3 grid, bool pdl, cudaStream_t stream)
{
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = dim3(twm::mma::threads_for(mp), 1, 1);       // more stager warps from four rows on
    cfg.dynamicSmemBytes = sizeof(twm::mma::Smem);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (pdl) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (p.cluster_reduce) {          // the K slices of one tile (grid y) form one cluster;
        attr[na].id = cudaLaunchAttributeClusterDimension;      // with a weighted expert sum, so do the slots (grid z)
        attr[na].val.clusterDim.x = 1;
        attr[na].val.clusterDim.y = grid.y;
        attr[na].val.clusterDim.z = (p.n_experts && p.expert_weights) ? grid.z : 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    cudaError_t e;
    if (p.a_kind != 0) {            // gated-activation prologue: one activation row only (expert GEMVs)
        if (mp != 1) return TWM_EINVAL;
        if (p.group == 128) e = p.a_kind == 1 ? cudaLaunchKernelEx(&cfg, twm::mma::gemv_kernel<1, 2, 1>, p)
                                              : cudaLaunchKernelEx(&cfg, twm::mma::gemv_kernel<1, 2, 2>, p);
        else e = p.a_kind == 1 ? cudaLaunchKernelEx(&cfg, twm::mma::gemv_kernel<1, 0, 1>, p)
                               : cudaLaunchKernelEx(&cfg, twm::mma::gemv_kernel<1, 0, 2>, p);
    } else if (p.group == 128) {
        switch (mp) {
            case 1: e = cudaLaunchKernelEx(&cfg, twm::mma::gemv_kernel<1, 2>, p); break;
            case 2: e = cudaLaunchKernelEx(&cfg, twm::mma::gemv_kernel<2, 2>, p); break;
            case 4: e = cudaLaunchKernelEx(&cfg, twm::mma::gemv_kernel<4, 2>, p); break;
            default: e = cudaLaunchKernelEx(&cfg, twm::mma::gemv_kernel<8, 2>, p); break;
        }
    } else {
        switch (mp) {
            case 1: e = cudaLaunchKernelEx(&cfg, twm::mma::gemv_kernel<1, 0>, p); break;
            case 2: e = cudaLaunchKernelEx(&cfg, twm::mma::gemv_kernel<2, 0>, p); break;
            case 4: e = cudaLaunchKernelEx(&cfg, twm::mma::gemv_kernel<4, 0>, p); break;
            default: e = cudaLaunchKernelEx(&cfg, twm::mma::gemv_kernel<8, 0>, p); break;
        }
    }
    if (e != cudaSuccess) { set_error("launch mma::gemv_kernel", e); return TWM_ELAUNCH; }
    return TWM_OK;
}

twm_status launch_simt(const twm::GemmParams& p, int mmax, dim3 grid, bool pdl, cudaStream_t stream)
{
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid;
    cfg.blockDim = dim3(twm::simt::THREADS, 1, 1);
    cfg.dynamicSmemBytes = sizeof(twm::simt::Smem);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    cudaError_t e;
    switch (mmax) {
        case 1: e = cudaLaunchKernelEx(&cfg, twm::simt::gemv_kernel<1>, p); break;
        case 2: e = cudaLaunchKernelEx(&cfg, twm::simt::gemv_kernel<2>, p); break;
        case 4: e = cudaLaunchKernelEx(&cfg, twm::simt::gemv_kernel<4>, p); break;
        default: e = cudaLaunchKernelEx(&cfg, twm::simt::gemv_kernel<8>, p); break;
    }
    if (e != cudaSuccess) { set_error("launch gemv_kernel", e); return TWM_ELAUNCH; }
    return TWM_OK;
}

// Scratch for twm_gemm_w4a16_static_ws: split-K tile counters (first 16 KB) and FP32
// partial sums.  It lives in the library's own device image, so every GPU that loads
// the library carries these 8 MiB until the process exits.
constexpr size_t kStaticWsBytes = 8u << 20;
static __device__ __align__(256) unsigned char g_static_ws[kStaticWsBytes];

// Device address of g_static_ws per device.  In host code the array's name is only a
// handle for the runtime, not a pointer a kernel could use; the real address comes from
// cudaGetSymbolAddress, asked once per device while that device is current.
void* g_static_ws_ptr[kMaxDevices] = {nullptr};
std::mutex g_static_ws_mutex;

twm_status static_ws_address(void** out)
{
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) { set_error("cudaGetDevice", e); return TWM_ELAUNCH; }
    if (dev < 0 || dev >= kMaxDevices) return TWM_EINVAL;
    std::lock_guard<std::mutex> lock(g_static_ws_mutex);
    if (g_static_ws_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_ws);
        if (e != cudaSuccess || ptr == nullptr) {
            set_error("cudaGetSymbolAddress(g_static_ws)", e);
            return TWM_ELAUNCH;
        }
        g_static_ws_ptr[dev] = ptr;
    }
    *out = g_static_ws_ptr[dev];
    return TWM_OK;
}

}  // namespace

namespace {
constexpr int kArgmaxParts = 592;   // 4 CTAs per SM

template <typename... KArgs, typename... Args>
twm_status launch_op(const char* name, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, int flags,
                     void* stream_, Args... args)
{
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = (cudaStream_t)stream_;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & TWM_FLAG_PDL) ? 1 : 0;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
    if (e != cudaSuccess) { set_error(name, e); return TWM_ELAUNCH; }
    return TWM_OK;
}

// twm_gemm_args.next: which bytes the GEMM after this one starts with, under its own plan.
twm::NextHead next_head_for(const twm_gemm_args* nx, int sm_count)
{
    twm::NextHead h;
    memset(&h, 0, sizeof(h));
    if (!nx || !nx->packed || !nx->scales || nx->packed_offsets) return h;
    if (!shape_ok(nx->M, nx->N, nx->K, nx->group_size) || (reinterpret_cast<uintptr_t>(nx->packed) & 15)) return h;
    const int kernel = resolve_kernel(nx);
    twm_plan_t pl;
    if (twm_plan(nx->M, nx->N, nx->K, nx->group_size, sm_count, nx->splits_override, kernel, &pl) != TWM_OK) return h;
    if (pl.workspace_bytes > 0 && (!nx->workspace || nx->workspace_bytes < pl.workspace_bytes) && kernel != TWM_KERNEL_TC &&
        kernel != TWM_KERNEL_TCW && nx->splits_override == 0 &&
        twm_plan(nx->M, nx->N, nx->K, nx->group_size, sm_count, 1, kernel, &pl) != TWM_OK)
        return h;
    const long row_bytes = (long)nx->N * twm::kBlockBytes;           // one 32-block of K over all columns
    const int gblocks = nx->group_size / 32;
    const int nkb = nx->K / 32;
    const int last = nkb - (pl.splits - 1) * pl.blocks_per_split;    // blocks of the last (shortest) K slice
    long hb = (16L << 20) / ((long)pl.splits * row_bytes);
    hb = std::min<long>(hb, std::min(pl.blocks_per_split, last));
    hb = hb / gblocks * gblocks;
    if (hb < gblocks) hb = std::min(gblocks, std::min(pl.blocks_per_split, last));
    if (hb < 1) return h;
    h.packed = nx->packed;
    h.regions = (unsigned)pl.splits;
    h.packed_stride = (unsigned long long)pl.blocks_per_split * row_bytes;
    h.packed_bytes = (unsigned)(hb * row_bytes);
    if ((nx->N & 7) == 0 && (reinterpret_cast<uintptr_t>(nx->scales) & 15) == 0 && pl.blocks_per_split % gblocks == 0) {
        h.scales = nx->scales;
        h.scales_stride = (unsigned long long)(pl.blocks_per_split / gblocks) * nx->N * 2;
        h.scales_bytes = (unsigned)(((hb + gblocks - 1) / gblocks) * nx->N * 2);
    }
    return h;
}

// The pre-pass of the tcgen05 kernels: the launch's rows in [K/8][rows][8] order.
twm_status launch_prepass(__half* xp, const __half* a, long lda, int rows, int K, unsigned flags, void* stream)
{
    const int items = rows * (K / 8);
    return launch_op("permute_activations_kernel", twm::tc::permute_activations_kernel, dim3((items + 255) / 256), dim3(256), 0,
                     flags & TWM_FLAG_PDL, stream, xp, a, lda, rows, K / 8);
}

// 9..32 rows on the streaming MMA kernel: the pre-pass that stages the rows as B fragments, then the GEMM
twm_status launch_mma_rows(twm::GemmParams& p, char* stage_buf, dim3 grid, unsigned flags, cudaStream_t stream)
{
    const int mp = mma_rows_for(p.M);
    p.rows_b = (const uint8_t*)stage_buf;
    p.rows_asum = (const float*)(stage_buf + mma_rows_b_bytes(p.M, p.K));
    const int items = p.nkb * mp * 4;
    twm_status st;
    auto stage = [&](auto kern) {
        return launch_op("stage_rows_kernel", kern, dim3((items + 255) / 256), dim3(256), 0, flags & TWM_FLAG_PDL, stream,
                         (uint8_t*)stage_buf, (float*)p.rows_asum, (const __half*)p.a, p.lda, p.M, mp, p.K, p.nkb);
    };
    // (a gated-activation prologue is applied here, once, while the rows are staged)
    if (p.group == 128)
        st = p.a_kind == 0 ? stage(twm::mma::stage_rows_kernel<2, 0>) : (p.a_kind == 1 ? stage(twm::mma::stage_rows_kernel<2, 1>) : stage(twm::mma::stage_rows_kernel<2, 2>));
    else
        st = p.a_kind == 0 ? stage(twm::mma::stage_rows_kernel<0, 0>) : (p.a_kind == 1 ? stage(twm::mma::stage_rows_kernel<0, 1>) : stage(twm::mma::stage_rows_kernel<0, 2>));
    if (st != TWM_OK) return st;
    auto go = [&](auto k128, auto k32, size_t smem) {
        return p.group == 128 ? launch_op("mma::gemm_rows_kernel", k128, grid, dim3(twm::mma::THREADS), smem, flags & TWM_FLAG_PDL, stream, p)
                              : launch_op("mma::gemm_rows_kernel", k32, grid, dim3(twm::mma::THREADS), smem, flags & TWM_FLAG_PDL, stream, p);
    };
    if (mp == 8) return go(twm::mma::gemm_rows_kernel<8, 2>, twm::mma::gemm_rows_kernel<8, 0>, sizeof(twm::mma::RowsSmem<8>));
    if (mp == 16) return go(twm::mma::gemm_rows_kernel<16, 2>, twm::mma::gemm_rows_kernel<16, 0>, sizeof(twm::mma::RowsSmem<16>));
    if (mp == 24) return go(twm::mma::gemm_rows_kernel<24, 2>, twm::mma::gemm_rows_kernel<24, 0>, sizeof(twm::mma::RowsSmem<24>));
    return go(twm::mma::gemm_rows_kernel<32, 2>, twm::mma::gemm_rows_kernel<32, 0>, sizeof(twm::mma::RowsSmem<32>));
}

// twm_plan; prepass (streaming MMA kernel's staging pre-pass) 0: not used (up to eight rows), 1: by the size rule,
// 2: from two rows on whatever the size
twm_status plan_impl(int M, int N, int K, int group_size, int sm_count, int splits_override,
                     int kernel_override, int prepass, twm_plan_t* out)
{
    if (!out || !shape_ok(M, N, K, group_size)) return TWM_EINVAL;
    if (splits_override < 0 || splits_override > kMaxSplits) return TWM_EINVAL;
    if (sm_count <= 0) sm_count = kDefaultSms;
    const int nkb = K / 32;
    int kernel = kernel_override;
    if (kernel == TWM_KERNEL_AUTO) kernel = auto_kernel(M, N, K, group_size, true, false, splits_override);
    if (kernel != TWM_KERNEL_SIMT && kernel != TWM_KERNEL_TC && kernel != TWM_KERNEL_MMA && kernel != TWM_KERNEL_TCW &&
        kernel != TWM_KERNEL_TCR)
        return TWM_EINVAL;
    if ((kernel == TWM_KERNEL_TCW || kernel == TWM_KERNEL_TCR) && (group_size != 128 || N < 128)) return TWM_EINVAL;
    if (kernel == TWM_KERNEL_TCR) {          // 256-column tiles over the whole K: no slices, no scratch but the reordered activations
        if (splits_override > 1) return TWM_EINVAL;
        const int rows_r = std::min(M, kTcrRows);
        out->kernel = kernel;
        out->n_tile = twm::tcr::NT;
        out->splits = 1;
        out->blocks_per_split = K / 32;
        out->grid_x = (N + twm::tcr::NT - 1) / twm::tcr::NT;
        out->grid_y = 1;
        out->workspace_bytes = kCounterBytes + 256 + (size_t)rows_r * K * 2;
        out->cluster_reduce = 0;
        return TWM_OK;
    }
    // rows one launch carries; more rows are served by further launches
    const int rows = std::min(M, kernel == TWM_KERNEL_TC ? kTcRows : (kernel == TWM_KERNEL_TCW ? kTcwRows : (kernel == TWM_KERNEL_MMA ? mma_rows_for(M) : 8)));
    const int n_tiles = (N + twm::simt::NT - 1) / twm::simt::NT;
    const int slots = kernel == TWM_KERNEL_TCW ? sm_count
                                               : sm_count * ((kernel != TWM_KERNEL_SIMT || mmax_for(rows) <= 4) ? 2 : 1);
    const int max_bps = nkb;
    const int align = (kernel == TWM_KERNEL_MMA || kernel == TWM_KERNEL_TC || kernel == TWM_KERNEL_TCW) ? group_size / 32 : 1;   // whole scale groups per slice
    // up to two rows on the streaming MMA kernel: K slices add up inside a cluster (at most 16 slices)
    const bool can_cluster = (kernel == TWM_KERNEL_MMA) && rows <= twm::mma::CLUSTER_ROWS;
    int splits, bps;
    if (splits_override > 0) {
        bps = (nkb + splits_override - 1) / splits_override;
        bps = (bps + align - 1) / align * align;
        if (bps > max_bps) return TWM_EINVAL;
        splits = (nkb + bps - 1) / bps;
    } else if (kernel == TWM_KERNEL_TCW) {
        // Measured (128 rows): a 128-K stage costs about 0.8 us, a K slice about 7 us of its own (partials out, count,
        // the last arriver's sum).  Slices pay only with few tiles and a long K: N=3584, K=18944: 124 us unsplit,
        // 64 us in five slices; N=3584, K=3584: 29 us unsplit, 36 us in two.
        const int stages = nkb / align;
        int want = 1;
        if (stages >= 64 && 2 * n_tiles <= slots) want = std::min(std::min(slots / n_tiles, stages / 28), kMaxSplits);
        bps = (stages + want - 1) / want * align;
        splits = (nkb + bps - 1) / bps;
    } else {
        choose_splits(n_tiles, nkb, slots, sm_count, max_bps, align, can_cluster ? twm::mma::MAX_CLUSTER / rows : kMaxSplits,
                      can_cluster, &splits, &bps);
        if (bps > max_bps) return TWM_EINVAL;
    }
    const bool cluster = can_cluster && splits > 1 && splits * rows <= twm::mma::MAX_CLUSTER;
    out->kernel = kernel;
    out->n_tile = twm::simt::NT;
    out->splits = splits;
    out->blocks_per_split = bps;
    out->grid_x = n_tiles;
    out->grid_y = splits;
    out->workspace_bytes = (splits > 1 && !cluster) ? kCounterBytes + (size_t)splits * rows * N * sizeof(float) : 0;
    if (kernel == TWM_KERNEL_TC || kernel == TWM_KERNEL_TCW)    // + the launch's activations in the MMA's K order, behind the split-K part
        out->workspace_bytes = kCounterBytes + (splits > 1 ? (size_t)splits * rows * N * sizeof(float) : 0) + 256 + (size_t)rows * K * 2;
    if (kernel == TWM_KERNEL_MMA && (mma_prepass(rows, K, N) || (prepass == 2 && rows >= 2))) {      // + the rows staged as B fragments with their group sums
        if (prepass)
            out->workspace_bytes = kCounterBytes + (splits > 1 ? (size_t)splits * rows * N * sizeof(float) : 0) + 256 + mma_rows_stage_bytes(rows, K, group_size);
        else if (rows > 8)
            return TWM_EINVAL;
    }
    out->cluster_reduce = cluster ? 1 : 0;
    return TWM_OK;
}
}  // namespace

extern "C" {

twm_status twm_plan(int M, int N, int K, int group_size, int sm_count, int splits_override,
                    int kernel_override, twm_plan_t* out)
{
    return plan_impl(M, N, K, group_size, sm_count, splits_override, kernel_override, 1, out);
}

size_t twm_workspace_bytes(int M, int N, int K, int group_size)
{
    // the larger of the two kernels' needs: which one runs depends on the activation dtype
    twm_plan_t tc, simt;
    size_t need = 0;
    if (twm_plan(M, N, K, group_size, kDefaultSms, 0, TWM_KERNEL_TC, &tc) == TWM_OK) need = tc.workspace_bytes;
    if (twm_plan(M, N, K, group_size, kDefaultSms, 0, TWM_KERNEL_TCW, &tc) == TWM_OK) need = std::max(need, tc.workspace_bytes);
    if (twm_plan(M, N, K, group_size, kDefaultSms, 0, TWM_KERNEL_TCR, &tc) == TWM_OK) need = std::max(need, tc.workspace_bytes);
    if (twm_plan(M, N, K, group_size, kDefaultSms, 0, TWM_KERNEL_SIMT, &simt) == TWM_OK)
        need = std::max(need, simt.workspace_bytes);
    // (the streaming MMA kernel with its staging pre-pass whatever the size: a push to peers asks for it)
    if (plan_impl(M, N, K, group_size, kDefaultSms, 0, TWM_KERNEL_MMA, 2, &simt) == TWM_OK)
        need = std::max(need, simt.workspace_bytes);
    return need;
}

twm_status twm_gemm_w4a16(const twm_gemm_args* a, void* stream_)
{
    if (!a) return TWM_EINVAL;
    if (!shape_ok(a->M, a->N, a->K, a->group_size)) return TWM_EINVAL;
    if (!a->a || !a->packed || !a->scales || !a->c) return TWM_EINVAL;
    if ((a->a_dtype != TWM_F32 && a->a_dtype != TWM_F16) || (a->c_dtype != TWM_F32 && a->c_dtype != TWM_F16))
        return TWM_EINVAL;
    if (a->lda < a->K || a->ldc < a->N) return TWM_EINVAL;
    if (a->a_prologue < TWM_A_PLAIN || a->a_prologue > TWM_A_GEGLU) return TWM_EINVAL;
    if (a->a_prologue != TWM_A_PLAIN && (a->M > 32 || a->a_dtype != TWM_F16 || a->lda < 2L * a->K)) return TWM_EINVAL;
    if ((a->packed_offsets == nullptr) != (a->scales_offsets == nullptr)) return TWM_EINVAL;
    if (a->packed_offsets && a->expert_idx < 0) return TWM_EINVAL;
    if (reinterpret_cast<uintptr_t>(a->packed) & 15) return TWM_EALIGN;
    if (reinterpret_cast<uintptr_t>(a->scales) & 1) return TWM_EALIGN;
    if (reinterpret_cast<uintptr_t>(a->a) & (a->a_dtype == TWM_F16 ? 1 : 3)) return TWM_EALIGN;
    if (reinterpret_cast<uintptr_t>(a->c) & (a->c_dtype == TWM_F16 ? 1 : 3)) return TWM_EALIGN;

    int sm_count = kDefaultSms;
    twm_status st = ensure_device(&sm_count);
    if (st != TWM_OK) return st;

    // The tensor-core kernel takes FP16 activations; FP32 activations (the
    // reference's own signature) run on the FP32 streaming kernel.
    const int kernel = resolve_kernel(a);
    if (kernel != TWM_KERNEL_SIMT && a->a_dtype != TWM_F16) return TWM_EINVAL;
    if (a->a_prologue != TWM_A_PLAIN && kernel != TWM_KERNEL_MMA) return TWM_EINVAL;
    // streaming MMA kernel: three rows or more on a large matrix, and nine or more on any, are staged by a pre-pass
    // (a push to tensor-parallel peers of three rows or more always is: the pre-pass form carries the push; and so is
    //  a gated-activation prologue on two rows or more: the pre-pass applies it)
    int prepass = 0;
    if (kernel == TWM_KERNEL_MMA) {
        if ((a->comm && a->M >= 3) || (a->a_prologue != TWM_A_PLAIN && a->M >= 2)) prepass = 2;
        else if (mma_prepass(std::min(a->M, mma_rows_for(a->M)), a->K, a->N)) prepass = 1;
    }
    if (prepass && a->packed_offsets != nullptr) {
        if (a->M > 8 || prepass == 2) return TWM_EINVAL;
        prepass = 0;                             // the CTAs' own stager warps
    }
    twm_plan_t pl;
    st = plan_impl(a->M, a->N, a->K, a->group_size, sm_count, a->splits_override, kernel, prepass, &pl);
    if (st != TWM_OK) return st;
    if (prepass == 1 && a->M <= 8 && (!a->workspace || a->workspace_bytes < pl.workspace_bytes)) {
        prepass = 0;                             // no room for the staged rows: the stager warps need none
        st = plan_impl(a->M, a->N, a->K, a->group_size, sm_count, a->splits_override, kernel, 0, &pl);
        if (st != TWM_OK) return st;
    }
    if (pl.workspace_bytes > 0 && (!a->workspace || a->workspace_bytes < pl.workspace_bytes) &&
        kernel != TWM_KERNEL_TC && a->splits_override == 0) {
        // The reference's call has no scratch argument (its split-K adds into C with atomics,
        // quantize.rs:1337-1357).  A caller that passes none still gets its GEMM: one K slice per
        // tile, nothing to add up, at the price of fewer CTAs on small N.
        st = plan_impl(a->M, a->N, a->K, a->group_size, sm_count, 1, kernel, prepass, &pl);
        if (st != TWM_OK) return st;
    }
    if (pl.workspace_bytes > 0) {
        if (!a->workspace || a->workspace_bytes < pl.workspace_bytes) return TWM_EWORKSPACE;
        if (reinterpret_cast<uintptr_t>(a->workspace) & 15) return TWM_EALIGN;
    }

    if (a->comm) {
        // pushing the result to tensor-parallel peers: streaming MMA kernel, no workspace-based split
        const twm_comm* cm = a->comm;
        const bool mma_ok = kernel == TWM_KERNEL_MMA &&
                            ((a->M <= twm::mma::CLUSTER_ROWS && (pl.splits == 1 || pl.cluster_reduce)) || (prepass && a->M <= 32));
        const bool tc_ok = kernel == TWM_KERNEL_TC && a->M <= 64;           // one launch: one operation of the flag protocol
        if (!mma_ok && !tc_ok) return TWM_EINVAL;
        if (cm->n_ranks < 1 || cm->n_ranks > 8 || cm->rank < 0 || cm->rank >= cm->n_ranks || !cm->state) return TWM_EINVAL;
        if (cm->slot_elems < (long)a->M * a->ldc) return TWM_EINVAL;
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    const size_t a_elt = a->a_dtype == TWM_F16 ? 2 : 4;
    const size_t c_elt = a->c_dtype == TWM_F16 ? 2 : 4;
    if ((kernel == TWM_KERNEL_TCW || kernel == TWM_KERNEL_TCR) && (a->packed_offsets != nullptr || a->comm)) return TWM_EINVAL;
    const int row_step = kernel == TWM_KERNEL_TC ? kTcRows : (kernel == TWM_KERNEL_TCW ? kTcwRows : (kernel == TWM_KERNEL_TCR ? kTcrRows : (kernel == TWM_KERNEL_MMA ? mma_rows_for(a->M) : 8)));
    CUtensorMap packed_map;
    int map_rows = 0;
    if (a->packed_offsets == nullptr && a->N >= 128 && kernel != TWM_KERNEL_SIMT) {
        const int want = kernel == TWM_KERNEL_MMA ? twm::mma::SB : (kernel == TWM_KERNEL_TCR ? twm::tcr::SB : twm::tc::WSTAGE_BLOCKS);      // (the wide kernel's stage is four blocks too)
        if (make_packed_map(&packed_map, a->packed, a->N, a->K / 32, want)) map_rows = want;
    }
    for (int m0 = 0; m0 < a->M; m0 += row_step) {
        const int rows = std::min(row_step, a->M - m0);
        twm::GemmParams p;
        memset(&p, 0, sizeof(p));
        p.M = rows; p.N = a->N; p.K = a->K; p.group = a->group_size; p.nkb = a->K / 32;
        p.a_is_f16 = a->a_dtype == TWM_F16; p.c_is_f16 = a->c_dtype == TWM_F16;
        p.a = (const char*)a->a + (size_t)m0 * a->lda * a_elt; p.lda = a->lda;
        p.packed = a->packed; p.scales = a->scales;
        p.c = (char*)a->c + (size_t)m0 * a->ldc * c_elt; p.ldc = a->ldc;
        p.ws_counters = (unsigned int*)a->workspace;
        p.ws_partials = a->workspace ? (float*)((char*)a->workspace + kCounterBytes) : nullptr;
        p.splits = pl.splits; p.blocks_per_split = pl.blocks_per_split;
        p.reduce_slices = pl.splits;
        p.cluster_reduce = (pl.cluster_reduce && rows <= twm::mma::CLUSTER_ROWS) ? 1 : 0;
        p.accumulate = (a->flags & TWM_FLAG_ACCUMULATE) ? 1 : 0;
        p.no_wait = ((a->flags & TWM_FLAG_INDEPENDENT) && (a->flags & TWM_FLAG_PDL) && kernel == TWM_KERNEL_MMA &&
                     pl.workspace_bytes == 0 && !p.accumulate && a->packed_offsets == nullptr && !a->comm) ? 1 : 0;
        p.packed_offsets = a->packed_offsets; p.scales_offsets = a->scales_offsets; p.expert_idx = a->expert_idx;
        p.a_kind = a->a_prologue;
        if (kernel == TWM_KERNEL_MMA && m0 + row_step >= a->M) p.next = next_head_for(a->next, sm_count);
        if (a->comm) {
            p.n_peers = a->comm->n_ranks; p.peer_rank = a->comm->rank; p.peer_slot_elems = a->comm->slot_elems;
            for (int r = 0; r < a->comm->n_ranks; ++r) { p.peer_data[r] = a->comm->data[r]; p.peer_flags[r] = a->comm->flags[r]; }
            p.comm_state = a->comm->state;
        }
        p.map_rows = map_rows;
        if (map_rows) p.packed_map = packed_map;
        const bool pdl = (a->flags & TWM_FLAG_PDL) != 0;
        if (kernel == TWM_KERNEL_TCR) {
            if (!map_rows) {
                snprintf(t_last_error, sizeof(t_last_error), "cuTensorMapEncodeTiled failed for the packed map of the 256-column tcgen05 kernel");
                return TWM_ELAUNCH;
            }
            char* xp = (char*)a->workspace + kCounterBytes;
            if (!make_act_map_wide(&p.act_map, xp, rows, a->K, twm::tcr::KCORES)) {
                snprintf(t_last_error, sizeof(t_last_error), "cuTensorMapEncodeTiled failed for the activation map");
                return TWM_ELAUNCH;
            }
            st = launch_prepass((__half*)xp, (const __half*)p.a, p.lda, rows, a->K, a->flags, stream_);
            if (st != TWM_OK) return st;
            st = launch_tcr(p, rows, dim3(pl.grid_x, 1, 1), pdl, stream);
        }
        else if (kernel == TWM_KERNEL_TCW) {
            if (!map_rows) {
                snprintf(t_last_error, sizeof(t_last_error), "cuTensorMapEncodeTiled failed for the packed map of the wide tcgen05 kernel");
                return TWM_ELAUNCH;
            }
            const size_t part_bytes = pl.splits > 1 ? (size_t)pl.splits * std::min(a->M, kTcwRows) * a->N * sizeof(float) : 0;
            char* xp = (char*)a->workspace + kCounterBytes + ((part_bytes + 255) / 256) * 256;
            if (!make_act_map_wide(&p.act_map, xp, rows, a->K)) {
                snprintf(t_last_error, sizeof(t_last_error), "cuTensorMapEncodeTiled failed for the activation map");
                return TWM_ELAUNCH;
            }
            st = launch_prepass((__half*)xp, (const __half*)p.a, p.lda, rows, a->K, a->flags, stream_);
            if (st != TWM_OK) return st;
            st = launch_tcw(p, dim3(pl.grid_x, pl.grid_y, 1), pdl, stream);
        }
        else if (kernel == TWM_KERNEL_TC) {
            // pre-pass: this launch's rows in [K/8][rows][8] order, then the GEMM loads them by TMA
            const size_t part_bytes = pl.splits > 1 ? (size_t)pl.splits * std::min(a->M, kTcRows) * a->N * sizeof(float) : 0;
            char* xp = (char*)a->workspace + kCounterBytes + ((part_bytes + 255) / 256) * 256;
            const int nb_rows = rows <= 16 ? 16 : (rows <= 32 ? 32 : 64);
            if (!make_act_map(&p.act_map, xp, rows, a->K, nb_rows)) {
                snprintf(t_last_error, sizeof(t_last_error), "cuTensorMapEncodeTiled failed for the activation map");
                return TWM_ELAUNCH;
            }
            st = launch_prepass((__half*)xp, (const __half*)p.a, p.lda, rows, a->K, a->flags, stream_);
            if (st != TWM_OK) return st;
            st = launch_tc(p, rows, dim3(pl.grid_x, pl.grid_y, 1), pdl, stream);
        }
        else if (kernel == TWM_KERNEL_MMA && prepass && rows >= (prepass == 2 ? 2 : 3)) {
            const size_t part_bytes = pl.splits > 1 ? (size_t)pl.splits * std::min(a->M, row_step) * a->N * sizeof(float) : 0;
            char* stage = (char*)a->workspace + kCounterBytes + ((part_bytes + 255) / 256) * 256;
            st = launch_mma_rows(p, stage, dim3(pl.grid_x, pl.grid_y, 1), a->flags, stream);
        }
        else if (kernel == TWM_KERNEL_MMA)
            st = launch_mma(p, mmax_for(rows), dim3(pl.grid_x, pl.grid_y, 1), pdl, stream);
        else
            st = launch_simt(p, mmax_for(rows), dim3(pl.grid_x, pl.grid_y, 1), pdl, stream);
        if (st != TWM_OK) return st;
    }
    return TWM_OK;
}

twm_status twm_gemm_w4a16_static_ws(const twm_gemm_args* a, void* stream_)
{
    // everything twm_gemm_w4a16 checks before it enqueues, checked here first: a call that is going
    // to be refused must not have put the counter clearing on the stream already
    if (!a) return TWM_EINVAL;
    if (!shape_ok(a->M, a->N, a->K, a->group_size)) return TWM_EINVAL;
    if (!a->a || !a->packed || !a->scales || !a->c) return TWM_EINVAL;
    if ((a->a_dtype != TWM_F32 && a->a_dtype != TWM_F16) || (a->c_dtype != TWM_F32 && a->c_dtype != TWM_F16))
        return TWM_EINVAL;
    if (a->lda < a->K || a->ldc < a->N) return TWM_EINVAL;
    if ((a->packed_offsets == nullptr) != (a->scales_offsets == nullptr)) return TWM_EINVAL;
    if (a->packed_offsets && a->expert_idx < 0) return TWM_EINVAL;
    if (reinterpret_cast<uintptr_t>(a->packed) & 15) return TWM_EALIGN;
    if (reinterpret_cast<uintptr_t>(a->scales) & 1) return TWM_EALIGN;
    if (reinterpret_cast<uintptr_t>(a->a) & (a->a_dtype == TWM_F16 ? 1 : 3)) return TWM_EALIGN;
    if (reinterpret_cast<uintptr_t>(a->c) & (a->c_dtype == TWM_F16 ? 1 : 3)) return TWM_EALIGN;
    int sm_count = kDefaultSms;
    twm_status st = ensure_device(&sm_count);
    if (st != TWM_OK) return st;
    void* ws = nullptr;
    st = static_ws_address(&ws);
    if (st != TWM_OK) return st;
    // The call that will run: the caller's arguments with the built-in array as its workspace.  The
    // kernel choice and the plan are made for THAT call (a workspace of this size decides
    // whether three to eight rows are staged by a pre-pass), so the capacity check and the clearing below match what runs.
    twm_gemm_args b = *a;
    b.workspace = ws;
    b.workspace_bytes = kStaticWsBytes;
    const int kernel = resolve_kernel(&b);
    if (kernel != TWM_KERNEL_SIMT && a->a_dtype != TWM_F16) return TWM_EINVAL;
    twm_plan_t pl;
    st = twm_plan(a->M, a->N, a->K, a->group_size, sm_count, a->splits_override, kernel, &pl);
    if (st != TWM_OK) return st;
    if (pl.workspace_bytes > kStaticWsBytes && kernel == TWM_KERNEL_MMA && a->M <= 8) {
        // as twm_gemm_w4a16 will: up to eight rows can do without the staging pre-pass
        st = plan_impl(a->M, a->N, a->K, a->group_size, sm_count, a->splits_override, kernel, 0, &pl);
        if (st != TWM_OK) return st;
    }
    if (pl.workspace_bytes > kStaticWsBytes) {
        snprintf(t_last_error, sizeof(t_last_error),
                 "twm_gemm_w4a16_static_ws: this shape needs %zu bytes of split-K scratch, the built-in array holds %zu; "
                 "use twm_gemm_w4a16 with a caller-owned workspace", pl.workspace_bytes, kStaticWsBytes);
        return TWM_EWORKSPACE;
    }
    if (pl.workspace_bytes > 0) {
        // The array keeps whatever the last call left.  Partial sums are always written before
        // they are read; the tile counters must start at zero, so they are cleared here.
        cudaError_t e = cudaMemsetAsync(ws, 0, (size_t)pl.grid_x * sizeof(unsigned int), (cudaStream_t)stream_);
        if (e != cudaSuccess) { set_error("cudaMemsetAsync(static scratch counters)", e); return TWM_ELAUNCH; }
    }
    return twm_gemm_w4a16(&b, stream_);
}

size_t twm_static_ws_capacity(void) { return kStaticWsBytes; }

// ------------------------------------------------------- batched expert GEMVs (MoE) --
namespace {
struct MoePlan { int splits, bps, cluster; size_t workspace_bytes; };

// K slices so that n_tiles x top_k x splits CTAs come close to the resident slots; a sum over the
// slots runs inside a cluster when K slices x slots fit one, else through the workspace.
MoePlan moe_plan(int top_k, int N, int K, int group_size, int sm_count, bool weighted)
{
    const int nkb = K / 32, align = group_size / 32;
    const int n_tiles = (N + twm::mma::NT - 1) / twm::mma::NT;
    const int slots = 2 * sm_count;
    const int max_by_k = std::max(1, nkb / std::max(align, 4));          // at least four 32-blocks per slice
    int splits = std::max(1, slots / std::max(1, n_tiles * top_k));
    splits = std::min(splits, max_by_k);
    if (!weighted) splits = std::min(splits, twm::mma::MAX_CLUSTER);
    else if (splits * top_k > twm::mma::MAX_CLUSTER && top_k <= twm::mma::MAX_CLUSTER)
        splits = std::max(1, std::min(splits, twm::mma::MAX_CLUSTER / top_k)) ;    // prefer the cluster: no workspace traffic
    splits = std::min(splits, kMaxSplits);
    int bps = (nkb + splits - 1) / splits;
    bps = (bps + align - 1) / align * align;
    splits = (nkb + bps - 1) / bps;
    MoePlan pl;
    pl.splits = splits; pl.bps = bps;
    const int slices = weighted ? splits * top_k : splits;
    pl.cluster = (slices > 1 && slices <= twm::mma::MAX_CLUSTER) ? 1 : 0;
    pl.workspace_bytes = (slices > 1 && !pl.cluster) ? kCounterBytes + (size_t)slices * N * sizeof(float) : 0;
    return pl;
}

twm_status moe_launch(const twm_moe_args* a, bool weighted, void* stream_)
{
    if (!a) return TWM_EINVAL;
    if (!shape_ok(1, a->N, a->K, a->group_size) || a->top_k < 1 || a->top_k > 64) return TWM_EINVAL;
    if (!a->a || !a->packed_base || !a->scales_base || !a->topk_ids || !a->c) return TWM_EINVAL;
    if (weighted != (a->topk_weights != nullptr)) return TWM_EINVAL;
    if (a->c_dtype != TWM_F32 && a->c_dtype != TWM_F16) return TWM_EINVAL;
    if (a->a_prologue < TWM_A_PLAIN || a->a_prologue > TWM_A_GEGLU) return TWM_EINVAL;
    if (a->a_slot_stride < 0 || (!weighted && a->c_slot_stride < a->N)) return TWM_EINVAL;
    if ((reinterpret_cast<uintptr_t>(a->packed_base) & 15) || (a->packed_bytes_per_expert & 15)) return TWM_EALIGN;
    if ((reinterpret_cast<uintptr_t>(a->scales_base) & 1) || (reinterpret_cast<uintptr_t>(a->a) & 1)) return TWM_EALIGN;
    if (reinterpret_cast<uintptr_t>(a->c) & (a->c_dtype == TWM_F16 ? 1 : 3)) return TWM_EALIGN;
    int sm_count = kDefaultSms;
    twm_status st = ensure_device(&sm_count);
    if (st != TWM_OK) return st;
    const MoePlan pl = moe_plan(a->top_k, a->N, a->K, a->group_size, sm_count, weighted);
    if (pl.workspace_bytes > 0) {
        if (!a->workspace || a->workspace_bytes < pl.workspace_bytes) return TWM_EWORKSPACE;
        if (reinterpret_cast<uintptr_t>(a->workspace) & 15) return TWM_EALIGN;
    }
    twm::GemmParams p;
    memset(&p, 0, sizeof(p));
    p.M = 1; p.N = a->N; p.K = a->K; p.group = a->group_size; p.nkb = a->K / 32;
    p.a_is_f16 = 1; p.c_is_f16 = a->c_dtype == TWM_F16;
    p.a = a->a; p.lda = a->a_prologue == TWM_A_PLAIN ? a->K : 2L * a->K;
    p.packed = a->packed_base; p.scales = a->scales_base;
    p.c = a->c; p.ldc = a->N;
    p.ws_counters = (unsigned int*)a->workspace;
    p.ws_partials = a->workspace ? (float*)((char*)a->workspace + kCounterBytes) : nullptr;
    p.splits = pl.splits; p.blocks_per_split = pl.bps;
    p.reduce_slices = weighted ? pl.splits * a->top_k : pl.splits;
    p.cluster_reduce = pl.cluster;
    p.accumulate = (a->flags & TWM_FLAG_ACCUMULATE) ? 1 : 0;
    p.n_experts = a->top_k;
    p.a_kind = a->a_prologue;
    p.expert_ids = a->topk_ids;
    p.expert_weights = weighted ? a->topk_weights : nullptr;
    p.packed_expert_stride = a->packed_bytes_per_expert;
    p.scales_expert_stride = a->scales_per_expert;
    p.a_expert_stride = a->a_slot_stride;
    p.c_expert_stride = a->c_slot_stride;
    p.map_rows = 0;                 // the expert is chosen on the device: rows are copied one by one, no tensor map
    const int n_tiles = (a->N + twm::mma::NT - 1) / twm::mma::NT;
    return launch_mma(p, 1, dim3(n_tiles, pl.splits, a->top_k), (a->flags & TWM_FLAG_PDL) != 0, (cudaStream_t)stream_);
}
}  // namespace

size_t twm_moe_workspace_bytes(int top_k, int N, int K, int group_size)
{
    if (!shape_ok(1, N, K, group_size) || top_k < 1 || top_k > 64) return 0;
    return std::max(moe_plan(top_k, N, K, group_size, kDefaultSms, true).workspace_bytes,
                    moe_plan(top_k, N, K, group_size, kDefaultSms, false).workspace_bytes);
}

twm_status twm_moe_gate_up(const twm_moe_args* args, void* stream) { return moe_launch(args, false, stream); }

twm_status twm_moe_down_axpy(const twm_moe_args* args, void* stream) { return moe_launch(args, true, stream); }

// ------------------------------------------------------------------ GEMM chains --
struct twm_chain {
    int device = 0;
    int count = 0;
    int grid = 0;
    int rows = 1;                 // MP of the kernel
    void* mem = nullptr;          // one allocation: state, counters, partials, GEMM table
    size_t bytes = 0;
    twm::chain::State* state = nullptr;
    unsigned int* done = nullptr;
    twm::chain::Op* ops = nullptr;
    int split_tiles = 0;
    int max_pieces = 1;
};

namespace {
size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

const void* chain_kernel_for(int rows)
{
    switch (rows) {
        case 1: return (const void*)twm::chain::chain_kernel<1>;
        case 2: return (const void*)twm::chain::chain_kernel<2>;
        case 4: return (const void*)twm::chain::chain_kernel<4>;
        default: return (const void*)twm::chain::chain_kernel<8>;
    }
}
}  // namespace

twm_status twm_chain_partition(int n_tiles, int nkb, int grid, int rank, int max_out, int* out5, int* n_out)
{
    if (n_tiles < 1 || nkb < 1 || grid < 1 || rank < 0 || rank >= grid || max_out < 0 || !n_out || (max_out > 0 && !out5))
        return TWM_EINVAL;
    const int upt = (nkb + twm::chain::UNIT - 1) / twm::chain::UNIT;
    const long long total = (long long)n_tiles * upt;
    if (total > 0x7fffffffLL) return TWM_EINVAL;
    const int ranks = (int)std::min<long long>(grid, total);
    twm::chain::Walker w;
    w.start(rank, (int)total, ranks, upt, nkb);
    twm::chain::Piece pc;
    int n = 0;
    while (w.next(pc)) {
        if (n < max_out) {
            int* o = out5 + 5 * n;
            o[0] = pc.tile; o[1] = pc.blk0; o[2] = pc.blk1; o[3] = pc.slot; o[4] = pc.n_pieces;
        }
        ++n;
    }
    *n_out = n;
    return TWM_OK;
}

twm_status twm_chain_create(const twm_chain_op* ops, int count, twm_chain** out)
{
    if (!ops || !out || count < 1 || count > 4096) return TWM_EINVAL;
    *out = nullptr;
    int sm_count = kDefaultSms;
    twm_status st = ensure_device(&sm_count);
    if (st != TWM_OK) return st;
    int max_m = 1;
    for (int i = 0; i < count; ++i) {
        const twm_gemm_args& a = ops[i].gemm;
        if (!shape_ok(a.M, a.N, a.K, a.group_size) || a.M > 8) return TWM_EINVAL;
        if (!a.a || !a.packed || !a.scales || !a.c) return TWM_EINVAL;
        if (a.a_dtype != TWM_F16 || (a.c_dtype != TWM_F32 && a.c_dtype != TWM_F16)) return TWM_EINVAL;
        if (a.a_prologue != TWM_A_PLAIN && a.a_prologue != TWM_A_SILU_MUL) return TWM_EINVAL;
        if (a.lda < (a.a_prologue == TWM_A_SILU_MUL ? 2L * a.K : (long)a.K) || a.ldc < a.N) return TWM_EINVAL;
        if (a.packed_offsets || a.scales_offsets || a.comm || a.splits_override || a.kernel_override) return TWM_EINVAL;
        if (reinterpret_cast<uintptr_t>(a.packed) & 15) return TWM_EALIGN;
        if ((reinterpret_cast<uintptr_t>(a.scales) & 1) || (reinterpret_cast<uintptr_t>(a.a) & 1)) return TWM_EALIGN;
        if (reinterpret_cast<uintptr_t>(a.c) & (a.c_dtype == TWM_F16 ? 1 : 3)) return TWM_EALIGN;
        max_m = std::max(max_m, a.M);
    }
    twm_chain* ch = new (std::nothrow) twm_chain();
    if (!ch) return TWM_ELAUNCH;
    cudaGetDevice(&ch->device);
    ch->count = count;
    ch->rows = mmax_for(max_m);
    int per_sm = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, chain_kernel_for(ch->rows), twm::chain::THREADS,
                                                                  sizeof(twm::chain::Smem));
    if (e != cudaSuccess || per_sm < 1) {
        if (e != cudaSuccess) set_error("cudaOccupancyMaxActiveBlocksPerMultiprocessor(chain_kernel)", e);
        else snprintf(t_last_error, sizeof(t_last_error), "chain_kernel does not fit on an SM");
        delete ch;
        return TWM_ELAUNCH;
    }
    ch->grid = sm_count * std::min(per_sm, twm::chain::CTAS_PER_SM);

    // the deal of every GEMM: pieces per tile decide the partial scratch
    std::vector<twm::chain::Op> table(count);
    std::vector<size_t> part_off(count), cnt_off(count);
    size_t part_bytes = 0, n_counters = 0;
    int dependent_from = 0;          // first GEMM a dependent GEMM must wait for
    for (int i = 0; i < count; ++i) {
        const twm_gemm_args& a = ops[i].gemm;
        twm::chain::Op& op = table[i];
        memset(&op, 0, sizeof(op));
        op.packed = a.packed; op.scales = a.scales; op.a = a.a; op.c = a.c;
        op.lda = a.lda; op.ldc = a.ldc;
        op.M = a.M; op.N = a.N; op.K = a.K; op.nkb = a.K / 32;
        op.gshift = a.group_size == 128 ? 2 : 0;
        op.n_tiles = (a.N + twm::chain::NT - 1) / twm::chain::NT;
        op.units_per_tile = (op.nkb + twm::chain::UNIT - 1) / twm::chain::UNIT;
        const long long total = (long long)op.n_tiles * op.units_per_tile;
        if (total > 0x7fffffffLL) { delete ch; return TWM_EINVAL; }
        op.total_units = (int)total;
        op.ranks = (int)std::min<long long>(ch->grid, total);
        op.rot = (int)(((long long)i * 97) % ch->grid);
        op.a_kind = a.a_prologue == TWM_A_SILU_MUL ? twm::chain::A_SILU_MUL : twm::chain::A_F16;
        op.c_is_f16 = a.c_dtype == TWM_F16;
        op.accumulate = (a.flags & TWM_FLAG_ACCUMULATE) ? 1 : 0;
        if (a.flags & TWM_FLAG_INDEPENDENT) {
            op.wait_from = i;                       // waits for nothing
        } else {
            op.wait_from = dependent_from;          // everything since (and including) the last dependent GEMM
            dependent_from = i;
        }
        op.use_maps = 0;
        if (a.N >= 128 && make_packed_map(&op.map8, a.packed, a.N, op.nkb, twm::chain::SB) &&
            make_packed_map(&op.map4, a.packed, a.N, op.nkb, twm::chain::UNIT))
            op.use_maps = 1;
        int max_pieces = 1;
        for (int t = 0; t < op.n_tiles; ++t) {
            const int first = twm::chain::rank_of_unit((long long)t * op.units_per_tile, op.total_units, op.ranks);
            const int last = twm::chain::rank_of_unit((long long)(t + 1) * op.units_per_tile - 1, op.total_units, op.ranks);
            const int pieces = last - first + 1;
            max_pieces = std::max(max_pieces, pieces);
            if (pieces > 1) ++ch->split_tiles;
        }
        op.max_pieces = max_pieces;
        ch->max_pieces = std::max(ch->max_pieces, max_pieces);
        part_off[i] = part_bytes;
        if (max_pieces > 1) part_bytes += round_up((size_t)op.n_tiles * max_pieces * a.M * twm::chain::NT * sizeof(float), 256);
        cnt_off[i] = n_counters;
        n_counters += op.n_tiles;
    }
    const size_t off_done = sizeof(twm::chain::State);
    const size_t off_cnt = off_done + round_up((size_t)count * 4, 256);
    const size_t off_part = off_cnt + round_up(n_counters * 4, 256);
    const size_t off_ops = off_part + part_bytes;
    ch->bytes = off_ops + (size_t)count * sizeof(twm::chain::Op);
    e = cudaMalloc(&ch->mem, ch->bytes);
    if (e == cudaSuccess) e = cudaMemset(ch->mem, 0, off_part);      // state and counters start at zero
    if (e != cudaSuccess) {
        set_error("twm_chain_create (allocation)", e);
        if (ch->mem) cudaFree(ch->mem);
        delete ch;
        return TWM_ELAUNCH;
    }
    char* base = (char*)ch->mem;
    ch->state = (twm::chain::State*)base;
    ch->done = (unsigned int*)(base + off_done);
    ch->ops = (twm::chain::Op*)(base + off_ops);
    for (int i = 0; i < count; ++i) {
        table[i].partials = (float*)(base + off_part + part_off[i]);
        table[i].tile_counters = (unsigned int*)(base + off_cnt) + cnt_off[i];
    }
    twm::chain::State hs;
    memset(&hs, 0, sizeof(hs));
    hs.n_tile_counters = (unsigned int)n_counters;
    hs.all_tile_counters = (unsigned int*)(base + off_cnt);
    e = cudaMemcpy(ch->state, &hs, sizeof(hs), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(ch->ops, table.data(), (size_t)count * sizeof(twm::chain::Op), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        set_error("twm_chain_create (copy)", e);
        cudaFree(ch->mem);
        delete ch;
        return TWM_ELAUNCH;
    }
    *out = ch;
    return TWM_OK;
}

twm_status twm_chain_launch(twm_chain* ch, void* stream_)
{
    if (!ch || !ch->mem) return TWM_EINVAL;
    int dev = -1;
    cudaGetDevice(&dev);
    if (dev != ch->device) {
        snprintf(t_last_error, sizeof(t_last_error), "twm_chain_launch: the chain was created on device %d, current device is %d",
                 ch->device, dev);
        return TWM_ELAUNCH;
    }
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(ch->grid, 1, 1);
    cfg.blockDim = dim3(twm::chain::THREADS, 1, 1);
    cfg.dynamicSmemBytes = sizeof(twm::chain::Smem);
    cfg.stream = (cudaStream_t)stream_;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;     // the CTAs wait on one another: all of them must be resident
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    const twm::chain::Op* ops = ch->ops;
    cudaError_t e;
    switch (ch->rows) {
        case 1: e = cudaLaunchKernelEx(&cfg, twm::chain::chain_kernel<1>, ops, ch->count, ch->state, ch->done); break;
        case 2: e = cudaLaunchKernelEx(&cfg, twm::chain::chain_kernel<2>, ops, ch->count, ch->state, ch->done); break;
        case 4: e = cudaLaunchKernelEx(&cfg, twm::chain::chain_kernel<4>, ops, ch->count, ch->state, ch->done); break;
        default: e = cudaLaunchKernelEx(&cfg, twm::chain::chain_kernel<8>, ops, ch->count, ch->state, ch->done); break;
    }
    if (e != cudaSuccess) { set_error("launch chain::chain_kernel", e); return TWM_ELAUNCH; }
    return TWM_OK;
}

twm_status twm_chain_info(const twm_chain* ch, twm_chain_info_t* out)
{
    if (!ch || !out) return TWM_EINVAL;
    out->count = ch->count; out->grid = ch->grid; out->rows = ch->rows; out->device_bytes = ch->bytes;
    out->split_tiles = ch->split_tiles; out->max_pieces = ch->max_pieces;
    return TWM_OK;
}

twm_status twm_chain_destroy(twm_chain* ch)
{
    if (!ch) return TWM_EINVAL;
    cudaError_t e = ch->mem ? cudaFree(ch->mem) : cudaSuccess;
    delete ch;
    if (e != cudaSuccess) { set_error("twm_chain_destroy", e); return TWM_ELAUNCH; }
    return TWM_OK;
}

twm_status twm_dequant(const uint8_t* packed, const uint16_t* scales, void* out, int out_dtype,
                       int K, int N, int group_size, void* stream_)
{
    if (!packed || !scales || !out || !shape_ok(1, N, K, group_size)) return TWM_EINVAL;
    if (out_dtype != TWM_F32 && out_dtype != TWM_F16) return TWM_EINVAL;
    if (reinterpret_cast<uintptr_t>(packed) & 15) return TWM_EALIGN;
    twm_status st = ensure_device(nullptr);
    if (st != TWM_OK) return st;
    dim3 grid((N + 127) / 128, K / 32, 1);
    if (grid.y > 65535) return TWM_EINVAL;
    cudaStream_t stream = (cudaStream_t)stream_;
    if (out_dtype == TWM_F16)
        twm::layout::dequant_kernel<__half><<<grid, 128, 0, stream>>>(packed, scales, (__half*)out, K, N, group_size);
    else
        twm::layout::dequant_kernel<float><<<grid, 128, 0, stream>>>(packed, scales, (float*)out, K, N, group_size);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_error("launch dequant_kernel", e); return TWM_ELAUNCH; }
    return TWM_OK;
}

twm_status twm_quantize_pack(const float* w, int w_is_nk, int K, int N, int group_size,
                             uint8_t* packed, uint16_t* scales, void* stream_)
{
    if (!w || !packed || !scales || !shape_ok(1, N, K, group_size)) return TWM_EINVAL;
    if (reinterpret_cast<uintptr_t>(packed) & 15) return TWM_EALIGN;
    twm_status st = ensure_device(nullptr);
    if (st != TWM_OK) return st;
    dim3 grid((N + 127) / 128, K / group_size, 1);
    if (grid.y > 65535) return TWM_EINVAL;
    cudaStream_t stream = (cudaStream_t)stream_;
    if (group_size == 32)
        twm::layout::quantize_pack_kernel<32><<<grid, 128, 0, stream>>>(w, w_is_nk, K, N, packed, scales);
    else
        twm::layout::quantize_pack_kernel<128><<<grid, 128, 0, stream>>>(w, w_is_nk, K, N, packed, scales);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_error("launch quantize_pack_kernel", e); return TWM_ELAUNCH; }
    return TWM_OK;
}

twm_status twm_reorder_to_tw_marlin(const uint8_t* col_major_q4, int K, int N, uint8_t* packed, uint16_t* scales,
                                    void* stream_)
{
    if (!col_major_q4 || !packed || !scales || K < 32 || (K % 32) || N < 1) return TWM_EINVAL;
    if ((reinterpret_cast<uintptr_t>(col_major_q4) & 3) || (reinterpret_cast<uintptr_t>(packed) & 15) ||
        (reinterpret_cast<uintptr_t>(scales) & 1))
        return TWM_EALIGN;
    twm_status st = ensure_device(nullptr);
    if (st != TWM_OK) return st;
    const int nkb = K / 32;
    dim3 grid((nkb + 31) / 32, (N + 31) / 32, 1);
    if (grid.y > 65535) return TWM_EINVAL;
    twm::layout::reorder_q4_0_kernel<<<grid, dim3(32, 32, 1), 0, (cudaStream_t)stream_>>>(
        reinterpret_cast<const uint32_t*>(col_major_q4), nkb, N, packed, scales);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_error("launch reorder_q4_0_kernel", e); return TWM_ELAUNCH; }
    return TWM_OK;
}

twm_status twm_fuse_n(const uint8_t* const* packed_srcs, const uint16_t* const* scales_srcs,
                      const int* ns, int count, int K, int group_size, uint8_t* packed_dst,
                      uint16_t* scales_dst, void* stream_)
{
    if (!packed_srcs || !scales_srcs || !ns || count < 1 || !packed_dst || !scales_dst) return TWM_EINVAL;
    if (K < 32 || (group_size != 32 && group_size != 128) || K % group_size) return TWM_EINVAL;
    long total = 0;
    for (int i = 0; i < count; ++i) {
        if (ns[i] < 1 || !packed_srcs[i] || !scales_srcs[i]) return TWM_EINVAL;
        total += ns[i];
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    long off = 0;
    for (int i = 0; i < count; ++i) {
        // one strided copy per source: K/32 rows of ns[i]*16 bytes, K/G rows of ns[i]*2 bytes
        cudaError_t e = cudaMemcpy2DAsync(packed_dst + off * 16, (size_t)total * 16, packed_srcs[i],
                                          (size_t)ns[i] * 16, (size_t)ns[i] * 16, K / 32,
                                          cudaMemcpyDeviceToDevice, stream);
        if (e == cudaSuccess)
            e = cudaMemcpy2DAsync(scales_dst + off, (size_t)total * 2, scales_srcs[i], (size_t)ns[i] * 2,
                                  (size_t)ns[i] * 2, K / group_size, cudaMemcpyDeviceToDevice, stream);
        if (e != cudaSuccess) { set_error("twm_fuse_n copy", e); return TWM_ELAUNCH; }
        off += ns[i];
    }
    return TWM_OK;
}

twm_status twm_slice_n(const uint8_t* packed_src, const uint16_t* scales_src, int K, int N,
                       int group_size, int n0, int n_len, uint8_t* packed_dst,
                       uint16_t* scales_dst, void* stream_)
{
    if (!packed_src || !scales_src || !packed_dst || !scales_dst) return TWM_EINVAL;
    if (K < 32 || (group_size != 32 && group_size != 128) || K % group_size) return TWM_EINVAL;
    if (n0 < 0 || n_len < 1 || n0 + n_len > N) return TWM_EINVAL;
    cudaStream_t stream = (cudaStream_t)stream_;
    cudaError_t e = cudaMemcpy2DAsync(packed_dst, (size_t)n_len * 16, packed_src + (size_t)n0 * 16,
                                      (size_t)N * 16, (size_t)n_len * 16, K / 32,
                                      cudaMemcpyDeviceToDevice, stream);
    if (e == cudaSuccess)
        e = cudaMemcpy2DAsync(scales_dst, (size_t)n_len * 2, scales_src + n0, (size_t)N * 2,
                              (size_t)n_len * 2, K / group_size, cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) { set_error("twm_slice_n copy", e); return TWM_ELAUNCH; }
    return TWM_OK;
}

twm_status twm_slice_k_offsets(int K, int N, int group_size, int k0, int k_len,
                               size_t* packed_byte_offset, size_t* scales_elem_offset)
{
    if (!packed_byte_offset || !scales_elem_offset) return TWM_EINVAL;
    if ((group_size != 32 && group_size != 128) || K % group_size || N < 1) return TWM_EINVAL;
    if (k0 < 0 || k_len < group_size || k0 % group_size || k_len % group_size || k0 + k_len > K) return TWM_EINVAL;
    *packed_byte_offset = (size_t)(k0 / 32) * N * 16;
    *scales_elem_offset = (size_t)(k0 / group_size) * N;
    return TWM_OK;
}

twm_status twm_device_error(void* stream_, unsigned int* word)
{
    if (!word) return TWM_EINVAL;
    cudaStream_t stream = (cudaStream_t)stream_;
    unsigned int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbolAsync(word, twm::g_error_word, sizeof(unsigned int), 0,
                                              cudaMemcpyDeviceToHost, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e == cudaSuccess && *word != 0)
        e = cudaMemcpyToSymbolAsync(twm::g_error_word, &zero, sizeof(unsigned int), 0, cudaMemcpyHostToDevice, stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) { set_error("twm_device_error", e); return TWM_ELAUNCH; }
    return *word ? TWM_ETIMEOUT : TWM_OK;
}

// ------------------------------------------------------------ decode-step kernels --
twm_status twm_embed(float* x, const void* table, const int* tokens, int rows, int hidden, int flags, void* stream)
{
    if (!x || !table || !tokens || rows < 1 || hidden < 1) return TWM_EINVAL;
    twm_status st = ensure_device(nullptr);
    if (st != TWM_OK) return st;
    return launch_op("twm_embed", twm::ops::embed_kernel, dim3((hidden + 255) / 256, rows), dim3(256), 0, flags, stream,
                     x, (const __half*)table, tokens, hidden);
}

twm_status twm_rmsnorm(void* y, const float* x, const float* gamma, int rows, int hidden, float eps, int flags,
                       void* stream)
{
    if (!y || !x || !gamma || rows < 1 || hidden < 1) return TWM_EINVAL;
    twm_status st = ensure_device(nullptr);
    if (st != TWM_OK) return st;
    return launch_op("twm_rmsnorm", twm::ops::rmsnorm_kernel, dim3(rows), dim3(256), 0, flags, stream, (__half*)y,
                     const_cast<float*>(x), (const float*)nullptr, gamma, hidden, eps);
}

twm_status twm_add_rmsnorm(void* y, float* x, const float* add, const float* gamma, int rows, int hidden, float eps,
                           int flags, void* stream)
{
    if (!x || !add || (y && !gamma) || rows < 1 || hidden < 1) return TWM_EINVAL;
    twm_status st = ensure_device(nullptr);
    if (st != TWM_OK) return st;
    return launch_op("twm_add_rmsnorm", twm::ops::rmsnorm_kernel, dim3(rows), dim3(256), 0, flags, stream, (__half*)y, x,
                     add, gamma, hidden, eps);
}

twm_status twm_rope_append(void* q_out, void* k_cache, void* v_cache, const void* qkv, const float* bias, int rows,
                           int num_heads, int num_kv_heads, int head_dim, const int* pos_buf, int max_seq,
                           float rope_base, int flags, void* stream)
{
    if (!q_out || !k_cache || !v_cache || !qkv || !pos_buf || rows < 1) return TWM_EINVAL;
    if (num_heads < 1 || num_kv_heads < 1 || head_dim < 2 || (head_dim & 1) || max_seq < 1) return TWM_EINVAL;
    twm_status st = ensure_device(nullptr);
    if (st != TWM_OK) return st;
    const int total = (num_heads + num_kv_heads) * head_dim;
    return launch_op("twm_rope_append", twm::ops::rope_append_kernel, dim3((total + 255) / 256, rows), dim3(256), 0, flags,
                     stream, (__half*)q_out, (__half*)k_cache, (__half*)v_cache, (const __half*)qkv, bias, num_heads,
                     num_kv_heads, head_dim, pos_buf, max_seq, rope_base);
}

size_t twm_attn_scratch_bytes(int rows, int num_heads, int head_dim, int max_seq)
{
    if (rows < 1 || num_heads < 1 || head_dim < 1 || max_seq < 1) return 0;
    const size_t chunks = (size_t)(max_seq + twm::ops::ATT_CHUNK - 1) / twm::ops::ATT_CHUNK;
    return (size_t)rows * num_heads * chunks * (head_dim + 2) * sizeof(float);
}

namespace {
twm_status attn_decode_common(void* out, const void* q_or_qkv, void* k_cache, void* v_cache, int rows, int num_heads,
                              int num_kv_heads, int head_dim, const int* len_buf, int max_seq, void* scratch,
                              size_t scratch_bytes, const float* bias, const float* rope_table, const int* pos_buf,
                              int flags, void* stream)
{
    if (!out || !q_or_qkv || !k_cache || !v_cache || !len_buf || !scratch || rows < 1 || rows > 65535) return TWM_EINVAL;
    if (head_dim != 128 || num_heads < 1 || num_kv_heads < 1 || num_heads % num_kv_heads) return TWM_EINVAL;
    if (num_heads / num_kv_heads > twm::ops::ATT_MAX_GROUP) return TWM_EINVAL;
    if (scratch_bytes < twm_attn_scratch_bytes(rows, num_heads, head_dim, max_seq)) return TWM_EWORKSPACE;
    if (reinterpret_cast<uintptr_t>(q_or_qkv) & 7) return TWM_EALIGN;
    twm_status st = ensure_device(nullptr);
    if (st != TWM_OK) return st;
    const int chunks = (max_seq + twm::ops::ATT_CHUNK - 1) / twm::ops::ATT_CHUNK;
    if (chunks > 1024) return TWM_EINVAL;          // the merge pass keeps one weight per chunk in shared memory
    // one 32-token chunk per CTA while that is at most two waves of CTAs (four fit an SM); beyond that
    // (many sequences in lock step) each CTA walks 2, 4 or 8 chunks
    int sms = kDefaultSms;
    st = ensure_device(&sms);
    if (st != TWM_OK) return st;
    int span = 1;
    while (span < 8 && (long)((chunks + span - 1) / span) * num_kv_heads * rows > 2L * 4 * sms) span *= 2;
    const int parts = (chunks + span - 1) / span;
    // CTAs that walk several chunks run the tensor-core form of the pass (four warps, 8 tokens of a chunk each)
    const dim3 grid(parts, num_kv_heads, rows), block(span > 1 ? 32 * twm::ops::ATT_MMA_WARPS : 32 * (num_heads / num_kv_heads));
    float* sp = (float*)scratch;
    const __half* qp = (const __half*)q_or_qkv;
    __half *kp = (__half*)k_cache, *vp = (__half*)v_cache;
    const float* nof = nullptr;
    const int* noi = nullptr;
    if (rope_table && span > 1)
        st = launch_op("twm_attn_decode_rope(spans)", twm::ops::attn_span_mma_kernel<128, true>, grid, block, twm::ops::ATT_MMA_SMEM_BYTES, flags, stream,
                       sp, qp, kp, vp, num_heads, num_kv_heads, len_buf, parts, span, max_seq, bias, rope_table, pos_buf);
    else if (rope_table)
        st = launch_op("twm_attn_decode_rope(chunks)", twm::ops::attn_chunk_kernel<128, true>, grid, block, 0, flags, stream,
                       sp, qp, kp, vp, num_heads, num_kv_heads, len_buf, parts, span, max_seq, bias, rope_table, pos_buf);
    else if (span > 1)
        st = launch_op("twm_attn_decode(spans)", twm::ops::attn_span_mma_kernel<128, false>, grid, block, twm::ops::ATT_MMA_SMEM_BYTES, flags, stream,
                       sp, qp, kp, vp, num_heads, num_kv_heads, len_buf, parts, span, max_seq, nof, nof, noi);
    else
        st = launch_op("twm_attn_decode(chunks)", twm::ops::attn_chunk_kernel<128, false>, grid, block, 0, flags, stream,
                       sp, qp, kp, vp, num_heads, num_kv_heads, len_buf, parts, span, max_seq, nof, nof, noi);
    if (st != TWM_OK) return st;
    return launch_op("twm_attn_decode(merge)", twm::ops::attn_merge_kernel<128>, dim3(num_heads, rows), dim3(128 * twm::ops::ATT_MERGE_PARTS), 0, flags,
                     stream, (__half*)out, (const float*)scratch, len_buf, parts, span);
}
}  // namespace

twm_status twm_attn_decode(void* out, const void* q, const void* k_cache, const void* v_cache, int rows, int num_heads,
                           int num_kv_heads, int head_dim, const int* len_buf, int max_seq, void* scratch,
                           size_t scratch_bytes, int flags, void* stream)
{
    return attn_decode_common(out, q, const_cast<void*>(k_cache), const_cast<void*>(v_cache), rows, num_heads, num_kv_heads,
                              head_dim, len_buf, max_seq, scratch, scratch_bytes, nullptr, nullptr, nullptr, flags, stream);
}

twm_status twm_rope_table(float* table, const int* pos_buf, int head_dim, float rope_base, int flags, void* stream)
{
    if (!table || !pos_buf || head_dim < 2 || (head_dim & 1)) return TWM_EINVAL;
    twm_status st = ensure_device(nullptr);
    if (st != TWM_OK) return st;
    return launch_op("twm_rope_table", twm::ops::rope_table_kernel, dim3((head_dim / 2 + 255) / 256), dim3(256), 0, flags, stream,
                     table, pos_buf, head_dim, rope_base);
}

twm_status twm_attn_decode_rope(void* out, const void* qkv, const float* bias, const float* rope_table, void* k_cache,
                                void* v_cache, int rows, int num_heads, int num_kv_heads, int head_dim, const int* pos_buf,
                                const int* len_buf, int max_seq, void* scratch, size_t scratch_bytes, int flags, void* stream)
{
    if (!rope_table || !pos_buf) return TWM_EINVAL;
    return attn_decode_common(out, qkv, k_cache, v_cache, rows, num_heads, num_kv_heads, head_dim, len_buf, max_seq, scratch,
                              scratch_bytes, bias, rope_table, pos_buf, flags, stream);
}

twm_status twm_silu_mul(void* act, const void* gate_up, int rows, int ffn, int flags, void* stream)
{
    if (!act || !gate_up || rows < 1 || ffn < 1) return TWM_EINVAL;
    twm_status st = ensure_device(nullptr);
    if (st != TWM_OK) return st;
    return launch_op("twm_silu_mul", twm::ops::silu_mul_kernel, dim3((rows * ffn + 255) / 256), dim3(256), 0, flags,
                     stream, (__half*)act, (const __half*)gate_up, ffn, rows);
}

twm_status twm_lm_head(float* logits, const void* x, const void* w, int hidden, int vocab, int flags, void* stream)
{
    if (!logits || !x || !w || hidden < 8 || (hidden & 7) || vocab < 1 || hidden > 24576) return TWM_EINVAL;
    if ((reinterpret_cast<uintptr_t>(w) & 15) || (reinterpret_cast<uintptr_t>(x) & 1)) return TWM_EALIGN;
    int sms = kDefaultSms;
    twm_status st = ensure_device(&sms);
    if (st != TWM_OK) return st;
    const int grid = std::min((vocab + 7) / 8, sms * 8);
    return launch_op("twm_lm_head", twm::ops::lm_head_kernel, dim3(grid), dim3(256), (size_t)hidden * 2, flags, stream,
                     logits, (const __half*)x, (const __half*)w, hidden, vocab);
}

// ------------------------------------------------------- tensor-parallel plumbing --
namespace {
constexpr size_t kCommHeaderBytes = 4096;      // state words (first 256 bytes) and flags (from byte 1024)
}

size_t twm_comm_bytes(int n_ranks, long slot_elems)
{
    if (n_ranks < 1 || n_ranks > 8 || slot_elems < 1) return 0;
    return kCommHeaderBytes + (size_t)2 * n_ranks * slot_elems * sizeof(float);
}

twm_status twm_comm_layout(void* base, int n_ranks, long slot_elems, float** data, unsigned int** flags,
                           unsigned int** state)
{
    if (!base || n_ranks < 1 || n_ranks > 8 || slot_elems < 1) return TWM_EINVAL;
    if (reinterpret_cast<uintptr_t>(base) & 255) return TWM_EALIGN;
    if (state) *state = (unsigned int*)base;
    if (flags) *flags = (unsigned int*)((char*)base + 1024);
    if (data) *data = (float*)((char*)base + kCommHeaderBytes);
    return TWM_OK;
}

twm_status twm_allreduce_add_rmsnorm(void* y, float* x, const twm_comm* comm, const float* gamma, int rows, int hidden,
                                     float eps, int flags, void* stream)
{
    if (!x || !comm || (y && !gamma) || rows < 1 || rows > 65535 || hidden < 1) return TWM_EINVAL;
    if (comm->n_ranks < 1 || comm->n_ranks > 8 || comm->rank < 0 || comm->rank >= comm->n_ranks) return TWM_EINVAL;
    if (comm->slot_elems < (long)rows * hidden || (hidden & 3) || (comm->slot_elems & 3)) return TWM_EINVAL;
    if (hidden > 4 * twm::ops::RMS_SEG_VECS * twm::ops::ARN_MAX_SEGS) return TWM_EINVAL;
    if ((reinterpret_cast<uintptr_t>(x) & 15) || (gamma && (reinterpret_cast<uintptr_t>(gamma) & 15)) ||
        (y && (reinterpret_cast<uintptr_t>(y) & 7)))
        return TWM_EALIGN;
    twm_status st = ensure_device(nullptr);
    if (st != TWM_OK) return st;
    // one 256-vector segment of the row per CTA up to eight CTAs (one cluster per row), two beyond that
    const int nseg = (hidden / 4 + twm::ops::RMS_SEG_VECS - 1) / twm::ops::RMS_SEG_VECS;
    const int ncta = std::min(nseg, 8);
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(ncta, rows, 1);
    cfg.blockDim = dim3(twm::ops::ARN_THREADS, 1, 1);
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = ncta;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (flags & TWM_FLAG_PDL) ? 2 : 1;
    const unsigned long long wait_ns = comm->wait_ns ? comm->wait_ns : 2000000000ull;     // two seconds unless the caller says otherwise
    cudaError_t e = cudaLaunchKernelEx(&cfg, twm::ops::allreduce_add_rmsnorm_kernel, (__half*)y, x,
                                       (const float*)comm->data[comm->rank], (const unsigned int*)comm->flags[comm->rank],
                                       comm->state, gamma, hidden, eps, comm->n_ranks, comm->slot_elems, wait_ns);
    if (e != cudaSuccess) { set_error("twm_allreduce_add_rmsnorm", e); return TWM_ELAUNCH; }
    return TWM_OK;
}

twm_status twm_ipc_alloc(size_t bytes, void** ptr)
{
    if (!ptr || bytes == 0) return TWM_EINVAL;
    cudaError_t e = cudaMalloc(ptr, bytes);
    if (e == cudaSuccess) e = cudaMemset(*ptr, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) { set_error("twm_ipc_alloc", e); return TWM_ELAUNCH; }
    return TWM_OK;
}

twm_status twm_ipc_free(void* ptr)
{
    cudaError_t e = cudaFree(ptr);
    if (e != cudaSuccess) { set_error("twm_ipc_free", e); return TWM_ELAUNCH; }
    return TWM_OK;
}

twm_status twm_ipc_get_handle(void* ptr, unsigned char handle[64])
{
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    if (!ptr || !handle) return TWM_EINVAL;
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
    if (e != cudaSuccess) { set_error("cudaIpcGetMemHandle", e); return TWM_ELAUNCH; }
    memcpy(handle, &h, 64);
    return TWM_OK;
}

twm_status twm_ipc_open(const unsigned char handle[64], void** ptr)
{
    if (!ptr || !handle) return TWM_EINVAL;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, 64);
    cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) { set_error("cudaIpcOpenMemHandle", e); return TWM_ELAUNCH; }
    return TWM_OK;
}

twm_status twm_ipc_close(void* ptr)
{
    cudaError_t e = cudaIpcCloseMemHandle(ptr);
    if (e != cudaSuccess) { set_error("cudaIpcCloseMemHandle", e); return TWM_ELAUNCH; }
    return TWM_OK;
}

size_t twm_argmax_scratch_bytes(void) { return (size_t)kArgmaxParts * 8; }

twm_status twm_argmax_advance(int* token_out, int* history, int history_capacity, int* pos_buf, int* len_buf,
                              int* step_buf, const float* logits, int n, void* scratch, size_t scratch_bytes, int flags,
                              void* stream)
{
    if (!token_out || !pos_buf || !len_buf || !step_buf || !logits || !scratch || n < 1) return TWM_EINVAL;
    if (history && history_capacity < 1) return TWM_EINVAL;
    if (scratch_bytes < twm_argmax_scratch_bytes()) return TWM_EWORKSPACE;
    twm_status st = ensure_device(nullptr);
    if (st != TWM_OK) return st;
    float* pval = (float*)scratch;
    int* pidx = (int*)((char*)scratch + (size_t)kArgmaxParts * 4);
    st = launch_op("twm_argmax(partial)", twm::ops::argmax_partial_kernel, dim3(kArgmaxParts), dim3(256), 0, flags, stream,
                   pval, pidx, logits, n);
    if (st != TWM_OK) return st;
    return launch_op("twm_argmax(final)", twm::ops::argmax_final_kernel, dim3(1), dim3(256), 0, flags, stream, token_out,
                     history, history_capacity, pos_buf, len_buf, step_buf, (const float*)pval, (const int*)pidx, kArgmaxParts, n);
}

const char* twm_status_string(twm_status s)
{
    switch (s) {
        case TWM_OK: return "ok";
        case TWM_EINVAL: return "invalid argument (shape, dtype, group size or null pointer)";
        case TWM_EALIGN: return "pointer alignment (packed and workspace need 16 bytes)";
        case TWM_EWORKSPACE: return "split-K workspace missing or too small (see twm_workspace_bytes)";
        case TWM_ELAUNCH: return "CUDA launch or copy failed (see twm_last_error)";
        case TWM_EARCH: return "device is not sm_100 (B200)";
        case TWM_ETIMEOUT: return "a bounded device-side wait expired";
    }
    return "unknown status";
}

const char* twm_last_error(void) { return t_last_error; }

const char* twm_version(void) { return "twmarlin 0.1 sm_100a"; }

}  // extern "C"
