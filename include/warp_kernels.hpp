// warp_kernels.hpp — C++ host mirror of the reference's `warp_kernels::quantize` TW-Marlin interface
// over the C ABI of libtwmarlin.so (twmarlin.h).
//
// The reference's host side is Rust (crates/kernels/src/quantize.rs); this header keeps its function
// names, argument order and error behaviour so that a caller written against the Rust crate reads the
// same in C++:
//
//   gemm_tw_marlin_m1              quantize.rs:1301-1360
//   gemm_tw_marlin_m1_from_buffer  quantize.rs:1731-1782
//   gemm_tw_marlin_m1_indirect     quantize_indirect.rs:228-253
//   quantize_f32_to_tw_marlin      quantize.rs:1171-1180
//   fuse_tw_marlin_n               quantize.rs:1018-1063
//   TWMarlinWeights                quantize.rs:1067-1165
//
// Differences that follow from the ahead-of-time kernels: there is no KernelCache argument (nothing is
// compiled at run time) and no WarpDevice (the device is the current CUDA device; the stream is passed
// explicitly).  A failed call throws DeviceError where the Rust functions return Err(DeviceError).
// Header only; link with -ltwmarlin.  Tensors are non-owning views of device memory.
#pragma once

#include <cstddef>
#include <cstdint>
#include <stdexcept>
#include <string>
#include <vector>

#include "twmarlin.h"

namespace warp_kernels {

constexpr uint32_t BLOCK_SIZE = 32;   // quantize.rs:25

struct DeviceError : std::runtime_error {
    twm_status status;
    DeviceError(twm_status st, const std::string& where)
        : std::runtime_error(where + ": " + twm_status_string(st) + (twm_last_error()[0] ? std::string(" (") + twm_last_error() + ")" : std::string())),
          status(st) {}
};

inline void check(twm_status st, const char* where) {
    if (st != TWM_OK) throw DeviceError(st, where);
}

// A view of device memory holding `numel` elements of T (stands in for GpuTensor<T>).
template <typename T>
struct GpuTensor {
    T* data = nullptr;
    size_t numel = 0;
};

struct f16 { uint16_t bits; };   // IEEE binary16 storage (half::f16 in the reference)

template <typename T> struct dtype_of;
template <> struct dtype_of<float> { static constexpr int value = TWM_F32; };
template <> struct dtype_of<f16> { static constexpr int value = TWM_F16; };

// Split-K scratch shared by the GEMMs of one stream (the reference allocates its scratch inside the
// launcher; here the caller owns it: twm_workspace_bytes says how much, zero it once).
struct Workspace {
    void* ptr = nullptr;
    size_t bytes = 0;
};

namespace quantize {

namespace detail {
template <typename TA, typename TC>
inline void gemm(const TA* a, long lda, const uint8_t* packed, const uint16_t* scales, TC* c, long ldc, uint32_t m, uint32_t n,
                 uint32_t k, uint32_t group_size, const Workspace& ws, void* stream, int flags, const uint32_t* packed_offsets,
                 const uint32_t* scales_offsets, int expert_idx) {
    twm_gemm_args args{};
    args.M = (int)m; args.N = (int)n; args.K = (int)k; args.group_size = (int)group_size;
    args.a_dtype = dtype_of<TA>::value; args.c_dtype = dtype_of<TC>::value;
    args.a = a; args.lda = lda; args.packed = packed; args.scales = scales; args.c = c; args.ldc = ldc;
    args.workspace = ws.ptr; args.workspace_bytes = ws.bytes;
    args.flags = flags;
    args.packed_offsets = packed_offsets; args.scales_offsets = scales_offsets; args.expert_idx = expert_idx;
    check(twm_gemm_w4a16(&args, stream), "twm_gemm_w4a16");
}
}  // namespace detail

// C[1,n] = A[1,k] x dequant(packed, scales).  The reference asserts k % 32 == 0 (quantize.rs:1311); so does this.
template <typename TA, typename TC>
inline void gemm_tw_marlin_m1(const GpuTensor<TA>& a, const GpuTensor<uint8_t>& packed, const GpuTensor<f16>& scales,
                              GpuTensor<TC>& c, uint32_t n, uint32_t k, const Workspace& ws = {}, void* stream = nullptr,
                              uint32_t group_size = BLOCK_SIZE, int flags = 0) {
    if (k % BLOCK_SIZE != 0) throw DeviceError(TWM_EINVAL, "gemm_tw_marlin_m1: k % 32 != 0");
    if (a.numel < k || c.numel < n || packed.numel < (size_t)(k / 32) * n * 16 || scales.numel < (size_t)(k / group_size) * n)
        throw DeviceError(TWM_EINVAL, "gemm_tw_marlin_m1: a tensor is smaller than the stated shape");
    detail::gemm(a.data, (long)k, packed.data, reinterpret_cast<const uint16_t*>(scales.data), c.data, (long)n, 1, n, k, group_size,
                 ws, stream, flags, nullptr, nullptr, 0);
}

// The M > 1 form (no counterpart in the reference, whose TW-Marlin kernel is M = 1 only).
template <typename TA, typename TC>
inline void gemm_tw_marlin(const GpuTensor<TA>& a, const GpuTensor<uint8_t>& packed, const GpuTensor<f16>& scales,
                           GpuTensor<TC>& c, uint32_t m, uint32_t n, uint32_t k, const Workspace& ws, void* stream = nullptr,
                           uint32_t group_size = BLOCK_SIZE, int flags = 0) {
    if (a.numel < (size_t)m * k || c.numel < (size_t)m * n) throw DeviceError(TWM_EINVAL, "gemm_tw_marlin: A or C too small");
    detail::gemm(a.data, (long)k, packed.data, reinterpret_cast<const uint16_t*>(scales.data), c.data, (long)n, m, n, k, group_size,
                 ws, stream, flags, nullptr, nullptr, 0);
}

// Sub-ranges of two big buffers: packed_offset in bytes, scales_offset in elements (quantize.rs:1731-1741).
template <typename TA, typename TC>
inline void gemm_tw_marlin_m1_from_buffer(const GpuTensor<TA>& a, const GpuTensor<uint8_t>& packed_buf, size_t packed_offset,
                                          const GpuTensor<f16>& scales_buf, size_t scales_offset, GpuTensor<TC>& c, uint32_t n,
                                          uint32_t k, const Workspace& ws = {}, void* stream = nullptr,
                                          uint32_t group_size = BLOCK_SIZE, int flags = 0) {
    if (packed_offset > packed_buf.numel || scales_offset > scales_buf.numel)
        throw DeviceError(TWM_EINVAL, "gemm_tw_marlin_m1_from_buffer: offset past the buffer");
    GpuTensor<uint8_t> p{packed_buf.data + packed_offset, packed_buf.numel - packed_offset};
    GpuTensor<f16> s{scales_buf.data + scales_offset, scales_buf.numel - scales_offset};
    gemm_tw_marlin_m1(a, p, s, c, n, k, ws, stream, group_size, flags);
}

// Expert-indexed form (quantize_indirect.rs:228-237): the kernel itself reads packed_offsets[expert_idx]
// (bytes) and scales_offsets[expert_idx] (elements) from device memory.
template <typename TA, typename TC>
inline void gemm_tw_marlin_m1_indirect(const GpuTensor<TA>& a, const GpuTensor<uint8_t>& packed_buf,
                                       const GpuTensor<uint32_t>& packed_offsets, const GpuTensor<f16>& scales_buf,
                                       const GpuTensor<uint32_t>& scales_offsets, uint32_t expert_idx, GpuTensor<TC>& c,
                                       uint32_t n, uint32_t k, const Workspace& ws = {}, void* stream = nullptr,
                                       uint32_t group_size = BLOCK_SIZE, int flags = 0) {
    if (k % BLOCK_SIZE != 0) throw DeviceError(TWM_EINVAL, "gemm_tw_marlin_m1_indirect: k % 32 != 0");
    if (expert_idx >= packed_offsets.numel || expert_idx >= scales_offsets.numel)
        throw DeviceError(TWM_EINVAL, "gemm_tw_marlin_m1_indirect: expert index past the offset tables");
    detail::gemm(a.data, (long)k, packed_buf.data, reinterpret_cast<const uint16_t*>(scales_buf.data), c.data, (long)n, 1, n, k,
                 group_size, ws, stream, flags, packed_offsets.data, scales_offsets.data, (int)expert_idx);
}

// F32 weights [k, n] (or [n, k] with w_is_nk) -> packed u8 [k/32, n, 16] and scales f16 [k/group, n], both
// preallocated by the caller.
inline void quantize_f32_to_tw_marlin(const GpuTensor<float>& weights, uint32_t k, uint32_t n, GpuTensor<uint8_t>& packed,
                                      GpuTensor<f16>& scales, uint32_t group_size = BLOCK_SIZE, bool w_is_nk = false,
                                      void* stream = nullptr) {
    if (weights.numel < (size_t)k * n || packed.numel < (size_t)(k / 32) * n * 16 || scales.numel < (size_t)(k / group_size) * n)
        throw DeviceError(TWM_EINVAL, "quantize_f32_to_tw_marlin: a tensor is smaller than the stated shape");
    check(twm_quantize_pack(weights.data, w_is_nk ? 1 : 0, (int)k, (int)n, (int)group_size, packed.data,
                            reinterpret_cast<uint16_t*>(scales.data), stream),
          "twm_quantize_pack");
}

// One quantised matrix (quantize.rs:1067-1165).
struct TWMarlinWeights {
    GpuTensor<uint8_t> packed;
    GpuTensor<f16> scales;
    uint32_t k = 0, n = 0, group_size = BLOCK_SIZE;
};

// Concatenate matrices that share K along N (fused QKV, fused gate+up): quantize.rs:1018-1063.
inline void fuse_tw_marlin_n(const std::vector<TWMarlinWeights>& parts, TWMarlinWeights& out, void* stream = nullptr) {
    if (parts.empty()) throw DeviceError(TWM_EINVAL, "fuse_tw_marlin_n: nothing to fuse");
    std::vector<const uint8_t*> ps;
    std::vector<const uint16_t*> ss;
    std::vector<int> ns;
    uint32_t total = 0;
    for (const TWMarlinWeights& w : parts) {
        if (w.k != parts[0].k || w.group_size != parts[0].group_size)
            throw DeviceError(TWM_EINVAL, "fuse_tw_marlin_n: parts differ in K or group size");
        ps.push_back(w.packed.data);
        ss.push_back(reinterpret_cast<const uint16_t*>(w.scales.data));
        ns.push_back((int)w.n);
        total += w.n;
    }
    if (out.n != total || out.k != parts[0].k || out.group_size != parts[0].group_size)
        throw DeviceError(TWM_EINVAL, "fuse_tw_marlin_n: destination shape does not match the parts");
    check(twm_fuse_n(ps.data(), ss.data(), ns.data(), (int)parts.size(), (int)out.k, (int)out.group_size, out.packed.data,
                     reinterpret_cast<uint16_t*>(out.scales.data), stream),
          "twm_fuse_n");
}

}  // namespace quantize
}  // namespace warp_kernels
