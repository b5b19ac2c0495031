// Exercises include/warp_kernels.hpp.  Without arguments: host-only checks (no CUDA call is
// reached).  With "gpu <dir>": quantises seeded weights, runs gemm_tw_marlin_m1 (FP32 and FP16),
// the from_buffer and indirect forms and fuse_tw_marlin_n on the current device and writes inputs
// and outputs as raw files into <dir> for the Python test to check against the oracle.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "warp_kernels.hpp"

using namespace warp_kernels;
using namespace warp_kernels::quantize;

static int host_checks() {
    int bad = 0;
    GpuTensor<float> a{reinterpret_cast<float*>(0x1000), 64};
    GpuTensor<uint8_t> p{reinterpret_cast<uint8_t*>(0x2000), 64};
    GpuTensor<f16> s{reinterpret_cast<f16*>(0x3000), 64};
    GpuTensor<float> c{reinterpret_cast<float*>(0x4000), 64};
    try { gemm_tw_marlin_m1(a, p, s, c, 64, 100); ++bad; }                       // k % 32 != 0
    catch (const DeviceError& e) { if (e.status != TWM_EINVAL) ++bad; }
    try { gemm_tw_marlin_m1(a, p, s, c, 64, 64); ++bad; }                        // packed too small for the shape
    catch (const DeviceError& e) { if (e.status != TWM_EINVAL) ++bad; }
    try { std::vector<TWMarlinWeights> none; TWMarlinWeights out; fuse_tw_marlin_n(none, out); ++bad; }
    catch (const DeviceError& e) { if (e.status != TWM_EINVAL) ++bad; }
    twm_plan_t pl;
    if (twm_plan(1, 4608, 3584, 128, 148, 0, 0, &pl) != TWM_OK || pl.grid_x * pl.grid_y < 100) ++bad;
    std::printf("host checks: %s\n", bad ? "FAILED" : "ok");
    return bad;
}

template <typename T>
static void dump(const std::string& path, const std::vector<T>& v) {
    FILE* f = std::fopen(path.c_str(), "wb");
    if (!f) { std::perror(path.c_str()); std::exit(2); }
    std::fwrite(v.data(), sizeof(T), v.size(), f);
    std::fclose(f);
}
#define CUDA_OK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { std::fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_)); std::exit(3); } } while (0)
template <typename T>
static GpuTensor<T> dev_alloc(size_t n) { GpuTensor<T> t; t.numel = n; CUDA_OK(cudaMalloc(reinterpret_cast<void**>(&t.data), n * sizeof(T))); CUDA_OK(cudaMemset(t.data, 0, n * sizeof(T))); return t; }

static uint16_t f32_to_f16_bits(float f) {           // round to nearest even; inputs here are small normals
    uint32_t x; std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    int32_t e = (int32_t)((x >> 23) & 0xff) - 127 + 15;
    uint32_t m = x & 0x7fffffu;
    if (e <= 0) return (uint16_t)sign;
    uint32_t h = sign | ((uint32_t)e << 10) | (m >> 13);
    const uint32_t rem = m & 0x1fffu;
    if (rem > 0x1000u || (rem == 0x1000u && (h & 1u))) ++h;
    return (uint16_t)h;
}

static int gpu_run(const std::string& dir) {
    const uint32_t k = 1024, n1 = 384, n2 = 256, n = n1 + n2, group = 128;
    uint32_t lcg = 12345u;
    auto rnd = [&]() { lcg = lcg * 1664525u + 1013904223u; return ((lcg >> 8) & 0xffff) / 65536.0f - 0.5f; };
    std::vector<float> w1((size_t)k * n1), w2((size_t)k * n2), a32(k);
    for (float& v : w1) v = 0.08f * rnd();
    for (float& v : w2) v = 0.08f * rnd();
    for (float& v : a32) v = 4.0f * rnd();
    std::vector<uint16_t> a16(k);
    for (uint32_t i = 0; i < k; ++i) a16[i] = f32_to_f16_bits(a32[i]);

    GpuTensor<float> dw1 = dev_alloc<float>(w1.size()), dw2 = dev_alloc<float>(w2.size()), da32 = dev_alloc<float>(k);
    GpuTensor<f16> da16 = dev_alloc<f16>(k);
    CUDA_OK(cudaMemcpy(dw1.data, w1.data(), w1.size() * 4, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(dw2.data, w2.data(), w2.size() * 4, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(da32.data, a32.data(), k * 4, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(da16.data, a16.data(), k * 2, cudaMemcpyHostToDevice));

    TWMarlinWeights q1{dev_alloc<uint8_t>((size_t)(k / 32) * n1 * 16), dev_alloc<f16>((size_t)(k / group) * n1), k, n1, group};
    TWMarlinWeights q2{dev_alloc<uint8_t>((size_t)(k / 32) * n2 * 16), dev_alloc<f16>((size_t)(k / group) * n2), k, n2, group};
    TWMarlinWeights qf{dev_alloc<uint8_t>((size_t)(k / 32) * n * 16), dev_alloc<f16>((size_t)(k / group) * n), k, n, group};
    quantize_f32_to_tw_marlin(dw1, k, n1, q1.packed, q1.scales, group);
    quantize_f32_to_tw_marlin(dw2, k, n2, q2.packed, q2.scales, group);
    fuse_tw_marlin_n({q1, q2}, qf);

    Workspace ws;
    ws.bytes = twm_workspace_bytes(1, (int)n, (int)k, (int)group);
    if (ws.bytes) { CUDA_OK(cudaMalloc(&ws.ptr, ws.bytes)); CUDA_OK(cudaMemset(ws.ptr, 0, ws.bytes)); }

    GpuTensor<float> c32 = dev_alloc<float>(n);
    GpuTensor<f16> c16 = dev_alloc<f16>(n), c16b = dev_alloc<f16>(n2), c16i = dev_alloc<f16>(n1);
    gemm_tw_marlin_m1(da32, qf.packed, qf.scales, c32, n, k, ws, nullptr, group);            // the reference's f32 signature
    gemm_tw_marlin_m1(da16, qf.packed, qf.scales, c16, n, k, ws, nullptr, group);
    // q2 again, addressed as a sub-range of "big buffers" (here: q2's own tensors at offset 0)
    gemm_tw_marlin_m1_from_buffer(da16, q2.packed, 0, q2.scales, 0, c16b, n2, k, ws, nullptr, group);
    // q1 through device-side offset tables with two entries (the second one selected)
    const uint32_t offs_host[2] = {0xffffff00u, 0u};
    GpuTensor<uint32_t> po = dev_alloc<uint32_t>(2), so = dev_alloc<uint32_t>(2);
    CUDA_OK(cudaMemcpy(po.data, offs_host, 8, cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(so.data, offs_host, 8, cudaMemcpyHostToDevice));
    gemm_tw_marlin_m1_indirect(da16, q1.packed, po, q1.scales, so, 1, c16i, n1, k, ws, nullptr, group);
    CUDA_OK(cudaDeviceSynchronize());
    unsigned int word = 0;
    if (twm_device_error(nullptr, &word) != TWM_OK || word != 0) { std::fprintf(stderr, "device error word %u\n", word); return 4; }

    std::vector<uint8_t> hp((size_t)(k / 32) * n * 16);
    std::vector<uint16_t> hs((size_t)(k / group) * n), h16(n), h16b(n2), h16i(n1);
    std::vector<float> h32(n);
    CUDA_OK(cudaMemcpy(hp.data(), qf.packed.data, hp.size(), cudaMemcpyDeviceToHost));
    CUDA_OK(cudaMemcpy(hs.data(), qf.scales.data, hs.size() * 2, cudaMemcpyDeviceToHost));
    CUDA_OK(cudaMemcpy(h32.data(), c32.data, n * 4, cudaMemcpyDeviceToHost));
    CUDA_OK(cudaMemcpy(h16.data(), c16.data, n * 2, cudaMemcpyDeviceToHost));
    CUDA_OK(cudaMemcpy(h16b.data(), c16b.data, n2 * 2, cudaMemcpyDeviceToHost));
    CUDA_OK(cudaMemcpy(h16i.data(), c16i.data, n1 * 2, cudaMemcpyDeviceToHost));
    dump(dir + "/w1.f32", w1); dump(dir + "/w2.f32", w2); dump(dir + "/a.f32", a32); dump(dir + "/a.f16", a16);
    dump(dir + "/packed.u8", hp); dump(dir + "/scales.u16", hs);
    dump(dir + "/c.f32", h32); dump(dir + "/c.f16", h16); dump(dir + "/c_from_buffer.f16", h16b); dump(dir + "/c_indirect.f16", h16i);
    std::printf("gpu run: ok k=%u n1=%u n2=%u group=%u\n", k, n1, n2, group);
    return 0;
}

int main(int argc, char** argv) {
    if (argc >= 3 && std::strcmp(argv[1], "gpu") == 0) return gpu_run(argv[2]);
    return host_checks();
}
