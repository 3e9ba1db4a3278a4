// A read-only pass over a device buffer: 32-bit checksum (XOR of all 32-bit words, each rotated by its
// position inside its 16-byte group so that swapped words show).  Used to verify that a weight upload
// arrived intact without reading it back, and, because it only reads, as the read-only HBM bandwidth
// probe the benchmark reports beside the copy bandwidth.  No reference counterpart.
#include <algorithm>

#include "vx_internal.h"

namespace {

constexpr int kThreads = 512;
constexpr int kUnroll = 8;   // 16-byte loads in flight per thread

__device__ __forceinline__ uint32_t fold(uint4 v) {
    return v.x ^ __funnelshift_l(v.y, v.y, 8) ^ __funnelshift_l(v.z, v.z, 16) ^ __funnelshift_l(v.w, v.w, 24);
}

__global__ void __launch_bounds__(kThreads) checksum_kernel(const uint4* __restrict__ in, size_t n16, uint32_t* out) {
    const size_t stride = (size_t)gridDim.x * kThreads;
    size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x;
    uint32_t acc = 0;
    for (; i + (kUnroll - 1) * stride < n16; i += kUnroll * stride) {
        uint4 v[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) v[u] = __ldcs(in + i + u * stride);   // streaming: read once
#pragma unroll
        for (int u = 0; u < kUnroll; ++u) acc ^= fold(v[u]);
    }
    for (; i < n16; i += stride) acc ^= fold(__ldcs(in + i));
    for (int off = 16; off > 0; off >>= 1) acc ^= __shfl_xor_sync(0xffffffffu, acc, off);
    if ((threadIdx.x & 31) == 0 && acc != 0) atomicXor(out, acc);   // XOR commutes: the result does not depend on the order
}

}  // namespace

extern "C" vx_status vx_checksum_u32(vx_context* ctx, const void* device_ptr, size_t bytes, uint32_t* device_out) {
    VX_REQUIRE(ctx && device_out && (device_ptr || bytes == 0), VX_ERR_INVALID_ARGUMENT, "vx_checksum_u32: null argument");
    VX_REQUIRE(bytes % 16 == 0 && (reinterpret_cast<uintptr_t>(device_ptr) & 15u) == 0, VX_ERR_INVALID_ARGUMENT,
               "vx_checksum_u32 takes 16-byte aligned buffers of whole 16-byte groups (%zu bytes given)", bytes);
    vx::DeviceGuard guard(ctx->device);
    VX_CUDA(cudaMemsetAsync(device_out, 0, 4, ctx->stream));
    const size_t n16 = bytes / 16;
    if (n16 == 0) return VX_OK;
    const unsigned blocks = (unsigned)std::min<size_t>((n16 + kThreads - 1) / kThreads, (size_t)ctx->sm_count * 4);
    checksum_kernel<<<blocks, kThreads, 0, ctx->stream>>>(static_cast<const uint4*>(device_ptr), n16, device_out);
    VX_CUDA(cudaGetLastError());
    ctx->launches++;
    return VX_OK;
}

extern "C" vx_status vx_qweights_checksum(vx_context* ctx, const vx_qweights* w, uint32_t* device_out) {
    VX_REQUIRE(ctx && w && device_out, VX_ERR_INVALID_ARGUMENT, "vx_qweights_checksum: null argument");
    VX_REQUIRE(w->device == ctx->device, VX_ERR_INVALID_ARGUMENT, "weights live on device %d, context on %d", w->device,
               ctx->device);
    return vx_checksum_u32(ctx, w->d_base, w->device_bytes, device_out);
}
