// Internal declarations shared by the translation units of libvortx_b200.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <map>
#include <string>

#include "../../include/vortx_b200.h"
#include "../../include/vortx_b200_host.h"

namespace vx {

// Records the message for vx_last_error() and returns `code`, so call sites can
// `return fail(VX_ERR_..., "...")`.
vx_status fail(vx_status code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));
void clear_error();

#define VX_CUDA(expr)                                                                      \
    do {                                                                                   \
        cudaError_t vx_e_ = (expr);                                                        \
        if (vx_e_ != cudaSuccess) {                                                        \
            (void)cudaGetLastError();                                                      \
            return ::vx::fail(vx_e_ == cudaErrorMemoryAllocation ? VX_ERR_OUT_OF_MEMORY    \
                                                                 : VX_ERR_CUDA,            \
                              "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(vx_e_),   \
                              __FILE__, __LINE__);                                         \
        }                                                                                  \
    } while (0)

#define VX_REQUIRE(cond, code, ...)                      \
    do {                                                 \
        if (!(cond)) return ::vx::fail(code, __VA_ARGS__); \
    } while (0)

// Sets the context's device for the lifetime of the guard and restores the previous one.
struct DeviceGuard {
    int prev = -1;
    bool changed = false;
    explicit DeviceGuard(int device) {
        if (cudaGetDevice(&prev) == cudaSuccess && prev != device) {
            changed = cudaSetDevice(device) == cudaSuccess;
        }
    }
    ~DeviceGuard() {
        if (changed) cudaSetDevice(prev);
    }
};

// Status word the bounded device-side waits report into (tcgen05 GEMM pipeline).
struct DeviceStatus {
    uint32_t code;    // 0 ok; otherwise which wait gave up
    uint32_t detail;  // block index that reported
};

}  // namespace vx

struct vx_context {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int sm_count = 0;
    int cc_major = 0, cc_minor = 0;
    size_t l2_bytes = 0;
    uint64_t launches = 0;
    int last_gemm_kernel = 0;
    vx::DeviceStatus* d_status = nullptr;  // device
    vx::DeviceStatus* h_status = nullptr;  // pinned host mirror
    bool status_dirty = false;             // a kernel that may write d_status ran since the last check
    bool weights_fresh = false;            // a kernel of this stream has written quantised weights since the last GEMV launch
    void* reduce_scratch = nullptr;        // per-block partials of the wide reduction (device)
    // scratch of the tensor-core batch GEMV (device, grown on demand): x as fixed-point planes
    void* mma_planes = nullptr;
    size_t mma_planes_bytes = 0;
    void* host_streams = nullptr;          // vx::HostStreams of vx_gemv_batch_run_host, made on first use
    std::map<std::string, int64_t> options;
};

struct vx_qweights {
    vx_qtype type;
    size_t rows = 0, cols = 0;
    size_t blocks_per_row = 0;
    size_t quant_row_bytes = 0;   // bytes of quants per row (16 B per Q4_0 block, 32 B per Q8_0 block)
    uint8_t* d_base = nullptr;    // one allocation: quants plane, then scales plane
    uint8_t* d_quants = nullptr;  // rows * quant_row_bytes
    uint16_t* d_scales = nullptr; // rows * blocks_per_row f16
    size_t device_bytes = 0;
    int device = 0;
};

namespace vx {

int64_t option(const vx_context* ctx, const char* key, int64_t fallback);

// Frees the copy streams and events of vx_gemv_batch_run_host (vx_host_stages.cu), if any were made.
void host_streams_free(vx_context* ctx);

// Budget of the device-side waits on exchange vectors and peer barriers, in SM clocks: the option
// "wait_cycles", or about 0.2 s.
inline long long wait_cycles(const vx_context* ctx) {
    const int64_t v = option(ctx, "wait_cycles", 0);
    return v > 0 ? (long long)v : 400ll * 1000 * 1000;
}

// Every device allocation of the library goes through here (cudaMalloc on the current device).  The option
// "debug.fail_alloc_after" = n makes the n-th call from now return cudaErrorMemoryAllocation without
// allocating, so that the out-of-memory paths can be tested without filling a device.
cudaError_t device_malloc(vx_context* ctx, void** ptr, size_t bytes);

// SIMT kernels (vx_gemm_simt.cu)
vx_status launch_gemm_naive(vx_context* ctx, float* out, const float* lhs, const float* rhs,
                            const vx_shapes3& s);
// Returns the kernel id it used in *kernel (2 vector, 4 generic).
vx_status launch_gemm_simt_exact(vx_context* ctx, float* out, const float* lhs, const float* rhs,
                                 const vx_shapes3& s, int* kernel);

// tcgen05 kernel (vx_gemm_tf32.cu).  *eligible = false when the operands cannot be
// described to TMA (strides, alignment, batch); nothing is launched then.
// out_peer / n_peer: further full-width C buffers (peer GPUs') that receive every tile at the same
// position, or null / 0; with peers the launch also requires one matrix, n % 32 == 0 and 16-byte
// aligned rows.
constexpr int kMaxPeers = 7;
vx_status launch_gemm_tf32(vx_context* ctx, float* out, const float* lhs, const float* rhs,
                           const vx_shapes3& s, bool* eligible, float* const* out_peer = nullptr,
                           uint32_t n_peer = 0);

// Streaming GEMV (vx_gemv_stream.cu), one vector.  *eligible = false when the row shape does
// not fit its shared-memory ring or register-resident x; nothing is launched then.
// y_peer / n_peer: further buffers that receive every row as well (peer GPUs' y), or null / 0.
// Arrival flags of the cross-GPU barrier: flags[r] is rank r's array of `world` counters (its
// own memory for r == this rank, a mapped peer pointer otherwise).
struct PeerFlags {
    uint32_t* flags[kMaxPeers + 1];
};
// Fused exchange of the row-sharded GEMV through exchange vectors (256-byte header, then one
// {f32, generation} pair per element; see StreamParams in vx_gemv_stream.cu).  x_vec: flagged x to
// read instead of the plain x, or null.  y_vec: this rank's full-length vector that receives the
// slab at elements y_row0 + r * y_stride, with peer_y_vec[d] the same vector of each peer; or null.
constexpr size_t kExchangeHeader = 256;
struct Exchange {
    const void* x_vec;
    void* y_vec;
    void* const* peer_y_vec;
    uint32_t n_peers;
    size_t y_row0;
    size_t y_stride;  // row r of the slab goes to element y_row0 + r * y_stride
};
vx_status launch_gemv_stream(vx_context* ctx, const vx_qweights* w, size_t row0, uint32_t nrows,
                             const float* x, float* y, float* const* y_peer, uint32_t n_peer,
                             const Exchange* xch, bool* eligible, uint32_t batch = 1, size_t x_stride = 0,
                             size_t y_stride = 0);

// Tensor-core batch GEMV (vx_gemv_mma.cu): up to 8 vectors per pass over the weights of `n_mats` slabs (rows
// [row0[i], row0[i] + nrows[i]) of ws[i] into ys[i]; one type, one column count) that share the vectors.
// *eligible = false (nothing launched) when the shape does not fit it.
vx_status launch_gemv_mma(vx_context* ctx, const vx_qweights* const* ws, const size_t* row0, const uint32_t* nrows,
                          float* const* ys, size_t n_mats, const float* x, size_t x_stride, size_t y_stride,
                          uint32_t batch, bool* eligible);

}  // namespace vx
