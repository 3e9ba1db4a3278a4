// Multi-GPU plumbing for the row-sharded GEMV without a collective: CUDA IPC mapping of peer
// buffers (one process per GPU), the GEMV whose epilogue also stores every row into the peers'
// copies of y, and a small cross-GPU arrival barrier.
//
// vortx has no multi-device notion beyond a device ordinal (src/linalg/gemm.rs:353); nothing here
// has a reference counterpart.  Design rules: a GPU only ever STORES to a peer (plain st.global
// through an NVLink-mapped pointer) and only loads from its own memory; no TMA touches peer
// memory; every device-side wait is bounded and reports through the context's status word.
#include <algorithm>
#include <cstring>

#include "vx_internal.h"

namespace {

using vx::fail;

// Each rank owns a sync block of 64 u32 in its own memory: entries [40, 40 + world) are the
// barrier's arrival counters and entry 32 is the rank's own count of barriers executed.  A barrier takes the next epoch e from
// that count (so a replayed CUDA graph keeps advancing, and all ranks, which run the same
// sequence of barriers, agree on e), stores e into entry [rank] of EVERY rank's array (its own
// included), then waits until all world entries of its own array have reached e.  Stores made
// before the announcement (the GEMV's rows, written by an earlier kernel of the same stream) are
// ordered before it by the system-scope fence.
constexpr uint32_t kEpochSlot = 32;
constexpr uint32_t kArrivalBase = 40;

__global__ void peer_barrier_kernel(vx::PeerFlags peers, uint32_t world, uint32_t rank, vx::DeviceStatus* status,
                                    long long wait_cycles) {
    const uint32_t t = threadIdx.x;
    // Let a dependent-launch GEMV behind this kernel become resident and prefetch its weights
    // now; it reads x and writes y only after this kernel has completed.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    uint32_t epoch = 0;
    if (t == 0) {
        epoch = peers.flags[rank][kEpochSlot] + 1;
        peers.flags[rank][kEpochSlot] = epoch;
    }
    epoch = __shfl_sync(0xffffffffu, epoch, 0);
    if (t < world) {
        __threadfence_system();
        volatile uint32_t* dst = peers.flags[t] + kArrivalBase + rank;  // my entry in rank t's block
        *dst = epoch;
        __threadfence_system();
        // wait for rank t's announcement in my own array (bounded: ~0.2 s of SM clocks)
        volatile uint32_t* mine = peers.flags[rank] + kArrivalBase + t;
        const long long start = clock64();
        bool ok = false;
        while (!ok) {
            for (int i = 0; i < 32 && !ok; ++i) ok = (int32_t)(*mine - epoch) >= 0;
            if (!ok && clock64() - start > wait_cycles) break;
        }
        if (!ok) {
            volatile vx::DeviceStatus* v = status;
            v->detail = t;
            v->code = 31;
            __threadfence_system();
        }
        __threadfence_system();
    }
}

// Exchange vector -> plain f32.  Pairs that do not carry the vector's generation yet are still
// on their way from a peer: re-read them, for at most about 0.2 s of SM clocks.
__global__ void xvec_unpack_kernel(const uint32_t* hdr, const uint64_t* pairs, uint32_t n, float* out,
                                   vx::DeviceStatus* status, long long wait_cycles) {
    const uint32_t gen = *(volatile const uint32_t*)hdr;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const volatile uint64_t* src = pairs + i;
        uint64_t v = *src;
        if ((uint32_t)(v >> 32) != gen) {
            const long long start = clock64();
            while ((uint32_t)((v = *src) >> 32) != gen) {
                if (clock64() - start > wait_cycles) {
                    volatile vx::DeviceStatus* st = status;
                    st->detail = i;
                    st->code = 32;
                    __threadfence_system();
                    break;
                }
            }
        }
        out[i] = __uint_as_float((uint32_t)v);
    }
}

}  // namespace

extern "C" {

vx_status vx_ipc_export(vx_context* ctx, const void* device_ptr, void* handle64) {
    VX_REQUIRE(ctx && device_ptr && handle64, VX_ERR_INVALID_ARGUMENT, "vx_ipc_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    vx::DeviceGuard guard(ctx->device);
    cudaIpcMemHandle_t h;
    VX_CUDA(cudaIpcGetMemHandle(&h, const_cast<void*>(device_ptr)));
    memcpy(handle64, &h, 64);
    return VX_OK;
}

vx_status vx_ipc_import(vx_context* ctx, const void* handle64, void** device_ptr) {
    VX_REQUIRE(ctx && handle64 && device_ptr, VX_ERR_INVALID_ARGUMENT, "vx_ipc_import: null argument");
    *device_ptr = nullptr;
    vx::DeviceGuard guard(ctx->device);
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    VX_CUDA(cudaIpcOpenMemHandle(device_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return VX_OK;
}

vx_status vx_ipc_release(vx_context* ctx, void* device_ptr) {
    VX_REQUIRE(ctx, VX_ERR_INVALID_ARGUMENT, "vx_ipc_release: null context");
    if (!device_ptr) return VX_OK;
    vx::DeviceGuard guard(ctx->device);
    VX_CUDA(cudaStreamSynchronize(ctx->stream));
    VX_CUDA(cudaIpcCloseMemHandle(device_ptr));
    return VX_OK;
}

static vx_status gemv_scatter_impl(const char* who, vx_context* ctx, const vx_qweights* w, size_t row0, size_t nrows,
                                   const float* x, float* y, float* const* peer_y, size_t n_peers,
                                   const vx::Exchange* xch) {
    VX_REQUIRE(ctx && w, VX_ERR_INVALID_ARGUMENT, "%s: null context or weights", who);
    VX_REQUIRE(w->device == ctx->device, VX_ERR_INVALID_ARGUMENT, "weights live on device %d, context on %d",
               w->device, ctx->device);
    VX_REQUIRE(row0 <= w->rows && nrows <= w->rows - row0, VX_ERR_OUT_OF_BOUNDS,
               "rows [%zu, %zu) outside a matrix of %zu rows", row0, row0 + nrows, w->rows);
    VX_REQUIRE(n_peers <= (size_t)vx::kMaxPeers, VX_ERR_INVALID_ARGUMENT, "at most %d peers", vx::kMaxPeers);
    // With a fused exchange every rank must launch, or its vector's generation falls behind the others'.
    VX_REQUIRE(nrows > 0 || !xch, VX_ERR_INVALID_ARGUMENT, "%s: a rank without rows cannot take part", who);
    if (nrows == 0) return VX_OK;
    VX_REQUIRE(x && (y || xch) && (peer_y || n_peers == 0), VX_ERR_INVALID_ARGUMENT, "%s: null vector", who);
    for (size_t i = 0; i < n_peers; ++i)
        VX_REQUIRE(peer_y[i], VX_ERR_INVALID_ARGUMENT, "peer buffer %zu is null", i);
    vx::DeviceGuard guard(ctx->device);
    bool eligible = false;
    vx_status st = vx::launch_gemv_stream(ctx, w, row0, (uint32_t)nrows, x, y, peer_y, (uint32_t)n_peers, xch,
                                          &eligible);
    if (st != VX_OK) return st;
    VX_REQUIRE(eligible, VX_ERR_UNSUPPORTED, "rows of %zu columns do not fit the streaming kernel", w->cols);
    return VX_OK;
}

vx_status vx_gemv_q_rows_scatter(vx_context* ctx, const vx_qweights* w, size_t row0, size_t nrows, const float* x,
                                 float* y, float* const* peer_y, size_t n_peers) {
    return gemv_scatter_impl("vx_gemv_q_rows_scatter", ctx, w, row0, nrows, x, y, peer_y, n_peers, nullptr);
}

size_t vx_xvec_bytes(size_t n) { return vx::kExchangeHeader + 8 * n; }

vx_status vx_gemv_q_rows_exchange(vx_context* ctx, const vx_qweights* w, size_t row0, size_t nrows, const void* x_xvec,
                                  const float* x, float* y, void* y_xvec, void* const* peer_y_xvec, size_t n_peers,
                                  size_t y_row0, size_t y_stride) {
    VX_REQUIRE(y_xvec && (peer_y_xvec || n_peers == 0), VX_ERR_INVALID_ARGUMENT,
               "vx_gemv_q_rows_exchange: null exchange vector");
    VX_REQUIRE(n_peers <= (size_t)vx::kMaxPeers, VX_ERR_INVALID_ARGUMENT, "at most %d peers", vx::kMaxPeers);
    VX_REQUIRE(x_xvec || x, VX_ERR_INVALID_ARGUMENT, "vx_gemv_q_rows_exchange: no x");
    VX_REQUIRE(y_stride >= 1 && y_stride <= 0xFFFFu, VX_ERR_INVALID_ARGUMENT, "element stride %zu", y_stride);
    VX_REQUIRE((reinterpret_cast<uintptr_t>(y_xvec) & 15u) == 0 && (reinterpret_cast<uintptr_t>(x_xvec) & 15u) == 0,
               VX_ERR_INVALID_ARGUMENT, "exchange vectors are 16-byte aligned");
    for (size_t i = 0; i < n_peers; ++i)
        VX_REQUIRE(peer_y_xvec[i] && (reinterpret_cast<uintptr_t>(peer_y_xvec[i]) & 15u) == 0, VX_ERR_INVALID_ARGUMENT,
                   "exchange vector of peer %zu is null or misaligned", i);
    vx::Exchange xch{x_xvec, y_xvec, peer_y_xvec, (uint32_t)n_peers, y_row0, y_stride};
    // No plain peer copies here: the exchange vectors carry the rows.
    return gemv_scatter_impl("vx_gemv_q_rows_exchange", ctx, w, row0, nrows, x_xvec ? reinterpret_cast<const float*>(x_xvec) : x,
                             y, nullptr, 0, &xch);
}

vx_status vx_xvec_unpack(vx_context* ctx, const void* xvec, size_t n, float* out) {
    VX_REQUIRE(ctx && xvec && (out || n == 0), VX_ERR_INVALID_ARGUMENT, "vx_xvec_unpack: null argument");
    VX_REQUIRE(n <= 0xFFFFFFFFull, VX_ERR_INVALID_ARGUMENT, "vx_xvec_unpack: %zu elements", n);
    if (n == 0) return VX_OK;
    vx::DeviceGuard guard(ctx->device);
    const uint32_t threads = 256;
    const uint32_t blocks = (uint32_t)std::min<size_t>((n + threads - 1) / threads, (size_t)ctx->sm_count * 4);
    xvec_unpack_kernel<<<blocks, threads, 0, ctx->stream>>>(
        static_cast<const uint32_t*>(xvec),
        reinterpret_cast<const uint64_t*>(static_cast<const uint8_t*>(xvec) + vx::kExchangeHeader), (uint32_t)n, out,
        ctx->d_status, vx::wait_cycles(ctx));
    VX_CUDA(cudaGetLastError());
    ctx->launches++;
    ctx->status_dirty = true;
    return VX_OK;
}

vx_status vx_gemm_tf32_scatter(vx_context* ctx, float* out, const float* lhs, const float* rhs,
                               const vx_shapes3* shapes, float* const* peer_out, size_t n_peers) {
    VX_REQUIRE(ctx && out && lhs && rhs && shapes, VX_ERR_INVALID_ARGUMENT, "vx_gemm_tf32_scatter: null argument");
    VX_REQUIRE(n_peers <= (size_t)vx::kMaxPeers && (peer_out || n_peers == 0), VX_ERR_INVALID_ARGUMENT,
               "at most %d peers", vx::kMaxPeers);
    for (size_t i = 0; i < n_peers; ++i)
        VX_REQUIRE(peer_out[i], VX_ERR_INVALID_ARGUMENT, "peer buffer %zu is null", i);
    const vx_shapes3& s = *shapes;
    VX_REQUIRE(s.out.h == s.lhs.h && s.out.w == s.rhs.w && s.lhs.w == s.rhs.h, VX_ERR_SHAPE,
               "out %ux%u, lhs %ux%u, rhs %ux%u do not form a product", s.out.h, s.out.w, s.lhs.h, s.lhs.w, s.rhs.h, s.rhs.w);
    vx::DeviceGuard guard(ctx->device);
    bool eligible = false;
    vx_status st = vx::launch_gemm_tf32(ctx, out, lhs, rhs, s, &eligible, peer_out, (uint32_t)n_peers);
    if (st != VX_OK) return st;
    VX_REQUIRE(eligible, VX_ERR_UNSUPPORTED,
               "the panel must be one matrix with unit column strides and 16-byte aligned bases and row pitches");
    ctx->last_gemm_kernel = 3;
    return VX_OK;
}

vx_status vx_peer_barrier(vx_context* ctx, uint32_t* const* flags, size_t world, size_t rank) {
    VX_REQUIRE(ctx && flags, VX_ERR_INVALID_ARGUMENT, "vx_peer_barrier: null argument");
    VX_REQUIRE(world >= 1 && world <= (size_t)vx::kMaxPeers + 1 && rank < world, VX_ERR_INVALID_ARGUMENT,
               "world %zu / rank %zu out of range", world, rank);
    vx::PeerFlags p;
    for (size_t i = 0; i < (size_t)vx::kMaxPeers + 1; ++i) {
        p.flags[i] = i < world ? flags[i] : nullptr;
        VX_REQUIRE(i >= world || flags[i], VX_ERR_INVALID_ARGUMENT, "flag array of rank %zu is null", i);
    }
    vx::DeviceGuard guard(ctx->device);
    peer_barrier_kernel<<<1, 32, 0, ctx->stream>>>(p, (uint32_t)world, (uint32_t)rank, ctx->d_status, vx::wait_cycles(ctx));
    VX_CUDA(cudaGetLastError());
    ctx->launches++;
    ctx->status_dirty = true;
    return VX_OK;
}

}  // extern "C"
