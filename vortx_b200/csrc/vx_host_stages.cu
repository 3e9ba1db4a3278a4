// Lists of products with HOST buffers, copies overlapped with the kernels (vx_gemv_batch_run_host).
//
// A caller whose activations and results live in host memory (the reference's own test builds its tensors
// from host matrices, submits, synchronises and reads the result back with `slow_read_buffer`,
// src/linalg/gemm.rs:378-426) pays, per step, one copy up, the kernels, one copy down, in a row.  Here the step is cut into stages:
// stage i's inputs go up on a copy stream while stage i - 1 runs, and its results come down on a second
// copy stream while stage i + 1 runs; uploads and downloads use different copy engines, so both hide behind
// the kernels.  What stays exposed is the first stage's copy up and the last stage's copy down.
#include <vector>

#include "vx_internal.h"

namespace vx {

struct HostStreams {
    cudaStream_t up = nullptr, down = nullptr;
    std::vector<cudaEvent_t> events;     // grown on demand, reused by every call
};

vx_status host_streams(vx_context* ctx, size_t n_events, HostStreams** out) {
    if (!ctx->host_streams) ctx->host_streams = new HostStreams();
    HostStreams* h = static_cast<HostStreams*>(ctx->host_streams);
    if (!h->up) VX_CUDA(cudaStreamCreateWithFlags(&h->up, cudaStreamNonBlocking));
    if (!h->down) VX_CUDA(cudaStreamCreateWithFlags(&h->down, cudaStreamNonBlocking));
    while (h->events.size() < n_events) {
        cudaEvent_t e;
        VX_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        h->events.push_back(e);
    }
    *out = h;
    return VX_OK;
}

void host_streams_free(vx_context* ctx) {
    HostStreams* h = static_cast<HostStreams*>(ctx->host_streams);
    if (!h) return;
    for (cudaEvent_t e : h->events) cudaEventDestroy(e);
    if (h->up) cudaStreamDestroy(h->up);
    if (h->down) cudaStreamDestroy(h->down);
    delete h;
    ctx->host_streams = nullptr;
}

}  // namespace vx

extern "C" {

vx_status vx_gemv_batch_run_host(vx_context* ctx, const vx_host_stage* stages, size_t n_stages) {
    using vx::fail;
    VX_REQUIRE(ctx, VX_ERR_INVALID_ARGUMENT, "vx_gemv_batch_run_host: null context");
    if (n_stages == 0) return VX_OK;
    VX_REQUIRE(stages, VX_ERR_INVALID_ARGUMENT, "vx_gemv_batch_run_host: null stages");
    for (size_t i = 0; i < n_stages; ++i) {
        const vx_host_stage& s = stages[i];
        VX_REQUIRE(s.batch, VX_ERR_INVALID_ARGUMENT, "stage %zu: no list", i);
        VX_REQUIRE(s.up_bytes == 0 || (s.up_device && s.up_host), VX_ERR_INVALID_ARGUMENT, "stage %zu: null upload pointer", i);
        const bool down = s.down_width_bytes != 0 && s.down_rows != 0;
        VX_REQUIRE(!down || (s.down_host && s.down_device), VX_ERR_INVALID_ARGUMENT, "stage %zu: null download pointer", i);
        VX_REQUIRE(!down || (s.down_host_pitch >= s.down_width_bytes && s.down_device_pitch >= s.down_width_bytes),
                   VX_ERR_INVALID_ARGUMENT, "stage %zu: pitches (%zu, %zu) shorter than a row of %zu bytes", i,
                   s.down_host_pitch, s.down_device_pitch, s.down_width_bytes);
        VX_REQUIRE(!s.barrier_flags || (s.world >= 1 && s.rank < s.world), VX_ERR_INVALID_ARGUMENT,
                   "stage %zu: world %zu / rank %zu out of range", i, s.world, s.rank);
    }
    vx::DeviceGuard guard(ctx->device);
    vx::HostStreams* h = nullptr;
    vx_status st = vx::host_streams(ctx, 2 * n_stages + 1, &h);
    if (st != VX_OK) return st;
    cudaEvent_t* up_done = h->events.data();
    cudaEvent_t* run_done = h->events.data() + n_stages;
    cudaEvent_t start = h->events[2 * n_stages];

    // the copy streams start after whatever the context's stream has been given before this call
    VX_CUDA(cudaEventRecord(start, ctx->stream));
    VX_CUDA(cudaStreamWaitEvent(h->up, start, 0));
    VX_CUDA(cudaStreamWaitEvent(h->down, start, 0));
    for (size_t i = 0; i < n_stages; ++i) {
        const vx_host_stage& s = stages[i];
        if (s.up_bytes) {
            VX_CUDA(cudaMemcpyAsync(s.up_device, s.up_host, s.up_bytes, cudaMemcpyHostToDevice, h->up));
            VX_CUDA(cudaEventRecord(up_done[i], h->up));
        }
    }
    for (size_t i = 0; i < n_stages; ++i) {
        const vx_host_stage& s = stages[i];
        if (s.up_bytes) VX_CUDA(cudaStreamWaitEvent(ctx->stream, up_done[i], 0));
        st = vx_gemv_batch_launch(ctx, s.batch);
        if (st == VX_OK && s.barrier_flags) st = vx_peer_barrier(ctx, s.barrier_flags, s.world, s.rank);
        if (st != VX_OK) break;
        if (s.down_width_bytes != 0 && s.down_rows != 0) {
            VX_CUDA(cudaEventRecord(run_done[i], ctx->stream));
            VX_CUDA(cudaStreamWaitEvent(h->down, run_done[i], 0));
            VX_CUDA(cudaMemcpy2DAsync(s.down_host, s.down_host_pitch, s.down_device, s.down_device_pitch, s.down_width_bytes,
                                      s.down_rows, cudaMemcpyDeviceToHost, h->down));
        }
    }
    // everything of this call is over before it returns, also after an error part-way
    const cudaError_t e1 = cudaStreamSynchronize(h->up);
    const cudaError_t e2 = cudaStreamSynchronize(h->down);
    const vx_status sync = vx_synchronize(ctx);
    if (st != VX_OK) return st;
    VX_CUDA(e1);
    VX_CUDA(e2);
    return sync;
}

}  // extern "C"
