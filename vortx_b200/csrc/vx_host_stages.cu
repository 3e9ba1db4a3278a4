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

// A step recorded once as a CUDA graph (vx_host_pipeline): with eight GPUs a step's kernels take 0.1 ms, less
// than the dozen runtime calls that issue its copies, events and launches one by one.
struct vx_host_pipeline {
    vx_context* ctx = nullptr;
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
};

namespace {

vx_status check_stages(const vx_host_stage* stages, size_t n_stages) {
    using vx::fail;
    VX_REQUIRE(stages, VX_ERR_INVALID_ARGUMENT, "host stages: null stages");
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
    return VX_OK;
}

// Gives every stage's copies and kernels to the three streams.  The copy streams fork from the context's stream
// at `start` and, with `join`, are waited for by it at the end (what a stream capture needs; the immediate form
// synchronises the streams from the host instead).
vx_status issue_stages(vx_context* ctx, vx::HostStreams* h, const vx_host_stage* stages, size_t n_stages, bool join) {
    using vx::fail;
    cudaEvent_t* up_done = h->events.data();
    cudaEvent_t* run_done = h->events.data() + n_stages;
    cudaEvent_t start = h->events[2 * n_stages];
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
    vx_status st = VX_OK;
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
    if (join) {
        cudaEvent_t up_end = h->events[2 * n_stages + 1], down_end = h->events[2 * n_stages + 2];
        VX_CUDA(cudaEventRecord(up_end, h->up));
        VX_CUDA(cudaEventRecord(down_end, h->down));
        VX_CUDA(cudaStreamWaitEvent(ctx->stream, up_end, 0));
        VX_CUDA(cudaStreamWaitEvent(ctx->stream, down_end, 0));
    }
    return st;
}

}  // namespace

extern "C" {

vx_status vx_gemv_batch_run_host(vx_context* ctx, const vx_host_stage* stages, size_t n_stages) {
    using vx::fail;
    VX_REQUIRE(ctx, VX_ERR_INVALID_ARGUMENT, "vx_gemv_batch_run_host: null context");
    if (n_stages == 0) return VX_OK;
    vx_status st = check_stages(stages, n_stages);
    if (st != VX_OK) return st;
    vx::DeviceGuard guard(ctx->device);
    vx::HostStreams* h = nullptr;
    st = vx::host_streams(ctx, 2 * n_stages + 3, &h);
    if (st != VX_OK) return st;
    st = issue_stages(ctx, h, stages, n_stages, false);
    // everything of this call is over before it returns, also after an error part-way
    const cudaError_t e1 = cudaStreamSynchronize(h->up);
    const cudaError_t e2 = cudaStreamSynchronize(h->down);
    const vx_status sync = vx_synchronize(ctx);
    if (st != VX_OK) return st;
    VX_CUDA(e1);
    VX_CUDA(e2);
    return sync;
}

vx_status vx_host_pipeline_create(vx_context* ctx, const vx_host_stage* stages, size_t n_stages, vx_host_pipeline** out) {
    using vx::fail;
    VX_REQUIRE(ctx && out, VX_ERR_INVALID_ARGUMENT, "vx_host_pipeline_create: null argument");
    *out = nullptr;
    VX_REQUIRE(n_stages >= 1, VX_ERR_INVALID_ARGUMENT, "vx_host_pipeline_create: no stages");
    vx_status st = check_stages(stages, n_stages);
    if (st != VX_OK) return st;
    vx::DeviceGuard guard(ctx->device);
    // a copy from pageable memory cannot be recorded
    for (size_t i = 0; i < n_stages; ++i) {
        const void* host[2] = {stages[i].up_bytes ? stages[i].up_host : nullptr,
                               stages[i].down_width_bytes && stages[i].down_rows ? stages[i].down_host : nullptr};
        for (const void* p : host) {
            if (!p) continue;
            cudaPointerAttributes attr{};
            const cudaError_t e = cudaPointerGetAttributes(&attr, p);
            (void)cudaGetLastError();
            VX_REQUIRE(e == cudaSuccess && attr.type == cudaMemoryTypeHost, VX_ERR_INVALID_ARGUMENT,
                       "stage %zu: the host buffers of a recorded step must be page-locked (vx_host_alloc)", i);
        }
    }
    vx::HostStreams* h = nullptr;
    st = vx::host_streams(ctx, 2 * n_stages + 3, &h);
    if (st != VX_OK) return st;
    VX_CUDA(cudaStreamSynchronize(ctx->stream));
    // one plain run first: every kernel of the lists sets its attributes and loads outside the recording
    st = vx_gemv_batch_run_host(ctx, stages, n_stages);
    if (st != VX_OK) return st;
    auto* p = new vx_host_pipeline();
    p->ctx = ctx;
    cudaError_t e = cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal);
    if (e == cudaSuccess) {
        st = issue_stages(ctx, h, stages, n_stages, true);
        e = cudaStreamEndCapture(ctx->stream, &p->graph);      // also ends a recording that an error left open
        if (st == VX_OK && e == cudaSuccess) e = cudaGraphInstantiate(&p->exec, p->graph, 0);
    }
    if (st != VX_OK || e != cudaSuccess) {
        (void)cudaGetLastError();
        if (p->exec) cudaGraphExecDestroy(p->exec);
        if (p->graph) cudaGraphDestroy(p->graph);
        delete p;
        if (st != VX_OK) return st;
        return fail(VX_ERR_CUDA, "vx_host_pipeline_create: recording the step failed: %s", cudaGetErrorString(e));
    }
    *out = p;
    return VX_OK;
}

vx_status vx_host_pipeline_run(vx_host_pipeline* p) {
    using vx::fail;
    VX_REQUIRE(p && p->exec, VX_ERR_INVALID_ARGUMENT, "vx_host_pipeline_run: null pipeline");
    vx::DeviceGuard guard(p->ctx->device);
    VX_CUDA(cudaGraphLaunch(p->exec, p->ctx->stream));
    p->ctx->status_dirty = true;
    return vx_synchronize(p->ctx);
}

vx_status vx_host_pipeline_free(vx_host_pipeline* p) {
    if (!p) return VX_OK;
    vx::DeviceGuard guard(p->ctx->device);
    cudaStreamSynchronize(p->ctx->stream);
    if (p->exec) cudaGraphExecDestroy(p->exec);
    if (p->graph) cudaGraphDestroy(p->graph);
    delete p;
    return VX_OK;
}

}  // extern "C"
