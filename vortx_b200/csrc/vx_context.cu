// Context, stream-ordered memory and error plumbing of libvortx_b200.
#include <cstring>
#include <new>

#include "vx_internal.h"

namespace vx {

static thread_local std::string g_last_error;

vx_status fail(vx_status code, const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

void clear_error() { g_last_error.clear(); }

int64_t option(const vx_context* ctx, const char* key, int64_t fallback) {
    auto it = ctx->options.find(key);
    return it == ctx->options.end() ? fallback : it->second;
}

cudaError_t device_malloc(vx_context* ctx, void** ptr, size_t bytes) {
    auto it = ctx->options.find("debug.fail_alloc_after");
    if (it != ctx->options.end() && it->second > 0 && --it->second == 0) {
        *ptr = nullptr;
        return cudaErrorMemoryAllocation;
    }
    return cudaMalloc(ptr, bytes);
}

static const char* const kKnownOptions[] = {
    "gemv.variant",       // 2 (default) = TMA streaming kernel; 0 / 1 = register-staged kernels
    "gemv.stages",        // ring depth of the streaming kernel (0 = as many as fit)
    "gemv.tile_rows",     // rows per TMA tile of the streaming kernel: 8 (default) or 4
    "gemv.pdl",           // 1 (default): launch the streaming kernel with programmatic dependent launch
    "gemv.rows_per_warp", // rows a warp carries at once
    "gemv.block_threads", // CTA size of the GEMV kernels
    "gemv.ctas_per_sm",   // persistent grid = SMs x this
    "gemv.batch_mma",     // batches of vectors on the tensor cores: -1 (default) for 2 and more vectors, 0 never, 1 also for one vector
    "debug.timeline_ptr", // timeline build only (-DVX_TIMELINE): device buffer [blocks][entries][8] u64 for the list kernel's stamps
    "gemv.mma_units_per_cta",  // tensor-core batch GEMV: most 16-row tiles a launch gives one thread block (default 14)
    "gemv.mma_nbw",       // tensor-core batch GEMV: most 32-column blocks per warp and column tile (8, 4, 2 or 1; 0 or less = default: 8, 4 for Q8_0 with three and more vectors)
    "gemv.mma_max_stages",  // tensor-core batch GEMV: cap on the depth of the weight ring (default 8)
    "gemv.block_wait",    // flagged x in a list: 1 one warp waits for the block, 0 every thread for its own chunk, -1 (default) by tiles per block
    "gemm.simt.force_generic",  // 1: always take the generic-stride SIMT kernel
    "gemm.tf32.stages",   // TMA pipeline depth
    "gemm.tf32.raster",   // tile rasterisation group height
    "gemm.tf32.tma_store",  // 1 (default): the epilogue hands C blocks to tiled TMA stores; 0: plain stores
    "gemm.tf32.round_nearest",  // 1 (default): TMA rounds A and B to TF32 to nearest on load; 0: the tensor core truncates
    "gemm.tf32.tile_m",   // 128 or 256 forces the tile height of the TF32 kernel (0 = by problem size)
    "elementwise.fast",   // 1 (default): op_assign / contiguous / repeat take their row and tile forms where the layout allows; 0: the general kernels
    "reduce.blocks_per_sm",  // WIDE reductions: thread blocks per SM (1..8, default 8)
    "elementwise.flat",   // 1 (default): dense operands of op_assign / contiguous take the one-dimensional form
    "bounds_check",       // 1 (default): refuse layouts that reach beyond the stated capacity
    "wait_cycles",        // budget, in SM clocks, of the device-side waits on exchange vectors and peer barriers (0 = about 0.2 s)
    "debug.fail_alloc_after",  // n > 0: the n-th device allocation from now fails as if the device were full (tests)
};

static bool known_option(const char* key) {
    for (const char* k : kKnownOptions)
        if (std::strcmp(k, key) == 0) return true;
    return false;
}

}  // namespace vx

using vx::fail;

extern "C" {

const char* vx_last_error(void) { return vx::g_last_error.c_str(); }
const char* vx_version(void) { return "vortx_b200 0.1 (sm_100a)"; }

static vx_status create_context(int32_t device, void* stream, bool adopt, vx_context** out) {
    VX_REQUIRE(out, VX_ERR_INVALID_ARGUMENT, "vx_context_create: out is null");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        (void)cudaGetLastError();
        return fail(VX_ERR_NO_DEVICE, "no CUDA device available: %s",
                    e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    }
    VX_REQUIRE(device >= 0 && device < count, VX_ERR_INVALID_ARGUMENT,
               "device ordinal %d out of range (0..%d)", device, count - 1);
    vx::DeviceGuard guard(device);
    cudaDeviceProp prop;
    VX_CUDA(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10) {
        return fail(VX_ERR_NO_DEVICE,
                    "device %d is compute capability %d.%d; this library holds sm_100a code only",
                    device, prop.major, prop.minor);
    }
    vx_context* ctx = new (std::nothrow) vx_context();
    VX_REQUIRE(ctx, VX_ERR_OUT_OF_MEMORY, "host allocation failed");
    ctx->device = device;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->cc_major = prop.major;
    ctx->cc_minor = prop.minor;
    ctx->l2_bytes = (size_t)prop.l2CacheSize;
    if (adopt) {
        ctx->stream = (cudaStream_t)stream;
        ctx->owns_stream = false;
    } else {
        cudaError_t se = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
        if (se != cudaSuccess) {
            delete ctx;
            return fail(VX_ERR_CUDA, "cudaStreamCreate failed: %s", cudaGetErrorString(se));
        }
        ctx->owns_stream = true;
    }
    // The status word lives in mapped host memory: kernels write it only when a bounded wait
    // gives up, and the host reads it after a stream synchronisation without any copy.
    cudaError_t a1 = cudaHostAlloc(&ctx->h_status, sizeof(vx::DeviceStatus), cudaHostAllocMapped);
    cudaError_t a2 = a1 == cudaSuccess ? cudaHostGetDevicePointer(&ctx->d_status, ctx->h_status, 0) : a1;
    if (a1 != cudaSuccess || a2 != cudaSuccess) {
        if (ctx->h_status) cudaFreeHost(ctx->h_status);
        if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
        delete ctx;
        (void)cudaGetLastError();
        return fail(VX_ERR_OUT_OF_MEMORY, "could not allocate the context status word");
    }
    std::memset(ctx->h_status, 0, sizeof(vx::DeviceStatus));
    ctx->options["bounds_check"] = 1;
    *out = ctx;
    return VX_OK;
}

vx_status vx_context_create(int32_t device, vx_context** out) {
    return create_context(device, nullptr, false, out);
}

vx_status vx_context_create_on_stream(int32_t device, void* cuda_stream, vx_context** out) {
    return create_context(device, cuda_stream, true, out);
}

vx_status vx_context_destroy(vx_context* ctx) {
    if (!ctx) return VX_OK;
    vx::DeviceGuard guard(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->reduce_scratch) cudaFree(ctx->reduce_scratch);
    vx::host_streams_free(ctx);
    if (ctx->mma_planes) cudaFree(ctx->mma_planes);
    if (ctx->h_status) cudaFreeHost(ctx->h_status);
    if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
    (void)cudaGetLastError();
    delete ctx;
    return VX_OK;
}

vx_status vx_synchronize(vx_context* ctx) {
    VX_REQUIRE(ctx, VX_ERR_INVALID_ARGUMENT, "vx_synchronize: null context");
    vx::DeviceGuard guard(ctx->device);
    VX_CUDA(cudaStreamSynchronize(ctx->stream));
    if (!ctx->status_dirty) return VX_OK;
    // A kernel with bounded device-side waits ran since the last check: look at its status word.
    ctx->status_dirty = false;
    volatile vx::DeviceStatus* hs = ctx->h_status;
    if (hs->code != 0) {
        const uint32_t code = hs->code, detail = hs->detail;
        hs->code = 0;
        hs->detail = 0;
        return fail(VX_ERR_DEVICE_TIMEOUT,
                    "a bounded device-side wait gave up (stage code %u, block %u); results of the "
                    "affected kernel are invalid",
                    code, detail);
    }
    return VX_OK;
}

vx_status vx_context_device(const vx_context* ctx, int32_t* device) {
    VX_REQUIRE(ctx && device, VX_ERR_INVALID_ARGUMENT, "vx_context_device: null argument");
    *device = ctx->device;
    return VX_OK;
}

vx_status vx_context_stream(const vx_context* ctx, void** cuda_stream) {
    VX_REQUIRE(ctx && cuda_stream, VX_ERR_INVALID_ARGUMENT, "vx_context_stream: null argument");
    *cuda_stream = (void*)ctx->stream;
    return VX_OK;
}

vx_status vx_context_launch_count(const vx_context* ctx, uint64_t* count) {
    VX_REQUIRE(ctx && count, VX_ERR_INVALID_ARGUMENT, "vx_context_launch_count: null argument");
    *count = ctx->launches;
    return VX_OK;
}

vx_status vx_alloc(vx_context* ctx, size_t bytes, void** device_ptr) {
    VX_REQUIRE(ctx && device_ptr, VX_ERR_INVALID_ARGUMENT, "vx_alloc: null argument");
    *device_ptr = nullptr;
    vx::DeviceGuard guard(ctx->device);
    // A zero-length tensor (Tensor::with_capacity(0), an emptied vector) still needs a handle.
    VX_CUDA(vx::device_malloc(ctx, device_ptr, bytes ? bytes : 16));
    return VX_OK;
}

vx_status vx_free(vx_context* ctx, void* device_ptr) {
    VX_REQUIRE(ctx, VX_ERR_INVALID_ARGUMENT, "vx_free: null context");
    if (!device_ptr) return VX_OK;
    vx::DeviceGuard guard(ctx->device);
    // Work queued on the stream may still use the buffer.
    VX_CUDA(cudaStreamSynchronize(ctx->stream));
    VX_CUDA(cudaFree(device_ptr));
    return VX_OK;
}

vx_status vx_upload(vx_context* ctx, void* dst, const void* src, size_t bytes) {
    VX_REQUIRE(ctx, VX_ERR_INVALID_ARGUMENT, "vx_upload: null context");
    if (bytes == 0) return VX_OK;
    VX_REQUIRE(dst && src, VX_ERR_INVALID_ARGUMENT, "vx_upload: null pointer");
    vx::DeviceGuard guard(ctx->device);
    VX_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return VX_OK;
}

vx_status vx_download(vx_context* ctx, void* dst, const void* src, size_t bytes) {
    VX_REQUIRE(ctx, VX_ERR_INVALID_ARGUMENT, "vx_download: null context");
    if (bytes != 0) {
        VX_REQUIRE(dst && src, VX_ERR_INVALID_ARGUMENT, "vx_download: null pointer");
        vx::DeviceGuard guard(ctx->device);
        VX_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    }
    return vx_synchronize(ctx);
}

vx_status vx_download_2d(vx_context* ctx, void* dst, size_t dst_pitch, const void* src, size_t src_pitch,
                         size_t width_bytes, size_t rows) {
    VX_REQUIRE(ctx, VX_ERR_INVALID_ARGUMENT, "vx_download_2d: null context");
    if (width_bytes != 0 && rows != 0) {
        VX_REQUIRE(dst && src, VX_ERR_INVALID_ARGUMENT, "vx_download_2d: null pointer");
        VX_REQUIRE(dst_pitch >= width_bytes && src_pitch >= width_bytes, VX_ERR_INVALID_ARGUMENT,
                   "vx_download_2d: pitches (%zu, %zu) shorter than a row of %zu bytes", dst_pitch, src_pitch, width_bytes);
        vx::DeviceGuard guard(ctx->device);
        VX_CUDA(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyDeviceToHost, ctx->stream));
    }
    return vx_synchronize(ctx);
}

vx_status vx_copy(vx_context* ctx, void* dst, const void* src, size_t bytes) {
    VX_REQUIRE(ctx, VX_ERR_INVALID_ARGUMENT, "vx_copy: null context");
    if (bytes == 0) return VX_OK;
    VX_REQUIRE(dst && src, VX_ERR_INVALID_ARGUMENT, "vx_copy: null pointer");
    vx::DeviceGuard guard(ctx->device);
    VX_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, ctx->stream));
    return VX_OK;
}

vx_status vx_memset(vx_context* ctx, void* dst, int value, size_t bytes) {
    VX_REQUIRE(ctx, VX_ERR_INVALID_ARGUMENT, "vx_memset: null context");
    if (bytes == 0) return VX_OK;
    VX_REQUIRE(dst, VX_ERR_INVALID_ARGUMENT, "vx_memset: null pointer");
    vx::DeviceGuard guard(ctx->device);
    VX_CUDA(cudaMemsetAsync(dst, value, bytes, ctx->stream));
    return VX_OK;
}

vx_status vx_host_alloc(size_t bytes, void** host_ptr) {
    VX_REQUIRE(host_ptr, VX_ERR_INVALID_ARGUMENT, "vx_host_alloc: null argument");
    *host_ptr = nullptr;
    VX_CUDA(cudaMallocHost(host_ptr, bytes ? bytes : 16));
    return VX_OK;
}

vx_status vx_host_free(void* host_ptr) {
    if (!host_ptr) return VX_OK;
    VX_CUDA(cudaFreeHost(host_ptr));
    return VX_OK;
}

vx_status vx_set_option(vx_context* ctx, const char* key, int64_t value) {
    VX_REQUIRE(ctx && key, VX_ERR_INVALID_ARGUMENT, "vx_set_option: null argument");
    VX_REQUIRE(vx::known_option(key), VX_ERR_INVALID_ARGUMENT, "unknown option '%s'", key);
    ctx->options[key] = value;
    return VX_OK;
}

vx_status vx_get_option(const vx_context* ctx, const char* key, int64_t* value) {
    VX_REQUIRE(ctx && key && value, VX_ERR_INVALID_ARGUMENT, "vx_get_option: null argument");
    VX_REQUIRE(vx::known_option(key), VX_ERR_INVALID_ARGUMENT, "unknown option '%s'", key);
    *value = vx::option(ctx, key, 0);
    return VX_OK;
}

}  // extern "C"
