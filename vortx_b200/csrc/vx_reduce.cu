// Reductions of a vector to one value: sum, product, min, max for f32 / u32 / i32 and the f32
// squared norm — vortx's Reduce (src/linalg/reduce.rs:79-207) over its thirteen kernels
// (vortx-shaders/src/linalg/reduce.rs:19-367).
//
// As in the reference only the w axis of the shape is walked (reduce.rs:45-51: element i is
// input[shape.it(0, 0, 0, i)]) and the result lands in output[0].
//
// Two kernels:
//   * ORDERED: one block of 128 threads that folds elements t, t+128, ... per thread and then
//     combines the 128 partials with the stride-64..1 tree — the reference kernel's exact order, so
//     f32 sums, products and norms come out bit-identical to it.  Latency-bound for long vectors,
//     like the reference.
//   * WIDE: a grid of blocks, each reducing a contiguous slice to one partial in a scratch array in
//     global memory, and a second one-block kernel that folds the partials in index order.
//     Integer results and f32 min / max are the same values as ORDERED; f32 sum / product / norm
//     differ from it by rounding order only.  Deterministic run to run.
#include <atomic>

#include "vx_internal.h"

namespace {

using vx::fail;

enum Op { SUM = 0, PROD = 1, MIN = 2, MAX = 3, SQNORM = 4 };

template <class T> struct Limits;
// The reference starts its f32 min / max from +-1e18, not the type's limits (reduce.rs:292-295).
template <> struct Limits<float> { __host__ __device__ static float hi() { return 1.0e18f; } __host__ __device__ static float lo() { return -1.0e18f; } };
template <> struct Limits<uint32_t> { __host__ __device__ static uint32_t hi() { return 0xFFFFFFFFu; } __host__ __device__ static uint32_t lo() { return 0u; } };
template <> struct Limits<int32_t> { __host__ __device__ static int32_t hi() { return 2147483647; } __host__ __device__ static int32_t lo() { return -2147483647 - 1; } };

template <class T, int OP> __device__ __forceinline__ T identity() {
    if (OP == SUM || OP == SQNORM) return (T)0;
    if (OP == PROD) return (T)1;
    if (OP == MIN) return Limits<T>::hi();
    return Limits<T>::lo();
}

__device__ __forceinline__ float fold_add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float fold_mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ uint32_t fold_add(uint32_t a, uint32_t b) { return a + b; }
__device__ __forceinline__ uint32_t fold_mul(uint32_t a, uint32_t b) { return a * b; }
__device__ __forceinline__ int32_t fold_add(int32_t a, int32_t b) { return (int32_t)((uint32_t)a + (uint32_t)b); }
__device__ __forceinline__ int32_t fold_mul(int32_t a, int32_t b) { return (int32_t)((uint32_t)a * (uint32_t)b); }

template <class T, int OP> __device__ __forceinline__ T fold(T a, T b) {
    if (OP == SUM || OP == SQNORM) return fold_add(a, b);
    if (OP == PROD) return fold_mul(a, b);
    if (OP == MIN) return b < a ? b : a;  // f32: a NaN operand is ignored, as Rust's f32::min does
    return b > a ? b : a;
}
// For f32 min / max the comparison above keeps `a` when b is NaN and takes b when a is NaN only if
// b compares true, which it never does against NaN; make the f32 forms follow fminf / fmaxf exactly.
template <> __device__ __forceinline__ float fold<float, MIN>(float a, float b) { return fminf(a, b); }
template <> __device__ __forceinline__ float fold<float, MAX>(float a, float b) { return fmaxf(a, b); }

template <class T, int OP> __device__ __forceinline__ T prepare(T v) {
    if (OP == SQNORM) return fold_mul(v, v);
    return v;
}

// ---- ORDERED: the reference's workgroup -----------------------------------------------------
template <class T, int OP>
__global__ void __launch_bounds__(128)
reduce_ordered_kernel(const T* __restrict__ in, uint32_t n, uint32_t stride, T* __restrict__ out) {
    __shared__ T ws[128];
    const uint32_t t = threadIdx.x;
    T a = identity<T, OP>();
    // 4 loads in flight per thread; the folds stay in index order.
    uint32_t i = t;
    for (; i + 3 * 128 < n; i += 4 * 128) {
        const T v0 = in[(size_t)i * stride], v1 = in[(size_t)(i + 128) * stride];
        const T v2 = in[(size_t)(i + 256) * stride], v3 = in[(size_t)(i + 384) * stride];
        a = fold<T, OP>(a, prepare<T, OP>(v0));
        a = fold<T, OP>(a, prepare<T, OP>(v1));
        a = fold<T, OP>(a, prepare<T, OP>(v2));
        a = fold<T, OP>(a, prepare<T, OP>(v3));
    }
    for (; i < n; i += 128) a = fold<T, OP>(a, prepare<T, OP>(in[(size_t)i * stride]));
    ws[t] = a;
    __syncthreads();
    // SQNORM partials are plain sums from here on.
    constexpr int TREE = OP == SQNORM ? SUM : OP;
    for (uint32_t s = 64; s >= 1; s >>= 1) {
        if (t < s) ws[t] = fold<T, TREE>(ws[t], ws[t + s]);
        __syncthreads();
    }
    if (t == 0) out[0] = ws[0];
}

// ---- WIDE: grid of partials + fold ------------------------------------------------------------
constexpr int kWideThreads = 256;

template <class T>
__device__ __forceinline__ T bits_to(uint32_t w);
template <>
__device__ __forceinline__ float bits_to<float>(uint32_t w) { return __uint_as_float(w); }
template <>
__device__ __forceinline__ uint32_t bits_to<uint32_t>(uint32_t w) { return w; }
template <>
__device__ __forceinline__ int32_t bits_to<int32_t>(uint32_t w) { return (int32_t)w; }

template <class T, int OP>
__device__ __forceinline__ T block_fold(T a, T* ws) {
    constexpr int TREE = OP == SQNORM ? SUM : OP;
    const uint32_t t = threadIdx.x;
    ws[t] = a;
    __syncthreads();
    for (uint32_t s = kWideThreads / 2; s >= 1; s >>= 1) {
        if (t < s) ws[t] = fold<T, TREE>(ws[t], ws[t + s]);
        __syncthreads();
    }
    return ws[0];
}

template <class T, int OP>
__global__ void __launch_bounds__(kWideThreads)
reduce_wide_partials_kernel(const T* __restrict__ in, uint32_t n, uint32_t stride, T* partials, uint32_t* done, T* out) {
    __shared__ T ws[kWideThreads];
    __shared__ bool is_last;
    // contiguous slice per block (a multiple of 4 elements), so that the partials' order is the index order
    const uint32_t per = ((n + gridDim.x - 1) / gridDim.x + 3) & ~3u;
    const uint32_t lo = min(n, blockIdx.x * per), hi = min(n, lo + per);
    T a = identity<T, OP>();
    if (stride == 1 && (reinterpret_cast<uintptr_t>(in) & 15u) == 0) {
        // unit stride: 16-byte streaming loads, four running results per thread (element 4 k + j goes to result j),
        // four loads in flight; the thread's four results are folded as (0 with 1) with (2 with 3)
        constexpr int TREE = OP == SQNORM ? SUM : OP;
        constexpr int kInFlight = 4;
        T acc[4] = {a, a, a, a};
        const uint4* v = reinterpret_cast<const uint4*>(in + lo);
        const uint32_t nv = (hi - lo) / 4;
        uint32_t i = threadIdx.x;
        for (; i + (kInFlight - 1) * kWideThreads < nv; i += kInFlight * kWideThreads) {
            uint4 p[kInFlight];
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) p[u] = __ldcs(v + i + u * kWideThreads);
#pragma unroll
            for (int u = 0; u < kInFlight; ++u) {
                const uint32_t pw[4] = {p[u].x, p[u].y, p[u].z, p[u].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[j] = fold<T, OP>(acc[j], prepare<T, OP>(bits_to<T>(pw[j])));
            }
        }
        for (; i < nv; i += kWideThreads) {
            const uint4 p = __ldcs(v + i);
            const uint32_t pw[4] = {p.x, p.y, p.z, p.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] = fold<T, OP>(acc[j], prepare<T, OP>(bits_to<T>(pw[j])));
        }
        a = fold<T, TREE>(fold<T, TREE>(acc[0], acc[1]), fold<T, TREE>(acc[2], acc[3]));
        // the slice's last 1..3 elements (only the last block has any)
        const uint32_t rest = lo + nv * 4 + threadIdx.x;
        if (rest < hi) a = fold<T, TREE>(a, prepare<T, OP>(in[rest]));
    } else {
        for (uint32_t i = lo + threadIdx.x; i < hi; i += kWideThreads) a = fold<T, OP>(a, prepare<T, OP>(in[(size_t)i * stride]));
    }
    const T r = block_fold<T, OP>(a, ws);
    if (done == nullptr) {          // the partials are folded by reduce_wide_final_kernel
        if (threadIdx.x == 0) partials[blockIdx.x] = r;
        return;
    }
    // With a counter, the block that finishes last folds the partials itself, in the same order as
    // reduce_wide_final_kernel: which block that is does not change the result.  atomicInc wraps to 0 at the
    // last arrival, so the counter is ready for the next call.
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = r;
        __threadfence();
        is_last = atomicInc(done, gridDim.x - 1) == gridDim.x - 1;
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    constexpr int TREE = OP == SQNORM ? SUM : OP;
    T f = identity<T, OP>();
    for (uint32_t i = threadIdx.x; i < gridDim.x; i += kWideThreads) f = fold<T, TREE>(f, __ldcg(partials + i));
    const T total = block_fold<T, TREE>(f, ws);
    if (threadIdx.x == 0) out[0] = total;
}

template <class T, int OP>
__global__ void __launch_bounds__(kWideThreads)
reduce_wide_final_kernel(const T* __restrict__ partials, uint32_t count, T* __restrict__ out) {
    __shared__ T ws[kWideThreads];
    constexpr int TREE = OP == SQNORM ? SUM : OP;
    T a = identity<T, OP>();
    for (uint32_t i = threadIdx.x; i < count; i += kWideThreads) a = fold<T, TREE>(a, partials[i]);
    const T r = block_fold<T, TREE>(a, ws);
    if (threadIdx.x == 0) out[0] = r;
}

template <class T, int OP>
vx_status run(vx_context* ctx, bool wide, const T* in, uint32_t n, uint32_t stride, T* out, T* partials,
              uint32_t max_partials) {
    if (!wide) {
        reduce_ordered_kernel<T, OP><<<1, 128, 0, ctx->stream>>>(in, n, stride, out);
        VX_CUDA(cudaGetLastError());
        ctx->launches += 1;
        return VX_OK;
    }
    uint32_t blocks = (n + kWideThreads * 8 - 1) / (kWideThreads * 8);
    blocks = std::max(1u, std::min(blocks, std::min<uint32_t>(max_partials, (uint32_t)ctx->sm_count * (uint32_t)std::clamp<long long>(vx::option(ctx, "reduce.blocks_per_sm", 8), 1, 8))));
    // one launch: the counter behind the partials lets the last block finish the fold
    uint32_t* done = reinterpret_cast<uint32_t*>(partials + max_partials);
    reduce_wide_partials_kernel<T, OP><<<blocks, kWideThreads, 0, ctx->stream>>>(in, n, stride, partials, done, out);
    VX_CUDA(cudaGetLastError());
    ctx->launches += 1;
    return VX_OK;
}

template <class T>
vx_status run_op(vx_context* ctx, int op, bool wide, const void* in, uint32_t n, uint32_t stride, void* out,
                 void* partials, uint32_t max_partials) {
    const T* i = static_cast<const T*>(in);
    T* o = static_cast<T*>(out);
    T* p = static_cast<T*>(partials);
    switch (op) {
        case SUM: return run<T, SUM>(ctx, wide, i, n, stride, o, p, max_partials);
        case PROD: return run<T, PROD>(ctx, wide, i, n, stride, o, p, max_partials);
        case MIN: return run<T, MIN>(ctx, wide, i, n, stride, o, p, max_partials);
        case MAX: return run<T, MAX>(ctx, wide, i, n, stride, o, p, max_partials);
        default: return run<T, SQNORM>(ctx, wide, i, n, stride, o, p, max_partials);
    }
}

vx_status check_args(vx_context* ctx, vx_reduce_op op, vx_dtype dtype, const void* in, const vx_shape* shape,
                     void* out) {
    VX_REQUIRE(ctx && shape && out, VX_ERR_INVALID_ARGUMENT, "vx_reduce: null argument");
    VX_REQUIRE(op >= VX_REDUCE_SUM && op <= VX_REDUCE_SQNORM, VX_ERR_INVALID_ARGUMENT, "unknown reduction %d", (int)op);
    VX_REQUIRE(dtype >= VX_F32 && dtype <= VX_I32, VX_ERR_INVALID_ARGUMENT, "unknown element type %d", (int)dtype);
    VX_REQUIRE(op != VX_REDUCE_SQNORM || dtype == VX_F32, VX_ERR_UNSUPPORTED,
               "the squared norm exists for f32 only (vortx-shaders/src/linalg/reduce.rs:311)");
    VX_REQUIRE(in || shape->w == 0, VX_ERR_INVALID_ARGUMENT, "vx_reduce: null input");
    return VX_OK;
}

}  // namespace

extern "C" {

vx_status vx_reduce(vx_context* ctx, vx_reduce_op op, vx_dtype dtype, vx_reduce_mode mode, const void* in,
                    const vx_shape* shape, uint64_t cap_in, void* out) {
    vx_status st = check_args(ctx, op, dtype, in, shape, out);
    if (st != VX_OK) return st;
    VX_REQUIRE(mode >= VX_REDUCE_ORDERED && mode <= VX_REDUCE_WIDE, VX_ERR_INVALID_ARGUMENT, "unknown mode %d", (int)mode);
    const uint32_t n = shape->w, stride = shape->w_stride;
    if (cap_in != 0 && n != 0 && vx::option(ctx, "bounds_check", 1) != 0)
        VX_REQUIRE((uint64_t)(n - 1) * stride + 1 <= cap_in, VX_ERR_OUT_OF_BOUNDS,
                   "input layout reaches element %llu of a buffer holding %llu",
                   (unsigned long long)((uint64_t)(n - 1) * stride), (unsigned long long)cap_in);
    vx::DeviceGuard guard(ctx->device);
    const bool wide = mode == VX_REDUCE_WIDE;
    void* partials = nullptr;
    const uint32_t max_partials = (uint32_t)ctx->sm_count * 8;
    if (wide) {
        // Scratch for the partials: owned by the context, allocated on first use.
        // (max_partials values, then the arrival counter of the last-block fold, zero between calls)
        if (!ctx->reduce_scratch) {
            VX_CUDA(vx::device_malloc(ctx, &ctx->reduce_scratch, (size_t)max_partials * 4 + 16));
            VX_CUDA(cudaMemsetAsync(static_cast<char*>(ctx->reduce_scratch) + (size_t)max_partials * 4, 0, 16, ctx->stream));
        }
        partials = ctx->reduce_scratch;
    }
    switch (dtype) {
        case VX_F32: return run_op<float>(ctx, (int)op, wide, in, n, stride, out, partials, max_partials);
        case VX_U32: return run_op<uint32_t>(ctx, (int)op, wide, in, n, stride, out, partials, max_partials);
        default: return run_op<int32_t>(ctx, (int)op, wide, in, n, stride, out, partials, max_partials);
    }
}

}  // extern "C"

// ------------------------------------------------------- reduction without any allocation ----
// vx_reduce_static is the WIDE reduction for hosts that must not allocate when they call it: a
// process that handed the whole device to its own arena at start-up and forbids driver
// allocations afterwards, or a latency-critical loop in which a cudaMalloc (which can stall the
// whole device) is not acceptable.  It therefore takes no vx_context either (creating one
// allocates): just a device ordinal and a stream.
//
// Its scratch — one partial per block — is the fixed array below, part of the library's device
// image: every GPU that loads the library carries these 4 KB until the process exits.  The array
// name is a host-side handle, not a device address; the address a kernel can use is obtained once
// per device with cudaGetSymbolAddress (static_partials_for) and cached.
namespace {

constexpr uint32_t kStaticPartials = 1024;           // blocks, hence partials, per call at most
constexpr uint32_t kStaticPerBlock = 65536;          // elements one block folds at most
constexpr uint64_t kStaticMaxElements = (uint64_t)kStaticPartials * kStaticPerBlock;  // 67 108 864
static __device__ __align__(256) unsigned char g_static_partials[kStaticPartials * 4];

// With lazy module loading (the CUDA default) a kernel's code reaches the device at its first launch, and
// that load may allocate device memory.  Asking for the attributes of every instantiation the entry point
// can launch loads them all now, so that only the first call on a device ever loads anything.
template <class T, int OP>
cudaError_t warm_pair() {
    cudaFuncAttributes a;
    cudaError_t e = cudaFuncGetAttributes(&a, reduce_wide_partials_kernel<T, OP>);
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, reduce_wide_final_kernel<T, OP>);
    return e;
}
template <class T>
cudaError_t warm_type(bool with_sqnorm) {
    cudaError_t e = warm_pair<T, SUM>();
    if (e == cudaSuccess) e = warm_pair<T, PROD>();
    if (e == cudaSuccess) e = warm_pair<T, MIN>();
    if (e == cudaSuccess) e = warm_pair<T, MAX>();
    if (e == cudaSuccess && with_sqnorm) e = warm_pair<T, SQNORM>();
    return e;
}

// Device address of g_static_partials on `device`, looked up on the first call for that device
// (with that device current) and remembered; the same first call loads the code of every kernel the
// entry point can launch.  No allocation by this library: the symbol already exists.  Two threads that
// make the first call at once both look the address up and store the same value.
vx_status static_partials_for(int device, void** out) {
    static std::atomic<void*> cached[64];
    VX_REQUIRE(device >= 0 && device < 64, VX_ERR_INVALID_ARGUMENT, "device ordinal %d out of range", device);
    void* p = cached[device].load(std::memory_order_acquire);
    if (!p) {
        VX_CUDA(cudaGetSymbolAddress(&p, g_static_partials));
        VX_CUDA(warm_type<float>(true));
        VX_CUDA(warm_type<uint32_t>(false));
        VX_CUDA(warm_type<int32_t>(false));
        cached[device].store(p, std::memory_order_release);
    }
    *out = p;
    return VX_OK;
}

template <class T, int OP>
vx_status run_static(cudaStream_t stream, const T* in, uint32_t n, uint32_t stride, T* out, T* partials) {
    uint32_t blocks = (n + kWideThreads * 8 - 1) / (kWideThreads * 8);
    blocks = std::max(1u, std::min(blocks, kStaticPartials));
    // Every partial the second kernel reads is written by the first one of the same call, so
    // nothing in the shared array has to be cleared between calls.
    reduce_wide_partials_kernel<T, OP><<<blocks, kWideThreads, 0, stream>>>(in, n, stride, partials, nullptr, nullptr);
    VX_CUDA(cudaGetLastError());
    reduce_wide_final_kernel<T, OP><<<1, kWideThreads, 0, stream>>>(partials, blocks, out);
    VX_CUDA(cudaGetLastError());
    return VX_OK;
}

template <class T>
vx_status run_static_op(int op, cudaStream_t stream, const void* in, uint32_t n, uint32_t stride, void* out,
                        void* partials) {
    const T* i = static_cast<const T*>(in);
    T* o = static_cast<T*>(out);
    T* p = static_cast<T*>(partials);
    switch (op) {
        case SUM: return run_static<T, SUM>(stream, i, n, stride, o, p);
        case PROD: return run_static<T, PROD>(stream, i, n, stride, o, p);
        case MIN: return run_static<T, MIN>(stream, i, n, stride, o, p);
        case MAX: return run_static<T, MAX>(stream, i, n, stride, o, p);
        default: return run_static<T, SQNORM>(stream, i, n, stride, o, p);
    }
}

}  // namespace

extern "C" {

vx_status vx_reduce_static(int32_t device, void* cuda_stream, vx_reduce_op op, vx_dtype dtype, const void* in,
                           const vx_shape* shape, void* out) {
    VX_REQUIRE(shape && out, VX_ERR_INVALID_ARGUMENT, "vx_reduce_static: null argument");
    VX_REQUIRE(op >= VX_REDUCE_SUM && op <= VX_REDUCE_SQNORM, VX_ERR_INVALID_ARGUMENT, "unknown reduction %d", (int)op);
    VX_REQUIRE(dtype >= VX_F32 && dtype <= VX_I32, VX_ERR_INVALID_ARGUMENT, "unknown element type %d", (int)dtype);
    VX_REQUIRE(op != VX_REDUCE_SQNORM || dtype == VX_F32, VX_ERR_UNSUPPORTED, "the squared norm exists for f32 only");
    VX_REQUIRE(in || shape->w == 0, VX_ERR_INVALID_ARGUMENT, "vx_reduce_static: null input");
    VX_REQUIRE((uint64_t)shape->w <= kStaticMaxElements, VX_ERR_UNSUPPORTED,
               "vx_reduce_static takes at most %llu elements (its scratch is a fixed %u-entry array); got %u",
               (unsigned long long)kStaticMaxElements, kStaticPartials, shape->w);
    int device_count = 0;
    VX_CUDA(cudaGetDeviceCount(&device_count));
    VX_REQUIRE(device >= 0 && device < device_count, VX_ERR_INVALID_ARGUMENT,
               "device ordinal %d out of range (0..%d)", device, device_count - 1);
    vx::DeviceGuard guard(device);
    void* partials = nullptr;
    vx_status st = static_partials_for(device, &partials);
    if (st != VX_OK) return st;
    cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
    switch (dtype) {
        case VX_F32: return run_static_op<float>((int)op, stream, in, shape->w, shape->w_stride, out, partials);
        case VX_U32: return run_static_op<uint32_t>((int)op, stream, in, shape->w, shape->w_stride, out, partials);
        default: return run_static_op<int32_t>((int)op, stream, in, shape->w, shape->w_stride, out, partials);
    }
}

}  // extern "C"
