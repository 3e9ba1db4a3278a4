// Multi-GPU group behind the C ABI: one process (or thread) per GPU, one vx_group per context.
//
// vortx knows one device ordinal (src/linalg/gemm.rs:353); nothing here has a reference counterpart.  A group is
// an NCCL communicator over the ranks (for the collective forms: all-gather, broadcast, and for handing CUDA
// IPC handles around) plus what the fused forms need: buffers that every rank can store into (allocated on
// their owner, mapped into the others through IPC) and the arrival flags of vx_peer_barrier.  With it a host
// that has no Python and no torch runs the row-sharded GEMV and the column-sharded GEMM:
//     vx_group_unique_id on rank 0 -> the 128 bytes reach the other ranks by any means -> vx_group_create
//     vx_group_peer_alloc (y or C on every rank) -> vx_group_gemv_q / vx_group_gemm_tf32 -> vx_group_destroy.
// NCCL is loaded at run time (libnccl.so.2, or the path in VX_NCCL_LIBRARY): the library itself has no link-time
// dependency on it, and a process that already holds NCCL (through torch, say) gets that very copy.
#include <dlfcn.h>

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "vx_internal.h"

namespace {

using vx::fail;

// The handful of NCCL entry points used, as declared by nccl.h (the types are fixed by NCCL's ABI).
struct NcclId {
    char internal[128];
};
using ncclComm_t = void*;
enum { kNcclSuccess = 0, kNcclUint8 = 1, kNcclSum = 0 };
struct Nccl {
    int (*GetUniqueId)(NcclId*) = nullptr;
    int (*CommInitRank)(ncclComm_t*, int, NcclId, int) = nullptr;
    int (*CommDestroy)(ncclComm_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    int (*Broadcast)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    void* handle = nullptr;
    std::string why;
};

Nccl* nccl() {
    static Nccl n;
    static std::once_flag once;
    std::call_once(once, [] {
        const char* env = std::getenv("VX_NCCL_LIBRARY");
        const char* names[] = {env, "libnccl.so.2", "libnccl.so"};
        for (const char* name : names) {
            if (!name || !*name) continue;
            n.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (n.handle) break;
            n.why = dlerror();
        }
        if (!n.handle) return;
        auto sym = [&](const char* s) { return dlsym(n.handle, s); };
        n.GetUniqueId = reinterpret_cast<decltype(n.GetUniqueId)>(sym("ncclGetUniqueId"));
        n.CommInitRank = reinterpret_cast<decltype(n.CommInitRank)>(sym("ncclCommInitRank"));
        n.CommDestroy = reinterpret_cast<decltype(n.CommDestroy)>(sym("ncclCommDestroy"));
        n.AllGather = reinterpret_cast<decltype(n.AllGather)>(sym("ncclAllGather"));
        n.Broadcast = reinterpret_cast<decltype(n.Broadcast)>(sym("ncclBroadcast"));
        n.GetErrorString = reinterpret_cast<decltype(n.GetErrorString)>(sym("ncclGetErrorString"));
        if (!n.GetUniqueId || !n.CommInitRank || !n.CommDestroy || !n.AllGather || !n.Broadcast || !n.GetErrorString) {
            n.why = "the NCCL library lacks an expected entry point";
            n.handle = nullptr;
        }
    });
    return n.handle ? &n : nullptr;
}

#define VX_NCCL(expr)                                                                                       \
    do {                                                                                                    \
        const int vx_r_ = (expr);                                                                           \
        if (vx_r_ != kNcclSuccess)                                                                          \
            return fail(VX_ERR_COLLECTIVE, "%s failed: %s", #expr, nccl()->GetErrorString(vx_r_));          \
    } while (0)

}  // namespace

struct vx_group {
    vx_context* ctx = nullptr;
    size_t world = 1, rank = 0;
    ncclComm_t comm = nullptr;
    uint32_t* flags[vx::kMaxPeers + 1] = {};   // arrival flags of vx_peer_barrier: own block and the mapped peers'
    uint8_t* staging = nullptr;                // device scratch for handing IPC handles around: world x 64 bytes
};

namespace {

// Exchanges one 64-byte IPC handle per rank and maps the peers' buffers; ptrs[rank] = mine.
vx_status exchange(vx_group* g, void* mine, void** ptrs) {
    vx_context* ctx = g->ctx;
    for (size_t r = 0; r < g->world; ++r) ptrs[r] = nullptr;
    ptrs[g->rank] = mine;
    if (g->world == 1) return VX_OK;
    uint8_t handle[64];
    vx_status st = vx_ipc_export(ctx, mine, handle);
    if (st != VX_OK) return st;
    VX_CUDA(cudaMemcpyAsync(g->staging + 64 * g->rank, handle, 64, cudaMemcpyHostToDevice, ctx->stream));
    VX_NCCL(nccl()->AllGather(g->staging + 64 * g->rank, g->staging, 64, kNcclUint8, g->comm, ctx->stream));
    std::vector<uint8_t> all(64 * g->world);
    VX_CUDA(cudaMemcpyAsync(all.data(), g->staging, all.size(), cudaMemcpyDeviceToHost, ctx->stream));
    VX_CUDA(cudaStreamSynchronize(ctx->stream));
    for (size_t r = 0; r < g->world; ++r) {
        if (r == g->rank) continue;
        st = vx_ipc_import(ctx, all.data() + 64 * r, &ptrs[r]);
        if (st != VX_OK) return st;
    }
    return VX_OK;
}

}  // namespace

extern "C" {

vx_status vx_group_unique_id(void* id128) {
    VX_REQUIRE(id128, VX_ERR_INVALID_ARGUMENT, "vx_group_unique_id: null argument");
    Nccl* n = nccl();
    VX_REQUIRE(n, VX_ERR_COLLECTIVE, "NCCL is not available: %s", n ? "" : "libnccl.so.2 could not be loaded (set VX_NCCL_LIBRARY)");
    NcclId id;
    VX_NCCL(n->GetUniqueId(&id));
    std::memcpy(id128, &id, 128);
    return VX_OK;
}

vx_status vx_group_create(vx_context* ctx, size_t world, size_t rank, const void* id128, vx_group** out) {
    VX_REQUIRE(ctx && out, VX_ERR_INVALID_ARGUMENT, "vx_group_create: null argument");
    *out = nullptr;
    VX_REQUIRE(world >= 1 && world <= (size_t)vx::kMaxPeers + 1 && rank < world, VX_ERR_INVALID_ARGUMENT,
               "world %zu / rank %zu out of range (at most %d GPUs of one node)", world, rank, vx::kMaxPeers + 1);
    vx::DeviceGuard guard(ctx->device);
    vx_group* g = new (std::nothrow) vx_group();
    VX_REQUIRE(g, VX_ERR_OUT_OF_MEMORY, "host allocation failed");
    g->ctx = ctx;
    g->world = world;
    g->rank = rank;
    auto cleanup = [&](vx_status st) {
        vx_group_destroy(g);
        return st;
    };
    void* own = nullptr;
    if (vx::device_malloc(ctx, &own, 64 * sizeof(uint32_t)) != cudaSuccess) return cleanup(fail(VX_ERR_OUT_OF_MEMORY, "allocating the group's flags failed"));
    g->flags[rank] = static_cast<uint32_t*>(own);
    if (cudaMemsetAsync(own, 0, 64 * sizeof(uint32_t), ctx->stream) != cudaSuccess) return cleanup(fail(VX_ERR_CUDA, "clearing the group's flags failed"));
    if (world > 1) {
        VX_REQUIRE(id128, VX_ERR_INVALID_ARGUMENT, "vx_group_create: a group of %zu ranks needs the unique id of rank 0", world);
        Nccl* n = nccl();
        if (!n) return cleanup(fail(VX_ERR_COLLECTIVE, "NCCL is not available: libnccl.so.2 could not be loaded (set VX_NCCL_LIBRARY)"));
        // No NVLink multicast objects bound to this process's buffers: a rank that ends while its memory is bound
        // to one raises faults on the others.  (An explicit setting of the variable by the host is respected.)
        setenv("NCCL_NVLS_ENABLE", "0", 0);
        NcclId id;
        std::memcpy(&id, id128, 128);
        const int r = n->CommInitRank(&g->comm, (int)world, id, (int)rank);
        if (r != kNcclSuccess) return cleanup(fail(VX_ERR_COLLECTIVE, "ncclCommInitRank failed: %s", n->GetErrorString(r)));
        void* staging = nullptr;
        if (vx::device_malloc(ctx, &staging, 64 * world) != cudaSuccess) return cleanup(fail(VX_ERR_OUT_OF_MEMORY, "allocating the group's staging buffer failed"));
        g->staging = static_cast<uint8_t*>(staging);
        void* ptrs[vx::kMaxPeers + 1];
        const vx_status st = exchange(g, own, ptrs);
        if (st != VX_OK) return cleanup(st);
        for (size_t i = 0; i < world; ++i) g->flags[i] = static_cast<uint32_t*>(ptrs[i]);
    }
    if (cudaStreamSynchronize(ctx->stream) != cudaSuccess) return cleanup(fail(VX_ERR_CUDA, "synchronising after the group's set-up failed"));
    *out = g;
    return VX_OK;
}

vx_status vx_group_destroy(vx_group* g) {
    if (!g) return VX_OK;
    vx_context* ctx = g->ctx;
    vx::DeviceGuard guard(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    for (size_t r = 0; r < g->world; ++r)
        if (r != g->rank && g->flags[r]) cudaIpcCloseMemHandle(g->flags[r]);
    if (g->flags[g->rank]) cudaFree(g->flags[g->rank]);
    if (g->staging) cudaFree(g->staging);
    if (g->comm && nccl()) nccl()->CommDestroy(g->comm);
    (void)cudaGetLastError();
    delete g;
    return VX_OK;
}

vx_status vx_group_info(const vx_group* g, size_t* world, size_t* rank) {
    VX_REQUIRE(g, VX_ERR_INVALID_ARGUMENT, "vx_group_info: null group");
    if (world) *world = g->world;
    if (rank) *rank = g->rank;
    return VX_OK;
}

vx_status vx_group_all_gather(vx_group* g, const void* send, void* recv, size_t bytes_per_rank) {
    VX_REQUIRE(g && recv, VX_ERR_INVALID_ARGUMENT, "vx_group_all_gather: null argument");
    if (bytes_per_rank == 0) return VX_OK;
    vx_context* ctx = g->ctx;
    vx::DeviceGuard guard(ctx->device);
    uint8_t* mine = static_cast<uint8_t*>(recv) + bytes_per_rank * g->rank;
    if (!send) send = mine;       // in place: this rank's part already sits at its position
    if (g->world == 1) {
        if (send != mine) VX_CUDA(cudaMemcpyAsync(mine, send, bytes_per_rank, cudaMemcpyDeviceToDevice, ctx->stream));
        return VX_OK;
    }
    VX_NCCL(nccl()->AllGather(send, recv, bytes_per_rank, kNcclUint8, g->comm, ctx->stream));
    return VX_OK;
}

vx_status vx_group_broadcast(vx_group* g, void* buffer, size_t bytes, size_t root) {
    VX_REQUIRE(g && (buffer || bytes == 0), VX_ERR_INVALID_ARGUMENT, "vx_group_broadcast: null argument");
    VX_REQUIRE(root < g->world, VX_ERR_INVALID_ARGUMENT, "root %zu outside a group of %zu", root, g->world);
    if (bytes == 0 || g->world == 1) return VX_OK;
    vx::DeviceGuard guard(g->ctx->device);
    VX_NCCL(nccl()->Broadcast(buffer, buffer, bytes, kNcclUint8, (int)root, g->comm, g->ctx->stream));
    return VX_OK;
}

vx_status vx_group_peer_alloc(vx_group* g, size_t bytes, void** ptrs) {
    VX_REQUIRE(g && ptrs, VX_ERR_INVALID_ARGUMENT, "vx_group_peer_alloc: null argument");
    vx_context* ctx = g->ctx;
    vx::DeviceGuard guard(ctx->device);
    void* mine = nullptr;
    VX_CUDA(vx::device_malloc(ctx, &mine, bytes ? bytes : 16));
    cudaError_t e = cudaMemsetAsync(mine, 0, bytes ? bytes : 16, ctx->stream);
    if (e != cudaSuccess) {
        cudaFree(mine);
        return fail(VX_ERR_CUDA, "clearing a peer buffer failed: %s", cudaGetErrorString(e));
    }
    const vx_status st = exchange(g, mine, ptrs);
    if (st != VX_OK) {
        for (size_t r = 0; r < g->world; ++r)
            if (r != g->rank && ptrs[r]) cudaIpcCloseMemHandle(ptrs[r]);
        cudaFree(mine);
        for (size_t r = 0; r < g->world; ++r) ptrs[r] = nullptr;
        return st;
    }
    VX_CUDA(cudaStreamSynchronize(ctx->stream));
    return VX_OK;
}

vx_status vx_group_peer_free(vx_group* g, void* const* ptrs) {
    VX_REQUIRE(g && ptrs, VX_ERR_INVALID_ARGUMENT, "vx_group_peer_free: null argument");
    vx_context* ctx = g->ctx;
    vx::DeviceGuard guard(ctx->device);
    VX_CUDA(cudaStreamSynchronize(ctx->stream));
    for (size_t r = 0; r < g->world; ++r)
        if (r != g->rank && ptrs[r]) cudaIpcCloseMemHandle(ptrs[r]);
    if (ptrs[g->rank]) cudaFree(ptrs[g->rank]);
    (void)cudaGetLastError();
    return VX_OK;
}

vx_status vx_group_barrier(vx_group* g) {
    VX_REQUIRE(g, VX_ERR_INVALID_ARGUMENT, "vx_group_barrier: null group");
    if (g->world == 1) return VX_OK;
    return vx_peer_barrier(g->ctx, g->flags, g->world, g->rank);
}

vx_status vx_group_gemv_q(vx_group* g, const vx_qweights* slab, size_t row0, const float* x, void* const* y_all,
                          size_t y_offset) {
    VX_REQUIRE(g && slab && x && y_all, VX_ERR_INVALID_ARGUMENT, "vx_group_gemv_q: null argument");
    float* mine = reinterpret_cast<float*>(static_cast<uint8_t*>(y_all[g->rank]) + y_offset) + row0;
    float* peers[vx::kMaxPeers];
    size_t n = 0;
    for (size_t r = 0; r < g->world; ++r) {
        VX_REQUIRE(y_all[r], VX_ERR_INVALID_ARGUMENT, "vx_group_gemv_q: y of rank %zu is null", r);
        if (r != g->rank) peers[n++] = reinterpret_cast<float*>(static_cast<uint8_t*>(y_all[r]) + y_offset) + row0;
    }
    const vx_status st = vx_gemv_q_rows_scatter(g->ctx, slab, 0, slab->rows, x, mine, peers, n);
    if (st != VX_OK) return st;
    return vx_group_barrier(g);
}

vx_status vx_group_gemm_tf32(vx_group* g, const float* lhs, const float* rhs_panel, size_t m, size_t n, size_t k,
                             size_t col0, size_t ncols, size_t rhs_stride, void* const* c_all) {
    VX_REQUIRE(g && lhs && rhs_panel && c_all, VX_ERR_INVALID_ARGUMENT, "vx_group_gemm_tf32: null argument");
    VX_REQUIRE(col0 + ncols <= n && m <= 0xFFFFFFFFull && n <= 0xFFFFFFFFull && k <= 0xFFFFFFFFull && rhs_stride <= 0xFFFFFFFFull,
               VX_ERR_SHAPE, "panel [%zu, %zu) outside %zu columns", col0, col0 + ncols, n);
    vx_shapes3 s{};
    auto set = [](vx_shape& sh, size_t h, size_t w, size_t hs) {
        sh.n = sh.c = 1;
        sh.h = (uint32_t)h;
        sh.w = (uint32_t)w;
        sh.n_stride = sh.c_stride = (uint32_t)(h * hs);
        sh.h_stride = (uint32_t)hs;
        sh.w_stride = 1;
    };
    set(s.out, m, ncols, n);
    set(s.lhs, m, k, k);
    set(s.rhs, k, ncols, rhs_stride);
    float* peers[vx::kMaxPeers];
    size_t np = 0;
    for (size_t r = 0; r < g->world; ++r) {
        VX_REQUIRE(c_all[r], VX_ERR_INVALID_ARGUMENT, "vx_group_gemm_tf32: C of rank %zu is null", r);
        if (r != g->rank) peers[np++] = static_cast<float*>(c_all[r]) + col0;
    }
    if (ncols != 0) {
        const vx_status st = vx_gemm_tf32_scatter(g->ctx, static_cast<float*>(c_all[g->rank]) + col0, lhs, rhs_panel, &s, peers, np);
        if (st != VX_OK) return st;
    }
    return vx_group_barrier(g);
}

}  // extern "C"
