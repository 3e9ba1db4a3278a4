// f32 GEMM on the 5th-generation tensor cores: TF32 inputs, f32 accumulation in tensor memory.
//
// out[M,N] = lhs[M,K] * rhs[K,N], all row-major f32 (vortx's layout: src/tensor/tensor_impl.rs:543-555).
// Same semantics as gemm_tiled (vortx-shaders/src/linalg/gemm.rs:41-194) — overwrite, no alpha /
// beta — but the products are formed from TF32 operands and summed in an order of the hardware's
// choosing, so results agree with the SIMT kernel to about 1e-3 relative, not bit for bit.
//
// One persistent CTA per SM, 192 threads:
//   warp 0   TMA producer: per k-block of 32, one box of A (K-major, 128-byte swizzle) and eight
//            32 x 32 boxes of B (N-major: the natural form of a row-major K x N matrix) into a
//            shared-memory ring, completion on one mbarrier per stage.
//   warp 1   MMA issuer: allocates all 512 columns of tensor memory (two 128 x 256 f32
//            accumulators), issues tcgen05.mma.kind::tf32 128x256x8 from one thread, commits each
//            stage back to the producer and, after the last k-block, the accumulators to the epilogue.
//   warps 2-5  epilogue: tcgen05.ld the accumulators (each warp its 32 lanes), store rows to global
//            memory, hand the accumulators back.
// Two tile shapes share the code (template parameter HALVES):
//   HALVES = 1  128 x 256 tiles, the two accumulators alternate between consecutive tiles so that the
//               epilogue of one tile runs under the MMAs of the next; 4 stages of 48 KB.
//   HALVES = 2  256 x 256 tiles, the two accumulators are the upper and lower half of one tile and
//               every stage of B feeds both.  With 4-byte operands the kernel is bound by the bytes
//               that must reach shared memory per FLOP (measured: 12.5 TB/s from L2 at 128 x 256,
//               tensor pipe 61 % busy); sharing B across 256 rows cuts that by a third, at the price
//               of an epilogue that is no longer hidden (about 2 % of a tile at K = 8192).  3 stages
//               of 64 KB.
// B needs no transposing pre-pass: the instruction descriptor marks it MN-major.  For a 32-bit
// MN-major operand the tensor core accepts exactly one shared-memory form, the 128-byte swizzle
// with 32-byte atoms (measured: the 16-byte-atom form yields zeros), so B's tensor map uses
// CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B and its descriptor walks 32-column atoms (leading offset
// 4 KB) of 4-row k groups (stride offset 512 B).
#include <cuda.h>

#include <atomic>
#include <mutex>

#include <algorithm>
#include <cstring>

#include "vx_internal.h"
#include "vx_sm100.cuh"

namespace {

using namespace sm100;

constexpr int BMMA = 128, BN = 256, BK = 32;  // one MMA's M, N; BK floats = 128 bytes = one swizzle span
constexpr int UMMA_K = 8;                     // k per tcgen05.mma for 32-bit inputs
constexpr uint32_t kAHalfBytes = BMMA * BK * 4;        // 16 KB: 128 rows of A
constexpr uint32_t kBAtomBytes = 32 * BK * 4;          // one 32-column atom: 32 k-rows x 128 B = 4 KB
constexpr uint32_t kBBytes = (BN / 32) * kBAtomBytes;  // 32 KB
constexpr uint32_t kTmemCols = 2 * BN;                 // 512: both accumulators
constexpr int kThreads = 192;
constexpr int kMaxStages = 4;

template <int HALVES> struct Cfg {
    static constexpr int BM = BMMA * HALVES;                 // rows of C per tile
    static constexpr uint32_t kABytes = kAHalfBytes * HALVES;
    static constexpr uint32_t kStageBytes = kABytes + kBBytes;  // 48 KB or 64 KB
    static constexpr int kStages = HALVES == 1 ? 4 : 3;
    static constexpr int kAccStages = HALVES == 1 ? 2 : 1;   // tiles in flight in tensor memory
};

struct Tf32Params {
    float* out;
    uint32_t m, n, k;
    uint64_t ldc;
    uint32_t tiles_m, tiles_n;
    uint32_t raster;  // tiles of M walked together before moving along N
    uint32_t out_vec; // rows of out are 16-byte aligned
    // Column-sharded use: every tile is also stored at the same position of these buffers (the
    // full-width C of each peer GPU, mapped into this process).  Plain stores over NVLink.
    uint32_t n_peer;
    uint32_t tma_store;  // the epilogue sends blocks with tiled TMA stores (always with peers)
    float* out_peer[vx::kMaxPeers];
    vx::DeviceStatus* status;
};

// With peers, each epilogue warp stages a 32 x 32 block of C (one row per lane, as tensor memory hands it
// out) in shared memory in the 128-byte-swizzled box layout and one lane sends it with tiled TMA stores to
// this GPU's C and to every peer's: the copies run asynchronously (the warp goes on to the next block, two
// staging buffers per warp) and leave as whole 128-byte rows over NVLink.
constexpr uint32_t kStageBoxBytes = 32 * 32 * 4;                 // 4 KB
constexpr uint32_t kXposeBytes = 4 * 2 * kStageBoxBytes;         // four epilogue warps, two buffers each
struct PeerMaps {
    CUtensorMap c[vx::kMaxPeers + 1];  // [0] this GPU's panel of C, then the peers'
};

struct SharedTail {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
};

__device__ __forceinline__ void report(vx::DeviceStatus* st, uint32_t code) {
    volatile vx::DeviceStatus* v = st;
    v->detail = blockIdx.x;
    v->code = code;
    __threadfence_system();
}

__device__ __forceinline__ void tile_coords(const Tf32Params& p, uint32_t t, uint32_t& tm, uint32_t& tn) {
    // Groups of `raster` M-tiles are walked column by column, so that CTAs running at the same
    // time share a few panels of A and of B in L2.
    const uint32_t per_group = p.raster * p.tiles_n;
    const uint32_t g = t / per_group, r = t % per_group;
    const uint32_t first_m = g * p.raster;
    const uint32_t height = min(p.raster, p.tiles_m - first_m);
    tm = first_m + r % height;
    tn = r / height;
}

// Instruction descriptor of tcgen05.mma.kind::tf32: f32 accumulate (bits 4-5 = 1), A and B TF32
// (bits 7-9, 10-12 = 2), A K-major (bit 15 = 0), B MN-major (bit 16 = 1), N / 8 at bit 17, M / 16 at bit 24.
constexpr uint32_t kIdesc = (1u << 4) | (2u << 7) | (2u << 10) | (0u << 15) | (1u << 16) |
                            ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BMMA >> 4) << 24);

template <int HALVES>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ Tf32Params p, const __grid_constant__ PeerMaps maps_c) {
    using C = Cfg<HALVES>;
    constexpr int kStages = C::kStages, kAccStages = C::kAccStages;
    constexpr uint32_t kStageBytes = C::kStageBytes, kABytes = C::kABytes;

    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // The ring must start on a 1024-byte boundary (128-byte swizzle repeats every 8 rows).
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    SharedTail* tail = reinterpret_cast<SharedTail*>(smem + kStages * kStageBytes);
    uint8_t* stage_all = smem + kStages * kStageBytes + 1024;  // used with peers only; 1024-byte aligned
    volatile uint32_t* abort_flag = &tail->abort_flag;

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t num_tiles = p.tiles_m * p.tiles_n;
    const uint32_t num_kb = (p.k + BK - 1) / BK;

    if (threadIdx.x == 0) {
        tail->abort_flag = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_addr(&tail->full[s]), 1);
            mbar_init(smem_addr(&tail->empty[s]), 1);
        }
        for (int a = 0; a < kAccStages; ++a) {
            mbar_init(smem_addr(&tail->acc_full[a]), 1);
            mbar_init(smem_addr(&tail->acc_empty[a]), 4);  // one arrival per epilogue warp
        }
        mbar_init_fence();
        tma_prefetch_desc(&map_a);
        tma_prefetch_desc(&map_b);
    }
    if (warp == 1) {
        tmem_alloc(smem_addr(&tail->tmem_base), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tail->tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer ----
        if (lane == 0) {
            uint32_t it = 0;  // k-blocks issued so far, across tiles
            for (uint32_t t = blockIdx.x; t < num_tiles; t += gridDim.x) {
                uint32_t tm, tn;
                tile_coords(p, t, tm, tn);
                for (uint32_t kb = 0; kb < num_kb; ++kb, ++it) {
                    const uint32_t s = it % kStages, use = it / kStages;
                    if (use > 0 && !mbar_wait(smem_addr(&tail->empty[s]), (use - 1) & 1, abort_flag))
                        report(p.status, 21);
                    const uint32_t full = smem_addr(&tail->full[s]);
                    const uint32_t dst_a = smem_addr(smem + s * kStageBytes);
                    const uint32_t dst_b = dst_a + kABytes;
                    mbar_arrive_expect_tx(full, kStageBytes);
                    // A: one box of BM rows x 32 floats (the box of map_a is BM rows tall)
                    tma_load_2d(dst_a, &map_a, (int32_t)(kb * BK), (int32_t)(tm * C::BM), full);
#pragma unroll
                    for (int a = 0; a < BN / 32; ++a)
                        tma_load_2d(dst_b + a * kBAtomBytes, &map_b, (int32_t)(tn * BN + a * 32), (int32_t)(kb * BK), full);
                }
            }
            // Leave only once every copy into this CTA's shared memory has landed and been used.
            for (uint32_t s = 0; s < (uint32_t)kStages && s < it; ++s) {
                const uint32_t last = ((it - 1 - s) / kStages) * kStages + s;
                if (!mbar_wait(smem_addr(&tail->empty[s]), (last / kStages) & 1, abort_flag)) report(p.status, 22);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------- MMA issuer ----
        if (lane == 0) {
            uint32_t it = 0, tile_it = 0;
            for (uint32_t t = blockIdx.x; t < num_tiles; t += gridDim.x, ++tile_it) {
                const uint32_t as = tile_it % kAccStages, ause = tile_it / kAccStages;
                if (ause > 0 && !mbar_wait(smem_addr(&tail->acc_empty[as]), (ause - 1) & 1, abort_flag))
                    report(p.status, 23);
                tc_fence_after_sync();
                // HALVES = 1: accumulator `as` (256 columns).  HALVES = 2: both, upper half first.
                const uint32_t d_tmem = tmem_base + (HALVES == 1 ? as * BN : 0);
                for (uint32_t kb = 0; kb < num_kb; ++kb, ++it) {
                    const uint32_t s = it % kStages;
                    if (!mbar_wait(smem_addr(&tail->full[s]), (it / kStages) & 1, abort_flag)) report(p.status, 24);
                    tc_fence_after_sync();
                    const uint32_t a_addr = smem_addr(smem + s * kStageBytes);
                    const uint32_t b_addr = a_addr + kABytes;
#pragma unroll
                    for (int ks = 0; ks < BK / UMMA_K; ++ks) {
                        // B: MN-major with 32-byte swizzle atoms: 32-column atoms 4 KB apart (leading
                        // offset), groups of 4 k-rows of 128 B 512 B apart (stride offset); a k-step of 8
                        // rows is 1 KB.
                        const uint64_t db = smem_desc(b_addr + ks * UMMA_K * 128, kBAtomBytes, 512, kSwizzle128BAtom32B);
#pragma unroll
                        for (int h = 0; h < HALVES; ++h) {
                            // A: K-major, rows of 128 B, 8-row groups 1 KB apart; a k-step is 32 B along the
                            // row; the lower half of a 256-row tile starts 16 KB further.
                            const uint64_t da = smem_desc_sw128(a_addr + h * kAHalfBytes + ks * UMMA_K * 4, 16, 1024);
                            mma_tf32(d_tmem + h * BN, da, db, kIdesc, (kb | ks) != 0 ? 1u : 0u);
                        }
                    }
                    mma_commit(smem_addr(&tail->empty[s]));  // stage reusable once these MMAs have read it
                }
                mma_commit(smem_addr(&tail->acc_full[as]));  // accumulator(s) complete
            }
        }
    } else {
        // --------------------------------------------------------------------- epilogue ----
        const uint32_t quad = warp & 3;  // a warp may only touch tensor-memory lanes 32*(warp%4) ..
        uint32_t tile_it = 0, chunk_it = 0;
        for (uint32_t t = blockIdx.x; t < num_tiles; t += gridDim.x, ++tile_it) {
            uint32_t tm, tn;
            tile_coords(p, t, tm, tn);
            const uint32_t as = tile_it % kAccStages;
            if (!mbar_wait(smem_addr(&tail->acc_full[as]), (tile_it / kAccStages) & 1, abort_flag))
                report(p.status, 25);
            tc_fence_after_sync();
            const uint32_t col0 = tn * BN;
#pragma unroll 1
            for (int h = 0; h < HALVES; ++h) {
                const uint32_t row = tm * C::BM + h * BMMA + quad * 32 + lane;
                float* dst_row = p.out + (size_t)row * p.ldc + col0;
                const uint32_t taddr = tmem_base + ((quad * 32) << 16) + (HALVES == 1 ? as * BN : h * BN);
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t v[32];
                    tmem_ld_32x32(taddr + c * 32, v);
                    tmem_ld_wait();
                    const uint32_t col = col0 + c * 32;
                    if (p.tma_store) {
                        // (the host only takes this path when TMA can describe every C: 16-byte aligned bases and
                        // row pitches)
                        const uint32_t use = chunk_it++;
                        uint8_t* box = stage_all + (quad * 2 + (use & 1)) * kStageBoxBytes;
                        // the copies that last read this buffer (two blocks ago) must have read it
                        if (lane == 0) bulk_wait_group_read<1>();
                        __syncwarp();
                        // 128-byte swizzle: 16-byte unit j of row r sits at position j ^ (r & 7)
                        uint8_t* mine = box + lane * 128;
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            *reinterpret_cast<float4*>(mine + ((j ^ (lane & 7)) << 4)) =
                                make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                            __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                        fence_proxy_async_smem();
                        __syncwarp();
                        const uint32_t row_base = tm * C::BM + h * BMMA + quad * 32;
                        if (lane == 0) {
                            if (row_base < p.m && col < p.n) {
                                const uint32_t src = smem_addr(box);
                                for (uint32_t d = 0; d <= p.n_peer; ++d)
                                    tma_store_2d(&maps_c.c[d], (int32_t)col, (int32_t)row_base, src);
                            }
                            bulk_commit_group();
                        }
                    } else if (row < p.m) {
                        if (p.out_vec && col + 32 <= p.n) {
                            float4* d4 = reinterpret_cast<float4*>(dst_row + c * 32);
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                d4[j] = make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                    __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col + j < p.n) dst_row[c * 32 + j] = __uint_as_float(v[j]);
                        }
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_addr(&tail->acc_empty[as]));
        }
        // every TMA store of this warp has been performed before the block leaves
        if (p.tma_store && lane == 0) bulk_wait_group<0>();
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// cuTensorMapEncodeTiled, fetched from the driver at run time so that the library carries no
// link-time dependency on libcuda (it must load on machines without a driver).
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
    // contexts of different devices may call from different threads: looked up once, under a lock
    static std::once_flag once;
    static EncodeFn fn = nullptr;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeFn>(sym);
        (void)cudaGetLastError();
    });
    return fn;
}

// 2-D f32 tensor map: inner dimension `inner` (unit stride), outer dimension `outer` with
// `stride_elems` between rows; box inner_box x outer_box; zero fill out of bounds.
// `round_tf32`: the copy engine rounds each f32 to TF32 (to nearest) on its way into shared memory; the tensor
// core otherwise just drops the low 13 mantissa bits.
bool make_map(CUtensorMap* map, const float* base, uint64_t inner, uint64_t outer, uint64_t stride_elems,
              uint32_t inner_box, uint32_t outer_box, CUtensorMapSwizzle swizzle, bool round_tf32 = false) {
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {stride_elems * sizeof(float)};
    const cuuint32_t box[2] = {inner_box, outer_box};
    const cuuint32_t elem[2] = {1, 1};
    return fn(map, round_tf32 ? CU_TENSOR_MAP_DATA_TYPE_TFLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
              const_cast<float*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <int HALVES>
vx_status launch_tiles(vx_context* ctx, const CUtensorMap& map_a, const CUtensorMap& map_b, Tf32Params p,
                       const PeerMaps& maps_c) {
    using C = Cfg<HALVES>;
    const size_t smem = (size_t)C::kStages * C::kStageBytes + 1024 + kXposeBytes + 1024;
    static_assert(sizeof(SharedTail) <= 1024, "barriers sit in the first KB after the ring, the staging boxes after it");
    static std::atomic<bool> attr_set[64];
    if (!attr_set[ctx->device & 63].load(std::memory_order_acquire)) {
        VX_CUDA(cudaFuncSetAttribute(gemm_tf32_kernel<HALVES>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[ctx->device & 63].store(true, std::memory_order_release);
    }
    p.tiles_m = (p.m + C::BM - 1) / C::BM;
    p.tiles_n = (p.n + BN - 1) / BN;
    const uint32_t tiles = p.tiles_m * p.tiles_n;
    dim3 grid(std::min<uint32_t>(tiles, (uint32_t)ctx->sm_count));
    gemm_tf32_kernel<HALVES><<<grid, kThreads, smem, ctx->stream>>>(map_a, map_b, p, maps_c);
    VX_CUDA(cudaGetLastError());
    return VX_OK;
}

}  // namespace

namespace vx {

vx_status launch_gemm_tf32(vx_context* ctx, float* out, const float* lhs, const float* rhs,
                           const vx_shapes3& s, bool* eligible, float* const* out_peer, uint32_t n_peer) {
    *eligible = false;
    if (n_peer > 0) {
        // The peer path sends 32 x 32 blocks with tiled TMA stores: every C must be describable.
        if (s.out.n != 1 || s.out.c != 1 || !aligned16(out) || s.out.h_stride % 4 != 0 || s.out.h_stride < s.out.w) return VX_OK;
        for (uint32_t d = 0; d < n_peer; ++d)
            if (!aligned16(out_peer[d])) return VX_OK;
    }
    const uint32_t m = s.out.h, n = s.out.w, k = s.lhs.w;
    // What TMA can describe: unit stride along the rows, 16-byte aligned bases and row pitches.
    if (m == 0 || n == 0 || k == 0) return VX_OK;
    if (s.lhs.w_stride != 1 || s.rhs.w_stride != 1 || s.out.w_stride != 1) return VX_OK;
    if (!aligned16(lhs) || !aligned16(rhs)) return VX_OK;
    if (s.lhs.h_stride % 4 != 0 || s.rhs.h_stride % 4 != 0) return VX_OK;
    if (s.lhs.h_stride < k || s.rhs.h_stride < n) return VX_OK;  // overlapping rows: leave to the generic kernel
    const uint64_t batches = (uint64_t)s.out.n * s.out.c;
    if (batches > 1 && (s.lhs.n_stride % 4 || s.lhs.c_stride % 4 || s.rhs.n_stride % 4 || s.rhs.c_stride % 4))
        return VX_OK;
    if (batches > 4096) return VX_OK;
    if (!encode_fn()) return VX_OK;

    // 256-row tiles as soon as they fill the SMs once (measured at 4096^3, 1.7 waves: 709 against
    // 537 TFLOP/s); below that the finer 128-row tiles spread better.  "gemm.tf32.tile_m" forces one.
    const uint64_t tiles256 = (uint64_t)((m + 255) / 256) * ((n + BN - 1) / BN);
    int halves = tiles256 >= (uint64_t)ctx->sm_count ? 2 : 1;
    const int64_t forced = option(ctx, "gemm.tf32.tile_m", 0);
    if (forced == 128) halves = 1;
    if (forced == 256) halves = 2;

    for (uint32_t bn = 0; bn < s.out.n; ++bn)
        for (uint32_t bc = 0; bc < s.out.c; ++bc) {
            const float* a = lhs + (size_t)bn * s.lhs.n_stride + (size_t)bc * s.lhs.c_stride;
            const float* b = rhs + (size_t)bn * s.rhs.n_stride + (size_t)bc * s.rhs.c_stride;
            float* c = out + (size_t)bn * s.out.n_stride + (size_t)bc * s.out.c_stride;
            CUtensorMap map_a, map_b;
            const bool rn = option(ctx, "gemm.tf32.round_nearest", 1) != 0;
            if (!make_map(&map_a, a, k, m, s.lhs.h_stride, BK, BMMA * halves, CU_TENSOR_MAP_SWIZZLE_128B, rn) ||
                !make_map(&map_b, b, n, k, s.rhs.h_stride, 32, BK, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, rn)) {
                if (bn == 0 && bc == 0) return VX_OK;  // nothing launched yet: let the caller fall back
                return fail(VX_ERR_CUDA, "cuTensorMapEncodeTiled refused a batch matrix after the first");
            }
            Tf32Params p;
            p.out = c;
            p.m = m;
            p.n = n;
            p.k = k;
            p.ldc = s.out.h_stride;
            p.tiles_m = p.tiles_n = 0;  // set by launch_tiles
            p.raster = (uint32_t)std::max<int64_t>(1, option(ctx, "gemm.tf32.raster", halves == 2 ? 2 : 8));
            p.out_vec = (aligned16(c) && s.out.h_stride % 4 == 0) ? 1u : 0u;
            p.status = ctx->d_status;
            p.n_peer = std::min<uint32_t>(n_peer, kMaxPeers);
            for (uint32_t d = 0; d < (uint32_t)kMaxPeers; ++d) p.out_peer[d] = d < p.n_peer ? out_peer[d] : nullptr;
            PeerMaps maps_c;
            memset(&maps_c, 0, sizeof(maps_c));
            // One map per destination: the panel (n columns wide, rows ldc apart), 32 x 32 boxes in the
            // 128-byte-swizzled layout the epilogue stages.  Without peers the TMA epilogue is a choice
            // ("gemm.tf32.tma_store", default on when C can be described): the warps hand their blocks to the
            // copy engine instead of storing them themselves.
            p.tma_store = 0;
            const bool describable = aligned16(c) && s.out.h_stride % 4 == 0 && s.out.h_stride >= n;
            if (p.n_peer > 0 || (describable && option(ctx, "gemm.tf32.tma_store", 1) != 0)) {
                p.tma_store = 1;
                for (uint32_t d = 0; d <= p.n_peer; ++d) {
                    float* dst = d == 0 ? c : out_peer[d - 1];
                    if (!make_map(&maps_c.c[d], dst, n, m, s.out.h_stride, 32, 32, CU_TENSOR_MAP_SWIZZLE_128B)) {
                        if (p.n_peer == 0) {
                            p.tma_store = 0;
                            break;
                        }
                        return fail(VX_ERR_UNSUPPORTED, "cuTensorMapEncodeTiled refused the C panel of destination %u", d);
                    }
                }
            }
            vx_status st = halves == 2 ? launch_tiles<2>(ctx, map_a, map_b, p, maps_c)
                                       : launch_tiles<1>(ctx, map_a, map_b, p, maps_c);
            if (st != VX_OK) return st;
            ctx->launches++;
            ctx->status_dirty = true;
        }
    *eligible = true;
    return VX_OK;
}

}  // namespace vx
