// Streaming GEMV for block-quantised weights: TMA-fed, x-stationary, integer dot products.
//
// Shape of the kernel (8 consumer warps + 1 producer warp + 1 epilogue warp per CTA):
//   * The producer thread streams tiles of TR consecutive rows (their quants, and their f16
//     scales) from HBM into a ring of shared-memory stages with untiled TMA bulk copies,
//     completion counted on one mbarrier per stage.  Bytes in flight are set by the ring,
//     not by registers or occupancy.
//   * Every consumer thread owns the same 16-byte chunk position(s) of every row (32 Q4_0
//     weights or 16 Q8_0 weights) and keeps the matching slice of x in registers for a whole
//     product, so x is read from memory once per CTA and product and never touches shared memory.
//   * x is held as fixed point: per chunk, x_i = sx * X_i with |X_i| < 2^23, and X_i split into
//     three byte planes (signed high, unsigned middle and low).  A chunk-row product is then
//     6 (Q4_0: 24, Q8_0: 12) dp4a on the raw quants — exact integer arithmetic — followed by
//     one f32 multiply-add with d * sx.  The rounding of x to 24 bits relative to the chunk
//     maximum is of the order of one f32 ulp, and the block sums are exact, so the result is at
//     least as accurate as an f32-accumulated product.  The "- 8" of Q4_0 is folded into the
//     initial value of the integer accumulators (-8 * sum of the digits).
//   * Per tile, the TR partial sums per thread are combined with a transposed shuffle
//     reduction (values halve as lanes pair up); each warp then drops its partials into a small
//     shared-memory buffer and signals an mbarrier.  A tenth warp adds the warps' partials and
//     writes y, so the consumer warps never meet at a CTA barrier.
//   * One launch runs a LIST of GEMVs of one row shape (a batch): the three roles walk the
//     list with one continuous ring, so the weight stream of the next product is already in
//     flight while the last rows of the current one are reduced, and prologue, tail and launch
//     latency are paid once per list, not once per product.  Products of a list that depend on
//     each other exchange their vectors as flagged pairs (below), which needs no grid barrier.
// No scratch memory in global memory, no split along K, every weight byte read once.
#include <cuda_fp16.h>

#include <algorithm>
#include <atomic>
#include <memory>
#include <vector>

#include "vx_internal.h"
#include "vx_sm100.cuh"

namespace {

using namespace sm100;

constexpr int kConsumers = 256;            // consumer threads of a CTA (8 warps)
constexpr int kRedBufs = 4;                // partial-sum buffers between consumers and the epilogue warp

constexpr int kMaxVecs = 8;
constexpr int kInlineOps = 8;  // GEMVs of a list that travel in the kernel parameters

// One GEMV of the list.
struct OpParams {
    const uint8_t* quants;
    const uint8_t* scales;  // f16 plane, addressed in bytes
    uint64_t row0;
    uint32_t nrows;
    uint32_t x_aligned;     // x is 16-byte aligned
    const float* x;
    float* y;               // plain f32 rows, or null
    // Row-sharded use: besides y, every finished row is stored into these buffers (the same slab
    // of the full-length y on each peer GPU, mapped into this process), so that no collective is
    // needed afterwards.  Plain stores to peer memory; nothing is ever loaded from a peer.
    float* y_peer[vx::kMaxPeers];
    uint32_t n_peer;
    // Fused exchange (optional).  An exchange vector is a 256-byte header (word 0: how many times
    // the vector has been written completely, its generation; word 1: thread blocks of the
    // current launch that have finished) followed by one 8-byte pair {f32 value, u32 generation}
    // per element.  A value and the generation that says it has arrived travel in ONE 64-bit
    // store, so neither side needs a fence or a flag: the writer stores pairs tagged with the
    // next generation into its own vector and into every peer's, the reader knows which
    // generation to expect from its own header and re-reads any pair that does not carry it yet.
    // Headers only change when the last block of a launch retires; within a launch the expected
    // generation is the header's value plus the number of earlier writes of the list.
    int32_t x_vec;                        // index into StreamParams::vec_hdr, or -1: plain x
    uint32_t x_gen_add;
    int32_t y_vec;                        // or -1: no flagged output
    uint32_t y_gen_add;
    const uint64_t* x_pairs;
    // x may be a window of a longer flagged vector: `x_seg_len` consecutive elements, starting at element
    // `x_seg_first`, out of every `x_seg_stride` (a piece of each rank's slab, when the vector holds one slab
    // per rank).  x_seg_len == 0: x is the vector's first cols elements.
    uint32_t x_seg_len, x_seg_stride, x_seg_first;
    uint64_t* y_pairs;                    // this rank's vector, advanced to the slab's first element
    uint64_t* y_pairs_peer[vx::kMaxPeers];
    uint32_t n_pair_peer;
    uint32_t y_pair_stride;               // row r of the slab is element r * stride of y_pairs
};

struct StreamParams {
    uint32_t nchunks;        // 16-byte chunks per row
    uint32_t nb;             // blocks per row
    uint32_t tpr;            // threads per row group (multiple of 32)
    uint32_t stages;
    uint32_t stage_bytes;
    uint32_t q_stage_bytes;  // TR * row bytes: where the scales start inside a stage
    uint32_t n_ops;          // up to kInlineOps: inline_ops; more: ops[] in device memory
    uint32_t block_wait;     // flagged x: one warp waits for the block (see the consumers)
    uint32_t n_vec;
    long long wait_cycles;   // budget of the flagged-x waits, in SM clocks
#ifdef VX_TIMELINE
    unsigned long long* timeline;   // [block][entry][8] globaltimer stamps, or null (option "debug.timeline_ptr")
#endif
    const OpParams* ops;
    uint32_t* vec_hdr[kMaxVecs];   // headers of the exchange vectors the list touches (own memory)
    uint32_t vec_writes[kMaxVecs]; // how often the list writes each of them
    vx::DeviceStatus* status;
    OpParams inline_ops[kInlineOps];
};

__device__ __forceinline__ void report(vx::DeviceStatus* st, uint32_t code) {
    // Mapped host memory, written only on failure; which failing block wins does not matter.
    volatile vx::DeviceStatus* v = st;
    v->detail = blockIdx.x;
    v->code = code;
    __threadfence_system();
}

template <int NR>
__device__ __forceinline__ float transposed_reduce(float (&v)[NR], uint32_t lane) {
    // After the call lane l holds the full warp sum of v[row(l)], where row(l) is read off the
    // lane's high bits: NR = 8 -> bits 4,3,2; NR = 4 -> bits 4,3; NR = 2 -> bit 4; NR = 1 -> none.
    int off = 16;
#pragma unroll
    for (int n = NR; n > 1; n >>= 1, off >>= 1) {
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < n / 2; ++i) {
            const float send = upper ? v[i] : v[i + n / 2];
            const float keep = upper ? v[i + n / 2] : v[i];
            v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    }
    float r = v[0];
    for (; off > 0; off >>= 1) r += __shfl_xor_sync(0xffffffffu, r, off);
    return r;
}

// First tile of GEMV `op` that this block takes; it then strides by the grid.  When the tiles do
// not divide evenly, the blocks that take one more rotate from one GEMV of the list to the next.
__device__ __forceinline__ uint32_t first_tile(uint32_t op, uint32_t tiles) {
    const uint32_t rot = (uint32_t)(((uint64_t)op * (tiles % gridDim.x)) % gridDim.x);
    const uint32_t t = blockIdx.x + gridDim.x - rot;
    return t >= gridDim.x ? t - gridDim.x : t;
}

// QT: 0 = Q8_0 (16 weights per 16-byte chunk), 1 = Q4_0 (32 weights per chunk).
// CPT: chunk positions per thread.  RP: row groups working side by side.  TR: rows per tile.
// XCH: reads a flagged x and / or writes flagged pairs (the cross-GPU exchange); a template
// switch so that the plain kernel keeps its register count (two CTAs per SM need <= 102).
// NCW: consumer warps, 8 everywhere.  (The plain kernel gets 16 warps per SM from two CTAs.  A flagged
// CTA of 16 consumer warps, x held twice, measured slower than 8: 17.9 against 15.2 us per chained
// 14336 x 8192 product.)
// Timeline build (nvcc -DVX_TIMELINE, `python -m vortx_b200.build --timeline`): thread 0 of the consumers and
// lane 0 of the epilogue warp stamp %globaltimer (nanoseconds; it ticks every 256 ns here) per list entry:
//   [0] entry begins  [1] after the block's wait for x (the block-wait form; else = [0])  [2] x read (the threads'
//   own waits included) and converted  [3] first tile present  ([7] of entry 0: the thread block starts)
//   [4] last tile computed  [5] rows of the last tile stored  [6] rows of the first tile stored
// The product build carries none of this.
#ifdef VX_TIMELINE
#define VX_TL(...) do { __VA_ARGS__; } while (0)
__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
#else
#define VX_TL(...) do { } while (0)
#endif

template <int QT, int CPT, int RP, int TR, bool XCH, int NCW>
__global__ void __launch_bounds__(NCW * 32 + 64, 1)
gemv_stream_kernel(const __grid_constant__ StreamParams p) {
    constexpr int kWarps = NCW;
    constexpr int kConsumers = NCW * 32;  // then one producer warp and one epilogue warp
    constexpr int W = QT == 1 ? 32 : 16;
    constexpr int DR = W / 4;   // registers per digit plane per chunk
    constexpr int NR = TR / RP; // rows per thread per tile
    static_assert(TR % RP == 0 && NR >= 1 && NR <= 8, "bad tile split");

    extern __shared__ __align__(128) uint8_t smem[];
    float* red = reinterpret_cast<float*>(smem + (size_t)p.stages * p.stage_bytes);  // [kRedBufs][TR][kWarps]
    uint64_t* bars = reinterpret_cast<uint64_t*>(red + kRedBufs * TR * kWarps);
    // full[S], empty[S], red_full[kRedBufs], red_empty[kRedBufs]
    const uint32_t bar0 = smem_addr(bars);
    auto full = [&](uint32_t s) { return bar0 + 8u * s; };
    auto empty = [&](uint32_t s) { return bar0 + 8u * (p.stages + s); };
    auto red_full = [&](uint32_t b) { return bar0 + 8u * (2 * p.stages + b); };
    auto red_empty = [&](uint32_t b) { return bar0 + 8u * (2 * p.stages + kRedBufs + b); };
    // Set by the first bounded wait that gives up; see sm100::mbar_wait.
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 2 * 16 + 2 * kRedBufs);

    const uint32_t tid = threadIdx.x;
    VX_TL(if (p.timeline && tid == 0) p.timeline[(size_t)blockIdx.x * p.n_ops * 8 + 7] = gtime());
    // Programmatic dependent launch: let the next kernel in the stream start its own prologue
    // as soon as this grid's CTAs are all under way.  Nothing here depends on that kernel.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (tid == 0) {
        *abort_flag = 0u;
        for (uint32_t s = 0; s < p.stages; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), kWarps);
        }
        for (uint32_t b = 0; b < kRedBufs; ++b) {
            mbar_init(red_full(b), kWarps);
            mbar_init(red_empty(b), 1);
        }
        mbar_init_fence();
    }
    __syncthreads();

    const OpParams* const ops = p.ops ? p.ops : p.inline_ops;
    const uint32_t row_bytes = p.nchunks * 16;
    const uint32_t wpr = p.tpr >> 5;  // warps per row group

    if (tid >= kConsumers + 32) {
        // ---------------------------------------------------------------- epilogue ----
        const uint32_t lane = tid & 31;
        // y may still be read by the previous kernel in the stream: write it only once that
        // kernel has completed.
        asm volatile("griddepcontrol.wait;" ::: "memory");
        uint32_t k = 0;
        for (uint32_t o = 0; o < p.n_ops; ++o) {
            const OpParams& op = ops[o];
            const uint32_t nrows = op.nrows;
            const uint32_t tiles = (nrows + TR - 1) / TR;
            uint32_t t = first_tile(o, tiles);
            if (t >= tiles) continue;
            float* const y = op.y;
            const uint32_t n_peer = op.n_peer;
            uint64_t* const y_pairs = XCH ? op.y_pairs : nullptr;
            const uint32_t n_pair_peer = XCH ? op.n_pair_peer : 0;
            const uint32_t stride = XCH ? op.y_pair_stride : 1;
            // Generation this GEMV writes.
            const uint32_t gen = XCH && y_pairs ? *(volatile const uint32_t*)p.vec_hdr[op.y_vec] + op.y_gen_add : 0;
#ifdef VX_TIMELINE
            bool tl_first_store = true;
#endif
            for (; t < tiles; t += gridDim.x, ++k) {
                const uint32_t b = k % kRedBufs;
                if (!mbar_wait(red_full(b), (k / kRedBufs) & 1, abort_flag)) report(p.status, 14);
                const float* slot = red + (size_t)b * TR * kWarps;
                const uint32_t row = t * TR + lane;
                if (lane < (uint32_t)TR && row < nrows) {
                    float sum = 0.0f;
                    for (uint32_t wv = 0; wv < wpr; ++wv) sum += slot[lane * kWarps + wv];
                    if (y) y[row] = sum;
                    for (uint32_t d = 0; d < n_peer; ++d) op.y_peer[d][row] = sum;
                    if (XCH && y_pairs) {
                        const uint64_t pair = ((uint64_t)gen << 32) | __float_as_uint(sum);
                        const size_t at = (size_t)row * stride;
                        st_relaxed_sys_u64(y_pairs + at, pair);
                        for (uint32_t d = 0; d < n_pair_peer; ++d) st_relaxed_sys_u64(op.y_pairs_peer[d] + at, pair);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(red_empty(b));
                VX_TL(if (p.timeline && lane == 0) {
                    unsigned long long* d = p.timeline + ((size_t)blockIdx.x * p.n_ops + o) * 8;
                    const unsigned long long now = gtime();
                    d[5] = now;
                    if (tl_first_store) d[6] = now;
                    tl_first_store = false;
                });
            }
        }
        if (XCH && p.n_vec > 0 && lane == 0) {
            // The last block to retire publishes the new generations to later kernels of this GPU.
            if (atomicAdd(p.vec_hdr[0] + 1, 1u) == gridDim.x - 1) {
                for (uint32_t v = 0; v < p.n_vec; ++v)
                    *(volatile uint32_t*)p.vec_hdr[v] = *(volatile uint32_t*)p.vec_hdr[v] + p.vec_writes[v];
                *(volatile uint32_t*)(p.vec_hdr[0] + 1) = 0;
            }
        }
        return;
    }
    if (tid >= kConsumers) {
        // ---------------------------------------------------------------- producer ----
        if (tid == kConsumers) {
            const uint64_t policy = policy_evict_first();
            uint32_t k = 0;
            for (uint32_t o = 0; o < p.n_ops; ++o) {
                const OpParams& op = ops[o];
                const uint32_t nrows = op.nrows;
                const uint32_t tiles = (nrows + TR - 1) / TR;
                const uint8_t* const quants = op.quants;
                const uint8_t* const scales = op.scales;
                const uint64_t row0 = op.row0;
                for (uint32_t t = first_tile(o, tiles); t < tiles; t += gridDim.x, ++k) {
                    const uint32_t s = k % p.stages, use = k / p.stages;
                    if (use > 0 && !mbar_wait(empty(s), (use - 1) & 1, abort_flag)) report(p.status, 11);
                    const uint32_t tr = min((uint32_t)TR, nrows - t * TR);
                    const uint64_t first = row0 + (uint64_t)t * TR;
                    const uint32_t qbytes = tr * row_bytes;
                    const uint64_t soff = first * p.nb * 2;
                    const uint64_t salign = soff & ~(uint64_t)15;
                    const uint32_t sbytes = (uint32_t)(((soff - salign) + (uint64_t)tr * p.nb * 2 + 15) & ~(uint64_t)15);
                    const uint32_t dst = smem_addr(smem + (size_t)s * p.stage_bytes);
                    mbar_arrive_expect_tx(full(s), qbytes + sbytes);
                    bulk_g2s_hint(dst, quants + first * row_bytes, qbytes, full(s), policy);
                    bulk_g2s_hint(dst + p.q_stage_bytes, scales + salign, sbytes, full(s), policy);
                }
            }
            // Do not leave while copies into this CTA's shared memory are still in flight:
            // wait until the consumers have released the last use of every stage.
            for (uint32_t s = 0; s < p.stages && s < k; ++s) {
                const uint32_t last_k = ((k - 1 - s) / p.stages) * p.stages + s;  // last tile index on stage s
                if (!mbar_wait(empty(s), (last_k / p.stages) & 1, abort_flag)) report(p.status, 12);
            }
        }
        return;
    }

    // -------------------------------------------------------------------- consumers ----
    const uint32_t lane = tid & 31, warp = tid >> 5;
    const uint32_t rp = warp / wpr;           // this warp's row group
    const bool active = rp < (uint32_t)RP;
    const uint32_t tc = tid - rp * p.tpr;     // position inside the group

    // x may be the output of the previous kernel in the stream: wait for it (the producer
    // warp is already streaming weights, which no kernel writes).
    asm volatile("griddepcontrol.wait;" ::: "memory");

    // x -> three byte planes per chunk, kept in registers for one GEMV of the list.
    uint32_t DA[CPT][DR], DB[CPT][DR], DC[CPT][DR];
    float sxs[CPT];
    int initA[CPT], initB[CPT], initC[CPT];
    const float* held_x = nullptr;  // plain x the registers hold; GEMVs of a list often share it

    uint32_t k = 0;
    for (uint32_t o = 0; o < p.n_ops; ++o) {
        const OpParams& op = ops[o];
        const uint32_t tiles = (op.nrows + TR - 1) / TR;
        uint32_t t = first_tile(o, tiles);
        if (t >= tiles) continue;
        const uint64_t* const x_pairs = XCH && op.x_vec >= 0 ? op.x_pairs : nullptr;
        const float* const x = op.x;
#ifdef VX_TIMELINE
        unsigned long long* const tl = p.timeline && tid == 0 ? p.timeline + ((size_t)blockIdx.x * p.n_ops + o) * 8 : nullptr;
        bool tl_first = true;
#endif
        VX_TL(if (tl) tl[0] = gtime());
        if (x_pairs || x != held_x) {
            held_x = x_pairs ? nullptr : x;
            const uint32_t x_gen = x_pairs ? *(volatile const uint32_t*)p.vec_hdr[op.x_vec] + op.x_gen_add : 0;
            const uint32_t x_aligned = op.x_aligned;
            const uint32_t seg_len = XCH ? op.x_seg_len : 0, seg_stride = XCH ? op.x_seg_stride : 0;
            const uint32_t seg_first = XCH ? op.x_seg_first : 0;
            if (XCH && x_pairs && p.block_wait) {
                // One warp waits for the whole block: it re-reads the last two pairs of every chunk of x until
                // they all carry the generation; the other consumer warps sleep at a hardware barrier
                // meanwhile.  (Eight warps re-reading their own chunks at full rate took the issue slots and
                // the load pipe from this SM's epilogue warp, which still had the rows to deliver that other
                // blocks were waiting for: with 3 tiles per block and product, at 8 GPUs, a fully dependent
                // chained product took 26 us.)  What the probes do not cover is caught by each thread's own
                // read below.  The extra round of probes costs about 2 us per product, so the host only asks
                // for it when a block has few tiles per product and waiting dominates.
                if (warp == 0) {
                    const long long start = clock64();
                    for (;;) {
                        bool all = true;
                        // eight probes per lane in flight at a time (256 chunks per round)
                        for (uint32_t c0 = 0; c0 < p.nchunks; c0 += 256) {
                            uint64_t pa[8], pb[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) {
                                const uint32_t c = min(c0 + lane + 32u * i, p.nchunks - 1);
                                const uint32_t e = c * W + (W - 2);
                                ld_volatile_v2_u64(x_pairs + (seg_len ? (size_t)(e / seg_len) * seg_stride + seg_first + e % seg_len : (size_t)e),
                                                   pa[i], pb[i]);
                            }
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                all = all && (uint32_t)(pa[i] >> 32) == x_gen && (uint32_t)(pb[i] >> 32) == x_gen;
                        }
                        if (__all_sync(0xffffffffu, all)) break;
                        // one decision for the whole warp: the lanes must leave the loop together
                        if (__any_sync(0xffffffffu, *abort_flag != 0u || clock64() - start > p.wait_cycles)) break;   // the reads below report it
                    }
                }
                asm volatile("bar.sync 1, %0;" ::"n"(kConsumers) : "memory");
            }
            VX_TL(if (tl) tl[1] = gtime());
#pragma unroll
            for (int j = 0; j < CPT; ++j) {
                const uint32_t c = tc + j * p.tpr;
                const bool valid = active && c < p.nchunks;
                float xv[W];
                if (XCH && valid && x_pairs) {
                    // Flagged x: two pairs per 16-byte load; anything that does not carry this vector's
                    // generation yet is still on its way (from a peer, or from another block of this
                    // grid) and is read again (bounded).
                    const uint32_t e = c * W;  // first element of the chunk; segments are whole chunks
                    const uint64_t* src = x_pairs + (seg_len ? (size_t)(e / seg_len) * seg_stride + seg_first + e % seg_len : (size_t)e);
                    const long long start = clock64();
                    bool ok = false;
                    while (!ok) {
                        ok = true;
                        // 16 values (eight 16-byte loads) at a time: the temporaries of the loads are what
                        // sets the kernel's register count
#pragma unroll
                        for (int h = 0; h < W / 16; ++h) {
                            uint64_t v[16];
#pragma unroll
                            for (int i = 0; i < 8; ++i) ld_volatile_v2_u64(src + 16 * h + 2 * i, v[2 * i], v[2 * i + 1]);
                            uint32_t good = 1;
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                good &= (uint32_t)(v[i] >> 32) == x_gen ? 1u : 0u;
                                xv[16 * h + i] = __uint_as_float((uint32_t)v[i]);
                            }
                            // pins this group's values before the next group's loads are issued
                            asm volatile("" : "+r"(good) : "f"(xv[16 * h]), "f"(xv[16 * h + 5]), "f"(xv[16 * h + 10]), "f"(xv[16 * h + 15]));
                            ok = ok && good != 0;
                        }
                        if (!ok) {
                            if (*abort_flag != 0u || clock64() - start > p.wait_cycles) break;
                            // No __nanosleep here: measured on B200, a block whose warps sleep while they wait runs
                            // its next tiles about three times slower for tens of microseconds (a chained product
                            // took 33 us instead of 17.5 us when every block had to wait for the rows computed last).
                        }
                    }
                    if (!ok) {
                        if (*abort_flag == 0u) report(p.status, 16);
                        *abort_flag = 1u;
                    }
                } else if (valid) {
                    const float* src = x + (size_t)c * W;
                    if (x_aligned) {
#pragma unroll
                        for (int i = 0; i < W / 4; ++i) {
                            const float4 v = __ldg(reinterpret_cast<const float4*>(src) + i);
                            xv[4 * i + 0] = v.x; xv[4 * i + 1] = v.y; xv[4 * i + 2] = v.z; xv[4 * i + 3] = v.w;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < W; ++i) xv[i] = __ldg(src + i);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < W; ++i) xv[i] = 0.0f;
                }
#ifdef VX_TIMELINE
                // plain x: [1] = the first and the last 16 bytes of the thread's first chunk have arrived
                if (tl && j == 0 && !x_pairs) {
                    float probe = xv[0] + xv[W - 1];
                    asm volatile("" ::"f"(probe));
                    tl[1] = gtime();
                }
#endif
                float amax = 0.0f, poison = 0.0f;
#pragma unroll
                for (int i = 0; i < W; ++i) {
                    amax = fmaxf(amax, fabsf(xv[i]));
                    poison = fmaf(xv[i], 0.0f, poison);   // NaN as soon as one value is NaN or infinite (fmaxf skips NaN)
                }
                // |x * inv| <= 8388606.5 before rounding, so X stays within 24 signed bits without a clamp.
                float inv = amax > 0.0f ? 8388606.0f / amax : 0.0f;
                float sx = amax / 8388606.0f;
                // a chunk whose largest value is below 8388606 / FLT_MAX: the quotient would overflow; scale by
                // an exact power of two instead (|X| stays below 2^23, sx * inv == 1)
                if (amax > 0.0f && amax < 4.9e-32f) { inv = 0x1p126f; sx = 0x1p-126f; }
                // a NaN or an infinity in x reaches every row as NaN, as it would through f32 products and sums
                // of mixed signs (an f32 accumulation could also end on +-inf; this kernel does not tell them apart)
                if (poison != poison) { inv = 0.0f; sx = poison; }
                sxs[j] = valid ? sx : 0.0f;
                int sa = 0, sb = 0, sc = 0;
#pragma unroll
                for (int r = 0; r < DR; ++r) {
                    const uint32_t X0 = (uint32_t)__float2int_rn(xv[4 * r + 0] * inv);
                    const uint32_t X1 = (uint32_t)__float2int_rn(xv[4 * r + 1] * inv);
                    const uint32_t X2 = (uint32_t)__float2int_rn(xv[4 * r + 2] * inv);
                    const uint32_t X3 = (uint32_t)__float2int_rn(xv[4 * r + 3] * inv);
                    // byte n of each X gathered into one register: n = 2 signed high, 1 middle, 0 low
                    DA[j][r] = __byte_perm(__byte_perm(X0, X1, 0x0062), __byte_perm(X2, X3, 0x0062), 0x5410);
                    DB[j][r] = __byte_perm(__byte_perm(X0, X1, 0x0051), __byte_perm(X2, X3, 0x0051), 0x5410);
                    DC[j][r] = __byte_perm(__byte_perm(X0, X1, 0x0040), __byte_perm(X2, X3, 0x0040), 0x5410);
                    sa = dp4a_ss(0x01010101u, DA[j][r], sa);
                    sb = dp4a_su(0x01010101u, DB[j][r], sb);
                    sc = dp4a_su(0x01010101u, DC[j][r], sc);
                }
                initA[j] = QT == 1 ? -8 * sa : 0;
                initB[j] = QT == 1 ? -8 * sb : 0;
                initC[j] = QT == 1 ? -8 * sc : 0;
            }
        }
        VX_TL(if (tl) tl[2] = gtime());

        const uint64_t row0 = op.row0;
        for (; t < tiles; t += gridDim.x, ++k) {
            const uint32_t s = k % p.stages;
            if (!mbar_wait(full(s), (k / p.stages) & 1, abort_flag)) report(p.status, 13);
            VX_TL(if (tl && tl_first) { tl[3] = gtime(); tl_first = false; });
            const uint8_t* sq = smem + (size_t)s * p.stage_bytes;
            const uint64_t soff = (row0 + (uint64_t)t * TR) * p.nb * 2;
            const uint8_t* ss = sq + p.q_stage_bytes + (uint32_t)(soff & 15);

            float acc[NR];
#pragma unroll
            for (int i = 0; i < NR; ++i) acc[i] = 0.0f;

            if (active) {
#pragma unroll
                for (int j = 0; j < CPT; ++j) {
                    // a chunk position past the row's end reads chunk 0 with sx = 0
                    const uint32_t cj = tc + j * p.tpr;
                    const uint32_t c = cj < p.nchunks ? cj : 0;
                    const uint32_t blk = QT == 1 ? c : (c >> 1);
                    // All shared-memory reads of the tile first, so that the integer chains of the
                    // NR rows can overlap.
                    uint4 q[NR];
                    uint16_t dh[NR];
#pragma unroll
                    for (int i = 0; i < NR; ++i) {
                        const uint32_t r = rp + i * RP;  // row inside the tile
                        q[i] = *reinterpret_cast<const uint4*>(sq + ((size_t)r * p.nchunks + c) * 16);
                        dh[i] = *reinterpret_cast<const uint16_t*>(ss + ((size_t)r * p.nb + blk) * 2);
                    }
#pragma unroll
                    for (int i = 0; i < NR; ++i) {
                        const uint32_t w[4] = {q[i].x, q[i].y, q[i].z, q[i].w};
                        int sa = initA[j], sb = initB[j], sc = initC[j];
                        if (QT == 1) {
#pragma unroll
                            for (int m = 0; m < 4; ++m) {
                                const uint32_t lo = w[m] & 0x0F0F0F0Fu, hi = (w[m] >> 4) & 0x0F0F0F0Fu;
                                sa = dp4a_ss(lo, DA[j][m], sa);
                                sb = dp4a_su(lo, DB[j][m], sb);
                                sc = dp4a_su(lo, DC[j][m], sc);
                                sa = dp4a_ss(hi, DA[j][4 + m], sa);
                                sb = dp4a_su(hi, DB[j][4 + m], sb);
                                sc = dp4a_su(hi, DC[j][4 + m], sc);
                            }
                        } else {
#pragma unroll
                            for (int m = 0; m < 4; ++m) {
                                sa = dp4a_ss(w[m], DA[j][m], sa);
                                sb = dp4a_su(w[m], DB[j][m], sb);
                                sc = dp4a_su(w[m], DC[j][m], sc);
                            }
                        }
                        // sum q X = 65536 sa + 256 sb + sc; |256 sb + sc| < 2^31 for both formats.
                        const float tsum = fmaf((float)sa, 65536.0f, (float)(sb * 256 + sc));
                        const float d = __half2float(__ushort_as_half(dh[i]));
                        acc[i] = fmaf(d * sxs[j], tsum, acc[i]);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty(s));  // this warp has finished reading the stage

            const float total = transposed_reduce<NR>(acc, lane);
            const uint32_t b = k % kRedBufs;
            if (k >= kRedBufs && !mbar_wait(red_empty(b), ((k / kRedBufs) - 1) & 1, abort_flag)) report(p.status, 15);
            float* slot = red + (size_t)b * TR * kWarps;
            if (active) {
                // lanes whose low bits are zero hold one row each
                constexpr uint32_t low_mask = NR == 8 ? 3u : NR == 4 ? 7u : NR == 2 ? 15u : 31u;
                if ((lane & low_mask) == 0) {
                    const uint32_t i = NR == 8 ? (((lane >> 4) & 1u) * 4 + ((lane >> 3) & 1u) * 2 + ((lane >> 2) & 1u))
                                     : NR == 4 ? (((lane >> 4) & 1u) * 2 + ((lane >> 3) & 1u))
                                     : NR == 2 ? ((lane >> 4) & 1u) : 0u;
                    slot[(rp + i * RP) * kWarps + (warp - rp * wpr)] = total;
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(red_full(b));
            VX_TL(if (tl) tl[4] = gtime());
        }
    }
}

template <int QT, int CPT, int RP, int TR, bool XCH, int NCW = 8>
vx_status launch_one(vx_context* ctx, const StreamParams& p, dim3 grid, size_t smem) {
    auto kernel = gemv_stream_kernel<QT, CPT, RP, TR, XCH, NCW>;
    // Raise the dynamic shared-memory limit once per device and kernel instance.
    // (contexts of different devices may launch from different threads: the record is atomic, and setting
    // the attribute twice is harmless)
    static std::atomic<size_t> granted[64];
    const int dev = ctx->device & 63;
    if (granted[dev].load(std::memory_order_acquire) < smem) {
        VX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        granted[dev].store(smem, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(NCW * 32 + 64);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    // Weights quantised on the device by the kernel just before this one (vx_qweights_from_device) are only
    // guaranteed visible once that kernel has completed, and the producer warp reads weights before
    // griddepcontrol.wait: such a launch is an ordinary, fully serialised one.
    cfg.numAttrs = vx::option(ctx, "gemv.pdl", 1) != 0 && !ctx->weights_fresh ? 1 : 0;
    ctx->weights_fresh = false;
    VX_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
    return VX_OK;
}

template <int QT, int TR, bool XCH>
vx_status launch_qt(vx_context* ctx, int cpt, int rp, int ncw, const StreamParams& p, dim3 grid, size_t smem) {
    (void)ncw;
    if (cpt == 1) {
        switch (rp) {
            case 1: return launch_one<QT, 1, 1, TR, XCH>(ctx, p, grid, smem);
            case 2: return launch_one<QT, 1, 2, TR, XCH>(ctx, p, grid, smem);
            default: return launch_one<QT, 1, 4, TR, XCH>(ctx, p, grid, smem);
        }
    }
    if (cpt == 2) return launch_one<QT, 2, 1, TR, XCH>(ctx, p, grid, smem);
    return launch_one<QT, 4, 1, TR, XCH>(ctx, p, grid, smem);
}

// How one row shape maps onto the kernel.
struct StreamConfig {
    uint32_t tr, tpr, stages, stage_bytes, q_stage;
    int cpt, rp, ncw;
    int64_t per_sm;
    size_t smem;
};

template <bool XCH>
vx_status launch_tr(vx_context* ctx, int qtype, const StreamConfig& c, const StreamParams& p, dim3 grid) {
    if (c.tr == 8)
        return qtype == VX_Q4_0 ? launch_qt<1, 8, XCH>(ctx, c.cpt, c.rp, c.ncw, p, grid, c.smem)
                                : launch_qt<0, 8, XCH>(ctx, c.cpt, c.rp, c.ncw, p, grid, c.smem);
    return qtype == VX_Q4_0 ? launch_qt<1, 4, XCH>(ctx, c.cpt, c.rp, c.ncw, p, grid, c.smem)
                            : launch_qt<0, 4, XCH>(ctx, c.cpt, c.rp, c.ncw, p, grid, c.smem);
}


// false: the row is too long for the shared-memory ring or the register-resident x.
bool choose_config_tr(vx_context* ctx, uint32_t tile_rows, uint32_t nchunks, uint32_t nb, uint32_t max_tiles_hint_rows,
                      bool flagged, StreamConfig* c) {
    using vx::option;
    c->tr = tile_rows;
    if (nchunks > 4 * kConsumers) return false;
    c->cpt = nchunks <= kConsumers ? 1 : nchunks <= 2 * kConsumers ? 2 : 4;
    uint32_t tpr = ((nchunks + c->cpt - 1) / c->cpt + 31) / 32 * 32;
    c->tpr = std::min<uint32_t>(tpr, kConsumers);
    c->rp = 1;
    c->ncw = 8;
    if (c->cpt == 1) {
        const uint32_t fit = (uint32_t)c->ncw * 32 / c->tpr;  // 1..16
        c->rp = fit >= 4 ? 4 : fit >= 2 ? 2 : 1;
    }
    c->q_stage = c->tr * nchunks * 16;
    const uint32_t s_stage = (c->tr * nb * 2 + 32 + 15) / 16 * 16;
    c->stage_bytes = (c->q_stage + s_stage + 127) / 128 * 128;
    const size_t fixed = kRedBufs * c->tr * c->ncw * sizeof(float) + (2 * 16 + 2 * kRedBufs + 1) * sizeof(uint64_t);
    const uint32_t tiles = (max_tiles_hint_rows + c->tr - 1) / c->tr;
    // Measured on B200: two CTAs per SM pay off once every CTA slot streams many tiles; short
    // launches do better with one CTA per SM, which also balances their few tiles better.  The
    // ring stays at two stages by default so that a CTA takes well under half of the SM's
    // shared memory: the next kernel of a dependent-launch chain can then become resident and
    // prefetch its first tiles while this one is still running.
    int64_t per_sm = option(ctx, "gemv.ctas_per_sm", 0);
    if (per_sm <= 0) per_sm = tiles >= 16u * (uint32_t)ctx->sm_count ? 2 : 1;
    // One flagged CTA per SM.  Its blocks wait on each other's rows by re-reading memory, and a block that
    // spins next to a working one on the same SM takes its issue slots: with two per SM (the kernel fits in 86
    // registers when asked) a fully dependent chained product measured 104 us instead of 18 us.
    if (flagged) per_sm = 1;
    per_sm = std::min<int64_t>(per_sm, 4);
    const size_t budget = (size_t)(200 * 1024) / (size_t)per_sm - fixed;
    // (Also for flagged lists, whose CTAs have the SM to themselves: with a ring of six stages, a block's whole
    // share of a product prefetched while it waits for x, a chained 14336-row product took 85 us instead of
    // 17.6 us on two GPUs.  The prefetch traffic of future products queues ahead of the exchange's stores and polls.)
    int64_t want_stages = option(ctx, "gemv.stages", 0);
    if (want_stages <= 0) want_stages = 2;
    uint32_t stages = (uint32_t)std::min<size_t>(16, budget / c->stage_bytes);
    stages = std::min<uint32_t>(stages, (uint32_t)want_stages);
    if (stages < 2) {
        // a long row: give one CTA the whole SM
        per_sm = 1;
        stages = (uint32_t)std::min<size_t>(2, ((size_t)(227 * 1024) - 1024 - fixed) / c->stage_bytes);
        if (stages < 2) return false;
    }
    c->stages = stages;
    c->per_sm = per_sm;
    c->smem = (size_t)stages * c->stage_bytes + fixed;
    return true;
}

// Tiles of 8 rows (or what "gemv.tile_rows" asks for); rows too long for two stages of those (beyond about
// 28 000 Q4_0 / 14 000 Q8_0 weights) take tiles of 4 rows.
bool choose_config(vx_context* ctx, uint32_t nchunks, uint32_t nb, uint32_t max_tiles_hint_rows, bool flagged,
                   StreamConfig* c) {
    const uint32_t first = vx::option(ctx, "gemv.tile_rows", 8) == 4 ? 4 : 8;
    if (choose_config_tr(ctx, first, nchunks, nb, max_tiles_hint_rows, flagged, c)) return true;
    return first == 8 && choose_config_tr(ctx, 4, nchunks, nb, max_tiles_hint_rows, flagged, c);
}

void fill_common(StreamParams* p, const StreamConfig& c, uint32_t nchunks, uint32_t nb, vx_context* ctx) {
    p->nchunks = nchunks;
    p->nb = nb;
    p->tpr = c.tpr;
    p->stages = c.stages;
    p->stage_bytes = c.stage_bytes;
    p->q_stage_bytes = c.q_stage;
    p->status = ctx->d_status;
    p->wait_cycles = vx::wait_cycles(ctx);
#ifdef VX_TIMELINE
    p->timeline = reinterpret_cast<unsigned long long*>(vx::option(ctx, "debug.timeline_ptr", 0));
#endif
}

// Which rows of a producing entry a reading entry waits for, and whether that covers every thread block.
//
// A flagged reader only waits for the elements it reads.  A block of the PRODUCING entry none of whose rows
// are among them is never waited for: it may still be reading its own x (the vector written two entries
// ago) when a faster rank, already one entry further, writes that vector again.  A chain over two vectors
// is therefore only safe when every block that takes part in the producing entry owns at least one awaited
// row: nobody can then run ahead of a block that has not finished reading.  Tiles are dealt out to blocks
// in turn (see first_tile), so the test is per block, and a grid that fails it is shrunk until it passes.
struct AwaitedRows {
    // element e of the vector is awaited iff awaited(e); rows of the producer map to elements row0 + r * stride
    uint64_t cols = 0, seg_len = 0, seg_stride = 0, seg_first = 0;
    bool awaited(uint64_t e) const {
        if (seg_len == 0) return e < cols;
        const uint64_t s = e / seg_stride, o = e % seg_stride;
        return s < cols / seg_len && o >= seg_first && o < seg_first + seg_len;
    }
};

// true when, with `grid` blocks and tiles of `tr` rows, every block that has a tile of producer entry
// `op_index` (nrows rows, row r at element y_row0 + r * y_stride) also has a tile with an awaited row.
bool every_block_awaited(const AwaitedRows& a, uint32_t op_index, uint32_t nrows, uint64_t y_row0, uint64_t y_stride,
                         uint32_t tr, uint32_t grid) {
    const uint32_t tiles = (nrows + tr - 1) / tr;
    const uint32_t rot = (uint32_t)(((uint64_t)op_index * (tiles % grid)) % grid);
    std::vector<uint8_t> seen(grid, 0);
    for (uint32_t t = 0; t < tiles; ++t) {
        bool hit = false;
        for (uint32_t r = t * tr; r < std::min(nrows, (t + 1) * tr) && !hit; ++r) hit = a.awaited(y_row0 + (uint64_t)r * y_stride);
        if (hit) seen[(t + rot) % grid] = 1;
    }
    const uint32_t taking_part = std::min(tiles, grid);
    uint32_t covered = 0;
    for (uint32_t b = 0; b < grid; ++b) {
        const uint32_t first = (b + grid - rot) % grid;   // first_tile of block b
        if (first < tiles && seen[b]) ++covered;
    }
    return covered == taking_part;
}

void fill_plain_op(OpParams* o, const vx_qweights* w, size_t row0, uint32_t nrows, const float* x, float* y,
                   float* const* y_peer, uint32_t n_peer) {
    *o = OpParams{};
    o->quants = w->d_quants;
    o->scales = reinterpret_cast<const uint8_t*>(w->d_scales);
    o->row0 = row0;
    o->nrows = nrows;
    o->x = x;
    o->x_aligned = (reinterpret_cast<uintptr_t>(x) & 15u) == 0 ? 1u : 0u;
    o->y = y;
    o->n_peer = std::min<uint32_t>(n_peer, vx::kMaxPeers);
    for (uint32_t d = 0; d < o->n_peer; ++d) o->y_peer[d] = y_peer[d];
    o->x_vec = -1;
    o->y_vec = -1;
    o->y_pair_stride = 1;
}

}  // namespace

// A list of GEMVs prepared for one launch.
struct vx_gemv_batch {
    int device = 0;
    int qtype = 0;
    bool flagged = false;
    StreamConfig cfg{};
    StreamParams params{};
    dim3 grid;
    OpParams* d_ops = nullptr;
    size_t n_ops = 0;
};

namespace vx {

// `batch` vectors (at most kInlineOps; more than one only without peers or exchange) in one launch:
// a list whose entries share the weights, so that the later vectors find them in L2 when the
// matrix fits there.  *eligible = false (nothing launched) when the row is too long for the
// shared-memory ring or the register-resident x.
vx_status launch_gemv_stream(vx_context* ctx, const vx_qweights* w, size_t row0, uint32_t nrows,
                             const float* x, float* y, float* const* y_peer, uint32_t n_peer,
                             const Exchange* xch, bool* eligible, uint32_t batch, size_t x_stride,
                             size_t y_stride) {
    *eligible = false;
    const uint32_t nb = (uint32_t)w->blocks_per_row;
    const uint32_t nchunks = (uint32_t)(w->quant_row_bytes / 16);
    const bool flagged = xch && (xch->x_vec || xch->y_vec);
    StreamConfig c;
    if (batch < 1 || batch > (uint32_t)kInlineOps || (batch > 1 && (flagged || n_peer))) return VX_OK;
    if (!choose_config(ctx, nchunks, nb, nrows * batch, flagged, &c)) return VX_OK;

    StreamParams p{};
    fill_common(&p, c, nchunks, nb, ctx);
    p.n_ops = batch;
    OpParams& o = p.inline_ops[0];
    for (uint32_t v = 0; v < batch; ++v)
        fill_plain_op(&p.inline_ops[v], w, row0, nrows, x + v * x_stride, y + v * y_stride, y_peer, n_peer);
    if (flagged) {
        // vector table: the written vector first (its header carries the retire counter)
        if (xch->y_vec) {
            o.y_vec = (int32_t)p.n_vec;
            p.vec_hdr[p.n_vec] = static_cast<uint32_t*>(xch->y_vec);
            p.vec_writes[p.n_vec++] = 1;
            o.y_gen_add = 1;
            auto pairs = [&](void* base) {
                return reinterpret_cast<uint64_t*>(static_cast<uint8_t*>(base) + kExchangeHeader) + xch->y_row0;
            };
            o.y_pairs = pairs(xch->y_vec);
            o.y_pair_stride = (uint32_t)xch->y_stride;
            o.n_pair_peer = std::min<uint32_t>(xch->n_peers, kMaxPeers);
            for (uint32_t d = 0; d < o.n_pair_peer; ++d) o.y_pairs_peer[d] = pairs(xch->peer_y_vec[d]);
        }
        if (xch->x_vec) {
            // reading and writing one vector in the same GEMV is refused by the caller
            o.x_vec = (int32_t)p.n_vec;
            p.vec_hdr[p.n_vec] = const_cast<uint32_t*>(static_cast<const uint32_t*>(xch->x_vec));
            p.vec_writes[p.n_vec++] = 0;
            o.x_gen_add = 0;
            o.x_pairs = reinterpret_cast<const uint64_t*>(static_cast<const uint8_t*>(xch->x_vec) + kExchangeHeader);
        }
    }

    const uint32_t tiles = (nrows + c.tr - 1) / c.tr;
    const uint32_t slots = (uint32_t)std::max<int64_t>(1, ctx->sm_count * c.per_sm);
    dim3 grid(std::min(tiles, slots));
    if (flagged && xch->y_vec) {
        // The next link of the chain reads the first `cols` elements of the vector written here (every rank
        // issues the same launches on matrices of one shape).  Every block of this grid must own one of those
        // rows, or nobody ever waits for it and a faster rank could rewrite the vector it still reads as x.
        AwaitedRows a;
        a.cols = w->cols;
        uint32_t g = grid.x;
        while (g > 1 && !every_block_awaited(a, 0, nrows, xch->y_row0, xch->y_stride, c.tr, g)) --g;
        if (!every_block_awaited(a, 0, nrows, xch->y_row0, xch->y_stride, c.tr, g))
            return fail(VX_ERR_UNSUPPORTED,
                        "vx_gemv_q_rows_exchange: none of rows [%zu, +%u) (stride %zu) lies among the first %zu elements "
                        "the next link reads, so no rank would ever wait for this one; deal the rows out in turn "
                        "(y_stride = world) or use a list with a windowed x",
                        xch->y_row0, nrows, xch->y_stride, w->cols);
        grid.x = g;
    }
    const vx_status st = flagged ? launch_tr<true>(ctx, w->type, c, p, grid) : launch_tr<false>(ctx, w->type, c, p, grid);
    if (st != VX_OK) return st;
    ctx->launches++;
    ctx->status_dirty = true;
    *eligible = true;
    return VX_OK;
}

}  // namespace vx

extern "C" {

vx_status vx_gemv_batch_create(vx_context* ctx, const vx_gemv_op* ops, size_t n_ops, vx_gemv_batch** out) {
    using vx::fail;
    VX_REQUIRE(ctx && ops && out && n_ops >= 1, VX_ERR_INVALID_ARGUMENT, "vx_gemv_batch_create: null or empty argument");
    *out = nullptr;
    VX_REQUIRE(n_ops <= 4096, VX_ERR_INVALID_ARGUMENT, "at most 4096 GEMVs in a list (%zu given)", n_ops);
    const vx_qweights* w0 = ops[0].w;
    VX_REQUIRE(w0, VX_ERR_INVALID_ARGUMENT, "GEMV 0 has no weights");
    std::unique_ptr<vx_gemv_batch> b(new vx_gemv_batch());
    b->device = ctx->device;
    b->qtype = w0->type;
    b->n_ops = n_ops;
    std::vector<OpParams> host(n_ops);
    StreamParams& p = b->params;
    uint32_t max_rows = 0;
    auto vec_index = [&](const void* hdr) -> int32_t {
        for (uint32_t v = 0; v < p.n_vec; ++v)
            if (p.vec_hdr[v] == hdr) return (int32_t)v;
        if (p.n_vec == (uint32_t)kMaxVecs) return -1;
        p.vec_hdr[p.n_vec] = const_cast<uint32_t*>(static_cast<const uint32_t*>(hdr));
        p.vec_writes[p.n_vec] = 0;
        return (int32_t)p.n_vec++;
    };
    // Written vectors first, so that entry 0 (whose header carries the retire counter) is one this list owns.
    for (size_t i = 0; i < n_ops; ++i)
        if (ops[i].y_xvec) VX_REQUIRE(vec_index(ops[i].y_xvec) >= 0, VX_ERR_UNSUPPORTED, "more than %d exchange vectors", kMaxVecs);
    for (size_t i = 0; i < n_ops; ++i) {
        const vx_gemv_op& g = ops[i];
        VX_REQUIRE(g.w, VX_ERR_INVALID_ARGUMENT, "GEMV %zu has no weights", i);
        VX_REQUIRE(g.w->device == ctx->device, VX_ERR_INVALID_ARGUMENT, "weights of GEMV %zu live on device %d", i, g.w->device);
        VX_REQUIRE(g.w->type == w0->type && g.w->cols == w0->cols, VX_ERR_UNSUPPORTED,
                   "GEMV %zu: a list holds one quantisation type and one column count", i);
        VX_REQUIRE(g.row0 <= g.w->rows && g.nrows <= g.w->rows - g.row0 && g.nrows >= 1 && g.nrows <= 0xFFFFFFFFull,
                   VX_ERR_OUT_OF_BOUNDS, "GEMV %zu: rows [%zu, %zu) outside a matrix of %zu rows", i, g.row0,
                   g.row0 + g.nrows, g.w->rows);
        VX_REQUIRE(g.x_xvec || g.x, VX_ERR_INVALID_ARGUMENT, "GEMV %zu has no x", i);
        VX_REQUIRE(g.y || g.y_xvec, VX_ERR_INVALID_ARGUMENT, "GEMV %zu has no y", i);
        VX_REQUIRE(g.n_peers <= (size_t)vx::kMaxPeers && (g.n_peers == 0 || (g.y_xvec && g.peer_y_xvec)),
                   VX_ERR_INVALID_ARGUMENT, "GEMV %zu: peers need exchange vectors (at most %d)", i, vx::kMaxPeers);
        VX_REQUIRE(!g.y_xvec || g.x_xvec != g.y_xvec, VX_ERR_INVALID_ARGUMENT, "GEMV %zu reads the vector it writes", i);
        VX_REQUIRE((reinterpret_cast<uintptr_t>(g.x_xvec) & 15u) == 0 && (reinterpret_cast<uintptr_t>(g.y_xvec) & 15u) == 0,
                   VX_ERR_INVALID_ARGUMENT, "GEMV %zu: exchange vectors are 16-byte aligned", i);
        OpParams& o = host[i];
        VX_REQUIRE(g.n_peer_y <= (size_t)vx::kMaxPeers && (g.n_peer_y == 0 || (g.peer_y && g.y)), VX_ERR_INVALID_ARGUMENT,
                   "GEMV %zu: plain peer rows need y and at most %d buffers", i, vx::kMaxPeers);
        for (size_t d = 0; d < g.n_peer_y; ++d)
            VX_REQUIRE(g.peer_y[d], VX_ERR_INVALID_ARGUMENT, "GEMV %zu: peer buffer %zu is null", i, d);
        fill_plain_op(&o, g.w, g.row0, (uint32_t)g.nrows, g.x_xvec ? nullptr : g.x, g.y, g.peer_y, (uint32_t)g.n_peer_y);
        if (g.x_xvec) {
            const int32_t v = vec_index(g.x_xvec);
            VX_REQUIRE(v >= 0, VX_ERR_UNSUPPORTED, "more than %d exchange vectors", kMaxVecs);
            o.x_vec = v;
            o.x_gen_add = p.vec_writes[v];  // writes by the GEMVs before this one
            o.x_pairs = reinterpret_cast<const uint64_t*>(static_cast<const uint8_t*>(g.x_xvec) + vx::kExchangeHeader);
            VX_REQUIRE(g.x_seg_len == 0 || (g.x_seg_len % 32 == 0 && g.x_seg_first % 2 == 0 &&
                                            g.x_seg_first + g.x_seg_len <= g.x_seg_stride && g.x_seg_stride % 2 == 0 &&
                                            g.x_seg_stride <= 0xFFFFFFFFull && g.w->cols % g.x_seg_len == 0),
                       VX_ERR_INVALID_ARGUMENT, "GEMV %zu: x window of %zu elements from %zu, every %zu", i, g.x_seg_len,
                       g.x_seg_first, g.x_seg_stride);
            o.x_seg_len = (uint32_t)g.x_seg_len;
            o.x_seg_stride = (uint32_t)g.x_seg_stride;
            o.x_seg_first = (uint32_t)g.x_seg_first;
            b->flagged = true;
        }
        if (g.y_xvec) {
            const int32_t v = vec_index(g.y_xvec);
            o.y_vec = v;
            o.y_gen_add = ++p.vec_writes[v];
            VX_REQUIRE(g.y_stride >= 1 && g.y_stride <= 0xFFFFu, VX_ERR_INVALID_ARGUMENT, "GEMV %zu: element stride %zu", i, g.y_stride);
            auto pairs = [&](void* base) {
                return reinterpret_cast<uint64_t*>(static_cast<uint8_t*>(base) + vx::kExchangeHeader) + g.y_row0;
            };
            o.y_pairs = pairs(g.y_xvec);
            o.y_pair_stride = (uint32_t)g.y_stride;
            o.n_pair_peer = (uint32_t)g.n_peers;
            for (size_t d = 0; d < g.n_peers; ++d) {
                VX_REQUIRE(g.peer_y_xvec[d] && (reinterpret_cast<uintptr_t>(g.peer_y_xvec[d]) & 15u) == 0,
                           VX_ERR_INVALID_ARGUMENT, "GEMV %zu: exchange vector of peer %zu is null or misaligned", i, d);
                o.y_pairs_peer[d] = pairs(g.peer_y_xvec[d]);
            }
            b->flagged = true;
        }
        max_rows = std::max<uint32_t>(max_rows, (uint32_t)g.nrows);
    }
    const uint32_t nb = (uint32_t)w0->blocks_per_row;
    const uint32_t nchunks = (uint32_t)(w0->quant_row_bytes / 16);
    // A list streams like one long GEMV: size the launch for the sum of its rows.
    uint64_t total_rows = 0;
    for (size_t i = 0; i < n_ops; ++i) total_rows += ops[i].nrows;
    VX_REQUIRE(choose_config(ctx, nchunks, nb, (uint32_t)std::min<uint64_t>(total_rows, 0xFFFFFFFFull), b->flagged, &b->cfg),
               VX_ERR_UNSUPPORTED, "rows of %zu columns do not fit the streaming kernel", w0->cols);
    fill_common(&p, b->cfg, nchunks, nb, ctx);
    p.n_ops = (uint32_t)n_ops;
    const uint32_t tiles = (max_rows + b->cfg.tr - 1) / b->cfg.tr;
    const uint32_t slots = (uint32_t)std::max<int64_t>(1, ctx->sm_count * b->cfg.per_sm);
    b->grid = dim3(std::min(tiles, slots));
    if (b->flagged) {
        // Every flagged read must wait for at least one row of every block of the entry that produces the
        // vector (see AwaitedRows); the producer of entry i's x is the latest earlier entry that writes the
        // vector, or, for a list that is launched again and again, the last one of the list that does.
        auto producer_of = [&](size_t i) -> long {
            for (size_t j = i; j-- > 0;)
                if (ops[j].y_xvec == ops[i].x_xvec) return (long)j;
            for (size_t j = n_ops; j-- > i + 1;)
                if (ops[j].y_xvec == ops[i].x_xvec) return (long)j;
            return -1;   // written outside this list
        };
        auto safe = [&](uint32_t g, size_t* reader, size_t* producer) {
            for (size_t i = 0; i < n_ops; ++i) {
                if (!ops[i].x_xvec) continue;
                const long j = producer_of(i);
                if (j < 0) continue;
                AwaitedRows a;
                a.cols = ops[i].w->cols;
                a.seg_len = ops[i].x_seg_len;
                a.seg_stride = ops[i].x_seg_stride;
                a.seg_first = ops[i].x_seg_first;
                if (!every_block_awaited(a, (uint32_t)j, (uint32_t)ops[j].nrows, ops[j].y_row0, ops[j].y_stride, b->cfg.tr, g)) {
                    *reader = i;
                    *producer = (size_t)j;
                    return false;
                }
            }
            return true;
        };
        size_t reader = 0, producer = 0;
        uint32_t g = b->grid.x;
        while (g > 1 && !safe(g, &reader, &producer)) --g;
        VX_REQUIRE(safe(g, &reader, &producer), VX_ERR_UNSUPPORTED,
                   "GEMV %zu reads none of the rows this rank produces in GEMV %zu, so no rank would ever wait for "
                   "this one and the vectors could be rewritten under it: give x a window over every rank's slab "
                   "(x_seg_*) or deal the rows out in turn (y_stride = world)", reader, producer);
        b->grid.x = g;
    }
    // few tiles per block and product: the blocks mostly wait for each other, let one warp do it
    const int64_t bw = vx::option(ctx, "gemv.block_wait", -1);
    p.block_wait = bw >= 0 ? (bw != 0) : (tiles < 5 * b->grid.x ? 1u : 0u);
    vx::DeviceGuard guard(ctx->device);
    if (n_ops <= (size_t)kInlineOps) {
        for (size_t i = 0; i < n_ops; ++i) p.inline_ops[i] = host[i];
    } else {
        VX_CUDA(vx::device_malloc(ctx, reinterpret_cast<void**>(&b->d_ops), n_ops * sizeof(OpParams)));
        const cudaError_t e = cudaMemcpy(b->d_ops, host.data(), n_ops * sizeof(OpParams), cudaMemcpyHostToDevice);
        if (e != cudaSuccess) {
            cudaFree(b->d_ops);
            return fail(VX_ERR_CUDA, "uploading the GEMV list: %s", cudaGetErrorString(e));
        }
        p.ops = b->d_ops;
    }
    *out = b.release();
    return VX_OK;
}

vx_status vx_gemv_batch_launch(vx_context* ctx, const vx_gemv_batch* b) {
    using vx::fail;
    VX_REQUIRE(ctx && b, VX_ERR_INVALID_ARGUMENT, "vx_gemv_batch_launch: null argument");
    VX_REQUIRE(b->device == ctx->device, VX_ERR_INVALID_ARGUMENT, "the list was made for device %d", b->device);
    vx::DeviceGuard guard(ctx->device);
    StreamParams p = b->params;
    p.status = ctx->d_status;
    p.wait_cycles = vx::wait_cycles(ctx);
#ifdef VX_TIMELINE
    p.timeline = reinterpret_cast<unsigned long long*>(vx::option(ctx, "debug.timeline_ptr", 0));
#endif
    const StreamConfig& c = b->cfg;
    const vx_status st = b->flagged ? launch_tr<true>(ctx, b->qtype, c, p, b->grid) : launch_tr<false>(ctx, b->qtype, c, p, b->grid);
    if (st != VX_OK) return st;
    ctx->launches++;
    ctx->status_dirty = true;
    return VX_OK;
}

vx_status vx_gemv_batch_free(vx_context* ctx, vx_gemv_batch* b) {
    using vx::fail;
    VX_REQUIRE(ctx, VX_ERR_INVALID_ARGUMENT, "vx_gemv_batch_free: null context");
    if (!b) return VX_OK;
    vx::DeviceGuard guard(ctx->device);
    VX_CUDA(cudaStreamSynchronize(ctx->stream));
    if (b->d_ops) cudaFree(b->d_ops);
    delete b;
    return VX_OK;
}

}  // extern "C"
