// Batched GEMV for block-quantised weights on the tensor cores: up to eight activation vectors per pass
// over the weights, every weight byte read from HBM once.
//
// With one vector the streaming kernel (vx_gemv_stream.cu) does its dot products with dp4a on the integer
// pipe, which is already 60 % busy at HBM speed; eight vectors would need eight passes over the weights.
// Here the block sums are integer matrix products instead: per 32-weight block,
//     S[row, vec] = sum_i q[row, i] * X[vec, i]
// is an m16 n8 k32 tensor-core MMA on the raw quants (A, 16 rows) and on x held as fixed point (B, 8
// columns).  x is split into three signed byte planes (balanced digits: X = 65536 a + 256 b + c with
// a, b, c in [-128, 127]), and the block's f16 scale is applied to the exact integer sums in f32, as in
// the streaming kernel.  Two forms:
//   FULL    3 to 8 vectors: the 8 columns are 8 vectors, one MMA per plane, and the three int32 results
//           are recombined exactly (65536 sa + 256 sb + sc) before the scale is applied;
//   SINGLE  1 or 2 vectors: the 8 columns are (vector, plane) pairs, ONE MMA per block; every column keeps
//           its own f32 sum and the planes are added, with their weights 65536 / 256 / 1, at the end.
//
//   * A pre-pass kernel turns the batch's x into the planes ONCE, in the register layout the MMA wants for
//     its B operand, in scratch memory of the context: per 32 columns 3 (FULL) or 1 (SINGLE) planes of
//     32 lanes x 8 bytes, then, for Q4_0, -8 * sum X per column (the "- 8" of the format, added to the
//     accumulator's initial value).
//     X is fixed point relative to the largest |x| of its vector inside a slice of 32 * NBW columns
//     (256 for the usual shapes): |X| < 2^22 for Q4_0 and < 2^19 for Q8_0, so that a block's recombined
//     sum still fits 32 bits.  The slice sums are scaled by the slice's factor in f32.
//   * The main kernel is persistent, one CTA per SM: producer thread (one tiled TMA load per 16-row tile,
//     128-byte swizzle so that fragment loads hit 32 different banks) and 8 consumer warps.
//     A CTA owns whole rows.  The planes (25 bytes per column, 9 in the SINGLE form) must sit in its shared
//     memory, so the columns are walked in PHASES of one column tile (32 NBW x 8 warps columns): the tile's
//     planes sit in one of two slots (the next phase's arrive meanwhile), the tile is streamed for all the
//     CTA's row tiles (at most `sg_units` of them at a time: a pass), their sums wait in shared memory, and
//     so on; the last phase writes y.  No sums cross CTAs.  The 8 warps of a CTA split a tile's columns
//     further and keep their B fragments in registers for the whole pass.
//   * One launch walks up to 8 matrices of one type and column count that share the vectors (their row tiles
//     are numbered through and dealt out evenly); the planes are made once for all of them.
//   * Partial sums meet in shared memory: every consumer thread leaves its four sums of a row tile there (its
//     own 16 bytes, no synchronisation per tile); at the end of a pass over the set's row tiles the warps add
//     them up, the 8 warps of a CTA and then the phases, both in a fixed order.  (A hand-off of every tile to an
//     epilogue warp through barriers cost a fifth of a tile visit.)
// Measured on B200 while building this (they shaped the design): an SM completes about one untiled bulk
// copy per 75 cycles whatever its size, and one thread issues one per 450, so row-by-row copies of 1 KB
// top out near 3 TB/s (hence one tiled load per tile); mma.sync m16n8k32 s8 has 20 cycles latency and a
// rate of one per 8 cycles per SM sub-partition, far from limiting; splitting the columns over CTAs that
// exchange sums through global memory cost a GPU-scope fence per row tile (it doubled the kernel's time) or,
// with tagged 64-bit pairs instead of fences, CTAs that wait for each other and must start together (no
// early start under the launch before).  What limits the kernel now is the integer epilogue of every
// block (unpack, recombine, convert, scale): the consumers wait for data less than a tenth of their time.
// All waits are bounded (see vx_sm100.cuh).
#include <cuda.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <atomic>
#include <vector>

#include "vx_internal.h"
#include "vx_sm100.cuh"

namespace {

using namespace sm100;

constexpr int kVecs = 8;                 // vectors per pass (the MMA's n)
constexpr int kUnitRows = 16;            // rows per tile (the MMA's m)
constexpr uint32_t kAccUnit = 8 * 32 * 16;   // bytes of partial sums per row tile: a float4 per consumer thread
constexpr uint32_t kPartUnit = 32 * 16;      // bytes of sums between phases per row tile: a float4 per lane
enum { SINGLE = 0, FULL = 1 };
// Consumer warps per CTA.  (16 warps of 4 blocks each measured no faster than 8 warps of 8 in the FULL form:
// 2.65 against 2.85 TB/s on 28672 x 4096 Q4_0.)
constexpr int kWarps = 8;
constexpr int kMaxStages = 8;
// bytes of planes per 32 columns: 3 (FULL) or 1 (SINGLE) x 256, then 8 x int32
__host__ __device__ constexpr uint32_t block_planes(int mode) { return mode == FULL ? 800u : 288u; }

constexpr int kMaxMats = 8;              // matrices one launch walks (they share the vectors)

// The matrices of a launch: their row tiles are numbered through, matrix after matrix.
struct MmaMat {
    float* y;
    uint32_t row0;                // first row of the slab inside its matrix
    uint32_t nrows;
    uint32_t unit0;               // number of the slab's first row tile
};

struct MmaMaps {
    CUtensorMap q[kMaxMats], s[kMaxMats];
};

struct MmaParams {
    MmaMat mat[kMaxMats];
    uint32_t n_mats;
    uint32_t units;               // row tiles of all the matrices
    uint32_t nb;                  // blocks per row
    uint32_t phases;              // column tiles of 32 NBW kWarps columns, walked one after the other
    uint32_t slot_bytes;          // shared memory per slot of planes (a column tile's planes, then its slice factors)
    uint32_t sg_units;            // row tiles whose sums wait in shared memory between phases
    uint32_t stages, stage_bytes, s_off;
    uint32_t ring_off;            // offset of the ring in shared memory (1024-byte aligned: the swizzle works on address bits)
    const uint8_t* planes;        // [nb][block_planes(MODE)]
    const float* sx;              // [slices][kVecs]: per column, the factor its slice sums are scaled by
    uint64_t y_stride;
    uint32_t batch;
    vx::DeviceStatus* status;
};

__device__ __forceinline__ void report(vx::DeviceStatus* st, uint32_t code) {
    volatile vx::DeviceStatus* v = st;
    v->detail = blockIdx.x;
    v->code = code;
    __threadfence_system();
}

// D = A * B + C, A 16 x 32 bytes (row; unsigned nibbles of Q4_0 or signed bytes of Q8_0), B 32 x 8 signed
// bytes (col), int32 accumulators.
template <bool A_SIGNED>
__device__ __forceinline__ void mma_i8(int (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1, const int (&c)[4]) {
    if constexpr (A_SIGNED)
        asm("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
    else
        asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
                     : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(c[0]), "r"(c[1]), "r"(c[2]), "r"(c[3]));
}

// ------------------------------------------------------------------------ pre-pass ----
// One CTA per slice of 32 * NBW columns, one warp per column of the MMA's B operand: a vector (FULL), or a
// (vector, plane) pair (SINGLE: column n is plane n % 3 of vector n / 3).  Word w of the slice (4 matrix
// columns) belongs to block w / 8; inside the block, words 0..3 are the first B register of lanes t = 0..3
// and words 4..7 the second one (the MMA's k = 4 t + i and 16 + 4 t + i).
template <int QT, int MODE>
__global__ void __launch_bounds__(256) xplanes_kernel(const float* __restrict__ x, uint64_t x_stride, uint32_t batch,
                                                      uint32_t nbw, uint8_t* __restrict__ planes, float* __restrict__ sx) {
    // Programmatic dependent launch on both sides: the main kernel may become resident and start streaming
    // weights while this one runs (it reads the planes only after this grid has completed), and this grid
    // may start under the tail of the kernel before it, whose output x may be and whose planes these are.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
    constexpr float kXMax = QT == 1 ? 4194302.0f : 524286.0f;
    constexpr uint32_t kBP = block_planes(MODE);
    const uint32_t slice = blockIdx.x, col = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t vec = MODE == FULL ? col : col / 3, plane = col % 3;
    const uint32_t words = 8 * nbw;                  // 4-column words per slice: 8 .. 64
    const bool live = vec < batch && (MODE == FULL || col < 6);
    const float* src = x + (size_t)vec * x_stride + (size_t)slice * 32 * nbw;
    const bool aligned = (reinterpret_cast<uintptr_t>(src) & 15u) == 0;
    float v[2][4];
    float amax = 0.0f, poison = 0.0f;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint32_t w = lane + 32 * r;
#pragma unroll
        for (int i = 0; i < 4; ++i) v[r][i] = 0.0f;
        if (live && w < words) {
            if (aligned) {
                const float4 f = __ldg(reinterpret_cast<const float4*>(src) + w);
                v[r][0] = f.x; v[r][1] = f.y; v[r][2] = f.z; v[r][3] = f.w;
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) v[r][i] = __ldg(src + 4 * w + i);
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            amax = fmaxf(amax, fabsf(v[r][i]));
            poison = fmaf(v[r][i], 0.0f, poison);
        }
    }
    for (int off = 16; off > 0; off >>= 1) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
        poison += __shfl_xor_sync(0xffffffffu, poison, off);
    }
    // a slice whose values are all tiny: scale it up by an exact power of two first, so that neither the
    // quotient below nor its inverse leaves the normal range
    const bool tiny = amax < 1.0e-20f;
    if (tiny) {
        amax *= 0x1p64f;
#pragma unroll
        for (int r = 0; r < 2; ++r)
#pragma unroll
            for (int i = 0; i < 4; ++i) v[r][i] *= 0x1p64f;
    }
    float inv = amax > 0.0f ? kXMax / amax : 0.0f;
    float s = amax / kXMax;
    if (tiny) s *= 0x1p-64f;
    if (poison != poison) { inv = 0.0f; s = poison; }                                // NaN or infinity in x: NaN in y
    if (lane == 0) {
        const float weight = MODE == FULL ? 1.0f : plane == 0 ? 65536.0f : plane == 1 ? 256.0f : 1.0f;
        sx[(size_t)slice * kVecs + col] = live ? s * weight : 0.0f;
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint32_t w = lane + 32 * r;
        // balanced digits: X = 65536 a + 256 b + c, every digit a signed byte
        uint32_t da = 0, db = 0, dc = 0;
        int sum = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int X = __float2int_rn(v[r][i] * inv);
            const int c = (int)(int8_t)(X & 0xFF);
            const int X1 = (X - c) >> 8;
            const int b = (int)(int8_t)(X1 & 0xFF);
            const int a = (X1 - b) >> 8;
            da |= (uint32_t)(a & 0xFF) << (8 * i);
            db |= (uint32_t)(b & 0xFF) << (8 * i);
            dc |= (uint32_t)(c & 0xFF) << (8 * i);
            sum += MODE == FULL ? X : plane == 0 ? a : plane == 1 ? b : c;
        }
        // the 8 words of a block sit in 8 consecutive lanes
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        sum += __shfl_xor_sync(0xffffffffu, sum, 4);
        if (w < words) {
            const uint32_t blk = slice * nbw + w / 8, q = w & 7, t = q & 3, reg = q >> 2;
            uint8_t* base = planes + (size_t)blk * kBP;
            const uint32_t at = ((col * 4 + t) * 2 + reg) * 4;     // lane (col, t) of the MMA, register `reg`
            if (MODE == FULL) {
                *reinterpret_cast<uint32_t*>(base + at) = da;
                *reinterpret_cast<uint32_t*>(base + 256 + at) = db;
                *reinterpret_cast<uint32_t*>(base + 512 + at) = dc;
            } else {
                *reinterpret_cast<uint32_t*>(base + at) = plane == 0 ? da : plane == 1 ? db : dc;
            }
            if (q == 0) *reinterpret_cast<int*>(base + (kBP - 32) + col * 4) = QT == 1 && live ? -8 * sum : 0;
        }
    }
}

// ------------------------------------------------------------------------ main kernel ----
// Work of a CTA: row tiles [u0, u1), walked `sg_units` at a time; per such set every phase (column tile),
// and inside a phase the set's row tiles.  Producer and consumers walk the same order.
__device__ __forceinline__ void my_units(const MmaParams& p, uint32_t* u0, uint32_t* u1) {
    *u0 = (uint32_t)((uint64_t)p.units * blockIdx.x / gridDim.x);
    *u1 = (uint32_t)((uint64_t)p.units * (blockIdx.x + 1) / gridDim.x);
}
// The matrix row tile `u` belongs to (tiles are numbered matrix after matrix).
__device__ __forceinline__ uint32_t mat_of(const MmaParams& p, uint32_t u) {
    uint32_t m = 0;
    while (m + 1 < p.n_mats && u >= p.mat[m + 1].unit0) ++m;
    return m;
}

template <int QT, int NBW, int MODE>
__global__ void __launch_bounds__(kWarps * 32 + 32, 1)
gemv_mma_kernel(const __grid_constant__ MmaParams p, const __grid_constant__ MmaMaps maps) {
    constexpr int QB = QT == 1 ? 16 : 32;   // bytes of quants per block
    constexpr int NP = MODE == FULL ? 3 : 1;
    constexpr uint32_t kBP = block_planes(MODE);
    constexpr uint32_t kt_blocks = NBW * kWarps;             // blocks per column tile
    constexpr uint32_t q_tile_bytes = kt_blocks * QB;        // quants per row and tile
    constexpr uint32_t plane_bytes = kt_blocks * kBP;        // planes of a column tile
    constexpr uint32_t sx_bytes = kWarps * kVecs * 4;        // [kWarps][kVecs] slice factors of a column tile
    constexpr bool S_SWZ = kt_blocks == 64;   // the scales of a tile are 128 bytes per row: swizzled like the quants
    extern __shared__ __align__(128) uint8_t smem_raw[];
    // the swizzle of the tiled copies works on shared-memory address bits: start the layout on a 1024-byte boundary
    uint8_t* smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    // [2 slots of planes + slice factors][ring][partial sums of the set's row tiles][sums between phases][barriers]
    uint8_t* ring = smem + p.ring_off;
    float4* s_acc = reinterpret_cast<float4*>(ring + (size_t)p.stages * p.stage_bytes);   // [sg_units][kWarps][32]
    float4* s_part = s_acc + (size_t)p.sg_units * kWarps * 32;                             // [sg_units][32], if phases > 1
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_part + (p.phases > 1 ? (size_t)p.sg_units * 32 : 0));
    const uint32_t bar0 = smem_addr(bars);
    auto full = [&](uint32_t s) { return bar0 + 8u * s; };
    auto empty = [&](uint32_t s) { return bar0 + 8u * (kMaxStages + s); };
    auto planes_bar = [&](uint32_t slot) { return bar0 + 8u * (2 * kMaxStages + slot); };
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 2 * kMaxStages + 2);

    const uint32_t tid = threadIdx.x;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (tid == 0) {
        *abort_flag = 0u;
        for (uint32_t s = 0; s < p.stages; ++s) {
            mbar_init(full(s), 1);
            mbar_init(empty(s), kWarps);
        }
        mbar_init(planes_bar(0), 1);
        mbar_init(planes_bar(1), 1);
        mbar_init_fence();
    }
    __syncthreads();

    uint32_t u0, u1;
    my_units(p, &u0, &u1);

    if (tid >= kWarps * 32) {
        // ------------------------------------------------------------ producer warp ----
        // One thread, two tiled TMA loads per stage: the tile's quants as a box of 128 bytes x 16 rows x the
        // tile's 128-byte column chunks (shared memory: [chunk][row][128 bytes], 128-byte swizzle, so that the
        // eight rows a fragment load touches sit in eight different bank groups), and its scales.  Rows beyond
        // the matrix read as zeros.  (Row-by-row bulk copies of 1 KB do not keep up: an SM completes about
        // one bulk copy per 75 cycles whatever its size.)
        if (tid == kWarps * 32) {
            for (uint32_t m = 0; m < p.n_mats; ++m) {
                tma_prefetch_desc(&maps.q[m]);
                tma_prefetch_desc(&maps.s[m]);
            }
            uint32_t s = 0, use = 0;                         // ring stage and how often it has been filled before
            for (uint32_t sg0 = u0; sg0 < u1; sg0 += p.sg_units) {
                const uint32_t sg1 = min(sg0 + p.sg_units, u1);
                for (uint32_t ph = 0; ph < p.phases; ++ph) {
                    const uint32_t blk0 = ph * kt_blocks;                  // first block of the tile in the row
                    for (uint32_t u = sg0; u < sg1; ++u) {
                        if (use > 0 && !mbar_wait(empty(s), (use - 1) & 1, abort_flag)) report(p.status, 41);
                        const uint32_t m = mat_of(p, u);
                        const int32_t row = (int32_t)(p.mat[m].row0 + (u - p.mat[m].unit0) * kUnitRows);
                        const uint32_t dst = smem_addr(ring + (size_t)s * p.stage_bytes);
                        mbar_arrive_expect_tx(full(s), kUnitRows * (q_tile_bytes + (S_SWZ ? 128u : kt_blocks * 2)));
                        tma_load_3d(dst, &maps.q[m], 0, row, (int32_t)(blk0 * QB / 128), full(s));
                        tma_load_2d(dst + p.s_off, &maps.s[m], (int32_t)(blk0 * 2), row, full(s));
                        if (++s == p.stages) {
                            s = 0;
                            ++use;
                        }
                    }
                }
            }
            // do not leave while copies into this CTA's shared memory may still be in flight: stage i has been
            // filled `use` times, once more if the last round reached it
            for (uint32_t i = 0; i < p.stages; ++i) {
                const uint32_t fills = use + (i < s ? 1u : 0u);
                if (fills > 0 && !mbar_wait(empty(i), (fills - 1) & 1, abort_flag)) report(p.status, 42);
            }
        }
        return;
    }

    // ---------------------------------------------------------------- consumer warps ----
    const uint32_t lane = tid & 31, warp = tid >> 5;
    const uint32_t g = lane >> 2, t = lane & 3;
    // The planes of a phase sit in one of two slots; the next phase's are fetched while this one is worked on.
    auto load_planes = [&](uint32_t ph, uint32_t slot) {
        uint8_t* dst = smem + (size_t)slot * p.slot_bytes;
        mbar_arrive_expect_tx(planes_bar(slot), plane_bytes + sx_bytes);
        bulk_g2s(smem_addr(dst), p.planes + (size_t)ph * plane_bytes, plane_bytes, planes_bar(slot));
        bulk_g2s(smem_addr(dst + plane_bytes), p.sx + (size_t)ph * (kWarps * kVecs), sx_bytes, planes_bar(slot));
    };
    // the planes are the pre-pass kernel's output: wait for it
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (tid == 0 && u0 < u1) load_planes(0, 0);

    uint32_t n = 0;                     // passes walked (a set of row tiles x a phase)
    uint32_t s = 0, s_par = 0;          // ring stage and the parity of its use
    for (uint32_t sg0 = u0; sg0 < u1; sg0 += p.sg_units) {
        const uint32_t sg1 = min(sg0 + p.sg_units, u1);
        for (uint32_t ph = 0; ph < p.phases; ++ph, ++n) {
            // Every consumer warp has left the pass before: its planes' slot may take the planes of the next
            // phase, and the partial sums it left in shared memory have been added up.
            if (n > 0) asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory");
            uint32_t slot = 0;
            if (p.phases > 1) {
                slot = n & 1;
                if (tid == 0) {
                    if (ph + 1 < p.phases) load_planes(ph + 1, slot ^ 1);
                    else if (sg1 < u1) load_planes(0, slot ^ 1);
                }
                if (!mbar_wait(planes_bar(slot), (n >> 1) & 1, abort_flag)) report(p.status, 45);
            } else if (n == 0) {
                if (!mbar_wait(planes_bar(0), 0, abort_flag)) report(p.status, 45);    // one phase: its planes stay
            }
            const uint8_t* s_planes = smem + (size_t)slot * p.slot_bytes;
            const float2 sxv = *reinterpret_cast<const float2*>(s_planes + plane_bytes + (warp * kVecs + 2 * t) * 4);
            {
                // this warp's B fragments for its NBW blocks of the tile, kept in registers over the set's row tiles
                uint32_t B[NBW][NP][2];
                int init[NBW][2];
#pragma unroll
                for (int j = 0; j < NBW; ++j) {
                    const uint8_t* pb = s_planes + (size_t)(warp * NBW + j) * kBP;
#pragma unroll
                    for (int pl = 0; pl < NP; ++pl) {
                        const uint2 v = *reinterpret_cast<const uint2*>(pb + pl * 256 + lane * 8);
                        B[j][pl][0] = v.x;
                        B[j][pl][1] = v.y;
                    }
                    const int2 iv = *reinterpret_cast<const int2*>(pb + (kBP - 32) + t * 8);
                    init[j][0] = iv.x;
                    init[j][1] = iv.y;
                }

#pragma unroll 1
                for (uint32_t u = sg0; u < sg1; ++u) {
                    if (!mbar_wait(full(s), s_par, abort_flag)) report(p.status, 43);
                    const uint8_t* sq = ring + (size_t)s * p.stage_bytes;
                    const uint8_t* ss = sq + p.s_off;
                    // the NBW scales of rows g and g + 8 (rows of 2 NBW kWarps bytes; when that is 128, 16-byte group
                    // number n of a row sits at position n ^ row inside it)
                    __align__(16) __half dlo[NBW], dhi[NBW];
                    {
                        const uint32_t srow = kt_blocks * 2;
                        const uint32_t o = warp * NBW * 2;
                        const uint32_t at = S_SWZ ? ((((o >> 4) ^ g) << 4) | (o & 15u)) : o;
                        const uint8_t* a = ss + g * srow + at;
                        const uint8_t* b = a + 8 * srow;
                        if constexpr (NBW == 8) {
                            *reinterpret_cast<uint4*>(dlo) = *reinterpret_cast<const uint4*>(a);
                            *reinterpret_cast<uint4*>(dhi) = *reinterpret_cast<const uint4*>(b);
                        } else if constexpr (NBW == 4) {
                            *reinterpret_cast<uint2*>(dlo) = *reinterpret_cast<const uint2*>(a);
                            *reinterpret_cast<uint2*>(dhi) = *reinterpret_cast<const uint2*>(b);
                        } else if constexpr (NBW == 2) {
                            *reinterpret_cast<uint32_t*>(dlo) = *reinterpret_cast<const uint32_t*>(a);
                            *reinterpret_cast<uint32_t*>(dhi) = *reinterpret_cast<const uint32_t*>(b);
                        } else {
                            dlo[0] = *reinterpret_cast<const __half*>(a);
                            dhi[0] = *reinterpret_cast<const __half*>(b);
                        }
                    }
                    // row g of the tile: [chunk][row][128 bytes]; 16-byte group `sub` of a row sits at sub ^ (row & 7)
                    const uint8_t* qrow = sq + g * 128 + t * 4;
                    float sacc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                    for (int j = 0; j < NBW; ++j) {
                        const uint32_t off = (warp * NBW + j) * QB;                       // byte offset of the block in the tile's row
                        const uint8_t* qa = qrow + (off >> 7) * 2048 + ((((off >> 4) & 7) ^ g) << 4);
                        const uint8_t* qb = qa + 1024;                                      // row g + 8: same swizzle
                        uint32_t A[4];
                        if constexpr (QT == 1) {
                            const uint32_t wa = *reinterpret_cast<const uint32_t*>(qa);
                            const uint32_t wb = *reinterpret_cast<const uint32_t*>(qb);
                            A[0] = wa & 0x0F0F0F0Fu;
                            A[1] = wb & 0x0F0F0F0Fu;
                            A[2] = (wa >> 4) & 0x0F0F0F0Fu;
                            A[3] = (wb >> 4) & 0x0F0F0F0Fu;
                        } else {
                            // the block's second 16 bytes: the next group of the row
                            const uint8_t* qa2 = qrow + (off >> 7) * 2048 + (((((off >> 4) & 7) + 1) ^ g) << 4);
                            A[0] = *reinterpret_cast<const uint32_t*>(qa);
                            A[1] = *reinterpret_cast<const uint32_t*>(qb);
                            A[2] = *reinterpret_cast<const uint32_t*>(qa2);
                            A[3] = *reinterpret_cast<const uint32_t*>(qa2 + 1024);
                        }
                        const int c_init[4] = {init[j][0], init[j][1], init[j][0], init[j][1]};
                        const float dl = __half2float(dlo[j]), dh = __half2float(dhi[j]);
                        if constexpr (MODE == FULL) {
                            const int zero[4] = {0, 0, 0, 0};
                            int ca[4], cb[4], cc[4];
                            mma_i8<QT == 0>(ca, A, B[j][0][0], B[j][0][1], zero);
                            mma_i8<QT == 0>(cb, A, B[j][1][0], B[j][1][1], zero);
                            mma_i8<QT == 0>(cc, A, B[j][2][0], B[j][2][1], c_init);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                // sum q X = 65536 sa + 256 sb + sc, exact in 32 bits by the bound on |X|
                                const int tsum = ca[e] * 65536 + (cb[e] * 256 + cc[e]);
                                sacc[e] = fmaf(e < 2 ? dl : dh, (float)tsum, sacc[e]);
                            }
                        } else {
                            int c[4];
                            mma_i8<QT == 0>(c, A, B[j][0][0], B[j][0][1], c_init);
#pragma unroll
                            for (int e = 0; e < 4; ++e) sacc[e] = fmaf(e < 2 ? dl : dh, (float)c[e], sacc[e]);
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty(s));
                    if (++s == p.stages) {
                        s = 0;
                        s_par ^= 1u;
                    }
                    // this warp's columns of the tile are done: its sums wait in shared memory for the pass's end
                    s_acc[((size_t)(u - sg0) * kWarps + warp) * 32 + lane] =
                        make_float4(sxv.x * sacc[0], sxv.y * sacc[1], sxv.x * sacc[2], sxv.y * sacc[3]);
                }
            }
            // ---- the pass's end: add the 8 warps' sums of every row tile (warp w takes tiles w, w + 8, ..), in
            // warp order, then the phases in phase order; the last phase writes y
            asm volatile("bar.sync 1, %0;" ::"n"(kWarps * 32) : "memory");
            const uint32_t n_units = sg1 - sg0;
            const bool last_phase = ph + 1 == p.phases;
            for (uint32_t uu = warp; uu < n_units; uu += kWarps) {
                const float4* src = s_acc + (size_t)uu * kWarps * 32 + lane;
                float4 r = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                for (int w = 0; w < kWarps; ++w) {
                    const float4 v = src[w * 32];
                    r.x += v.x;
                    r.y += v.y;
                    r.z += v.z;
                    r.w += v.w;
                }
                // r: rows g (x, y) and g + 8 (z, w) of the tile, MMA columns 2 t and 2 t + 1
                uint32_t v0 = 2 * t, v1 = 2 * t + 1;
                bool writer = true;
                if constexpr (MODE == SINGLE) {
                    // the columns are (vector, plane) pairs, column 3 v + pl: collect a vector's three planes from
                    // the lanes of the quad and add them, each already weighted by 65536 / 256 / 1, high plane last
                    const uint32_t base = lane & ~3u;
                    float lo[6], hi[6];
#pragma unroll
                    for (int q = 0; q < 3; ++q) {
                        lo[2 * q] = __shfl_sync(0xffffffffu, r.x, base + q);
                        lo[2 * q + 1] = __shfl_sync(0xffffffffu, r.y, base + q);
                        hi[2 * q] = __shfl_sync(0xffffffffu, r.z, base + q);
                        hi[2 * q + 1] = __shfl_sync(0xffffffffu, r.w, base + q);
                    }
                    r.x = (lo[2] + lo[1]) + lo[0];
                    r.y = (lo[5] + lo[4]) + lo[3];
                    r.z = (hi[2] + hi[1]) + hi[0];
                    r.w = (hi[5] + hi[4]) + hi[3];
                    v0 = 0;
                    v1 = 1;
                    writer = t == 0;
                }
                if (writer) {
                    if (p.phases > 1) {
                        float4* part = s_part + (size_t)uu * 32 + lane;      // only this thread touches it
                        if (ph > 0) {
                            const float4 q = *part;
                            r.x += q.x;
                            r.y += q.y;
                            r.z += q.z;
                            r.w += q.w;
                        }
                        if (!last_phase) *part = r;
                    }
                    if (last_phase) {
                        const MmaMat& mt = p.mat[mat_of(p, sg0 + uu)];
                        const uint32_t row_lo = (sg0 + uu - mt.unit0) * kUnitRows + g, row_hi = row_lo + 8;
                        if (v0 < p.batch) {
                            if (row_lo < mt.nrows) mt.y[(size_t)v0 * p.y_stride + row_lo] = r.x;
                            if (row_hi < mt.nrows) mt.y[(size_t)v0 * p.y_stride + row_hi] = r.z;
                        }
                        if (v1 < p.batch) {
                            if (row_lo < mt.nrows) mt.y[(size_t)v1 * p.y_stride + row_lo] = r.y;
                            if (row_hi < mt.nrows) mt.y[(size_t)v1 * p.y_stride + row_hi] = r.w;
                        }
                    }
                }
            }
        }
    }
}

struct MmaConfig {
    uint32_t phases, nbw, stages, stage_bytes, s_off, ring_off, slot_bytes, sg_units;
    int mode;
    size_t smem;
};

// false: the shape does not fit (columns not a multiple of 256).  `units_per_cta`: the most row tiles one
// CTA will own.
bool choose(const vx_qweights* w, uint32_t batch, uint32_t units_per_cta, uint32_t nbw_max, uint32_t max_stages, MmaConfig* c) {
    const uint32_t nb = (uint32_t)w->blocks_per_row;
    const uint32_t qb = w->type == VX_Q4_0 ? 16 : 32;
    c->mode = batch <= 2 ? SINGLE : FULL;
    const uint32_t bp = block_planes(c->mode);
    if (nb % kWarps != 0) return false;
    units_per_cta = std::max(units_per_cta, 1u);
    // Shared memory: the planes' slots, the ring, and per row tile of a set 4 KB of partial sums (+ 512 B of
    // sums between phases).  Wanted: three ring stages (deeper rings measured no faster) and room for all of
    // a CTA's row tiles, or at least 8, in one set (every further set walks the phases again); column tiles
    // of fewer blocks per warp make that room when the widest ones do not.
    const size_t limit = (size_t)227 * 1024 - 1024;         // 1024: the dynamic window's own alignment
    for (int pass = 0; pass < 2; ++pass) {
        for (uint32_t nbw = nbw_max; nbw >= 1; nbw >>= 1) {
            if (nb % (nbw * kWarps) != 0) continue;
            const uint32_t kt_blocks = nbw * kWarps;
            c->nbw = nbw;
            c->phases = nb / kt_blocks;
            c->s_off = kUnitRows * kt_blocks * qb;              // a multiple of 2048
            c->stage_bytes = (c->s_off + kUnitRows * kt_blocks * 2 + 1023) & ~1023u;
            c->slot_bytes = (kt_blocks * bp + kWarps * kVecs * 4 + 127) & ~127u;
            c->ring_off = ((c->phases > 1 ? 2 : 1) * c->slot_bytes + 1023) & ~1023u;
            const size_t per_unit = kAccUnit + (c->phases > 1 ? kPartUnit : 0);
            const size_t bars = (2 * kMaxStages + 4) * 8;
            const uint32_t want_stages = pass == 0 ? 3 : 2;
            const size_t fixed = c->ring_off + (size_t)want_stages * c->stage_bytes + bars;
            if (fixed + per_unit > limit) continue;
            const uint32_t fit = (uint32_t)std::min<size_t>((limit - fixed) / per_unit, 0x10000);
            const uint32_t sg = std::min(units_per_cta, fit);
            if (pass == 0 && sg < std::min(units_per_cta, 8u)) continue;
            c->sg_units = sg;
            const size_t rest = limit - c->ring_off - bars - (size_t)sg * per_unit;
            c->stages = (uint32_t)std::min<size_t>(std::min<uint32_t>(max_stages, 6), rest / c->stage_bytes);
            if (c->stages < 2) continue;
            c->smem = c->ring_off + (size_t)c->stages * c->stage_bytes + (size_t)sg * per_unit + bars + 1024;
            return true;
        }
    }
    return false;
}

// cuTensorMapEncodeTiled, fetched from the driver at run time (no link-time dependency on libcuda).
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeFn encode_fn() {
    static std::atomic<EncodeFn> fn{nullptr};
    EncodeFn f = fn.load(std::memory_order_acquire);
    if (!f) {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            f = reinterpret_cast<EncodeFn>(sym);
        (void)cudaGetLastError();
        fn.store(f, std::memory_order_release);
    }
    return f;
}

// The quants plane as bytes [column chunk of 128][row][128]: box = 128 bytes x 16 rows x the tile's chunks.
// The scales plane as bytes [row][2 nb]: box = the tile's scales x 16 rows.
bool make_maps(const vx_qweights* w, const MmaConfig& c, CUtensorMap* map_q, CUtensorMap* map_s) {
    EncodeFn fn = encode_fn();
    if (!fn) return false;
    const uint32_t qb = w->type == VX_Q4_0 ? 16 : 32;
    const uint32_t kt_blocks = c.nbw * (uint32_t)kWarps;
    const cuuint32_t ones[3] = {1, 1, 1};
    {
        const cuuint64_t dims[3] = {128, w->rows, w->quant_row_bytes / 128};
        const cuuint64_t strides[2] = {w->quant_row_bytes, 128};
        const cuuint32_t box[3] = {128, (cuuint32_t)kUnitRows, kt_blocks * qb / 128};
        if (fn(map_q, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, w->d_quants, dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    {
        const cuuint64_t dims[2] = {w->blocks_per_row * 2, w->rows};
        const cuuint64_t strides[1] = {w->blocks_per_row * 2};
        const cuuint32_t box[2] = {kt_blocks * 2, (cuuint32_t)kUnitRows};
        if (fn(map_s, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, w->d_scales, dims, strides, box, ones, CU_TENSOR_MAP_INTERLEAVE_NONE,
               kt_blocks == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return false;
    }
    return true;
}

template <int QT, int NBW, int MODE>
vx_status launch_main(vx_context* ctx, const MmaParams& p, const MmaMaps& maps, uint32_t grid, size_t smem) {
    auto kernel = gemv_mma_kernel<QT, NBW, MODE>;
    static std::atomic<size_t> granted[64];
    const int dev = ctx->device & 63;
    if (granted[dev].load(std::memory_order_acquire) < smem) {
        VX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        granted[dev].store(smem, std::memory_order_release);
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kWarps * 32 + 32);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    // the weights may have been written by a kernel of this stream (device quantiser): then no early start
    cfg.numAttrs = vx::option(ctx, "gemv.pdl", 1) != 0 && !ctx->weights_fresh ? 1 : 0;
    ctx->weights_fresh = false;
    VX_CUDA(cudaLaunchKernelEx(&cfg, kernel, p, maps));
    return VX_OK;
}

template <int QT, int MODE>
vx_status launch_nbw(vx_context* ctx, uint32_t nbw, const MmaParams& p, const MmaMaps& maps, uint32_t grid, size_t smem) {
    switch (nbw) {
        case 8: return launch_main<QT, 8, MODE>(ctx, p, maps, grid, smem);
        case 4: return launch_main<QT, 4, MODE>(ctx, p, maps, grid, smem);
        case 2: return launch_main<QT, 2, MODE>(ctx, p, maps, grid, smem);
        default: return launch_main<QT, 1, MODE>(ctx, p, maps, grid, smem);
    }
}

// Grows one of the context's scratch buffers (never shrinks); new memory is zeroed.
vx_status ensure(vx_context* ctx, void** buf, size_t* have, size_t want) {
    if (*have >= want) return VX_OK;
    VX_CUDA(cudaStreamSynchronize(ctx->stream));     // earlier launches may still use the old buffer
    if (*buf) cudaFree(*buf);
    *buf = nullptr;
    *have = 0;
    VX_CUDA(vx::device_malloc(ctx, buf, want));
    VX_CUDA(cudaMemsetAsync(*buf, 0, want, ctx->stream));
    *have = want;
    return VX_OK;
}

}  // namespace

namespace vx {

// `batch` vectors (1..8) times `n_mats` slabs (rows [row0[i], row0[i] + nrows[i]) of ws[i]; all of one type and
// column count) in one pass: the vectors' planes are made once, then one persistent launch per kMaxMats slabs
// walks their row tiles.  *eligible = false (nothing launched) when the shape does not fit this kernel; the
// caller then takes the streaming kernel.
vx_status launch_gemv_mma(vx_context* ctx, const vx_qweights* const* ws_in, const size_t* row0_in, const uint32_t* nrows_in,
                          float* const* ys_in, size_t n_in, const float* x, size_t x_stride, size_t y_stride,
                          uint32_t batch, bool* eligible) {
    *eligible = false;
    if (n_in == 0) return VX_OK;
    const vx_qweights* w = ws_in[0];
    for (size_t i = 1; i < n_in; ++i)
        if (ws_in[i]->type != w->type || ws_in[i]->cols != w->cols) return VX_OK;
    MmaConfig c;
    // blocks per warp and column tile: 8, or what "gemv.mma_nbw" asks for (a power of two up to 8); Q8_0 with three
    // and more vectors does better with 4 (7.2 against 8.2 us at 4096 x 4096: its stages are twice the bytes)
    const int64_t nbw_opt = vx::option(ctx, "gemv.mma_nbw", 0);
    uint32_t nbw_max = w->type == VX_Q8_0 && batch > 2 ? 4 : 8;
    if (nbw_opt > 0) nbw_max = nbw_opt >= 8 ? 8 : nbw_opt >= 4 ? 4 : nbw_opt >= 2 ? 2 : 1;
    const uint32_t max_stages =
        (uint32_t)std::min<int64_t>(kMaxStages, std::max<int64_t>(2, vx::option(ctx, "gemv.mma_max_stages", kMaxStages)));
    if (batch < 1 || batch > (uint32_t)kVecs) return VX_OK;
    // How many row tiles per CTA fit one set (their sums wait in shared memory over the phases)?  A launch takes
    // up to kMaxMats slabs, and no more of them than keep its CTAs within one set where that is possible:
    // measured, a launch whose CTAs walk several sets is slower per matrix than several launches of one set each
    // (28672 x 8192 Q4_0, 8 vectors: 38.8 us per matrix with eight matrices in one launch, 33.9 with two).
    if (!choose(w, batch, 0x10000, nbw_max, max_stages, &c)) return VX_OK;
    // (and no more than 14 row tiles per CTA and launch: with one or two vectors, whose planes leave room for far
    // larger sets, 8192 x 8192 Q4_0 takes 8.7 us per matrix at 10 tiles per CTA and 10.6 us at 28)
    const uint32_t units_cap = (uint32_t)std::max<int64_t>(1, vx::option(ctx, "gemv.mma_units_per_cta", 14));
    const uint64_t set_units = (uint64_t)std::min(c.sg_units, units_cap) * (uint32_t)ctx->sm_count;
    // slabs taller than that are cut into pieces of that many row tiles, each a slab of its own
    std::vector<const vx_qweights*> ws;
    std::vector<size_t> row0;
    std::vector<uint32_t> nrows;
    std::vector<float*> ys;
    for (size_t i = 0; i < n_in; ++i) {
        const uint64_t piece_rows = set_units * kUnitRows;
        for (uint64_t done = 0; done < nrows_in[i]; done += piece_rows) {
            ws.push_back(ws_in[i]);
            row0.push_back(row0_in[i] + (size_t)done);
            nrows.push_back((uint32_t)std::min<uint64_t>(piece_rows, nrows_in[i] - done));
            ys.push_back(ys_in[i] + done);
        }
    }
    const size_t n_mats = ws.size();
    if (n_mats == 0) return VX_OK;
    std::vector<size_t> first;            // first slab of every launch
    uint32_t most_units = 0;              // the most row tiles a CTA owns in any of the launches
    {
        uint64_t units = 0;
        size_t count = 0;
        for (size_t i = 0; i <= n_mats; ++i) {
            const uint64_t u = i < n_mats ? (nrows[i] + kUnitRows - 1) / kUnitRows : 0;
            if (i == n_mats || (count > 0 && (count == (size_t)kMaxMats || units + u > set_units))) {
                const uint32_t grid = (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>((uint64_t)ctx->sm_count, units));
                most_units = std::max(most_units, (uint32_t)((units + grid - 1) / grid));
                units = 0;
                count = 0;
            }
            if (i == n_mats) break;
            if (count == 0) first.push_back(i);
            units += u;
            ++count;
        }
    }
    if (!choose(w, batch, most_units, nbw_max, max_stages, &c)) return VX_OK;
    // every slab's tensor maps first: nothing is launched unless all of them can be made
    std::vector<MmaMaps> all_maps(first.size());
    for (size_t l = 0; l < first.size(); ++l) {
        const size_t end = l + 1 < first.size() ? first[l + 1] : n_mats;
        for (size_t i = first[l]; i < end; ++i)
            if (!make_maps(ws[i], c, &all_maps[l].q[i - first[l]], &all_maps[l].s[i - first[l]])) return VX_OK;
    }
    const uint32_t nb = (uint32_t)w->blocks_per_row;
    const uint32_t slices = nb / c.nbw;
    const size_t planes_bytes = ((size_t)nb * block_planes(c.mode) + 255) & ~(size_t)255;
    vx_status st = ensure(ctx, &ctx->mma_planes, &ctx->mma_planes_bytes, planes_bytes + (size_t)slices * kVecs * 4);
    if (st != VX_OK) return st;
    uint8_t* planes = static_cast<uint8_t*>(ctx->mma_planes);
    float* sx = reinterpret_cast<float*>(planes + planes_bytes);

    const bool q4 = w->type == VX_Q4_0;
    {
        auto pre = c.mode == FULL ? (q4 ? xplanes_kernel<1, FULL> : xplanes_kernel<0, FULL>)
                                  : (q4 ? xplanes_kernel<1, SINGLE> : xplanes_kernel<0, SINGLE>);
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(slices);
        cfg.blockDim = dim3(256);
        cfg.stream = ctx->stream;
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = vx::option(ctx, "gemv.pdl", 1) != 0 ? 1 : 0;
        VX_CUDA(cudaLaunchKernelEx(&cfg, pre, x, (uint64_t)x_stride, batch, c.nbw, planes, sx));
    }
    VX_CUDA(cudaGetLastError());
    ctx->launches++;

    for (size_t l = 0; l < first.size(); ++l) {
        const size_t m0 = first[l];
        MmaParams p{};
        p.n_mats = (uint32_t)((l + 1 < first.size() ? first[l + 1] : n_mats) - m0);
        uint32_t units = 0;
        for (uint32_t i = 0; i < p.n_mats; ++i) {
            p.mat[i].y = ys[m0 + i];
            p.mat[i].row0 = (uint32_t)row0[m0 + i];
            p.mat[i].nrows = nrows[m0 + i];
            p.mat[i].unit0 = units;
            units += (nrows[m0 + i] + kUnitRows - 1) / kUnitRows;
        }
        p.units = units;
        p.nb = nb;
        p.phases = c.phases;
        p.sg_units = c.sg_units;
        p.slot_bytes = c.slot_bytes;
        p.stages = c.stages;
        p.stage_bytes = c.stage_bytes;
        p.s_off = c.s_off;
        p.ring_off = c.ring_off;
        p.planes = planes;
        p.sx = sx;
        p.y_stride = y_stride;
        p.batch = batch;
        p.status = ctx->d_status;
        const uint32_t grid = std::max(1u, std::min((uint32_t)ctx->sm_count, units));
        const MmaMaps& maps = all_maps[l];
        if (c.mode == FULL)
            st = q4 ? launch_nbw<1, FULL>(ctx, c.nbw, p, maps, grid, c.smem) : launch_nbw<0, FULL>(ctx, c.nbw, p, maps, grid, c.smem);
        else
            st = q4 ? launch_nbw<1, SINGLE>(ctx, c.nbw, p, maps, grid, c.smem) : launch_nbw<0, SINGLE>(ctx, c.nbw, p, maps, grid, c.smem);
        if (st != VX_OK) return st;
        ctx->launches++;
    }
    ctx->status_dirty = true;
    *eligible = true;
    return VX_OK;
}

}  // namespace vx
