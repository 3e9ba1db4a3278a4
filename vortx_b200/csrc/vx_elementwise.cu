// Strided element-wise kernels around the matmul path: in-place binary operations with
// broadcast strides (vortx-shaders/src/linalg/op_assign.rs:29-187), the strided-to-row-major
// gather (contiguous.rs:18-85) and the wrap-around tiling copy (repeat.rs:15-43).
//
// Index arithmetic follows the shaders exactly — a linear id is decomposed over the first
// shape's sizes (shape.rs:76-86) and re-composed through each operand's strides (shape.rs:52-54),
// all in wrapping u32 — so results are the very same bits wherever the reference is defined.
// The general kernels are one grid-stride loop each; adjacent threads take adjacent linear ids, which are
// adjacent addresses whenever the innermost stride is 1.  They spend three integer divisions per element and
// run at a third of the HBM rate, so the layouts that matter get forms that compute the same indices without
// them (all bit-identical: the operations are exact per element, only the order of the elements changes):
//   flat   both operands are one dense row-major block: a one-dimensional float4 pass, 16 KB per thread block;
//   rows   a block walks whole rows (n, c, h) and its threads the w axis: one decomposition per row; float4
//          accesses when both innermost strides are 1 (or b's is 0) and every row starts 16-byte aligned;
//          rows of 4096 elements or more get a thread block each, shorter ones resident blocks;
//   tile   b is read across its unit-stride axis h (a transposed view): 64 x 64 tiles through shared memory.
// Every form issues a batch of loads before the stores that depend on them: a and the result are the same
// array, so the compiler cannot move a later load above an earlier store by itself.
// They are taken when no index can wrap around 2^32 (the general kernels keep the wrapping arithmetic).
#include <algorithm>

#include "vx_internal.h"

namespace {

using vx::fail;

struct Idx4 {
    uint32_t n, c, h, w;
};

// vortx-shaders/src/linalg/shape.rs:76-86 (checked_div(..).unwrap_or(0) for empty dimensions)
__host__ __device__ __forceinline__ Idx4 decompose(const vx_shape& s, uint32_t i) {
    const uint32_t chw = s.c * s.h * s.w, hw = s.h * s.w;
    const uint32_t i3 = chw ? i / chw : 0;
    const uint32_t r3 = i - i3 * chw;
    const uint32_t i2 = hw ? r3 / hw : 0;
    const uint32_t r2 = r3 - i2 * hw;
    const uint32_t i1 = s.w ? r2 / s.w : 0;
    return Idx4{i3, i2, i1, r2 - i1 * s.w};
}
__host__ __device__ __forceinline__ uint32_t compose(const vx_shape& s, const Idx4& id) {
    return id.n * s.n_stride + id.c * s.c_stride + id.h * s.h_stride + id.w * s.w_stride;
}
__host__ __device__ __forceinline__ uint32_t shape_len(const vx_shape& s) { return s.n * s.c * s.h * s.w; }

template <int OP>
__device__ __forceinline__ float apply(float a, float b) {
    if (OP == VX_OP_ADD) return __fadd_rn(a, b);
    if (OP == VX_OP_SUB) return __fsub_rn(a, b);
    if (OP == VX_OP_MUL) return __fmul_rn(a, b);
    if (OP == VX_OP_DIV) return __fdiv_rn(a, b);
    return b;
}

// (n, c, h) of row r, as decompose() finds them for the row's elements
__device__ __forceinline__ Idx4 row_of(const vx_shape& s, uint32_t r) {
    const uint32_t t = r / s.h;
    return Idx4{t / s.c, t % s.c, r % s.h, 0};
}

// rows form.  VEC: float4 along w (b's innermost stride 1, or 0 with BCAST: one b value per row).
template <int OP, bool VEC, bool BCAST>
__global__ void __launch_bounds__(256)
op_assign_rows_kernel(float* __restrict__ a, const float* __restrict__ b, const vx_shape sa, const vx_shape sb,
                      uint32_t off_a, uint32_t off_b) {
    const uint32_t rows = sa.n * sa.c * sa.h;
    for (uint32_t r = blockIdx.x; r < rows; r += gridDim.x) {
        Idx4 id = row_of(sa, r);
        const uint32_t base_a = off_a + compose(sa, id), base_b = off_b + compose(sb, id);
        if (VEC) {
            float4* pa = reinterpret_cast<float4*>(a + base_a);
            const float4* pb = reinterpret_cast<const float4*>(b + base_b);
            const float bv = BCAST ? b[base_b] : 0.0f;
            // four float4 of a (and of b) in flight per thread: a load after a store to the same array would wait
            const uint32_t w4 = sa.w / 4;
            for (uint32_t w0 = threadIdx.x; w0 < w4; w0 += 4 * blockDim.x) {
                float4 va[4], vb[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t w = w0 + k * blockDim.x;
                    if (w < w4) {
                        if (OP != VX_OP_COPY) va[k] = pa[w];
                        vb[k] = BCAST ? make_float4(bv, bv, bv, bv) : pb[w];
                    }
                }
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const uint32_t w = w0 + k * blockDim.x;
                    if (w < w4) {
                        float4 r;
                        r.x = apply<OP>(OP != VX_OP_COPY ? va[k].x : 0.0f, vb[k].x);
                        r.y = apply<OP>(OP != VX_OP_COPY ? va[k].y : 0.0f, vb[k].y);
                        r.z = apply<OP>(OP != VX_OP_COPY ? va[k].z : 0.0f, vb[k].z);
                        r.w = apply<OP>(OP != VX_OP_COPY ? va[k].w : 0.0f, vb[k].w);
                        pa[w] = r;
                    }
                }
            }
        } else {
            for (uint32_t w = threadIdx.x; w < sa.w; w += blockDim.x) {
                const uint32_t ia = base_a + w * sa.w_stride;
                a[ia] = apply<OP>(a[ia], b[base_b + w * sb.w_stride]);
            }
        }
    }
}

// flat form: both operands are the same dense row-major block (16-byte aligned, length a multiple of 4): one
// 1-D pass, every thread block takes 1024 consecutive float4 and every thread four of them, loads before stores.
template <int OP>
__global__ void __launch_bounds__(256)
op_assign_flat_kernel(float4* __restrict__ a, const float4* __restrict__ b, uint32_t len4) {
    const uint32_t base = blockIdx.x * 1024u + threadIdx.x;
    float4 va[4], vb[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t i = base + 256u * k;
        if (i < len4) {
            if (OP != VX_OP_COPY) va[k] = a[i];
            vb[k] = b[i];
        }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t i = base + 256u * k;
        if (i < len4) {
            float4 r;
            r.x = apply<OP>(OP != VX_OP_COPY ? va[k].x : 0.0f, vb[k].x);
            r.y = apply<OP>(OP != VX_OP_COPY ? va[k].y : 0.0f, vb[k].y);
            r.z = apply<OP>(OP != VX_OP_COPY ? va[k].z : 0.0f, vb[k].z);
            r.w = apply<OP>(OP != VX_OP_COPY ? va[k].w : 0.0f, vb[k].w);
            a[i] = r;
        }
    }
}

// tile form: a's innermost stride is 1, b's unit stride is along h.  Tile (th, tw) of plane (n, c): b is read
// with h fastest, a is updated with w fastest; the 64 x 65 shared tile turns one into the other (runs of 256
// bytes on both sides).  Measured alternatives, none faster: 32 x 32 tiles (15 % slower), 128 x 64, 64 x 128,
// 256 x 32 and 128 x 128 tiles (3 to 60 % slower), one thread block per tile instead of resident blocks, and a
// diagonal order of the tiles (no change: the power-of-two pitch does not camp on memory channels), and rings of
// 4, 6 and 13 tiles per block filled by 4-byte asynchronous copies (8 to 15 % slower: more bytes in flight do
// not help, the 256-byte runs themselves are what the memory system serves at 0.8 of its dense rate).
constexpr int kTile = 64;
template <int OP>
__global__ void __launch_bounds__(256)
op_assign_tile_kernel(float* __restrict__ a, const float* __restrict__ b, const vx_shape sa, const vx_shape sb,
                      uint32_t off_a, uint32_t off_b) {
    __shared__ float tile[kTile][kTile + 1];
    const uint32_t tiles_w = (sa.w + kTile - 1) / kTile, tiles_h = (sa.h + kTile - 1) / kTile;
    const uint32_t per_plane = tiles_w * tiles_h, total = per_plane * sa.n * sa.c;
    const uint32_t x = threadIdx.x & (kTile - 1), y = threadIdx.x / kTile;     // 64 x 4 threads
    constexpr int kPer = kTile / 4;
    for (uint32_t t = blockIdx.x; t < total; t += gridDim.x) {
        const uint32_t plane = t / per_plane, in_plane = t - plane * per_plane;
        const uint32_t th = in_plane / tiles_w, tw = in_plane - th * tiles_w;
        const Idx4 pl = Idx4{plane / sa.c, plane % sa.c, 0, 0};
        const uint32_t base_a = off_a + compose(sa, pl), base_b = off_b + compose(sb, pl);
        __syncthreads();                                            // the tile of the round before has been used
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            const uint32_t h = th * kTile + x, w = tw * kTile + y + 4 * k;
            if (h < sa.h && w < sa.w) tile[y + 4 * k][x] = b[base_b + h * sb.h_stride + w * sb.w_stride];
        }
        __syncthreads();
        // all of a's elements first, then the stores: a load after a store to the same array would wait for it
        // (a quarter of the time of the whole pass, measured)
        float va[kPer];
        if (OP != VX_OP_COPY) {
#pragma unroll
            for (int k = 0; k < kPer; ++k) {
                const uint32_t h = th * kTile + y + 4 * k, w = tw * kTile + x;
                va[k] = (h < sa.h && w < sa.w) ? a[base_a + h * sa.h_stride + w * sa.w_stride] : 0.0f;
            }
        }
#pragma unroll
        for (int k = 0; k < kPer; ++k) {
            const uint32_t h = th * kTile + y + 4 * k, w = tw * kTile + x;
            if (h < sa.h && w < sa.w)
                a[base_a + h * sa.h_stride + w * sa.w_stride] = apply<OP>(OP != VX_OP_COPY ? va[k] : 0.0f, tile[x][y + 4 * k]);
        }
    }
}

// rows form of the tiling copy: the source's (n, c, h) wrap once per row, its w index by increments.
// VEC: both innermost strides are 1, both widths multiples of 4 and every row 16-byte aligned: float4 moves
// (a float4 of the result never straddles the source's wrap).
template <bool VEC>
__global__ void __launch_bounds__(256)
repeat_rows_kernel(float* __restrict__ result, const float* __restrict__ source, const vx_shape sr, const vx_shape ss) {
    const uint32_t rows = sr.n * sr.c * sr.h;
    const uint32_t src_w = VEC ? ss.w / 4 : ss.w, res_w = VEC ? sr.w / 4 : sr.w;
    const uint32_t step = blockDim.x % src_w;
    for (uint32_t r = blockIdx.x; r < rows; r += gridDim.x) {
        const Idx4 id = row_of(sr, r);
        const Idx4 wr = Idx4{id.n % ss.n, id.c % ss.c, id.h % ss.h, 0};
        const uint32_t base_r = compose(sr, id), base_s = compose(ss, wr);
        uint32_t ws = threadIdx.x % src_w;
        for (uint32_t w = threadIdx.x; w < res_w; w += blockDim.x) {
            if (VEC)
                reinterpret_cast<float4*>(result + base_r)[w] = reinterpret_cast<const float4*>(source + base_s)[ws];
            else
                result[base_r + w * sr.w_stride] = source[base_s + ws * ss.w_stride];
            ws += step;
            if (ws >= src_w) ws -= src_w;
        }
    }
}

template <int OP>
__global__ void __launch_bounds__(256)
op_assign_kernel(float* __restrict__ a, const float* __restrict__ b, const vx_shape sa, const vx_shape sb,
                 uint32_t off_a, uint32_t off_b) {
    const uint32_t len = shape_len(sa);
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < len; i += gridDim.x * blockDim.x) {
        const Idx4 id = decompose(sa, i);
        const uint32_t ia = off_a + compose(sa, id), ib = off_b + compose(sb, id);
        a[ia] = apply<OP>(a[ia], b[ib]);
    }
}

__global__ void __launch_bounds__(256)
contiguous_kernel(uint32_t* __restrict__ dest, const uint32_t* __restrict__ src, const vx_shape s, uint32_t offset) {
    const uint32_t len = shape_len(s);
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < len; i += gridDim.x * blockDim.x) {
        const Idx4 id = decompose(s, i);
        dest[i] = src[offset + compose(s, id)];
    }
}

__global__ void __launch_bounds__(256)
repeat_kernel(float* __restrict__ result, const float* __restrict__ source, const vx_shape sr, const vx_shape ss) {
    const uint32_t len = shape_len(sr);
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < len; i += gridDim.x * blockDim.x) {
        const Idx4 id = decompose(sr, i);
        // shape.rs:72-74: the source index wraps around each source dimension
        const Idx4 w = Idx4{ss.n ? id.n % ss.n : 0, ss.c ? id.c % ss.c : 0, ss.h ? id.h % ss.h : 0, ss.w ? id.w % ss.w : 0};
        result[compose(sr, id)] = source[compose(ss, w)];
    }
}

uint64_t span(const vx_shape& s) {
    if (s.n == 0 || s.c == 0 || s.h == 0 || s.w == 0) return 0;
    return (uint64_t)(s.n - 1) * s.n_stride + (uint64_t)(s.c - 1) * s.c_stride + (uint64_t)(s.h - 1) * s.h_stride +
           (uint64_t)(s.w - 1) * s.w_stride + 1;
}

unsigned grid_for(const vx_context* ctx, uint32_t len) {
    const unsigned want = (len + 255) / 256;
    return std::max(1u, std::min(want, (unsigned)ctx->sm_count * 16));
}

// No index of `s` walked over `sizes` (plus offset) reaches 2^32: the fast forms may then compute indices
// in any order.
bool no_wrap(const vx_shape& sizes, const vx_shape& s, uint64_t offset) {
    if (sizes.n == 0 || sizes.c == 0 || sizes.h == 0 || sizes.w == 0) return true;
    const uint64_t last = offset + (uint64_t)(sizes.n - 1) * s.n_stride + (uint64_t)(sizes.c - 1) * s.c_stride +
                          (uint64_t)(sizes.h - 1) * s.h_stride + (uint64_t)(sizes.w - 1) * s.w_stride;
    return last < (1ull << 32);
}
bool rows_aligned(const void* base, const vx_shape& s, uint64_t offset) {
    return (reinterpret_cast<uintptr_t>(base) & 15u) == 0 && offset % 4 == 0 && s.n_stride % 4 == 0 && s.c_stride % 4 == 0 &&
           s.h_stride % 4 == 0;
}

// The strides of `s`, walked over the extents of `sizes`, are row-major without gaps (a dimension of extent 1
// may carry any stride).  b is indexed with a's ids, so its strides are judged over a's extents.
bool is_dense(const vx_shape& sizes, const vx_shape& s) {
    return (sizes.w == 1 || s.w_stride == 1) && (sizes.h == 1 || s.h_stride == sizes.w) &&
           (sizes.c == 1 || s.c_stride == sizes.h * sizes.w) && (sizes.n == 1 || s.n_stride == sizes.c * sizes.h * sizes.w);
}

// Picks the form for a op= b (see the head of this file) and launches it.
template <int OP>
void launch_op_assign(vx_context* ctx, float* a, const float* b, const vx_shape& sa, const vx_shape& sb, uint32_t off_a,
                      uint32_t off_b) {
    const uint32_t len = shape_len(sa);
    const bool fast = vx::option(ctx, "elementwise.fast", 1) != 0 && no_wrap(sa, sa, off_a) && no_wrap(sa, sb, off_b);
    const uint32_t rows = sa.n * sa.c * sa.h;
    // long rows: a thread block per row (blocks that come and go keep the memory system fuller than resident
    // ones walking rows, measured); short rows: resident blocks that walk rows
    const unsigned row_grid = sa.w >= 4096 ? std::max(1u, rows) : std::max(1u, std::min(rows, (unsigned)ctx->sm_count * 8));
    if (fast && vx::option(ctx, "elementwise.flat", 1) != 0 && len % 4 == 0 && is_dense(sa, sa) && is_dense(sa, sb) &&
        (reinterpret_cast<uintptr_t>(a + off_a) & 15u) == 0 && (reinterpret_cast<uintptr_t>(b + off_b) & 15u) == 0) {
        op_assign_flat_kernel<OP><<<(len / 4 + 1023) / 1024, 256, 0, ctx->stream>>>(
            reinterpret_cast<float4*>(a + off_a), reinterpret_cast<const float4*>(b + off_b), len / 4);
    } else if (fast && sa.w >= 32 && sa.h >= 32 && sa.w_stride == 1 && sb.h_stride == 1 && sb.w_stride != 1 && sb.w_stride != 0) {
        const uint32_t tiles = ((sa.w + kTile - 1) / kTile) * ((sa.h + kTile - 1) / kTile) * sa.n * sa.c;
        op_assign_tile_kernel<OP><<<std::min(tiles, (uint32_t)ctx->sm_count * 16), 256, 0, ctx->stream>>>(a, b, sa, sb, off_a, off_b);
    } else if (fast && sa.w >= 128) {
        const bool vec = sa.w % 4 == 0 && sa.w_stride == 1 && rows_aligned(a, sa, off_a) && rows_aligned(b, sb, off_b);
        if (vec && sb.w_stride == 1)
            op_assign_rows_kernel<OP, true, false><<<row_grid, 256, 0, ctx->stream>>>(a, b, sa, sb, off_a, off_b);
        else if (sa.w % 4 == 0 && sa.w_stride == 1 && sb.w_stride == 0 && rows_aligned(a, sa, off_a))
            op_assign_rows_kernel<OP, true, true><<<row_grid, 256, 0, ctx->stream>>>(a, b, sa, sb, off_a, off_b);
        else
            op_assign_rows_kernel<OP, false, false><<<row_grid, 256, 0, ctx->stream>>>(a, b, sa, sb, off_a, off_b);
    } else {
        op_assign_kernel<OP><<<grid_for(ctx, len), 256, 0, ctx->stream>>>(a, b, sa, sb, off_a, off_b);
    }
}

vx_status cap_check(const vx_context* ctx, const char* what, const vx_shape& s, uint64_t offset, uint64_t cap) {
    if (cap == 0 || vx::option(ctx, "bounds_check", 1) == 0) return VX_OK;
    const uint64_t sp = span(s);
    if (sp != 0 && offset + sp > cap)
        return fail(VX_ERR_OUT_OF_BOUNDS, "%s layout reaches element %llu of a buffer holding %llu", what,
                    (unsigned long long)(offset + sp - 1), (unsigned long long)cap);
    return VX_OK;
}

}  // namespace

extern "C" {

vx_status vx_op_assign(vx_context* ctx, vx_op op, float* a, const vx_shape* shape_a, uint64_t cap_a, const float* b,
                       const vx_shape* shape_b, uint64_t cap_b, uint32_t offset_a, uint32_t offset_b) {
    VX_REQUIRE(ctx && shape_a && shape_b, VX_ERR_INVALID_ARGUMENT, "vx_op_assign: null argument");
    VX_REQUIRE(op >= VX_OP_ADD && op <= VX_OP_COPY, VX_ERR_INVALID_ARGUMENT, "unknown operation %d", (int)op);
    const uint32_t len = shape_len(*shape_a);
    if (len == 0) return VX_OK;
    VX_REQUIRE(a && b, VX_ERR_INVALID_ARGUMENT, "vx_op_assign: null device pointer");
    // b is indexed with a's ids: what it touches is a's extent walked with b's strides
    vx_shape touched_b = *shape_b;
    touched_b.n = shape_a->n; touched_b.c = shape_a->c; touched_b.h = shape_a->h; touched_b.w = shape_a->w;
    vx_status st;
    if ((st = cap_check(ctx, "a", *shape_a, offset_a, cap_a)) != VX_OK) return st;
    if ((st = cap_check(ctx, "b", touched_b, offset_b, cap_b)) != VX_OK) return st;
    vx::DeviceGuard guard(ctx->device);
    switch (op) {
        case VX_OP_ADD: launch_op_assign<VX_OP_ADD>(ctx, a, b, *shape_a, *shape_b, offset_a, offset_b); break;
        case VX_OP_SUB: launch_op_assign<VX_OP_SUB>(ctx, a, b, *shape_a, *shape_b, offset_a, offset_b); break;
        case VX_OP_MUL: launch_op_assign<VX_OP_MUL>(ctx, a, b, *shape_a, *shape_b, offset_a, offset_b); break;
        case VX_OP_DIV: launch_op_assign<VX_OP_DIV>(ctx, a, b, *shape_a, *shape_b, offset_a, offset_b); break;
        default: launch_op_assign<VX_OP_COPY>(ctx, a, b, *shape_a, *shape_b, offset_a, offset_b); break;
    }
    VX_CUDA(cudaGetLastError());
    ctx->launches++;
    return VX_OK;
}

vx_status vx_contiguous(vx_context* ctx, void* dest, uint64_t cap_dest, const void* src, const vx_shape* shape_src,
                        uint64_t cap_src, uint32_t offset) {
    VX_REQUIRE(ctx && shape_src, VX_ERR_INVALID_ARGUMENT, "vx_contiguous: null argument");
    const uint32_t len = shape_len(*shape_src);
    if (len == 0) return VX_OK;
    VX_REQUIRE(dest && src, VX_ERR_INVALID_ARGUMENT, "vx_contiguous: null device pointer");
    VX_REQUIRE(cap_dest == 0 || len <= cap_dest, VX_ERR_OUT_OF_BOUNDS, "destination holds %llu elements, %u needed",
               (unsigned long long)cap_dest, len);
    vx_status st = cap_check(ctx, "source", *shape_src, offset, cap_src);
    if (st != VX_OK) return st;
    vx::DeviceGuard guard(ctx->device);
    // dest[i] = src[..] is "a = b" with a the row-major tensor of src's sizes: the copy forms of op_assign move
    // the 4-byte elements as they are (no arithmetic touches them)
    vx_shape sd = *shape_src;
    sd.w_stride = 1;
    sd.h_stride = sd.w;
    sd.c_stride = sd.h * sd.w;
    sd.n_stride = sd.c * sd.h * sd.w;
    if (vx::option(ctx, "elementwise.fast", 1) != 0 && (uint64_t)shape_src->n * shape_src->c * shape_src->h * shape_src->w < (1ull << 32))
        launch_op_assign<VX_OP_COPY>(ctx, static_cast<float*>(dest), static_cast<const float*>(src), sd, *shape_src, 0, offset);
    else
        contiguous_kernel<<<grid_for(ctx, len), 256, 0, ctx->stream>>>(static_cast<uint32_t*>(dest),
                                                                       static_cast<const uint32_t*>(src), *shape_src, offset);
    VX_CUDA(cudaGetLastError());
    ctx->launches++;
    return VX_OK;
}

vx_status vx_repeat(vx_context* ctx, float* result, const vx_shape* shape_result, uint64_t cap_result,
                    const float* source, const vx_shape* shape_source, uint64_t cap_source) {
    VX_REQUIRE(ctx && shape_result && shape_source, VX_ERR_INVALID_ARGUMENT, "vx_repeat: null argument");
    const uint32_t len = shape_len(*shape_result);
    if (len == 0) return VX_OK;
    VX_REQUIRE(result && source, VX_ERR_INVALID_ARGUMENT, "vx_repeat: null device pointer");
    VX_REQUIRE(shape_len(*shape_source) != 0, VX_ERR_SHAPE, "vx_repeat: empty source");
    vx_status st;
    if ((st = cap_check(ctx, "result", *shape_result, 0, cap_result)) != VX_OK) return st;
    if ((st = cap_check(ctx, "source", *shape_source, 0, cap_source)) != VX_OK) return st;
    vx::DeviceGuard guard(ctx->device);
    if (vx::option(ctx, "elementwise.fast", 1) != 0 && shape_result->w >= 128 && no_wrap(*shape_result, *shape_result, 0) &&
        no_wrap(*shape_source, *shape_source, 0)) {
        const uint32_t rows = shape_result->n * shape_result->c * shape_result->h;
        const unsigned grid = shape_result->w >= 4096 ? std::max(1u, rows) : std::max(1u, std::min(rows, (unsigned)ctx->sm_count * 8));
        const bool vec = shape_result->w_stride == 1 && shape_source->w_stride == 1 && shape_result->w % 4 == 0 &&
                         shape_source->w % 4 == 0 && rows_aligned(result, *shape_result, 0) && rows_aligned(source, *shape_source, 0);
        if (vec)
            repeat_rows_kernel<true><<<grid, 256, 0, ctx->stream>>>(result, source, *shape_result, *shape_source);
        else
            repeat_rows_kernel<false><<<grid, 256, 0, ctx->stream>>>(result, source, *shape_result, *shape_source);
    } else {
        repeat_kernel<<<grid_for(ctx, len), 256, 0, ctx->stream>>>(result, source, *shape_result, *shape_source);
    }
    VX_CUDA(cudaGetLastError());
    ctx->launches++;
    return VX_OK;
}

// OpAssign::launch / Repeat::launch level (src/linalg/op_assign.rs:38-143, src/linalg/repeat.rs:24-88):
// broadcast_assign the two layouts (VX_ERR_SHAPE where the reference panics), canonicalise, apply the
// view offsets, launch.  is_repeat selects the tiling copy.
vx_status vx_op_assign_dispatch(vx_context* ctx, vx_op op, int32_t is_repeat, float* a, const vx_layout* layout_a,
                                uint64_t cap_a, const float* b, const vx_layout* layout_b, uint64_t cap_b) {
    VX_REQUIRE(ctx && layout_a && layout_b, VX_ERR_INVALID_ARGUMENT, "vx_op_assign_dispatch: null argument");
    vx_layout ta, tb, ca, cb;
    vx_status st = vx_layout_broadcast_assign(layout_a, layout_b, &ta, &tb);
    if (st != VX_OK) return st;
    if ((st = vx_layout_canonicalize(&ta, &ca)) != VX_OK) return st;
    if ((st = vx_layout_canonicalize(&tb, &cb)) != VX_OK) return st;
    vx_shape sa, sb;
    vx_layout_to_shape(&ca, &sa);
    vx_layout_to_shape(&cb, &sb);
    VX_REQUIRE(cap_a == 0 || layout_a->offset <= cap_a, VX_ERR_OUT_OF_BOUNDS, "a view offset beyond its buffer");
    VX_REQUIRE(cap_b == 0 || layout_b->offset <= cap_b, VX_ERR_OUT_OF_BOUNDS, "b view offset beyond its buffer");
    float* pa = a ? a + layout_a->offset : nullptr;
    const float* pb = b ? b + layout_b->offset : nullptr;
    const uint64_t ra = cap_a ? std::max<uint64_t>(1, cap_a - layout_a->offset) : 0;
    const uint64_t rb = cap_b ? std::max<uint64_t>(1, cap_b - layout_b->offset) : 0;
    if (is_repeat) return vx_repeat(ctx, pa, &sa, ra, pb, &sb, rb);
    return vx_op_assign(ctx, op, pa, &sa, ra, pb, &sb, rb, 0, 0);
}

}  // extern "C"
