// GEMM entry points: the kernel-call level (vx_gemm_f32) and the Gemm::dispatch level
// (vx_gemm_dispatch) of vortx's src/linalg/gemm.rs.
#include "vx_internal.h"

namespace {

using vx::fail;

// Largest element index the shape reaches, plus one; 0 if the shape is empty.
uint64_t shape_span(const vx_shape& s) {
    if (s.n == 0 || s.c == 0 || s.h == 0 || s.w == 0) return 0;
    return (uint64_t)(s.n - 1) * s.n_stride + (uint64_t)(s.c - 1) * s.c_stride +
           (uint64_t)(s.h - 1) * s.h_stride + (uint64_t)(s.w - 1) * s.w_stride + 1;
}

// cap < 0 means "not stated": no check.
vx_status check_capacity(const char* what, const vx_shape& s, int64_t cap) {
    if (cap < 0) return VX_OK;
    const uint64_t span = shape_span(s);
    if (span > (uint64_t)cap)
        return fail(VX_ERR_OUT_OF_BOUNDS, "%s layout reaches element %llu of a buffer holding %llu",
                    what, (unsigned long long)(span - 1), (unsigned long long)cap);
    return VX_OK;
}

vx_status gemm_impl(vx_context* ctx, vx_gemm_mode mode, float* out, const float* lhs,
                    const float* rhs, const vx_shapes3& s, int64_t cap_out, int64_t cap_lhs,
                    int64_t cap_rhs) {
    const bool empty = shape_span(s.out) == 0;
    VX_REQUIRE(empty || (out && (lhs || s.lhs.w == 0) && (rhs || s.lhs.w == 0)), VX_ERR_INVALID_ARGUMENT,
               "vx_gemm_f32: null device pointer");
    VX_REQUIRE(mode == VX_GEMM_AUTO || mode == VX_GEMM_NAIVE || mode == VX_GEMM_SIMT_EXACT ||
                   mode == VX_GEMM_TF32,
               VX_ERR_INVALID_ARGUMENT, "vx_gemm_f32: unknown mode %d", (int)mode);

    if (vx::option(ctx, "bounds_check", 1) != 0) {
        // The kernels index lhs with (row < out.h, k < lhs.w) and rhs with (k < lhs.w,
        // col < out.w): check what they will actually touch.
        vx_shape touched_lhs = s.lhs, touched_rhs = s.rhs;
        touched_lhs.n = touched_rhs.n = s.out.n;
        touched_lhs.c = touched_rhs.c = s.out.c;
        touched_lhs.h = s.out.h;
        touched_rhs.h = s.lhs.w;
        touched_rhs.w = s.out.w;
        vx_status st;
        if ((st = check_capacity("out", s.out, cap_out)) != VX_OK) return st;
        if (s.lhs.w != 0) {
            if ((st = check_capacity("lhs", touched_lhs, cap_lhs)) != VX_OK) return st;
            if ((st = check_capacity("rhs", touched_rhs, cap_rhs)) != VX_OK) return st;
        }
    }
    if (empty) {
        ctx->last_gemm_kernel = 0;
        return VX_OK;
    }

    vx::DeviceGuard guard(ctx->device);
    int kernel = 0;
    vx_status st = VX_OK;
    switch (mode) {
        case VX_GEMM_NAIVE:
            st = vx::launch_gemm_naive(ctx, out, lhs, rhs, s);
            kernel = 1;
            break;
        case VX_GEMM_AUTO:
            // src/linalg/gemm.rs:111-112
            if (s.out.h >= 32 || s.out.w >= 32) {
                st = vx::launch_gemm_simt_exact(ctx, out, lhs, rhs, s, &kernel);
            } else {
                st = vx::launch_gemm_naive(ctx, out, lhs, rhs, s);
                kernel = 1;
            }
            break;
        case VX_GEMM_SIMT_EXACT:
            st = vx::launch_gemm_simt_exact(ctx, out, lhs, rhs, s, &kernel);
            break;
        case VX_GEMM_TF32: {
            bool eligible = false;
            st = vx::launch_gemm_tf32(ctx, out, lhs, rhs, s, &eligible);
            if (st == VX_OK && eligible) {
                kernel = 3;
            } else if (st == VX_OK) {
                st = vx::launch_gemm_simt_exact(ctx, out, lhs, rhs, s, &kernel);
            }
            break;
        }
    }
    if (st == VX_OK) ctx->last_gemm_kernel = kernel;
    return st;
}

}  // namespace

extern "C" {

vx_status vx_gemm_f32(vx_context* ctx, vx_gemm_mode mode, float* out, const float* lhs,
                      const float* rhs, const vx_shapes3* shapes, uint64_t cap_out,
                      uint64_t cap_lhs, uint64_t cap_rhs) {
    VX_REQUIRE(ctx && shapes, VX_ERR_INVALID_ARGUMENT, "vx_gemm_f32: null context or shapes");
    auto cap = [](uint64_t c) -> int64_t { return c == 0 ? -1 : (int64_t)c; };
    return gemm_impl(ctx, mode, out, lhs, rhs, *shapes, cap(cap_out), cap(cap_lhs), cap(cap_rhs));
}

vx_status vx_gemm_last_kernel(const vx_context* ctx, int32_t* kernel) {
    VX_REQUIRE(ctx && kernel, VX_ERR_INVALID_ARGUMENT, "vx_gemm_last_kernel: null argument");
    *kernel = ctx->last_gemm_kernel;
    return VX_OK;
}

vx_status vx_gemm_dispatch(vx_context* ctx, vx_dispatch_kind kind, float* out,
                           const vx_layout* out_layout, uint64_t out_cap, const float* lhs,
                           const vx_layout* lhs_layout, uint64_t lhs_cap, const float* rhs,
                           const vx_layout* rhs_layout, uint64_t rhs_cap) {
    VX_REQUIRE(ctx && out_layout && lhs_layout && rhs_layout, VX_ERR_INVALID_ARGUMENT,
               "vx_gemm_dispatch: null argument");
    VX_REQUIRE(kind >= VX_DISPATCH && kind <= VX_DISPATCH_TF32, VX_ERR_INVALID_ARGUMENT,
               "vx_gemm_dispatch: unknown kind %d", (int)kind);
    vx_layout lo, ll, lr;
    vx_status st;
    if ((st = vx_layout_canonicalize(out_layout, &lo)) != VX_OK) return st;
    if ((st = vx_layout_canonicalize(lhs_layout, &ll)) != VX_OK) return st;
    if ((st = vx_layout_canonicalize(rhs_layout, &lr)) != VX_OK) return st;

    if (kind == VX_DISPATCH || kind == VX_DISPATCH_TF32) {
        // The seven assert_eq! of src/linalg/gemm.rs:70-104, in their order.
        const bool ok = lo.size[0] == ll.size[0] && lo.size[1] == ll.size[1] &&
                        ll.size[0] == lr.size[0] && ll.size[1] == lr.size[1] &&
                        lo.size[2] == ll.size[2] && lo.size[3] == lr.size[3] &&
                        ll.size[3] == lr.size[2];
        if (!ok)
            return fail(VX_ERR_SHAPE,
                        "incompatible gemm shapes: [%u,%u,%u,%u] = [%u,%u,%u,%u] x [%u,%u,%u,%u]",
                        lo.size[0], lo.size[1], lo.size[2], lo.size[3], ll.size[0], ll.size[1],
                        ll.size[2], ll.size[3], lr.size[0], lr.size[1], lr.size[2], lr.size[3]);
    }

    vx_shapes3 s;
    vx_layout_to_shape(&lo, &s.out);
    vx_layout_to_shape(&ll, &s.lhs);
    vx_layout_to_shape(&lr, &s.rhs);

    // TensorRef::buffer() = buffer.slice(offset..) — src/tensor/tensor_ref.rs:101-103.
    VX_REQUIRE(out_cap == 0 || out_layout->offset <= out_cap, VX_ERR_OUT_OF_BOUNDS,
               "out view offset %u beyond its buffer (%llu)", out_layout->offset, (unsigned long long)out_cap);
    VX_REQUIRE(lhs_cap == 0 || lhs_layout->offset <= lhs_cap, VX_ERR_OUT_OF_BOUNDS,
               "lhs view offset %u beyond its buffer (%llu)", lhs_layout->offset, (unsigned long long)lhs_cap);
    VX_REQUIRE(rhs_cap == 0 || rhs_layout->offset <= rhs_cap, VX_ERR_OUT_OF_BOUNDS,
               "rhs view offset %u beyond its buffer (%llu)", rhs_layout->offset, (unsigned long long)rhs_cap);
    float* o = out ? out + out_layout->offset : nullptr;
    const float* l = lhs ? lhs + lhs_layout->offset : nullptr;
    const float* r = rhs ? rhs + rhs_layout->offset : nullptr;
    auto remaining = [](uint64_t cap, uint32_t off) -> int64_t {
        return cap == 0 ? -1 : (int64_t)(cap - off);
    };

    vx_gemm_mode mode = VX_GEMM_AUTO;
    switch (kind) {
        case VX_DISPATCH: mode = VX_GEMM_AUTO; break;
        case VX_DISPATCH_NAIVE: mode = VX_GEMM_NAIVE; break;
        case VX_DISPATCH_TILED: mode = VX_GEMM_SIMT_EXACT; break;
        case VX_DISPATCH_TF32: mode = VX_GEMM_TF32; break;
    }
    return gemm_impl(ctx, mode, o, l, r, s, remaining(out_cap, out_layout->offset),
                     remaining(lhs_cap, lhs_layout->offset), remaining(rhs_cap, rhs_layout->offset));
}

}  // extern "C"
