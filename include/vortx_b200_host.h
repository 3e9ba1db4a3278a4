/*
 * vortx_b200 — host side of the matmul path: the view/stride algebra of
 * vortx's TensorLayout and the Gemm::dispatch entry that consumes it.
 *
 * In a Rust build these stay in vortx's own src/shapes.rs and src/linalg/gemm.rs and
 * only vortx_b200.h is bound.  They are provided here, in C, for hosts without that
 * code; argument meaning and results follow the reference function named beside each
 * declaration.  Where the reference panics, these return VX_ERR_INVALID_ARGUMENT
 * (VX_ERR_SHAPE for Gemm::dispatch's shape asserts) and leave *out untouched.
 */
#ifndef VORTX_B200_HOST_H
#define VORTX_B200_HOST_H

#include "vortx_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* src/shapes.rs:49-60 — sizes, strides (elements), rank and buffer offset of a view. */
typedef struct {
    uint32_t size[4];
    uint32_t stride[4];
    uint32_t rank;
    uint32_t offset;
} vx_layout;

/* src/shapes.rs:85-99 */
VX_API vx_status vx_layout_contiguous(const uint32_t* size, uint32_t rank, vx_layout* out);
/* src/shapes.rs:20-47 — sizes beyond the rank become 1 and take the last real stride. */
VX_API vx_status vx_layout_to_shape(const vx_layout* l, vx_shape* out);
/* src/shapes.rs:145-155 — pads to rank 4 with ones on the left; the offset is dropped. */
VX_API vx_status vx_layout_canonicalize(const vx_layout* l, vx_layout* out);
/* src/shapes.rs:115-141 — VX_ERR_UNSUPPORTED where the reference returns None. */
VX_API vx_status vx_layout_unsqueeze_to_rank(const vx_layout* l, uint32_t rank, vx_layout* out);
/* src/shapes.rs:161-175 — VX_ERR_UNSUPPORTED where the reference returns None (rank already 4,
 * axis > rank); axis 3 makes the reference index stride[4] and panic: VX_ERR_INVALID_ARGUMENT. */
VX_API vx_status vx_layout_unsqueeze(const vx_layout* l, uint32_t axis, vx_layout* out);
/* src/shapes.rs:177-200 */
VX_API vx_status vx_layout_squeeze_axis(const vx_layout* l, uint32_t axis, vx_layout* out);
/* src/shapes.rs:202-230 */
VX_API vx_status vx_layout_squeeze(const vx_layout* l, vx_layout* out);
/* src/shapes.rs:232-234 */
VX_API vx_status vx_layout_index(const vx_layout* l, uint32_t i, vx_layout* out);
/* src/shapes.rs:238-254 */
VX_API vx_status vx_layout_transpose(const vx_layout* l, uint32_t axis_a, uint32_t axis_b,
                                     vx_layout* out);
/* src/shapes.rs:256-259 */
VX_API vx_status vx_layout_transpose_last_dims(const vx_layout* l, vx_layout* out);
/* src/shapes.rs:268-329 */
VX_API vx_status vx_layout_permute(const vx_layout* l, const uint32_t perm[4], vx_layout* out);
/* src/shapes.rs:262-265 */
VX_API vx_status vx_layout_permute_ggml(const vx_layout* l, const uint32_t perm[4], vx_layout* out);
/* src/shapes.rs:332-343 */
VX_API int32_t vx_layout_is_contiguous(const vx_layout* l);
/* src/shapes.rs:346-389 — VX_ERR_SHAPE when the shapes cannot be broadcast (None). */
VX_API vx_status vx_layout_broadcast(const vx_layout* a, const vx_layout* b, vx_layout* out_a,
                                     vx_layout* out_b);
/* src/shapes.rs:393-404 */
VX_API vx_status vx_layout_broadcast_assign(const vx_layout* target, const vx_layout* source,
                                            vx_layout* out_target, vx_layout* out_source);
/* src/shapes.rs:407-441 — stride_set[k] != 0 means stride[k] is given (Some), else derived. */
VX_API vx_status vx_layout_view(const vx_layout* l, uint32_t offset, const uint32_t* shape,
                                uint32_t shape_len, const uint32_t* stride,
                                const uint8_t* stride_set, uint32_t stride_len, vx_layout* out);
/* src/shapes.rs:108-110 */
VX_API vx_status vx_layout_reshape(const vx_layout* l, const uint32_t* shape, uint32_t shape_len,
                                   vx_layout* out);
/* src/shapes.rs:443-464 */
VX_API vx_status vx_layout_narrow(const vx_layout* l, uint32_t axis, uint32_t first,
                                  uint32_t count, vx_layout* out);
/* src/shapes.rs:467-489 — matrix narrows axis 2, columns axis 1, rows axis 0. */
VX_API vx_status vx_layout_matrix(const vx_layout* l, uint32_t matrix_id, vx_layout* out);
VX_API vx_status vx_layout_columns(const vx_layout* l, uint32_t first, uint32_t count,
                                   vx_layout* out);
VX_API vx_status vx_layout_rows(const vx_layout* l, uint32_t first, uint32_t count, vx_layout* out);
/* src/shapes.rs:492-519 */
VX_API vx_status vx_layout_f32_to_vec4(const vx_layout* l, vx_layout* out);
/* src/shapes.rs:527-533 — product of the sizes within the rank, at least 1. */
VX_API uint64_t vx_layout_len(const vx_layout* l);
/* Largest element index a canonical layout reaches, plus one (0 for an empty view). */
VX_API uint64_t vx_layout_span(const vx_layout* l);

/* Which entry of src/linalg/gemm.rs the call stands for. */
typedef enum {
    VX_DISPATCH = 0,       /* Gemm::dispatch — :47-187: shape asserts, then the tiled/naive rule */
    VX_DISPATCH_NAIVE = 1, /* Gemm::dispatch_naive — :190-246: no asserts                      */
    VX_DISPATCH_TILED = 2, /* Gemm::dispatch_tiled — :249-305: no asserts                      */
    VX_DISPATCH_TF32 = 3   /* asserts as VX_DISPATCH, then the tensor-core kernel (no reference
                              counterpart; same result within TF32 rounding)                  */
} vx_dispatch_kind;

/* out/lhs/rhs are the BASE device pointers of the underlying buffers and *_cap their
 * lengths in elements; the view offset in each layout is applied here, as
 * TensorRef::buffer() does (src/tensor/tensor_ref.rs:101-103). */
VX_API vx_status vx_gemm_dispatch(vx_context* ctx, vx_dispatch_kind kind, float* out,
                                  const vx_layout* out_layout, uint64_t out_cap, const float* lhs,
                                  const vx_layout* lhs_layout, uint64_t lhs_cap, const float* rhs,
                                  const vx_layout* rhs_layout, uint64_t rhs_cap);

/* OpAssign::launch — src/linalg/op_assign.rs:38-143 — and, with is_repeat != 0, Repeat::launch —
 * src/linalg/repeat.rs:24-88: broadcast_assign(a, b) (VX_ERR_SHAPE where the reference panics on
 * incompatible shapes), canonicalise both, apply the view offsets, launch.  a and b are the base
 * pointers of the underlying buffers, *_cap their lengths in elements. */
VX_API vx_status vx_op_assign_dispatch(vx_context* ctx, vx_op op, int32_t is_repeat, float* a,
                                       const vx_layout* layout_a, uint64_t cap_a, const float* b,
                                       const vx_layout* layout_b, uint64_t cap_b);

#ifdef __cplusplus
}
#endif
#endif /* VORTX_B200_HOST_H */
