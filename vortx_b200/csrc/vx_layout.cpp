// Host view/stride algebra (vx_layout_*), following vortx's TensorLayout in src/shapes.rs.
// Every function validates first and writes *out only on success.
#include <algorithm>
#include <cstring>

#include "vx_internal.h"

namespace {

using vx::fail;

vx_layout make_contiguous(const uint32_t size_in[4], uint32_t rank) {
    vx_layout l;
    for (int k = 0; k < 4; ++k) {
        l.size[k] = (uint32_t)k < rank ? size_in[k] : 1u;
        l.stride[k] = 1;
    }
    uint32_t run = 1;
    for (int k = (int)rank - 1; k >= 0; --k) {
        l.stride[k] = run;
        run *= l.size[k];
    }
    l.rank = rank;
    l.offset = 0;
    return l;
}

bool valid(const vx_layout* l) { return l != nullptr && l->rank <= 4; }

bool contiguous(const vx_layout& l) {
    uint32_t expect = 1;
    for (int i = (int)l.rank - 1; i >= 0; --i) {
        if (l.stride[i] != 0 && l.stride[i] != expect) return false;
        expect *= l.size[i];
    }
    return true;
}

}  // namespace

extern "C" {

vx_status vx_layout_contiguous(const uint32_t* size, uint32_t rank, vx_layout* out) {
    VX_REQUIRE(out && (size || rank == 0), VX_ERR_INVALID_ARGUMENT, "vx_layout_contiguous: null argument");
    VX_REQUIRE(rank <= 4, VX_ERR_INVALID_ARGUMENT, "tensors of ranks > 4 not supported");
    uint32_t padded[4] = {1, 1, 1, 1};
    for (uint32_t k = 0; k < rank; ++k) padded[k] = size[k];
    *out = make_contiguous(padded, rank);
    return VX_OK;
}

vx_status vx_layout_to_shape(const vx_layout* l, vx_shape* out) {
    VX_REQUIRE(valid(l) && out, VX_ERR_INVALID_ARGUMENT, "vx_layout_to_shape: bad argument");
    uint32_t size[4], stride[4];
    std::memcpy(size, l->size, sizeof size);
    std::memcpy(stride, l->stride, sizeof stride);
    for (uint32_t k = l->rank; k < 4; ++k) {
        size[k] = 1;
        stride[k] = l->rank > 0 ? stride[l->rank - 1] : 1;
    }
    *out = vx_shape{size[0], size[1], size[2], size[3], stride[0], stride[1], stride[2], stride[3]};
    return VX_OK;
}

vx_status vx_layout_canonicalize(const vx_layout* l, vx_layout* out) {
    VX_REQUIRE(valid(l) && out, VX_ERR_INVALID_ARGUMENT, "vx_layout_canonicalize: bad argument");
    if (l->rank == 4) {
        *out = *l;
        return VX_OK;
    }
    const uint32_t pad = 4 - l->rank;
    uint32_t size[4] = {1, 1, 1, 1};
    for (uint32_t k = 0; k < l->rank; ++k) size[pad + k] = l->size[k];
    vx_layout r = make_contiguous(size, 4);
    for (uint32_t k = 0; k < l->rank; ++k) r.stride[pad + k] = l->stride[k];
    *out = r;  // offset 0: the view offset travels with the buffer slice instead
    return VX_OK;
}

vx_status vx_layout_unsqueeze_to_rank(const vx_layout* l, uint32_t rank, vx_layout* out) {
    VX_REQUIRE(valid(l) && out, VX_ERR_INVALID_ARGUMENT, "vx_layout_unsqueeze_to_rank: bad argument");
    // The reference returns None here, not a panic.
    VX_REQUIRE(rank <= 4 && rank >= l->rank, VX_ERR_UNSUPPORTED,
               "cannot unsqueeze rank %u to rank %u", l->rank, rank);
    vx_layout r = *l;
    if (l->rank == rank) {
        *out = r;
        return VX_OK;
    }
    if (l->rank == 0) {
        for (int k = 0; k < 4; ++k) r.size[k] = r.stride[k] = 1;
    } else {
        const uint32_t tail = l->stride[l->rank - 1] * l->size[l->rank - 1];
        for (uint32_t k = l->rank; k < 4; ++k) {
            r.size[k] = 1;
            r.stride[k] = tail;
        }
    }
    r.rank = rank;
    *out = r;
    return VX_OK;
}

vx_status vx_layout_unsqueeze(const vx_layout* l, uint32_t axis, vx_layout* out) {
    VX_REQUIRE(valid(l) && out, VX_ERR_INVALID_ARGUMENT, "vx_layout_unsqueeze: bad argument");
    // The reference returns None here, not a panic.
    VX_REQUIRE(l->rank < 4 && axis <= l->rank, VX_ERR_UNSUPPORTED,
               "Not enough rank available for unsqueezing (rank %u, axis %u)", l->rank, axis);
    // Appending an axis to a rank-3 layout reads stride[4] in the reference and panics there.
    VX_REQUIRE(axis < 3, VX_ERR_INVALID_ARGUMENT, "unsqueeze at axis 3 indexes past the stride array");
    vx_layout r = *l;
    for (int i = 2; i >= (int)axis; --i) {
        r.size[i + 1] = r.size[i];
        r.stride[i + 1] = r.stride[i];
    }
    r.size[axis] = 1;
    r.stride[axis] = r.stride[axis + 1];  // keeps is_contiguous true for contiguous inputs
    r.rank = l->rank + 1;
    *out = r;
    return VX_OK;
}

vx_status vx_layout_squeeze_axis(const vx_layout* l, uint32_t axis, vx_layout* out) {
    VX_REQUIRE(valid(l) && out, VX_ERR_INVALID_ARGUMENT, "vx_layout_squeeze_axis: bad argument");
    VX_REQUIRE(axis < l->rank, VX_ERR_INVALID_ARGUMENT, "axis out of bounds");
    VX_REQUIRE(l->size[axis] == 1, VX_ERR_INVALID_ARGUMENT, "can only squeeze an axis with length 1");
    vx_layout r = *l;
    for (uint32_t k = axis; k + 1 < l->rank; ++k) {
        r.size[k] = r.size[k + 1];
        r.stride[k] = r.stride[k + 1];
    }
    r.rank = l->rank - 1;
    r.size[r.rank] = 1;
    if (r.rank > 0) {
        uint32_t prod = 1;
        for (uint32_t k = 0; k + 1 < r.rank; ++k) prod *= r.size[k];
        r.stride[r.rank] = prod;
    }
    *out = r;
    return VX_OK;
}

vx_status vx_layout_squeeze(const vx_layout* l, vx_layout* out) {
    VX_REQUIRE(valid(l) && out, VX_ERR_INVALID_ARGUMENT, "vx_layout_squeeze: bad argument");
    vx_layout r = *l;
    uint32_t kept = 0;
    for (uint32_t k = 0; k < l->rank; ++k)
        if (l->size[k] != 1) {
            r.size[kept] = l->size[k];
            r.stride[kept] = l->stride[k];
            ++kept;
        }
    if (kept == 0) {
        for (int k = 0; k < 4; ++k) r.size[k] = r.stride[k] = 1;
        r.rank = 0;
    } else {
        const uint32_t tail = r.stride[kept - 1] * r.size[kept - 1];
        for (uint32_t k = kept; k < 4; ++k) {
            r.size[k] = 1;
            r.stride[k] = tail;
        }
        r.rank = kept;
    }
    *out = r;
    return VX_OK;
}

vx_status vx_layout_index(const vx_layout* l, uint32_t i, vx_layout* out) {
    vx_layout t;
    vx_status st = vx_layout_narrow(l, 0, i, 1, &t);
    if (st != VX_OK) return st;
    return vx_layout_squeeze_axis(&t, 0, out);
}

vx_status vx_layout_transpose(const vx_layout* l, uint32_t a, uint32_t b, vx_layout* out) {
    VX_REQUIRE(valid(l) && out, VX_ERR_INVALID_ARGUMENT, "vx_layout_transpose: bad argument");
    VX_REQUIRE(a < l->rank, VX_ERR_INVALID_ARGUMENT, "transpose axis index out of bounds: %u >= %u", a, l->rank);
    VX_REQUIRE(b < l->rank, VX_ERR_INVALID_ARGUMENT, "transpose axis index out of bounds: %u >= %u", b, l->rank);
    vx_layout r = *l;
    std::swap(r.size[a], r.size[b]);
    std::swap(r.stride[a], r.stride[b]);
    *out = r;
    return VX_OK;
}

vx_status vx_layout_transpose_last_dims(const vx_layout* l, vx_layout* out) {
    VX_REQUIRE(valid(l) && out, VX_ERR_INVALID_ARGUMENT, "vx_layout_transpose_last_dims: bad argument");
    VX_REQUIRE(l->rank >= 2, VX_ERR_INVALID_ARGUMENT, "transpose_last_dims needs rank >= 2");
    return vx_layout_transpose(l, l->rank - 2, l->rank - 1, out);
}

vx_status vx_layout_permute(const vx_layout* l, const uint32_t perm[4], vx_layout* out) {
    VX_REQUIRE(valid(l) && perm && out, VX_ERR_INVALID_ARGUMENT, "vx_layout_permute: bad argument");
    for (int i = 0; i < 4; ++i) {
        VX_REQUIRE(perm[i] < 4, VX_ERR_INVALID_ARGUMENT, "permutation index %u out of range", perm[i]);
        for (int j = i + 1; j < 4; ++j)
            VX_REQUIRE(perm[i] != perm[j], VX_ERR_INVALID_ARGUMENT, "Permutation indices must not overlap.");
    }
    for (uint32_t k = 0; k < l->rank; ++k)
        VX_REQUIRE(perm[k] < l->rank, VX_ERR_INVALID_ARGUMENT,
                   "permutation index %u exceeds this matrix rank %u", perm[k], l->rank);
    for (uint32_t k = l->rank; k < 4; ++k)
        VX_REQUIRE(perm[k] == k, VX_ERR_INVALID_ARGUMENT,
                   "Indices exceeding the tensor rank %u must be identity", l->rank);
    vx_layout r = *l;
    for (int k = 0; k < 4; ++k) {
        r.size[perm[k]] = l->size[k];
        r.stride[perm[k]] = l->stride[k];
    }
    *out = r;
    return VX_OK;
}

vx_status vx_layout_permute_ggml(const vx_layout* l, const uint32_t perm[4], vx_layout* out) {
    VX_REQUIRE(perm, VX_ERR_INVALID_ARGUMENT, "vx_layout_permute_ggml: bad argument");
    // GGML swaps the two leading dimensions (src/shapes.rs:15-18): swap the first two
    // entries, then map every entry through [1, 0, 2, 3].
    static const uint32_t ggml_ids[4] = {1, 0, 2, 3};
    uint32_t p[4] = {perm[1], perm[0], perm[2], perm[3]};
    for (int i = 0; i < 4; ++i) {
        VX_REQUIRE(p[i] < 4, VX_ERR_INVALID_ARGUMENT, "permutation index %u out of range", p[i]);
        p[i] = ggml_ids[p[i]];
    }
    return vx_layout_permute(l, p, out);
}

int32_t vx_layout_is_contiguous(const vx_layout* l) { return valid(l) && contiguous(*l) ? 1 : 0; }

vx_status vx_layout_broadcast(const vx_layout* a_in, const vx_layout* b_in, vx_layout* out_a,
                              vx_layout* out_b) {
    VX_REQUIRE(valid(a_in) && valid(b_in) && out_a && out_b, VX_ERR_INVALID_ARGUMENT,
               "vx_layout_broadcast: bad argument");
    // Work with the lower-rank operand in `lo`.
    const bool flipped = a_in->rank > b_in->rank;
    vx_layout lo = flipped ? *b_in : *a_in;
    vx_layout hi = flipped ? *a_in : *b_in;

    const uint32_t shift = hi.rank - lo.rank;
    for (int k = (int)lo.rank - 1; k >= 0; --k) {
        lo.size[k + shift] = lo.size[k];
        lo.stride[k + shift] = lo.stride[k];
    }
    for (uint32_t k = 0; k < shift; ++k) lo.size[k] = 1;
    lo.rank = hi.rank;

    for (uint32_t k = 0; k < lo.rank; ++k) {
        if (lo.size[k] == 1) lo.stride[k] = 0;
        if (hi.size[k] == 1) hi.stride[k] = 0;
    }
    for (uint32_t k = 0; k < lo.rank; ++k)
        if (lo.size[k] != 1 && hi.size[k] != 1 && lo.size[k] != hi.size[k])
            return fail(VX_ERR_SHAPE, "shapes cannot be broadcast along axis %u (%u vs %u)", k,
                        lo.size[k], hi.size[k]);

    *out_a = flipped ? hi : lo;
    *out_b = flipped ? lo : hi;
    return VX_OK;
}

vx_status vx_layout_broadcast_assign(const vx_layout* target, const vx_layout* source,
                                     vx_layout* out_target, vx_layout* out_source) {
    vx_layout t, s;
    vx_status st = vx_layout_broadcast(target, source, &t, &s);
    if (st != VX_OK) return st;
    for (uint32_t k = 0; k < t.rank; ++k)
        if (t.size[k] < s.size[k])
            return fail(VX_ERR_SHAPE, "assignment would grow the target along axis %u", k);
    *out_target = t;
    *out_source = s;
    return VX_OK;
}

vx_status vx_layout_view(const vx_layout* l, uint32_t offset, const uint32_t* shape,
                         uint32_t shape_len, const uint32_t* stride, const uint8_t* stride_set,
                         uint32_t stride_len, vx_layout* out) {
    VX_REQUIRE(valid(l) && out && (shape || shape_len == 0), VX_ERR_INVALID_ARGUMENT,
               "vx_layout_view: bad argument");
    VX_REQUIRE(shape_len <= 4 && stride_len <= shape_len, VX_ERR_INVALID_ARGUMENT,
               "view: shape longer than 4 or stride list longer than the shape");
    VX_REQUIRE(stride_len == 0 || (stride && stride_set), VX_ERR_INVALID_ARGUMENT, "view: null strides");
    VX_REQUIRE(contiguous(*l), VX_ERR_INVALID_ARGUMENT, "Cannot take a view of a non-contiguous tensor.");

    // u32 products, wrapping, as in the reference.
    uint32_t available = 1;
    for (int k = 0; k < 4; ++k) available *= l->size[k];
    uint32_t needed = 1;
    for (uint32_t k = 0; k < shape_len; ++k) needed *= shape[k];
    needed += offset;
    VX_REQUIRE(needed <= available, VX_ERR_INVALID_ARGUMENT,
               "Source tensor is too small for reshaping. Expected at least %u elements, found %u",
               needed, available);

    vx_layout r;
    for (int k = 0; k < 4; ++k) {
        r.size[k] = (uint32_t)k < shape_len ? shape[k] : 1u;
        r.stride[k] = 0;
    }
    uint32_t run = 1;
    for (int k = (int)shape_len - 1; k >= 0; --k) {
        const bool given = (uint32_t)k < stride_len && stride_set[k];
        r.stride[k] = given ? stride[k] : run;
        run = r.stride[k] * r.size[k];
    }
    r.rank = shape_len;
    r.offset = l->offset + offset;
    *out = r;
    return VX_OK;
}

vx_status vx_layout_reshape(const vx_layout* l, const uint32_t* shape, uint32_t shape_len,
                            vx_layout* out) {
    return vx_layout_view(l, 0, shape, shape_len, nullptr, nullptr, 0, out);
}

vx_status vx_layout_narrow(const vx_layout* l, uint32_t axis, uint32_t first, uint32_t count,
                           vx_layout* out) {
    VX_REQUIRE(valid(l) && out, VX_ERR_INVALID_ARGUMENT, "vx_layout_narrow: bad argument");
    VX_REQUIRE(axis < l->rank, VX_ERR_INVALID_ARGUMENT, "Axis index out of bounds.");
    VX_REQUIRE((uint64_t)first + count <= l->size[axis], VX_ERR_INVALID_ARGUMENT,
               "narrow: %u + %u > %u", first, count, l->size[axis]);
    vx_layout r = *l;
    r.size[axis] = count;
    r.offset = l->offset + l->stride[axis] * first;
    *out = r;
    return VX_OK;
}

vx_status vx_layout_matrix(const vx_layout* l, uint32_t id, vx_layout* out) {
    return vx_layout_narrow(l, 2, id, 1, out);
}
vx_status vx_layout_columns(const vx_layout* l, uint32_t first, uint32_t count, vx_layout* out) {
    return vx_layout_narrow(l, 1, first, count, out);
}
vx_status vx_layout_rows(const vx_layout* l, uint32_t first, uint32_t count, vx_layout* out) {
    return vx_layout_narrow(l, 0, first, count, out);
}

vx_status vx_layout_f32_to_vec4(const vx_layout* l, vx_layout* out) {
    VX_REQUIRE(valid(l) && out, VX_ERR_INVALID_ARGUMENT, "vx_layout_f32_to_vec4: bad argument");
    const uint32_t dim = std::max<uint32_t>(l->rank, 1) - 1;
    VX_REQUIRE(l->stride[dim] == 1, VX_ERR_INVALID_ARGUMENT,
               "Cannot convert from f32 to vec4 with a stride[%u] of %u != 1", dim, l->stride[dim]);
    VX_REQUIRE(l->size[dim] % 4 == 0, VX_ERR_INVALID_ARGUMENT, "Matrix row count no properly aligned.");
    vx_layout r = *l;
    for (int k = 0; k < 4; ++k) {
        VX_REQUIRE(l->stride[k] == 1 || l->stride[k] % 4 == 0, VX_ERR_INVALID_ARGUMENT,
                   "stride[%d] = %u is neither 1 nor a multiple of 4", k, l->stride[k]);
        r.stride[k] = (l->stride[k] + 3) / 4;
    }
    r.size[dim] = l->size[dim] / 4;
    *out = r;
    return VX_OK;
}

uint64_t vx_layout_len(const vx_layout* l) {
    if (!valid(l)) return 0;
    uint64_t n = 1;
    for (uint32_t k = 0; k < l->rank; ++k) n *= l->size[k];
    return std::max<uint64_t>(n, 1);
}

uint64_t vx_layout_span(const vx_layout* l) {
    if (!valid(l)) return 0;
    uint64_t last = 0;
    for (uint32_t k = 0; k < l->rank; ++k) {
        if (l->size[k] == 0) return 0;
        last += (uint64_t)(l->size[k] - 1) * l->stride[k];
    }
    return last + 1;
}

}  // extern "C"
