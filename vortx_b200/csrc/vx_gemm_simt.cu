// SIMT f32 GEMM kernels whose results are bit-identical to vortx's shaders.
//
// vortx-shaders/src/linalg/gemm.rs computes every output element as
//     acc = 0; for k ascending: acc = round(acc + round(a[k] * b[k]))
// (gemm_naive :225-236, gemm_tiled :137-167 — the tiled kernel only changes which
// invocation owns which element and pads K with zero terms, which leave acc unchanged).
// The kernels here keep exactly that per-element order and rounding — __fmul_rn then
// __fadd_rn, never a fused multiply-add, never a split of the k range — and are free to
// tile M and N differently.
#include "vx_internal.h"

namespace {

__device__ __forceinline__ uint32_t shape_it(const vx_shape& s, uint32_t n, uint32_t c, uint32_t h,
                                             uint32_t w) {
    // vortx-shaders/src/linalg/shape.rs:46-48 (u32, wrapping)
    return n * s.n_stride + c * s.c_stride + h * s.h_stride + w * s.w_stride;
}

// ---------------------------------------------------------------- naive -------
// One thread per output element and per batch matrix (gemm_naive walks n serially in the
// thread; the order across n does not touch any element's sum).
__global__ void __launch_bounds__(256)
gemm_naive_kernel(float* __restrict__ out, const float* __restrict__ lhs,
                  const float* __restrict__ rhs, const vx_shapes3 s) {
    const uint32_t col = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t row = blockIdx.y * blockDim.y + threadIdx.y;
    if (col >= s.out.w || row >= s.out.h) return;
    const uint32_t c = blockIdx.z % s.out.c;
    const uint32_t n = blockIdx.z / s.out.c;
    const uint32_t k = s.lhs.w;
    float sum = 0.0f;
    for (uint32_t j = 0; j < k; ++j) {
        const float a = lhs[shape_it(s.lhs, n, c, row, j)];
        const float b = rhs[shape_it(s.rhs, n, c, j, col)];
        sum = __fadd_rn(sum, __fmul_rn(a, b));
    }
    out[shape_it(s.out, n, c, row, col)] = sum;
}

// --------------------------------------------------------- generic strides ----
// 64x64 output tile, K stepped by 16, 4x4 outputs per thread, any strides: the shape of
// the reference kernel, used when the operands do not allow vector loads.
constexpr int G_TM = 64, G_TN = 64, G_TK = 16;

__global__ void __launch_bounds__(256)
gemm_tiled_generic_kernel(float* __restrict__ out, const float* __restrict__ lhs,
                          const float* __restrict__ rhs, const vx_shapes3 s) {
    __shared__ float sa[G_TK][G_TM + 1];
    __shared__ float sb[G_TK][G_TN + 1];

    const uint32_t tid = threadIdx.x;
    const uint32_t tx = tid % 16, ty = tid / 16;
    const uint32_t tile_row = blockIdx.y * G_TM, tile_col = blockIdx.x * G_TN;
    const uint32_t c = blockIdx.z % s.out.c;
    const uint32_t n = blockIdx.z / s.out.c;
    const uint32_t m = s.out.h, nn = s.out.w, k = s.lhs.w;

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (uint32_t k0 = 0; k0 < k; k0 += G_TK) {
        for (uint32_t i = tid; i < G_TM * G_TK; i += 256) {
            const uint32_t r = i / G_TK, kk = i % G_TK;
            const uint32_t gr = tile_row + r, gk = k0 + kk;
            sa[kk][r] = (gr < m && gk < k) ? lhs[shape_it(s.lhs, n, c, gr, gk)] : 0.0f;
        }
        for (uint32_t i = tid; i < G_TK * G_TN; i += 256) {
            const uint32_t kk = i / G_TN, cc = i % G_TN;
            const uint32_t gk = k0 + kk, gc = tile_col + cc;
            sb[kk][cc] = (gk < k && gc < nn) ? rhs[shape_it(s.rhs, n, c, gk, gc)] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < G_TK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = sa[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = sb[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], b[j]));
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t r = tile_row + ty * 4 + i;
        if (r >= m) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t cc = tile_col + tx * 4 + j;
            if (cc < nn) out[shape_it(s.out, n, c, r, cc)] = acc[i][j];
        }
    }
}

// ------------------------------------------------------------ vector path -----
// Row-major operands (unit stride along w, rows and bases 16-byte aligned): BM x 128 output
// tile (BM = 128, or 64 when 128-row tiles would leave SMs without work), K stepped by 8,
// (BM / 16) x 8 outputs per thread held as 4-wide pieces so that every shared-memory read is a
// conflict-free 128-bit load.  Global tiles for step t+1 are fetched into registers while step t is
// multiplied (one barrier per step).  Every output element is still accumulated k ascending,
// multiply then add: the tile shape does not change a bit of the result.
constexpr int V_BN = 128, V_BK = 8;

template <int V_BM>
__global__ void __launch_bounds__(256, 2)
gemm_tiled_vec_kernel(float* __restrict__ out, const float* __restrict__ lhs,
                      const float* __restrict__ rhs, const vx_shapes3 s) {
    constexpr int V_AS = V_BM + 4;       // padded row of the transposed A tile
    constexpr int RH = V_BM / 64;        // 4-row pieces per thread: rows ty*4.. and (RH = 2) 64 + ty*4..
    constexpr int RT = 4 * RH;           // rows per thread
    __shared__ __align__(16) float sa[2][V_BK][V_AS];
    __shared__ __align__(16) float sb[2][V_BK][V_BN];

    const uint32_t tid = threadIdx.x;
    const uint32_t tx = tid % 16, ty = tid / 16;
    const uint32_t tile_row = blockIdx.y * V_BM, tile_col = blockIdx.x * V_BN;
    const uint32_t c = blockIdx.z % s.out.c;
    const uint32_t n = blockIdx.z / s.out.c;
    const uint32_t m = s.out.h, nn = s.out.w, k = s.lhs.w;

    const float* __restrict__ A = lhs + (size_t)n * s.lhs.n_stride + (size_t)c * s.lhs.c_stride;
    const float* __restrict__ B = rhs + (size_t)n * s.rhs.n_stride + (size_t)c * s.rhs.c_stride;
    float* __restrict__ C = out + (size_t)n * s.out.n_stride + (size_t)c * s.out.c_stride;
    const size_t lda = s.lhs.h_stride, ldb = s.rhs.h_stride, ldc = s.out.h_stride;

    // Loader roles: A tile BM rows x 8 k = 2 BM float4 (threads below 2 BM take one each); B tile 8 k x 128 =
    // 256 float4 (one per thread).
    const bool a_loader = tid < 2 * V_BM;
    const uint32_t a_row = tid / 2, a_k = (tid % 2) * 4;
    const uint32_t b_k = tid / 32, b_col = (tid % 32) * 4;

    auto load_a = [&](uint32_t k0) -> float4 {
        const uint32_t gr = tile_row + a_row, gk = k0 + a_k;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (a_loader && gr < m) {
            const float* p = A + (size_t)gr * lda + gk;
            if (gk + 3 < k) {
                v = *reinterpret_cast<const float4*>(p);
            } else {
                if (gk + 0 < k) v.x = p[0];
                if (gk + 1 < k) v.y = p[1];
                if (gk + 2 < k) v.z = p[2];
            }
        }
        return v;
    };
    auto load_b = [&](uint32_t k0) -> float4 {
        const uint32_t gk = k0 + b_k, gc = tile_col + b_col;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (gk < k) {
            const float* p = B + (size_t)gk * ldb + gc;
            if (gc + 3 < nn) {
                v = *reinterpret_cast<const float4*>(p);
            } else {
                if (gc + 0 < nn) v.x = p[0];
                if (gc + 1 < nn) v.y = p[1];
                if (gc + 2 < nn) v.z = p[2];
            }
        }
        return v;
    };
    auto store_tiles = [&](int buf, const float4& va, const float4& vb) {
        if (a_loader) {
            sa[buf][a_k + 0][a_row] = va.x;
            sa[buf][a_k + 1][a_row] = va.y;
            sa[buf][a_k + 2][a_row] = va.z;
            sa[buf][a_k + 3][a_row] = va.w;
        }
        *reinterpret_cast<float4*>(&sb[buf][b_k][b_col]) = vb;
    };

    float acc[RT][8];
#pragma unroll
    for (int i = 0; i < RT; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.0f;

    float4 ra = load_a(0), rb = load_b(0);
    store_tiles(0, ra, rb);
    __syncthreads();

    int buf = 0;
    for (uint32_t k0 = 0; k0 < k; k0 += V_BK) {
        const bool more = k0 + V_BK < k;
        if (more) {
            ra = load_a(k0 + V_BK);
            rb = load_b(k0 + V_BK);
        }
#pragma unroll
        for (int kk = 0; kk < V_BK; ++kk) {
            float a[RT];
#pragma unroll
            for (int h = 0; h < RH; ++h) {
                const float4 av = *reinterpret_cast<const float4*>(&sa[buf][kk][h * 64 + ty * 4]);
                a[4 * h + 0] = av.x; a[4 * h + 1] = av.y; a[4 * h + 2] = av.z; a[4 * h + 3] = av.w;
            }
            const float4 b0 = *reinterpret_cast<const float4*>(&sb[buf][kk][tx * 4]);
            const float4 b1 = *reinterpret_cast<const float4*>(&sb[buf][kk][64 + tx * 4]);
            const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for (int i = 0; i < RT; ++i)
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], b[j]));
        }
        if (more) {
            store_tiles(buf ^ 1, ra, rb);
            __syncthreads();
            buf ^= 1;
        }
    }

#pragma unroll
    for (int i = 0; i < RT; ++i) {
        const uint32_t r = tile_row + (i / 4) * 64 + ty * 4 + (i % 4);
        if (r >= m) continue;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const uint32_t cc = tile_col + h * 64 + tx * 4;
            float* p = C + (size_t)r * ldc + cc;
            if (cc + 3 < nn) {
                *reinterpret_cast<float4*>(p) =
                    make_float4(acc[i][h * 4 + 0], acc[i][h * 4 + 1], acc[i][h * 4 + 2], acc[i][h * 4 + 3]);
            } else {
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    if (cc + j < nn) p[j] = acc[i][h * 4 + j];
            }
        }
    }
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Unit stride along w and every row / matrix start 16-byte aligned.
bool vector_friendly(const void* base, const vx_shape& s) {
    if (s.w_stride != 1 && s.w > 1) return false;
    if (!aligned16(base)) return false;
    if (s.h > 1 && s.h_stride % 4 != 0) return false;
    if (s.c > 1 && s.c_stride % 4 != 0) return false;
    if (s.n > 1 && s.n_stride % 4 != 0) return false;
    return true;
}

}  // namespace

namespace vx {

vx_status launch_gemm_naive(vx_context* ctx, float* out, const float* lhs, const float* rhs,
                            const vx_shapes3& s) {
    const uint64_t batches = (uint64_t)s.out.n * s.out.c;
    if (s.out.h == 0 || s.out.w == 0 || batches == 0) return VX_OK;
    VX_REQUIRE(batches <= 65535, VX_ERR_UNSUPPORTED, "more than 65535 batch matrices (%llu)",
               (unsigned long long)batches);
    dim3 block(32, 8, 1);
    dim3 grid((s.out.w + 31) / 32, (s.out.h + 7) / 8, (unsigned)batches);
    VX_REQUIRE(grid.y <= 65535, VX_ERR_UNSUPPORTED, "too many rows for the naive kernel (%u)", s.out.h);
    gemm_naive_kernel<<<grid, block, 0, ctx->stream>>>(out, lhs, rhs, s);
    VX_CUDA(cudaGetLastError());
    ctx->launches++;
    return VX_OK;
}

vx_status launch_gemm_simt_exact(vx_context* ctx, float* out, const float* lhs, const float* rhs,
                                 const vx_shapes3& s, int* kernel) {
    const uint64_t batches = (uint64_t)s.out.n * s.out.c;
    if (kernel) *kernel = 0;
    if (s.out.h == 0 || s.out.w == 0 || batches == 0) return VX_OK;
    VX_REQUIRE(batches <= 65535, VX_ERR_UNSUPPORTED, "more than 65535 batch matrices (%llu)",
               (unsigned long long)batches);
    const bool vec = option(ctx, "gemm.simt.force_generic", 0) == 0 && vector_friendly(out, s.out) &&
                     vector_friendly(lhs, s.lhs) && vector_friendly(rhs, s.rhs);
    if (vec) {
        // 128-row tiles unless they would leave SMs idle (1024^3: 64 tiles for 148 SMs): then 64-row tiles
        const uint64_t tiles128 = (uint64_t)((s.out.w + V_BN - 1) / V_BN) * ((s.out.h + 127) / 128) * batches;
        const int bm = tiles128 >= 2ull * (uint64_t)ctx->sm_count ? 128 : 64;
        dim3 grid((s.out.w + V_BN - 1) / V_BN, (s.out.h + bm - 1) / bm, (unsigned)batches);
        VX_REQUIRE(grid.y <= 65535, VX_ERR_UNSUPPORTED, "too many rows (%u)", s.out.h);
        if (bm == 128) gemm_tiled_vec_kernel<128><<<grid, 256, 0, ctx->stream>>>(out, lhs, rhs, s);
        else gemm_tiled_vec_kernel<64><<<grid, 256, 0, ctx->stream>>>(out, lhs, rhs, s);
        if (kernel) *kernel = 2;
    } else {
        dim3 grid((s.out.w + G_TN - 1) / G_TN, (s.out.h + G_TM - 1) / G_TM, (unsigned)batches);
        VX_REQUIRE(grid.y <= 65535, VX_ERR_UNSUPPORTED, "too many rows (%u)", s.out.h);
        gemm_tiled_generic_kernel<<<grid, 256, 0, ctx->stream>>>(out, lhs, rhs, s);
        if (kernel) *kernel = 4;
    }
    VX_CUDA(cudaGetLastError());
    ctx->launches++;
    return VX_OK;
}

}  // namespace vx
