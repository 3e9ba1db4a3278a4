// Block-quantised weights (Q8_0, Q4_0): host quantisers, the planar device form, device
// dequantisation and the GEMV kernels.
//
// vortx has no quantised type; its matrix-times-vector is Gemm::dispatch with a [K,1]
// right-hand side (src/linalg/gemm.rs:46, :373-387).  These entry points keep that
// calling shape (weights, x, y on the device; overwrite y) for weights stored as blocks
// of 32 with one f16 scale each.
//
// Device form.  A host block stream interleaves a 2-byte scale with 16 or 32 bytes of
// quants, so no block starts on a 16-byte boundary.  vx_qweights_upload splits the same
// bytes into two planes, quants (row-major, 16 / 32 bytes per block) and scales (row-major
// f16), each starting on a 256-byte boundary.  Every device load is then a full, aligned
// 128-bit vector of quants or a 16-bit scale, and the bytes moved per GEMV are exactly
// the 18 / 34 bytes per block of the stream.
//
// GEMV kernels are HBM-bound by design: each weight byte is read once, x is staged once
// per CTA in shared memory (swizzled so that the 128-bit reads of 32 lanes holding 32
// different blocks hit 32 different banks), partial sums stay in registers and are
// combined with warp shuffles.  There is no split along K and no scratch memory.
#include <cuda_fp16.h>

#include <algorithm>
#include <memory>
#include <cmath>
#include <cstring>
#include <new>
#include <vector>

#include "vx_internal.h"

namespace {

using vx::fail;

constexpr int QK = 32;
constexpr size_t kQ8BlockBytes = 34, kQ4BlockBytes = 18;

size_t block_bytes(vx_qtype t) { return t == VX_Q8_0 ? kQ8BlockBytes : kQ4BlockBytes; }
size_t quant_bytes(vx_qtype t) { return t == VX_Q8_0 ? 32 : 16; }
size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// f32 -> f16 (round to nearest even) and back, on the host.
uint16_t host_f2h(float f) {
    return static_cast<__half_raw>(__float2half_rn(f)).x;
}
float host_h2f(uint16_t u) {
    __half_raw raw;
    raw.x = u;
    return __half2float(__half(raw));
}

// ------------------------------------------------------------------ device ------

__device__ __forceinline__ float h2f(uint16_t u) { return __half2float(__ushort_as_half(u)); }

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
    // Weights are read exactly once: keep them out of L1.
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Stages x (B vectors of nb*32 floats) into shared memory as float4 chunks; chunk k of
// block b lands at slot (k + b) & 7 of that block.  Also leaves the per-block sums of x in
// sx when WANT_SUMS.  x must be 16-byte aligned with x_stride % 4 == 0 when `vec` is set.
template <int B, bool WANT_SUMS>
__device__ __forceinline__ void stage_x(float4* xs, float* sx, const float* __restrict__ x,
                                        size_t x_stride, uint32_t nb, bool vec) {
    const uint32_t chunks = nb * 8;
    for (uint32_t v = 0; v < B; ++v) {
        const float* xv = x + (size_t)v * x_stride;
        // Uniform trip count per CTA so that every lane reaches the ballot.
        for (uint32_t base = 0; base < chunks; base += blockDim.x) {
            const uint32_t i = base + threadIdx.x;
            const bool live = i < chunks;
            const unsigned mask = __ballot_sync(0xffffffffu, live);
            if (!live) continue;
            const uint32_t b = i >> 3, k = i & 7;
            float4 val;
            if (vec) {
                val = __ldg(reinterpret_cast<const float4*>(xv) + i);
            } else {
                val.x = __ldg(xv + 4 * i + 0);
                val.y = __ldg(xv + 4 * i + 1);
                val.z = __ldg(xv + 4 * i + 2);
                val.w = __ldg(xv + 4 * i + 3);
            }
            xs[(size_t)v * chunks + b * 8 + ((k + b) & 7)] = val;
            if (WANT_SUMS) {
                // The 8 chunks of a block sit in 8 consecutive lanes, all live or all not.
                float s = (val.x + val.y) + (val.z + val.w);
                s += __shfl_xor_sync(mask, s, 1);
                s += __shfl_xor_sync(mask, s, 2);
                s += __shfl_xor_sync(mask, s, 4);
                if (k == 0) sx[(size_t)v * nb + b] = s;
            }
        }
    }
}

// ---- Q4_0 ----------------------------------------------------------------------
// Lane l of a warp owns blocks l, l+32, ... of the R rows the warp carries; one 128-bit
// load brings the 32 nibbles of a block.  Two unpack schemes:
//   VARIANT 0: nibble -> exact float through the 2^23 magic (shift, lop3, fadd, ffma).
//   VARIANT 1: nibbles are dropped into the top mantissa bits of 0.5, giving 0.5 + q/32
//              with one prmt per weight after two shift/mask pairs per word; the affine
//              offset is removed once per block with the block sum of x:
//                  sum (q-8) x = 32 * sum (0.5 + q/32) x - 24 * sum x.
template <int R, int B, int VARIANT>
__global__ void __launch_bounds__(256)
gemv_q4_0_kernel(const uint8_t* __restrict__ quants, const uint16_t* __restrict__ scales,
                 uint32_t nb, size_t row0, uint32_t nrows, const float* __restrict__ x,
                 size_t x_stride, float* __restrict__ y, size_t y_stride, int x_vec) {
    extern __shared__ float4 smem4[];
    float4* xs = smem4;
    float* sx = reinterpret_cast<float*>(xs + (size_t)B * nb * 8);

    stage_x<B, VARIANT == 1>(xs, sx, x, x_stride, nb, x_vec != 0);
    __syncthreads();

    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpc = blockDim.x >> 5;
    const uint32_t groups = (nrows + R - 1) / R;
    const uint32_t chunks = nb * 8;

    for (uint32_t g = blockIdx.x * wpc + warp; g < groups; g += gridDim.x * wpc) {
        const uint32_t lr0 = g * R;  // first local row of the group
        float acc[R][B];
#pragma unroll
        for (int i = 0; i < R; ++i)
#pragma unroll
            for (int v = 0; v < B; ++v) acc[i][v] = 0.0f;

#pragma unroll 2
        for (uint32_t b = lane; b < nb; b += 32) {
            uint4 q[R];
            float d[R];
#pragma unroll
            for (int i = 0; i < R; ++i) {
                const bool ok = lr0 + i < nrows;
                const size_t row = row0 + lr0 + (ok ? i : 0);
                q[i] = ldg_stream(reinterpret_cast<const uint4*>(quants) + row * nb + b);
                d[i] = ok ? h2f(__ldg(scales + row * nb + b)) : 0.0f;
            }
            float s[R][B];
#pragma unroll
            for (int i = 0; i < R; ++i)
#pragma unroll
                for (int v = 0; v < B; ++v)
                    s[i][v] = (VARIANT == 1) ? -0.75f * sx[(size_t)v * nb + b] : 0.0f;

#pragma unroll
            for (int k = 0; k < 8; ++k) {
                float4 xv[B];
#pragma unroll
                for (int v = 0; v < B; ++v)
                    xv[v] = xs[(size_t)v * chunks + b * 8 + ((k + lane) & 7)];
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    const uint32_t w = (k & 3) == 0 ? q[i].x : (k & 3) == 1 ? q[i].y
                                     : (k & 3) == 2 ? q[i].z : q[i].w;
                    float f0, f1, f2, f3;
                    if (VARIANT == 1) {
                        // low nibbles for k < 4, high nibbles for k >= 4, moved to bits 6..3 of each byte
                        const uint32_t t = (k < 4) ? ((w << 3) & 0x78787878u) : ((w >> 1) & 0x78787878u);
                        f0 = __uint_as_float(__byte_perm(t, 0x3F000000u, 0x7044));
                        f1 = __uint_as_float(__byte_perm(t, 0x3F000000u, 0x7144));
                        f2 = __uint_as_float(__byte_perm(t, 0x3F000000u, 0x7244));
                        f3 = __uint_as_float(__byte_perm(t, 0x3F000000u, 0x7344));
                    } else {
                        const uint32_t t = (k < 4) ? w : (w >> 4);
                        const float magic = 8388616.0f;  // 2^23 + 8
                        f0 = __uint_as_float(0x4B000000u | (t & 0xFu)) - magic;
                        f1 = __uint_as_float(0x4B000000u | ((t >> 8) & 0xFu)) - magic;
                        f2 = __uint_as_float(0x4B000000u | ((t >> 16) & 0xFu)) - magic;
                        f3 = __uint_as_float(0x4B000000u | ((t >> 24) & 0xFu)) - magic;
                    }
#pragma unroll
                    for (int v = 0; v < B; ++v) {
                        s[i][v] = fmaf(f0, xv[v].x, s[i][v]);
                        s[i][v] = fmaf(f1, xv[v].y, s[i][v]);
                        s[i][v] = fmaf(f2, xv[v].z, s[i][v]);
                        s[i][v] = fmaf(f3, xv[v].w, s[i][v]);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < R; ++i) {
                const float dd = (VARIANT == 1) ? 32.0f * d[i] : d[i];
#pragma unroll
                for (int v = 0; v < B; ++v) acc[i][v] = fmaf(dd, s[i][v], acc[i][v]);
            }
        }

#pragma unroll
        for (int i = 0; i < R; ++i)
#pragma unroll
            for (int v = 0; v < B; ++v) {
                const float t = warp_sum(acc[i][v]);
                if (lane == 0 && lr0 + i < nrows) y[(size_t)v * y_stride + lr0 + i] = t;
            }
    }
}

// ---- Q8_0 ----------------------------------------------------------------------
// A block holds 32 bytes of quants: lane l owns half-blocks l, l+32, ... (16 int8, one
// 128-bit load) so that a warp load is one contiguous 512-byte run.  int8 -> float goes
// through one xor per word (bias to unsigned), one prmt per weight into the low byte of
// 2^23, and one fadd that removes 2^23 + 128.
template <int R, int B>
__global__ void __launch_bounds__(256)
gemv_q8_0_kernel(const uint8_t* __restrict__ quants, const uint16_t* __restrict__ scales,
                 uint32_t nb, size_t row0, uint32_t nrows, const float* __restrict__ x,
                 size_t x_stride, float* __restrict__ y, size_t y_stride, int x_vec) {
    extern __shared__ float4 smem4[];
    float4* xs = smem4;

    stage_x<B, false>(xs, nullptr, x, x_stride, nb, x_vec != 0);
    __syncthreads();

    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, wpc = blockDim.x >> 5;
    const uint32_t groups = (nrows + R - 1) / R;
    const uint32_t chunks = nb * 8;
    const uint32_t nhalf = nb * 2;

    for (uint32_t g = blockIdx.x * wpc + warp; g < groups; g += gridDim.x * wpc) {
        const uint32_t lr0 = g * R;
        float acc[R][B];
#pragma unroll
        for (int i = 0; i < R; ++i)
#pragma unroll
            for (int v = 0; v < B; ++v) acc[i][v] = 0.0f;

#pragma unroll 2
        for (uint32_t h = lane; h < nhalf; h += 32) {
            const uint32_t b = h >> 1, half = h & 1;
            uint4 q[R];
            float d[R];
#pragma unroll
            for (int i = 0; i < R; ++i) {
                const bool ok = lr0 + i < nrows;
                const size_t row = row0 + lr0 + (ok ? i : 0);
                q[i] = ldg_stream(reinterpret_cast<const uint4*>(quants) + row * nhalf + h);
                d[i] = ok ? h2f(__ldg(scales + row * nb + b)) : 0.0f;
            }
            float s[R][B];
#pragma unroll
            for (int i = 0; i < R; ++i)
#pragma unroll
                for (int v = 0; v < B; ++v) s[i][v] = 0.0f;

#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                float4 xv[B];
#pragma unroll
                for (int v = 0; v < B; ++v)
                    xv[v] = xs[(size_t)v * chunks + b * 8 + ((half * 4 + kk + b) & 7)];
#pragma unroll
                for (int i = 0; i < R; ++i) {
                    const uint32_t w = (kk == 0 ? q[i].x : kk == 1 ? q[i].y : kk == 2 ? q[i].z : q[i].w) ^ 0x80808080u;
                    const float magic = 8388736.0f;  // 2^23 + 128
                    const float f0 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440)) - magic;
                    const float f1 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7441)) - magic;
                    const float f2 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7442)) - magic;
                    const float f3 = __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7443)) - magic;
#pragma unroll
                    for (int v = 0; v < B; ++v) {
                        s[i][v] = fmaf(f0, xv[v].x, s[i][v]);
                        s[i][v] = fmaf(f1, xv[v].y, s[i][v]);
                        s[i][v] = fmaf(f2, xv[v].z, s[i][v]);
                        s[i][v] = fmaf(f3, xv[v].w, s[i][v]);
                    }
                }
            }
#pragma unroll
            for (int i = 0; i < R; ++i)
#pragma unroll
                for (int v = 0; v < B; ++v) acc[i][v] = fmaf(d[i], s[i][v], acc[i][v]);
        }

#pragma unroll
        for (int i = 0; i < R; ++i)
#pragma unroll
            for (int v = 0; v < B; ++v) {
                const float t = warp_sum(acc[i][v]);
                if (lane == 0 && lr0 + i < nrows) y[(size_t)v * y_stride + lr0 + i] = t;
            }
    }
}

// ---- dequantisation --------------------------------------------------------------
// One thread per block; w = float(d) * float(q), which is exact in f32 (11 x 8 significant bits).
__global__ void dequant_q8_0_kernel(const uint8_t* __restrict__ quants,
                                    const uint16_t* __restrict__ scales, size_t nblocks,
                                    float* __restrict__ out) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    const float d = h2f(scales[b]);
    const int8_t* q = reinterpret_cast<const int8_t*>(quants) + b * 32;
    float* o = out + b * 32;
#pragma unroll
    for (int i = 0; i < 32; ++i) o[i] = __fmul_rn(d, (float)q[i]);
}

__global__ void dequant_q4_0_kernel(const uint8_t* __restrict__ quants,
                                    const uint16_t* __restrict__ scales, size_t nblocks,
                                    float* __restrict__ out) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nblocks) return;
    const float d = h2f(scales[b]);
    const uint8_t* q = quants + b * 16;
    float* o = out + b * 32;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        o[i] = __fmul_rn(d, (float)((int)(q[i] & 0x0F) - 8));
        o[i + 16] = __fmul_rn(d, (float)((int)(q[i] >> 4) - 8));
    }
}

// ---- launch helpers -------------------------------------------------------------

template <int R, int B>
vx_status launch_q4(vx_context* ctx, int variant, dim3 grid, dim3 block, size_t smem,
                    const vx_qweights* w, size_t row0, uint32_t nrows, const float* x,
                    size_t x_stride, float* y, size_t y_stride, int x_vec) {
    auto go = [&](auto kernel) -> vx_status {
        VX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kernel<<<grid, block, smem, ctx->stream>>>(w->d_quants, w->d_scales, (uint32_t)w->blocks_per_row,
                                                   row0, nrows, x, x_stride, y, y_stride, x_vec);
        VX_CUDA(cudaGetLastError());
        return VX_OK;
    };
    return variant == 0 ? go(gemv_q4_0_kernel<R, B, 0>) : go(gemv_q4_0_kernel<R, B, 1>);
}

template <int R, int B>
vx_status launch_q8(vx_context* ctx, dim3 grid, dim3 block, size_t smem, const vx_qweights* w,
                    size_t row0, uint32_t nrows, const float* x, size_t x_stride, float* y,
                    size_t y_stride, int x_vec) {
    auto kernel = gemv_q8_0_kernel<R, B>;
    VX_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<grid, block, smem, ctx->stream>>>(w->d_quants, w->d_scales, (uint32_t)w->blocks_per_row,
                                               row0, nrows, x, x_stride, y, y_stride, x_vec);
    VX_CUDA(cudaGetLastError());
    return VX_OK;
}

template <int B>
vx_status launch_batch(vx_context* ctx, const vx_qweights* w, size_t row0, uint32_t nrows,
                       const float* x, size_t x_stride, float* y, size_t y_stride) {
    const int variant = vx::option(ctx, "gemv.variant", 1) == 0 ? 0 : 1;
    int rpw = (int)vx::option(ctx, "gemv.rows_per_warp", 2);
    if (B >= 4) rpw = 1;  // keep the accumulators in registers
    const int threads = (int)vx::option(ctx, "gemv.block_threads", 256);
    const int per_sm = (int)vx::option(ctx, "gemv.ctas_per_sm", 4);
    VX_REQUIRE(threads >= 32 && threads <= 256 && threads % 32 == 0, VX_ERR_INVALID_ARGUMENT,
               "gemv.block_threads must be a multiple of 32 in [32, 256]");
    VX_REQUIRE(rpw == 1 || rpw == 2 || rpw == 4, VX_ERR_INVALID_ARGUMENT,
               "gemv.rows_per_warp must be 1, 2 or 4");

    const uint32_t nb = (uint32_t)w->blocks_per_row;
    const size_t smem = (size_t)B * nb * 8 * sizeof(float4) + (size_t)B * nb * sizeof(float);
    const uint32_t wpc = threads / 32;
    const uint32_t groups = (nrows + rpw - 1) / rpw;
    const uint32_t want = (groups + wpc - 1) / wpc;
    const uint32_t cap = (uint32_t)std::max(1, ctx->sm_count * per_sm);
    dim3 grid(std::min(want, cap)), block(threads);
    const int x_vec = ((reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (x_stride % 4 == 0 || B == 1)) ? 1 : 0;

    vx_status st;
    if (w->type == VX_Q4_0) {
        if (rpw == 1) st = launch_q4<1, B>(ctx, variant, grid, block, smem, w, row0, nrows, x, x_stride, y, y_stride, x_vec);
        else if (rpw == 2) st = launch_q4<2, B>(ctx, variant, grid, block, smem, w, row0, nrows, x, x_stride, y, y_stride, x_vec);
        else st = launch_q4<4, B>(ctx, variant, grid, block, smem, w, row0, nrows, x, x_stride, y, y_stride, x_vec);
    } else {
        if (rpw == 1) st = launch_q8<1, B>(ctx, grid, block, smem, w, row0, nrows, x, x_stride, y, y_stride, x_vec);
        else if (rpw == 2) st = launch_q8<2, B>(ctx, grid, block, smem, w, row0, nrows, x, x_stride, y, y_stride, x_vec);
        else st = launch_q8<4, B>(ctx, grid, block, smem, w, row0, nrows, x, x_stride, y, y_stride, x_vec);
    }
    if (st == VX_OK) ctx->launches++;
    return st;
}

}  // namespace

// Device quantiser: one thread per block of 32 weights, the same arithmetic as the host quantiser below
// (IEEE division, f16 scale rounded to nearest even before the quants are formed, round half away from zero),
// writing the planar layout directly.  `row_stride` is the distance between rows of w in elements.
template <int QT>
__global__ void quantize_planar_kernel(const float* __restrict__ w, size_t rows, size_t nb, size_t row_stride,
                                       uint8_t* __restrict__ quants, uint16_t* __restrict__ scales) {
    const size_t total = rows * nb;
    for (size_t blk = (size_t)blockIdx.x * blockDim.x + threadIdx.x; blk < total; blk += (size_t)gridDim.x * blockDim.x) {
        const size_t r = blk / nb, b = blk % nb;
        const float* src = w + r * row_stride + b * QK;
        float v[QK];
        if ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) {
#pragma unroll
            for (int i = 0; i < QK / 4; ++i) {
                const float4 f = __ldg(reinterpret_cast<const float4*>(src) + i);
                v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < QK; ++i) v[i] = __ldg(src + i);
        }
        // The element of largest magnitude (first one on ties) fixes the scale.
        float amax = 0.0f, signed_max = 0.0f;
#pragma unroll
        for (int i = 0; i < QK; ++i) {
            const float a = fabsf(v[i]);
            if (a > amax) {
                amax = a;
                signed_max = v[i];
            }
        }
        const __half dh = __float2half_rn(QT == 0 ? __fdiv_rn(amax, 127.0f) : __fdiv_rn(signed_max, 7.0f));
        const float d = __half2float(dh);
        scales[blk] = __half_as_ushort(dh);
        if (QT == 0) {
            uint32_t packed[QK / 4];
#pragma unroll
            for (int i = 0; i < QK; ++i) {
                float q = d != 0.0f ? roundf(__fdiv_rn(v[i], d)) : 0.0f;   // roundf: half away from zero
                q = fminf(127.0f, fmaxf(-127.0f, q));
                const uint32_t byte = (uint32_t)(int)q & 0xFFu;
                if (i % 4 == 0) packed[i / 4] = 0;
                packed[i / 4] |= byte << (8 * (i % 4));
            }
            uint4* dst = reinterpret_cast<uint4*>(quants + blk * 32);
            dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        } else {
            uint32_t q[QK];
#pragma unroll
            for (int i = 0; i < QK; ++i) {
                float t = d != 0.0f ? roundf(__fdiv_rn(v[i], d)) + 8.0f : 8.0f;
                t = fminf(15.0f, fmaxf(0.0f, t));
                q[i] = (uint32_t)(int)t;
            }
            uint32_t packed[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                packed[k] = 0;
#pragma unroll
                for (int j = 0; j < 4; ++j) packed[k] |= (q[4 * k + j] | (q[4 * k + j + 16] << 4)) << (8 * j);
            }
            *reinterpret_cast<uint4*>(quants + blk * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
    }
}

extern "C" {

size_t vx_qblock_bytes(vx_qtype t) { return (t == VX_Q8_0 || t == VX_Q4_0) ? block_bytes(t) : 0; }

vx_status vx_quantize(vx_qtype t, const float* w, size_t rows, size_t cols, void* blocks) {
    VX_REQUIRE(t == VX_Q8_0 || t == VX_Q4_0, VX_ERR_INVALID_ARGUMENT, "vx_quantize: unknown type %d", (int)t);
    VX_REQUIRE(cols % QK == 0, VX_ERR_INVALID_ARGUMENT, "cols (%zu) must be a multiple of 32", cols);
    if (rows == 0 || cols == 0) return VX_OK;
    VX_REQUIRE(w && blocks, VX_ERR_INVALID_ARGUMENT, "vx_quantize: null pointer");
    const size_t nb = cols / QK;
    uint8_t* out = static_cast<uint8_t*>(blocks);
    for (size_t r = 0; r < rows; ++r)
        for (size_t b = 0; b < nb; ++b) {
            const float* src = w + r * cols + b * QK;
            uint8_t* dst = out + (r * nb + b) * block_bytes(t);
            // The element of largest magnitude (first one on ties) fixes the scale.
            float amax = 0.0f, signed_max = 0.0f;
            for (int i = 0; i < QK; ++i) {
                const float a = std::fabs(src[i]);
                if (a > amax) {
                    amax = a;
                    signed_max = src[i];
                }
            }
            if (t == VX_Q8_0) {
                // d = max|w| / 127; q = round-half-away(w / d16) in [-127, 127].
                const uint16_t d16 = host_f2h(amax / 127.0f);
                const float d = host_h2f(d16);
                std::memcpy(dst, &d16, 2);
                for (int i = 0; i < QK; ++i) {
                    long q = d != 0.0f ? std::lround(src[i] / d) : 0;
                    q = std::max(-127l, std::min(127l, q));
                    dst[2 + i] = (uint8_t)(int8_t)q;
                }
            } else {
                // d = (signed element of largest magnitude) / 7; q = round-half-away(w / d16) + 8 in [0, 15].
                const uint16_t d16 = host_f2h(signed_max / 7.0f);
                const float d = host_h2f(d16);
                std::memcpy(dst, &d16, 2);
                uint8_t q[QK];
                for (int i = 0; i < QK; ++i) {
                    long v = d != 0.0f ? std::lround(src[i] / d) + 8 : 8;
                    q[i] = (uint8_t)std::max(0l, std::min(15l, v));
                }
                for (int i = 0; i < 16; ++i) dst[2 + i] = (uint8_t)(q[i] | (q[i + 16] << 4));
            }
        }
    return VX_OK;
}

vx_status vx_dequantize_host(vx_qtype t, const void* blocks, size_t rows, size_t cols, float* w) {
    VX_REQUIRE(t == VX_Q8_0 || t == VX_Q4_0, VX_ERR_INVALID_ARGUMENT, "vx_dequantize_host: unknown type %d", (int)t);
    VX_REQUIRE(cols % QK == 0, VX_ERR_INVALID_ARGUMENT, "cols (%zu) must be a multiple of 32", cols);
    if (rows == 0 || cols == 0) return VX_OK;
    VX_REQUIRE(w && blocks, VX_ERR_INVALID_ARGUMENT, "vx_dequantize_host: null pointer");
    const size_t nblocks = rows * (cols / QK);
    const uint8_t* in = static_cast<const uint8_t*>(blocks);
    for (size_t b = 0; b < nblocks; ++b) {
        const uint8_t* src = in + b * block_bytes(t);
        uint16_t d16;
        std::memcpy(&d16, src, 2);
        const float d = host_h2f(d16);
        float* o = w + b * QK;
        if (t == VX_Q8_0) {
            for (int i = 0; i < QK; ++i) o[i] = d * (float)(int8_t)src[2 + i];
        } else {
            for (int i = 0; i < 16; ++i) {
                o[i] = d * (float)((int)(src[2 + i] & 0x0F) - 8);
                o[i + 16] = d * (float)((int)(src[2 + i] >> 4) - 8);
            }
        }
    }
    return VX_OK;
}

vx_status vx_qweights_upload(vx_context* ctx, vx_qtype t, const void* blocks, size_t rows,
                             size_t cols, vx_qweights** out) {
    VX_REQUIRE(ctx && out, VX_ERR_INVALID_ARGUMENT, "vx_qweights_upload: null argument");
    *out = nullptr;
    VX_REQUIRE(t == VX_Q8_0 || t == VX_Q4_0, VX_ERR_INVALID_ARGUMENT, "unknown quantised type %d", (int)t);
    VX_REQUIRE(cols % QK == 0 && cols > 0 && rows > 0, VX_ERR_INVALID_ARGUMENT,
               "rows (%zu) and cols (%zu) must be positive and cols a multiple of 32", rows, cols);
    VX_REQUIRE(blocks, VX_ERR_INVALID_ARGUMENT, "vx_qweights_upload: null block stream");
    VX_REQUIRE(rows <= 0xFFFFFFFFull && cols / QK <= 0x03FFFFFFull, VX_ERR_UNSUPPORTED, "matrix too large");

    vx::DeviceGuard guard(ctx->device);
    vx_qweights* w = new (std::nothrow) vx_qweights();
    VX_REQUIRE(w, VX_ERR_OUT_OF_MEMORY, "host allocation failed");
    w->type = t;
    w->rows = rows;
    w->cols = cols;
    w->blocks_per_row = cols / QK;
    w->quant_row_bytes = w->blocks_per_row * quant_bytes(t);
    w->device = ctx->device;
    const size_t nblocks = rows * w->blocks_per_row;
    const size_t qplane = round_up(nblocks * quant_bytes(t), 256);
    const size_t splane = round_up(nblocks * 2, 256);
    w->device_bytes = qplane + splane;

    // Split the stream into the two planes on the host, then one upload.
    uint8_t* staging = nullptr;
    cudaError_t e = cudaMallocHost(&staging, w->device_bytes);
    if (e != cudaSuccess) {
        const size_t wanted = w->device_bytes;
        delete w;
        (void)cudaGetLastError();
        return fail(VX_ERR_OUT_OF_MEMORY, "pinned staging allocation of %zu bytes failed: %s", wanted,
                    cudaGetErrorString(e));
    }
    std::memset(staging + nblocks * quant_bytes(t), 0, qplane - nblocks * quant_bytes(t));
    std::memset(staging + qplane + nblocks * 2, 0, splane - nblocks * 2);
    const uint8_t* in = static_cast<const uint8_t*>(blocks);
    const size_t bb = block_bytes(t), qb = quant_bytes(t);
    for (size_t b = 0; b < nblocks; ++b) {
        std::memcpy(staging + qplane + b * 2, in + b * bb, 2);
        std::memcpy(staging + b * qb, in + b * bb + 2, qb);
    }
    e = vx::device_malloc(ctx, reinterpret_cast<void**>(&w->d_base), w->device_bytes);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(w->d_base, staging, w->device_bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFreeHost(staging);
    if (e != cudaSuccess) {
        if (w->d_base) cudaFree(w->d_base);
        delete w;
        (void)cudaGetLastError();
        return fail(e == cudaErrorMemoryAllocation ? VX_ERR_OUT_OF_MEMORY : VX_ERR_CUDA,
                    "uploading quantised weights failed: %s", cudaGetErrorString(e));
    }
    w->d_quants = w->d_base;
    w->d_scales = reinterpret_cast<uint16_t*>(w->d_base + qplane);
    *out = w;
    return VX_OK;
}

vx_status vx_qweights_from_device(vx_context* ctx, vx_qtype t, const float* w_device, size_t rows, size_t cols,
                                  size_t row_stride, vx_qweights** out) {
    VX_REQUIRE(ctx && out, VX_ERR_INVALID_ARGUMENT, "vx_qweights_from_device: null argument");
    *out = nullptr;
    VX_REQUIRE(t == VX_Q8_0 || t == VX_Q4_0, VX_ERR_INVALID_ARGUMENT, "unknown quantised type %d", (int)t);
    VX_REQUIRE(cols % QK == 0 && cols > 0 && rows > 0, VX_ERR_INVALID_ARGUMENT,
               "rows (%zu) and cols (%zu) must be positive and cols a multiple of 32", rows, cols);
    VX_REQUIRE(w_device && row_stride >= cols, VX_ERR_INVALID_ARGUMENT, "null weights or rows %zu elements apart", row_stride);
    VX_REQUIRE(rows <= 0xFFFFFFFFull && cols / QK <= 0x03FFFFFFull, VX_ERR_UNSUPPORTED, "matrix too large");
    vx::DeviceGuard guard(ctx->device);
    std::unique_ptr<vx_qweights> w(new (std::nothrow) vx_qweights());
    VX_REQUIRE(w, VX_ERR_OUT_OF_MEMORY, "host allocation failed");
    w->type = t;
    w->rows = rows;
    w->cols = cols;
    w->blocks_per_row = cols / QK;
    w->quant_row_bytes = w->blocks_per_row * quant_bytes(t);
    w->device = ctx->device;
    const size_t nblocks = rows * w->blocks_per_row;
    const size_t qplane = round_up(nblocks * quant_bytes(t), 256);
    const size_t splane = round_up(nblocks * 2, 256);
    w->device_bytes = qplane + splane;
    cudaError_t e = vx::device_malloc(ctx, reinterpret_cast<void**>(&w->d_base), w->device_bytes);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return fail(VX_ERR_OUT_OF_MEMORY, "allocating %zu bytes of quantised weights failed: %s", w->device_bytes,
                    cudaGetErrorString(e));
    }
    w->d_quants = w->d_base;
    w->d_scales = reinterpret_cast<uint16_t*>(w->d_base + qplane);
    // the padding behind each plane is read by whole-tile copies: keep it defined
    e = cudaMemsetAsync(w->d_base, 0, w->device_bytes, ctx->stream);
    if (e == cudaSuccess) {
        const unsigned threads = 128;
        const unsigned blocks = (unsigned)std::min<size_t>((nblocks + threads - 1) / threads, (size_t)ctx->sm_count * 16);
        if (t == VX_Q8_0)
            quantize_planar_kernel<0><<<blocks, threads, 0, ctx->stream>>>(w_device, rows, w->blocks_per_row, row_stride,
                                                                        w->d_quants, w->d_scales);
        else
            quantize_planar_kernel<1><<<blocks, threads, 0, ctx->stream>>>(w_device, rows, w->blocks_per_row, row_stride,
                                                                        w->d_quants, w->d_scales);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        cudaFree(w->d_base);
        return fail(VX_ERR_CUDA, "device quantisation failed: %s", cudaGetErrorString(e));
    }
    ctx->launches++;
    ctx->weights_fresh = true;
    *out = w.release();
    return VX_OK;
}

vx_status vx_qweights_free(vx_context* ctx, vx_qweights* w) {
    VX_REQUIRE(ctx, VX_ERR_INVALID_ARGUMENT, "vx_qweights_free: null context");
    if (!w) return VX_OK;
    vx::DeviceGuard guard(ctx->device);
    VX_CUDA(cudaStreamSynchronize(ctx->stream));
    if (w->d_base) VX_CUDA(cudaFree(w->d_base));
    delete w;
    return VX_OK;
}

vx_status vx_qweights_info(const vx_qweights* w, int32_t* qtype, size_t* rows, size_t* cols,
                           size_t* device_bytes) {
    VX_REQUIRE(w, VX_ERR_INVALID_ARGUMENT, "vx_qweights_info: null weights");
    if (qtype) *qtype = (int32_t)w->type;
    if (rows) *rows = w->rows;
    if (cols) *cols = w->cols;
    if (device_bytes) *device_bytes = w->device_bytes;
    return VX_OK;
}

vx_status vx_dequantize(vx_context* ctx, const vx_qweights* w, float* device_out) {
    VX_REQUIRE(ctx && w && device_out, VX_ERR_INVALID_ARGUMENT, "vx_dequantize: null argument");
    VX_REQUIRE(w->device == ctx->device, VX_ERR_INVALID_ARGUMENT, "weights live on device %d, context on %d",
               w->device, ctx->device);
    vx::DeviceGuard guard(ctx->device);
    const size_t nblocks = w->rows * w->blocks_per_row;
    const unsigned threads = 128;
    const size_t grid = (nblocks + threads - 1) / threads;
    VX_REQUIRE(grid <= 0x7FFFFFFFull, VX_ERR_UNSUPPORTED, "matrix too large");
    if (w->type == VX_Q8_0)
        dequant_q8_0_kernel<<<(unsigned)grid, threads, 0, ctx->stream>>>(w->d_quants, w->d_scales, nblocks, device_out);
    else
        dequant_q4_0_kernel<<<(unsigned)grid, threads, 0, ctx->stream>>>(w->d_quants, w->d_scales, nblocks, device_out);
    VX_CUDA(cudaGetLastError());
    ctx->launches++;
    return VX_OK;
}

vx_status vx_gemv_q_multi(vx_context* ctx, const vx_qweights* const* ws, size_t n, const float* x, size_t x_stride,
                          float* const* ys, size_t y_stride, size_t batch) {
    VX_REQUIRE(ctx, VX_ERR_INVALID_ARGUMENT, "vx_gemv_q_multi: null context");
    if (n == 0 || batch == 0) return VX_OK;
    VX_REQUIRE(ws && ys && x, VX_ERR_INVALID_ARGUMENT, "vx_gemv_q_multi: null argument");
    size_t most_rows = 0;
    for (size_t i = 0; i < n; ++i) {
        VX_REQUIRE(ws[i] && ys[i], VX_ERR_INVALID_ARGUMENT, "vx_gemv_q_multi: matrix %zu or its y is null", i);
        VX_REQUIRE(ws[i]->device == ctx->device, VX_ERR_INVALID_ARGUMENT, "weights %zu live on device %d, context on %d", i,
                   ws[i]->device, ctx->device);
        VX_REQUIRE(ws[i]->type == ws[0]->type && ws[i]->cols == ws[0]->cols, VX_ERR_SHAPE,
                   "matrix %zu (type %d, %zu columns) does not match matrix 0 (type %d, %zu columns)", i, (int)ws[i]->type,
                   ws[i]->cols, (int)ws[0]->type, ws[0]->cols);
        most_rows = std::max(most_rows, ws[i]->rows);
    }
    VX_REQUIRE(batch == 1 || (x_stride >= ws[0]->cols && y_stride >= most_rows), VX_ERR_INVALID_ARGUMENT,
               "batch strides (x %zu, y %zu) shorter than the vectors (%zu, %zu)", x_stride, y_stride, ws[0]->cols, most_rows);
    vx::DeviceGuard guard(ctx->device);
    if (vx::option(ctx, "gemv.variant", 2) == 2 && vx::option(ctx, "gemv.batch_mma", -1) != 0) {
        std::vector<size_t> row0(n, 0);
        std::vector<uint32_t> nrows(n);
        bool any = false;
        for (size_t i = 0; i < n; ++i) {
            nrows[i] = (uint32_t)ws[i]->rows;
            any = any || nrows[i] != 0;
        }
        if (!any) return VX_OK;
        size_t v = 0;
        while (v < batch) {
            const uint32_t take = (uint32_t)std::min<size_t>(8, batch - v);
            std::vector<float*> yv(n);
            for (size_t i = 0; i < n; ++i) yv[i] = ys[i] + v * y_stride;
            bool eligible = false;
            vx_status st = vx::launch_gemv_mma(ctx, ws, row0.data(), nrows.data(), yv.data(), n, x + v * x_stride, x_stride,
                                               y_stride, take, &eligible);
            if (st != VX_OK) return st;
            if (!eligible) break;
            v += take;
        }
        if (v == batch) return VX_OK;
        x += v * x_stride;
        batch -= v;
        for (size_t i = 0; i < n; ++i) {
            vx_status st = vx_gemv_q_rows(ctx, ws[i], 0, ws[i]->rows, x, x_stride, ys[i] + v * y_stride, y_stride, batch);
            if (st != VX_OK) return st;
        }
        return VX_OK;
    }
    for (size_t i = 0; i < n; ++i) {
        vx_status st = vx_gemv_q_rows(ctx, ws[i], 0, ws[i]->rows, x, x_stride, ys[i], y_stride, batch);
        if (st != VX_OK) return st;
    }
    return VX_OK;
}

vx_status vx_gemv_q_rows(vx_context* ctx, const vx_qweights* w, size_t row0, size_t nrows,
                         const float* x, size_t x_stride, float* y, size_t y_stride, size_t batch) {
    VX_REQUIRE(ctx && w, VX_ERR_INVALID_ARGUMENT, "vx_gemv_q: null context or weights");
    VX_REQUIRE(w->device == ctx->device, VX_ERR_INVALID_ARGUMENT, "weights live on device %d, context on %d",
               w->device, ctx->device);
    VX_REQUIRE(row0 <= w->rows && nrows <= w->rows - row0, VX_ERR_OUT_OF_BOUNDS,
               "rows [%zu, %zu) outside a matrix of %zu rows", row0, row0 + nrows, w->rows);
    if (nrows == 0 || batch == 0) return VX_OK;
    VX_REQUIRE(x && y, VX_ERR_INVALID_ARGUMENT, "vx_gemv_q: null vector");
    VX_REQUIRE(batch == 1 || (x_stride >= w->cols && y_stride >= nrows), VX_ERR_INVALID_ARGUMENT,
               "batch strides (x %zu, y %zu) shorter than the vectors (%zu, %zu)", x_stride, y_stride,
               w->cols, nrows);
    vx::DeviceGuard guard(ctx->device);

    // Default: the TMA-fed streaming kernel, up to eight vectors per launch (a list whose entries
    // share the weights: the later vectors find them in L2 when the matrix fits there).
    // "gemv.variant" 0 / 1 select the register-staged kernels below, which also take over when a
    // row does not fit the ring.
    if (vx::option(ctx, "gemv.variant", 2) == 2) {
        size_t v = 0;
        // Two and more vectors: the tensor-core kernel, eight vectors per pass over the weights.
        const int64_t use_mma = vx::option(ctx, "gemv.batch_mma", -1);
        if (use_mma != 0 && (batch >= 2 || use_mma == 1)) {
            while (v < batch) {
                const uint32_t take = (uint32_t)std::min<size_t>(8, batch - v);
                bool eligible = false;
                const uint32_t nr = (uint32_t)nrows;
                float* yv = y + v * y_stride;
                vx_status st = vx::launch_gemv_mma(ctx, &w, &row0, &nr, &yv, 1, x + v * x_stride, x_stride, y_stride,
                                                   take, &eligible);
                if (st != VX_OK) return st;
                if (!eligible) break;
                v += take;
            }
        }
        while (v < batch) {
            const uint32_t take = (uint32_t)std::min<size_t>(8, batch - v);
            bool eligible = false;
            vx_status st = vx::launch_gemv_stream(ctx, w, row0, (uint32_t)nrows, x + v * x_stride,
                                                  y + v * y_stride, nullptr, 0, nullptr, &eligible, take, x_stride,
                                                  y_stride);
            if (st != VX_OK) return st;
            if (!eligible) break;
            v += take;
        }
        if (v == batch) return VX_OK;
        x += v * x_stride;
        y += v * y_stride;
        batch -= v;
    }

    // Shared memory bounds how many x vectors one launch can stage.
    const size_t per_vec = w->blocks_per_row * (8 * sizeof(float4) + sizeof(float));
    const size_t budget = 200 * 1024;
    VX_REQUIRE(per_vec <= budget, VX_ERR_UNSUPPORTED,
               "rows of %zu columns do not fit the shared-memory staging of x (limit %zu)", w->cols,
               (budget / (8 * sizeof(float4) + sizeof(float))) * QK);
    size_t max_b = std::min<size_t>(4, budget / per_vec);
    size_t done = 0;
    while (done < batch) {
        size_t b = std::min(max_b, batch - done);
        if (b == 3) b = 2;
        const float* xv = x + done * x_stride;
        float* yv = y + done * y_stride;
        vx_status st;
        switch (b) {
            case 1: st = launch_batch<1>(ctx, w, row0, (uint32_t)nrows, xv, x_stride, yv, y_stride); break;
            case 2: st = launch_batch<2>(ctx, w, row0, (uint32_t)nrows, xv, x_stride, yv, y_stride); break;
            default: st = launch_batch<4>(ctx, w, row0, (uint32_t)nrows, xv, x_stride, yv, y_stride); break;
        }
        if (st != VX_OK) return st;
        done += b;
    }
    return VX_OK;
}

vx_status vx_gemv_q(vx_context* ctx, const vx_qweights* w, const float* x, size_t x_stride, float* y,
                    size_t y_stride, size_t batch) {
    VX_REQUIRE(w, VX_ERR_INVALID_ARGUMENT, "vx_gemv_q: null weights");
    return vx_gemv_q_rows(ctx, w, 0, w->rows, x, x_stride, y, y_stride, batch);
}

}  // extern "C"
