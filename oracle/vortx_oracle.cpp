// CPU oracle for the vortx matmul hot path.  TEST INFRASTRUCTURE ONLY — see vortx_oracle.h.
//
// Compile with -ffp-contract=off: the reference's Rust source writes `acc += a * b`,
// which rounds the product and the sum separately; a fused multiply-add here would
// change the bits.
#include "vortx_oracle.h"

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstring>
#include <thread>
#include <vector>

namespace {

// vortx-shaders/src/linalg/gemm.rs:15-31
constexpr uint32_t TILE_M = 64, TILE_N = 64, TILE_K = 16;
constexpr uint32_t WG_M = 16, WG_N = 16;
constexpr uint32_t THREAD_M = TILE_M / WG_M, THREAD_N = TILE_N / WG_N;
constexpr uint32_t SMEM_A_STRIDE = TILE_K + 1, SMEM_B_STRIDE = TILE_N + 1;
constexpr size_t SMEM_A_SIZE = TILE_M * SMEM_A_STRIDE, SMEM_B_SIZE = TILE_K * SMEM_B_STRIDE;

inline uint32_t it(const orc_shape& s, uint32_t n, uint32_t c, uint32_t h, uint32_t w) {
    return n * s.n_stride + c * s.c_stride + h * s.h_stride + w * s.w_stride;
}

template <class F>
void parallel_for(size_t count, int nthreads, F&& body) {
    if (nthreads <= 1 || count <= 1) {
        for (size_t i = 0; i < count; ++i) body(i);
        return;
    }
    std::atomic<size_t> next{0};
    std::vector<std::thread> pool;
    const int nt = (int)std::min<size_t>((size_t)nthreads, count);
    for (int t = 0; t < nt; ++t)
        pool.emplace_back([&] {
            for (;;) {
                size_t i = next.fetch_add(1);
                if (i >= count) break;
                body(i);
            }
        });
    for (auto& th : pool) th.join();
}

// One workgroup of gemm_tiled (vortx-shaders/src/linalg/gemm.rs:69-193).  The 256
// invocations are run phase by phase between the two barriers of the k loop, which is
// what the barriers guarantee on a device.
void tiled_workgroup(float* out, const float* lhs, const float* rhs, const orc_shape& so,
                     const orc_shape& sl, const orc_shape& sr, uint32_t wg_x, uint32_t wg_y,
                     uint32_t wg_z) {
    float smem_a[SMEM_A_SIZE];
    float smem_b[SMEM_B_SIZE];
    std::vector<float> acc_all(256 * 16);

    const uint32_t tile_row = wg_y * TILE_M;
    const uint32_t tile_col = wg_x * TILE_N;
    const uint32_t m = so.h, n = so.w, k = sl.w;

    for (uint32_t batch = 0; batch < so.n; ++batch) {
        const uint32_t batch_c = wg_z % so.c;
        std::fill(acc_all.begin(), acc_all.end(), 0.0f);

        for (uint32_t k_tile = 0; k_tile < k; k_tile += TILE_K) {
            for (uint32_t linear_tid = 0; linear_tid < WG_M * WG_N; ++linear_tid) {
                for (uint32_t i = linear_tid; i < TILE_M * TILE_K; i += WG_M * WG_N) {
                    uint32_t row = i / TILE_K, col = i % TILE_K;
                    uint32_t gr = tile_row + row, gc = k_tile + col;
                    float v = (gr < m && gc < k) ? lhs[it(sl, batch, batch_c, gr, gc)] : 0.0f;
                    smem_a[row * SMEM_A_STRIDE + col] = v;
                }
                for (uint32_t i = linear_tid; i < TILE_K * TILE_N; i += WG_M * WG_N) {
                    uint32_t row = i / TILE_N, col = i % TILE_N;
                    uint32_t gr = k_tile + row, gc = tile_col + col;
                    float v = (gr < k && gc < n) ? rhs[it(sr, batch, batch_c, gr, gc)] : 0.0f;
                    smem_b[row * SMEM_B_STRIDE + col] = v;
                }
            }
            // barrier
            for (uint32_t tid_y = 0; tid_y < WG_M; ++tid_y)
                for (uint32_t tid_x = 0; tid_x < WG_N; ++tid_x) {
                    float* acc = &acc_all[(tid_y * WG_N + tid_x) * 16];
                    const uint32_t a_row_base = tid_y * THREAD_M;
                    const uint32_t b_col_base = tid_x * THREAD_N;
                    for (uint32_t kk = 0; kk < TILE_K; ++kk) {
                        float a[4], b[4];
                        for (uint32_t r = 0; r < 4; ++r)
                            a[r] = smem_a[(a_row_base + r) * SMEM_A_STRIDE + kk];
                        for (uint32_t c = 0; c < 4; ++c)
                            b[c] = smem_b[kk * SMEM_B_STRIDE + b_col_base + c];
                        for (uint32_t r = 0; r < 4; ++r)
                            for (uint32_t c = 0; c < 4; ++c) {
                                float p = a[r] * b[c];
                                acc[r * 4 + c] = acc[r * 4 + c] + p;
                            }
                    }
                }
            // barrier
        }

        for (uint32_t tid_y = 0; tid_y < WG_M; ++tid_y)
            for (uint32_t tid_x = 0; tid_x < WG_N; ++tid_x) {
                const float* acc = &acc_all[(tid_y * WG_N + tid_x) * 16];
                const uint32_t out_row = tile_row + tid_y * THREAD_M;
                const uint32_t out_col = tile_col + tid_x * THREAD_N;
                for (uint32_t i = 0; i < THREAD_M; ++i) {
                    uint32_t row = out_row + i;
                    if (row >= m) continue;
                    for (uint32_t j = 0; j < THREAD_N; ++j) {
                        uint32_t col = out_col + j;
                        if (col < n) out[it(so, batch, batch_c, row, col)] = acc[i * THREAD_N + j];
                    }
                }
            }
    }
}

inline uint16_t load_u16(const uint8_t* p) { return (uint16_t)(p[0] | (p[1] << 8)); }
inline void store_u16(uint8_t* p, uint16_t v) {
    p[0] = (uint8_t)(v & 0xff);
    p[1] = (uint8_t)(v >> 8);
}

// Round half away from zero, the rounding the quantiser states for q.
inline int round_away(float v) { return (int)std::lround(v); }

}  // namespace

extern "C" {

uint32_t orc_shape_it(const orc_shape* s, uint32_t n, uint32_t c, uint32_t h, uint32_t w) {
    return it(*s, n, c, h, w);
}

void orc_gemm_naive(float* out, const float* lhs, const float* rhs, const orc_shape* so,
                    const orc_shape* sl, const orc_shape* sr) {
    // Grid (src/linalg/gemm.rs:307-309): x over out.w, y over out.h, z over out.c.
    for (uint32_t z = 0; z < so->c; ++z)
        for (uint32_t y = 0; y < so->h; ++y)
            for (uint32_t x = 0; x < so->w; ++x) {
                for (uint32_t n = 0; n < so->n; ++n) {
                    float sum = 0.0f;
                    for (uint32_t j = 0; j < sl->w; ++j) {
                        float p = lhs[it(*sl, n, z, y, j)] * rhs[it(*sr, n, z, j, x)];
                        sum = sum + p;
                    }
                    out[it(*so, n, z, y, x)] = sum;
                }
            }
}

void orc_gemm_tiled(float* out, const float* lhs, const float* rhs, const orc_shape* so,
                    const orc_shape* sl, const orc_shape* sr, int nthreads) {
    // Workgroup counts, src/linalg/gemm.rs:311-321 (thread counts there, /16 here).
    const uint32_t gx = (so->w + TILE_N - 1) / TILE_N;
    const uint32_t gy = (so->h + TILE_M - 1) / TILE_M;
    const uint32_t gz = so->c;
    const size_t total = (size_t)gx * gy * gz;
    parallel_for(total, nthreads, [&](size_t idx) {
        uint32_t wx = (uint32_t)(idx % gx);
        uint32_t wy = (uint32_t)((idx / gx) % gy);
        uint32_t wz = (uint32_t)(idx / ((size_t)gx * gy));
        tiled_workgroup(out, lhs, rhs, *so, *sl, *sr, wx, wy, wz);
    });
}

void orc_gemm_dispatch(float* out, const float* lhs, const float* rhs, const orc_shape* so,
                       const orc_shape* sl, const orc_shape* sr, int nthreads) {
    if (so->h >= 32 || so->w >= 32)
        orc_gemm_tiled(out, lhs, rhs, so, sl, sr, nthreads);
    else
        orc_gemm_naive(out, lhs, rhs, so, sl, sr);
}

void orc_gemm_f64(double* out, const float* lhs, const float* rhs, uint32_t m, uint32_t n,
                  uint32_t k) {
    for (uint32_t i = 0; i < m; ++i)
        for (uint32_t j = 0; j < n; ++j) {
            double s = 0.0;
            for (uint32_t p = 0; p < k; ++p)
                s += (double)lhs[(size_t)i * k + p] * (double)rhs[(size_t)p * n + j];
            out[(size_t)i * n + j] = s;
        }
}

// ---- f16 <-> f32, bit level -------------------------------------------------

uint16_t orc_f32_to_f16(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    const uint32_t absx = x & 0x7fffffffu;
    if (absx >= 0x7f800000u) {  // inf / nan
        return (uint16_t)(sign | 0x7c00u | ((absx > 0x7f800000u) ? 0x0200u : 0u));
    }
    if (absx >= 0x477ff000u) {  // rounds to >= 65520 -> inf
        return (uint16_t)(sign | 0x7c00u);
    }
    if (absx < 0x33000001u) {  // <= 2^-25: rounds to zero (ties to even -> 0)
        return (uint16_t)sign;
    }
    int32_t exp = (int32_t)(absx >> 23) - 127;
    uint32_t man = (absx & 0x007fffffu) | 0x00800000u;  // 24-bit significand
    uint32_t shift;
    uint32_t hexp;
    if (exp < -14) {  // subnormal half
        shift = (uint32_t)(13 + (-14 - exp));
        hexp = 0;
    } else {
        shift = 13;
        hexp = (uint32_t)(exp + 15);
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q += 1;
    uint32_t h;
    if (hexp == 0) {
        h = q;  // may carry into the exponent field: that is the smallest normal
    } else {
        h = ((hexp << 10) + (q - 0x400u));  // q has the implicit bit at 0x400; carry propagates
    }
    return (uint16_t)(sign | h);
}

float orc_f16_to_f32(uint16_t h) {
    const uint32_t sign = ((uint32_t)h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ffu;
    uint32_t x;
    if (exp == 0) {
        if (man == 0) {
            x = sign;
        } else {
            int e = -1;
            do {
                man <<= 1;
                ++e;
            } while (!(man & 0x400u));
            man &= 0x3ffu;
            x = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        x = sign | 0x7f800000u | (man << 13);
    } else {
        x = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &x, 4);
    return f;
}

// ---- quantisers ---------------------------------------------------------------
// Q8_0: d = max|w| / 127, stored as f16; q = round_half_away(w / float(d16)), clamped to
// [-127, 127]; a block whose stored scale is zero stores q = 0.
void orc_quantize_q8_0(const float* w, size_t rows, size_t cols, uint8_t* blocks) {
    const size_t nb = cols / ORC_QK;
    for (size_t r = 0; r < rows; ++r)
        for (size_t b = 0; b < nb; ++b) {
            const float* src = w + r * cols + b * ORC_QK;
            uint8_t* dst = blocks + (r * nb + b) * ORC_Q8_0_BLOCK_BYTES;
            float amax = 0.0f;
            for (int i = 0; i < ORC_QK; ++i) amax = std::max(amax, std::fabs(src[i]));
            const uint16_t d16 = orc_f32_to_f16(amax / 127.0f);
            const float d = orc_f16_to_f32(d16);
            store_u16(dst, d16);
            for (int i = 0; i < ORC_QK; ++i) {
                int q = (d != 0.0f) ? round_away(src[i] / d) : 0;
                q = std::max(-127, std::min(127, q));
                dst[2 + i] = (uint8_t)(int8_t)q;
            }
        }
}

// Q4_0: m = the element of largest magnitude, sign kept; d = m / 7 stored as f16;
// q = round_half_away(w / float(d16)) + 8 clamped to [0, 15]; zero scale stores q = 8.
void orc_quantize_q4_0(const float* w, size_t rows, size_t cols, uint8_t* blocks) {
    const size_t nb = cols / ORC_QK;
    for (size_t r = 0; r < rows; ++r)
        for (size_t b = 0; b < nb; ++b) {
            const float* src = w + r * cols + b * ORC_QK;
            uint8_t* dst = blocks + (r * nb + b) * ORC_Q4_0_BLOCK_BYTES;
            float amax = 0.0f, m = 0.0f;
            for (int i = 0; i < ORC_QK; ++i) {
                float a = std::fabs(src[i]);
                if (a > amax) {
                    amax = a;
                    m = src[i];
                }
            }
            const uint16_t d16 = orc_f32_to_f16(m / 7.0f);
            const float d = orc_f16_to_f32(d16);
            store_u16(dst, d16);
            uint8_t q[ORC_QK];
            for (int i = 0; i < ORC_QK; ++i) {
                int v = (d != 0.0f) ? round_away(src[i] / d) + 8 : 8;
                q[i] = (uint8_t)std::max(0, std::min(15, v));
            }
            for (int i = 0; i < 16; ++i) dst[2 + i] = (uint8_t)(q[i] | (q[i + 16] << 4));
        }
}

void orc_dequantize_q8_0(const uint8_t* blocks, size_t rows, size_t cols, float* w) {
    const size_t nb = cols / ORC_QK;
    for (size_t r = 0; r < rows; ++r)
        for (size_t b = 0; b < nb; ++b) {
            const uint8_t* src = blocks + (r * nb + b) * ORC_Q8_0_BLOCK_BYTES;
            const float d = orc_f16_to_f32(load_u16(src));
            for (int i = 0; i < ORC_QK; ++i)
                w[r * cols + b * ORC_QK + i] = d * (float)(int8_t)src[2 + i];
        }
}

void orc_dequantize_q4_0(const uint8_t* blocks, size_t rows, size_t cols, float* w) {
    const size_t nb = cols / ORC_QK;
    for (size_t r = 0; r < rows; ++r)
        for (size_t b = 0; b < nb; ++b) {
            const uint8_t* src = blocks + (r * nb + b) * ORC_Q4_0_BLOCK_BYTES;
            const float d = orc_f16_to_f32(load_u16(src));
            for (int i = 0; i < 16; ++i) {
                w[r * cols + b * ORC_QK + i] = d * (float)((int)(src[2 + i] & 0x0f) - 8);
                w[r * cols + b * ORC_QK + 16 + i] = d * (float)((int)(src[2 + i] >> 4) - 8);
            }
        }
}

// ---- GEMV ---------------------------------------------------------------------

}  // extern "C"

namespace {
inline void unpack_q8(const uint8_t* blk, float* d, int* q) {
    *d = orc_f16_to_f32(load_u16(blk));
    for (int i = 0; i < ORC_QK; ++i) q[i] = (int)(int8_t)blk[2 + i];
}
inline void unpack_q4(const uint8_t* blk, float* d, int* q) {
    *d = orc_f16_to_f32(load_u16(blk));
    for (int i = 0; i < 16; ++i) {
        q[i] = (int)(blk[2 + i] & 0x0f) - 8;
        q[i + 16] = (int)(blk[2 + i] >> 4) - 8;
    }
}

template <class Unpack>
void gemv_f32(const uint8_t* blocks, size_t block_bytes, size_t rows, size_t cols, const float* x,
              size_t batch, float* y, int nthreads, Unpack unpack) {
    const size_t nb = cols / ORC_QK;
    parallel_for(rows, nthreads, [&](size_t r) {
        for (size_t v = 0; v < batch; ++v) {
            const float* xv = x + v * cols;
            float acc = 0.0f;
            for (size_t b = 0; b < nb; ++b) {
                float d;
                int q[ORC_QK];
                unpack(blocks + (r * nb + b) * block_bytes, &d, q);
                float s = 0.0f;
                for (int i = 0; i < ORC_QK; ++i) {
                    float p = (float)q[i] * xv[b * ORC_QK + i];
                    s = s + p;
                }
                float t = d * s;
                acc = acc + t;
            }
            y[v * rows + r] = acc;
        }
    });
}

template <class Unpack>
void gemv_f64(const uint8_t* blocks, size_t block_bytes, size_t rows, size_t cols, const float* x,
              size_t batch, double* y, double* absdot, Unpack unpack) {
    const size_t nb = cols / ORC_QK;
    parallel_for(rows, orc_hardware_threads(), [&](size_t r) {
        for (size_t v = 0; v < batch; ++v) {
            const float* xv = x + v * cols;
            double acc = 0.0, aacc = 0.0;
            for (size_t b = 0; b < nb; ++b) {
                float d;
                int q[ORC_QK];
                unpack(blocks + (r * nb + b) * block_bytes, &d, q);
                for (int i = 0; i < ORC_QK; ++i) {
                    double t = (double)d * (double)q[i] * (double)xv[b * ORC_QK + i];
                    acc += t;
                    aacc += std::fabs(t);
                }
            }
            y[v * rows + r] = acc;
            if (absdot) absdot[v * rows + r] = aacc;
        }
    });
}
}  // namespace

extern "C" {

void orc_gemv_q8_0(const uint8_t* blocks, size_t rows, size_t cols, const float* x, size_t batch,
                   float* y, int nthreads) {
    gemv_f32(blocks, ORC_Q8_0_BLOCK_BYTES, rows, cols, x, batch, y, nthreads, unpack_q8);
}
void orc_gemv_q4_0(const uint8_t* blocks, size_t rows, size_t cols, const float* x, size_t batch,
                   float* y, int nthreads) {
    gemv_f32(blocks, ORC_Q4_0_BLOCK_BYTES, rows, cols, x, batch, y, nthreads, unpack_q4);
}
void orc_gemv_q8_0_f64(const uint8_t* blocks, size_t rows, size_t cols, const float* x,
                       size_t batch, double* y, double* absdot) {
    gemv_f64(blocks, ORC_Q8_0_BLOCK_BYTES, rows, cols, x, batch, y, absdot, unpack_q8);
}
void orc_gemv_q4_0_f64(const uint8_t* blocks, size_t rows, size_t cols, const float* x,
                       size_t batch, double* y, double* absdot) {
    gemv_f64(blocks, ORC_Q4_0_BLOCK_BYTES, rows, cols, x, batch, y, absdot, unpack_q4);
}

// ---- reductions -----------------------------------------------------------------
// vortx-shaders/src/linalg/reduce.rs:19-367, the 128-invocation workgroup form: each
// invocation folds elements tid, tid+128, ... along w, then a shared-memory tree with
// strides 64..1 combines the 128 partials.  Only shape.w is walked (reduce.rs:45-51).
// The f32 min / max kernels start from +-1.0e18, not from the type's limits (reduce.rs:292-295).
}  // extern "C"

namespace {
template <class T, class Op>
T reduce_wg(const T* v, const orc_shape& s, T init, Op op, bool square) {
    constexpr uint32_t WG = 128;
    T ws[WG];
    for (uint32_t t = 0; t < WG; ++t) {
        T a = init;
        for (uint32_t i = t; i < s.w; i += WG) {
            T val = v[it(s, 0, 0, 0, i)];
            if (square) val = val * val;
            a = op(a, val);
        }
        ws[t] = a;
    }
    for (uint32_t stride = 64; stride >= 1; stride /= 2)
        for (uint32_t t = 0; t < stride; ++t) ws[t] = op(ws[t], ws[t + stride]);
    return ws[0];
}
}  // namespace

extern "C" {

float orc_reduce_f32(const float* v, const orc_shape* s, int op) {
    switch (op) {
        case 0: return reduce_wg<float>(v, *s, 0.0f, [](float a, float b) { return a + b; }, false);
        case 1: return reduce_wg<float>(v, *s, 1.0f, [](float a, float b) { return a * b; }, false);
        case 2: return reduce_wg<float>(v, *s, 1.0e18f, [](float a, float b) { return std::fmin(a, b); }, false);
        case 3: return reduce_wg<float>(v, *s, -1.0e18f, [](float a, float b) { return std::fmax(a, b); }, false);
        default: return reduce_wg<float>(v, *s, 0.0f, [](float a, float b) { return a + b; }, true);
    }
}
uint32_t orc_reduce_u32(const uint32_t* v, const orc_shape* s, int op) {
    switch (op) {
        case 0: return reduce_wg<uint32_t>(v, *s, 0u, [](uint32_t a, uint32_t b) { return a + b; }, false);
        case 1: return reduce_wg<uint32_t>(v, *s, 1u, [](uint32_t a, uint32_t b) { return a * b; }, false);
        case 2: return reduce_wg<uint32_t>(v, *s, 0xffffffffu, [](uint32_t a, uint32_t b) { return std::min(a, b); }, false);
        default: return reduce_wg<uint32_t>(v, *s, 0u, [](uint32_t a, uint32_t b) { return std::max(a, b); }, false);
    }
}
int32_t orc_reduce_i32(const int32_t* v, const orc_shape* s, int op) {
    // Sum and product wrap, as release-mode Rust integer arithmetic on the device does.
    auto wadd = [](int32_t a, int32_t b) { return (int32_t)((uint32_t)a + (uint32_t)b); };
    auto wmul = [](int32_t a, int32_t b) { return (int32_t)((uint32_t)a * (uint32_t)b); };
    switch (op) {
        case 0: return reduce_wg<int32_t>(v, *s, 0, wadd, false);
        case 1: return reduce_wg<int32_t>(v, *s, 1, wmul, false);
        case 2: return reduce_wg<int32_t>(v, *s, INT32_MAX, [](int32_t a, int32_t b) { return std::min(a, b); }, false);
        default: return reduce_wg<int32_t>(v, *s, INT32_MIN, [](int32_t a, int32_t b) { return std::max(a, b); }, false);
    }
}

int orc_hardware_threads(void) {
    unsigned n = std::thread::hardware_concurrency();
    return n ? (int)n : 1;
}

}  // extern "C"

// ---- element-wise kernels -----------------------------------------------------------------------
// vortx-shaders/src/linalg/op_assign.rs:29-187, contiguous.rs:18-85, repeat.rs:15-43, with
// Shape::decompose (shape.rs:76-86) and it_vec / it_repeating_vec (shape.rs:52-74).
namespace {
struct Idx4 { uint32_t n, c, h, w; };
inline Idx4 decompose(const orc_shape& s, uint32_t i) {
    const uint32_t chw = s.c * s.h * s.w, hw = s.h * s.w;
    const uint32_t i3 = chw ? i / chw : 0;
    const uint32_t r3 = i - i3 * chw;
    const uint32_t i2 = hw ? r3 / hw : 0;
    const uint32_t r2 = r3 - i2 * hw;
    const uint32_t i1 = s.w ? r2 / s.w : 0;
    return Idx4{i3, i2, i1, r2 - i1 * s.w};
}
inline uint32_t it_vec(const orc_shape& s, const Idx4& id) {
    return id.n * s.n_stride + id.c * s.c_stride + id.h * s.h_stride + id.w * s.w_stride;
}
}  // namespace

extern "C" {

void orc_op_assign(int op, float* a, const orc_shape* sa, const float* b, const orc_shape* sb, uint32_t off_a,
                   uint32_t off_b) {
    const uint32_t len = sa->n * sa->c * sa->h * sa->w;
    for (uint32_t i = 0; i < len; ++i) {
        const Idx4 id = decompose(*sa, i);
        const uint32_t ia = off_a + it_vec(*sa, id), ib = off_b + it_vec(*sb, id);
        switch (op) {
            case 0: a[ia] = a[ia] + b[ib]; break;
            case 1: a[ia] = a[ia] - b[ib]; break;
            case 2: a[ia] = a[ia] * b[ib]; break;
            case 3: a[ia] = a[ia] / b[ib]; break;
            default: a[ia] = b[ib]; break;
        }
    }
}

void orc_contiguous(uint32_t* dest, const uint32_t* src, const orc_shape* s, uint32_t offset) {
    const uint32_t len = s->n * s->c * s->h * s->w;
    for (uint32_t i = 0; i < len; ++i) {
        // contiguous.rs:66-76 spells the decomposition out with div and mod; same values
        const uint32_t h_stride = s->w, c_stride = s->h * s->w, n_stride = s->c * s->h * s->w;
        const uint32_t n = i / n_stride, c = (i % n_stride) / c_stride, h = (i % c_stride) / h_stride, w = i % h_stride;
        dest[i] = src[offset + it(*s, n, c, h, w)];
    }
}

void orc_repeat(float* result, const orc_shape* sr, const float* source, const orc_shape* ss) {
    const uint32_t len = sr->n * sr->c * sr->h * sr->w;
    for (uint32_t i = 0; i < len; ++i) {
        const Idx4 id = decompose(*sr, i);
        const Idx4 w{id.n % ss->n, id.c % ss->c, id.h % ss->h, id.w % ss->w};
        result[it_vec(*sr, id)] = source[it_vec(*ss, w)];
    }
}

}  // extern "C"
