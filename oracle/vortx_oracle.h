/*
 * CPU oracle for the vortx matmul hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * This library restates, on the host, the arithmetic of the reference's GEMM
 * shaders and defines the block-quantised GEMV the reference does not have.
 * It is the checker the CUDA path is compared with; nothing in the product
 * path may link, load or call it.
 *
 * Parity status
 *   - f32 GEMM: restated loop-for-loop from vortx-shaders/src/linalg/gemm.rs.
 *     The reference holds no golden vectors for it.  The only pin it offers is
 *     the property its own test checks (src/linalg/gemm.rs:365-444): a 256x256
 *     matrix times a 256-vector agrees with a plain host product to 1e-3.
 *     That property is replayed in the tests.
 *   - Q8_0 / Q4_0 GEMV: PARITY UNPINNED.  The reference has no quantised code,
 *     no test and no fixture for it; the format below is this library's own
 *     statement of the block layout.
 */
#ifndef VORTX_ORACLE_H
#define VORTX_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* vortx-shaders/src/linalg/shape.rs:9-29 — eight u32, sizes then strides, in elements. */
typedef struct {
    uint32_t n, c, h, w;
    uint32_t n_stride, c_stride, h_stride, w_stride;
} orc_shape;

/* vortx-shaders/src/linalg/shape.rs:46-48 — u32 wrapping index arithmetic. */
uint32_t orc_shape_it(const orc_shape* s, uint32_t n, uint32_t c, uint32_t h, uint32_t w);

/* vortx-shaders/src/linalg/gemm.rs:197-237 — one invocation per (x=col, y=row, z=c). */
void orc_gemm_naive(float* out, const float* lhs, const float* rhs,
                    const orc_shape* so, const orc_shape* sl, const orc_shape* sr);

/* vortx-shaders/src/linalg/gemm.rs:41-194 — 16x16 workgroups, 64x64x16 tiles, 4x4 per thread.
 * grid_x / grid_y / grid_z are workgroup counts (src/linalg/gemm.rs:311-321 divided by 16). */
void orc_gemm_tiled(float* out, const float* lhs, const float* rhs,
                    const orc_shape* so, const orc_shape* sl, const orc_shape* sr,
                    int nthreads);

/* Host dispatch rule, src/linalg/gemm.rs:111-112: tiled iff M >= 32 || N >= 32. */
void orc_gemm_dispatch(float* out, const float* lhs, const float* rhs,
                       const orc_shape* so, const orc_shape* sl, const orc_shape* sr,
                       int nthreads);

/* f64-accumulated product, the stand-in for the nalgebra host product the
 * reference test compares with (src/linalg/gemm.rs:429). Contiguous row-major. */
void orc_gemm_f64(double* out, const float* lhs, const float* rhs,
                  uint32_t m, uint32_t n, uint32_t k);

/* ---- block quantisation (format defined here; no reference counterpart) ----
 * Q8_0 block, 34 bytes: f16 scale d (little endian) then 32 int8 q.   w = d * q.
 * Q4_0 block, 18 bytes: f16 scale d then 16 bytes; byte i holds element i in
 * its low nibble and element i+16 in its high nibble.                  w = d * (q - 8).
 */
#define ORC_QK 32
#define ORC_Q8_0_BLOCK_BYTES 34
#define ORC_Q4_0_BLOCK_BYTES 18

uint16_t orc_f32_to_f16(float f);  /* round to nearest even */
float orc_f16_to_f32(uint16_t h);

/* rows x cols f32 (cols % 32 == 0) -> rows*cols/32 blocks, row after row. */
void orc_quantize_q8_0(const float* w, size_t rows, size_t cols, uint8_t* blocks);
void orc_quantize_q4_0(const float* w, size_t rows, size_t cols, uint8_t* blocks);
void orc_dequantize_q8_0(const uint8_t* blocks, size_t rows, size_t cols, float* w);
void orc_dequantize_q4_0(const uint8_t* blocks, size_t rows, size_t cols, float* w);

/* y[v*rows + r] = sum_b float(d) * sum_i float(q) * x[v*cols + 32b+i], f32, in that order.
 * batch vectors of x are contiguous, batch vectors of y are contiguous. */
void orc_gemv_q8_0(const uint8_t* blocks, size_t rows, size_t cols,
                   const float* x, size_t batch, float* y, int nthreads);
void orc_gemv_q4_0(const uint8_t* blocks, size_t rows, size_t cols,
                   const float* x, size_t batch, float* y, int nthreads);
/* The same sums carried in f64: the yardstick for the tolerance tests.
 * absdot[v*rows+r] (may be NULL) receives sum |w*x|, the conditioning of the row. */
void orc_gemv_q8_0_f64(const uint8_t* blocks, size_t rows, size_t cols,
                       const float* x, size_t batch, double* y, double* absdot);
void orc_gemv_q4_0_f64(const uint8_t* blocks, size_t rows, size_t cols,
                       const float* x, size_t batch, double* y, double* absdot);

/* Serial reductions, vortx-shaders/src/linalg/reduce.rs (workgroup of 128, stride loop
 * then tree) restated; op: 0 sum, 1 product, 2 min, 3 max, 4 squared norm. */
float orc_reduce_f32(const float* v, const orc_shape* s, int op);
uint32_t orc_reduce_u32(const uint32_t* v, const orc_shape* s, int op);
int32_t orc_reduce_i32(const int32_t* v, const orc_shape* s, int op);

/* Element-wise kernels: vortx-shaders/src/linalg/op_assign.rs:29-187 (op: 0 add, 1 sub, 2 mul, 3 div,
 * 4 copy; offsets as in gpu_copy_with_offsets), contiguous.rs:18-85, repeat.rs:15-43. */
void orc_op_assign(int op, float* a, const orc_shape* sa, const float* b, const orc_shape* sb,
                   uint32_t off_a, uint32_t off_b);
void orc_contiguous(uint32_t* dest, const uint32_t* src, const orc_shape* s, uint32_t offset);
void orc_repeat(float* result, const orc_shape* sr, const float* source, const orc_shape* ss);

int orc_hardware_threads(void);

#ifdef __cplusplus
}
#endif
#endif
