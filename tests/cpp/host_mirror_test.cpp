// The C++ host mirror (include/vortx_b200.hpp) driven the way vortx's own tests drive the Rust API.
//
//   layout    the ten broadcast_* unit tests of src/shapes.rs:646-782 and the view algebra: host only, needs no GPU
//   gpu       gpu_gemm_generic of src/linalg/gemm.rs:365-444 (256x256 matrix times a 256-vector within 1e-3 of a
//             host product) for dispatch / dispatch_naive / dispatch_tiled / dispatch_tf32, Gemm::dispatch's shape
//             asserts, a transposed view, OpAssign / Reduce / Contiguous, and the quantised GEMV as single
//             products and as a list
// Usage: host_mirror_test layout | gpu.  Exit code 0 and a last line "ok" on success.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <memory>
#include <random>

#include "vortx_b200.hpp"

using namespace vortx;

static int failures = 0;
#define EXPECT(cond)                                                            \
    do {                                                                        \
        if (!(cond)) {                                                          \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);       \
            ++failures;                                                         \
        }                                                                       \
    } while (0)

static bool sizes_are(const TensorLayout& l, std::array<uint32_t, 4> size, std::array<uint32_t, 4> stride) {
    for (int i = 0; i < 4; ++i)
        if (l.size(i) != size[i] || l.stride(i) != stride[i]) return false;
    return true;
}

static void layout_tests() {
    // The properties src/shapes.rs:646-782 pins: ranks are equalised by padding on the left, sizes stay as
    // they are, and every axis of size 1 gets stride 0; incompatible sizes give None.
    {
        auto a = TensorLayout::contiguous({3, 4}), b = TensorLayout::contiguous({3, 4});
        auto r = TensorLayout::broadcast(a, b);
        EXPECT(r && r->first.size(0) == 3 && r->first.size(1) == 4 && r->first.stride(0) == 4 && r->first.stride(1) == 1);
        EXPECT(r && r->second.stride(0) == 4 && r->second.stride(1) == 1);
    }
    {
        auto scalar = TensorLayout::contiguous({1}), m = TensorLayout::contiguous({3, 4});
        auto r = TensorLayout::broadcast(scalar, m);
        EXPECT(r && r->first.rank() == 2 && r->second.rank() == 2);
        EXPECT(r && r->first.size(0) == 1 && r->first.size(1) == 1 && r->first.stride(0) == 0 && r->first.stride(1) == 0);
        EXPECT(r && r->second.size(0) == 3 && r->second.size(1) == 4);
    }
    {
        auto col = TensorLayout::contiguous({3, 1}), m = TensorLayout::contiguous({3, 4});
        auto r = TensorLayout::broadcast(col, m);
        EXPECT(r && r->first.size(0) == 3 && r->first.size(1) == 1 && r->first.stride(1) == 0);
    }
    {
        auto row = TensorLayout::contiguous({1, 4}), m = TensorLayout::contiguous({3, 4});
        auto r = TensorLayout::broadcast(row, m);
        EXPECT(r && r->first.size(0) == 1 && r->first.size(1) == 4 && r->first.stride(0) == 0);
    }
    {
        auto a = TensorLayout::contiguous({4, 1}), b = TensorLayout::contiguous({1, 3});
        auto r = TensorLayout::broadcast(a, b);
        EXPECT(r && r->first.stride(1) == 0 && r->second.stride(0) == 0 && r->first.size(0) == 4 && r->second.size(1) == 3);
    }
    {
        auto a = TensorLayout::contiguous({4, 3}), b = TensorLayout::contiguous({2, 3});
        EXPECT(!TensorLayout::broadcast(a, b));   // incompatible: None
    }
    // view algebra
    auto m = TensorLayout::contiguous({6, 8});
    EXPECT(m.len() == 48 && m.is_contiguous());
    auto t = m.transpose_last_dims();
    EXPECT(t.size(0) == 8 && t.size(1) == 6 && t.stride(0) == 1 && t.stride(1) == 8 && !t.is_contiguous());
    auto c = m.canonicalize();
    EXPECT(sizes_are(c, {1, 1, 6, 8}, {48, 48, 8, 1}));
    auto rows = m.rows(2, 3);
    EXPECT(rows.offset() == 16 && rows.size(0) == 3 && rows.size(1) == 8);
    auto cols = m.columns(5, 2);
    EXPECT(cols.offset() == 5 && cols.size(1) == 2 && cols.stride(0) == 8);
    EXPECT(!TensorLayout::contiguous({2, 2, 2, 2}).unsqueeze(0));   // rank already 4: None
    bool threw = false;
    try {
        m.rows(5, 3);   // past the end: the reference panics
    } catch (const Error&) {
        threw = true;
    }
    EXPECT(threw);
    vx_shape s = m.canonicalize().into_gpu();
    EXPECT(s.h == 6 && s.w == 8 && s.n == 1 && s.c == 1 && s.h_stride == 8 && s.w_stride == 1);
}

static std::vector<float> random_vec(size_t n, uint32_t seed, float lo = -1.0f, float hi = 1.0f) {
    std::mt19937 rng(seed);
    std::uniform_real_distribution<float> d(lo, hi);
    std::vector<float> v(n);
    for (auto& x : v) x = d(rng);
    return v;
}

static void gpu_tests() {
    GpuBackend backend(0);
    // ---- gpu_gemm_generic, src/linalg/gemm.rs:365-444
    const uint32_t NROWS = 256, NCOLS = 256;
    const auto m1 = random_vec((size_t)NROWS * NCOLS, 1), v1 = random_vec(NCOLS, 2);
    std::vector<double> want(NROWS, 0.0);
    for (uint32_t i = 0; i < NROWS; ++i)
        for (uint32_t k = 0; k < NCOLS; ++k) want[i] += (double)m1[(size_t)i * NCOLS + k] * v1[k];
    auto gm = Tensor<float>::matrix(backend, NROWS, NCOLS, m1);
    auto gv = Tensor<float>::matrix(backend, NCOLS, 1, v1);
    using Fn = void (*)(const GpuBackend&, const TensorMut<float>&, const TensorRef<float>&, const TensorRef<float>&);
    const Fn entries[] = {&Gemm::dispatch, &Gemm::dispatch_naive, &Gemm::dispatch_tiled, &Gemm::dispatch_tf32};
    for (Fn entry : entries) {
        auto result = Tensor<float>::matrix_uninit(backend, NROWS, 1);
        entry(backend, result.as_view_mut(), gm.as_view(), gv.as_view());
        backend.synchronize();
        const auto got = result.read();
        for (uint32_t i = 0; i < NROWS; ++i) EXPECT(std::fabs(got[i] - want[i]) <= 1.0e-3);   // epsilon = 1.0e-3, :442
    }
    // ---- the shape asserts of Gemm::dispatch (:70-104) panic in the reference
    {
        auto bad = Tensor<float>::matrix_uninit(backend, NROWS + 1, 1);
        bool threw = false;
        try {
            Gemm::dispatch(backend, bad.as_view_mut(), gm.as_view(), gv.as_view());
        } catch (const ShapeMismatch&) {
            threw = true;
        }
        EXPECT(threw);
    }
    // ---- a transposed view as lhs: out = m1^T v
    {
        std::vector<double> wt(NCOLS, 0.0);
        for (uint32_t i = 0; i < NROWS; ++i)
            for (uint32_t k = 0; k < NCOLS; ++k) wt[k] += (double)m1[(size_t)i * NCOLS + k] * v1[i];
        auto result = Tensor<float>::matrix_uninit(backend, NCOLS, 1);
        Gemm::dispatch(backend, result.as_view_mut(), gm.as_view().transpose_last_dims(), gv.as_view());
        const auto got = result.read();
        for (uint32_t i = 0; i < NCOLS; ++i) EXPECT(std::fabs(got[i] - wt[i]) <= 1.0e-3);
    }
    // ---- TF32 on a size its tensor-core kernel takes
    {
        const uint32_t n = 512;
        const auto a = random_vec((size_t)n * n, 3), b = random_vec((size_t)n * n, 4);
        auto ga = Tensor<float>::matrix(backend, n, n, a), gb = Tensor<float>::matrix(backend, n, n, b);
        auto gc = Tensor<float>::matrix_uninit(backend, n, n);
        Gemm::dispatch_tf32(backend, gc.as_view_mut(), ga.as_view(), gb.as_view());
        EXPECT(Gemm::last_kernel(backend) == 3);
        const auto got = gc.read();
        double num = 0, den = 0;
        for (uint32_t i = 0; i < n; i += 7)
            for (uint32_t j = 0; j < n; j += 5) {
                double t = 0;
                for (uint32_t k = 0; k < n; ++k) t += (double)a[(size_t)i * n + k] * b[(size_t)k * n + j];
                num += (got[(size_t)i * n + j] - t) * (got[(size_t)i * n + j] - t);
                den += t * t;
            }
        EXPECT(std::sqrt(num / den) <= 5e-3);
    }
    // ---- OpAssign with broadcast, Reduce, Contiguous
    {
        const auto a = random_vec(12, 5), row = random_vec(4, 6);
        auto ga = Tensor<float>::matrix(backend, 3, 4, a);
        auto gr = Tensor<float>::vector(backend, row);
        OpAssign::launch(backend, OpAssignVariant::Add, ga.as_view_mut(), gr.as_view());
        auto got = ga.read();
        for (int i = 0; i < 12; ++i) EXPECT(got[i] == a[i] + row[i % 4]);
        auto sum = Tensor<float>::scalar(backend, 0.0f);
        Reduce::launch(backend, ReduceVariant::Max, gr.as_view(), sum.as_view_mut());
        float mx = row[0];
        for (float x : row) mx = std::fmax(mx, x);
        EXPECT(sum.read()[0] == mx);
        auto tr = Tensor<float>::matrix_uninit(backend, 4, 3);
        Contiguous::launch(backend, tr.as_view_mut(), ga.as_view().transpose_last_dims());
        const auto gt = tr.read();
        for (int i = 0; i < 3; ++i)
            for (int j = 0; j < 4; ++j) EXPECT(gt[j * 3 + i] == got[i * 4 + j]);
    }
    // ---- quantised GEMV: single products and the same products as one list
    {
        const size_t rows = 96, cols = 1024;
        const auto x = random_vec(cols, 9);
        auto gx = Tensor<float>::vector(backend, x);
        std::vector<std::unique_ptr<QuantizedMatrix>> ws;
        std::vector<Tensor<float>> single, listed;
        for (int i = 0; i < 3; ++i) {
            ws.emplace_back(new QuantizedMatrix(backend, VX_Q4_0, random_vec(rows * cols, 10 + i, -0.05f, 0.05f), rows, cols));
            single.push_back(Tensor<float>::vector_uninit(backend, rows));
            listed.push_back(Tensor<float>::vector_uninit(backend, rows));
            Gemv::dispatch(backend, single.back().as_view_mut(), *ws.back(), gx.as_view());
        }
        std::vector<vx_gemv_op> ops(3);
        for (int i = 0; i < 3; ++i) {
            std::memset(&ops[i], 0, sizeof(vx_gemv_op));
            ops[i].w = ws[i]->handle();
            ops[i].nrows = rows;
            ops[i].x = gx.buffer().ptr();
            ops[i].y = listed[i].buffer().ptr();
            ops[i].y_stride = 1;
        }
        GemvBatch batch(backend, ops);
        batch.launch();
        backend.synchronize();
        for (int i = 0; i < 3; ++i) {
            const auto a = single[i].read(), b = listed[i].read();
            EXPECT(std::memcmp(a.data(), b.data(), rows * sizeof(float)) == 0);
        }
        // the same three matrices times the same vector in one call (vx_gemv_q_multi), and with two vectors; then the
        // list with host buffers, recorded once and replayed (vx_host_pipeline): pinned x up, the list, y down
        {
            const vx_qweights* wp[3] = {ws[0]->handle(), ws[1]->handle(), ws[2]->handle()};
            std::vector<Tensor<float>> multi;
            float* yp[3];
            for (int i = 0; i < 3; ++i) {
                multi.push_back(Tensor<float>::vector_uninit(backend, 2 * rows));
                yp[i] = multi.back().buffer().ptr();
            }
            std::vector<float> x2(2 * cols);
            for (size_t c = 0; c < cols; ++c) {
                x2[c] = x[c];
                x2[cols + c] = 0.5f * x[cols - 1 - c];
            }
            auto gx2 = Tensor<float>::vector(backend, x2);
            check(vx_gemv_q_multi(backend.ctx(), wp, 3, gx2.buffer().ptr(), cols, yp, rows, 2));
            backend.synchronize();
            for (int i = 0; i < 3; ++i) {
                const auto a = single[i].read(), b = multi[i].read();
                double worst = 0, largest = 0;
                for (size_t r = 0; r < rows; ++r) {
                    worst = std::fmax(worst, std::fabs((double)a[r] - b[r]));
                    largest = std::fmax(largest, std::fabs((double)a[r]));
                }
                EXPECT(worst / largest <= 1e-5);          // the tensor-core kernel against the streaming kernel
            }
            void *hx = nullptr, *hy = nullptr;
            check(vx_host_alloc(cols * sizeof(float), &hx));
            check(vx_host_alloc(3 * rows * sizeof(float), &hy));
            std::memcpy(hx, x.data(), cols * sizeof(float));
            auto gxh = Tensor<float>::vector_uninit(backend, cols);
            auto gyh = Tensor<float>::vector_uninit(backend, 3 * rows);
            std::vector<vx_gemv_op> hops(3);
            for (int i = 0; i < 3; ++i) {
                std::memset(&hops[i], 0, sizeof(vx_gemv_op));
                hops[i].w = ws[i]->handle();
                hops[i].nrows = rows;
                hops[i].x = gxh.buffer().ptr();
                hops[i].y = gyh.buffer().ptr() + i * rows;
                hops[i].y_stride = 1;
            }
            GemvBatch hbatch(backend, hops);
            vx_host_stage stage;
            std::memset(&stage, 0, sizeof(stage));
            stage.batch = hbatch.handle();
            stage.up_device = gxh.buffer().ptr();
            stage.up_host = hx;
            stage.up_bytes = cols * sizeof(float);
            stage.down_host = hy;
            stage.down_host_pitch = stage.down_device_pitch = stage.down_width_bytes = 3 * rows * sizeof(float);
            stage.down_device = gyh.buffer().ptr();
            stage.down_rows = 1;
            vx_host_pipeline* pipe = nullptr;
            check(vx_host_pipeline_create(backend.ctx(), &stage, 1, &pipe));
            for (int rep = 0; rep < 2; ++rep) {
                std::memset(hy, 0xFF, 3 * rows * sizeof(float));
                check(vx_host_pipeline_run(pipe));
                for (int i = 0; i < 3; ++i) {
                    const auto a = single[i].read();
                    EXPECT(std::memcmp(a.data(), static_cast<float*>(hy) + i * rows, rows * sizeof(float)) == 0);
                }
            }
            check(vx_host_pipeline_free(pipe));
            check(vx_host_free(hx));
            check(vx_host_free(hy));
        }
        // both block formats against a host product over the dequantised weights: 1e-4 of the largest output
        for (vx_qtype qt : {VX_Q8_0, VX_Q4_0}) {
            const auto w = random_vec(rows * cols, 20 + (int)qt, -0.05f, 0.05f);
            std::vector<uint8_t> blocks(rows * (cols / 32) * vx_qblock_bytes(qt));
            check(vx_quantize(qt, w.data(), rows, cols, blocks.data()));
            std::vector<float> deq(rows * cols);
            check(vx_dequantize_host(qt, blocks.data(), rows, cols, deq.data()));
            QuantizedMatrix qm(backend, qt, w, rows, cols);
            auto gy = Tensor<float>::vector_uninit(backend, rows);
            Gemv::dispatch(backend, gy.as_view_mut(), qm, gx.as_view());
            const auto got = gy.read();
            double worst = 0, largest = 0;
            for (size_t r = 0; r < rows; ++r) {
                double t = 0;
                for (size_t c = 0; c < cols; ++c) t += (double)deq[r * cols + c] * x[c];
                worst = std::fmax(worst, std::fabs(got[r] - t));
                largest = std::fmax(largest, std::fabs(t));
            }
            EXPECT(worst / largest <= 1e-4);
        }
    }
    std::printf("kernels launched: %llu\n", (unsigned long long)backend.launch_count());
}

int main(int argc, char** argv) {
    const std::string what = argc > 1 ? argv[1] : "layout";
    try {
        layout_tests();
        if (what == "gpu") gpu_tests();
    } catch (const std::exception& e) {
        std::printf("exception: %s\n", e.what());
        return 2;
    }
    if (failures) {
        std::printf("%d check(s) failed\n", failures);
        return 1;
    }
    std::printf("ok\n");
    return 0;
}
