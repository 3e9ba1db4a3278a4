// A host without Python or torch drives the multi-GPU layer through the C ABI alone: one process per GPU.
//
//   group_test <world> <rank> <id-file>
// Rank 0 creates the NCCL unique id and writes it to <id-file>; the other ranks wait for the file.  Every rank
// then: creates its context and group; all-gathers and broadcasts a pattern; runs the row-sharded Q4_0 GEMV
// (rows of every rank stored on every GPU by the kernel's epilogue + the group's barrier) and checks the whole y
// against the same product computed on its own GPU from the whole matrix; runs the column-sharded TF32 GEMM the
// same way.  With world = 1 it needs neither NCCL nor a second GPU.  Exit code 0 and a last line "ok".
#include <unistd.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <random>
#include <vector>

#include "vortx_b200.h"

#define CHECK(expr)                                                                              \
    do {                                                                                         \
        const vx_status st_ = (expr);                                                            \
        if (st_ != VX_OK) {                                                                      \
            std::printf("FAILED %s:%d: %s -> %d (%s)\n", __FILE__, __LINE__, #expr, st_, vx_last_error()); \
            return 1;                                                                            \
        }                                                                                        \
    } while (0)
#define EXPECT(cond)                                                        \
    do {                                                                    \
        if (!(cond)) {                                                      \
            std::printf("FAILED %s:%d: %s\n", __FILE__, __LINE__, #cond);   \
            return 1;                                                       \
        }                                                                   \
    } while (0)

int main(int argc, char** argv) {
    if (argc != 4) {
        std::printf("usage: group_test <world> <rank> <id-file>\n");
        return 2;
    }
    const size_t world = (size_t)std::atoi(argv[1]), rank = (size_t)std::atoi(argv[2]);
    const char* id_file = argv[3];
    vx_context* ctx = nullptr;
    CHECK(vx_context_create((int32_t)rank, &ctx));

    unsigned char id[128] = {};
    if (world > 1) {
        if (rank == 0) {
            CHECK(vx_group_unique_id(id));
            std::string tmp = std::string(id_file) + ".tmp";
            FILE* f = std::fopen(tmp.c_str(), "wb");
            EXPECT(f && std::fwrite(id, 1, 128, f) == 128);
            std::fclose(f);
            EXPECT(std::rename(tmp.c_str(), id_file) == 0);
        } else {
            FILE* f = nullptr;
            for (int tries = 0; tries < 3000 && !f; ++tries) {
                f = std::fopen(id_file, "rb");
                if (!f) usleep(10000);
            }
            EXPECT(f && std::fread(id, 1, 128, f) == 128);
            std::fclose(f);
        }
    }
    vx_group* g = nullptr;
    CHECK(vx_group_create(ctx, world, rank, id, &g));
    size_t w2 = 0, r2 = 0;
    CHECK(vx_group_info(g, &w2, &r2));
    EXPECT(w2 == world && r2 == rank);

    // ---- collectives: every rank contributes 256 bytes of its own pattern
    {
        void* buf = nullptr;
        CHECK(vx_alloc(ctx, 256 * world, &buf));
        std::vector<unsigned char> mine(256), all(256 * world);
        for (int i = 0; i < 256; ++i) mine[i] = (unsigned char)(i * 7 + rank * 31);
        CHECK(vx_upload(ctx, static_cast<unsigned char*>(buf) + 256 * rank, mine.data(), 256));
        CHECK(vx_group_all_gather(g, nullptr, buf, 256));
        CHECK(vx_download(ctx, all.data(), buf, all.size()));
        for (size_t r = 0; r < world; ++r)
            for (int i = 0; i < 256; ++i) EXPECT(all[256 * r + i] == (unsigned char)(i * 7 + r * 31));
        // broadcast: every rank puts its own pattern at the front, the last rank's one wins everywhere
        CHECK(vx_upload(ctx, buf, mine.data(), 256));
        CHECK(vx_group_broadcast(g, buf, 256, world - 1));
        CHECK(vx_download(ctx, all.data(), buf, 256));
        for (int i = 0; i < 256; ++i) EXPECT(all[i] == (unsigned char)(i * 7 + (world - 1) * 31));
        CHECK(vx_free(ctx, buf));
    }

    // ---- row-sharded Q4_0 GEMV against the unsharded product on this GPU
    {
        const size_t rows = 1024 * world, cols = 2048, shard = rows / world;
        std::mt19937 rng(7);
        std::normal_distribution<float> nw(0.0f, 0.02f), nx(0.0f, 1.0f);
        std::vector<float> w(rows * cols), x(cols);
        for (auto& v : w) v = nw(rng);
        for (auto& v : x) v = nx(rng);
        std::vector<unsigned char> blocks(rows * cols / 32 * 18);
        CHECK(vx_quantize(VX_Q4_0, w.data(), rows, cols, blocks.data()));
        vx_qweights *whole = nullptr, *slab = nullptr;
        CHECK(vx_qweights_upload(ctx, VX_Q4_0, blocks.data(), rows, cols, &whole));
        CHECK(vx_qweights_upload(ctx, VX_Q4_0, blocks.data() + rank * shard * (cols / 32 * 18), shard, cols, &slab));
        void *xd = nullptr, *yref = nullptr;
        CHECK(vx_alloc(ctx, cols * 4, &xd));
        CHECK(vx_alloc(ctx, rows * 4, &yref));
        CHECK(vx_upload(ctx, xd, x.data(), cols * 4));
        CHECK(vx_gemv_q(ctx, whole, static_cast<float*>(xd), cols, static_cast<float*>(yref), rows, 1));
        std::vector<void*> y_all(world);
        CHECK(vx_group_peer_alloc(g, rows * 4, y_all.data()));
        for (int rep = 0; rep < 3; ++rep)
            CHECK(vx_group_gemv_q(g, slab, rank * shard, static_cast<float*>(xd), y_all.data(), 0));
        std::vector<float> want(rows), got(rows);
        CHECK(vx_download(ctx, want.data(), yref, rows * 4));
        CHECK(vx_download(ctx, got.data(), y_all[rank], rows * 4));
        EXPECT(std::memcmp(want.data(), got.data(), rows * 4) == 0);      // same kernel, same rows: the same bits
        double norm = 0;
        for (float v : got) norm += (double)v * v;
        EXPECT(norm > 0);
        CHECK(vx_group_barrier(g));                                        // nobody frees while a peer may still store
        CHECK(vx_synchronize(ctx));
        CHECK(vx_group_peer_free(g, y_all.data()));
        CHECK(vx_qweights_free(ctx, whole));
        CHECK(vx_qweights_free(ctx, slab));
        CHECK(vx_free(ctx, xd));
        CHECK(vx_free(ctx, yref));
    }

    // ---- column-sharded TF32 GEMM against the unsharded tensor-core product on this GPU
    {
        const size_t m = 512, k = 256, n = 256 * world, ncols = n / world, col0 = rank * ncols;
        std::mt19937 rng(11);
        std::uniform_real_distribution<float> u(-1.0f, 1.0f);
        std::vector<float> a(m * k), b(k * n);
        for (auto& v : a) v = u(rng);
        for (auto& v : b) v = u(rng);
        void *ad = nullptr, *bd = nullptr, *cref = nullptr;
        CHECK(vx_alloc(ctx, a.size() * 4, &ad));
        CHECK(vx_alloc(ctx, b.size() * 4, &bd));
        CHECK(vx_alloc(ctx, m * n * 4, &cref));
        CHECK(vx_upload(ctx, ad, a.data(), a.size() * 4));
        CHECK(vx_upload(ctx, bd, b.data(), b.size() * 4));
        vx_shapes3 s{};
        auto set = [](vx_shape& sh, size_t h, size_t w, size_t hs) {
            sh.n = sh.c = 1; sh.h = (uint32_t)h; sh.w = (uint32_t)w;
            sh.n_stride = sh.c_stride = (uint32_t)(h * hs); sh.h_stride = (uint32_t)hs; sh.w_stride = 1;
        };
        set(s.out, m, n, n); set(s.lhs, m, k, k); set(s.rhs, k, n, n);
        CHECK(vx_gemm_f32(ctx, VX_GEMM_TF32, static_cast<float*>(cref), static_cast<float*>(ad), static_cast<float*>(bd), &s, 0, 0, 0));
        std::vector<void*> c_all(world);
        CHECK(vx_group_peer_alloc(g, m * n * 4, c_all.data()));
        for (int rep = 0; rep < 2; ++rep)
            CHECK(vx_group_gemm_tf32(g, static_cast<float*>(ad), static_cast<float*>(bd) + col0, m, n, k, col0, ncols, n, c_all.data()));
        std::vector<float> want(m * n), got(m * n);
        CHECK(vx_download(ctx, want.data(), cref, m * n * 4));
        CHECK(vx_download(ctx, got.data(), c_all[rank], m * n * 4));
        EXPECT(std::memcmp(want.data(), got.data(), m * n * 4) == 0);
        // and within the TF32 bar of the f64 product, on a sample of rows
        double num = 0, den = 0;
        for (size_t i = 0; i < m; i += 37)
            for (size_t j = 0; j < n; ++j) {
                double acc = 0;
                for (size_t kk = 0; kk < k; ++kk) acc += (double)a[i * k + kk] * b[kk * n + j];
                num += (got[i * n + j] - acc) * (got[i * n + j] - acc);
                den += acc * acc;
            }
        EXPECT(std::sqrt(num / den) <= 5e-3);
        CHECK(vx_group_barrier(g));
        CHECK(vx_synchronize(ctx));
        CHECK(vx_group_peer_free(g, c_all.data()));
        CHECK(vx_free(ctx, ad));
        CHECK(vx_free(ctx, bd));
        CHECK(vx_free(ctx, cref));
    }
    CHECK(vx_group_barrier(g));
    CHECK(vx_synchronize(ctx));
    CHECK(vx_group_destroy(g));
    CHECK(vx_context_destroy(ctx));
    std::printf("rank %zu of %zu: ok\n", rank, world);
    return 0;
}
