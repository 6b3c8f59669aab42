// Multi-GPU GEMM through the C++ API, one process per GPU:
//     test_engine_sharded <rank> <nranks> <id_file>
// Every rank builds the same global problem from a seeded generator, multiplies its row block with
// engine.blas().gemm_row_sharded and checks the gathered C against a host fp64 reference.
#include <cstdlib>
#include <random>
#include <vector>
#include <SushiBLAS/SushiBLAS.h>
#include "check.hpp"

static int g_rank = 0, g_nranks = 1;
static std::string g_id_file;

static sr::Execution::RuntimeContext& runtime()
{
    static sr::Execution::DistributedConfig cfg{g_rank, g_nranks, g_rank, g_id_file, 60, "test_engine_sharded"};
    static sr::Execution::RuntimeContext ctx(cfg);
    return ctx;
}

static std::vector<float> random_vec(size_t n, unsigned seed)
{
    std::mt19937 g(seed);
    std::uniform_real_distribution<float> d(-1.0f, 1.0f);
    std::vector<float> v(n);
    for (auto& x : v) x = d(g);
    return v;
}

TEST_CASE(RowShardedGemmGathersTheFullResult)
{
    auto& rt = runtime();
    EXPECT_EQ(rt.rank(), g_rank); EXPECT_EQ(rt.nranks(), g_nranks);
    sb::Engine engine(rt);
    auto dev = sr::Memory::AllocStrategy::DEVICE;
    for (auto [m, n, k, alpha, beta] : {std::tuple{1024, 512, 256, 1.0f, 0.0f}, std::tuple{301, 64, 40, 1.5f, 0.5f}})
    {
        int64_t first = 0, count = 0;
        sushi_cuda_partition(m, g_nranks, g_rank, &first, &count);
        auto a = random_vec(size_t(m) * k, 1), b = random_vec(size_t(k) * n, 2), c = random_vec(size_t(m) * n, 3);
        auto A_local = engine.create_tensor({count, k}, dev), B = engine.create_tensor({k, n}, dev), C = engine.create_tensor({m, n}, dev);
        A_local.from_host(a.data() + size_t(first) * k); B.from_host(b.data()); C.from_host(c.data());
        engine.blas().gemm_row_sharded(A_local, B, C, false, false, alpha, beta);
        engine.execute().wait();
        std::vector<float> got(size_t(m) * n);
        C.to_host(got.data());
        for (int i = 0; i < m; i += 7)
            for (int j = 0; j < n; j += 5)
            {
                double s = 0;
                for (int p = 0; p < k; ++p) s += double(a[size_t(i) * k + p]) * double(b[size_t(p) * n + j]);
                EXPECT_NEAR(got[size_t(i) * n + j], alpha * s + beta * c[size_t(i) * n + j], 2e-4);
            }
    }
    // argument checks
    auto A_bad = engine.create_tensor({3, 5}, dev), B = engine.create_tensor({5, 8}, dev), C = engine.create_tensor({100, 8}, dev);
    EXPECT_THROWS(engine.blas().gemm_row_sharded(A_bad, B, C), "A_local must hold");
    auto H = engine.create_tensor({100, 8});
    EXPECT_THROWS(engine.blas().gemm_row_sharded(A_bad, B, H), "DEVICE tensors");
}

int main(int argc, char** argv)
{
    if (argc < 4) { std::fprintf(stderr, "usage: %s <rank> <nranks> <id_file>\n", argv[0]); return 2; }
    g_rank = std::atoi(argv[1]); g_nranks = std::atoi(argv[2]); g_id_file = argv[3];
    return check::run_all();
}
