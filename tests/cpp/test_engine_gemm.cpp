// GPU tests of the C++ Engine/Tensor API: the reference's own GEMM tests
// (tests/blas/level3/test_gemm.cpp:39-88) with their fixture helpers
// (tests/test_common.hpp:36-58: fill through data_as<T>() on the host, verify with an absolute
// tolerance of 1e-4), the caller shapes of tests/runtime/test_framework_sim.cpp:18-58,81-111 and
// tests/runtime/test_dependency_stress.cpp:17-45,67-83, examples/example.cpp:34-56, plus the
// cases the reference never tests (transposes, alpha/beta, rank-3 batches, DEVICE storage).
#include <chrono>
#include <memory>
#include <random>
#include <vector>
#include <SushiBLAS/SushiBLAS.h>
#include "check.hpp"

static sr::Execution::RuntimeContext& runtime() { static sr::Execution::RuntimeContext ctx; return ctx; }

template <typename T = float>
static void fill_tensor(sb::Tensor& t, const std::vector<T>& data)
{
    SB_THROW_IF(static_cast<int64_t>(data.size()) != t.num_elements, "Data size mismatch. Vector: {}, Tensor: {}",
                data.size(), t.num_elements);
    std::copy(data.begin(), data.end(), t.data_as<T>());
}

template <typename T = float>
static void verify_tensor(const sb::Tensor& t, const std::vector<T>& expected, float abs_error = 1e-4f)
{
    EXPECT_EQ(static_cast<int64_t>(expected.size()), t.num_elements);
    const T* p = t.data_as<T>();
    for (size_t i = 0; i < expected.size(); ++i) EXPECT_NEAR(p[i], expected[i], abs_error);
}

// fp64 reference on host vectors (row-major)
static std::vector<float> host_gemm(bool ta, bool tb, int m, int n, int k, float alpha, const std::vector<float>& a,
                                    const std::vector<float>& b, float beta, const std::vector<float>& c)
{
    std::vector<float> out(size_t(m) * n);
    for (int i = 0; i < m; ++i)
        for (int j = 0; j < n; ++j)
        {
            double s = 0;
            for (int p = 0; p < k; ++p)
                s += double(ta ? a[size_t(p) * m + i] : a[size_t(i) * k + p]) * double(tb ? b[size_t(j) * k + p] : b[size_t(p) * n + j]);
            out[size_t(i) * n + j] = float(alpha * s + (beta != 0 ? beta * double(c[size_t(i) * n + j]) : 0.0));
        }
    return out;
}

static std::vector<float> random_vec(size_t n, unsigned seed)
{
    std::mt19937 g(seed);
    std::uniform_real_distribution<float> d(-1.0f, 1.0f);
    std::vector<float> v(n);
    for (auto& x : v) x = d(g);
    return v;
}

TEST_CASE(SimpleGEMM3x3)
{
    sb::Engine engine(runtime(), sb::Core::Layout::ROW_MAJOR);
    const int N = 3;
    auto A = engine.create_tensor({N, N});
    auto B = engine.create_tensor({N, N});
    auto C = engine.create_tensor({N, N});
    fill_tensor(A, {1, 2, 3, 4, 5, 6, 7, 8, 9});
    fill_tensor(B, {2, 0, 0, 0, 2, 0, 0, 0, 2});
    fill_tensor(C, std::vector<float>(N * N, 0.0f));
    engine.blas().gemm(A, B, C);
    engine.execute().wait();
    verify_tensor(C, {2, 4, 6, 8, 10, 12, 14, 16, 18});
}

TEST_CASE(SimpleGEMMColumnMajor)
{
    sb::Engine engine(runtime(), sb::Core::Layout::COLUMN_MAJOR);
    const int M = 2, N = 2, K = 2;
    auto A = engine.create_tensor({M, K});
    auto B = engine.create_tensor({K, N});
    auto C = engine.create_tensor({M, N});
    fill_tensor(A, {1, 3, 2, 4});
    fill_tensor(B, {5, 7, 6, 8});
    engine.blas().gemm(A, B, C);
    engine.execute().wait();
    verify_tensor(C, {19, 43, 22, 50});
}

TEST_CASE(TransposesAlphaBeta)
{
    sb::Engine engine(runtime());
    const int m = 37, n = 29, k = 53;
    for (int ta = 0; ta < 2; ++ta)
        for (int tb = 0; tb < 2; ++tb)
        {
            auto A = ta ? engine.create_tensor({k, m}) : engine.create_tensor({m, k});
            auto B = tb ? engine.create_tensor({n, k}) : engine.create_tensor({k, n});
            auto C = engine.create_tensor({m, n});
            auto a = random_vec(size_t(m) * k, 1 + ta), b = random_vec(size_t(k) * n, 3 + tb), c = random_vec(size_t(m) * n, 5);
            fill_tensor(A, a); fill_tensor(B, b); fill_tensor(C, c);
            engine.blas().gemm(A, B, C, ta, tb, 1.5f, 0.5f);
            engine.execute().wait();
            verify_tensor(C, host_gemm(ta, tb, m, n, k, 1.5f, a, b, 0.5f, c), 1e-4f);
        }
}

TEST_CASE(BetaZeroNeverReadsC)
{
    sb::Engine engine(runtime());
    auto A = engine.create_tensor({8, 8}), B = engine.create_tensor({8, 8}), C = engine.create_tensor({8, 8});
    auto a = random_vec(64, 7), b = random_vec(64, 8);
    fill_tensor(A, a); fill_tensor(B, b);
    fill_tensor(C, std::vector<float>(64, std::numeric_limits<float>::quiet_NaN()));
    engine.blas().gemm(A, B, C);
    engine.execute().wait();
    verify_tensor(C, host_gemm(false, false, 8, 8, 8, 1.0f, a, b, 0.0f, a));
}

TEST_CASE(BatchedRank3AndLargeTensorCorePath)
{
    sb::Engine engine(runtime());
    const int batch = 3, m = 320, n = 272, k = 200;      // large enough for the tcgen05 path, ragged tiles
    auto A = engine.create_tensor({batch, m, k}), B = engine.create_tensor({batch, k, n}), C = engine.create_tensor({batch, m, n});
    auto a = random_vec(size_t(batch) * m * k, 11), b = random_vec(size_t(batch) * k * n, 12);
    fill_tensor(A, a); fill_tensor(B, b);
    engine.blas().gemm(A, B, C);
    engine.execute().wait();
    for (int bi = 0; bi < batch; ++bi)
    {
        std::vector<float> ab(a.begin() + size_t(bi) * m * k, a.begin() + size_t(bi + 1) * m * k);
        std::vector<float> bb(b.begin() + size_t(bi) * k * n, b.begin() + size_t(bi + 1) * k * n);
        auto ref = host_gemm(false, false, m, n, k, 1.0f, ab, bb, 0.0f, ab);
        const float* got = C.data_as<float>() + size_t(bi) * m * n;
        for (size_t i = 0; i < ref.size(); ++i) EXPECT_NEAR(got[i], ref[i], 2e-4);
    }
}

TEST_CASE(DeviceStorageWithExplicitStaging)
{
    sb::Engine engine(runtime());
    const int m = 300, n = 260, k = 256;
    auto dev = sr::Memory::AllocStrategy::DEVICE;
    auto A = engine.create_tensor({m, k}, dev), B = engine.create_tensor({k, n}, dev), C = engine.create_tensor({m, n}, dev);
    EXPECT_TRUE(!A.storage->host_resident());
    auto a = random_vec(size_t(m) * k, 21), b = random_vec(size_t(k) * n, 22), c = random_vec(size_t(m) * n, 23);
    A.from_host(a.data()); B.from_host(b.data()); C.from_host(c.data());
    engine.blas().gemm(A, B, C, false, false, 2.0f, -1.0f);
    engine.execute().wait();
    std::vector<float> out(size_t(m) * n);
    C.to_host(out.data());
    auto ref = host_gemm(false, false, m, n, k, 2.0f, a, b, -1.0f, c);
    for (size_t i = 0; i < ref.size(); ++i) EXPECT_NEAR(out[i], ref[i], 3e-4);
    // slices of the leading dimension are views into the same storage
    auto top = C.slice(0, 0, 100);
    std::vector<float> part(size_t(100) * n);
    top.to_host(part.data());
    EXPECT_EQ(part[5], out[5]);
}

TEST_CASE(ChainedGemmsKeepOrder)
{
    // x <- x * W repeated: each GEMM reads what the previous one wrote
    // (shape of DeepForwardPass, tests/runtime/test_framework_sim.cpp:18-58, scaled down)
    sb::Engine engine(runtime());
    const int batch = 64, hidden = 128, layers = 6;
    auto x0 = engine.create_tensor({batch, hidden}), x1 = engine.create_tensor({batch, hidden});
    auto W = engine.create_tensor({hidden, hidden});
    auto w = random_vec(size_t(hidden) * hidden, 31);
    for (auto& v : w) v *= 0.1f;
    auto x = random_vec(size_t(batch) * hidden, 32);
    fill_tensor(W, w); fill_tensor(x0, x);
    sb::Tensor* cur = &x0; sb::Tensor* nxt = &x1;
    for (int l = 0; l < layers; ++l) { engine.blas().gemm(*cur, W, *nxt); std::swap(cur, nxt); }
    EXPECT_EQ(engine.get_graph().pending(), size_t(layers));
    engine.execute().wait();
    std::vector<float> ref = x;
    for (int l = 0; l < layers; ++l) ref = host_gemm(false, false, batch, hidden, hidden, 1.0f, ref, w, 0.0f, ref);
    verify_tensor(*cur, ref, 1e-4f);
}

TEST_CASE(SimpleSYRK)
{
    // tests/blas/level3/test_syrk.cpp:39-63
    sb::Engine engine(runtime());
    const int N = 3, K = 2;
    auto A = engine.create_tensor({N, K});
    auto C = engine.create_tensor({N, N});
    fill_tensor(A, {1, 2, 3, 4, 5, 6});
    fill_tensor(C, std::vector<float>(N * N, 0.0f));
    engine.blas().syrk(A, C, false, false, 1.0f, 0.0f);
    engine.execute().wait();
    verify_tensor(C, {5, 0, 0, 11, 25, 0, 17, 39, 61});
}

TEST_CASE(SimpleSYRKColumnMajor)
{
    // tests/blas/level3/test_syrk.cpp:65-88
    sb::Engine engine(runtime(), sb::Core::Layout::COLUMN_MAJOR);
    const int N = 2, K = 3;
    auto A = engine.create_tensor({K, N});
    auto C = engine.create_tensor({N, N});
    fill_tensor(A, {1, 2, 3, 4, 5, 6});
    fill_tensor(C, std::vector<float>(N * N, 0.0f));
    engine.blas().syrk(A, C, false, true, 1.0f, 0.0f);
    engine.execute().wait();
    verify_tensor(C, {14, 32, 0, 77});
}

TEST_CASE(SyrkLargeUpperKeepsTheOtherTriangle)
{
    sb::Engine engine(runtime());
    const int n = 520, k = 300;                       // tensor-core path, ragged tiles
    auto A = engine.create_tensor({n, k}), C = engine.create_tensor({n, n});
    auto a = random_vec(size_t(n) * k, 51), c = random_vec(size_t(n) * n, 52);
    fill_tensor(A, a); fill_tensor(C, c);
    engine.blas().syrk(A, C, true, false, 2.0f, 0.5f);
    engine.execute().wait();
    const float* got = C.data_as<float>();
    for (int i = 0; i < n; i += 3)
        for (int j = 0; j < n; j += 5)
        {
            if (j < i) { EXPECT_EQ(got[size_t(i) * n + j], c[size_t(i) * n + j]); continue; }
            double s = 0;
            for (int p = 0; p < k; ++p) s += double(a[size_t(i) * k + p]) * double(a[size_t(j) * k + p]);
            EXPECT_NEAR(got[size_t(i) * n + j], 2.0 * s + 0.5 * c[size_t(i) * n + j], 3e-4);
        }
    auto R = engine.create_tensor({4, 5});
    EXPECT_THROWS(engine.blas().syrk(A, R), "square matrix");
    auto S = engine.create_tensor({7, 7});
    EXPECT_THROWS(engine.blas().syrk(A, S), "does not match C");
}

TEST_CASE(Float64GEMM)
{
    // FLOAT64 branch of the front-end (src/ops/blas/level3/gemm.cpp:158-169); the 3 x 3 known answer of
    // tests/blas/level3/test_gemm.cpp:39-62 in double, then a product whose low bits only fp64 keeps
    sb::Engine engine(runtime());
    auto A = engine.create_tensor({3, 3}, sb::Core::DataType::FLOAT64);
    auto B = engine.create_tensor({3, 3}, sb::Core::DataType::FLOAT64);
    auto C = engine.create_tensor({3, 3}, sb::Core::DataType::FLOAT64);
    for (int i = 0; i < 9; ++i) { A.data_as<double>()[i] = i + 1; B.data_as<double>()[i] = (i % 4 == 0) ? 1.0 : 0.0; C.data_as<double>()[i] = 0.0; }
    engine.blas().gemm(A, B, C);
    engine.execute().wait();
    for (int i = 0; i < 9; ++i) EXPECT_EQ(C.data_as<double>()[i], double(i + 1));

    const int m = 150, n = 140, k = 130;
    auto X = engine.create_tensor({m, k}, sb::Core::DataType::FLOAT64, sr::Memory::AllocStrategy::DEVICE);
    auto Y = engine.create_tensor({n, k}, sb::Core::DataType::FLOAT64, sr::Memory::AllocStrategy::DEVICE);
    auto Z = engine.create_tensor({m, n}, sb::Core::DataType::FLOAT64, sr::Memory::AllocStrategy::DEVICE);
    std::vector<double> x(size_t(m) * k), y(size_t(n) * k), z(size_t(m) * n, 1.0);
    for (size_t i = 0; i < x.size(); ++i) x[i] = 1.0 + double(i % 977) * 1e-9;
    for (size_t i = 0; i < y.size(); ++i) y[i] = 1.0 - double(i % 991) * 1e-9;
    X.from_host(x.data()); Y.from_host(y.data()); Z.from_host(z.data());
    engine.blas().gemm(X, Y, Z, false, true, 2.0f, 0.5f);
    engine.execute().wait();
    Z.to_host(z.data());
    for (int i = 0; i < m; i += 7)
        for (int j = 0; j < n; j += 11)
        {
            long double s = 0;
            for (int p = 0; p < k; ++p) s += (long double)x[size_t(i) * k + p] * (long double)y[size_t(j) * k + p];
            EXPECT_NEAR(z[size_t(i) * n + j], double(2.0L * s + 0.5L), 1e-11);     // fp32 would be off by ~1e-5
        }
    auto F = engine.create_tensor({3, 3});
    EXPECT_THROWS(engine.blas().gemm(A, F, C), "Data type mismatch");
}

TEST_CASE(SimpleTRSM)
{
    // tests/blas/level3/test_trsm.cpp:39-77: lower triangular, left side
    sb::Engine engine(runtime());
    auto A = engine.create_tensor({2, 2});
    auto B = engine.create_tensor({2, 2});
    fill_tensor(A, {2, 0, 1, 2});
    fill_tensor(B, {4, 6, 4, 7});
    engine.blas().trsm(A, B, true, false, false, false, 1.0f);
    engine.execute().wait();
    verify_tensor(B, {2, 3, 1, 2});
}

TEST_CASE(SimpleTRSMColumnMajor)
{
    // tests/blas/level3/test_trsm.cpp:79-: upper triangular, column-major engine
    sb::Engine engine(runtime(), sb::Core::Layout::COLUMN_MAJOR);
    auto A = engine.create_tensor({2, 2});
    auto B = engine.create_tensor({2, 2});
    fill_tensor(A, {2, 0, 1, 2});
    fill_tensor(B, {4, 4, 6, 7});
    engine.blas().trsm(A, B, true, true, false, false, 1.0f);
    engine.execute().wait();
    verify_tensor(B, {1.0f, 2.0f, 1.25f, 3.5f});
}

TEST_CASE(TrsmBlockedRightSideRoundTrip)
{
    // X * A^T = alpha * B with A 300 x 300 upper (three diagonal blocks, the last one ragged):
    // multiply the solution back and compare with alpha * B
    sb::Engine engine(runtime());
    const int m = 70, n = 300;
    auto A = engine.create_tensor({n, n}), B = engine.create_tensor({m, n});
    auto a = random_vec(size_t(n) * n, 61), b = random_vec(size_t(m) * n, 62);
    for (int i = 0; i < n; ++i)
        for (int j = 0; j < n; ++j)
            a[size_t(i) * n + j] = (i == j) ? 4.0f + 0.01f * float(i % 7) : 0.05f * a[size_t(i) * n + j];
    fill_tensor(A, a); fill_tensor(B, b);
    engine.blas().trsm(A, B, false, true, true, false, 0.5f);
    engine.execute().wait();
    const float* x = B.data_as<float>();
    for (int i = 0; i < m; i += 3)
        for (int j = 0; j < n; j += 7)
        {
            // (X * A^T)(i, j) = sum_p X(i, p) * A(j, p) over the upper triangle p >= j
            double s = 0;
            for (int p = j; p < n; ++p) s += double(x[size_t(i) * n + p]) * double(a[size_t(j) * n + p]);
            EXPECT_NEAR(s, 0.5 * b[size_t(i) * n + j], 2e-5);
        }
    auto R = engine.create_tensor({4, 5});
    EXPECT_THROWS(engine.blas().trsm(R, B), "square");
    auto S = engine.create_tensor({7, 7});
    EXPECT_THROWS(engine.blas().trsm(S, B, true), "must match rows of B");
    EXPECT_THROWS(engine.blas().trsm(S, B, false), "must match cols of B");
}

TEST_CASE(ReLUForward)
{
    // tests/math/nonlinear/test_relu.cpp:38-47
    sb::Engine engine(runtime());
    auto t = engine.create_tensor({4});
    fill_tensor(t, {-2.0f, -0.5f, 0.0f, 3.5f});
    engine.nonlinear().relu(t);
    EXPECT_EQ(engine.get_graph().pending(), size_t(1));        // nothing to fold into: its own task
    engine.execute().wait();
    verify_tensor(t, {0.0f, 0.0f, 0.0f, 3.5f});
}

TEST_CASE(GemmReluChainIsFusedAndEqualsUnfused)
{
    // H_{i+1} = relu(H_i * W_i) as in DeepForwardPass (tests/runtime/test_framework_sim.cpp:47-58):
    // each relu is folded into the GEMM recorded just before it; results equal the unfused run bit for bit
    const int batch = 96, hidden = 160, layers = 4;
    auto w = random_vec(size_t(hidden) * hidden, 41);
    for (auto& v : w) v *= 0.2f;
    auto x = random_vec(size_t(batch) * hidden, 42);
    std::vector<float> results[2];
    for (int fused = 0; fused < 2; ++fused)
    {
        sb::Engine engine(runtime());
        engine.get_graph().set_fusion(fused == 1);
        auto W = engine.create_tensor({hidden, hidden});
        auto h0 = engine.create_tensor({batch, hidden}), h1 = engine.create_tensor({batch, hidden});
        fill_tensor(W, w); fill_tensor(h0, x);
        sb::Tensor* cur = &h0; sb::Tensor* nxt = &h1;
        for (int l = 0; l < layers; ++l)
        {
            engine.blas().gemm(*cur, W, *nxt);
            if (l < layers - 1) engine.nonlinear().relu(*nxt);
            std::swap(cur, nxt);
        }
        EXPECT_EQ(engine.get_graph().pending(), size_t(fused ? layers : 2 * layers - 1));
        EXPECT_EQ(engine.get_graph().fused_count(), size_t(fused ? layers - 1 : 0));
        engine.execute().wait();
        results[fused].assign(cur->data_as<float>(), cur->data_as<float>() + cur->num_elements);
    }
    EXPECT_TRUE(results[0] == results[1]);
    // and against the host reference
    std::vector<float> ref = x;
    for (int l = 0; l < layers; ++l)
    {
        ref = host_gemm(false, false, batch, hidden, hidden, 1.0f, ref, w, 0.0f, ref);
        if (l < layers - 1) for (auto& v : ref) v = v > 0 ? v : 0;
    }
    for (size_t i = 0; i < ref.size(); ++i) EXPECT_NEAR(results[1][i], ref[i], 2e-4);
    // a relu on a different tensor, or on a slice of the output, is not folded
    sb::Engine engine(runtime());
    auto A = engine.create_tensor({8, 8}), B = engine.create_tensor({8, 8}), C = engine.create_tensor({8, 8});
    fill_tensor(A, std::vector<float>(64, 1.0f)); fill_tensor(B, std::vector<float>(64, -1.0f));
    engine.blas().gemm(A, B, C);
    auto top = C.slice(0, 0, 4);
    engine.nonlinear().relu(top);
    EXPECT_EQ(engine.get_graph().pending(), size_t(2));
    engine.execute().wait();
    EXPECT_EQ(C.data_as<float>()[0], 0.0f);          // top half clamped
    EXPECT_EQ(C.data_as<float>()[63], -8.0f);        // bottom half untouched
}

TEST_CASE(FrameworkSimShapesAndStress)
{
    // DeepForwardPass: 10 x (512x1024 * 1024x1024); ParallelBatchedInference: 24 x (256x256 * 256x512);
    // dependency stress: 5000 reader GEMMs of 32x32 after one writer, then 3000 independent 8x8 GEMMs.
    // Like the reference, only shapes and a positive duration are asserted; timings are printed.
    sb::Engine engine(runtime());
    auto dev = sr::Memory::AllocStrategy::DEVICE;
    {
        std::vector<sb::Tensor> act, wts;
        for (int l = 0; l <= 10; ++l) act.push_back(engine.create_tensor({512, 1024}, dev));
        for (int l = 0; l < 10; ++l) wts.push_back(engine.create_tensor({1024, 1024}, dev));
        std::vector<float> ones(size_t(1024) * 1024, 0.001f);
        for (auto& w : wts) w.from_host(ones.data());
        act[0].from_host(ones.data());
        double ms = 0.0;
        for (int pass = 0; pass < 2; ++pass)       // the first pass also allocates the library's scratch
        {
            auto t0 = std::chrono::steady_clock::now();
            for (int l = 0; l < 10; ++l)
            {
                engine.blas().gemm(act[l], wts[l], act[l + 1]);
                if (l < 9) engine.nonlinear().relu(act[l + 1]);
            }
            EXPECT_EQ(engine.get_graph().pending(), size_t(10));          // the nine ReLUs were folded
            engine.execute().wait();
            ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
            std::printf("       DeepForwardPass 10 x (512x1024x1024), pass %d: %.3f ms\n", pass, ms);
        }
        EXPECT_EQ(act[10].shape[0], 512); EXPECT_EQ(act[10].shape[1], 1024); EXPECT_TRUE(ms > 0);
    }
    {
        auto src = engine.create_tensor({32, 32}, dev), w = engine.create_tensor({32, 32}, dev);
        std::vector<sb::Tensor> outs;
        for (int i = 0; i < 5000; ++i) outs.push_back(engine.create_tensor({32, 32}, dev));
        std::vector<float> v(1024, 0.5f);
        src.from_host(v.data()); w.from_host(v.data());
        for (int grouped = 1; grouped >= 0; --grouped)
        {
            engine.get_graph().set_grouping(grouped == 1);
            const size_t before = engine.get_graph().grouped_count();
            auto t0 = std::chrono::steady_clock::now();
            engine.blas().gemm(w, w, src);
            for (auto& o : outs) engine.blas().gemm(src, w, o);
            engine.execute().wait();
            double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
            std::printf("       1 writer + 5000 reader GEMMs (32^3), %s: %.3f ms\n",
                        grouped ? "grouped launch" : "one launch each", ms);
            // the writer stays alone (the readers depend on it); the 5000 readers form one group
            EXPECT_EQ(engine.get_graph().grouped_count() - before, size_t(grouped ? 5000 : 0));
            std::vector<float> got(1024);
            outs[4999].to_host(got.data());
            EXPECT_NEAR(got[0], 32 * (32 * 0.25f) * 0.5f, 1e-3);
            outs[17].to_host(got.data());
            EXPECT_NEAR(got[1023], 128.0f, 1e-3);
            EXPECT_TRUE(ms > 0);
        }
        engine.get_graph().set_grouping(true);
    }
    {
        // 3000 independent 8x8 GEMMs on SHARED tensors (tests/runtime/test_dependency_stress.cpp:67-83):
        // inputs are staged up, one grouped launch, outputs staged back
        std::vector<sb::Tensor> as, bs, cs;
        for (int i = 0; i < 3000; ++i)
        {
            as.push_back(engine.create_tensor({8, 8})); bs.push_back(engine.create_tensor({8, 8})); cs.push_back(engine.create_tensor({8, 8}));
            std::fill_n(as.back().data_as<float>(), 64, float(i % 7)); std::fill_n(bs.back().data_as<float>(), 64, 0.5f);
        }
        auto t0 = std::chrono::steady_clock::now();
        for (int i = 0; i < 3000; ++i) engine.blas().gemm(as[i], bs[i], cs[i]);
        engine.execute().wait();
        double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        std::printf("       3000 independent GEMMs (8^3, SHARED tensors): %.3f ms\n", ms);
        for (int i : {0, 1, 6, 2999}) EXPECT_NEAR(cs[i].data_as<float>()[63], 8 * float(i % 7) * 0.5f, 1e-4);
    }
    {
        // dependent small GEMMs must not be grouped together: C1 = A*B, C2 = C1*B, C3 = C2*B
        auto A = engine.create_tensor({16, 16}), B = engine.create_tensor({16, 16});
        auto C1 = engine.create_tensor({16, 16}), C2 = engine.create_tensor({16, 16}), C3 = engine.create_tensor({16, 16});
        std::fill_n(A.data_as<float>(), 256, 1.0f); std::fill_n(B.data_as<float>(), 256, 0.25f);
        engine.blas().gemm(A, B, C1); engine.blas().gemm(C1, B, C2); engine.blas().gemm(C2, B, C3);
        const size_t before = engine.get_graph().grouped_count();
        engine.execute().wait();
        EXPECT_EQ(engine.get_graph().grouped_count(), before);
        EXPECT_NEAR(C3.data_as<float>()[100], 64.0f, 1e-4);      // (16*0.25)^3
    }
}

TEST_CASE(DeepForwardPassOnDefaultTensorsCrossesPcieOncePerTensor)
{
    // tests/runtime/test_framework_sim.cpp:18-72 exactly as the reference writes it: default (SHARED) tensors
    // filled through data_as<T>() (tests/test_common.hpp:36-46), ten GEMM + ReLU layers, one execute().wait().
    // Residency: X and every weight go up once, no activation crosses PCIe between layers, every written
    // activation comes down once, at the wait.
    sb::Engine engine(runtime());
    sushi_cuda_ctx* native = runtime().native_handle();
    const int batch = 512, features = 1024, layers = 10;
    auto X = engine.create_tensor({batch, features});
    fill_tensor(X, std::vector<float>(size_t(batch) * features, 1.0f));
    std::vector<sb::Tensor> weights, activations;
    activations.push_back(X);
    for (int i = 0; i < layers; ++i)
    {
        auto W = engine.create_tensor({features, features});
        fill_tensor(W, std::vector<float>(size_t(features) * features, 0.01f));
        weights.push_back(W);
        activations.push_back(engine.create_tensor({batch, features}));
    }
    const uint64_t act_bytes = uint64_t(batch) * features * 4, w_bytes = uint64_t(features) * features * 4;
    double ms = 0.0;
    for (int pass = 0; pass < 2; ++pass)          // the first pass also allocates mirrors and the library's scratch
    {
        uint64_t up0 = 0, down0 = 0, up1 = 0, down1 = 0;
        EXPECT_EQ(sushi_cuda_copy_bytes(native, &up0, &down0), SUSHI_CUDA_OK);
        auto t0 = std::chrono::steady_clock::now();
        for (int i = 0; i < layers; ++i)
        {
            engine.blas().gemm(activations[i], weights[i], activations[i + 1]);
            if (i < layers - 1) engine.nonlinear().relu(activations[i + 1]);
        }
        engine.execute().wait();
        ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
        EXPECT_EQ(sushi_cuda_copy_bytes(native, &up1, &down1), SUSHI_CUDA_OK);
        std::printf("       DeepForwardPass 10 x (512x1024x1024) on SHARED tensors, pass %d: %.3f ms, %.1f MB up, %.1f MB down\n",
                    pass, ms, double(up1 - up0) / 1e6, double(down1 - down0) / 1e6);
        EXPECT_EQ(up1 - up0, act_bytes + layers * w_bytes);          // X and the ten weights, once each
        EXPECT_EQ(down1 - down0, layers * act_bytes);                // H1 .. H10, once each, at the wait
    }
    // all ones times 0.01: H_l = 1024 * 0.01 * H_{l-1} = 10.24^l (ReLU changes nothing)
    double want = 1.0;
    for (int l = 1; l <= layers; ++l)
    {
        want *= 10.24;
        EXPECT_NEAR(activations[l].data_as<float>()[12345] / want, 1.0, 1e-4);
    }
    EXPECT_TRUE(ms > 0);

    // a second round reads what the first left on the device: H11 = H10 * W0 sends W0 up again (the host may
    // have rewritten it since the wait) but not H10, unless the host touches it -- a host write is picked up
    auto H11 = engine.create_tensor({batch, features});
    uint64_t up0 = 0, up1 = 0;
    sushi_cuda_copy_bytes(native, &up0, nullptr);
    engine.blas().gemm(activations[layers], weights[0], H11);
    engine.execute().wait();
    sushi_cuda_copy_bytes(native, &up1, nullptr);
    EXPECT_EQ(up1 - up0, act_bytes + w_bytes);                       // host-valid images are re-sent once per round
    EXPECT_NEAR(H11.data_as<float>()[777] / (want * 10.24), 1.0, 1e-4);
    std::fill_n(activations[layers].data_as<float>(), size_t(batch) * features, 2.0f);
    engine.blas().gemm(activations[layers], weights[0], H11);
    engine.execute().wait();
    EXPECT_NEAR(H11.data_as<float>()[777], 2.0f * 10.24f, 1e-3);

    // two rounds without a wait in between: the second reads the first's output from the device
    auto P = engine.create_tensor({64, 64}), Q = engine.create_tensor({64, 64}), R = engine.create_tensor({64, 64});
    auto S = engine.create_tensor({64, 64});
    std::fill_n(P.data_as<float>(), 4096, 1.0f); std::fill_n(Q.data_as<float>(), 4096, 0.5f);
    engine.blas().gemm(P, Q, R);
    engine.execute();
    engine.blas().gemm(R, Q, S);
    engine.execute().wait();
    EXPECT_NEAR(R.data_as<float>()[100], 32.0f, 1e-4);
    EXPECT_NEAR(S.data_as<float>()[100], 32.0f * 32.0f, 1e-3);

    // an operation that writes a slice keeps the rest of the storage: the whole image goes up first
    auto C = engine.create_tensor({8, 8}), A = engine.create_tensor({4, 8}), B = engine.create_tensor({8, 8});
    std::fill_n(C.data_as<float>(), 64, 7.0f); std::fill_n(A.data_as<float>(), 32, 1.0f); std::fill_n(B.data_as<float>(), 64, 1.0f);
    auto top = C.slice(0, 0, 4);
    engine.blas().gemm(A, B, top);
    engine.execute().wait();
    EXPECT_EQ(C.data_as<float>()[0], 8.0f);
    EXPECT_EQ(C.data_as<float>()[63], 7.0f);
}

TEST_CASE(ExampleFlowWithWaitAll)
{
    // examples/example.cpp:34-56: column-major engine, 1024^2 tensors, execute() then ctx.wait_all()
    sb::Engine sbe(runtime(), sb::Core::Layout::COLUMN_MAJOR);
    auto A = sbe.create_tensor({1024, 1024}, sr::Memory::AllocStrategy::SHARED);
    auto B = sbe.create_tensor({1024, 1024}, sr::Memory::AllocStrategy::SHARED);
    auto C = sbe.create_tensor({1024, 1024}, sr::Memory::AllocStrategy::SHARED);
    std::fill_n(A.data_as<float>(), A.num_elements, 1.0f);
    std::fill_n(B.data_as<float>(), B.num_elements, 0.5f);
    sbe.blas().gemm(A, B, C);
    sbe.execute();
    runtime().wait_all();
    EXPECT_NEAR(C.data_as<float>()[12345], 512.0f, 1e-3);
}

TEST_CASE(ActivationFamilyKnownAnswers)
{
    // Forward / Backward of tests/math/nonlinear/test_{leaky_relu,sigmoid,tanh,elu,silu,gelu,softplus}.cpp
    sb::Engine engine(runtime());
    auto t = engine.create_tensor({4});
    auto dy = engine.create_tensor({4}), x = engine.create_tensor({4}), dx = engine.create_tensor({4});
    auto fwd = [&](std::vector<float> in, std::vector<float> want, auto&& op) {
        fill_tensor(t, in); op(); engine.execute().wait(); verify_tensor(t, want);
    };
    auto bwd = [&](std::vector<float> g, std::vector<float> saved, std::vector<float> want, auto&& op) {
        fill_tensor(dy, g); fill_tensor(x, saved); fill_tensor(dx, {0, 0, 0, 0}); op(); engine.execute().wait(); verify_tensor(dx, want);
    };
    fwd({-2.0f, -0.5f, 0.0f, 3.5f}, {-0.02f, -0.005f, 0.0f, 3.5f}, [&] { engine.nonlinear().leaky_relu(t, 0.01f); });
    fwd({0.0f, 1.0f, -1.0f, 2.0f}, {0.5f, 0.731058f, 0.268941f, 0.880797f}, [&] { engine.nonlinear().sigmoid(t); });
    fwd({0.0f, 1.0f, -1.0f, 2.0f}, {0.0f, 0.761594f, -0.761594f, 0.964028f}, [&] { engine.nonlinear().tanh(t); });
    fwd({-1.0f, 0.0f, 1.0f, 2.0f}, {-0.632121f, 0.0f, 1.0f, 2.0f}, [&] { engine.nonlinear().elu(t, 1.0f); });
    fwd({-1.0f, 0.0f, 1.0f, 2.0f}, {-0.268941f, 0.0f, 0.731059f, 1.761594f}, [&] { engine.nonlinear().silu(t); });
    fwd({-1.0f, 0.0f, 1.0f, 2.0f}, {-0.158865f, 0.0f, 0.841135f, 1.954598f}, [&] { engine.nonlinear().gelu(t); });
    fwd({-1.0f, 0.0f, 1.0f, 2.0f}, {0.313262f, 0.693147f, 1.313262f, 2.126928f}, [&] { engine.nonlinear().softplus(t); });
    bwd({1, 2, 3, 4}, {-1.0f, 0.0f, 1.0f, 2.0f}, {0.0f, 0.0f, 3.0f, 4.0f}, [&] { engine.nonlinear().relu_backward(dy, x, dx); });
    bwd({1, 2, 3, 4}, {-1.0f, -0.5f, 1.0f, 2.0f}, {0.01f, 0.02f, 3.0f, 4.0f}, [&] { engine.nonlinear().leaky_relu_backward(dy, x, dx, 0.01f); });
    bwd({1, 1, 1, 1}, {0.5f, 0.731058f, 0.268941f, 0.880797f}, {0.25f, 0.196612f, 0.196612f, 0.104994f},
        [&] { engine.nonlinear().sigmoid_backward(dy, x, dx); });
    bwd({1, 1, 1, 1}, {0.0f, 0.761594f, -0.761594f, 0.964028f}, {1.0f, 0.419974f, 0.419974f, 0.070651f},
        [&] { engine.nonlinear().tanh_backward(dy, x, dx); });
    bwd({1, 1, 1, 1}, {-1.0f, 0.0f, 1.0f, 2.0f}, {0.367879f, 1.0f, 1.0f, 1.0f}, [&] { engine.nonlinear().elu_backward(dy, x, dx, 1.0f); });
    bwd({1, 1, 1, 1}, {-1.0f, 0.0f, 1.0f, 2.0f}, {0.072329f, 0.5f, 0.927671f, 1.090784f}, [&] { engine.nonlinear().silu_backward(dy, x, dx); });
    bwd({1, 1, 1, 1}, {-1.0f, 0.0f, 1.0f, 2.0f}, {-0.082937f, 0.5f, 1.082937f, 1.086099f}, [&] { engine.nonlinear().gelu_backward(dy, x, dx); });
    bwd({1, 1, 1, 1}, {-1.0f, 0.0f, 1.0f, 2.0f}, {0.268941f, 0.5f, 0.731059f, 0.880797f}, [&] { engine.nonlinear().softplus_backward(dy, x, dx); });

    // an activation recorded right after the GEMM that wrote the tensor is folded into the GEMM's epilogue
    auto A = engine.create_tensor({64, 48}), B = engine.create_tensor({48, 40}), C = engine.create_tensor({64, 40});
    auto a = random_vec(64 * 48, 71), b = random_vec(48 * 40, 72);
    fill_tensor(A, a); fill_tensor(B, b);
    engine.blas().gemm(A, B, C);
    engine.nonlinear().sigmoid(C);
    EXPECT_EQ(engine.get_graph().pending(), size_t(1));
    engine.execute().wait();
    auto ref = host_gemm(false, false, 64, 40, 48, 1.0f, a, b, 0.0f, a);
    for (size_t i = 0; i < ref.size(); ++i) EXPECT_NEAR(C.data_as<float>()[i], 1.0 / (1.0 + std::exp(-double(ref[i]))), 2e-5);
    auto D64 = engine.create_tensor({4}, sb::Core::DataType::FLOAT64);
    EXPECT_THROWS(engine.nonlinear().gelu(D64), "FLOAT32 only");
}

TEST_CASE(ErrorsAreRuntimeErrors)
{
    sb::Engine engine(runtime());
    auto A = engine.create_tensor({4, 4}), B = engine.create_tensor({4, 4});
    auto D = engine.create_tensor({4, 4}, sb::Core::DataType::FLOAT64);
    auto v = engine.create_tensor({4});
    sb::Tensor none;
    EXPECT_THROWS(engine.blas().gemm(v, B, A), "at least 2D");
    EXPECT_THROWS(engine.blas().gemm(A, B, D), "Data type mismatch");
    auto Z = engine.create_tensor({4, 4}, sb::Core::DataType::COMPLEX32);
    EXPECT_THROWS(engine.blas().gemm(Z, Z, Z), "serves FLOAT32 and FLOAT64");
    auto big = engine.create_tensor({64, 64});
    auto small = engine.create_tensor({2, 2});
    EXPECT_THROWS(engine.blas().gemm(small, B, big), "does not fit its storage");
    EXPECT_EQ(engine.get_graph().pending(), size_t(0));
}

int main() { return check::run_all(); }
