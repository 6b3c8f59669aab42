// File IO of the C++ API against numpy (reference: src/io.cpp:111-240; the reference has no IO
// test of its own).  Run as `test_io_npy <directory>`: the directory may hold files written by
// numpy.save (in_rowmajor.npy: float32 (6, 10) row-major = arange(60); in_fortran.npy: the same
// values as a Fortran-ordered (6, 10) array); this program loads them into DEVICE and SHARED
// tensors, writes them back (echo_*.npy, which must be byte-identical to numpy's files), saves
// the result of a GEMM on DEVICE tensors (gemm_c.npy) and a rank-1 tensor (vec.npy), and checks
// the loader's error paths.
#include <cstdio>
#include <fstream>
#include <numeric>
#include <string>
#include <vector>
#include <SushiBLAS/SushiBLAS.h>
#include "check.hpp"

namespace {
std::string g_dir;
sr::Execution::RuntimeContext& runtime() { static sr::Execution::RuntimeContext ctx; return ctx; }
bool exists(const std::string& p) { std::ifstream f(p, std::ios::binary); return f.good(); }
constexpr auto DEVICE = sr::Memory::AllocStrategy::DEVICE;
}

TEST_CASE(LoadNumpyFilesAndEchoThem)
{
    if (!exists(g_dir + "/in_rowmajor.npy")) { std::printf("  (no numpy input files: skipped)\n"); return; }
    sb::Engine engine(runtime());
    auto D = engine.create_tensor({6, 10}, DEVICE);
    engine.io().load_npy(D, g_dir + "/in_rowmajor.npy");
    std::vector<float> host(60);
    D.to_host(host.data());
    for (int i = 0; i < 60; ++i) EXPECT_EQ(host[i], float(i));
    engine.io().save_npy(D, g_dir + "/echo_rowmajor.npy");

    sb::Engine col(runtime(), sb::Core::Layout::COLUMN_MAJOR);
    auto F = col.create_tensor({6, 10});                       // SHARED, column-major
    col.io().load_npy(F, g_dir + "/in_fortran.npy");
    // element (i, j) = 10 i + j, stored first index fastest
    for (int j = 0; j < 10; ++j)
        for (int i = 0; i < 6; ++i) EXPECT_EQ(F.data_as<float>()[j * 6 + i], float(10 * i + j));
    col.io().save_npy(F, g_dir + "/echo_fortran.npy");

    // mismatches the loader must refuse
    auto wrong_shape = engine.create_tensor({10, 6});
    EXPECT_THROWS(engine.io().load_npy(wrong_shape, g_dir + "/in_rowmajor.npy"), "Shape dimension 0 mismatch");
    auto wrong_rank = engine.create_tensor({60});
    EXPECT_THROWS(engine.io().load_npy(wrong_rank, g_dir + "/in_rowmajor.npy"), "Rank mismatch");
    auto wrong_type = engine.create_tensor({6, 10}, sb::Core::DataType::FLOAT64);
    EXPECT_THROWS(engine.io().load_npy(wrong_type, g_dir + "/in_rowmajor.npy"), "Data type mismatch");
    auto wrong_order = engine.create_tensor({6, 10});
    EXPECT_THROWS(engine.io().load_npy(wrong_order, g_dir + "/in_fortran.npy"), "Memory order mismatch");
    EXPECT_THROWS(engine.io().load_npy(D, g_dir + "/does_not_exist.npy"), "Failed to open file for reading");
}

TEST_CASE(SaveFlushesPendingWorkAndStagesDeviceTensors)
{
    sb::Engine engine(runtime());
    const int M = 5, K = 7, N = 3;
    auto A = engine.create_tensor({M, K}, DEVICE), B = engine.create_tensor({K, N}, DEVICE), C = engine.create_tensor({M, N}, DEVICE);
    std::vector<float> a(M * K), b(K * N);
    std::iota(a.begin(), a.end(), 1.0f);
    for (int i = 0; i < K * N; ++i) b[i] = float(i % 4) - 1.0f;
    A.from_host(a.data()); B.from_host(b.data());
    engine.blas().gemm(A, B, C);
    EXPECT_EQ(engine.get_graph().pending(), size_t(1));
    engine.io().save_npy(C, g_dir + "/gemm_c.npy");            // runs the GEMM first (src/io.cpp:138)
    EXPECT_EQ(engine.get_graph().pending(), size_t(0));
    engine.io().save_npy(A, g_dir + "/gemm_a.npy");
    engine.io().save_npy(B, g_dir + "/gemm_b.npy");

    auto v = engine.create_tensor({4});
    for (int i = 0; i < 4; ++i) v.data_as<float>()[i] = 0.5f * float(i);
    engine.io().save_npy(v, g_dir + "/vec.npy");

    // raw bytes round trip through a DEVICE tensor
    engine.io().save_bin(C, g_dir + "/gemm_c.bin");
    auto C2 = engine.create_tensor({M, N}, DEVICE);
    engine.io().load_bin(C2, g_dir + "/gemm_c.bin");
    std::vector<float> c(M * N), c2(M * N);
    C.to_host(c.data()); C2.to_host(c2.data());
    EXPECT_TRUE(c == c2);
    // and the .npy round trip
    auto C3 = engine.create_tensor({M, N});
    engine.io().load_npy(C3, g_dir + "/gemm_c.npy");
    for (int i = 0; i < M * N; ++i) EXPECT_EQ(C3.data_as<float>()[i], c[i]);

    // not an .npy file
    EXPECT_THROWS(engine.io().load_npy(C3, g_dir + "/gemm_c.bin"), "Invalid .npy file magic");
    // truncated payload
    {
        std::ifstream in(g_dir + "/gemm_c.npy", std::ios::binary);
        std::vector<char> bytes((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
        std::ofstream out(g_dir + "/short.npy", std::ios::binary);
        out.write(bytes.data(), std::streamsize(bytes.size() - 8));
    }
    EXPECT_THROWS(engine.io().load_npy(C3, g_dir + "/short.npy"), "shorter than the tensor");
}

int main(int argc, char** argv)
{
    g_dir = argc > 1 ? argv[1] : ".";
    return check::run_all();
}
