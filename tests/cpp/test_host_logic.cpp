// Host-side logic of the C++ API, no GPU needed: Tensor metadata and views
// (reference include/SushiBLAS/tensor.hpp:92-300), Storage rounding (storage.hpp:78-95),
// GEMM parameter derivation and validation (src/ops/blas/level3/gemm.cpp:87-105), task
// metadata (task_types.hpp:35-129), the smart pointer, and the loud failure of
// RuntimeContext without a device.
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iterator>
#include <vector>
#include <unistd.h>
#include <SushiBLAS/SushiBLAS.h>
#include "check.hpp"

namespace {
// host-only allocator for tests: plain malloc, everything host-resident, no device view
struct MallocAllocator final : sr::Memory::USMAllocator
{
    int live = 0;
    std::size_t last_bytes = 0;
    void* allocate(std::size_t bytes, sr::Memory::AllocStrategy, std::size_t) override
    { ++live; last_bytes = bytes; return std::aligned_alloc(128, bytes); }
    void deallocate(void* p) override { --live; std::free(p); }
    bool is_host_resident(void*) override { return true; }
    void* device_view(void*) override { return nullptr; }
};

sb::Tensor make(sr::sushi_ptr<MallocAllocator> al, std::initializer_list<int64_t> dims,
                sb::Core::Layout l = sb::Core::Layout::ROW_MAJOR)
{
    std::size_t n = 1; for (auto d : dims) n *= d;
    auto st = sr::make_sushi<sb::Storage>(al, n * 4);
    return sb::Tensor(st, dims, 0, l);
}
}

TEST_CASE(storage_rounds_to_128_and_frees)
{
    auto al = sr::make_sushi<MallocAllocator>();
    {
        auto st = sr::make_sushi<sb::Storage>(al, 36);       // 3x3 floats
        EXPECT_EQ(st->requested_bytes, 36u);
        EXPECT_EQ(st->size_bytes, 128u);
        EXPECT_EQ(al->last_bytes, 128u);
        EXPECT_EQ(al->live, 1);
        auto copy = st;
        EXPECT_EQ(st->ref_count(), 2u);
    }
    EXPECT_EQ(al->live, 0);
    EXPECT_THROWS(sr::make_sushi<sb::Storage>(al, 0), "cannot be zero");
    EXPECT_THROWS(sr::make_sushi<sb::Storage>(sr::sushi_ptr<MallocAllocator>(), 16), "cannot be null");
}

TEST_CASE(tensor_strides_row_and_column_major)
{
    auto al = sr::make_sushi<MallocAllocator>();
    auto t = make(al, {4, 5, 6});
    EXPECT_EQ(t.rank, 3); EXPECT_EQ(t.num_elements, 120);
    EXPECT_EQ(t.strides[0], 30); EXPECT_EQ(t.strides[1], 6); EXPECT_EQ(t.strides[2], 1);
    auto c = make(al, {4, 5, 6}, sb::Core::Layout::COLUMN_MAJOR);
    EXPECT_EQ(c.strides[0], 1); EXPECT_EQ(c.strides[1], 4); EXPECT_EQ(c.strides[2], 20);
    EXPECT_TRUE(t.is_contiguous() && c.is_contiguous() && t.is_aligned());
    EXPECT_THROWS(make(al, {1, 1, 1, 1, 1, 1, 1}), "exceeds limit");
    // capacity check
    auto st = sr::make_sushi<sb::Storage>(al, 64);
    EXPECT_THROWS(sb::Tensor(st, {8, 8}), "capacity exceeded");
    EXPECT_THROWS(sb::Tensor(st, {2, 2}, -1), "negative");
    sb::Tensor empty;
    EXPECT_THROWS(empty.data(), "no storage");
}

TEST_CASE(tensor_views)
{
    auto al = sr::make_sushi<MallocAllocator>();
    auto t = make(al, {4, 6});
    float* p = t.data_as<float>();
    for (int i = 0; i < 24; ++i) p[i] = float(i);
    auto tr = t.transpose(0, 1);
    EXPECT_EQ(tr.shape[0], 6); EXPECT_EQ(tr.strides[0], 1); EXPECT_EQ(tr.strides[1], 6);
    EXPECT_TRUE(!tr.is_contiguous());
    EXPECT_THROWS(t.transpose(0, 2), "Invalid dimensions");
    auto r = t.reshape({2, 12});
    EXPECT_EQ(r.strides[0], 12); EXPECT_EQ(r.data(), t.data());
    EXPECT_THROWS(t.reshape({5, 5}), "Element count mismatch");
    EXPECT_THROWS(tr.reshape({24}), "must be contiguous");
    auto s = t.slice(0, 1, 3);                    // rows 1..2
    EXPECT_EQ(s.shape[0], 2); EXPECT_EQ(s.storage_offset, 6); EXPECT_EQ(s.data_as<float>()[0], 6.0f);
    auto neg = t.slice(0, -1, 100);               // last row, end clamped
    EXPECT_EQ(neg.shape[0], 1); EXPECT_EQ(neg.storage_offset, 18);
    EXPECT_THROWS(t.slice(2, 0, 1), "Invalid dimension");
    // host staging helpers on a host-resident tensor are plain copies
    std::vector<float> out(24);
    t.to_host(out.data());
    EXPECT_EQ(out[23], 23.0f);
}

TEST_CASE(gemm_parameter_derivation)
{
    auto al = sr::make_sushi<MallocAllocator>();
    auto A = make(al, {256, 512, 512}), B = make(al, {256, 512, 512}), C = make(al, {256, 512, 512});
    auto g = sb::detail::derive_gemm_call(A, B, C, false, false, 1.0f, 0.0f);
    EXPECT_EQ(g.m, 512); EXPECT_EQ(g.n, 512); EXPECT_EQ(g.k, 512); EXPECT_EQ(g.batch, 256);
    EXPECT_EQ(g.lda, 512); EXPECT_EQ(g.stride_a, 262144); EXPECT_EQ(g.stride_c, 262144);
    // k comes from A's second-to-last dim under transA
    auto At = make(al, {7, 3}), B2 = make(al, {7, 5}), C2 = make(al, {3, 5});
    g = sb::detail::derive_gemm_call(At, B2, C2, true, false, 2.0f, 0.5f);
    EXPECT_EQ(g.m, 3); EXPECT_EQ(g.n, 5); EXPECT_EQ(g.k, 7); EXPECT_EQ(g.lda, 3); EXPECT_EQ(g.batch, 1);
    EXPECT_EQ(g.stride_a, 0);
    // rank-4 batch = product of leading dims
    auto A4 = make(al, {2, 3, 8, 4}), B4 = make(al, {2, 3, 4, 6}), C4 = make(al, {2, 3, 8, 6});
    g = sb::detail::derive_gemm_call(A4, B4, C4, false, false, 1.0f, 0.0f);
    EXPECT_EQ(g.batch, 6); EXPECT_EQ(g.stride_a, 32); EXPECT_EQ(g.stride_b, 24); EXPECT_EQ(g.stride_c, 48);
    // validation
    auto v = make(al, {4});
    EXPECT_THROWS(sb::detail::derive_gemm_call(v, B2, C2, false, false, 1, 0), "at least 2D");
    auto D = make(al, {3, 5}); D.dtype = sb::Core::DataType::FLOAT64;
    EXPECT_THROWS(sb::detail::derive_gemm_call(At, B2, D, true, false, 1, 0), "Data type mismatch");
    EXPECT_THROWS(sb::detail::derive_gemm_call(At, B2, C, true, false, 1, 0), "rank >= 3");
}

TEST_CASE(column_major_maps_to_swapped_row_major)
{
    auto al = sr::make_sushi<MallocAllocator>();
    auto L = sb::Core::Layout::COLUMN_MAJOR;
    auto A = make(al, {5, 7}, L), B = make(al, {7, 3}, L), C = make(al, {5, 3}, L);
    auto g = sb::detail::derive_gemm_call(A, B, C, false, false, 1.0f, 0.0f);
    EXPECT_EQ(g.lda, 5); EXPECT_EQ(g.ldb, 7); EXPECT_EQ(g.ldc, 5); EXPECT_EQ(g.k, 7);
    bool swapped = false;
    auto r = sb::detail::row_major_equivalent(g, &swapped);
    EXPECT_TRUE(swapped);
    EXPECT_EQ(r.m, 3); EXPECT_EQ(r.n, 5); EXPECT_EQ(r.k, 7); EXPECT_EQ(r.lda, 7); EXPECT_EQ(r.ldb, 5); EXPECT_EQ(r.ldc, 5);
    auto rm = sb::detail::row_major_equivalent(sb::detail::derive_gemm_call(make(al, {5, 7}), make(al, {7, 3}),
                                                                            C = make(al, {5, 3}), false, true, 1, 0), &swapped);
    EXPECT_TRUE(!swapped && rm.trans_b);
    EXPECT_EQ(sb::detail::operand_extent(4, 3, 5, 100, 3), 2 * 100 + 3 * 5 + 3);
    EXPECT_EQ(sb::detail::operand_extent(0, 3, 5, 100, 3), 0);
}

TEST_CASE(task_metadata_and_op_id)
{
    using namespace sr::Graph::Literals;
    constexpr auto id = "blas.lvl3.gemm"_op;
    // FNV-1a 32-bit of the operation name
    std::uint32_t h = 2166136261u;
    for (const char* s = "blas.lvl3.gemm"; *s; ++s) { h ^= std::uint8_t(*s); h *= 16777619u; }
    EXPECT_EQ(id.value, h);
    EXPECT_TRUE("a"_op != "b"_op);
    sr::Graph::TaskMetadata m;
    m.set_param(0, 1.5f); m.set_param(2, true); m.set_param(9, 3);       // out-of-range index ignored
    EXPECT_EQ(m.get_param<float>(0), 1.5f); EXPECT_EQ(m.get_param<bool>(2), true); EXPECT_EQ(m.get_param<int>(9), 0);
}

TEST_CASE(npy_header_is_what_numpy_writes_and_parses_back)
{
    // src/io.cpp:149-169; the expected strings are the headers numpy.save writes for these arrays
    // numpy pads each of these dictionaries with spaces to 117 characters and closes it with '\n'
    auto numpy_header = [](const std::string& text) { return text + std::string(117 - text.size(), ' ') + "\n"; };
    int64_t s2[] = {3, 4};
    EXPECT_EQ(sb::detail::npy_header_dict(sb::Core::DataType::FLOAT32, sb::Core::Layout::ROW_MAJOR, s2, 2),
              numpy_header("{'descr': '<f4', 'fortran_order': False, 'shape': (3, 4), }"));
    int64_t s1[] = {5};
    EXPECT_EQ(sb::detail::npy_header_dict(sb::Core::DataType::FLOAT32, sb::Core::Layout::ROW_MAJOR, s1, 1),
              numpy_header("{'descr': '<f4', 'fortran_order': False, 'shape': (5,), }"));
    int64_t s3[] = {2, 3, 4};
    EXPECT_EQ(sb::detail::npy_header_dict(sb::Core::DataType::FLOAT64, sb::Core::Layout::COLUMN_MAJOR, s3, 3),
              numpy_header("{'descr': '<f8', 'fortran_order': True, 'shape': (2, 3, 4), }"));
    int64_t s4[] = {1024, 1024, 7};
    const std::string h4 = sb::detail::npy_header_dict(sb::Core::DataType::FLOAT32, sb::Core::Layout::ROW_MAJOR, s4, 3);
    EXPECT_EQ(h4, numpy_header("{'descr': '<f4', 'fortran_order': False, 'shape': (1024, 1024, 7), }"));
    EXPECT_EQ((10 + h4.size()) % 64, 0u);

    auto info = sb::detail::parse_npy_header(h4);
    EXPECT_EQ(info.descr, std::string("<f4"));
    EXPECT_TRUE(!info.fortran_order);
    EXPECT_EQ(info.shape.size(), 3u);
    EXPECT_EQ(info.shape[0], 1024); EXPECT_EQ(info.shape[1], 1024); EXPECT_EQ(info.shape[2], 7);
    // key order and spacing are free in the format; () is a scalar, (5,) one dimension
    info = sb::detail::parse_npy_header("{'shape': (5,), 'fortran_order': True, 'descr': '|f4'}");
    EXPECT_EQ(info.descr, std::string("|f4"));
    EXPECT_TRUE(info.fortran_order);
    EXPECT_EQ(info.shape.size(), 1u);
    EXPECT_EQ(sb::detail::parse_npy_header("{'descr': '<f8', 'fortran_order': False, 'shape': (), }").shape.size(), 0u);
    EXPECT_THROWS(sb::detail::parse_npy_header("{'descr': '<f4', 'shape': (3,)}"), "fortran_order");
    EXPECT_THROWS(sb::detail::parse_npy_header("{'descr': '<f4', 'fortran_order': 0, 'shape': (3,)}"), "neither True nor False");
    EXPECT_THROWS(sb::detail::parse_npy_header("{'descr': '<f4', 'fortran_order': False, 'shape': (3, x)}"), "bad character");
    EXPECT_THROWS(sb::detail::parse_npy_header("{'descr': '<f4', 'fortran_order': False, 'shape': (3, 4"), "unterminated shape");
}

TEST_CASE(npy_files_round_trip_on_the_host)
{
    // the file routines behind IO::save_npy / load_npy with host-resident tensors: no device involved
    const char* dir = std::getenv("SUSHI_TEST_TMPDIR");
    const std::string base = std::string(dir ? dir : "/tmp") + "/host_logic_";
    auto al = sr::make_sushi<MallocAllocator>();
    auto t = make(al, {3, 5});
    for (int i = 0; i < 15; ++i) t.data_as<float>()[i] = 0.25f * float(i) - 1.0f;
    sb::detail::save_npy_file(t, base + "rowmajor.npy");
    auto back = make(al, {3, 5});
    sb::detail::load_npy_file(back, base + "rowmajor.npy");
    for (int i = 0; i < 15; ++i) EXPECT_EQ(back.data_as<float>()[i], t.data_as<float>()[i]);
    // the file is 10 bytes of preamble, a header that ends on a 64-byte boundary, then the raw elements
    {
        std::ifstream f(base + "rowmajor.npy", std::ios::binary);
        std::vector<char> bytes((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
        EXPECT_EQ(bytes.size(), size_t(128 + 15 * 4));
        EXPECT_TRUE(std::memcmp(bytes.data(), "\x93NUMPY\x01\x00\x76\x00", 10) == 0);
        EXPECT_TRUE(std::memcmp(bytes.data() + 128, t.data(), 60) == 0);
    }
    auto col = make(al, {3, 5}, sb::Core::Layout::COLUMN_MAJOR);
    for (int i = 0; i < 15; ++i) col.data_as<float>()[i] = float(i);
    sb::detail::save_npy_file(col, base + "fortran.npy");
    EXPECT_THROWS(sb::detail::load_npy_file(back, base + "fortran.npy"), "Memory order mismatch");
    auto wrong = make(al, {5, 3});
    EXPECT_THROWS(sb::detail::load_npy_file(wrong, base + "rowmajor.npy"), "Shape dimension 0 mismatch");
    EXPECT_THROWS(sb::detail::load_npy_file(back, base + "missing.npy"), "Failed to open file for reading");
    auto view = t.transpose(0, 1);
    EXPECT_THROWS(sb::detail::save_npy_file(view, base + "view.npy"), "contiguous");

    // native container (src/io.cpp:40-109): 72-byte header at the offsets of the reference's struct, then the elements
    sb::detail::save_sushi_file(t, base + "native.sushi");
    {
        std::ifstream f(base + "native.sushi", std::ios::binary);
        std::vector<unsigned char> bytes((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
        EXPECT_EQ(bytes.size(), size_t(72 + 60));
        EXPECT_TRUE(std::memcmp(bytes.data(), "SUSHI\0", 6) == 0);
        int32_t version, rank, dtype, layout; int64_t d0, d1;
        std::memcpy(&version, &bytes[8], 4); std::memcpy(&rank, &bytes[12], 4);
        std::memcpy(&d0, &bytes[16], 8); std::memcpy(&d1, &bytes[24], 8);
        std::memcpy(&dtype, &bytes[64], 4); std::memcpy(&layout, &bytes[68], 4);
        EXPECT_EQ(version, 1); EXPECT_EQ(rank, 2); EXPECT_EQ(d0, 3); EXPECT_EQ(d1, 5);
        EXPECT_EQ(dtype, int32_t(sb::Core::DataType::FLOAT32)); EXPECT_EQ(layout, int32_t(sb::Core::Layout::ROW_MAJOR));
        EXPECT_TRUE(std::memcmp(&bytes[72], t.data(), 60) == 0);
    }
    auto again = make(al, {3, 5});
    sb::detail::load_sushi_file(again, base + "native.sushi");
    for (int i = 0; i < 15; ++i) EXPECT_EQ(again.data_as<float>()[i], t.data_as<float>()[i]);
    EXPECT_THROWS(sb::detail::load_sushi_file(wrong, base + "native.sushi"), "Dimension mismatch at index 0");
    auto rank1 = make(al, {15});
    EXPECT_THROWS(sb::detail::load_sushi_file(rank1, base + "native.sushi"), "Rank mismatch");
    EXPECT_THROWS(sb::detail::load_sushi_file(again, base + "rowmajor.npy"), "Invalid .sushi file magic");
}

TEST_CASE(tensor_text_form)
{
    // src/io.cpp:242-359: header line, nested rows, fixed decimals, "..." past 2 * edge_items entries
    auto al = sr::make_sushi<MallocAllocator>();
    auto t = make(al, {2, 3});
    for (int i = 0; i < 6; ++i) t.data_as<float>()[i] = float(i);
    EXPECT_EQ(sb::detail::format_tensor(t, 1, 3), std::string("Tensor(shape=[2, 3], dtype=f32):\n[[0.0, 1.0, 2.0],\n [3.0, 4.0, 5.0]]\n"));
    // a transposed view prints through its strides
    EXPECT_EQ(sb::detail::format_tensor(t.transpose(0, 1), 0, 3),
              std::string("Tensor(shape=[3, 2], dtype=f32):\n[[0, 3],\n [1, 4],\n [2, 5]]\n"));
    auto v = make(al, {8});
    for (int i = 0; i < 8; ++i) v.data_as<float>()[i] = float(i) * 0.5f;
    EXPECT_EQ(sb::detail::format_tensor(v, 2, 3), std::string("Tensor(shape=[8], dtype=f32):\n[0.00, 0.50, 1.00, ... 2.50, 3.00, 3.50]"));
    EXPECT_EQ(sb::detail::format_tensor(v, 1, 4), std::string("Tensor(shape=[8], dtype=f32):\n[0.0, 0.5, 1.0, 1.5, 2.0, 2.5, 3.0, 3.5]"));
    auto tall = make(al, {8, 1});
    for (int i = 0; i < 8; ++i) tall.data_as<float>()[i] = float(i);
    EXPECT_EQ(sb::detail::format_tensor(tall, 0, 3),
              std::string("Tensor(shape=[8, 1], dtype=f32):\n[[0],\n [1],\n [2],\n \n ...\n [5],\n [6],\n [7]]\n"));
}

TEST_CASE(runtime_context_fails_loudly_without_a_device)
{
    int count = 0;
    if (sushi_cuda_device_count(&count) == SUSHI_CUDA_OK && count > 0) return;     // a GPU is present
    EXPECT_THROWS(sr::Execution::RuntimeContext ctx, "cannot create the CUDA context");
}

TEST_CASE(nccl_id_file_of_another_job_is_not_accepted)
{
    // host half of the multi-GPU rendezvous: a waiting rank takes the id file only when it carries its job's token,
    // so what an earlier (crashed) job left at the same path is ignored
    const std::string path = "/tmp/sushiblas_host_logic_id_" + std::to_string(::getpid()) + ".bin";
    std::remove(path.c_str());
    EXPECT_TRUE(!sr::Execution::RuntimeContext::id_file_matches(path, "job-2"));          // no file
    {
        unsigned char image[192] = {0};
        std::memcpy(image + 128, "job-1", 5);
        std::FILE* f = std::fopen(path.c_str(), "wb");
        EXPECT_TRUE(f != nullptr);
        std::fwrite(image, 1, sizeof image, f);
        std::fclose(f);
    }
    EXPECT_TRUE(sr::Execution::RuntimeContext::id_file_matches(path, "job-1"));
    EXPECT_TRUE(!sr::Execution::RuntimeContext::id_file_matches(path, "job-2"));          // stale: another job's token
    EXPECT_TRUE(!sr::Execution::RuntimeContext::id_file_matches(path, ""));
    {
        std::FILE* f = std::fopen(path.c_str(), "wb");                                    // a bare 128-byte id: too short
        unsigned char id[128] = {0};
        std::fwrite(id, 1, sizeof id, f);
        std::fclose(f);
    }
    EXPECT_TRUE(!sr::Execution::RuntimeContext::id_file_matches(path, ""));
    EXPECT_TRUE(!sr::Execution::RuntimeContext::id_file_matches(path, std::string(64, 'x')));   // token too long
    std::remove(path.c_str());
}

int main() { return check::run_all(); }
