// io.hpp -- tensor persistence in the native ".sushi" container, in NumPy's .npy format and as raw bytes
// and as text (reference: include/SushiBLAS/io.hpp:47-125, src/io.cpp:40-359).  Same entry points and the same
// staging convention: pending work is flushed first (execute().wait()), a DEVICE tensor goes
// through a host buffer (src/io.cpp:73-78, 187-193), SHARED / HOST tensors are written from
// their host image.  The .npy writer emits format version 1.0 with the dictionary padded so
// that the data starts on a 64-byte boundary, i.e. the bytes numpy.save writes for the same
// array.  The loader parses the dictionary (versions 1.0 - 3.0) and, where the reference only
// looks for the digits of each extent somewhere after "'shape': (" (src/io.cpp:214-218),
// checks dtype, order and the exact shape, with the reference's messages for the failures the
// reference reports.
#pragma once

#include <cstdint>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

#include <SushiBLAS/core/common.hpp>
#include <SushiBLAS/core/logger.hpp>
#include <SushiBLAS/tensor.hpp>

namespace SushiBLAS
{
    class Engine;

    namespace detail
    {
        inline const char* npy_descr(Core::DataType dtype)
        {
            switch (dtype)
            {
                case Core::DataType::FLOAT32: return "<f4";
                case Core::DataType::FLOAT64: return "<f8";
                case Core::DataType::COMPLEX32: return "<c8";
                case Core::DataType::COMPLEX64: return "<c16";
                case Core::DataType::HALF: return "<f2";
                default: return "";
            }
        }

        inline std::size_t io_bytes_per_element(Core::DataType dtype)
        {
            if (dtype == Core::DataType::FLOAT64 || dtype == Core::DataType::COMPLEX32) return 8;
            if (dtype == Core::DataType::COMPLEX64) return 16;
            if (dtype == Core::DataType::HALF) return 2;
            return 4;
        }

        /// The header dictionary of a version-1.0 file, padded with spaces and closed by '\n' so
        /// that 10 + its length is a multiple of 64 (src/io.cpp:149-169).
        inline std::string npy_header_dict(Core::DataType dtype, Core::Layout layout, const int64_t* shape, int rank)
        {
            std::string dict = "{'descr': '";
            dict += npy_descr(dtype);
            dict += "', 'fortran_order': ";
            dict += (layout == Core::Layout::COLUMN_MAJOR) ? "True" : "False";
            dict += ", 'shape': (";
            for (int i = 0; i < rank; ++i)
            {
                dict += std::to_string(shape[i]);
                if (rank == 1 || i + 1 < rank) dict += ",";
                if (i + 1 < rank) dict += " ";
            }
            dict += "), }";
            while ((10 + dict.size() + 1) % 64 != 0) dict += ' ';
            dict += '\n';
            return dict;
        }

        struct NpyInfo
        {
            std::string descr;
            bool fortran_order = false;
            std::vector<int64_t> shape;
        };

        /// Parses the Python-literal dictionary of a .npy header.  Throws on anything that is not
        /// {'descr': '<str>', 'fortran_order': True|False, 'shape': (<ints>)} in any key order.
        inline NpyInfo parse_npy_header(const std::string& h)
        {
            NpyInfo info;
            auto value_after = [&](const char* key) -> std::size_t
            {
                std::size_t p = h.find(key);
                SB_THROW_IF(p == std::string::npos, "Malformed .npy header: missing {}", key);
                p = h.find(':', p + std::strlen(key));
                SB_THROW_IF(p == std::string::npos, "Malformed .npy header: missing value of {}", key);
                ++p;
                while (p < h.size() && h[p] == ' ') ++p;
                return p;
            };
            std::size_t p = value_after("'descr'");
            SB_THROW_IF(p >= h.size() || (h[p] != '\'' && h[p] != '"'), "Malformed .npy header: descr is not a string");
            const std::size_t q = h.find(h[p], p + 1);
            SB_THROW_IF(q == std::string::npos, "Malformed .npy header: unterminated descr");
            info.descr = h.substr(p + 1, q - p - 1);

            p = value_after("'fortran_order'");
            if (h.compare(p, 4, "True") == 0) info.fortran_order = true;
            else if (h.compare(p, 5, "False") == 0) info.fortran_order = false;
            else SB_THROW_IF(true, "Malformed .npy header: fortran_order is neither True nor False");

            p = value_after("'shape'");
            SB_THROW_IF(p >= h.size() || h[p] != '(', "Malformed .npy header: shape is not a tuple");
            ++p;
            while (p < h.size() && h[p] != ')')
            {
                if (h[p] == ' ' || h[p] == ',') { ++p; continue; }
                SB_THROW_IF(h[p] < '0' || h[p] > '9', "Malformed .npy header: bad character in shape");
                int64_t v = 0;
                while (p < h.size() && h[p] >= '0' && h[p] <= '9') v = v * 10 + (h[p++] - '0');
                if (p < h.size() && h[p] == 'L') ++p;          // Python 2 long suffix
                info.shape.push_back(v);
            }
            SB_THROW_IF(p >= h.size(), "Malformed .npy header: unterminated shape");
            return info;
        }
    } // namespace detail

    class IO
    {
        public:
            explicit IO(Engine& e) : engine_(e) {}

            /// Native ".sushi" container: a 72-byte header (magic, version, rank, extents, dtype, layout) and
            /// the raw elements (src/io.cpp:40-109).
            inline void save(const Tensor& t, const std::string& path);
            inline void load(Tensor& t, const std::string& path);
            /// Writes `t` as a NumPy .npy file that numpy.load() opens (src/io.cpp:136-196).
            /// Flushes the engine's pending tasks first.  The tensor must be contiguous.
            inline void save_npy(const Tensor& t, const std::string& path);
            /// Reads a .npy file into `t` (src/io.cpp:198-240); dtype, order and shape must match.
            inline void load_npy(Tensor& t, const std::string& path);
            /// Raw element bytes without a header (src/io.cpp:111-134); also serves DEVICE tensors.
            inline void save_bin(const Tensor& t, const std::string& path);
            inline void load_bin(Tensor& t, const std::string& path);
            /// Text form as numpy-style nested rows (src/io.cpp:242-359); print() writes it to stdout.
            inline std::string to_string(const Tensor& t, int precision = 4, int edge_items = 3);
            inline void print(const Tensor& t, int precision = 4, int edge_items = 3);

        private:
            Engine& engine_;
    };
} // namespace SushiBLAS
