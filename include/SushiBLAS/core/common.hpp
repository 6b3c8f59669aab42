// core/common.hpp -- enums shared by Tensor / Engine (same names and values as the reference's
// include/SushiBLAS/core/common.hpp:41-59).
#pragma once

#include <cstddef>
#include <cstdint>

namespace SushiBLAS
{
    namespace Core
    {
        enum class Layout : std::uint8_t
        {
            ROW_MAJOR,
            COLUMN_MAJOR
        };

        enum class DataType : std::uint8_t
        {
            HALF,
            FLOAT32,
            FLOAT64,
            COMPLEX32,
            COMPLEX64
        };

        inline constexpr std::size_t MAX_TENSOR_RANK = 6;
    } // namespace Core
} // namespace SushiBLAS

namespace sb = SushiBLAS;
