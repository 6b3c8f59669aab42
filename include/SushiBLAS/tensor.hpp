// tensor.hpp -- metadata view over a Storage (reference: include/SushiBLAS/tensor.hpp:54-301).
// Same public fields (shape, strides, rank, dtype, layout, num_elements, storage,
// storage_offset), same constructors and view operations, same error conditions.
// Added for cudaMalloc storage: from_host() / to_host() staging helpers, which are the
// explicit form of the queue.memcpy staging the reference applies to DEVICE tensors
// (src/io.cpp:73-78, 103-108).
#pragma once

#include <algorithm>
#include <array>
#include <cstdint>
#include <initializer_list>
#include <span>
#include <stdexcept>

#include <SushiBLAS/core/common.hpp>
#include <SushiBLAS/core/logger.hpp>
#include <SushiBLAS/storage.hpp>
#include <SushiRuntime/SushiRuntime.h>

namespace SushiBLAS
{
    struct Tensor
    {
        std::array<int64_t, Core::MAX_TENSOR_RANK> shape{};
        std::array<int64_t, Core::MAX_TENSOR_RANK> strides{};   ///< in elements
        int32_t rank = 0;
        Core::DataType dtype = Core::DataType::FLOAT32;
        Core::Layout layout = Core::Layout::ROW_MAJOR;
        int64_t num_elements = 0;
        SushiRuntime::sushi_ptr<Storage> storage;
        int64_t storage_offset = 0;                              ///< in elements

        Tensor() = default;

        /// Contiguous tensor of the given dims over `s`, starting `offset` elements in.
        /// Row-major: last dim fastest; column-major: first dim fastest (tensor.hpp:99-116).
        Tensor(SushiRuntime::sushi_ptr<Storage> s, std::span<const int64_t> dims, int64_t offset = 0,
               Core::Layout l = Core::Layout::ROW_MAJOR)
            : rank(static_cast<int32_t>(dims.size())), layout(l), storage(s), storage_offset(offset)
        {
            SB_THROW_IF(static_cast<std::size_t>(rank) > Core::MAX_TENSOR_RANK, "Rank {} exceeds limit of {}", rank,
                        Core::MAX_TENSOR_RANK);
            int64_t run = 1;
            for (int step = 0; step < rank; ++step)
            {
                const int i = (layout == Core::Layout::ROW_MAJOR) ? rank - 1 - step : step;
                shape[i] = dims[i];
                strides[i] = run;
                run *= dims[i];
            }
            num_elements = run;
            if (storage)
            {
                SB_THROW_IF(storage_offset < 0, "Storage offset cannot be negative ({})", storage_offset);
                // capacity is checked in units of sizeof(float), as the reference does (tensor.hpp:123)
                const std::size_t required_bytes = (static_cast<std::size_t>(num_elements) + storage_offset) * sizeof(float);
                SB_THROW_IF(required_bytes > storage->size_bytes,
                            "Storage capacity exceeded! Required: {} bytes, Available: {} bytes", required_bytes,
                            storage->size_bytes);
            }
        }

        Tensor(SushiRuntime::sushi_ptr<Storage> s, std::initializer_list<int64_t> dims, int64_t offset = 0,
               Core::Layout l = Core::Layout::ROW_MAJOR)
            : Tensor(s, std::span<const int64_t>(dims.begin(), dims.end()), offset, l) {}

        /// Bytes per element of this tensor's dtype as data() scales offsets (tensor.hpp:165).
        std::size_t offset_element_size() const { return dtype == Core::DataType::FLOAT64 ? 8 : 4; }

        /// Start of the tensor's data: a host pointer for SHARED / HOST storage, a device pointer
        /// for DEVICE storage.
        void* data() const
        {
            SB_THROW_IF(storage == nullptr, "Accessing data of a tensor with no storage");
            SB_THROW_IF(storage->data_ptr == nullptr, "Accessing data of a tensor with no data pointer");
            return static_cast<char*>(storage->data_ptr) + storage_offset * static_cast<int64_t>(offset_element_size());
        }

        template <typename T = float>
        T* data_as() const { return static_cast<T*>(data()); }

        bool is_contiguous() const
        {
            if (num_elements == 0) return true;
            int64_t expect = 1;
            for (int step = 0; step < rank; ++step)
            {
                const int i = (layout == Core::Layout::ROW_MAJOR) ? rank - 1 - step : step;
                if (shape[i] == 1) continue;
                if (strides[i] != expect) return false;
                expect *= shape[i];
            }
            return true;
        }

        bool is_aligned() const
        {
            SB_THROW_IF(data() == nullptr, "Alignment check on a tensor with no data pointer (Storage might be null)");
            return reinterpret_cast<std::uintptr_t>(data()) % SushiRuntime::Core::DEFAULT_ALIGNMENT == 0;
        }

        /// View with two dimensions exchanged (no data movement).
        Tensor transpose(int32_t dim0, int32_t dim1) const
        {
            SB_THROW_IF(dim0 >= rank || dim1 >= rank, "Invalid dimensions ({}, {}) for rank {}", dim0, dim1, rank);
            Tensor t = *this;
            std::swap(t.shape[dim0], t.shape[dim1]);
            std::swap(t.strides[dim0], t.strides[dim1]);
            return t;
        }

        /// Contiguous view with new dims and the same element count.
        Tensor reshape(std::initializer_list<int64_t> new_dims) const
        {
            std::span<const int64_t> dims(new_dims.begin(), new_dims.end());
            int64_t count = 1;
            for (int64_t d : dims) count *= d;
            SB_THROW_IF(count != num_elements, "Element count mismatch. Current: {}, New: {}", num_elements, count);
            SB_THROW_IF(!is_contiguous(), "Tensor must be contiguous for this operation");
            Tensor t(storage, dims, storage_offset, layout);
            t.dtype = dtype;
            return t;
        }

        /// Sub-range [start, end) of dimension `dim` (negative indices count from the end).
        /// As in the reference (tensor.hpp:280-300) the result is rebuilt as a contiguous tensor
        /// of the sliced shape at the new offset, so only slices that stay contiguous (leading
        /// dimension for row-major, trailing for column-major) describe the same elements.
        Tensor slice(int32_t dim, int64_t start, int64_t end) const
        {
            SB_THROW_IF(dim < 0 || dim >= rank, "Invalid dimension {}", dim);
            const int64_t extent = shape[dim];
            if (start < 0) start += extent;
            if (end < 0) end += extent;
            start = std::clamp<int64_t>(start, 0, extent);
            end = std::clamp<int64_t>(end, start, extent);
            std::array<int64_t, Core::MAX_TENSOR_RANK> dims = shape;
            dims[dim] = end - start;
            Tensor t(storage, std::span<const int64_t>(dims.data(), static_cast<std::size_t>(rank)),
                     storage_offset + start * strides[dim], layout);
            t.dtype = dtype;
            return t;
        }

        /// Copies num_elements contiguous elements from host memory into the tensor (blocking).
        void from_host(const void* src) const { stage(const_cast<void*>(src), true); }
        /// Copies the tensor's num_elements contiguous elements to host memory (blocking).
        void to_host(void* dst) const { stage(dst, false); }

    private:
        void stage(void* host, bool upload) const
        {
            SB_THROW_IF(!is_contiguous(), "Tensor must be contiguous for this operation");
            std::size_t elem = offset_element_size();
            if (dtype == Core::DataType::HALF) elem = 2;
            if (dtype == Core::DataType::COMPLEX32) elem = 8;
            if (dtype == Core::DataType::COMPLEX64) elem = 16;
            const std::size_t bytes = static_cast<std::size_t>(num_elements) * elem;
            if (storage->host_resident())
            {
                if (upload) std::memcpy(data(), host, bytes); else std::memcpy(host, data(), bytes);
                return;
            }
            sushi_cuda_ctx* ctx = storage->allocator->native_context();
            SB_THROW_IF(ctx == nullptr, "Tensor storage has no device context");
            int rc = upload ? sushi_cuda_memcpy_h2d(ctx, 0, data(), host, bytes)
                            : sushi_cuda_memcpy_d2h(ctx, 0, host, data(), bytes);
            if (rc == SUSHI_CUDA_OK) rc = sushi_cuda_sync(ctx, 0);
            SB_THROW_IF(rc != SUSHI_CUDA_OK, "Tensor staging failed: {}", sushi_cuda_last_error(ctx));
        }
    };
} // namespace SushiBLAS
