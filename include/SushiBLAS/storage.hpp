// storage.hpp -- reference-counted owner of one allocation (reference:
// include/SushiBLAS/storage.hpp:49-113).  Same public fields and constructor contract: the
// size is rounded up to 128 bytes, allocation goes through the USMAllocator with the chosen
// strategy, the destructor returns the block.  With the CUDA allocator, DEVICE is cudaMalloc
// memory and SHARED / HOST are pinned host images that operations stage through a device
// mirror (see sr::Memory::AllocStrategy).
#pragma once

#include <cstddef>

#include <SushiBLAS/core/common.hpp>
#include <SushiBLAS/core/logger.hpp>
#include <SushiRuntime/SushiRuntime.h>

namespace SushiBLAS
{
    class alignas(64) Storage : public SushiRuntime::Core::RefCounted
    {
        public:
            void* data_ptr = nullptr;          ///< host pointer (SHARED/HOST) or device pointer (DEVICE)
            std::size_t size_bytes = 0;        ///< allocated bytes (multiple of 128)
            std::size_t requested_bytes = 0;   ///< bytes asked for
            SushiRuntime::sushi_ptr<SushiRuntime::Memory::USMAllocator> allocator;
            SushiRuntime::Memory::AllocStrategy strategy;

            Storage(SushiRuntime::sushi_ptr<SushiRuntime::Memory::USMAllocator> alloc, std::size_t n_bytes,
                    SushiRuntime::Memory::AllocStrategy strat = SushiRuntime::Memory::AllocStrategy::SHARED)
                : requested_bytes(n_bytes), allocator(alloc), strategy(strat)
            {
                SB_THROW_IF(!allocator, "Allocator pointer cannot be null");
                SB_THROW_IF(n_bytes == 0, "Requested size cannot be zero");
                constexpr std::size_t align = SushiRuntime::Core::DEFAULT_ALIGNMENT;
                size_bytes = (n_bytes + align - 1) / align * align;
                data_ptr = allocator->allocate(size_bytes, strategy);
                SB_THROW_IF(!data_ptr, "Allocation failed for {} bytes", size_bytes);
            }

            Storage(const Storage&) = delete;
            Storage& operator=(const Storage&) = delete;

            /// True when data_ptr can be dereferenced on the host.
            bool host_resident() const { return allocator->is_host_resident(data_ptr); }

        protected:
            ~Storage() override
            {
                if (data_ptr && allocator) allocator->deallocate(data_ptr);
            }
    };
} // namespace SushiBLAS
