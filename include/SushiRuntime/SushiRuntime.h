// SushiRuntime.h -- the small public surface of the runtime that SushiBLAS callers touch,
// rewritten for the CUDA backend (no SYCL).  One header, header-only.
//
// What is kept, with the reference's spellings so that caller code compiles unchanged:
//   sr::Core::RefCounted, sr::sushi_ptr<T>, sr::make_sushi<T>     (include/SushiRuntime/core/ref_counted.hpp:38-80,
//                                                                  core/sushi_ptr.hpp:38-143)
//   sr::Core::DEFAULT_ALIGNMENT, MAX_SUPPORTED_XPU                (core/common.hpp:40-53)
//   sr::Memory::AllocStrategy, sr::Memory::USMAllocator           (memory/usm_allocator.hpp:33-71)
//   sr::Graph::TaskType / OpID / "_op" / TaskMetadata / TaskGraph (graph/task_types.hpp:35-129,
//                                                                  graph/task_graph.hpp:55-125)
//   sr::Execution::RuntimeContext                                 (execution/runtime_context.hpp:42-96)
// What changes: sycl::queue / sycl::event are gone.  A RuntimeContext owns one sushi_cuda_ctx
// (C ABI, include/sushiblas_cuda.h) with one in-order stream; TaskGraph is a deferred list of
// closures replayed in submission order on that stream, which satisfies every read/write
// dependency the reference infers from pointer sets; execute() returns an Event whose wait()
// synchronises the stream and raises std::runtime_error on any recorded failure.
// The work-stealing scheduler, the dependency tracker, the memory pool and the NUMA/topology
// layers of the reference are not rebuilt.
#pragma once

#include <atomic>
#include <chrono>
#include <cstdio>
#include <thread>
#include <cstddef>
#include <cstdint>
#include <cstring>
#include <functional>
#include <memory>
#include <mutex>
#include <stdexcept>
#include <string>
#include <type_traits>
#include <unordered_map>
#include <unordered_set>
#include <utility>
#include <vector>

#include "../sushiblas_cuda.h"

namespace SushiRuntime
{
    namespace Core
    {
        inline constexpr std::size_t DEFAULT_ALIGNMENT = 128;
        inline constexpr std::size_t MAX_SUPPORTED_XPU = 16;

        /// Intrusive reference count; objects are deleted when the count drops to zero.
        class RefCounted
        {
            public:
                RefCounted() = default;
                RefCounted(const RefCounted&) = delete;
                RefCounted& operator=(const RefCounted&) = delete;

                void add_ref() const noexcept { refs_.fetch_add(1, std::memory_order_relaxed); }
                void release() const noexcept
                {
                    if (refs_.fetch_sub(1, std::memory_order_acq_rel) == 1) delete this;
                }
                std::uint32_t ref_count() const noexcept { return refs_.load(std::memory_order_acquire); }

            protected:
                virtual ~RefCounted() = default;

            private:
                mutable std::atomic<std::uint32_t> refs_{0};
        };
    } // namespace Core

    /// Smart pointer for RefCounted objects.
    template <typename T>
    class sushi_ptr
    {
        public:
            sushi_ptr() noexcept = default;
            sushi_ptr(std::nullptr_t) noexcept {}
            explicit sushi_ptr(T* p) noexcept : p_(p) { acquire(); }
            sushi_ptr(const sushi_ptr& o) noexcept : p_(o.p_) { acquire(); }
            sushi_ptr(sushi_ptr&& o) noexcept : p_(o.p_) { o.p_ = nullptr; }
            template <typename U, typename = std::enable_if_t<std::is_convertible_v<U*, T*>>>
            sushi_ptr(const sushi_ptr<U>& o) noexcept : p_(o.get()) { acquire(); }
            ~sushi_ptr() { drop(); }

            sushi_ptr& operator=(const sushi_ptr& o) noexcept
            {
                if (p_ != o.p_) { drop(); p_ = o.p_; acquire(); }
                return *this;
            }
            sushi_ptr& operator=(sushi_ptr&& o) noexcept
            {
                if (this != &o) { drop(); p_ = o.p_; o.p_ = nullptr; }
                return *this;
            }
            sushi_ptr& operator=(std::nullptr_t) noexcept { drop(); p_ = nullptr; return *this; }

            T* get() const noexcept { return p_; }
            T* operator->() const noexcept { return p_; }
            T& operator*() const noexcept { return *p_; }
            explicit operator bool() const noexcept { return p_ != nullptr; }
            void reset() noexcept { drop(); p_ = nullptr; }

            friend bool operator==(const sushi_ptr& a, const sushi_ptr& b) noexcept { return a.p_ == b.p_; }
            friend bool operator!=(const sushi_ptr& a, const sushi_ptr& b) noexcept { return a.p_ != b.p_; }
            friend bool operator==(const sushi_ptr& a, std::nullptr_t) noexcept { return a.p_ == nullptr; }
            friend bool operator!=(const sushi_ptr& a, std::nullptr_t) noexcept { return a.p_ != nullptr; }

        private:
            void acquire() const noexcept { if (p_) p_->add_ref(); }
            void drop() const noexcept { if (p_) p_->release(); }
            T* p_ = nullptr;
    };

    template <typename T, typename... Args>
    sushi_ptr<T> make_sushi(Args&&... args)
    {
        return sushi_ptr<T>(new T(std::forward<Args>(args)...));
    }

    namespace Memory
    {
        /// Where a tensor's bytes live.  With cudaMalloc storage and explicit staging:
        ///  DEVICE: device memory only; data() is a device pointer.
        ///  SHARED: pinned host image the caller reads/writes, mirrored by a device buffer that operations
        ///          work on.  Residency is tracked per allocation: within one execute() round an
        ///          input goes up at most once, what an operation wrote stays on the device for the
        ///          operations after it (also in later rounds), and the host image is refreshed once,
        ///          when the caller waits (Event::wait / RuntimeContext::wait_all).  Between a wait
        ///          and the next execute() the host may rewrite any tensor: a host-valid image is sent
        ///          up again by the first operation of the next round that reads it.
        ///  HOST:   pinned host image, staged the same way.
        enum class AllocStrategy
        {
            DEVICE,
            SHARED,
            HOST
        };

        /// Allocation interface handed to Storage.  allocate()/deallocate() keep the reference's
        /// meaning; the three staging queries replace "which sycl::device owns this pointer".
        class USMAllocator : public Core::RefCounted
        {
            public:
                virtual void* allocate(std::size_t bytes, AllocStrategy strategy = AllocStrategy::SHARED,
                                       std::size_t alignment = Core::DEFAULT_ALIGNMENT) = 0;
                virtual void deallocate(void* ptr) = 0;

                /// True when `ptr` (an allocation base) is dereferenceable on the host.
                virtual bool is_host_resident(void* ptr) = 0;
                /// Device buffer backing `ptr`: the pointer itself for DEVICE allocations, a lazily
                /// created device mirror of equal size for SHARED / HOST ones; nullptr if unknown.
                virtual void* device_view(void* ptr) = 0;
                /// Native context the allocation belongs to (nullptr for host-only test allocators).
                virtual sushi_cuda_ctx* native_context() { return nullptr; }

                // -- residency of host-resident allocations (no-ops for allocators without a device)
                /// Starts an execute() round: host images may have been rewritten since the last one.
                virtual void begin_round() {}
                /// Device buffer of allocation `ptr` for an operation that is being enqueued.  With
                /// `contents` the buffer must hold what the allocation holds (the operation reads it, or
                /// writes only part of it): a host image newer than the mirror is uploaded first.
                /// Returns nullptr on failure (*rc receives the status when given).
                virtual void* device_for_operation(void* ptr, bool contents, int* rc = nullptr)
                {
                    (void)contents;
                    if (rc) *rc = 0;
                    return device_view(ptr);
                }
                /// An enqueued operation writes allocation `ptr` on the device: its host image is stale
                /// until flush_to_host().
                virtual void mark_device_written(void* ptr) { (void)ptr; }
                /// Enqueues the download of every allocation whose host image is stale; returns a status.
                virtual int flush_to_host() { return 0; }

            protected:
                ~USMAllocator() override = default;
        };
    } // namespace Memory

    namespace Graph
    {
        enum class TaskType : std::uint8_t
        {
            NONE = 0,
            MATH_OP,
            MEMORY_COPY,
            CUSTOM_HOST,
            CONTROL_FLOW
        };

        /// Operation identifier: 32-bit FNV-1a hash of the operation's dotted name.
        struct OpID
        {
            std::uint32_t value;

            constexpr OpID() : value(0) {}
            constexpr explicit OpID(std::uint32_t v) : value(v) {}

            static constexpr std::uint32_t hash_str(const char* s, std::size_t n)
            {
                std::uint32_t h = 0x811C9DC5u;           // FNV offset basis
                for (std::size_t i = 0; i < n; ++i)
                {
                    h ^= static_cast<std::uint8_t>(s[i]);
                    h *= 0x01000193u;                    // FNV prime
                }
                return h;
            }

            constexpr bool operator==(const OpID& o) const { return value == o.value; }
            constexpr bool operator!=(const OpID& o) const { return value != o.value; }
            constexpr bool operator<(const OpID& o) const { return value < o.value; }
        };

        namespace Literals
        {
            constexpr OpID operator""_op(const char* s, std::size_t n) { return OpID(OpID::hash_str(s, n)); }
        }

        /// Name, category, id and up to eight 64-bit scalar parameters of a task.
        struct TaskMetadata
        {
            const char* name = "unnamed_task";
            TaskType task_type = TaskType::NONE;
            OpID op_id = OpID(0);

            static constexpr std::size_t K_MAX_PARAMS = 8;
            std::uint64_t params[K_MAX_PARAMS] = {0};

            template <typename T>
            void set_param(int index, T value)
            {
                static_assert(std::is_trivially_copyable_v<T> && sizeof(T) <= sizeof(std::uint64_t));
                if (index < 0 || index >= static_cast<int>(K_MAX_PARAMS)) return;
                params[index] = 0;
                std::memcpy(&params[index], &value, sizeof(T));
            }

            template <typename T>
            T get_param(int index) const
            {
                static_assert(std::is_trivially_copyable_v<T> && sizeof(T) <= sizeof(std::uint64_t));
                T value{};
                if (index >= 0 && index < static_cast<int>(K_MAX_PARAMS)) std::memcpy(&value, &params[index], sizeof(T));
                return value;
            }
        };
    } // namespace Graph

    namespace Execution
    {
        class RuntimeContext;

        /// Completion handle returned by TaskGraph::execute() / Engine::execute().
        /// A default-constructed Event is already complete (what the reference's op calls return).
        class Event
        {
            public:
                Event() = default;
                explicit Event(RuntimeContext* ctx) : ctx_(ctx) {}
                /// Blocks until the context's stream has drained; throws std::runtime_error on failure.
                inline void wait();

            private:
                RuntimeContext* ctx_ = nullptr;
        };

        namespace detail
        {
            /// cudaMalloc / pinned-host allocator bound to one sushi_cuda_ctx.
            class CudaAllocator final : public Memory::USMAllocator
            {
                public:
                    explicit CudaAllocator(sushi_cuda_ctx* ctx) : ctx_(ctx) {}

                    void* allocate(std::size_t bytes, Memory::AllocStrategy strategy, std::size_t) override
                    {
                        void* p = nullptr;
                        const int rc = (strategy == Memory::AllocStrategy::DEVICE)
                                           ? sushi_cuda_malloc(ctx_, 0, bytes, &p)
                                           : sushi_cuda_host_alloc(ctx_, bytes, &p);
                        if (rc != SUSHI_CUDA_OK) return nullptr;
                        std::lock_guard<std::mutex> lock(mutex_);
                        blocks_[p] = Block{bytes, strategy, nullptr};
                        return p;
                    }

                    void deallocate(void* ptr) override
                    {
                        Block b;
                        {
                            std::lock_guard<std::mutex> lock(mutex_);
                            auto it = blocks_.find(ptr);
                            if (it == blocks_.end()) return;
                            b = it->second;
                            blocks_.erase(it);
                        }
                        // queued work may still reference the block
                        sushi_cuda_sync(ctx_, 0);
                        if (b.strategy == Memory::AllocStrategy::DEVICE) sushi_cuda_free(ctx_, 0, ptr);
                        else
                        {
                            if (b.mirror) sushi_cuda_free(ctx_, 0, b.mirror);
                            if (b.written) sushi_cuda_marker_destroy(ctx_, b.written);
                            sushi_cuda_host_free(ctx_, ptr);
                        }
                    }

                    bool is_host_resident(void* ptr) override
                    {
                        std::lock_guard<std::mutex> lock(mutex_);
                        auto it = blocks_.find(ptr);
                        return it != blocks_.end() && it->second.strategy != Memory::AllocStrategy::DEVICE;
                    }

                    void* device_view(void* ptr) override
                    {
                        std::lock_guard<std::mutex> lock(mutex_);
                        auto it = blocks_.find(ptr);
                        if (it == blocks_.end()) return nullptr;
                        Block& b = it->second;
                        if (b.strategy == Memory::AllocStrategy::DEVICE) return ptr;
                        if (!b.mirror && sushi_cuda_malloc(ctx_, 0, b.bytes, &b.mirror) != SUSHI_CUDA_OK) return nullptr;
                        return b.mirror;
                    }

                    sushi_cuda_ctx* native_context() override { return ctx_; }

                    void begin_round() override
                    {
                        std::lock_guard<std::mutex> lock(mutex_);
                        ++round_;
                        // uploads of this round may overtake its own operations, never those of earlier rounds
                        // (which may still read the mirrors about to be refreshed)
                        fence_status_ = sushi_cuda_upload_fence(ctx_, 0);
                    }

                    void* device_for_operation(void* ptr, bool contents, int* rc) override
                    {
                        std::lock_guard<std::mutex> lock(mutex_);
                        int status = fence_status_;
                        void* out = nullptr;
                        auto it = blocks_.find(ptr);
                        if (status == SUSHI_CUDA_OK && it == blocks_.end()) status = SUSHI_CUDA_ERR_INVALID_ARG;
                        if (status == SUSHI_CUDA_OK)
                        {
                            Block& b = it->second;
                            if (b.strategy == Memory::AllocStrategy::DEVICE) out = ptr;
                            else
                            {
                                if (!b.mirror) status = sushi_cuda_malloc(ctx_, 0, b.bytes, &b.mirror);
                                // the mirror is current when the device wrote it last (host image stale) or
                                // when it was brought up in the current execute() round
                                if (status == SUSHI_CUDA_OK && contents && !b.host_stale && b.valid_round != round_)
                                    status = sushi_cuda_upload_ahead(ctx_, 0, b.mirror, ptr, b.bytes);
                                if (status == SUSHI_CUDA_OK)
                                {
                                    if (contents) b.valid_round = round_;
                                    out = b.mirror;
                                }
                            }
                        }
                        if (rc) *rc = status;
                        return out;
                    }

                    void mark_device_written(void* ptr) override
                    {
                        std::lock_guard<std::mutex> lock(mutex_);
                        auto it = blocks_.find(ptr);
                        if (it == blocks_.end() || it->second.strategy == Memory::AllocStrategy::DEVICE) return;
                        Block& b = it->second;
                        if (!b.host_stale) stale_.push_back(ptr);
                        b.host_stale = true;
                        b.valid_round = round_;
                        // the point in the stream after which the mirror holds what this operation wrote; without
                        // a marker the download is ordered behind everything queued (flush_to_host)
                        if (!b.written && sushi_cuda_marker_create(ctx_, 0, &b.written) != SUSHI_CUDA_OK) b.written = nullptr;
                        if (b.written && sushi_cuda_marker_record(ctx_, 0, b.written) != SUSHI_CUDA_OK)
                        {
                            sushi_cuda_marker_destroy(ctx_, b.written);
                            b.written = nullptr;
                        }
                    }

                    int flush_to_host() override
                    {
                        std::lock_guard<std::mutex> lock(mutex_);
                        int status = SUSHI_CUDA_OK;
                        for (void* ptr : stale_)
                        {
                            auto it = blocks_.find(ptr);
                            if (it == blocks_.end() || !it->second.host_stale) continue;      // freed meanwhile
                            Block& b = it->second;
                            // each image comes down as soon as its last writer has finished, beside whatever
                            // the device still has queued
                            if (status == SUSHI_CUDA_OK)
                                status = b.written ? sushi_cuda_download_behind(ctx_, 0, ptr, b.mirror, b.bytes, b.written)
                                                   : sushi_cuda_memcpy_d2h(ctx_, 0, ptr, b.mirror, b.bytes);
                            b.host_stale = false;
                        }
                        stale_.clear();
                        return status;
                    }

                private:
                    struct Block
                    {
                        std::size_t bytes;
                        Memory::AllocStrategy strategy;
                        void* mirror;
                        std::uint64_t valid_round = 0;    ///< execute() round in which the mirror was last made current
                        bool host_stale = false;          ///< the device wrote the mirror after the host image
                        sushi_cuda_marker* written = nullptr;   ///< stream position of the last device write
                    };
                    std::uint64_t round_ = 1;
                    int fence_status_ = SUSHI_CUDA_OK;
                    std::vector<void*> stale_;
                    sushi_cuda_ctx* ctx_;
                    std::mutex mutex_;
                    std::unordered_map<void*, Block> blocks_;
            };
        } // namespace detail

        /// One process per GPU: which rank this process is, how many there are, which CUDA device it
        /// drives, and a file through which rank 0 hands the 128-byte NCCL id to the others (any
        /// path all ranks can read).  Rank 0 writes the id followed by `job_token` (at most 63 characters)
        /// and removes the file once every rank has joined; the other ranks accept a file only when its
        /// token equals theirs, so a file left behind by an earlier job -- a crashed one, since a finished
        /// one removes it -- is ignored as long as the jobs use different tokens (a launcher's job id, a
        /// timestamp), and otherwise the wait for a matching file ends after `timeout_s`.
        struct DistributedConfig
        {
            int rank = 0;
            int nranks = 1;
            int device = 0;
            std::string id_file;
            int timeout_s = 60;
            std::string job_token;
        };

        /// Owns the device context.  Construction needs a CUDA device (sm_100a): there is no CPU
        /// fallback, so it throws std::runtime_error otherwise.  The device is device 0 or the
        /// one named by $SUSHI_CUDA_DEVICE.
        class RuntimeContext
        {
            public:
                RuntimeContext()
                {
                    const int rc = sushi_cuda_init(nullptr, 0, &ctx_);
                    if (rc != SUSHI_CUDA_OK)
                        throw std::runtime_error(std::string("RuntimeContext: cannot create the CUDA context: ") +
                                                 sushi_cuda_last_error(nullptr));
                    allocator_ = make_sushi<detail::CudaAllocator>(ctx_);
                }

                /// Member of a multi-GPU job (the reference has no counterpart: its only multi-device
                /// hook is get_queue(xpu_index), runtime_context.hpp:65).  Creates the context on
                /// cfg.device and joins the NCCL communicator of cfg.nranks processes.
                explicit RuntimeContext(const DistributedConfig& cfg) : rank_(cfg.rank), nranks_(cfg.nranks)
                {
                    if (cfg.nranks < 1 || cfg.rank < 0 || cfg.rank >= cfg.nranks)
                        throw std::runtime_error("RuntimeContext: bad rank / nranks");
                    const int dev = cfg.device;
                    int rc = sushi_cuda_init(&dev, 1, &ctx_);
                    if (rc != SUSHI_CUDA_OK)
                        throw std::runtime_error(std::string("RuntimeContext: cannot create the CUDA context: ") +
                                                 sushi_cuda_last_error(nullptr));
                    allocator_ = make_sushi<detail::CudaAllocator>(ctx_);
                    if (cfg.nranks == 1) return;
                    // file image: 128 bytes of NCCL id, then the job token in 64 zero-padded bytes
                    unsigned char image[192] = {0}, want_token[64] = {0};
                    if (cfg.job_token.size() > 63) fail_plain("job_token is longer than 63 characters");
                    std::memcpy(want_token, cfg.job_token.data(), cfg.job_token.size());
                    if (cfg.rank == 0)
                    {
                        rc = sushi_cuda_comm_unique_id(image);
                        if (rc != SUSHI_CUDA_OK) fail("cannot create the NCCL id");
                        std::memcpy(image + 128, want_token, sizeof want_token);
                        std::remove(cfg.id_file.c_str());          // whatever an earlier job left there
                        const std::string tmp = cfg.id_file + ".tmp";
                        std::FILE* f = std::fopen(tmp.c_str(), "wb");
                        const bool written = f && std::fwrite(image, 1, sizeof image, f) == sizeof image;
                        if (f) std::fclose(f);
                        if (!written) fail("cannot write the NCCL id file");
                        if (std::rename(tmp.c_str(), cfg.id_file.c_str()) != 0) fail("cannot publish the NCCL id file");
                    }
                    else
                    {
                        // the host-side rendezvous is bounded: give up after timeout_s
                        const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(cfg.timeout_s);
                        bool got = false;
                        while (!got && std::chrono::steady_clock::now() < deadline)
                        {
                            if (std::FILE* f = std::fopen(cfg.id_file.c_str(), "rb"))
                            {
                                got = std::fread(image, 1, sizeof image, f) == sizeof image &&
                                      std::memcmp(image + 128, want_token, sizeof want_token) == 0;
                                std::fclose(f);
                            }
                            if (!got) std::this_thread::sleep_for(std::chrono::milliseconds(20));
                        }
                        if (!got) fail_plain("timed out waiting for the NCCL id file of rank 0 (none, or none with this job's token)");
                    }
                    rc = sushi_cuda_comm_init_rank(ctx_, 0, image, cfg.nranks, cfg.rank);
                    if (rc != SUSHI_CUDA_OK) fail("cannot join the NCCL communicator");
                    // the communicator exists on every rank, so every rank has read the file
                    if (cfg.rank == 0) std::remove(cfg.id_file.c_str());
                }

                /// Host half of the rendezvous alone (no device): true when `path` holds an id image whose
                /// token equals `job_token`.  What the waiting ranks test; exposed for host-only tests.
                static bool id_file_matches(const std::string& path, const std::string& job_token)
                {
                    unsigned char image[192] = {0}, want[64] = {0};
                    if (job_token.size() > 63) return false;
                    std::memcpy(want, job_token.data(), job_token.size());
                    std::FILE* f = std::fopen(path.c_str(), "rb");
                    if (!f) return false;
                    const bool ok = std::fread(image, 1, sizeof image, f) == sizeof image && std::memcmp(image + 128, want, sizeof want) == 0;
                    std::fclose(f);
                    return ok;
                }

                int rank() const { return rank_; }
                int nranks() const { return nranks_; }

                ~RuntimeContext()
                {
                    allocator_.reset();
                    if (ctx_) sushi_cuda_destroy(ctx_);
                }

                RuntimeContext(const RuntimeContext&) = delete;
                RuntimeContext& operator=(const RuntimeContext&) = delete;

                /// Kept for source compatibility; the single device is found at construction.
                void probe_hardware() {}

                sushi_ptr<Memory::USMAllocator> get_allocator() { return allocator_; }
                sushi_ptr<Memory::USMAllocator> get_allocator(int /*numa_id*/) { return allocator_; }

                /// Global synchronisation; throws std::runtime_error if anything queued has failed.  Host images
                /// of the SHARED / HOST allocations that queued operations wrote are refreshed here (one
                /// download each), behind everything queued, before the call returns.
                void wait_all()
                {
                    int rc = allocator_ ? allocator_->flush_to_host() : SUSHI_CUDA_OK;
                    if (rc == SUSHI_CUDA_OK) rc = sushi_cuda_sync(ctx_, 0);
                    if (rc != SUSHI_CUDA_OK)
                        throw std::runtime_error(std::string("wait_all: ") + sushi_cuda_last_error(ctx_));
                }

                /// The C-ABI handle (for the op front-ends).
                sushi_cuda_ctx* native_handle() const { return ctx_; }

            private:
                [[noreturn]] void fail(const char* what)
                {
                    std::string msg = std::string("RuntimeContext: ") + what + ": " + sushi_cuda_last_error(ctx_);
                    allocator_.reset();
                    if (ctx_) sushi_cuda_destroy(ctx_);
                    ctx_ = nullptr;
                    throw std::runtime_error(msg);
                }
                /// Same for failures of the host-side protocol (no library error text to append).
                [[noreturn]] void fail_plain(const char* what)
                {
                    allocator_.reset();
                    if (ctx_) sushi_cuda_destroy(ctx_);
                    ctx_ = nullptr;
                    throw std::runtime_error(std::string("RuntimeContext: ") + what);
                }
                sushi_cuda_ctx* ctx_ = nullptr;
                sushi_ptr<Memory::USMAllocator> allocator_;
                int rank_ = 0, nranks_ = 1;
        };

        inline void Event::wait()
        {
            if (ctx_) ctx_->wait_all();
        }
    } // namespace Execution

    namespace Graph
    {
        /// Work item of a task: enqueue onto the context's stream, return a sushi_cuda status.
        using HostWork = std::function<int(Execution::RuntimeContext&)>;

        /// Epilogue a producer task applies to its output; shared between the recorded closure and
        /// the graph so that a later element-wise task can be folded into the producer.
        struct EpilogueSlot
        {
            int activation = 0;        ///< sushi_cuda_activation_kind value
            float param = 0.0f;        ///< its parameter (leaky_relu slope, elu alpha)
        };

        /// What a producer task writes, for record-time fusion ("TaskMetadata ... for fusers",
        /// reference task_graph.hpp:99-105): `out_count` contiguous elements at `out_ptr`.
        struct FusionInfo
        {
            void* out_ptr = nullptr;
            std::int64_t out_count = 0;
            std::shared_ptr<EpilogueSlot> slot;
        };

        /// A task that is one GEMM and may be batched with its neighbours into a grouped launch:
        /// prepare() stages inputs and fills the descriptor with device addresses, finish() stages
        /// the output back.  Tasks without these run through their HostWork closure alone.
        struct GroupableGemm
        {
            std::function<int(Execution::RuntimeContext&, sushi_cuda_gemm_desc&)> prepare;
            std::function<int(Execution::RuntimeContext&)> finish;
            explicit operator bool() const { return static_cast<bool>(prepare); }
        };

        /// Deferred task list.  add_task() records; execute() replays in order on the stream.
        class TaskGraph
        {
            public:
                explicit TaskGraph(Execution::RuntimeContext& ctx) : ctx_(ctx) {}
                TaskGraph(const TaskGraph&) = delete;
                TaskGraph& operator=(const TaskGraph&) = delete;

                void add_task(const TaskMetadata& meta, const std::vector<void*>& read_access,
                              const std::vector<void*>& write_access, HostWork work, FusionInfo producer = {},
                              GroupableGemm groupable = {})
                {
                    tasks_.push_back(Task{meta, read_access, write_access, std::move(work), std::move(producer),
                                          std::move(groupable)});
                }

                /// Folds an in-place activation over `count` elements at `ptr` into the task recorded
                /// just before it, if that task produces exactly this range and has no activation yet.
                /// Returns true when folded (the caller then records no task of its own).
                bool try_fuse_activation(void* ptr, std::int64_t count, int activation, float param = 0.0f)
                {
                    if (!fusion_enabled_ || tasks_.empty()) return false;
                    FusionInfo& f = tasks_.back().producer;
                    if (!f.slot || f.out_ptr != ptr || f.out_count != count || f.slot->activation != 0) return false;
                    f.slot->activation = activation;
                    f.slot->param = param;
                    ++fused_;
                    return true;
                }

                /// Record-time fusion switch (on by default) and the number of tasks folded so far.
                void set_fusion(bool on) { fusion_enabled_ = on; }
                std::size_t fused_count() const { return fused_; }

                /// Number of tasks recorded and not yet executed.
                std::size_t pending() const { return tasks_.size(); }
                /// Metadata of a pending task (profilers / tests).
                const TaskMetadata& metadata(std::size_t i) const { return tasks_.at(i).meta; }
                const std::vector<void*>& reads(std::size_t i) const { return tasks_.at(i).reads; }
                const std::vector<void*>& writes(std::size_t i) const { return tasks_.at(i).writes; }

                /// Enqueues every pending task; the returned Event completes when the stream drains.
                /// Runs of consecutive small GEMM tasks that do not depend on one another (judged, as
                /// the reference's dependency tracker does, by the base pointers they read and write)
                /// go out as one grouped launch; everything else runs in submission order.
                Execution::Event execute()
                {
                    std::vector<Task> run;
                    run.swap(tasks_);
                    // host images may have been rewritten since the last round: inputs go up again, once
                    ctx_.get_allocator()->begin_round();
                    std::size_t i = 0;
                    while (i < run.size())
                    {
                        std::size_t j = i;
                        if (grouping_enabled_ && run[i].groupable)
                        {
                            std::unordered_set<void*> reads, writes;
                            auto touches = [](const std::unordered_set<void*>& set, const std::vector<void*>& ptrs) {
                                for (void* p : ptrs)
                                    if (set.count(p)) return true;
                                return false;
                            };
                            // grow the run while the next task neither reads nor writes an earlier output
                            // and does not write an earlier input
                            while (j < run.size() && run[j].groupable && !touches(writes, run[j].reads) &&
                                   !touches(writes, run[j].writes) && !touches(reads, run[j].writes))
                            {
                                writes.insert(run[j].writes.begin(), run[j].writes.end());
                                reads.insert(run[j].reads.begin(), run[j].reads.end());
                                ++j;
                            }
                        }
                        if (j - i >= 2)
                        {
                            std::vector<sushi_cuda_gemm_desc> descs(j - i);
                            for (std::size_t t = i; t < j; ++t) check(run[t], run[t].groupable.prepare(ctx_, descs[t - i]));
                            check(run[i], sushi_cuda_sgemm_grouped(ctx_.native_handle(), 0, descs.data(),
                                                                   static_cast<std::int64_t>(descs.size())));
                            for (std::size_t t = i; t < j; ++t) check(run[t], run[t].groupable.finish(ctx_));
                            grouped_ += j - i;
                            i = j;
                        }
                        else
                        {
                            check(run[i], run[i].work(ctx_));
                            ++i;
                        }
                    }
                    return Execution::Event(&ctx_);
                }

                /// Grouped-launch switch (on by default) and the number of tasks sent in groups so far.
                void set_grouping(bool on) { grouping_enabled_ = on; }
                std::size_t grouped_count() const { return grouped_; }

            private:
                struct Task
                {
                    TaskMetadata meta;
                    std::vector<void*> reads, writes;
                    HostWork work;
                    FusionInfo producer;
                    GroupableGemm groupable;
                };
                void check(const Task& t, int rc) const
                {
                    if (rc != SUSHI_CUDA_OK)
                        throw std::runtime_error(std::string(t.meta.name) + ": " + sushi_cuda_last_error(ctx_.native_handle()));
                }
                Execution::RuntimeContext& ctx_;
                std::vector<Task> tasks_;
                bool fusion_enabled_ = true, grouping_enabled_ = true;
                std::size_t fused_ = 0, grouped_ = 0;
        };
    } // namespace Graph
} // namespace SushiRuntime

namespace sr = SushiRuntime;
