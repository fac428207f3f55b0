// Lifecycle shared by all buffers (reference: `csrc/buffers/base.hpp:11-63`).
#pragma once

#include <cstdio>
#include <memory>

#include "../comm/context.hpp"

namespace deep_ep {

class BufferBase {
protected:
    bool explicitly_destroy;
    bool destroyed = false;

    // Called from the destructor of the concrete buffer.
    void destroy_on_destruction(const char* name) {
        if (destroyed) return;
        if (explicitly_destroy) {
            std::fprintf(stderr, "[deep_ep] WARNING: %s buffer released without destroy(); its symmetric memory is "
                                 "freed without a final barrier\n", name);
            release_without_barrier();
        } else {
            // destructors must not throw: a failed final barrier is reported and the memory is released anyway
            try { destroy(); } catch (const std::exception& e) {
                std::fprintf(stderr, "[deep_ep] WARNING: destroying %s buffer failed: %s\n", name, e.what());
            } catch (...) {
                std::fprintf(stderr, "[deep_ep] WARNING: destroying %s buffer failed\n", name);
            }
            if (not destroyed) release_without_barrier();
        }
    }
    virtual void release_without_barrier() {}

public:
    std::shared_ptr<comm::Context> main_context;

    explicit BufferBase(bool explicitly_destroy) : explicitly_destroy(explicitly_destroy) {}
    virtual ~BufferBase() = default;
    virtual void destroy() = 0;

    // Teardown after a failure, in two steps and without the device-side barrier of `destroy()` (a peer may be gone, or
    // the barrier's own state may be what broke): every rank first closes its mappings of the peers' memory, the caller
    // then makes the ranks meet on the host, and only then each rank frees its own allocation with `abort()`.
    void close_peer_mappings() {
        if (main_context != nullptr) main_context->close_peer_mappings();
    }
    void abort() {
        if (not destroyed) release_without_barrier();
        destroyed = true;
    }

    void print_memory_usage() const {
        EP_HOST_ASSERT(main_context != nullptr);
        const auto mib = [](int64_t b) { return static_cast<double>(b) / (1 << 20); };
        std::printf("[deep_ep] rank %d/%d: workspace %.1f MiB, buffer %.1f MiB, storage %.1f MiB\n",
                    main_context->rank_idx, main_context->num_ranks, mib(main_context->num_workspace_bytes),
                    mib(main_context->num_gpu_buffer_bytes), mib(main_context->num_rdma_storage_bytes));
        std::fflush(stdout);
    }
};

}  // namespace deep_ep
