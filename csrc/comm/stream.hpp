// The process-wide high-priority communication stream and a stream-to-stream wait
// (reference: `csrc/comm/stream.hpp:7-27`).
#pragma once

#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAStream.h>

namespace deep_ep::comm {

inline c10::cuda::CUDAStream get_comm_stream() {
    static c10::cuda::CUDAStream stream = c10::cuda::getStreamFromPool(/*isHighPriority=*/true);
    return stream;
}

// Make `waiter` wait for everything currently enqueued on `target`.
inline void stream_wait(const c10::cuda::CUDAStream& waiter, const c10::cuda::CUDAStream& target) {
    at::cuda::CUDAEvent event(cudaEventDisableTiming);
    event.record(target);
    event.block(waiter);
}

}  // namespace deep_ep::comm
