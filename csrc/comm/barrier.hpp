// Host entry of the cross-rank barrier (reference: `csrc/comm/barrier.hpp:9-33`): optionally join
// the communication stream before and after, launch the one-warp barrier kernel on the current
// stream, optionally wait on the host and surface device-side failures.
#pragma once

#include <c10/cuda/CUDAStream.h>

#include "../kernels/api.hpp"
#include "context.hpp"
#include "stream.hpp"

namespace deep_ep::comm {

inline void barrier(Context& context, bool with_cpu_sync = false, bool sequential = true, bool wait_comm_stream = true,
                    int repeats = 1) {
    (void) sequential;   // accepted for API parity; the kernel is always a single ordered barrier
    EP_HOST_ASSERT(context.peers_ready and context.common_signals != nullptr);
    const auto stream = c10::cuda::getCurrentCUDAStream();
    if (wait_comm_stream) stream_wait(stream, get_comm_stream());
    EP_HOST_ASSERT(repeats >= 1);
    kernels::BarrierArgs args = {context.common_signals, context.host_status_device, context.peers, context.num_gpu_timeout_ns, repeats};
    launch::barrier(args, stream);
    if (wait_comm_stream) stream_wait(get_comm_stream(), stream);
    if (with_cpu_sync) {
        CUDA_CHECK(cudaStreamSynchronize(stream));
        context.check_status();
    }
}

}  // namespace deep_ep::comm
