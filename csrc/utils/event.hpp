// `EventHandle`: an event recorded on the current (or a given) CUDA stream at construction
// (reference: `csrc/utils/event.hpp:10-25`). Without a GPU it degrades to a no-op so that the
// Python layer can be exercised on CPU.
#pragma once

#include <ATen/cuda/CUDAEvent.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include <memory>

namespace deep_ep {

struct EventHandle {
    std::shared_ptr<at::cuda::CUDAEvent> event;

    EventHandle() {
        if (torch::cuda::is_available()) {
            event = std::make_shared<at::cuda::CUDAEvent>(cudaEventDisableTiming);
            event->record(c10::cuda::getCurrentCUDAStream());
        }
    }
    explicit EventHandle(const c10::cuda::CUDAStream& stream) {
        event = std::make_shared<at::cuda::CUDAEvent>(cudaEventDisableTiming);
        event->record(stream);
    }

    void current_stream_wait() const {
        if (event != nullptr) event->block(c10::cuda::getCurrentCUDAStream());
    }
    void stream_wait(const c10::cuda::CUDAStream& stream) const {
        if (event != nullptr) event->block(stream);
    }
};

}  // namespace deep_ep
