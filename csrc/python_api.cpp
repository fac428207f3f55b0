// pybind11 module `deep_ep._C`: registers the host runtime (buffers, contexts, events, barrier,
// runtime knobs, sizing helpers). Counterpart of the reference's `csrc/python_api.cpp:18-74`.
#include <pybind11/functional.h>
#include <pybind11/stl.h>
#include <torch/extension.h>

#include "buffers/bucket.hpp"
#include "buffers/engram.hpp"
#include "buffers/ep.hpp"
#include "buffers/pp.hpp"
#include "comm/barrier.hpp"
#include "comm/stream.hpp"
#include "runtime/device.hpp"
#include "runtime/jit.hpp"
#include "utils/event.hpp"

namespace py = pybind11;
using namespace deep_ep;

namespace {

// The reference compares a device-side call against a host wait that runs out; this is the hook
// the failure-detection test uses: a bounded wait on a flag nobody sets, then the status check.
void run_bounded_wait_probe(comm::Context& context, double timeout_secs) {
    EP_HOST_ASSERT(context.common_signals != nullptr and context.host_status_device != nullptr);
    const cudaStream_t stream = c10::cuda::getCurrentCUDAStream().stream();
    launch::bounded_wait_probe(context.common_signals, context.host_status_device,
                               static_cast<long long>(timeout_secs * 1e9), stream);
    CUDA_CHECK(cudaStreamSynchronize(stream));
}

void clear_status(comm::Context& context) {
    CUDA_CHECK(cudaDeviceSynchronize());
    if (context.host_status != nullptr) context.host_status->code = 0;
    if (context.common_signals != nullptr) CUDA_CHECK(cudaMemset(&context.common_signals->status, 0, sizeof(int)));
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "deep_ep native runtime for NVIDIA B200 (sm_100a)";
    py::register_exception<EPException>(m, "EPException", PyExc_RuntimeError);

    m.attr("topk_idx_t") = py::reinterpret_borrow<py::object>(
        reinterpret_cast<PyObject*>(torch::getTHPDtype(c10::ScalarType::Long)));
    m.def("get_num_allocation_alignment", [] { return kNumAllocationAlignmentBytes; });
    m.def("get_num_rdma_alignment", [] { return kNumRDMAAlignmentBytes; });
    m.def("get_num_tma_alignment", [] { return kNumTMAAlignmentBytes; });
    m.attr("MAX_RANKS") = kMaxRanks;
    m.attr("MAX_BUCKETS") = kMaxBuckets;
    m.attr("MAX_CONTEXTS") = kMaxContexts;

    // runtime knobs
    m.def("get_num_sms", [] { return Runtime::get().get_num_sms(); });
    m.def("set_num_sms", [](int n) { Runtime::get().set_num_sms(n); });
    m.def("get_num_device_sms", [] { return Runtime::get().get_num_device_sms(); });
    m.def("get_arch", [] { return Runtime::get().get_arch(); });
    m.def("set_arch", [](const std::string& a) { Runtime::get().set_arch(a); });
    m.def("set_barrier_in_prologue", [](bool v) { return Runtime::get().set_barrier_in_prologue(v); });
    m.def("get_barrier_in_prologue", [] { return Runtime::get().get_barrier_in_prologue(); });
    jit::register_python_api(m);

    py::class_<EventHandle>(m, "EventHandle")
        .def(py::init<>())
        .def("current_stream_wait", &EventHandle::current_stream_wait);

    py::class_<comm::Context, std::shared_ptr<comm::Context>>(m, "Context")
        .def_readonly("rank_idx", &comm::Context::rank_idx)
        .def_readonly("num_ranks", &comm::Context::num_ranks)
        .def_readonly("context_idx", &comm::Context::context_idx)
        .def_readonly("num_workspace_bytes", &comm::Context::num_workspace_bytes)
        .def_readonly("num_gpu_buffer_bytes", &comm::Context::num_gpu_buffer_bytes)
        .def_readonly("num_rdma_storage_bytes", &comm::Context::num_rdma_storage_bytes)
        .def_readonly("peers_ready", &comm::Context::peers_ready)
        .def("get_local_handle", [](const comm::Context& c) { return py::bytes(c.get_local_handle()); })
        .def("set_peer_handles", [](comm::Context& c, const std::vector<py::bytes>& handles) {
            std::vector<std::string> raw;
            for (const auto& h : handles) raw.emplace_back(static_cast<std::string>(h));
            c.set_peer_handles(raw);
        })
        .def("get_physical_domain_size", &comm::Context::get_physical_domain_size)
        .def("get_logical_domain_size", &comm::Context::get_logical_domain_size)
        .def("check_status", &comm::Context::check_status)
        .def("status_code", [](const comm::Context& c) { return c.host_status ? static_cast<int>(c.host_status->code) : 0; })
        .def("clear_status", &clear_status)
        .def("bounded_wait_probe", &run_bounded_wait_probe);

    m.def("barrier", [](comm::Context& context, bool with_cpu_sync, bool sequential, bool wait_comm_stream) {
        comm::barrier(context, with_cpu_sync, sequential, wait_comm_stream);
    }, py::arg("context"), py::arg("with_cpu_sync") = false, py::arg("sequential") = true, py::arg("wait_comm_stream") = true);
    m.def("get_comm_stream", [] {
        const auto s = comm::get_comm_stream();
        return py::make_tuple(s.id(), static_cast<int>(s.device_index()), static_cast<int>(s.device_type()));
    });
    m.def("check_peer_access", [](int device, int peer) {
        int ok = 0;
        CUDA_CHECK(cudaDeviceCanAccessPeer(&ok, device, peer));
        return ok != 0;
    });

    py::class_<BufferBase, std::shared_ptr<BufferBase>>(m, "BufferBase")
        .def_readonly("main_context", &BufferBase::main_context)
        .def("print_memory_usage", &BufferBase::print_memory_usage)
        .def("destroy", &BufferBase::destroy);

    py::class_<EPBuffer, BufferBase, std::shared_ptr<EPBuffer>>(m, "EPBuffer")
        .def(py::init<int, int, const std::string&, int64_t, int64_t, bool, int, int, bool>())
        .def_readonly("context", &EPBuffer::context)
        .def_readonly("lb_storage", &EPBuffer::lb_storage)
        .def("dispatch", &EPBuffer::dispatch)
        .def("combine", &EPBuffer::combine)
        .def("check_status", &EPBuffer::check_status);
    m.def("calculate_ep_buffer_size", &EPBuffer::calculate_buffer_size);

    py::class_<PPBuffer, BufferBase, std::shared_ptr<PPBuffer>>(m, "PPBuffer")
        .def(py::init<int, int, const std::string&, int64_t, int, bool, int, bool>())
        .def_readonly("context", &PPBuffer::context)
        .def_readonly("storage", &PPBuffer::storage)
        .def("send", &PPBuffer::send)
        .def("recv", &PPBuffer::recv);

    py::class_<EngramBuffer, BufferBase, std::shared_ptr<EngramBuffer>>(m, "EngramBuffer")
        .def(py::init<int, int, const std::string&, int64_t, int64_t, bool, int, bool>())
        .def_readonly("context", &EngramBuffer::context)
        .def("set_config", &EngramBuffer::set_config)
        .def("write", &EngramBuffer::write)
        .def("fetch", &EngramBuffer::fetch);

    py::class_<BucketBuffer, BufferBase, std::shared_ptr<BucketBuffer>>(m, "BucketBuffer")
        .def(py::init<const std::vector<int>&, const std::vector<int>&, const std::vector<std::string>&, int64_t, bool, int, bool>())
        .def_readonly("contexts", &BucketBuffer::contexts)
        .def_readonly("storage", &BucketBuffer::storage)
        .def("all_gather", &BucketBuffer::all_gather);
}
