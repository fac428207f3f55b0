// Run-time shape specialisation of the four expert-parallel kernels (the way the reference instantiates every kernel with
// its shapes as template constants, `csrc/kernels/ep/dispatch.hpp:52-81`, `csrc/kernels/ep/combine.hpp:85-112`).
// On the first call with a new (kernel, ranks, top-k, hidden bytes, experts) combination a three-line translation unit
// that instantiates the kernel body template with those constants is compiled by `jit::Compiler` (nvcc -> cubin -> disk
// cache -> driver module) and the launchers of `launch.cu` use the resulting function from then on. The ahead-of-time
// kernels remain the fallback: without a compiler, on a compile error or with the switch off nothing changes.
// Switch: `EP_JIT_SPECIALIZE=1` in the environment or `_C.set_jit_specialization(True)`.
#pragma once

#include <algorithm>
#include <cstdio>
#include <map>
#include <mutex>
#include <sstream>
#include <string>

#include "../kernels/api.hpp"
#include "jit.hpp"

namespace deep_ep::jit {

class Specializer {
    std::map<std::string, void*> functions;       // key -> CUfunction, nullptr = tried and failed
    std::mutex mutex;
    bool enabled = get_env_flag("SPECIALIZE");

    struct KernelInfo {
        const char* header;
        const char* args_type;
        const char* body;
        const char* launch_bounds;
        bool with_experts;
    };

    static const KernelInfo* info(const std::string& kernel) {
        static const std::map<std::string, KernelInfo> table = {
            {"dispatch", {"ep_dispatch.cuh", "DispatchArgs", "ep_dispatch_body", "32 * 9, 1", true}},
            {"expand", {"ep_expand.cuh", "ExpandArgs", "ep_dispatch_expand_body", "32 * 8, 1", true}},
            {"combine", {"ep_combine.cuh", "CombineArgs", "ep_combine_body", "32 * 8, 1", false}},
            {"reduce", {"ep_combine.cuh", "CombineReduceArgs", "ep_combine_reduce_body", "32 * 8", true}},
        };
        const auto it = table.find(kernel);
        return it == table.end() ? nullptr : &it->second;
    }

public:
    static Specializer& get() {
        static Specializer instance;
        return instance;
    }

    bool set_enabled(bool value) { std::swap(value, enabled); return value; }
    bool get_enabled() const { return enabled; }

    static std::string source(const std::string& kernel, const launch::EPShape& shape) {
        const auto* k = info(kernel);
        EP_HOST_ASSERT_MSG(k != nullptr, "unknown kernel " + kernel);
        std::ostringstream out;
        // the reduce epilogue has two register budgets (see ep_combine.cuh): three CTAs per SM, or two for its few-rows variant
        const bool few_rows = std::min(shape.num_topk, shape.num_ranks) <= 2;
        const std::string bounds = kernel == "reduce" ? (few_rows ? "32 * 8, 2" : "32 * 8, 3") : k->launch_bounds;
        out << "#include <deep_ep/kernels/" << k->header << ">\n"
            << "extern \"C\" __global__ void __launch_bounds__(" << bounds << ") ep_specialized(\n"
            << "        const __grid_constant__ deep_ep::kernels::" << k->args_type << " a) {\n"
            << "    deep_ep::kernels::" << k->body << "<" << shape.num_ranks << ", " << shape.num_topk << ", " << shape.hidden_bytes;
        if (k->with_experts) out << ", " << shape.num_experts;
        // the reduce body also takes "a token has at most two partials" (see ep_combine.cuh)
        if (kernel == "reduce") out << ", " << (few_rows ? "true" : "false");
        out << ">(a);\n}\n";
        return out.str();
    }

    // The specialised function for this kernel and shape, or nullptr (switch off, no compiler, compile error).
    void* lookup(const char* kernel, const launch::EPShape& shape) {
        if (not enabled or Compiler::get().get_package_dir().empty()) return nullptr;
        std::ostringstream key;
        key << kernel << "_r" << shape.num_ranks << "_k" << shape.num_topk << "_h" << shape.hidden_bytes << "_e" << shape.num_experts;
        std::lock_guard<std::mutex> guard(mutex);
        const auto it = functions.find(key.str());
        if (it != functions.end()) return it->second;
        void* fn = nullptr;
        try {
            const auto cubin = Compiler::get().compile("ep_" + key.str(), source(kernel, shape));
            fn = reinterpret_cast<void*>(Compiler::get().load(cubin, "ep_specialized"));
        } catch (const std::exception& e) {
            std::fprintf(stderr, "[deep_ep jit] no specialised %s kernel, using the generic one: %s\n", key.str().c_str(), e.what());
        }
        functions[key.str()] = fn;
        return fn;
    }

    void install() {
        launch::set_specialized_kernel_provider([](const char* kernel, const launch::EPShape& shape) {
            return Specializer::get().lookup(kernel, shape);
        });
    }
};

inline void register_specialization_api(pybind11::module_& m) {
    Specializer::get().install();
    m.def("set_jit_specialization", [](bool value) { return Specializer::get().set_enabled(value); },
          "Compile and use shape-specialised EP kernels from the next call on; returns the previous setting");
    m.def("get_jit_specialization", [] { return Specializer::get().get_enabled(); });
    m.def("jit_specialized_source", [](const std::string& kernel, int num_ranks, int num_topk, int hidden_bytes, int num_experts) {
        return Specializer::source(kernel, launch::EPShape{num_ranks, num_topk, hidden_bytes, num_experts});
    });
}

}  // namespace deep_ep::jit
