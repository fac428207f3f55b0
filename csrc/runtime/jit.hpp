// Runtime kernel specialisation (the role DeepJIT plays for the reference, `csrc/runtime/jit.hpp:15-118`):
// generate a small translation unit that instantiates a kernel template with compile-time constants,
// compile it with nvcc for sm_100a into a cubin, cache it on disk by content hash, load it through
// the driver API and launch it. The ahead-of-time kernels linked into this extension remain the
// default path; the JIT is for specialisations chosen at run time.
#pragma once

#include <cuda.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <filesystem>
#include <fstream>
#include <functional>
#include <map>
#include <mutex>
#include <sstream>
#include <fcntl.h>
#include <spawn.h>
#include <sys/wait.h>
#include <unistd.h>
#include <cerrno>
#include <string>
#include <vector>

#include <deep_ep/common/exception.hpp>

#include "driver.hpp"

extern char** environ;

namespace deep_ep::jit {

// `EP_JIT_<NAME>` with `DJ_JIT_<NAME>` as fallback (the reference's environment contract).
inline std::string get_env(const std::string& name, const std::string& fallback = "") {
    for (const char* prefix : {"EP_JIT_", "DJ_JIT_"}) {
        const char* v = std::getenv((std::string(prefix) + name).c_str());
        if (v != nullptr and *v != '\0') return v;
    }
    return fallback;
}
inline bool get_env_flag(const std::string& name) {
    const auto v = get_env(name, "0");
    return v != "0" and v != "false" and v != "False";
}

inline uint64_t fnv1a(const std::string& s, uint64_t h = 1469598103934665603ull) {
    for (const unsigned char c : s) h = (h ^ c) * 1099511628211ull;
    return h;
}

// Runs `argv` (argv[0] = program path, looked up in PATH when it has no slash) as a child process, standard output and
// error appended to `log_path`; returns the exit code, or -1 when the process could not be started or was killed.
inline int run_process(const std::vector<std::string>& argv_text, const std::string& log_path, const std::string& working_dir = "") {
    std::vector<char*> argv;
    for (const auto& word : argv_text) argv.push_back(const_cast<char*>(word.c_str()));
    argv.push_back(nullptr);
    posix_spawn_file_actions_t actions;
    posix_spawn_file_actions_init(&actions);
    posix_spawn_file_actions_addopen(&actions, 1, log_path.c_str(), O_WRONLY | O_CREAT | O_TRUNC, 0644);
    posix_spawn_file_actions_adddup2(&actions, 1, 2);
    if (not working_dir.empty()) posix_spawn_file_actions_addchdir_np(&actions, working_dir.c_str());
    pid_t pid = 0;
    const int err = posix_spawnp(&pid, argv[0], &actions, nullptr, argv.data(), environ);
    posix_spawn_file_actions_destroy(&actions);
    if (err != 0) return -1;
    int status = 0;
    while (waitpid(pid, &status, 0) < 0)
        if (errno != EINTR) return -1;
    return WIFEXITED(status) ? WEXITSTATUS(status) : -1;
}

class Compiler {
    std::string package_dir;
    std::map<std::string, CUfunction> loaded;     // cache key -> function
    std::vector<CUmodule> modules;
    std::mutex mutex;

    // `EP_JIT_CACHE_DIR` may name several roots separated by colons: all are searched in order, misses are compiled
    // into the first (a read-only cache shipped with an image can sit behind a writable one).
    std::vector<std::string> cache_roots() const {
        auto dirs = get_env("CACHE_DIR");
        if (dirs.empty()) {
            const char* home = std::getenv("HOME");
            dirs = std::string(home != nullptr ? home : "/tmp") + "/.deep_ep_b200/cache";
        }
        std::vector<std::string> roots;
        std::stringstream stream(dirs);
        for (std::string item; std::getline(stream, item, ':');)
            if (not item.empty()) roots.push_back(item);
        EP_HOST_ASSERT_MSG(not roots.empty(), "EP_JIT_CACHE_DIR names no directory");
        std::filesystem::create_directories(roots.front());
        return roots;
    }

public:
    static Compiler& get() {
        static Compiler instance;
        return instance;
    }

    void init(const std::string& dir) { package_dir = dir; }
    const std::string& get_package_dir() const { return package_dir; }
    std::vector<std::string> get_cache_roots() const { return cache_roots(); }
    std::string include_dir() const { return package_dir + "/include"; }

    std::string nvcc_path() const {
        auto p = get_env("NVCC");
        if (not p.empty()) return p;
        const char* home = std::getenv("CUDA_HOME");
        return std::string(home != nullptr ? home : "/usr/local/cuda") + "/bin/nvcc";
    }

    // Compile `source` (a full translation unit) to a cubin; returns the cubin path. Cached by hash
    // of source + flags + arch.
    std::string compile(const std::string& name, const std::string& source, const std::string& arch = "sm_100a") {
        EP_HOST_ASSERT_MSG(not package_dir.empty(), "init_jit(package_dir) has not been called");
        std::string flags = "-std=c++20 -O3 --expt-relaxed-constexpr -cubin";
        if (get_env_flag("KERNEL_DEBUG_INFO")) flags += " -lineinfo";
        // EP_DEBUG=1: bounds-checked build of the kernels (every remote message store is checked against its landing area)
        if (const char* debug = std::getenv("EP_DEBUG"); debug != nullptr and std::string(debug) == "1") flags += " -DEP_DEBUG";
        const std::string arch_num = arch.substr(3);
        flags += " -gencode arch=compute_" + arch_num + ",code=" + arch;
        std::ostringstream key;
        key << std::hex << fnv1a(source, fnv1a(flags + " -I" + include_dir()));
        const auto roots = cache_roots();
        const auto entry = name + "-" + key.str();
        for (const auto& root : roots) {
            const auto hit = root + "/" + entry + "/kernel.cubin";
            std::error_code ignored;
            if (std::filesystem::exists(hit, ignored)) return hit;
        }
        const auto dir = roots.front() + "/" + entry;
        const auto cubin = dir + "/kernel.cubin";
        std::filesystem::create_directories(dir);
        const auto tmp = cubin + ".tmp." + std::to_string(::getpid());
        {
            // several ranks may compile the same entry at once: the source is published with a rename, so a compiler that
            // another rank has already started never reads a half-written file
            const auto source_tmp = dir + "/kernel.cu.tmp." + std::to_string(::getpid());
            {
                std::ofstream out(source_tmp);
                out << source;
            }
            std::filesystem::rename(source_tmp, dir + "/kernel.cu");
        }
        // the compiler runs as a child process with an argument vector (no shell: paths from the environment may hold
        // spaces or shell metacharacters), its output goes to `nvcc.log`. It runs INSIDE the entry's directory and is given
        // file names only, because nvcc passes the paths it receives on to its own sub-commands through a shell.
        std::vector<std::string> argv_text = {nvcc_path()};
        {
            std::stringstream words(flags);
            for (std::string word; words >> word;) argv_text.push_back(word);
        }
        argv_text.push_back("-I" + include_dir());
        argv_text.push_back("kernel.cu");
        argv_text.push_back("-o");
        argv_text.push_back(std::filesystem::path(tmp).filename().string());
        if (get_env_flag("PRINT_COMPILER_COMMAND") or get_env_flag("DEBUG")) {
            std::string line;
            for (const auto& word : argv_text) line += word + " ";
            std::fprintf(stderr, "[deep_ep jit] %s\n", line.c_str());
        }
        const int rc = run_process(argv_text, dir + "/nvcc.log", dir);
        if (rc != 0) {
            std::ifstream log(dir + "/nvcc.log");
            std::stringstream text;
            text << log.rdbuf();
            throw EPException("JIT compile", __FILE__, __LINE__, name + ": nvcc failed (" + std::to_string(rc) + ")\n" + text.str());
        }
        std::filesystem::rename(tmp, cubin);     // atomic publish: concurrent ranks may race on the same key
        return cubin;
    }

    // Load (once) and return the kernel `symbol` of a compiled cubin.
    CUfunction load(const std::string& cubin, const std::string& symbol) {
        std::lock_guard<std::mutex> guard(mutex);
        const auto key = cubin + "::" + symbol;
        auto it = loaded.find(key);
        if (it != loaded.end()) return it->second;
        CUmodule module;
        const auto t0 = std::chrono::steady_clock::now();
        DRV_CHECK(driver::cuModuleLoad()(&module, cubin.c_str()));
        if (get_env_flag("PRINT_LOAD_TIME") or get_env_flag("DEBUG")) {
            const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
            std::fprintf(stderr, "[deep_ep jit] loaded %s in %.2f ms\n", cubin.c_str(), ms);
        }
        modules.push_back(module);
        CUfunction fn;
        DRV_CHECK(driver::cuModuleGetFunction()(&fn, module, symbol.c_str()));
        loaded[key] = fn;
        return fn;
    }

    void launch(CUfunction fn, int grid, int block, int smem_bytes, CUstream stream, std::vector<void*>& args, bool cooperative = false) {
        if (smem_bytes > 48 * 1024)
            DRV_CHECK(driver::cuFuncSetAttribute()(fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, smem_bytes));
        CUlaunchConfig config = {};
        config.gridDimX = grid, config.gridDimY = 1, config.gridDimZ = 1;
        config.blockDimX = block, config.blockDimY = 1, config.blockDimZ = 1;
        config.sharedMemBytes = smem_bytes, config.hStream = stream;
        CUlaunchAttribute attr[1];
        attr[0].id = CU_LAUNCH_ATTRIBUTE_COOPERATIVE, attr[0].value.cooperative = cooperative ? 1 : 0;
        config.attrs = attr, config.numAttrs = 1;
        DRV_CHECK(driver::cuLaunchKernelEx()(&config, fn, args.data(), nullptr));
    }
};

inline void register_python_api(pybind11::module_& m) {
    m.def("init_jit", [](const std::string& package_dir) { Compiler::get().init(package_dir); });
    m.def("jit_compile", [](const std::string& name, const std::string& source, const std::string& arch) {
        return Compiler::get().compile(name, source, arch);
    }, pybind11::arg("name"), pybind11::arg("source"), pybind11::arg("arch") = "sm_100a");
    m.def("jit_include_dir", [] { return Compiler::get().include_dir(); });
    m.def("jit_cache_roots", [] { return Compiler::get().get_cache_roots(); });
    // `EP_JIT_LAUNCH_TIMEOUT` (seconds, default 300, 0 = none) is read for compatibility with the reference's launcher.
    // CUDA has no per-launch execution limit: what bounds a kernel here is the buffer's `num_gpu_timeout_secs`, after
    // which every device-side wait gives up and reports through the status word.
    m.def("jit_launch_timeout_secs", [] { return std::atoi(get_env("LAUNCH_TIMEOUT", "300").c_str()); });
    // Launch `symbol` of a compiled cubin on the current CUDA stream. Each argument is a `(kind, value)` pair with
    // kind in {"ptr", "i64", "i32", "f32"}; pointers are raw device addresses.
    m.def("jit_launch", [](const std::string& cubin, const std::string& symbol, int grid, int block, int smem_bytes,
                           const std::vector<std::pair<std::string, pybind11::object>>& args, bool cooperative,
                           uint64_t stream) {
        std::vector<uint64_t> storage(args.size(), 0);
        std::vector<void*> pointers(args.size(), nullptr);
        for (size_t i = 0; i < args.size(); ++i) {
            const auto& [kind, value] = args[i];
            if (kind == "ptr" or kind == "i64") storage[i] = static_cast<uint64_t>(value.cast<int64_t>());
            else if (kind == "i32") { const int32_t v = value.cast<int32_t>(); std::memcpy(&storage[i], &v, 4); }
            else if (kind == "f32") { const float v = value.cast<float>(); std::memcpy(&storage[i], &v, 4); }
            else throw EPException("JIT launch", __FILE__, __LINE__, "unknown argument kind " + kind);
            pointers[i] = &storage[i];
        }
        auto fn = Compiler::get().load(cubin, symbol);
        Compiler::get().launch(fn, grid, block, smem_bytes, reinterpret_cast<CUstream>(stream), pointers, cooperative);
    }, pybind11::arg("cubin"), pybind11::arg("symbol"), pybind11::arg("grid"), pybind11::arg("block"),
       pybind11::arg("smem_bytes"), pybind11::arg("args"), pybind11::arg("cooperative") = false, pybind11::arg("stream") = 0);
}

}  // namespace deep_ep::jit
