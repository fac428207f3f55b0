// Host-side error handling (reference: `common/exception.hpp:14-82`). Device code never traps:
// it records a status code and returns, and the host turns that code into an `EPException`.
#pragma once

#include <sstream>
#include <stdexcept>
#include <string>

namespace deep_ep {

class EPException : public std::runtime_error {
    static std::string format(const char* kind, const char* file, int line, const std::string& what) {
        std::ostringstream os;
        os << kind << " failed (" << file << ":" << line << "): " << what;
        return os.str();
    }

public:
    EPException(const char* kind, const char* file, int line, const std::string& what)
        : std::runtime_error(format(kind, file, line, what)) {}
};

}  // namespace deep_ep

#define EP_HOST_ASSERT(cond)                                                          \
    do {                                                                              \
        if (not(cond)) throw deep_ep::EPException("Assertion", __FILE__, __LINE__, #cond); \
    } while (0)

#define EP_HOST_ASSERT_MSG(cond, msg)                                                 \
    do {                                                                              \
        if (not(cond)) throw deep_ep::EPException("Assertion", __FILE__, __LINE__, std::string(#cond) + ": " + (msg)); \
    } while (0)

#define EP_HOST_UNREACHABLE(msg) throw deep_ep::EPException("Unreachable", __FILE__, __LINE__, msg)

#define CUDA_CHECK(expr)                                                              \
    do {                                                                              \
        cudaError_t e_ = (expr);                                                      \
        if (e_ != cudaSuccess)                                                        \
            throw deep_ep::EPException("CUDA runtime", __FILE__, __LINE__, std::string(#expr) + " -> " + cudaGetErrorString(e_)); \
    } while (0)
