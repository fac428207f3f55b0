// Optional second route to a symmetric allocation: CUDA virtual memory management instead of `cudaMalloc` + CUDA IPC.
// It exists for one reason: only memory created with `cuMemCreate` can be bound to an NVLink multicast object, which
// is what `multimem.*` instructions (one store reaching every GPU through the switch, loads reduced inside the switch)
// need. Pieces:
//   * `FdServer` / `receive_fds`: file descriptors of exported handles travel between the processes of one node over
//     an abstract-namespace unix socket (SCM_RIGHTS); the socket's name goes through the process group like an IPC handle.
//   * `VmmAllocation`: the local physical allocation, mapped and zero-filled.
//   * `VmmPeerMapping`: a peer's allocation imported from its descriptor and mapped into this process.
//   * `MulticastObject`: created by rank 0, imported by the others, every rank adds its device, binds its allocation and
//     maps the object: stores to that mapping land in all GPUs.
// The reference reaches peers through its own registered-memory service (`csrc/kernels/comm/hccl.hpp:72-77,173-194`);
// it has no multicast.
#pragma once

#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include <deep_ep/common/exception.hpp>

#include "../runtime/driver.hpp"

namespace deep_ep::comm {

namespace vmm_detail {

inline sockaddr_un abstract_address(const std::string& name, socklen_t& len) {
    sockaddr_un addr;
    std::memset(&addr, 0, sizeof(addr));
    addr.sun_family = AF_UNIX;
    EP_HOST_ASSERT(name.size() + 1 < sizeof(addr.sun_path));
    std::memcpy(addr.sun_path + 1, name.data(), name.size());          // leading NUL: abstract namespace, no file
    len = static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + name.size());
    return addr;
}

inline CUdevice current_device() {
    CUdevice dev;
    DRV_CHECK(driver::cuCtxGetDevice()(&dev));
    return dev;
}

inline CUmemAccessDesc read_write_access(CUdevice dev) {
    CUmemAccessDesc access;
    std::memset(&access, 0, sizeof(access));
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE, access.location.id = dev;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    return access;
}

}  // namespace vmm_detail

// Hands a fixed set of file descriptors to `num_clients` connecting processes, from a background thread.
class FdServer {
    int listen_fd = -1;
    std::vector<int> fds;
    std::thread worker;
    std::atomic<bool> stop{false};

    void serve(int num_clients, int timeout_secs) {
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(timeout_secs);
        for (int served = 0; served < num_clients and not stop.load();) {
            pollfd p = {listen_fd, POLLIN, 0};
            if (::poll(&p, 1, 100) <= 0) {
                if (std::chrono::steady_clock::now() > deadline) return;
                continue;
            }
            const int conn = ::accept(listen_fd, nullptr, nullptr);
            if (conn < 0) continue;
            // only processes of the same user may receive the descriptors
            ucred cred;
            socklen_t cred_len = sizeof(cred);
            if (::getsockopt(conn, SOL_SOCKET, SO_PEERCRED, &cred, &cred_len) != 0 or cred.uid != ::geteuid()) {
                ::close(conn);
                continue;
            }
            // one byte of payload carries the descriptors as ancillary data
            char payload = static_cast<char>(fds.size());
            iovec iov = {&payload, 1};
            std::vector<char> control(CMSG_SPACE(sizeof(int) * fds.size()), 0);
            msghdr msg;
            std::memset(&msg, 0, sizeof(msg));
            msg.msg_iov = &iov, msg.msg_iovlen = 1;
            msg.msg_control = control.data(), msg.msg_controllen = control.size();
            cmsghdr* cmsg = CMSG_FIRSTHDR(&msg);
            cmsg->cmsg_level = SOL_SOCKET, cmsg->cmsg_type = SCM_RIGHTS;
            cmsg->cmsg_len = CMSG_LEN(sizeof(int) * fds.size());
            std::memcpy(CMSG_DATA(cmsg), fds.data(), sizeof(int) * fds.size());
            if (::sendmsg(conn, &msg, 0) == 1) ++served;
            ::close(conn);
        }
    }

public:
    std::string name;

    FdServer(const std::vector<int>& fds, int num_clients, int timeout_secs = 300) : fds(fds) {
        static std::atomic<int> counter{0};
        name = "deep_ep." + std::to_string(::getpid()) + "." + std::to_string(counter.fetch_add(1)) + "." +
               std::to_string(std::chrono::steady_clock::now().time_since_epoch().count());
        listen_fd = ::socket(AF_UNIX, SOCK_STREAM, 0);
        EP_HOST_ASSERT(listen_fd >= 0);
        socklen_t len;
        const auto addr = vmm_detail::abstract_address(name, len);
        EP_HOST_ASSERT_MSG(::bind(listen_fd, reinterpret_cast<const sockaddr*>(&addr), len) == 0, "cannot bind the descriptor socket");
        EP_HOST_ASSERT(::listen(listen_fd, 64) == 0);
        worker = std::thread([this, num_clients, timeout_secs] { serve(num_clients, timeout_secs); });
    }
    FdServer(const FdServer&) = delete;
    ~FdServer() {
        stop.store(true);
        if (worker.joinable()) worker.join();
        if (listen_fd >= 0) ::close(listen_fd);
    }
};

// Connects to a peer's `FdServer` (retrying until it is up) and returns the descriptors it hands out.
inline std::vector<int> receive_fds(const std::string& name, int num_fds, int timeout_secs = 300) {
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::seconds(timeout_secs);
    socklen_t len;
    const auto addr = vmm_detail::abstract_address(name, len);
    while (true) {
        const int fd = ::socket(AF_UNIX, SOCK_STREAM, 0);
        EP_HOST_ASSERT(fd >= 0);
        if (::connect(fd, reinterpret_cast<const sockaddr*>(&addr), len) == 0) {
            char payload = 0;
            iovec iov = {&payload, 1};
            std::vector<char> control(CMSG_SPACE(sizeof(int) * num_fds), 0);
            msghdr msg;
            std::memset(&msg, 0, sizeof(msg));
            msg.msg_iov = &iov, msg.msg_iovlen = 1;
            msg.msg_control = control.data(), msg.msg_controllen = control.size();
            const auto got = ::recvmsg(fd, &msg, 0);
            ::close(fd);
            cmsghdr* cmsg = CMSG_FIRSTHDR(&msg);
            EP_HOST_ASSERT_MSG(got == 1 and cmsg != nullptr and cmsg->cmsg_level == SOL_SOCKET and cmsg->cmsg_type == SCM_RIGHTS and
                               cmsg->cmsg_len == CMSG_LEN(sizeof(int) * num_fds),
                               "a peer sent an unexpected number of descriptors");
            std::vector<int> out(num_fds);
            std::memcpy(out.data(), CMSG_DATA(cmsg), sizeof(int) * num_fds);
            return out;
        }
        ::close(fd);
        EP_HOST_ASSERT_MSG(std::chrono::steady_clock::now() < deadline, "timed out connecting to a peer's descriptor socket");
        std::this_thread::sleep_for(std::chrono::milliseconds(10));
    }
}

// Granularity that satisfies both the allocator and, when multicast is wanted, the switch.
inline size_t vmm_granularity(int num_devices, bool with_multicast) {
    CUmemAllocationProp prop;
    std::memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE, prop.location.id = vmm_detail::current_device();
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t gran = 0;
    DRV_CHECK(driver::cuMemGetAllocationGranularity()(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
    if (with_multicast) {
        CUmulticastObjectProp mc;
        std::memset(&mc, 0, sizeof(mc));
        mc.numDevices = static_cast<unsigned>(num_devices), mc.size = gran;
        mc.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        size_t mc_gran = 0;
        DRV_CHECK(driver::cuMulticastGetGranularity()(&mc_gran, &mc, CU_MULTICAST_GRANULARITY_RECOMMENDED));
        gran = std::max(gran, mc_gran);
    }
    return gran;
}

inline bool multicast_supported() {
    int value = 0;
    DRV_CHECK(driver::cuDeviceGetAttribute()(&value, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, vmm_detail::current_device()));
    return value != 0;
}

// Local physical allocation: created, exported as a descriptor, mapped read-write, zero-filled.
class VmmAllocation {
public:
    CUmemGenericAllocationHandle handle = 0;
    CUdeviceptr va = 0;
    size_t size = 0;
    int fd = -1;

    VmmAllocation(size_t num_bytes, size_t granularity) {
        size = (num_bytes + granularity - 1) / granularity * granularity;
        const CUdevice dev = vmm_detail::current_device();
        CUmemAllocationProp prop;
        std::memset(&prop, 0, sizeof(prop));
        prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE, prop.location.id = dev;
        prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        try {
            DRV_CHECK(driver::cuMemCreate()(&handle, size, &prop, 0));
            DRV_CHECK(driver::cuMemAddressReserve()(&va, size, granularity, 0, 0));
            DRV_CHECK(driver::cuMemMap()(va, size, 0, handle, 0));
            mapped = true;
            const auto access = vmm_detail::read_write_access(dev);
            DRV_CHECK(driver::cuMemSetAccess()(va, size, &access, 1));
            CUDA_CHECK(cudaMemset(reinterpret_cast<void*>(va), 0, size));
            CUDA_CHECK(cudaDeviceSynchronize());
            DRV_CHECK(driver::cuMemExportToShareableHandle()(&fd, handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
        } catch (...) {
            release();          // a constructor that throws runs no destructor
            throw;
        }
    }
    VmmAllocation(const VmmAllocation&) = delete;
    ~VmmAllocation() { release(); }

private:
    bool mapped = false;

    void release() {
        if (fd >= 0) ::close(fd), fd = -1;
        if (va != 0) {
            if (mapped) driver::cuMemUnmap()(va, size);
            driver::cuMemAddressFree()(va, size);
            va = 0, mapped = false;
        }
        if (handle != 0) driver::cuMemRelease()(handle), handle = 0;
    }
};

// A peer's allocation (or a multicast object) imported from a descriptor and mapped into this process.
class VmmPeerMapping {
public:
    CUmemGenericAllocationHandle handle = 0;
    CUdeviceptr va = 0;
    size_t size = 0;
    bool mapped = false;

    // takes ownership of `fd` (closed after the import, also when the import fails)
    VmmPeerMapping(int fd, size_t size, size_t granularity, bool map_now = true) : size(size) {
        const auto result = driver::cuMemImportFromShareableHandle()(&handle, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)),
                                                                     CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
        ::close(fd);
        DRV_CHECK(result);
        if (not map_now) return;
        try {
            map(granularity);
        } catch (...) {
            driver::cuMemRelease()(handle);
            handle = 0;
            throw;
        }
    }
    // wraps a handle this process created itself (rank 0's multicast object)
    VmmPeerMapping(CUmemGenericAllocationHandle own_handle, size_t size) : handle(own_handle), size(size) {}
    VmmPeerMapping(const VmmPeerMapping&) = delete;

    void map(size_t granularity) {
        EP_HOST_ASSERT(va == 0);
        DRV_CHECK(driver::cuMemAddressReserve()(&va, size, granularity, 0, 0));
        try {
            DRV_CHECK(driver::cuMemMap()(va, size, 0, handle, 0));
            mapped = true;
            const auto access = vmm_detail::read_write_access(vmm_detail::current_device());
            DRV_CHECK(driver::cuMemSetAccess()(va, size, &access, 1));
        } catch (...) {
            unmap();
            throw;
        }
    }

    void unmap() {
        if (va == 0) return;
        if (mapped) driver::cuMemUnmap()(va, size);
        driver::cuMemAddressFree()(va, size);
        va = 0, mapped = false;
    }

    ~VmmPeerMapping() {
        unmap();
        if (handle != 0) driver::cuMemRelease()(handle);
    }
};

// Creates (rank 0) the multicast object of a group of `num_devices` GPUs; the descriptor is in `fd` until it is closed.
inline CUmemGenericAllocationHandle create_multicast_object(int num_devices, size_t size, int& fd) {
    CUmulticastObjectProp prop;
    std::memset(&prop, 0, sizeof(prop));
    prop.numDevices = static_cast<unsigned>(num_devices), prop.size = size;
    prop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    CUmemGenericAllocationHandle handle = 0;
    DRV_CHECK(driver::cuMulticastCreate()(&handle, &prop));
    DRV_CHECK(driver::cuMemExportToShareableHandle()(&fd, handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
    return handle;
}

}  // namespace deep_ep::comm
