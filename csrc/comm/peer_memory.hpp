// Registration layer: where a rank's symmetric segment lives and how peers reach it.
//
// The reference has one substrate, a /dev/shm file per source that every rank mmaps and registers
// with cudaHostRegister (csrc/comm/advanced_shared_memory.hpp:143-288).  Here that is the fallback
// ("host_staged"); the primary substrate is device memory exported with CUDA IPC and mapped by
// every peer over NVLink ("peer").  Both produce the same thing for the kernels: a table of base
// pointers, one per rank, valid on this rank's GPU.
//
// Handles travel between processes through the caller's control group (gloo); nothing here talks
// to another process.
#pragma once

#include <cctype>
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <cuda_runtime.h>

namespace bep {

inline bool debug_enabled() {
    const char* v = std::getenv("PCIE_EP_B200_DEBUG");
    return v != nullptr && v[0] == '1';
}

inline void cuda_check(cudaError_t status, const char* what) {
    if (status != cudaSuccess) {
        throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(status));
    }
}

// ---- device segments (transport "peer") -------------------------------------------------------

struct DeviceSegment {
    void* ptr = nullptr;
    std::size_t bytes = 0;
};

// cudaMalloc (not the PyTorch caching allocator: an IPC handle names a whole allocation) + zero fill
inline DeviceSegment allocate_device_segment(std::size_t bytes) {
    DeviceSegment seg;
    seg.bytes = bytes;
    cuda_check(cudaMalloc(&seg.ptr, bytes), "cudaMalloc(segment)");
    cuda_check(cudaMemset(seg.ptr, 0, bytes), "cudaMemset(segment)");
    cuda_check(cudaDeviceSynchronize(), "cudaDeviceSynchronize(segment)");
    return seg;
}

inline std::string export_device_segment(void* ptr) {
    cudaIpcMemHandle_t handle;
    cuda_check(cudaIpcGetMemHandle(&handle, ptr), "cudaIpcGetMemHandle");
    return std::string(reinterpret_cast<const char*>(&handle), sizeof(handle));
}

inline void* import_device_segment(const std::string& bytes) {
    if (bytes.size() != sizeof(cudaIpcMemHandle_t)) throw std::runtime_error("malformed IPC handle");
    cudaIpcMemHandle_t handle;
    std::memcpy(&handle, bytes.data(), sizeof(handle));
    void* ptr = nullptr;
    cuda_check(cudaIpcOpenMemHandle(&ptr, handle, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
    return ptr;
}

inline void release_imported_segment(void* ptr) { cuda_check(cudaIpcCloseMemHandle(ptr), "cudaIpcCloseMemHandle"); }
inline void free_device_segment(void* ptr) { cuda_check(cudaFree(ptr), "cudaFree(segment)"); }

// ---- host segments (transport "host_staged") -------------------------------------------------

inline int device_numa_node(int device) {
    char bdf[64] = {0};
    if (cudaDeviceGetPCIBusId(bdf, static_cast<int>(sizeof(bdf)) - 1, device) != cudaSuccess) return -1;
    for (char* p = bdf; *p; ++p) *p = static_cast<char>(std::tolower(static_cast<unsigned char>(*p)));
    if (debug_enabled()) std::fprintf(stderr, "[pcie_ep_b200] device %d is %s\n", device, bdf);
    // C stdio on purpose: this header is compiled by a newer g++ than the libstdc++ some hosts load at
    // run time, and iostream locale machinery is where such a mismatch crashes.
    const std::string path = std::string("/sys/bus/pci/devices/") + bdf + "/numa_node";
    std::FILE* file = std::fopen(path.c_str(), "r");
    if (file == nullptr) return -1;
    int node = -1;
    if (std::fscanf(file, "%d", &node) != 1) node = -1;
    std::fclose(file);
    return node;
}

inline void create_host_segment(const std::string& path, std::size_t bytes) {
    const int fd = ::open(path.c_str(), O_RDWR | O_CREAT | O_EXCL, 0600);
    if (fd < 0) throw std::runtime_error("open(" + path + "): " + std::strerror(errno));
    const int rc = ::ftruncate(fd, static_cast<off_t>(bytes));
    const int saved = errno;
    ::close(fd);
    if (rc != 0) throw std::runtime_error("ftruncate(" + path + "): " + std::strerror(saved));
}

struct HostMapping {
    void* host = nullptr;
    void* device = nullptr;
    std::size_t bytes = 0;
    bool registered = false;
};

inline bool numa_placement_enabled() {
    const char* v = std::getenv("PCIE_EP_B200_NUMA_PLACEMENT");
    return v != nullptr && v[0] == '1';
}

// Owner side: map and first-touch by zeroing, so the pages land on the NUMA node of the touching
// thread (the kernel's default local-allocation policy).  An explicit placement request
// (mbind, MPOL_PREFERRED towards the GPU's node) is made only when PCIE_EP_B200_NUMA_PLACEMENT=1:
// in sandboxed containers the mbind system call can be fatal to the process rather than refused,
// and a library must not take its host down by default.  Returns whether a placement request was
// made and accepted.
inline bool first_touch_host_segment(const std::string& path, std::size_t bytes, int numa_node) {
    const int fd = ::open(path.c_str(), O_RDWR);
    if (fd < 0) throw std::runtime_error("open(" + path + "): " + std::strerror(errno));
    struct stat info {};
    if (::fstat(fd, &info) != 0 || static_cast<std::size_t>(info.st_size) < bytes) {
        ::close(fd);
        throw std::runtime_error("segment file " + path + " is smaller than the segment");
    }
    void* host = ::mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    ::close(fd);
    if (host == MAP_FAILED) throw std::runtime_error("mmap(" + path + "): " + std::strerror(errno));
    bool placed = false;
#ifdef SYS_mbind
    if (numa_placement_enabled() && numa_node >= 0 && numa_node < 64 &&
        ::access(("/sys/devices/system/node/node" + std::to_string(numa_node)).c_str(), F_OK) == 0) {
        unsigned long nodemask[2] = {1ul << numa_node, 0ul};
        placed = ::syscall(SYS_mbind, host, static_cast<unsigned long>(bytes), 1 /* MPOL_PREFERRED */, nodemask,
                           static_cast<unsigned long>(65), static_cast<unsigned long>(0)) == 0;
    }
#endif
    if (debug_enabled()) std::fprintf(stderr, "[pcie_ep_b200] first touch %s bytes=%zu node=%d placed=%d\n", path.c_str(), bytes, numa_node, placed ? 1 : 0);
    std::memset(host, 0, bytes);
    ::munmap(host, bytes);
    return placed;
}

inline HostMapping map_host_segment(const std::string& path, std::size_t bytes) {
    HostMapping m;
    m.bytes = bytes;
    const int fd = ::open(path.c_str(), O_RDWR);
    if (fd < 0) throw std::runtime_error("open(" + path + "): " + std::strerror(errno));
    m.host = ::mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    ::close(fd);
    if (m.host == MAP_FAILED) throw std::runtime_error("mmap(" + path + "): " + std::strerror(errno));
    const cudaError_t status = cudaHostRegister(m.host, bytes, cudaHostRegisterMapped | cudaHostRegisterPortable);
    if (status != cudaSuccess) {
        ::munmap(m.host, bytes);
        throw std::runtime_error(std::string("cudaHostRegister: ") + cudaGetErrorString(status));
    }
    m.registered = true;
    cuda_check(cudaHostGetDevicePointer(&m.device, m.host, 0), "cudaHostGetDevicePointer");
    return m;
}

// Keeps the mapping if unregistering fails: a peer GPU may still be touching it.
inline bool unmap_host_segment(HostMapping& m) {
    if (m.host == nullptr) return true;
    if (m.registered && cudaHostUnregister(m.host) != cudaSuccess) return false;
    m.registered = false;
    ::munmap(m.host, m.bytes);
    m.host = m.device = nullptr;
    return true;
}

// One mapped + registered host segment with RAII-free explicit close (close order is collective
// and decided by the Python layer).
class HostSegment {
   public:
    HostSegment(const std::string& path, std::size_t bytes, int device) {
        int previous = 0;
        cuda_check(cudaGetDevice(&previous), "cudaGetDevice");
        cuda_check(cudaSetDevice(device), "cudaSetDevice");
        try {
            mapping_ = map_host_segment(path, bytes);
        } catch (...) {
            cudaSetDevice(previous);
            throw;
        }
        cudaSetDevice(previous);
    }
    std::int64_t host_pointer() const { return reinterpret_cast<std::int64_t>(mapping_.host); }
    std::int64_t device_pointer() const { return reinterpret_cast<std::int64_t>(mapping_.device); }
    bool close() { return unmap_host_segment(mapping_); }

   private:
    HostMapping mapping_;
};

}  // namespace bep
