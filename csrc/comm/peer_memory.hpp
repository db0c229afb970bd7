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

#include <cerrno>
#include <cstdint>
#include <cstring>
#include <fstream>
#include <stdexcept>
#include <string>

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <sys/syscall.h>
#include <unistd.h>

#include <cuda_runtime.h>

namespace bep {

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
    char bdf[32] = {0};
    if (cudaDeviceGetPCIBusId(bdf, sizeof(bdf), device) != cudaSuccess) return -1;
    for (char* p = bdf; *p; ++p) *p = static_cast<char>(std::tolower(*p));
    std::ifstream file(std::string("/sys/bus/pci/devices/") + bdf + "/numa_node");
    int node = -1;
    if (!(file >> node)) return -1;
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

// Owner side: map, bind to the GPU's NUMA node when the kernel allows it, first-touch by zeroing.
// Returns whether the NUMA bind succeeded (it is advisory; containers often refuse it).
inline bool first_touch_host_segment(const std::string& path, std::size_t bytes, int numa_node) {
    const int fd = ::open(path.c_str(), O_RDWR);
    if (fd < 0) throw std::runtime_error("open(" + path + "): " + std::strerror(errno));
    void* host = ::mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    ::close(fd);
    if (host == MAP_FAILED) throw std::runtime_error("mmap(" + path + "): " + std::strerror(errno));
    bool bound = false;
#ifdef SYS_mbind
    if (numa_node >= 0 && numa_node < 64) {
        unsigned long nodemask = 1ul << numa_node;
        bound = ::syscall(SYS_mbind, host, bytes, 2 /* MPOL_BIND */, &nodemask, 65ul, 0u) == 0;
    }
#endif
    std::memset(host, 0, bytes);
    ::munmap(host, bytes);
    return bound;
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
