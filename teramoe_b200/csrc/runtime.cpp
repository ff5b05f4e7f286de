#include "runtime.h"

#include <cuda.h>
#include <unistd.h>

#include <cstring>
#include <stdexcept>

namespace tmoe {

namespace {
void check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("teramoe_b200 runtime: ") + what + ": " + cudaGetErrorString(e));
}

// The virtual-memory-management calls of the driver, looked up through the runtime (no link against libcuda).
struct VmmApi {
    CUresult (*get_granularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
    CUresult (*create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
    CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
    CUresult (*reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
    CUresult (*address_free)(CUdeviceptr, size_t) = nullptr;
    CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
    CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*set_access)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
    CUresult (*export_handle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
    CUresult (*import_handle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
    bool ok = false;
};

template <class F>
bool lookup(const char* name, F& fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) return false;
    fn = reinterpret_cast<F>(p);
    return true;
}

const VmmApi& vmm_api() {
    static VmmApi api = [] {
        VmmApi a;
        a.ok = lookup("cuMemGetAllocationGranularity", a.get_granularity) && lookup("cuMemCreate", a.create) &&
               lookup("cuMemRelease", a.release) && lookup("cuMemAddressReserve", a.reserve) &&
               lookup("cuMemAddressFree", a.address_free) && lookup("cuMemMap", a.map) && lookup("cuMemUnmap", a.unmap) &&
               lookup("cuMemSetAccess", a.set_access) && lookup("cuMemExportToShareableHandle", a.export_handle) &&
               lookup("cuMemImportFromShareableHandle", a.import_handle);
        return a;
    }();
    if (!api.ok) throw std::runtime_error("teramoe_b200 runtime: the driver's virtual memory management entry points were not found");
    return api;
}

void check_drv(CUresult r, const char* what) {
    if (r != CUDA_SUCCESS) throw std::runtime_error(std::string("teramoe_b200 runtime: ") + what + " failed with CUresult " + std::to_string((int)r));
}

CUmemAccessDesc rw_access(int device) {
    CUmemAccessDesc d{};
    d.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    d.location.id = device;
    d.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    return d;
}
}  // namespace

SymmetricArena::SymmetricArena(int rank, int world, size_t bytes, bool vmm, bool fabric)
    : rank_(rank), world_(world), bytes_(bytes), vmm_(vmm) {
    if (rank < 0 || rank >= world) throw std::invalid_argument("teramoe_b200 runtime: rank out of range");
    if (bytes == 0 || bytes % 128 != 0) throw std::invalid_argument("teramoe_b200 runtime: arena size must be a positive multiple of 128");
    check(cudaGetDevice(&device_), "cudaGetDevice");
    if (vmm_) {
        check(cudaFree(nullptr), "context creation");
        const VmmApi& api = vmm_api();
        CUmemAllocationProp prop{};
        prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
        prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
        prop.location.id = device_;
        prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        size_t gran = 0;
        check_drv(api.get_granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
        if (gran == 0) gran = 2u << 20;
        mapped_bytes_ = (bytes_ + gran - 1) / gran * gran;
        CUmemGenericAllocationHandle h = 0;
        CUresult r = CUDA_ERROR_NOT_SUPPORTED;
        if (fabric) {
            // a fabric handle next to the descriptor where the platform offers one (multi-node NVLink domains)
            CUmemAllocationProp both = prop;
            both.requestedHandleTypes = (CUmemAllocationHandleType)(CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR | CU_MEM_HANDLE_TYPE_FABRIC);
            r = api.create(&h, mapped_bytes_, &both, 0);
            fabric_ok_ = (r == CUDA_SUCCESS);
        }
        if (r != CUDA_SUCCESS) check_drv(api.create(&h, mapped_bytes_, &prop, 0), "cuMemCreate");
        handle_ = h;
        CUdeviceptr ptr = 0;
        r = api.reserve(&ptr, mapped_bytes_, gran, 0, 0);
        if (r != CUDA_SUCCESS) {
            api.release(h);
            check_drv(r, "cuMemAddressReserve");
        }
        r = api.map(ptr, mapped_bytes_, 0, h, 0);
        if (r == CUDA_SUCCESS) {
            const CUmemAccessDesc acc = rw_access(device_);
            r = api.set_access(ptr, mapped_bytes_, &acc, 1);
            if (r != CUDA_SUCCESS) api.unmap(ptr, mapped_bytes_);
        }
        if (r != CUDA_SUCCESS) {
            api.address_free(ptr, mapped_bytes_);
            api.release(h);
            check_drv(r, "cuMemMap / cuMemSetAccess");
        }
        local_ = reinterpret_cast<void*>(ptr);
    } else {
        check(cudaMalloc(&local_, bytes_), "cudaMalloc(arena)");
    }
    check(cudaMemset(local_, 0, bytes_), "cudaMemset(arena)");
    check(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    peers_.assign(world_, 0);
    peers_[rank_] = reinterpret_cast<uint64_t>(local_);
}

SymmetricArena::~SymmetricArena() {
    try {
        close();
    } catch (...) {
    }
}

std::string SymmetricArena::export_handle() const {
    if (vmm_) throw std::runtime_error("teramoe_b200 runtime: a vmm arena is shared through export_fd / open_peer_fds");
    cudaIpcMemHandle_t h;
    check(cudaIpcGetMemHandle(&h, local_), "cudaIpcGetMemHandle");
    return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
}

int SymmetricArena::export_fd() {
    if (!vmm_) throw std::runtime_error("teramoe_b200 runtime: only vmm arenas have a file descriptor");
    if (export_fd_ < 0) {
        int fd = -1;
        check_drv(vmm_api().export_handle(&fd, handle_, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
        export_fd_ = fd;
    }
    return export_fd_;
}

void SymmetricArena::open_peer_fds(const std::vector<int>& fds) {
    if (!vmm_) throw std::runtime_error("teramoe_b200 runtime: only vmm arenas open file descriptors");
    if ((int)fds.size() != world_) throw std::invalid_argument("teramoe_b200 runtime: need one descriptor per rank");
    if (open_) throw std::runtime_error("teramoe_b200 runtime: peers already open");
    const VmmApi& api = vmm_api();
    const CUmemAccessDesc acc = rw_access(device_);
    std::string error;
    for (int r = 0; r < world_; ++r) {
        if (r == rank_) continue;
        if (fds[r] < 0) {
            error = "negative descriptor for rank " + std::to_string(r);
            continue;
        }
        if (error.empty()) {
            // every rank allocates the same size with the same granularity, so the peer's mapping has our extent
            CUmemGenericAllocationHandle h = 0;
            CUresult res = api.import_handle(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fds[r])), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
            CUdeviceptr ptr = 0;
            if (res == CUDA_SUCCESS) {
                res = api.reserve(&ptr, mapped_bytes_, 0, 0, 0);
                if (res == CUDA_SUCCESS) {
                    res = api.map(ptr, mapped_bytes_, 0, h, 0);
                    if (res == CUDA_SUCCESS) {
                        res = api.set_access(ptr, mapped_bytes_, &acc, 1);
                        if (res != CUDA_SUCCESS) api.unmap(ptr, mapped_bytes_);
                    }
                    if (res != CUDA_SUCCESS) api.address_free(ptr, mapped_bytes_);
                }
                if (res != CUDA_SUCCESS) api.release(h);
            }
            if (res == CUDA_SUCCESS) {
                vmm_opened_.push_back({h, (unsigned long long)ptr, mapped_bytes_});
                peers_[r] = (uint64_t)ptr;
            } else {
                error = "mapping the allocation of rank " + std::to_string(r) + " failed with CUresult " + std::to_string((int)res);
            }
        }
        ::close(fds[r]);          // the import holds its own reference
    }
    if (!error.empty()) throw std::runtime_error("teramoe_b200 runtime: " + error);
    open_ = true;
}

void SymmetricArena::open_peers(const std::vector<std::string>& handles) {
    if (vmm_) throw std::runtime_error("teramoe_b200 runtime: a vmm arena is shared through export_fd / open_peer_fds");
    if ((int)handles.size() != world_) throw std::invalid_argument("teramoe_b200 runtime: need one handle per rank");
    if (open_) throw std::runtime_error("teramoe_b200 runtime: peers already open");
    for (int r = 0; r < world_; ++r) {
        if (r == rank_) continue;
        if (handles[r].size() != sizeof(cudaIpcMemHandle_t)) throw std::invalid_argument("teramoe_b200 runtime: malformed IPC handle");
        cudaIpcMemHandle_t h;
        std::memcpy(&h, handles[r].data(), sizeof(h));
        void* p = nullptr;
        check(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
        ipc_opened_.push_back(p);
        peers_[r] = reinterpret_cast<uint64_t>(p);
    }
    open_ = true;
}

void SymmetricArena::adopt_peer_pointers(const std::vector<uint64_t>& ptrs) {
    if ((int)ptrs.size() != world_) throw std::invalid_argument("teramoe_b200 runtime: need one pointer per rank");
    if (ptrs[rank_] != reinterpret_cast<uint64_t>(local_)) throw std::invalid_argument("teramoe_b200 runtime: own pointer mismatch");
    peers_ = ptrs;
    open_ = true;
}

void SymmetricArena::close() {
    if (closed_) return;
    closed_ = true;
    int cur = 0;
    cudaGetDevice(&cur);
    cudaSetDevice(device_);
    cudaDeviceSynchronize();
    for (void* p : ipc_opened_) cudaIpcCloseMemHandle(p);
    ipc_opened_.clear();
    if (vmm_) {
        const VmmApi& api = vmm_api();
        for (const PeerMap& m : vmm_opened_) {
            api.unmap((CUdeviceptr)m.ptr, m.bytes);
            api.address_free((CUdeviceptr)m.ptr, m.bytes);
            api.release((CUmemGenericAllocationHandle)m.handle);
        }
        vmm_opened_.clear();
        if (export_fd_ >= 0) ::close(export_fd_);
        export_fd_ = -1;
        if (local_ != nullptr) {
            api.unmap(reinterpret_cast<CUdeviceptr>(local_), mapped_bytes_);
            api.address_free(reinterpret_cast<CUdeviceptr>(local_), mapped_bytes_);
            api.release((CUmemGenericAllocationHandle)handle_);
        }
    } else if (local_ != nullptr) {
        cudaFree(local_);
    }
    local_ = nullptr;
    cudaSetDevice(cur);
}

}  // namespace tmoe
