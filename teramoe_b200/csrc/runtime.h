// Symmetric-memory runtime: one device allocation per rank that every peer of the node maps into its
// own address space, so kernels can store straight into a peer's buffers over NVLink.  Two ways to share it:
//   * CUDA IPC (default): cudaMalloc + a 64-byte handle that travels through the process group;
//   * virtual memory management ("vmm"): cuMemCreate with a shareable POSIX file descriptor, cuMemAddressReserve +
//     cuMemMap + cuMemSetAccess on both sides; the descriptor travels over a Unix socket (parallel/fdpass.py).  This
//     is the allocation kind that multicast objects and fabric handles build on; with `fabric` the allocation also
//     asks for a fabric handle and falls back to the descriptor where the platform has none.
//
// Reference counterparts: shared_memory::SharedMemoryAllocator (csrc/moe_extension.hpp:25-51,
// csrc/moe_extension.cpp:16-125) and the allocate / export / open / close parts of deep_ep::Buffer
// (csrc/moe_extension.cpp:129-229, :291-436).  There is no NVSHMEM or RDMA tier here: all ranks sit
// behind one NVSwitch.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>
#include <vector>

namespace tmoe {

class SymmetricArena {
public:
    SymmetricArena(int rank, int world, size_t bytes, bool vmm = false, bool fabric = false);
    ~SymmetricArena();
    SymmetricArena(const SymmetricArena&) = delete;
    SymmetricArena& operator=(const SymmetricArena&) = delete;

    // 64-byte CUDA IPC handle of the local allocation.
    std::string export_handle() const;
    // Map every peer (handles[rank] is ignored: the local pointer is used).
    void open_peers(const std::vector<std::string>& handles);
    // vmm arenas: a POSIX file descriptor of the local allocation (owned by the arena, closed with it) ...
    int export_fd();
    // ... and the peers' descriptors as received in THIS process (fds[rank] is ignored; the others are closed here).
    void open_peer_fds(const std::vector<int>& fds);
    bool is_vmm() const { return vmm_; }
    bool has_fabric_handle() const { return fabric_ok_; }
    // Several ranks emulated inside one process on one device: peers are plain pointers.
    void adopt_peer_pointers(const std::vector<uint64_t>& ptrs);
    void close();

    uint64_t local_ptr() const { return reinterpret_cast<uint64_t>(local_); }
    const std::vector<uint64_t>& peer_ptrs() const { return peers_; }
    size_t bytes() const { return bytes_; }
    int rank() const { return rank_; }
    int world() const { return world_; }
    bool is_open() const { return open_; }

private:
    int rank_, world_, device_ = 0;
    size_t bytes_;
    void* local_ = nullptr;
    std::vector<uint64_t> peers_;
    std::vector<void*> ipc_opened_;
    bool open_ = false;
    bool closed_ = false;
    // vmm state
    bool vmm_ = false, fabric_ok_ = false;
    size_t mapped_bytes_ = 0;                      // bytes_ rounded up to the allocation granularity
    unsigned long long handle_ = 0;                // CUmemGenericAllocationHandle of the local allocation
    int export_fd_ = -1;
    struct PeerMap { unsigned long long handle; unsigned long long ptr; size_t bytes; };
    std::vector<PeerMap> vmm_opened_;
};

}  // namespace tmoe
