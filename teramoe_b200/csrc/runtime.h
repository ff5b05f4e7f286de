// Symmetric-memory runtime: one device allocation per rank that every peer of the node maps into its
// own address space (CUDA IPC), so kernels can store straight into a peer's buffers over NVLink.
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
    SymmetricArena(int rank, int world, size_t bytes);
    ~SymmetricArena();
    SymmetricArena(const SymmetricArena&) = delete;
    SymmetricArena& operator=(const SymmetricArena&) = delete;

    // 64-byte CUDA IPC handle of the local allocation.
    std::string export_handle() const;
    // Map every peer (handles[rank] is ignored: the local pointer is used).
    void open_peers(const std::vector<std::string>& handles);
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
};

}  // namespace tmoe
