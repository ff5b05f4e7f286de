#include "runtime.h"

#include <cstring>
#include <stdexcept>

namespace tmoe {

namespace {
void check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string("teramoe_b200 runtime: ") + what + ": " + cudaGetErrorString(e));
}
}  // namespace

SymmetricArena::SymmetricArena(int rank, int world, size_t bytes) : rank_(rank), world_(world), bytes_(bytes) {
    if (rank < 0 || rank >= world) throw std::invalid_argument("teramoe_b200 runtime: rank out of range");
    if (bytes == 0 || bytes % 128 != 0) throw std::invalid_argument("teramoe_b200 runtime: arena size must be a positive multiple of 128");
    check(cudaGetDevice(&device_), "cudaGetDevice");
    check(cudaMalloc(&local_, bytes_), "cudaMalloc(arena)");
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
    cudaIpcMemHandle_t h;
    check(cudaIpcGetMemHandle(&h, local_), "cudaIpcGetMemHandle");
    return std::string(reinterpret_cast<const char*>(&h), sizeof(h));
}

void SymmetricArena::open_peers(const std::vector<std::string>& handles) {
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
    if (local_ != nullptr) cudaFree(local_);
    local_ = nullptr;
    cudaSetDevice(cur);
}

}  // namespace tmoe
