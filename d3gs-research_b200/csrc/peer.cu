// Buffers that the other ranks of a node can map, for the data-parallel update over NVLink peer memory.
//
// The reference trains on one GPU and has nothing of the kind.  One process per GPU: each rank allocates
// its flat gradient and parameter buffers here, sends the handles to the other ranks through the
// process group, and maps theirs.  Mapping a peer's buffer turns on peer access to its device
// (cudaIpcMemLazyEnablePeerAccess), after which kernels read and write it with ordinary loads and stores.
#include <cstring>

#include "common.cuh"

using namespace d3gs;

static_assert(sizeof(cudaIpcMemHandle_t) == D3GS_PEER_HANDLE_BYTES, "handle size");

extern "C" int32_t d3gs_peer_buffer_create(int64_t bytes, void** ptr, void* handle) {
    D3GS_REQUIRE(bytes > 0 && ptr != nullptr && handle != nullptr, "bad argument");
    void* p = nullptr;
    D3GS_CUDA(cudaMalloc(&p, (size_t)bytes));
    cudaError_t e = cudaMemset(p, 0, (size_t)bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    cudaIpcMemHandle_t h;
    if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
    if (e != cudaSuccess) {
        cudaFree(p);
        D3GS_CUDA(e);
    }
    memcpy(handle, &h, sizeof(h));
    *ptr = p;
    return D3GS_OK;
}

extern "C" int32_t d3gs_peer_buffer_open(const void* handle, void** ptr) {
    D3GS_REQUIRE(ptr != nullptr && handle != nullptr, "bad argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    D3GS_CUDA(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *ptr = p;
    return D3GS_OK;
}

extern "C" int32_t d3gs_peer_buffer_close(void* ptr) {
    D3GS_REQUIRE(ptr != nullptr, "NULL pointer");
    D3GS_CUDA(cudaIpcCloseMemHandle(ptr));
    return D3GS_OK;
}

extern "C" int32_t d3gs_peer_buffer_destroy(void* ptr) {
    D3GS_REQUIRE(ptr != nullptr, "NULL pointer");
    D3GS_CUDA(cudaFree(ptr));
    return D3GS_OK;
}
