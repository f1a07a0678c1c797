// Peer-visible device memory for the in-kernel tensor-parallel all-reduce.
//
// The reference has nothing of the kind (one GPU).  The exchange needs two small
// buffers per rank that the other ranks' kernels can store into: the tagged residual
// stream and a receive buffer for partial sums (every value carries its own tag, so
// there are no arrival counters).  Ranks are separate processes (one per GPU), so
// the memory is shared with CUDA IPC handles; the 64-byte handle travels through the
// host's own channel.  Host-only code: nothing here launches a kernel.
#include <cuda_runtime.h>

#include <cstring>

#include "../../include/mkb200.h"

namespace mkb {
int set_error(int code, const char* msg);
}

static_assert(sizeof(cudaIpcMemHandle_t) == MKB_PEER_HANDLE_BYTES, "handle size is part of the ABI");

extern "C" int mkb_peer_alloc(size_t bytes, void** device_ptr, unsigned char* handle) {
    if (!device_ptr || !handle || bytes == 0)
        return mkb::set_error(MKB_ERR_INVALID_ARGUMENT, "mkb_peer_alloc: NULL output or zero size");
    void* ptr = nullptr;
    if (cudaMalloc(&ptr, bytes) != cudaSuccess) {
        cudaGetLastError();
        return mkb::set_error(MKB_ERR_CUDA, "mkb_peer_alloc: cudaMalloc failed");
    }
    cudaIpcMemHandle_t h;
    if (cudaMemset(ptr, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
        cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(ptr);
        return mkb::set_error(MKB_ERR_CUDA, "mkb_peer_alloc: cudaIpcGetMemHandle failed");
    }
    memcpy(handle, &h, sizeof(h));
    *device_ptr = ptr;
    return MKB_OK;
}

extern "C" int mkb_peer_open(const unsigned char* handle, void** device_ptr) {
    if (!device_ptr || !handle) return mkb::set_error(MKB_ERR_INVALID_ARGUMENT, "mkb_peer_open: NULL argument");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void* ptr = nullptr;
    if (cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
        cudaGetLastError();
        return mkb::set_error(MKB_ERR_CUDA, "mkb_peer_open: cudaIpcOpenMemHandle failed (no peer access?)");
    }
    *device_ptr = ptr;
    return MKB_OK;
}

extern "C" int mkb_peer_close(void* device_ptr) {
    if (device_ptr && cudaIpcCloseMemHandle(device_ptr) != cudaSuccess) {
        cudaGetLastError();
        return mkb::set_error(MKB_ERR_CUDA, "mkb_peer_close: cudaIpcCloseMemHandle failed");
    }
    return MKB_OK;
}

extern "C" int mkb_peer_free(void* device_ptr) {
    if (device_ptr && cudaFree(device_ptr) != cudaSuccess) {
        cudaGetLastError();
        return mkb::set_error(MKB_ERR_CUDA, "mkb_peer_free: cudaFree failed");
    }
    return MKB_OK;
}
