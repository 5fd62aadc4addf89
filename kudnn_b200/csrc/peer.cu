// Output buffers that other processes on the same machine can map: the pieces a column-sharded Linear needs to
// write its slab of y straight into every rank's copy of the full tensor (kudnn_b200_linear_set_mirrors) instead of
// gathering afterwards.  A buffer is a plain cudaMalloc allocation plus its CUDA IPC handle; the handle (64 bytes)
// travels to the other ranks by whatever the host program uses (MPI, a torch.distributed all-gather, a pipe), and
// each of them opens it once.  Nothing here launches a kernel or waits on another GPU.
#include "kernels.cuh"

#include <cstring>

static_assert(sizeof(cudaIpcMemHandle_t) == KUDNN_B200_PEER_HANDLE_BYTES, "handle size of the C ABI");

extern "C" {

int kudnn_b200_peer_buffer_create(size_t bytes, void **dev_ptr, unsigned char *handle_out)
{
    if (bytes == 0 || dev_ptr == nullptr || handle_out == nullptr) {
        return kb::set_last_error(KUDNN_B200_BAD_ARGUMENTS, "peer_buffer_create: bad argument");
    }
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return kb::set_last_error(KUDNN_B200_ALLOC_FAILED, "peer_buffer_create: cudaMalloc failed");
    }
    cudaIpcMemHandle_t hnd;
    e = cudaIpcGetMemHandle(&hnd, p);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        cudaFree(p);
        return kb::set_last_error(KUDNN_B200_CUDA_ERROR, "peer_buffer_create: cudaIpcGetMemHandle failed");
    }
    std::memcpy(handle_out, &hnd, sizeof(hnd));
    *dev_ptr = p;
    return KUDNN_B200_OK;
}

int kudnn_b200_peer_buffer_open(const unsigned char *handle, void **dev_ptr)
{
    if (handle == nullptr || dev_ptr == nullptr) {
        return kb::set_last_error(KUDNN_B200_BAD_ARGUMENTS, "peer_buffer_open: bad argument");
    }
    cudaIpcMemHandle_t hnd;
    std::memcpy(&hnd, handle, sizeof(hnd));
    void *p = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&p, hnd, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        (void)cudaGetLastError();
        return kb::set_last_error(KUDNN_B200_CUDA_ERROR,
                                  "peer_buffer_open: cudaIpcOpenMemHandle failed (same process, or no peer access?)");
    }
    *dev_ptr = p;
    return KUDNN_B200_OK;
}

int kudnn_b200_peer_buffer_close(void *dev_ptr)
{
    if (dev_ptr == nullptr) {
        return KUDNN_B200_OK;
    }
    if (cudaIpcCloseMemHandle(dev_ptr) != cudaSuccess) {
        (void)cudaGetLastError();
        return kb::set_last_error(KUDNN_B200_CUDA_ERROR, "peer_buffer_close: cudaIpcCloseMemHandle failed");
    }
    return KUDNN_B200_OK;
}

int kudnn_b200_peer_buffer_destroy(void *dev_ptr)
{
    if (dev_ptr == nullptr) {
        return KUDNN_B200_OK;
    }
    if (cudaFree(dev_ptr) != cudaSuccess) {
        (void)cudaGetLastError();
        return kb::set_last_error(KUDNN_B200_CUDA_ERROR, "peer_buffer_destroy: cudaFree failed");
    }
    return KUDNN_B200_OK;
}

}  // extern "C"
