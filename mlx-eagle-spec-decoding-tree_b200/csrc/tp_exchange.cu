// Exchange buffers of the tensor-parallel persistent forward kernel: device memory that the other
// processes of one node map through CUDA IPC, so that a kernel on one GPU can read the fp32 partial
// products and write the flag words of its peers with plain loads and stores over NVLink.
#include <cuda_runtime.h>

#include <cstring>

#include "b200_eagle.h"
#include "common.cuh"

namespace {
int fail(cudaError_t e) {
    b200::g_last_cuda_error = (int)e;
    cudaGetLastError();            // clear the sticky-free error state
    return B200_ECUDA;
}
}  // namespace

extern "C" {

int b200_tp_exchange_alloc(size_t bytes, void** ptr, unsigned char* handle) {
    static_assert(sizeof(cudaIpcMemHandle_t) == B200_TP_HANDLE_BYTES, "handle size");
    if (!ptr || !handle || bytes == 0) return B200_EINVAL;
    void* q = nullptr;
    cudaError_t e = cudaMalloc(&q, bytes);
    if (e != cudaSuccess) return fail(e);
    cudaIpcMemHandle_t h;
    if ((e = cudaMemset(q, 0, bytes)) != cudaSuccess || (e = cudaDeviceSynchronize()) != cudaSuccess ||
        (e = cudaIpcGetMemHandle(&h, q)) != cudaSuccess) {
        cudaFree(q);
        return fail(e);
    }
    std::memcpy(handle, &h, sizeof(h));
    *ptr = q;
    return B200_OK;
}

int b200_tp_exchange_open(const unsigned char* handle, void** ptr) {
    if (!ptr || !handle) return B200_EINVAL;
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    void* q = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&q, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) return fail(e);
    *ptr = q;
    return B200_OK;
}

int b200_tp_exchange_close(void* ptr) {
    if (!ptr) return B200_EINVAL;
    const cudaError_t e = cudaIpcCloseMemHandle(ptr);
    return e == cudaSuccess ? B200_OK : fail(e);
}

int b200_tp_exchange_free(void* ptr) {
    if (!ptr) return B200_EINVAL;
    const cudaError_t e = cudaFree(ptr);
    return e == cudaSuccess ? B200_OK : fail(e);
}

}  // extern "C"
