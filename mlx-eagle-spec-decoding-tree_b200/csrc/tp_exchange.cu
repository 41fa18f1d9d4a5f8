// Exchange buffers of the tensor-parallel persistent forward kernel: device memory that the other
// processes of one node map through CUDA IPC, so that a kernel on one GPU can read the fp32 partial
// products and write the flag words of its peers with plain loads and stores over NVLink.
#include <cuda_runtime.h>

#include <cstring>

#include "b200_eagle.h"
#include "common.cuh"
#include "tp_layout.cuh"

namespace b200 {
namespace {

constexpr unsigned kCombineWaitLimit = 1u << 22;     // polls of one flag before giving up

__global__ void __launch_bounds__(32) tp_argmax_combine_kernel(unsigned long long* __restrict__ best_key, int R,
                                                               unsigned index_offset, TpPeers peers, int world, int rank,
                                                               unsigned wait_limit) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ int s_fail;
    unsigned char* own = peers.p[rank];
    const int t = threadIdx.x;
    const unsigned seq = *reinterpret_cast<const volatile unsigned*>(own + kTpKeyCount);
    unsigned long long* slot = reinterpret_cast<unsigned long long*>(own + kTpKeys) + (seq & 1u) * 32;
    if (t == 0) s_fail = 0;
    if (t < R) {
        // low word of a key: 0xffffffff - index, so a larger index is a smaller key
        *reinterpret_cast<volatile unsigned long long*>(slot + t) = best_key[t] - index_offset;
        __threadfence_system();
    }
    __syncthreads();
    if (t < world && t != rank) {
        st_release_sys(reinterpret_cast<unsigned*>(peers.p[t] + kTpKeyFlags + rank * kTpFlagStride), seq + 1);
        const unsigned* flag = reinterpret_cast<const unsigned*>(own + kTpKeyFlags + t * kTpFlagStride);
        bool ok = false;
        for (unsigned i = 0; i < wait_limit; i++) {
            if ((int)(ld_acquire_sys(flag) - (seq + 1)) >= 0) { ok = true; break; }
        }
        if (!ok) s_fail = 1;
    }
    __syncthreads();
    if (s_fail) {                                    // the count stays: the host has to reset the group
        if (t == 0) *reinterpret_cast<volatile int*>(own + kTpKeyErr) = 1;
        return;
    }
    if (t < R) {
        unsigned long long best = 0;
        for (int r = 0; r < world; r++) {
            const unsigned long long* src =
                reinterpret_cast<const unsigned long long*>(peers.p[r] + kTpKeys) + (seq & 1u) * 32 + t;
            unsigned long long v;
            asm volatile("ld.relaxed.sys.global.u64 %0, [%1];\n" : "=l"(v) : "l"(src) : "memory");
            best = v > best ? v : best;
        }
        best_key[t] = best;
    }
    __syncthreads();
    if (t == 0) *reinterpret_cast<volatile unsigned*>(own + kTpKeyCount) = seq + 1;
}

}  // namespace
}  // namespace b200

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

int b200_tp_exchange_error(const void* own_buffer) {
    if (!own_buffer) return B200_EINVAL;
    int v = 0;
    const cudaError_t e = cudaMemcpy(&v, static_cast<const char*>(own_buffer) + b200::kTpKeyErr, sizeof(int),
                                     cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return fail(e);
    return v != 0 ? 1 : 0;
}

int b200_tp_argmax_combine(unsigned long long* best_key, int R, unsigned int index_offset, int tp_world, int tp_rank,
                           void* const* tp_peers, void* stream) {
    if (!best_key || !tp_peers || R < 1 || R > 32 || tp_world < 2 || tp_world > b200::kMaxTp || tp_rank < 0 ||
        tp_rank >= tp_world)
        return B200_EINVAL;
    b200::TpPeers peers{};
    for (int r = 0; r < tp_world; r++) {
        if (!tp_peers[r]) return B200_EINVAL;
        peers.p[r] = static_cast<unsigned char*>(tp_peers[r]);
    }
    b200::launch_kernel(b200::tp_argmax_combine_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream),
                        best_key, R, index_offset, peers, tp_world, tp_rank,
                        b200::g_wait_limit ? b200::g_wait_limit : b200::kCombineWaitLimit);
    return b200::check_launch();
}

int b200_tp_exchange_reset(void* own_buffer, size_t bytes) {
    if (!own_buffer || bytes == 0) return B200_EINVAL;
    cudaError_t e = cudaMemset(own_buffer, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    return e == cudaSuccess ? B200_OK : fail(e);
}

int b200_tp_exchange_free(void* ptr) {
    if (!ptr) return B200_EINVAL;
    const cudaError_t e = cudaFree(ptr);
    return e == cudaSuccess ? B200_OK : fail(e);
}

}  // extern "C"
