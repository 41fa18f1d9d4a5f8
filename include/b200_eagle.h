/*
 * C ABI of libb200eagle.so: the B200 (sm_100a) kernels of the tree speculative
 * decoding path.  Plain pointers and sizes only; every pointer is a DEVICE
 * pointer unless stated otherwise, every call is asynchronous on `stream`
 * (a cudaStream_t passed as void*), never allocates device memory (except where a
 * function says so), never prints and never aborts.
 *
 * Return value: 0 on success, a negative B200_E* code otherwise (nothing was
 * launched in that case).  Launch failures reported by the CUDA runtime come
 * back as B200_ECUDA; b200_last_cuda_error() gives the runtime's code.
 *
 * File/line citations name the reference interface each entry point replaces
 * (paths inside 0seba/mlx-eagle-spec-decoding-tree).
 */
#ifndef B200_EAGLE_H
#define B200_EAGLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_OK 0
#define B200_EINVAL (-1)      /* bad shape / size / flag combination            */
#define B200_EALIGN (-2)      /* a pointer is not 16-byte aligned               */
#define B200_EUNSUPPORTED (-3) /* dtype / group size / bits not implemented      */
#define B200_EWORKSPACE (-4)  /* workspace too small for the requested launch   */
#define B200_ECUDA (-5)       /* CUDA runtime error; see b200_last_cuda_error() */

#define B200_DTYPE_F16 0

/* Epilogue selector of b200_qmm_fused. */
#define B200_EPI_NONE 0      /* y = fp16(acc) [+ bias, in fp16]                               */
#define B200_EPI_RESIDUAL 1  /* y = fp16(residual + fp16(acc))       (mlx_llama.py:246,248)  */
#define B200_EPI_SILU_MUL 2  /* y = silu(fp16(acc_gate)) * fp16(acc_up), two weight sets     */
                             /*                                       (mlx_llama.py:215)      */

int b200_version(void);
int b200_last_cuda_error(void);

/* Bytes of scratch b200_qmm / b200_qmm_fused want for a given problem (split-K partial sums and
 * tile counters).  0 means the problem runs without scratch. */
size_t b200_qmm_workspace_bytes(int M, int N, int K);

/*
 * Batched 4-bit affine quantised matmul  y[M,N] = x[M,K] . dequant(W[N,K])^T (+ bias[N]).
 * Replaces qmm_kernel.py:84-164 `matmul(x, w, s, b, group_size)` as bound at
 * mlx_eagle.py:704-708 and called from mlx_model_fwd_bench.py:69 (rows 8/16/24/32), and the
 * mx.quantized_matmul fallback for other row counts (mlx_model_fwd_bench.py:73).
 *   x        [M,K]   fp16, row-major                       M >= 1 (rows beyond 32 are processed
 *                                                          in passes of 32)
 *   wq       [N,K/8] uint32, element j of a pack in bits 4j..4j+3 (MLX layout)
 *   scales, biases [N,K/64] fp16;  group_size must be 64, K % 128 == 0, N % 8 == 0
 *   bias     [N] fp16 or NULL: added after the fp16 rounding of the product
 *            (mlx_model_fwd_bench.py:70-71)
 *   y        [M,N]   fp16
 *   workspace / workspace_bytes: scratch from b200_qmm_workspace_bytes (may be NULL/0: the
 *            kernel then runs without split-K).  The first 4 KiB must be zero before the first
 *            use; the library restores that state itself after every launch.  Launches
 *            sharing one workspace must be stream-ordered.
 */
int b200_qmm(const void* x, const uint32_t* wq, const void* scales, const void* biases,
             const void* bias, void* y, int M, int N, int K, int group_size, int dtype,
             void* workspace, size_t workspace_bytes, void* stream);

/*
 * Same product with a fused epilogue (the element-wise op that follows the linear layer in
 * mlx_llama.py:215,246,248).  For B200_EPI_SILU_MUL, (wq, scales, biases) is gate_proj and
 * (wq2, scales2, biases2) is up_proj, both [N,K]; `extra` is unused.  For B200_EPI_RESIDUAL,
 * `extra` is the residual [M,N] fp16 (may alias y).  M <= 32.
 */
int b200_qmm_fused(const void* x, const uint32_t* wq, const void* scales, const void* biases,
                   const uint32_t* wq2, const void* scales2, const void* biases2,
                   const void* bias, const void* extra, void* y, int M, int N, int K,
                   int group_size, int dtype, int epilogue,
                   void* workspace, size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_EAGLE_H */
