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
#define B200_ELIMIT (-6)      /* problem larger than a fixed built-in limit       */

#define B200_DTYPE_F16 0

/* Epilogue selector of b200_qmm_fused. */
#define B200_EPI_NONE 0      /* y = fp16(acc) [+ bias, in fp16]                               */
#define B200_EPI_RESIDUAL 1  /* y = fp16(residual + fp16(acc))       (mlx_llama.py:246,248)  */
#define B200_EPI_SILU_MUL 2  /* y = silu(fp16(acc_gate)) * fp16(acc_up), two weight sets     */
                             /*                                       (mlx_llama.py:215)      */
#define B200_EPI_F32 3       /* b200_qmm_tiled only: y is float [M,N] and receives the fp32     */
                             /* accumulator - the partial product of one K shard of a         */
                             /* row-parallel layer, to be all-reduced across GPUs              */

int b200_version(void);
int b200_last_cuda_error(void);
/* Kernels are launched with programmatic stream serialisation (a kernel may start while its
 * predecessor drains and waits on the device before touching dependent data); 0 turns the launch
 * attribute off (plain stream order).  Process-wide; default on. */
void b200_set_pdl(int enabled);
/* Every device-side wait on another CTA or another GPU (grid barrier and all-GPU barrier of b200_forward,
 * the peer flags of b200_tp_argmax_combine) polls a bounded number of times, then sets an error word the host
 * can read and lets the kernel run to its end.  `polls` replaces the built-in limits (a few seconds) for
 * launches made after the call; 0 restores them.  Process-wide.  Meant for hosts that want a tighter
 * failure-detection time, and for testing the give-up path without a failing peer. */
void b200_set_wait_limit(unsigned int polls);

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

/*
 * b200_qmm for callers that must not allocate.  (No counterpart in the reference: it exists for
 * hosts that embed this library where device allocation is off limits - a serving process whose
 * memory pool is owned by another runtime and handed out in full at start-up, a plug-in loaded into
 * a process that forbids cudaMalloc after initialisation, or code that runs where the CUDA
 * allocator may not be entered.)  Same product and arguments as b200_qmm with at most 32 rows, but
 * the split-K scratch is a fixed 4 MiB array inside the library image instead of a caller buffer:
 * nothing is allocated or freed, by this call or by anything it calls.  Every GPU that loads the
 * library carries those 4 MiB until the process exits.
 *   - Problems whose split-K scratch for the plain product (what b200_qmm itself would use; the
 *     gate/up pair counted by b200_qmm_workspace_bytes does not run here) exceeds
 *     b200_qmm_noalloc_max_scratch_bytes() are refused with B200_ELIMIT; nothing is launched
 *     (e.g. 32 rows x 3584 x 18944 wants 5.3 MiB: use b200_qmm with a caller buffer for those).
 *   - The first call on each device looks up the array's device address (with that device
 *     current); make that first call outside any stream capture, and do not let two host threads
 *     make their first call on the same device at the same time (the cached address is written
 *     without a lock; both would store the same value).
 *   - All calls on a device share the one array and it keeps the previous call's contents; the call
 *     re-zeroes the part that must start at zero.  Two calls that overlap on the GPU (different
 *     streams, no ordering) race on it: order them.
 */
size_t b200_qmm_noalloc_max_scratch_bytes(void);
int b200_qmm_noalloc(const void* x, const uint32_t* wq, const void* scales, const void* biases,
                     const void* bias, void* y, int M, int N, int K, int group_size, int dtype, void* stream);

/*
 * Streaming ("tiled") weight layout and the matmul kernel that reads it.  b200_qmm_relayout is the
 * one-off offline re-layout (counterpart of the reference's swizzle.py:41-57 /
 * kernels/swizzle.metal): records of 16 rows x 128 k = 1152 contiguous bytes, packs in the order the
 * lanes of a warp consume them followed by the {scale, bias} pairs; `out` needs b200_qmm_tiled_bytes.
 * b200_qmm_tiled computes the same product and epilogues as b200_qmm_fused (same arithmetic, same
 * rounding points) from that layout with persistent CTAs and bulk-copy rings; M <= 32, and a
 * workspace of at least b200_qmm_tiled_workspace_bytes is required (first 4 KiB zero before first use;
 * the last int of that block is an error flag set if a bounded wait on a bulk copy ever gives up).
 */
size_t b200_qmm_tiled_bytes(int N, int K);
int b200_qmm_relayout(const uint32_t* wq, const void* scales, const void* biases, void* out, int N, int K,
                      void* stream);
size_t b200_qmm_tiled_workspace_bytes(int M, int N, int K);
int b200_qmm_tiled(const void* x, const void* wt, const void* wt2, const void* bias, const void* extra, void* y,
                   int M, int N, int K, int epilogue, void* workspace, size_t workspace_bytes, void* stream);

/* The same product (plain epilogue: y = fp16(acc) [+ bias, in fp16]) on the tcgen05 tensor cores: sixteen warps
 * expand the packed records (exact q*s+b, rounded once) and write the fp16 weights with tcgen05.st straight into
 * 128-row tiles in tensor memory (the weights never pass through shared memory as fp16), one thread per CTA issues
 * tcgen05.mma (weights from tensor memory, activations read in place from the bulk-copied stage in shared memory)
 * with the accumulator in tensor memory.  Same streaming weight layout; M <= 128 (one weight read serves up to 128
 * token rows: the shape of prompt ingestion), N % 128 == 0, K % 128 == 0.  workspace: b200_qmm_umma_workspace_bytes
 * bytes (the activations in the tensor cores' K-major core-matrix order, written by a relayout kernel that this call
 * launches first, + an error word, int 0 of the workspace, non-zero if a bounded wait gave up; zero it before the
 * first use).  Replaces qmm_kernel.py:79-124 like b200_qmm. */
size_t b200_qmm_umma_workspace_bytes(int M, int K);
int b200_qmm_umma(const void* x, const void* w_tiled, const void* bias, void* y, int M, int N, int K,
                  void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------
 * Per-token model kernels (one decoder layer = rms_norm, qmm(+bias), rope_kv_append,
 * tree_attention, qmm(residual), rms_norm, qmm(silu-mul), qmm(residual)).
 * ------------------------------------------------------------------------------------------ */

/* Quantised embedding lookup, h[m,:] = dequant(E[tokens[m],:]).  Replaces `self.embed_tokens(inputs)`
 * (mlx_llama.py:273) on a 4-bit nn.QuantizedEmbedding.  out [M,H] fp16; H % 64 == 0. */
int b200_embed_gather(const int* tokens, const uint32_t* wq, const void* scales, const void* biases,
                      void* out, int M, int H, int V, void* stream);

/* RMSNorm, y = fp16((x * rsqrt(mean(x^2)+eps)) * w) with fp32 math.  Replaces nn.RMSNorm /
 * mx.fast.rms_norm (mlx_llama.py:225-228,240,247,263,286).  If row_index != NULL (device int),
 * output row i is computed from input row row_index[0] + i (used to pick the catch-up pass row,
 * mlx_eagle.py:404,408). */
int b200_rms_norm(const void* x, const void* w, void* y, const int* row_index, int M, int H, float eps,
                  void* stream);

/* Element-wise halves of the fused matmul epilogues, for prompt ingestion (mlx_eagle.py:522-535), whose matmuls run
 * 128 token rows at a time through b200_qmm_umma (plain epilogue): h = fp16(h + y) (the residual add of
 * mlx_llama.py:246,248) and out = silu(gate) * up with every op result rounded to fp16 (mlx_llama.py:215), the same
 * rounding points as B200_EPI_RESIDUAL / B200_EPI_SILU_MUL.  n = element count, a multiple of 8; fp16 device arrays,
 * 16-byte aligned. */
int b200_add_f16(void* h, const void* y, size_t n, void* stream);
int b200_silu_mul_f16(const void* gate, const void* up, void* out, size_t n, void* stream);

/* Tensor-parallel residual epilogue: h[M,N] = fp16(h + fp16(sum)) with `sum` the all-reduced fp32 partial
 * products of a row-parallel layer (o_proj / down_proj of mlx_llama.py:246,248 sharded along K).  No
 * counterpart in the reference, which runs on one device. */
int b200_residual_add_f32(void* h, const float* sum, int M, int N, void* stream);

/* Tree-position RoPE fused with the KV-cache append.  qkv [M,(Hq+2Hkv)*hd] fp16 holds q|k|v of M
 * tokens; q is rotated in place, k rotated and v copied into cache row prefix[0]+write_off+m of
 * kcache / vcache ([Hkv][cache_rows][hd] fp16 each).  pos[m] is the rotary position of token m.
 * Replaces the two rope_positions calls (mlx_llama.py:150-161), the flat_rope path (:141-143,
 * 162-176) and cache.update_and_fetch (:178). */
int b200_rope_kv_append(void* qkv, const int* pos, const float* inv_freq, float scaling, void* kcache,
                        void* vcache, const int* prefix, int write_off, int M, int Hq, int Hkv, int hd,
                        int cache_rows, void* stream);

/* Stand-alone RoPE with per-(batch, token) integer positions, tensors laid out (B,H,L,D) fp16,
 * offsets (B,L) int32, inv_freqs (D/2) fp32.  Replaces mlx_arrayed_rope_kernel.py:46-152
 * `rope_positions(inp, offsets, inv_freqs, scaling_factor)` (non-traditional layout, forward). */
int b200_rope_positions(const void* in, const int* offsets, const float* inv_freqs, float scaling_factor,
                        void* out, int B, int H, int L, int D, void* stream);

/* Tree-masked attention of M <= 32 query tokens, GQA.  Query m sees every cache row < prefix[0]
 * and cache row prefix[0]+j (j < tail <= 64) iff bit j of mask[m] is set; the new tokens' K/V
 * must already be in the cache.  q points at the rotated queries (token stride q_stride halves),
 * out is [M,Hq*hd] fp16.  max_kv bounds prefix+tail over the lifetime of the workspace (it sizes the
 * grid, so one launch shape serves a growing cache); workspace from
 * b200_tree_attention_workspace_bytes, first 256 bytes zero before first use.  hd in {64,128}.
 * Replaces mx.fast.scaled_dot_product_attention with the additive tree mask
 * (mlx_llama.py:185-192; masks built at mlx_eagle.py:143-146,171,207,336-338). */
size_t b200_tree_attention_workspace_bytes(int M, int Hq, int Hkv, int hd, int max_kv);
int b200_tree_attention(const void* q, int q_stride, const void* kcache, const void* vcache,
                        const unsigned long long* mask, const int* prefix, int tail, void* out,
                        int M, int Hq, int Hkv, int hd, int cache_rows, int max_kv, float scale,
                        void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------------
 * Whole forward pass as one persistent cooperative kernel.
 * Replaces one call of Model.__call__ (mlx_llama.py:298-313: embed_tokens, every TransformerBlock
 * :231-249 with Attention :121-196 and MLP :199-215, the final norm and lm_head / as_linear) for
 * M <= 32 tokens whose ids, rotary positions, tail masks and committed length are in device memory
 * (same meaning as in b200_rope_kv_append / b200_tree_attention).  All linear weights are in the
 * streaming layout of b200_qmm_relayout; the embedding stays in the MLX row-major layout.
 *
 * The descriptor itself is HOST memory (read during the call only); every pointer in it is a device
 * pointer.  layer_table is a device array of n_layers entries of 8 pointers each:
 *   { qkv weights (q|k|v rows concatenated), qkv bias [NQKV] fp16 or NULL, o_proj, gate_proj, up_proj,
 *     down_proj weights, input_layernorm weight [hidden] fp16, post_attention_layernorm weight }.
 * Buffers (all fp16): h [32][hidden]; qkv [32][(n_heads+2*n_kv_heads)*head_dim]; logits [rows_out][vocab];
 * hw, attn, act are scratch the kernel keeps in its own chunk-major padded layout and need
 * (width/128)*32*160 halves each, width = hidden, n_heads*head_dim, intermediate.  kv_cache is
 * [n_layers][2][n_kv_heads][cache_rows][head_dim] fp16; the K/V rows of the M new tokens are written
 * to cache row prefix[0]+write_off+m.  Output row r of logits belongs to token row_index[0]+r
 * (row_index may be NULL = 0).  RMSNorm is folded into the adjacent matmuls (h*w is rounded to fp16,
 * the per-token 1/rms multiplies the fp32 accumulator), which differs from the per-op kernels by
 * input-rounding noise only.
 *
 * workspace: b200_forward_workspace_bytes bytes, the first 4352 bytes zero before the first use (the
 * kernel restores that state).  Int word 2 of the workspace is an error flag: non-zero after a launch
 * means a bounded wait inside the kernel gave up; zero the first 4352 bytes before reusing it.
 * The launch is cooperative (one CTA per SM, all co-resident); launches sharing a workspace must be
 * stream-ordered.  hidden, intermediate and n_heads*head_dim must be multiples of 128, hidden <= 8192,
 * head_dim 64 or 128, tail <= 64, write_off + M <= tail.
 * ------------------------------------------------------------------------------------------ */
typedef struct b200_forward_desc {
    int M, rows_out;
    int hidden, intermediate, n_heads, n_kv_heads, head_dim, vocab, n_layers;
    int cache_rows, write_off, tail;
    float rms_eps, rope_scaling, attn_scale;
    int attn_split_blocks;  /* 0 = default (33): from this many 64-key blocks of cache on, attention splits the  */
                            /* keys across CTAs and merges in a second phase; below, one CTA per (kv head,      */
                            /* query tile) scores the key blocks on its warps side by side.  < 0 = always split  */
    const int* tokens;
    const int* pos;
    const unsigned long long* mask;
    const int* prefix;
    const int* row_index;
    const float* inv_freq;
    const uint32_t* embed_wq;
    const void* embed_scales;
    const void* embed_biases;
    const void* final_norm;
    const void* lm_head_tiled;
    const void* layer_table;
    void* h;
    void* hw;
    void* qkv;
    void* attn;
    void* act;
    void* logits;
    void* kv_cache;
    void* workspace;
    size_t workspace_bytes;
    void* timeline;         /* optional profiling hook, NULL = off: int64 [SMs][timeline_pitch][8]; CTA b  */
    int timeline_pitch;     /* stores the nanosecond timer when it arrives at / leaves device barrier i   */
    int phase_mask;         /* (i = 0 after the embedding, then 6 per layer) and, arrive only, at its end */
                            /* phase_mask: profiling only, 0 = run everything; else bit k set = run phase  */
                            /* kind k (0 embedding, 1 qkv, 2 attention, 3 merge, 4 o_proj, 5 gate/up,      */
                            /* 6 down_proj, 7 vocabulary projection); results are then meaningless         */
    /* Tensor parallelism over the GPUs of one node (tp_world <= 1 = off, all fields below zero).  The call
     * then runs shard tp_rank of tp_world: n_heads, n_kv_heads and intermediate are this shard's counts
     * (heads and MLP rows cut evenly; o_proj / down_proj weights hold this shard's K columns), head_rows
     * is the number of vocabulary rows in lm_head_tiled (logits [rows_out][head_rows]; 0 = vocab), the
     * embedding and the norms are whole.  tp_peers[r] is rank r's exchange buffer
     * (b200_forward_tp_buffer_bytes(hidden) bytes, zero before the first launch, 16-byte aligned) as
     * mapped into this process: peer-accessible device memory, e.g. a CUDA IPC or symmetric-memory
     * mapping.  o_proj and down_proj store their fp32 partial products into their rank's slot of every
     * GPU's buffer (or, in the pull form, leave them in the GPU's own buffer); every CTA then
     * adds one to an arrival counter in every GPU's buffer (remote atomics) and waits (bounded; error
     * code 12 in the workspace's error word on timeout) until its own GPU's counter shows all CTAs of all
     * GPUs; then every GPU adds all partial products in rank order (from its own memory; in the pull
     * form with plain loads over NVLink), so every GPU holds bit-identical hidden states.  The running count of
     * exchanges lives in the buffer (flags only grow), so a launch can be replayed from a CUDA graph.
     * Every rank must launch the same sequence of passes; the kernels of one pass run concurrently,
     * one per GPU, never two ranks on one GPU.  After an error code 12 the buffers of all ranks must
     * be zeroed (with no launch in flight anywhere) before the next pass. */
    int tp_world, tp_rank;
    int head_rows;
    int grid_ctas;          /* CTAs of the persistent kernel: 0 = one per SM.  A small model (a draft whose layer is
                             * a few MB) is bound by the latency of its device-wide phase boundaries, not by
                             * bandwidth: fewer CTAs make every boundary cheaper and 16 to 64 SMs already pull 2 to
                             * 6.5 TB/s.  Size the workspace with the same value. */
    void* tp_peers[8];
    int scales_in_fast_range;   /* non-zero: EVERY group scale of every matrix of layer_table and of lm_head_tiled has its
                                 * fp16 exponent field in 1..10 (2^-14 <= |scale| < 2^-4, never zero or subnormal): the
                                 * kernel then expands the nibbles with a shorter instruction sequence that gives the
                                 * same bits.  0 is always safe. */
    int tp_two_shot;            /* exchange of the row-parallel layers (o_proj, down_proj); the same value on every rank,
                                 * the same bits whichever form runs; zero the exchange buffers when switching.
                                 * 0 = the library's choice (the push form).
                                 * 3 = push form: every GPU stores its partial products into its slot of EVERY GPU's
                                 * buffer while the matmul phase runs (posted stores over NVLink); after one all-GPU
                                 * barrier each GPU adds up the slots in its own memory, so no load crosses NVLink.
                                 * 4 = pull form: every GPU keeps its partial products in its own buffer and, after the
                                 * all-GPU barrier, reads all ranks' products in full over NVLink.
                                 * 2 = the pull form behind a hierarchical all-GPU barrier: the CTAs of a GPU meet on a
                                 * local counter and only the last one adds to the peers' counters (7 remote atomics per
                                 * exchange and GPU at 8 GPUs instead of 148 x 7).
                                 * 1 = two-step form: each GPU reduces its slice of the columns (pulled) and stores the
                                 * result to every GPU (a second all-GPU barrier; needs hidden % (16 * tp_world) == 0,
                                 * else the pull form runs). */
    int requests;               /* 0 or 1: one request.  2..4: the M rows are `requests` groups of M / requests rows, one
                                 * group per request, so that several requests share every weight read (no counterpart in
                                 * the reference, which decodes one request).  Request r then has its own committed length
                                 * prefix[r], its own head-row offset row_index[r] (if row_index is given) and its own slab
                                 * of kv_cache, laid out [requests][layers][2][kv heads][cache_rows][head_dim]; write_off
                                 * and tail apply to each; attention never crosses requests; rows_out counts rows per
                                 * request and logits is [requests * rows_out][vocab].  Needs cache_rows <= 2048 (single-
                                 * phase attention) and tp_world <= 1. */
} b200_forward_desc;

size_t b200_forward_workspace_bytes(const b200_forward_desc* desc);
size_t b200_forward_tp_buffer_bytes(int hidden);

/* Exchange buffers for tp_peers.  alloc: `bytes` of zeroed device memory on the current device plus a
 * 64-byte handle to hand to the other processes of the node (any host channel); open: map a peer's
 * buffer into this process (peer access is enabled on demand); close / free undo them.  The buffers
 * must be zero and every rank must have opened all of them before the first tensor-parallel launch. */
#define B200_TP_HANDLE_BYTES 64
int b200_tp_exchange_alloc(size_t bytes, void** ptr, unsigned char* handle);
int b200_tp_exchange_open(const unsigned char* handle, void** ptr);
int b200_tp_exchange_close(void* ptr);
int b200_tp_exchange_free(void* ptr);
/* Zero this GPU's own buffer again (synchronous).  After a pass that reported a timeout every rank calls it with
 * no launch in flight anywhere (the host synchronises the ranks before and after), then passes may resume. */
int b200_tp_exchange_reset(void* own_buffer, size_t bytes);
/* Error word of the argmax combine in this GPU's own buffer: 0, or 1 after a combine that gave up waiting
 * for a peer (synchronous 4-byte copy; negative = B200_E*). */
int b200_tp_exchange_error(const void* own_buffer);

/* Vocabulary-parallel greedy argmax (the per-shard halves of evaluate_posterior_greedy's argmax,
 * mlx_eagle.py:311-313): best_key[R] holds this shard's keys from b200_logits_argmax (shard-local
 * indices); index_offset = first vocabulary row of the shard.  One small kernel per GPU shifts the keys
 * to global indices, publishes them in its exchange buffer, raises its flag at every peer, waits (bounded)
 * for the peers' flags and leaves the maximum over all shards in best_key on every GPU.  No host
 * synchronisation, safe inside a CUDA graph; R <= 32. */
int b200_tp_argmax_combine(unsigned long long* best_key, int R, unsigned int index_offset, int tp_world,
                           int tp_rank, void* const* tp_peers, void* stream);
int b200_forward(const b200_forward_desc* desc, void* stream);

/* Measurement aid, not part of the model interface: overrides the work split the planner would choose for the
 * matmul phases of later b200_forward calls.  spec = "A=kw:cps:splits,C=...,D=...,E=...,H=..." (A q|k|v, C o_proj,
 * D gate/up, E down_proj, H vocabulary projection; kw = K-parts inside a CTA, 1/2/4/8; cps = 128-column chunks of K
 * per ring stage; splits = split of K across CTAs); values that do not fit the shape are ignored; NULL or ""
 * restores the planner.  The workspace size depends on the split: query b200_forward_workspace_bytes again after a
 * hint.  The same string is read once from the environment variable B200_FWD_PLAN.  No counterpart in the reference. */
void b200_forward_plan_hint(const char* spec);

/* ------------------------------------------------------------------------------------------
 * Draft tree, acceptance and compaction.  One request; k = 8 children per node.
 * ctl is int32[16]: [0] committed length of the target cache, [1] of the draft cache, [2] accept
 * length of the previous step, [3] tokens generated, [4] step, [5] draft cache length after the
 * catch-up pass, [6] capacity of out_tokens, [7] best path of the last step, [8] capacity of the step log, [9] end-of-sequence
 * id + 1 (0 = none), [10] done flag, [11] token count at the stop, [12] seed and [13] draw count of sampling acceptance.
 * Ordering keys: (order-preserving image of the fp32 value) << 32 | (0xffffffff - index).
 * ------------------------------------------------------------------------------------------ */
int b200_topk_blocks(int V);
int b200_logits_rowstats(const void* logits, int R, int V, uint32_t* row_max, unsigned long long* row_sum,
                         void* stream);
int b200_logits_topk_candidates(const void* logits, int R, int V, const uint32_t* row_max,
                                const unsigned long long* row_sum, int by_score,
                                unsigned long long* cand, void* stream);
/* Root expansion (level < 0; mlx_eagle.py:410-412) or one tree level (level = i >= 0;
 * process_generate_tree_iteration, mlx_eagle.py:97-115, plus the per-level bookkeeping of
 * generate_draft_tree, :157-207).  Writes the candidate pool and the inputs (tokens, positions,
 * tail masks, prefix) of the next draft forward. */
int b200_tree_expand(const void* logits, int V, int level, const unsigned long long* cand, uint32_t* row_max,
                     unsigned long long* row_sum, int* ctl, float* pool_scores, int* pool_tokens,
                     uint32_t* pool_parents, float* cur_scores, uint32_t* topk_cs_index, int* fwd_tokens,
                     int* fwd_pos, unsigned long long* fwd_mask, int* fwd_prefix, void* stream);
/* Inputs of the draft catch-up pass: y padded to 8 tokens (mlx_eagle.py:400-408). */
int b200_prep_catchup(const int* ctl, const int* y, int* fwd_tokens, int* fwd_pos, unsigned long long* fwd_mask,
                      int* fwd_prefix, int* sel_row, void* stream);
/* process_draft_tree + search_sorted + post_process_draft_tree (mlx_eagle.py:61-93,217-295): stable
 * top-T of the pool, parents, ancestor masks, depths, verify inputs, root-to-leaf paths
 * (retrieve is [T][9] int32, -1 padded; tree_info[0] = leaves, [1] = max depth + 1). */
int b200_tree_finalize(int depth, int T, const float* pool_scores, const int* pool_tokens,
                       const uint32_t* pool_parents, const int* ctl, const int* y, int* fwd_tokens,
                       int* fwd_pos, unsigned long long* fwd_mask, int* fwd_prefix, int* tree_position_ids,
                       int* mask_index, int* draft_tokens, int* retrieve, int* tree_info, void* stream);
int b200_logits_argmax(const void* logits, int R, int V, unsigned long long* best_key, void* stream);
/* Vocabulary-parallel argmax across GPUs: turns the shard-local keys of b200_logits_argmax into global ones
 * (index_offset = first vocabulary row of this GPU's shard) and toggles the top bit so that a signed 64-bit MAX
 * all-reduce orders them; call again with index_offset 0 after the all-reduce to toggle the bit back. */
int b200_argmax_key_shift(unsigned long long* best_key, int R, unsigned int index_offset, void* stream);
/* evaluate_posterior_greedy (mlx_eagle.py:311-326) on per-node argmaxes, plus the loop bookkeeping of
 * generate_step (:587-599): next y, accept length, lengths of both caches, generated-token log.
 * accept_rows[0] = accept length, [1..] = accepted node indices (retrieve_indices[best, 1:1+a]). */
int b200_tree_accept(int T, unsigned long long* argmax_key, const int* draft_tokens, const int* retrieve,
                     const int* tree_info, int* ctl, int* y, int* accept_rows, int* out_tokens,
                     int* step_log, void* stream);

/* Sampling acceptance at temperature > 0 (no counterpart in the reference, which is greedy only: README.md:9;
 * the same role as evaluate_posterior_greedy + the bookkeeping of generate_step, mlx_eagle.py:311-326,587-599).
 * Speculative sampling on the verify tree: with p = softmax(logits[node] / temperature), walk down from the root; a
 * node's children are tried in node order, a child with token x is accepted with probability p(x) of what is left of
 * the node's distribution, a rejected token's mass is removed; when no child is accepted the bonus token is drawn from
 * what is left, so every emitted token is distributed as if sampled from the target alone.  Integer arithmetic
 * throughout (masses round(exp((l - max) / temperature) * 2^40) from the deterministic exponential of the tree
 * scores, 40-bit draws from splitmix64(seed = ctl[12], draw index = ctl[13])): a CPU restatement takes the same
 * decisions bit for bit.  logits [T+1, V] fp16 are the target logits of the tree nodes, mask_index[n] the parent of node
 * n + 1 (b200_tree_finalize); row_max / row_sum: [T+1] scratch, zero on entry, zero again on exit; workspace:
 * b200_tree_accept_sample_workspace_bytes(V) bytes, 16-byte aligned.  Outputs as b200_tree_accept (best path = 0). */
size_t b200_tree_accept_sample_workspace_bytes(int V);
int b200_tree_accept_sample(int T, int V, const void* logits, uint32_t* row_max, unsigned long long* row_sum,
                            const int* draft_tokens, const int* mask_index, double temperature, int* ctl, int* y,
                            int* accept_rows, int* out_tokens, int* step_log, void* workspace, size_t workspace_bytes,
                            void* stream);
/* One draw from softmax(logits_row / temperature) with the same integer arithmetic and generator (draw number `counter`
 * of the stream `seed`): the first token of a request in sampling mode (the reference takes it greedily,
 * mlx_eagle.py:536-538).  logits_row [V] fp16; row_max / row_sum: one word each, zero on entry and on exit; workspace as
 * for b200_tree_accept_sample; out_token: device int. */
int b200_sample_token(const void* logits_row, int V, double temperature, unsigned int seed, unsigned int counter,
                      uint32_t* row_max, unsigned long long* row_sum, void* workspace, size_t workspace_bytes,
                      int* out_token, void* stream);
/* b200_logits_rowstats with the logits divided by `temperature` before the exponential. */
int b200_logits_rowstats_temp(const void* logits, int R, int V, uint32_t* row_max, unsigned long long* row_sum,
                              double temperature, void* stream);
/* accept_candidate (mlx_eagle.py:349-376) over all layers; cache is [layers][2][Hkv][cache_rows][hd]. */
int b200_kv_compact(void* cache, int layers, int Hkv, int cache_rows, int hd, const int* accept_rows,
                    const int* ctl, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_EAGLE_H */
