// Draft-tree construction, verify-batch finalisation, greedy acceptance and KV compaction, all on
// the device: one request, k = 8 children per node, no host round trip inside a decode step.
//
// Ordering rule everywhere: larger value first, ties to the lower index.  It is implemented as a
// max over 64-bit keys (order-preserving image of the value << 32 | ~index), so parallel
// reductions give the same answer in any order.
//
// Log-probabilities use a fixed arithmetic that a CPU reproduces bit for bit: separately rounded
// double add/multiply (never fused), exp by range reduction + Taylor, the sum of exponentials in
// 2^-40 fixed point with integer adds (associative), log by the atanh series; the score of a token
// is float(logit - lse).
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kK = 8;                 // children per node (hard-wired in the reference, mlx_eagle.py:750)
constexpr int kTopkChunk = 4096;      // logits handled by one CTA of the top-k and argmax kernels
constexpr int kStatChunk = 1024;      // ... of the max and sum-of-exponentials kernels: four elements per thread (the fp64
                                      //     exponential is a long dependent chain; short chains, many CTAs)
constexpr int kMaxDepth = 7;
constexpr int kMaxPool = kK + kK * kK * kMaxDepth;

// ctl words
enum { CTL_BASE_LEN = 0, CTL_DRAFT_LEN = 1, CTL_ACCEPT = 2, CTL_NGEN = 3, CTL_STEP = 4, CTL_DRAFT_OFF = 5,
       CTL_OUT_CAP = 6, CTL_LAST_BEST = 7,
       CTL_LOG_CAP = 8,      // steps the step log can hold; later steps are counted but not logged
       CTL_EOS = 9,          // end-of-sequence token id + 1 (0 = none)
       CTL_DONE = 10,        // set once an accepted token was the end-of-sequence token
       CTL_STOP_N = 11,      // generated-token count up to and including that token
       CTL_SEED = 12,        // sampling acceptance: seed of the request's random stream ...
       CTL_DRAW = 13,        // ... and the number of draws made so far
       CTL_WORDS = 16 };

// ---------------------------------------------------------------- ordering keys
__device__ __forceinline__ uint32_t order_bits(float f) {
    f = f + 0.0f;                                     // -0 -> +0 so equal values share one key
    uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float unorder_bits(uint32_t u) {
    uint32_t b = (u & 0x80000000u) ? (u & 0x7fffffffu) : ~u;
    return __uint_as_float(b);
}
__device__ __forceinline__ unsigned long long make_key(float v, uint32_t idx) {
    return ((unsigned long long)order_bits(v) << 32) | (unsigned long long)(0xffffffffu - idx);
}
__device__ __forceinline__ uint32_t key_index(unsigned long long k) { return 0xffffffffu - (uint32_t)(k & 0xffffffffu); }
__device__ __forceinline__ float key_value(unsigned long long k) { return unorder_bits((uint32_t)(k >> 32)); }

__device__ __forceinline__ unsigned long long warp_max_key(unsigned long long k) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        unsigned long long other = __shfl_xor_sync(0xffffffffu, k, o);
        k = other > k ? other : k;
    }
    return k;
}

// ---------------------------------------------------------------- deterministic exp / log
__device__ __forceinline__ double exp_det(double d) {
    const double LOG2E = 1.4426950408889634;
    const double LN2_HI = 6.93147180369123816490e-01;
    const double LN2_LO = 1.90821492927058770002e-10;
    const double dd = fmax(d, -40.0);
    const double kf = rint(__dmul_rn(dd, LOG2E));
    const double r = __dsub_rn(__dsub_rn(dd, __dmul_rn(kf, LN2_HI)), __dmul_rn(kf, LN2_LO));
    const double c[14] = {1.0, 1.0, 1.0 / 2.0, 1.0 / 6.0, 1.0 / 24.0, 1.0 / 120.0, 1.0 / 720.0,
                          1.0 / 5040.0, 1.0 / 40320.0, 1.0 / 362880.0, 1.0 / 3628800.0,
                          1.0 / 39916800.0, 1.0 / 479001600.0, 1.0 / 6227020800.0};
    double p = c[13];
#pragma unroll
    for (int i = 12; i >= 0; i--) p = __dadd_rn(__dmul_rn(p, r), c[i]);
    const double out = scalbn(p, (int)kf);
    return d < -40.0 ? 0.0 : out;
}
__device__ __forceinline__ long long exp_fixed(double d) { return __double2ll_rn(scalbn(exp_det(d), 40)); }

__device__ __forceinline__ double log_det(unsigned long long total) {
    const double LN2_HI = 6.93147180369123816490e-01;
    const double LN2_LO = 1.90821492927058770002e-10;
    int e;
    double f = frexp(__ull2double_rn(total), &e);
    if (f < 0.70710678118654752440) { f = __dmul_rn(f, 2.0); e -= 1; }
    const double ed = (double)(e - 40);
    const double s = __ddiv_rn(__dsub_rn(f, 1.0), __dadd_rn(f, 1.0));
    const double z = __dmul_rn(s, s);
    const double c[12] = {1.0, 1.0 / 3.0, 1.0 / 5.0, 1.0 / 7.0, 1.0 / 9.0, 1.0 / 11.0, 1.0 / 13.0,
                          1.0 / 15.0, 1.0 / 17.0, 1.0 / 19.0, 1.0 / 21.0, 1.0 / 23.0};
    double q = c[11];
#pragma unroll
    for (int i = 10; i >= 0; i--) q = __dadd_rn(__dmul_rn(q, z), c[i]);
    const double lnf = __dmul_rn(__dmul_rn(2.0, s), q);
    return __dadd_rn(__dmul_rn(ed, LN2_HI), __dadd_rn(__dmul_rn(ed, LN2_LO), lnf));
}

__device__ __forceinline__ double row_lse(uint32_t max_enc, unsigned long long sum) {
    return __dadd_rn((double)unorder_bits(max_enc), log_det(sum));
}
__device__ __forceinline__ float score_of(float logit, double lse) {
    return __double2float_rn(__dsub_rn((double)logit, lse));
}

// ---------------------------------------------------------------- row kernels over logits [R, V]
__global__ void row_max_kernel(const __half* __restrict__ logits, int V, uint32_t* __restrict__ row_max) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.y;
    const int begin = blockIdx.x * kStatChunk, end = min(V, begin + kStatChunk);
    const __half* row = logits + (size_t)r * V;
    uint32_t best = 0;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) best = max(best, order_bits(__half2float(row[i])));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    if ((threadIdx.x & 31) == 0) atomicMax(row_max + r, best);
}

// temp: temperature the logits are divided by before the exponential (1.0: the plain soft-max; dividing by 1.0 is exact,
// so the draft tree's log-probabilities are what they were).
__global__ void row_sumexp_kernel(const __half* __restrict__ logits, int V, const uint32_t* __restrict__ row_max,
                                  unsigned long long* __restrict__ row_sum, double temp) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.y;
    const int begin = blockIdx.x * kStatChunk, end = min(V, begin + kStatChunk);
    const __half* row = logits + (size_t)r * V;
    const double mx = (double)unorder_bits(row_max[r]);
    unsigned long long acc = 0;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x)
        acc += (unsigned long long)exp_fixed(__ddiv_rn(__dsub_rn((double)__half2float(row[i]), mx), temp));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) atomicAdd(row_sum + r, acc);
}

// Local top-8 of one chunk of one row.  by_score == 0: order by the raw logit (root expansion,
// mlx_eagle.py:411); by_score == 1: order by the fp32 log-probability (tree levels, :104-105).
__global__ void __launch_bounds__(256) row_topk_kernel(const __half* __restrict__ logits, int V,
                                                       const uint32_t* __restrict__ row_max,
                                                       const unsigned long long* __restrict__ row_sum,
                                                       int by_score, unsigned long long* __restrict__ cand) {
    pdl_wait();
    pdl_launch_dependents();
    // Every thread keeps its 16 keys in registers; each warp selects the top 8 of its 512 keys with warp
    // shuffles only, then one warp selects the top 8 of the 64 survivors: one block-wide barrier in all.
    constexpr int PER = kTopkChunk / 256;
    __shared__ unsigned long long wtop[8 * kK];
    const int r = blockIdx.y;
    const int begin = blockIdx.x * kTopkChunk, end = min(V, begin + kTopkChunk);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const __half* row = logits + (size_t)r * V;
    double lse = 0.0;
    if (by_score) lse = row_lse(row_max[r], row_sum[r]);
    unsigned long long mine[PER];
#pragma unroll
    for (int j = 0; j < PER; j++) {
        const int i = begin + j * 256 + (int)threadIdx.x;
        mine[j] = 0ull;                                        // past the end: never selected
        if (i < end) {
            const float l = __half2float(row[i]);
            mine[j] = make_key(by_score ? score_of(l, lse) : l, (uint32_t)i);
        }
    }
    unsigned long long bound = ~0ull;
    for (int round = 0; round < kK; round++) {
        unsigned long long best = 0;
#pragma unroll
        for (int j = 0; j < PER; j++)
            if (mine[j] < bound && mine[j] > best) best = mine[j];
        best = warp_max_key(best);
        if (lane == 0) wtop[warp * kK + round] = best;         // 0 when the warp has run out
        bound = best ? best : 0ull;
    }
    __syncthreads();
    if (warp == 0) {
        const unsigned long long k0 = wtop[lane], k1 = wtop[lane + 32];
        unsigned long long* out = cand + ((size_t)r * gridDim.x + blockIdx.x) * kK;
        bound = ~0ull;
        for (int round = 0; round < kK; round++) {
            unsigned long long best = 0;
            if (k0 < bound && k0 > best) best = k0;
            if (k1 < bound && k1 > best) best = k1;
            best = warp_max_key(best);
            if (lane == 0) out[round] = best;                  // 0 when the chunk has run out
            bound = best ? best : 0ull;
        }
    }
}

__global__ void row_argmax_kernel(const __half* __restrict__ logits, int V, unsigned long long* __restrict__ best_key) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.y;
    const int begin = blockIdx.x * kTopkChunk, end = min(V, begin + kTopkChunk);
    const __half* row = logits + (size_t)r * V;
    unsigned long long best = 0;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const unsigned long long k = make_key(__half2float(row[i]), (uint32_t)i);
        best = k > best ? k : best;
    }
    best = warp_max_key(best);
    if ((threadIdx.x & 31) == 0) atomicMax(best_key + r, best);
}

__global__ void argmax_key_shift_kernel(unsigned long long* __restrict__ best_key, int R, unsigned int index_offset) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = threadIdx.x;
    if (r < R) best_key[r] = (best_key[r] - index_offset) ^ 0x8000000000000000ull;   // low word: 0xffffffff - index
}

// ---------------------------------------------------------------- tree expansion (1 CTA, 8 warps)
struct ExpandParams {
    const __half* logits;                // [R, V]
    int V, nblk, R;
    const unsigned long long* cand;      // [R][nblk][8]
    uint32_t* row_max;                   // [R]   (cleared on exit)
    unsigned long long* row_sum;         // [R]   (cleared on exit)
    int level;                           // -1: root expansion; i >= 0: tree level i
    int* ctl;
    float* pool_scores;                  // [8 + 64*D]
    int* pool_tokens;                    // [8 + 64*D]
    uint32_t* pool_parents;              // [1 + 8*D]
    float* cur_scores;                   // [8]
    uint32_t* topk_cs_index;             // [8]
    int* fwd_tokens;                     // draft forward inputs for the next level
    int* fwd_pos;
    unsigned long long* fwd_mask;
    int* fwd_prefix;
};

__global__ void __launch_bounds__(256) tree_expand_kernel(const ExpandParams p) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float s_val[kK][kK];      // per-row top-8 log-probabilities
    __shared__ int s_idx[kK][kK];        // per-row top-8 token ids
    __shared__ float s_cu[kK * kK];
    __shared__ unsigned long long s_oldmask[kK];
    const int lane = threadIdx.x & 31, r = threadIdx.x >> 5;
    const bool root = p.level < 0;

    if (r < p.R) {
        const double lse = row_lse(p.row_max[r], p.row_sum[r]);
        const unsigned long long* c = p.cand + (size_t)r * p.nblk * kK;
        const int n = p.nblk * kK;
        // the row's candidates stay in registers for the eight selection rounds (up to kCandRegs * 32 of them;
        // a larger vocabulary re-reads them from memory)
        constexpr int kCandRegs = 12;
        unsigned long long mine[kCandRegs];
#pragma unroll
        for (int j = 0; j < kCandRegs; j++) mine[j] = (lane + 32 * j < n) ? c[lane + 32 * j] : 0ull;
        unsigned long long bound = ~0ull;
        for (int round = 0; round < kK; round++) {
            unsigned long long best = 0;
#pragma unroll
            for (int j = 0; j < kCandRegs; j++)
                if (mine[j] < bound && mine[j] > best) best = mine[j];
            for (int i = lane + 32 * kCandRegs; i < n; i += 32) {
                const unsigned long long k = c[i];
                if (k < bound && k > best) best = k;
            }
            best = warp_max_key(best);
            bound = best;
            if (lane == 0) {
                const uint32_t tok = key_index(best);
                s_idx[r][round] = (int)tok;
                // root: key holds the logit, the score is logit - lse (mlx_eagle.py:410-412)
                s_val[r][round] = root ? score_of(__half2float(p.logits[(size_t)r * p.V + tok]), lse) : key_value(best);
            }
        }
    }
    __syncthreads();

    if (root) {
        if (threadIdx.x < kK) {
            const int j = threadIdx.x;
            const int off = p.ctl[CTL_DRAFT_LEN] + p.ctl[CTL_ACCEPT] + 1;   // draft cache length after catch-up
            p.pool_scores[j] = s_val[0][j];
            p.pool_tokens[j] = s_idx[0][j];
            p.cur_scores[j] = s_val[0][j];
            p.topk_cs_index[j] = (uint32_t)j;
            p.fwd_tokens[j] = s_idx[0][j];
            p.fwd_pos[j] = off;
            p.fwd_mask[j] = 1ull << j;
            if (j == 0) {
                p.pool_parents[0] = 0u;
                p.fwd_prefix[0] = off;
                p.ctl[CTL_DRAFT_OFF] = off;
            }
        }
    } else {
        const int i = p.level;
        if (threadIdx.x < kK * kK) {
            const int rr = threadIdx.x >> 3, cc = threadIdx.x & 7;
            const float cu = s_val[rr][cc] + p.cur_scores[rr];              // fp32 add (mlx_eagle.py:107)
            s_cu[threadIdx.x] = cu;
            const int flat = kK * (1 + kK * i + rr) + cc;
            p.pool_scores[flat] = cu;
            p.pool_tokens[flat] = s_idx[rr][cc];
        }
        if (threadIdx.x < kK) {
            // parents of this level's rows come from the previous level's selection (mlx_eagle.py:158-162)
            const uint32_t bias = 1u + (uint32_t)(kK * kK) * (uint32_t)max(0, i - 1) + (i > 0 ? (uint32_t)kK : 0u);
            p.pool_parents[1 + kK * i + threadIdx.x] = p.topk_cs_index[threadIdx.x] + bias;
            s_oldmask[threadIdx.x] = p.fwd_mask[threadIdx.x];
        }
        __syncthreads();
        if (r == 0) {
            // top-8 of the 64 cumulative scores, flat index order on ties (mlx_eagle.py:108)
            unsigned long long k0 = make_key(s_cu[lane], (uint32_t)lane);
            unsigned long long k1 = make_key(s_cu[lane + 32], (uint32_t)(lane + 32));
            unsigned long long bound = ~0ull;
            for (int round = 0; round < kK; round++) {
                unsigned long long best = 0;
                if (k0 < bound && k0 > best) best = k0;
                if (k1 < bound && k1 > best) best = k1;
                best = warp_max_key(best);
                bound = best;
                if (lane == 0) {
                    const uint32_t flat = key_index(best);
                    const int parent_row = (int)(flat >> 3);                // out_ids (mlx_eagle.py:109)
                    p.topk_cs_index[round] = flat;
                    p.cur_scores[round] = key_value(best);
                    p.fwd_tokens[round] = s_idx[parent_row][flat & 7];
                    p.fwd_pos[round] = p.ctl[CTL_DRAFT_OFF] + i + 1;
                    // the query inherits its parent's visible columns and sees itself (mlx_eagle.py:171,207)
                    p.fwd_mask[round] = s_oldmask[parent_row] | (1ull << (kK * (i + 1) + round));
                }
            }
        }
    }
    if (threadIdx.x < p.R) {
        p.row_max[threadIdx.x] = 0u;
        p.row_sum[threadIdx.x] = 0ull;
    }
}

// ---------------------------------------------------------------- catch-up pass inputs
// The draft model re-reads the tokens accepted in the previous step plus the bonus token, padded
// with zeros to 8 rows (mlx_eagle.py:400-408); logits of row `accept_len` are the ones used.
__global__ void prep_catchup_kernel(const int* __restrict__ ctl, const int* __restrict__ y, int* fwd_tokens,
                                    int* fwd_pos, unsigned long long* fwd_mask, int* fwd_prefix, int* sel_row) {
    pdl_wait();
    pdl_launch_dependents();
    const int m = threadIdx.x;
    if (m >= kK) return;
    const int dl = ctl[CTL_DRAFT_LEN], a = ctl[CTL_ACCEPT];
    fwd_tokens[m] = (m <= a) ? y[m] : 0;
    fwd_pos[m] = dl + m;
    fwd_mask[m] = (2ull << m) - 1ull;
    if (m == 0) {
        fwd_prefix[0] = dl;
        sel_row[0] = a;
    }
}

// ---------------------------------------------------------------- verify-batch finalisation (1 CTA)
struct FinalizeParams {
    int depth, T;
    const float* pool_scores;
    const int* pool_tokens;
    const uint32_t* pool_parents;
    const int* ctl;
    const int* y;
    int* fwd_tokens;                     // target forward inputs [T+1]
    int* fwd_pos;
    unsigned long long* fwd_mask;
    int* fwd_prefix;
    int* tree_position_ids;              // [T+1]
    int* mask_index;                     // [T]
    int* draft_tokens;                   // [T+1]
    int* retrieve;                       // [T][kMaxDepth + 2], -1 padded
    int* tree_info;                      // [0] leaf_num, [1] max_depth
};

__global__ void __launch_bounds__(512) tree_finalize_kernel(const FinalizeParams p) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ unsigned long long s_key[kMaxPool];
    __shared__ unsigned char s_sel[kMaxPool];
    __shared__ int s_selidx[32];
    __shared__ int s_parent[32];         // mask_index
    __shared__ unsigned long long s_anc[32];
    __shared__ int s_depth[32];
    __shared__ unsigned char s_nonleaf[32];
    const int ps = kK + kK * kK * p.depth;
    const int T = p.T;
    const int tid = threadIdx.x;
    if (tid < ps) s_key[tid] = make_key(p.pool_scores[tid], (uint32_t)tid);
    if (tid < 32) s_nonleaf[tid] = 0;
    __syncthreads();
    // stable top-T (mlx_eagle.py:229): rank by counting
    if (tid < ps) {
        const unsigned long long mine = s_key[tid];
        int rank = 0;
        for (int j = 0; j < ps; j++) rank += (s_key[j] > mine);
        s_sel[tid] = rank < T;
    }
    __syncthreads();
    // ... sorted by flat index (mlx_eagle.py:230)
    if (tid < ps && s_sel[tid]) {
        int pos = 0;
        for (int j = 0; j < tid; j++) pos += s_sel[j];
        s_selidx[pos] = tid;
    }
    __syncthreads();
    if (tid < T) {
        const int flat = s_selidx[tid];
        const uint32_t parent = p.pool_parents[flat >> 3];                   // mlx_eagle.py:235
        // bisection for (parent - 1) among the selected flat indices (mlx_eagle.py:61-93,236-237);
        // uint32 wrap for parent == 0 restated, then masked
        const uint32_t target = parent - 1u;
        uint32_t low = 0, high = (uint32_t)T;
        int steps = 0;
        while ((1 << steps) < T) steps++;
        for (int s = 0; s < steps; s++) {
            const uint32_t mid = (low + high) >> 1;
            const uint32_t mv = (uint32_t)s_selidx[min(mid, (uint32_t)(T - 1))];
            if (mv < target) low = mid + 1;
            if (mv >= target) high = mid;
        }
        const int mi = (parent == 0u) ? 0 : (int)low + 1;
        s_parent[tid] = mi;
        p.mask_index[tid] = mi;
        p.draft_tokens[tid + 1] = p.pool_tokens[flat];
    }
    __syncthreads();
    if (tid == 0) {
        // ancestor rows, built in node order like the reference's loop (mlx_eagle.py:239-243)
        s_anc[0] = 1ull;
        for (int n = 1; n <= T; n++) s_anc[n] = (1ull << n) | s_anc[s_parent[n - 1]];
        p.draft_tokens[0] = p.y[p.ctl[CTL_ACCEPT]];                          // _y[:, [-1]] (mlx_eagle.py:436)
        p.fwd_prefix[0] = p.ctl[CTL_BASE_LEN];
    }
    __syncthreads();
    if (tid <= T) {
        const int d = __popcll(s_anc[tid]) - 1;                              // mlx_eagle.py:245
        s_depth[tid] = d;
        p.tree_position_ids[tid] = d;
        p.fwd_pos[tid] = p.ctl[CTL_BASE_LEN] + d;                            // mlx_eagle.py:343
        p.fwd_mask[tid] = s_anc[tid];
        if (tid < T) s_nonleaf[s_parent[tid]] = 1;
    }
    __syncthreads();
    if (tid <= T) p.fwd_tokens[tid] = p.draft_tokens[tid];
    // root-to-leaf paths, leaves in ascending node order, -1 padded (mlx_eagle.py:254-295)
    constexpr int RW = kMaxDepth + 2;
    if (tid < T * RW) p.retrieve[tid] = -1;
    __syncthreads();
    if (tid <= T && !s_nonleaf[tid]) {
        int rid = 0;
        for (int j = 0; j < tid; j++) rid += !s_nonleaf[j];
        int cid = tid;
        for (int j = s_depth[tid]; j >= 0; j--) {
            p.retrieve[rid * RW + j] = cid;
            cid = (cid == 0) ? 0 : s_parent[cid - 1];
        }
    }
    if (tid == 0) {
        int leaves = 0, md = 0;
        for (int n = 0; n <= T; n++) {
            leaves += !s_nonleaf[n];
            md = max(md, s_depth[n]);
        }
        p.tree_info[0] = leaves;
        p.tree_info[1] = md + 1;
    }
}

// The end of a step (generate_step's bookkeeping, mlx_eagle.py:587-599), by one thread: the bonus token after the
// `accept` accepted ones (already in y and out_tokens), the step log, the end-of-sequence test, cache lengths, counters.
__device__ void commit_step(int* ctl, int* y, int* out_tokens, int* step_log, int accept, int best, int bonus) {
    const int P = ctl[CTL_BASE_LEN];
    const int n = ctl[CTL_NGEN];
    const int cap = ctl[CTL_OUT_CAP];
    y[accept] = bonus;
    if (n + accept < cap) out_tokens[n + accept] = bonus;
    const int step = ctl[CTL_STEP];
    if (step < ctl[CTL_LOG_CAP]) {                                      // the log has a fixed capacity; CTL_STEP keeps counting
        step_log[2 * step] = accept;
        step_log[2 * step + 1] = best;
    }
    const int eos1 = ctl[CTL_EOS];
    if (eos1 > 0 && !ctl[CTL_DONE]) {                                   // first end-of-sequence token among this step's tokens
        for (int j = 0; j <= accept; j++) {
            if (y[j] == eos1 - 1) {
                ctl[CTL_DONE] = 1;
                ctl[CTL_STOP_N] = n + j + 1;
                break;
            }
        }
    }
    ctl[CTL_DRAFT_LEN] = ctl[CTL_DRAFT_OFF];                            // draft cache rewound (mlx_eagle.py:593-594)
    ctl[CTL_BASE_LEN] = P + accept + 1;                                 // mlx_eagle.py:376
    ctl[CTL_ACCEPT] = accept;
    ctl[CTL_NGEN] = n + accept + 1;
    ctl[CTL_STEP] = step + 1;
    ctl[CTL_LAST_BEST] = best;
}

// ---------------------------------------------------------------- greedy acceptance (1 warp)
struct AcceptParams {
    int T;
    unsigned long long* argmax_key;      // [T+1] (cleared on exit)
    const int* draft_tokens;             // [T+1]
    const int* retrieve;                 // [T][kMaxDepth+2]
    const int* tree_info;
    int* ctl;
    int* y;                              // [8] tokens fed to the next step
    int* accept_rows;                    // [8]: [0] = count, [1..] = node index of each accepted token
    int* out_tokens;                     // generated-token log
    int* step_log;                       // [steps][2]: accept length, best path
};

__global__ void tree_accept_kernel(const AcceptParams p) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int RW = kMaxDepth + 2;
    const int lane = threadIdx.x;
    const int T = p.T;
    const int leaf_num = p.tree_info[0], max_depth = p.tree_info[1];
    // evaluate_posterior_greedy (mlx_eagle.py:311-326) on per-node argmaxes; -1 wraps to node T
    int len = -1;
    if (lane < leaf_num) {
        len = 0;
        bool alive = true;
        for (int j = 0; j + 1 < max_depth; j++) {
            int a = p.retrieve[lane * RW + j], b = p.retrieve[lane * RW + j + 1];
            a = a < 0 ? a + T + 1 : a;
            b = b < 0 ? b + T + 1 : b;
            const int pred = (int)key_index(p.argmax_key[a]);
            alive = alive && (p.draft_tokens[b] == pred);
            len += alive ? 1 : 0;
        }
    }
    // max length, first path on ties
    unsigned long long key = lane < leaf_num ? (((unsigned long long)(uint32_t)len << 32) | (0xffffffffu - (uint32_t)lane)) : 0ull;
    key = warp_max_key(key);
    const int accept = (int)(key >> 32);
    const int best = accept == 0 ? 0 : (int)key_index(key);
    if (lane == 0) {
        const int n = p.ctl[CTL_NGEN];
        const int cap = p.ctl[CTL_OUT_CAP];
        p.accept_rows[0] = accept;
        for (int j = 0; j < kK; j++) p.y[j] = 0;
        for (int j = 0; j < accept; j++) {
            const int node = p.retrieve[best * RW + 1 + j];           // may be -1 in the wrap case
            p.accept_rows[1 + j] = node;
            const int tok = p.draft_tokens[node < 0 ? node + T + 1 : node];
            p.y[j] = tok;
            if (n + j < cap) p.out_tokens[n + j] = tok;
        }
        int last = p.retrieve[best * RW + accept];
        last = last < 0 ? last + T + 1 : last;
        const int bonus = (int)key_index(p.argmax_key[last]);           // argmax(logits[best, accept])
        commit_step(p.ctl, p.y, p.out_tokens, p.step_log, accept, best, bonus);
    }
    __syncwarp();
    if (lane <= T) p.argmax_key[lane] = 0ull;
}

// ---------------------------------------------------------------- sampling acceptance
// Speculative sampling on the verify tree at temperature `temp` (the reference is greedy only, README.md:9).  With
// p = softmax(logits[node] / temp): walk down from the root; at a node, take its children in node order (descending
// draft probability); child with token x is accepted with probability p(x) of what is left of the distribution; a
// rejected token's mass is removed and the rest renormalised; when no child is accepted (or the node is a leaf) the
// bonus token is drawn from what is left.  Every emitted token is then distributed exactly as sampling from the target
// alone.  All arithmetic is in integers so that a CPU restatement takes the same decisions bit for bit: masses are
// e(v) = round(exp((l_v - max) / temp) * 2^40) with the deterministic exponential above, their row sums come from
// row_sumexp_kernel, random draws are 40-bit outputs of a counter-based generator (splitmix64 of seed and draw index).
struct SampleState {                    // what the acceptance walk leaves for the bonus draw
    int node, nremoved, accept, pad;
    unsigned long long rem_total, u;    // remaining mass of the node's row; 40-bit draw for the bonus token
    int removed[kK];
};

__device__ __forceinline__ unsigned long long rand40(unsigned int seed, unsigned int counter) {
    unsigned long long z = ((unsigned long long)seed << 32 | counter) + 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return z >> 24;
}
__device__ __forceinline__ unsigned long long mass_of(float logit, uint32_t max_enc, double temp) {
    return (unsigned long long)exp_fixed(__ddiv_rn(__dsub_rn((double)logit, (double)unorder_bits(max_enc)), temp));
}

struct SampleParams {
    int T, V;
    const __half* logits;               // [T+1, V] target logits of the tree nodes
    uint32_t* row_max;                  // [T+1] at temperature `temp` (cleared on exit)
    unsigned long long* row_sum;        // [T+1]
    const int* draft_tokens;            // [T+1]
    const int* mask_index;              // [T] parent node of node n+1
    double temp;
    int* ctl;
    int* y;
    int* accept_rows;
    int* out_tokens;
    int* step_log;
    SampleState* state;
    unsigned long long* chunk_sums;     // [ceil(V / kStatChunk)]
    int* out_token;                     // non-null: a plain draw from row 0 (the first token of a request); the token
                                        //   goes here and the step's bookkeeping is skipped
    unsigned int seed, counter;         // ... with this draw
};

// A plain draw from one row: the state the bonus kernels expect, without a tree walk.
__global__ void sample_init_kernel(const SampleParams p) {
    pdl_wait();
    pdl_launch_dependents();
    if (threadIdx.x != 0) return;
    p.state->node = 0;
    p.state->nremoved = 0;
    p.state->accept = 0;
    p.state->rem_total = p.row_sum[0];
    p.state->u = rand40(p.seed, p.counter);
    for (int j = 0; j < kK; j++) p.state->removed[j] = -1;
}

// The acceptance walk, by one thread (at most 7 levels of at most 8 children).
__global__ void tree_accept_sample_kernel(const SampleParams p) {
    pdl_wait();
    pdl_launch_dependents();
    if (threadIdx.x != 0) return;
    const unsigned int seed = (unsigned int)p.ctl[CTL_SEED];
    unsigned int draw = (unsigned int)p.ctl[CTL_DRAW];
    const int n0 = p.ctl[CTL_NGEN], cap = p.ctl[CTL_OUT_CAP];
    for (int j = 0; j < kK; j++) p.y[j] = 0;
    int cur = 0, accept = 0, nrem = 0;
    int removed[kK];
    unsigned long long rem = p.row_sum[0];
    while (true) {
        rem = p.row_sum[cur];
        nrem = 0;
        int taken = -1;
        for (int c = 1; c <= p.T && taken < 0 && accept < kK - 1; c++) {
            if (p.mask_index[c - 1] != cur) continue;
            const int x = p.draft_tokens[c];
            const unsigned long long ex = mass_of(__half2float(p.logits[(size_t)cur * p.V + x]), p.row_max[cur], p.temp);
            const unsigned long long u = rand40(seed, draw++);
            // accept iff u / 2^40 < ex / rem, compared as 128-bit integers: u * rem < ex * 2^40
            const unsigned long long lhi = __umul64hi(u, rem), llo = u * rem;
            const unsigned long long rhi = ex >> 24, rlo = ex << 40;
            if (lhi < rhi || (lhi == rhi && llo < rlo)) {
                taken = c;
            } else {
                rem -= ex;
                removed[nrem++] = x;
            }
        }
        if (taken < 0) break;
        p.accept_rows[1 + accept] = taken;
        p.y[accept] = p.draft_tokens[taken];
        if (n0 + accept < cap) p.out_tokens[n0 + accept] = p.draft_tokens[taken];
        accept++;
        cur = taken;
    }
    p.accept_rows[0] = accept;
    p.state->node = cur;
    p.state->nremoved = nrem;
    p.state->accept = accept;
    p.state->rem_total = rem;
    p.state->u = rand40(seed, draw++);
    for (int j = 0; j < kK; j++) p.state->removed[j] = j < nrem ? removed[j] : -1;
    p.ctl[CTL_DRAW] = (int)draw;
}

// Mass of every 1024-token chunk of the chosen node's row, rejected tokens left out.
__global__ void bonus_chunk_sums_kernel(const SampleParams p) {
    pdl_wait();
    pdl_launch_dependents();
    const int node = p.state->node, nrem = p.state->nremoved;
    const int begin = blockIdx.x * kStatChunk, end = min(p.V, begin + kStatChunk);
    const __half* row = p.logits + (size_t)node * p.V;
    const uint32_t mx = p.row_max[node];
    unsigned long long acc = 0;
    for (int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        bool gone = false;
        for (int j = 0; j < nrem; j++) gone = gone || (p.state->removed[j] == i);
        if (!gone) acc += mass_of(__half2float(row[i]), mx, p.temp);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    __shared__ unsigned long long ws[8];
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long t = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) t += ws[w];
        p.chunk_sums[blockIdx.x] = t;
    }
}

// The bonus token: the token whose cumulative mass (token order, rejected tokens left out) first exceeds
// u * remaining / 2^40; then the step's bookkeeping.  One CTA of 256 threads.
__global__ void __launch_bounds__(256) bonus_pick_kernel(const SampleParams p) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ unsigned long long s_target, s_base;
    __shared__ int s_chunk;
    __shared__ unsigned long long s_mass[kStatChunk];
    const int node = p.state->node, nrem = p.state->nremoved, accept = p.state->accept;
    const int nchunks = (p.V + kStatChunk - 1) / kStatChunk;
    if (threadIdx.x == 0) {
        const unsigned long long u = p.state->u, rem = p.state->rem_total;
        const unsigned long long target = (__umul64hi(u, rem) << 24) | ((u * rem) >> 40);     // floor(u * rem / 2^40) < rem
        unsigned long long cum = 0;
        int c = 0;
        for (; c < nchunks - 1; c++) {
            const unsigned long long t = p.chunk_sums[c];
            if (cum + t > target) break;
            cum += t;
        }
        s_target = target;
        s_base = cum;
        s_chunk = c;
    }
    __syncthreads();
    const int begin = s_chunk * kStatChunk, end = min(p.V, begin + kStatChunk);
    const __half* row = p.logits + (size_t)node * p.V;
    const uint32_t mx = p.row_max[node];
    for (int i = threadIdx.x; i < kStatChunk; i += 256) {
        const int v = begin + i;
        bool gone = v >= end;
        for (int j = 0; j < nrem; j++) gone = gone || (p.state->removed[j] == v);
        s_mass[i] = gone ? 0ull : mass_of(__half2float(row[v]), mx, p.temp);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned long long cum = s_base;
        int bonus = -1, lastpos = -1;
        for (int i = 0; i < end - begin; i++) {
            if (s_mass[i] == 0ull) continue;
            lastpos = i;
            if (cum + s_mass[i] > s_target) { bonus = begin + i; break; }
            cum += s_mass[i];
        }
        if (bonus < 0) bonus = begin + max(lastpos, 0);     // (unreachable when the sums are consistent)
        if (p.out_token != nullptr) *p.out_token = bonus;
        else commit_step(p.ctl, p.y, p.out_tokens, p.step_log, accept, 0, bonus);
    }
    __syncthreads();
    if ((int)threadIdx.x <= p.T) {                          // the statistics buffers start every use at zero
        p.row_max[threadIdx.x] = 0u;
        p.row_sum[threadIdx.x] = 0ull;
    }
}

// ---------------------------------------------------------------- KV compaction of the accepted path
// For every layer and kv head: rows old_base+1 .. old_base+a  <-  rows old_base + node[j]
// (mlx_eagle.py:366-374).  Sources are gathered before any store (array-assignment semantics).
__global__ void kv_compact_kernel(__half* __restrict__ cache, size_t layer_stride, size_t kv_stride,
                                  int cap, int hd, const int* __restrict__ accept_rows,
                                  const int* __restrict__ ctl) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __half* buf = reinterpret_cast<__half*>(smem_raw);
    const int a = accept_rows[0];
    if (a <= 0) return;
    const int old_base = ctl[CTL_BASE_LEN] - a - 1;                     // ctl already advanced
    __half* base = cache + blockIdx.y * layer_stride + blockIdx.z * kv_stride + (size_t)blockIdx.x * cap * hd;
    for (int i = threadIdx.x; i < a * hd; i += blockDim.x) {
        const int j = i / hd, c = i - j * hd;
        const int src = old_base + accept_rows[1 + j];
        buf[i] = base[(size_t)src * hd + c];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < a * hd; i += blockDim.x) {
        const int j = i / hd, c = i - j * hd;
        base[(size_t)(old_base + 1 + j) * hd + c] = buf[i];
    }
}

inline int nblk_for(int V) { return (V + kTopkChunk - 1) / kTopkChunk; }

}  // namespace
}  // namespace b200

extern "C" {

int b200_topk_blocks(int V) { return V < 1 ? 0 : b200::nblk_for(V); }

// Row maximum (order-preserving uint32 image) and fixed-point sum of exponentials of fp16 logits
// [R,V]; row_max / row_sum must be zero on entry (the expand kernels re-zero them).
int b200_logits_rowstats(const void* logits, int R, int V, uint32_t* row_max, unsigned long long* row_sum,
                         void* stream) {
    if (!logits || !row_max || !row_sum || R < 1 || R > 32 || V < 1) return B200_EINVAL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid((V + b200::kStatChunk - 1) / b200::kStatChunk, R);
    b200::launch_kernel(b200::row_max_kernel, dim3(grid), dim3(256), 0, st, static_cast<const __half*>(logits), V, row_max);
    b200::launch_kernel(b200::row_sumexp_kernel, dim3(grid), dim3(256), 0, st, static_cast<const __half*>(logits), V, row_max, row_sum, 1.0);
    return b200::check_launch();
}

int b200_logits_rowstats_temp(const void* logits, int R, int V, uint32_t* row_max, unsigned long long* row_sum,
                              double temperature, void* stream) {
    if (!logits || !row_max || !row_sum || R < 1 || R > 32 || V < 1 || !(temperature > 0.0)) return B200_EINVAL;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    dim3 grid((V + b200::kStatChunk - 1) / b200::kStatChunk, R);
    b200::launch_kernel(b200::row_max_kernel, dim3(grid), dim3(256), 0, st, static_cast<const __half*>(logits), V, row_max);
    b200::launch_kernel(b200::row_sumexp_kernel, dim3(grid), dim3(256), 0, st, static_cast<const __half*>(logits), V, row_max, row_sum,
                        temperature);
    return b200::check_launch();
}

// Per-chunk top-8 candidates of every row: cand [R][b200_topk_blocks(V)][8] keys.
int b200_logits_topk_candidates(const void* logits, int R, int V, const uint32_t* row_max,
                                const unsigned long long* row_sum, int by_score,
                                unsigned long long* cand, void* stream) {
    if (!logits || !row_max || !row_sum || !cand || R < 1 || R > 32 || V < 1) return B200_EINVAL;
    dim3 grid(b200::nblk_for(V), R);
    b200::launch_kernel(b200::row_topk_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const __half*>(logits), V, row_max, row_sum, by_score, cand);
    return b200::check_launch();
}

// level < 0: root expansion from the catch-up pass logits [1,V] (mlx_eagle.py:410-412);
// level >= 0: one tree level from logits [8,V] (mlx_eagle.py:97-115,157-207).
int b200_tree_expand(const void* logits, int V, int level, const unsigned long long* cand, uint32_t* row_max,
                     unsigned long long* row_sum, int* ctl, float* pool_scores, int* pool_tokens,
                     uint32_t* pool_parents, float* cur_scores, uint32_t* topk_cs_index, int* fwd_tokens,
                     int* fwd_pos, unsigned long long* fwd_mask, int* fwd_prefix, void* stream) {
    if (!logits || !cand || !row_max || !row_sum || !ctl || !pool_scores || !pool_tokens || !pool_parents ||
        !cur_scores || !topk_cs_index || !fwd_tokens || !fwd_pos || !fwd_mask || !fwd_prefix)
        return B200_EINVAL;
    if (V < 8 || level >= b200::kMaxDepth) return B200_EINVAL;
    b200::ExpandParams p{};
    p.logits = static_cast<const __half*>(logits);
    p.V = V; p.nblk = b200::nblk_for(V); p.R = level < 0 ? 1 : b200::kK;
    p.cand = cand; p.row_max = row_max; p.row_sum = row_sum; p.level = level; p.ctl = ctl;
    p.pool_scores = pool_scores; p.pool_tokens = pool_tokens; p.pool_parents = pool_parents;
    p.cur_scores = cur_scores; p.topk_cs_index = topk_cs_index;
    p.fwd_tokens = fwd_tokens; p.fwd_pos = fwd_pos; p.fwd_mask = fwd_mask; p.fwd_prefix = fwd_prefix;
    b200::launch_kernel(b200::tree_expand_kernel, dim3(1), dim3(256), 0, static_cast<cudaStream_t>(stream), p);
    return b200::check_launch();
}

int b200_prep_catchup(const int* ctl, const int* y, int* fwd_tokens, int* fwd_pos, unsigned long long* fwd_mask,
                      int* fwd_prefix, int* sel_row, void* stream) {
    if (!ctl || !y || !fwd_tokens || !fwd_pos || !fwd_mask || !fwd_prefix || !sel_row) return B200_EINVAL;
    b200::launch_kernel(b200::prep_catchup_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), ctl, y, fwd_tokens, fwd_pos,
                                                                               fwd_mask, fwd_prefix, sel_row);
    return b200::check_launch();
}

// process_draft_tree + post_process_draft_tree (mlx_eagle.py:217-295).
int b200_tree_finalize(int depth, int T, const float* pool_scores, const int* pool_tokens,
                       const uint32_t* pool_parents, const int* ctl, const int* y, int* fwd_tokens,
                       int* fwd_pos, unsigned long long* fwd_mask, int* fwd_prefix, int* tree_position_ids,
                       int* mask_index, int* draft_tokens, int* retrieve, int* tree_info, void* stream) {
    if (depth < 0 || depth > b200::kMaxDepth || T < 1 || T > 31 || T > b200::kK + 64 * depth) return B200_EINVAL;
    if (!pool_scores || !pool_tokens || !pool_parents || !ctl || !y || !fwd_tokens || !fwd_pos || !fwd_mask ||
        !fwd_prefix || !tree_position_ids || !mask_index || !draft_tokens || !retrieve || !tree_info)
        return B200_EINVAL;
    b200::FinalizeParams p{};
    p.depth = depth; p.T = T; p.pool_scores = pool_scores; p.pool_tokens = pool_tokens;
    p.pool_parents = pool_parents; p.ctl = ctl; p.y = y; p.fwd_tokens = fwd_tokens; p.fwd_pos = fwd_pos;
    p.fwd_mask = fwd_mask; p.fwd_prefix = fwd_prefix; p.tree_position_ids = tree_position_ids;
    p.mask_index = mask_index; p.draft_tokens = draft_tokens; p.retrieve = retrieve; p.tree_info = tree_info;
    b200::launch_kernel(b200::tree_finalize_kernel, dim3(1), dim3(512), 0, static_cast<cudaStream_t>(stream), p);
    return b200::check_launch();
}

// argmax of every row of fp16 logits [R,V] as ordering keys (first index on ties); best_key must be
// zero on entry (b200_tree_accept re-zeroes it).
int b200_logits_argmax(const void* logits, int R, int V, unsigned long long* best_key, void* stream) {
    if (!logits || !best_key || R < 1 || R > 32 || V < 1) return B200_EINVAL;
    dim3 grid(b200::nblk_for(V), R);
    b200::launch_kernel(b200::row_argmax_kernel, dim3(grid), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const __half*>(logits), V, best_key);
    return b200::check_launch();
}

// Vocabulary-parallel argmax: keys computed on a shard hold shard-local indices.  Shifts them to global
// indices (index_offset = first vocabulary row of the shard) and toggles the top bit, so that a signed 64-bit
// MAX all-reduce orders them like the unsigned keys; a second call with offset 0 toggles the bit back.
int b200_argmax_key_shift(unsigned long long* best_key, int R, unsigned int index_offset, void* stream) {
    if (!best_key || R < 1 || R > 1024) return B200_EINVAL;
    b200::launch_kernel(b200::argmax_key_shift_kernel, dim3(1), dim3(((R + 31) / 32) * 32), 0,
                        static_cast<cudaStream_t>(stream), best_key, R, index_offset);
    return b200::check_launch();
}

// evaluate_posterior_greedy + the bookkeeping of generate_step (mlx_eagle.py:311-326,582-599).
int b200_tree_accept(int T, unsigned long long* argmax_key, const int* draft_tokens, const int* retrieve,
                     const int* tree_info, int* ctl, int* y, int* accept_rows, int* out_tokens,
                     int* step_log, void* stream) {
    if (T < 1 || T > 31 || !argmax_key || !draft_tokens || !retrieve || !tree_info || !ctl || !y ||
        !accept_rows || !out_tokens || !step_log)
        return B200_EINVAL;
    b200::AcceptParams p{};
    p.T = T; p.argmax_key = argmax_key; p.draft_tokens = draft_tokens; p.retrieve = retrieve;
    p.tree_info = tree_info; p.ctl = ctl; p.y = y; p.accept_rows = accept_rows; p.out_tokens = out_tokens;
    p.step_log = step_log;
    b200::launch_kernel(b200::tree_accept_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), p);
    return b200::check_launch();
}

size_t b200_tree_accept_sample_workspace_bytes(int V) {
    if (V < 1) return 0;
    return 128 + sizeof(unsigned long long) * (size_t)((V + b200::kStatChunk - 1) / b200::kStatChunk);
}

int b200_tree_accept_sample(int T, int V, const void* logits, uint32_t* row_max, unsigned long long* row_sum,
                            const int* draft_tokens, const int* mask_index, double temperature, int* ctl, int* y,
                            int* accept_rows, int* out_tokens, int* step_log, void* workspace, size_t workspace_bytes,
                            void* stream) {
    if (T < 1 || T > 31 || V < 1 || !logits || !row_max || !row_sum || !draft_tokens || !mask_index || !ctl || !y ||
        !accept_rows || !out_tokens || !step_log || !workspace || !(temperature > 0.0))
        return B200_EINVAL;
    if (workspace_bytes < b200_tree_accept_sample_workspace_bytes(V)) return B200_EWORKSPACE;
    if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return B200_EALIGN;
    static_assert(sizeof(b200::SampleState) <= 128, "the walk's state must fit the head of the workspace");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc = b200_logits_rowstats_temp(logits, T + 1, V, row_max, row_sum, temperature, stream);
    if (rc != B200_OK) return rc;
    b200::SampleParams p{};
    p.T = T; p.V = V; p.logits = static_cast<const __half*>(logits); p.row_max = row_max; p.row_sum = row_sum;
    p.draft_tokens = draft_tokens; p.mask_index = mask_index; p.temp = temperature; p.ctl = ctl; p.y = y;
    p.accept_rows = accept_rows; p.out_tokens = out_tokens; p.step_log = step_log;
    p.state = static_cast<b200::SampleState*>(workspace);
    p.chunk_sums = reinterpret_cast<unsigned long long*>(static_cast<char*>(workspace) + 128);
    const int nchunks = (V + b200::kStatChunk - 1) / b200::kStatChunk;
    b200::launch_kernel(b200::tree_accept_sample_kernel, dim3(1), dim3(32), 0, st, p);
    b200::launch_kernel(b200::bonus_chunk_sums_kernel, dim3(nchunks), dim3(256), 0, st, p);
    b200::launch_kernel(b200::bonus_pick_kernel, dim3(1), dim3(256), 0, st, p);
    return b200::check_launch();
}

int b200_sample_token(const void* logits_row, int V, double temperature, unsigned int seed, unsigned int counter,
                      uint32_t* row_max, unsigned long long* row_sum, void* workspace, size_t workspace_bytes,
                      int* out_token, void* stream) {
    if (V < 1 || !logits_row || !row_max || !row_sum || !workspace || !out_token || !(temperature > 0.0)) return B200_EINVAL;
    if (workspace_bytes < b200_tree_accept_sample_workspace_bytes(V)) return B200_EWORKSPACE;
    if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return B200_EALIGN;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int rc = b200_logits_rowstats_temp(logits_row, 1, V, row_max, row_sum, temperature, stream);
    if (rc != B200_OK) return rc;
    b200::SampleParams p{};
    p.T = 0; p.V = V; p.logits = static_cast<const __half*>(logits_row); p.row_max = row_max; p.row_sum = row_sum;
    p.temp = temperature; p.out_token = out_token; p.seed = seed; p.counter = counter;
    p.state = static_cast<b200::SampleState*>(workspace);
    p.chunk_sums = reinterpret_cast<unsigned long long*>(static_cast<char*>(workspace) + 128);
    const int nchunks = (V + b200::kStatChunk - 1) / b200::kStatChunk;
    b200::launch_kernel(b200::sample_init_kernel, dim3(1), dim3(32), 0, st, p);
    b200::launch_kernel(b200::bonus_chunk_sums_kernel, dim3(nchunks), dim3(256), 0, st, p);
    b200::launch_kernel(b200::bonus_pick_kernel, dim3(1), dim3(256), 0, st, p);
    return b200::check_launch();
}

// accept_candidate (mlx_eagle.py:349-376) for all layers of one model.  cache: [layers][2][Hkv][rows][hd].
int b200_kv_compact(void* cache, int layers, int Hkv, int cache_rows, int hd, const int* accept_rows,
                    const int* ctl, void* stream) {
    if (!cache || !accept_rows || !ctl || layers < 1 || Hkv < 1 || cache_rows < 1 || hd < 1) return B200_EINVAL;
    const size_t kv_stride = (size_t)Hkv * cache_rows * hd;
    dim3 grid(Hkv, layers, 2);
    b200::launch_kernel(b200::kv_compact_kernel, dim3(grid), dim3(128), (size_t)b200::kK * hd * sizeof(__half), static_cast<cudaStream_t>(stream), static_cast<__half*>(cache), 2 * kv_stride, kv_stride, cache_rows, hd, accept_rows, ctl);
    return b200::check_launch();
}

}  // extern "C"
