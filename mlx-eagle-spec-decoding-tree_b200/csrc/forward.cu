// One forward pass of the 4-bit decoder (<= 32 tokens) as ONE persistent cooperative kernel, sm_100a.
//
// The per-op kernels of this library (rms_norm, qmm, rope_kv_append, tree_attention, ...) cost one
// launch each: nine per decoder layer, ~250 per pass, and at <= 32 tokens every one of them is shorter
// than its own launch/drain latency.  Here the whole pass of mlx_llama.py:298-313 (embedding ->
// layers -> final norm -> vocabulary projection) is one kernel: one CTA per SM, eight consumer
// warps plus one producer warp, and a device-wide barrier between the phases of a layer.
//
//   phase 0   quantised embedding gather, h and h*w_norm, per-tile sums of squares, RoPE cos/sin table
//   per layer A   q|k|v = rstd * ((h*w) . Wqkv^T) + bias            (RMSNorm folded, see below)
//             B1  RoPE of q and of the new k rows, KV append, tree-masked attention partials per
//                 (kv head, 64-key block)
//             B2  merge of the key blocks -> attn
//             C   h += attn . Wo^T ; also writes h*w_post and the sums of squares of the new h
//             D   act = silu(gate) * up   from  rstd * ((h*w) . W^T)
//             E   h += act . Wdown^T ; also h*w_next and sums of squares
//   head      logits = rstd * ((h*w_final) . Whead^T) on the selected rows
//
// RMSNorm is folded into the neighbouring matmuls: the producer of h also stores h*w (fp16, one
// rounding) and the per-128-column partial sums of h^2; the consumer matmul multiplies its fp32
// accumulator by rstd = rsqrt(mean(h^2)+eps) (a per-token scalar commutes with the product) before
// rounding.  This differs from the unfused graph (which rounds (h*rstd)*w to fp16 before the
// product) by input-rounding noise only; all other rounding points are those of the per-op kernels.
//
// The weight stream never stops at a phase boundary: the producer warp keeps filling the shared
// ring with the next phase's weights (which depend on nothing) while the grid barrier completes,
// and adds the activations of those stages once it has observed the barrier.  K/V blocks travel
// through the same ring.  Every wait (mbarrier, grid barrier) is bounded; on a timeout the CTA
// raises the error word of the workspace, stops waiting and runs to the end, so the kernel always
// terminates.  The kernel must be launched cooperatively (all CTAs co-resident).  No load here uses
// cluster multicast.
#include <cuda.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "pipeline.cuh"
#include "tp_layout.cuh"
#include "qmm_common.cuh"

namespace b200 {
namespace {

constexpr int kWN = 8;                        // consumer warps per CTA
constexpr int kNCons = kWN * 32;
constexpr int kMaxReq = 4;                   // requests that can share one pass
constexpr int kFwdThreads = kNCons + 32;      // + one producer warp
constexpr int kRec = 1152;                    // bytes per 16-row x 128-k weight record
constexpr int kWArea = 8 * 4 * kRec;          // weight bytes of a ring stage: 8 (block, chunk) cells of 4 records
// Matmul inputs that a phase of this kernel writes for a later phase (h*w, attention output, MLP
// activations) live in a chunk-major layout: [k chunk of 128][token row (MP of them)][128 halves], so that the
// activations of a stage's K range are ONE contiguous run (one bulk copy).  Inside a row the sixteen 16-byte
// units are swizzled, unit u of token row r sits at u ^ ((r & 1) << 2): the fragment loads of a quarter warp (rows
// g and g + 1, four units each) then hit eight different bank groups without any padding.
constexpr int kXRowH = 128;                   // halves per row of one chunk
constexpr int kXRow = kXRowH * 2;             // bytes
constexpr int kStageBytes = 57344;            // one ring stage (every row count)
constexpr int kMaxLayers = 128;               // layer pointer table kept in shared memory (64 bytes per layer)
constexpr int kLtabBytes = kMaxLayers * 64;
constexpr int kScratch = 36864;               // shared scratch for the K-part reduction of a tile
constexpr int kKeyBlock = 64;
constexpr float kLog2e = 1.4426950408889634f;
constexpr uint32_t kGridWaitLimit = 1u << 22;
constexpr int kSsqPitch = 32;                 // ssq[part][token]
constexpr int kMaxSsqParts = 512;             // one part per 16 columns of h: hidden <= 8192
constexpr int kCsPitch = 64;                  // cos/sin table: cs[token][i], i < head_dim/2 <= 64

// sync words (ints) at the head of the workspace
constexpr int kSyncExit = 1, kSyncErr = 2, kSyncBar = 8;   // exit count, error code, then kBarLanes arrival counters
constexpr int kBarLanes = 8;

enum { EPI_QKV = 0, EPI_SILU = 1, EPI_RESID = 2, EPI_HEAD = 3, EPI_TP = 4 };
enum { K_EMBED = 0, K_A = 1, K_B1 = 2, K_B2 = 3, K_C = 4, K_D = 5, K_E = 6, K_HEAD = 7, K_R = 8 };
constexpr uint32_t kTpWaitLimit = 1u << 22;   // polls of a peer's flag (a microsecond or so each) before giving up
enum { PLAN_A = 0, PLAN_C = 1, PLAN_D = 2, PLAN_E = 3, PLAN_HEAD = 4 };

struct LayerPtrs {                 // one entry per layer, in device memory (8 pointers = 64 bytes)
    const unsigned char* qkv_w;
    const __half* qkv_bias;
    const unsigned char* o_w;
    const unsigned char* gate_w;
    const unsigned char* up_w;
    const unsigned char* down_w;
    const __half* norm_in;
    const __half* norm_post;
};

struct PhasePlan {
    int row_items, splits, chunks_per_split;   // items along N, split-K ways across CTAs
    int kw, cps;                               // K-parts per tile inside a CTA (8/kw tiles per item), chunks of K per ring stage
};

struct FwdParams {
    int M, mp, rows_out, H, I, Hq, Hkv, HD, V, L, NQKV;   // mp: M rounded up to 8 (row count of the padded layout)
    float eps, rope_scale, scale_log2;
    const int* tokens;
    const int* pos;
    const unsigned long long* mask;
    const int* prefix;
    const int* row_index;
    const float* inv_freq;
    const uint32_t* emb_wq;
    const __half* emb_sc;
    const __half* emb_bi;
    const __half* final_norm;
    const unsigned char* head_w;
    const LayerPtrs* layers;
    __half *h, *hw, *qkv, *attn, *act, *logits;
    __half* kv;                    // [layers][2][Hkv][cap][HD]
    size_t kv_layer_stride, kv_half_stride;   // in halves
    int cap, write_off, tail;
    // Several requests in one pass (nreq > 1): the M rows are nreq groups of mr rows; request r has its own
    // committed length prefix[r], head-row offset row_index[r] and KV slab (kv + r * kv_req_stride); attention never
    // crosses requests, every other phase just sees M rows.
    int nreq, mr;
    size_t kv_req_stride;          // in halves
    int kv_req_rows;               // rows of the 2-D view of one request's slab (layers * 2 * Hkv * cap)
    int* sync;
    int* counter;
    float* ssq;
    float2* cs;
    float* part_ml;
    float* part_o;
    float* partial;
    int nkb, qrp;
    PhasePlan plan[5];
    // Tensor parallelism (tp_world > 1): this launch is rank tp_rank's shard.  o_proj / down_proj write fp32
    // partial products into this GPU's exchange buffer; after a handshake through flag words in the peers'
    // buffers every GPU adds the partial products of all ranks (plain loads over NVLink, rank order) and the
    // residual.  tp_peers[r] = rank r's exchange buffer as mapped into this process.
    // The count of exchanges done by earlier launches lives in the buffer (flags only ever grow).
    int tp_world, tp_rank;
    int tp_two_shot;               // reduce-scatter + all-gather through the exchange buffers instead of reading every peer in full
    int tp_hier;                   // all-GPU barrier with one remote arrival per GPU (the last CTA's) instead of one per CTA
    int tp_push;                   // partial products are stored into every GPU's buffer as they are made; the reduce reads local memory only
    unsigned char* tp_peers[kMaxTp];
    int head_rows;                 // rows of the vocabulary projection held here (a vocabulary shard under TP)
    int attn_fused_max;            // single-phase attention while the cache spans at most this many key blocks
    unsigned phase_mask;           // bit per phase kind (K_*): kinds to run; all ones normally
    uint32_t grid_wait_limit, tp_wait_limit;   // polls before a wait on other CTAs / other GPUs gives up
    int fast_scales;               // every group scale of every matrix has its fp16 exponent field in 1..10
    alignas(64) CUtensorMap kvmap; // the whole KV cache as a 2-D fp16 tensor [rows][head_dim], 64 x 64 boxes, 128-byte swizzle
    long long* timeline;           // optional [CTAs][timeline_pitch][8] timer stamps per barrier: arrive, leave, then
                                   // six stamps inside the matmul phase that ends at that barrier
    int timeline_pitch;
};

template <int MT>
struct Geo {
    static constexpr int MP = MT * 8;
    static constexpr int STAGE = kStageBytes;
    static constexpr int NST = 3;
    static constexpr int SMEM = NST * STAGE + 256 + kScratch + kLtabBytes;
};

struct QDesc {
    const __half* x;            // activations [xrows][K]
    const unsigned char* w0;
    const unsigned char* w1;    // up_proj in dual mode
    const __half* bias;
    const __half* wn;           // norm weights applied to the new h (EPI_RESID)
    __half* y;
    int N, K;
    PhasePlan pl;
    int xrows;                  // token rows of the pass
    int row_lo, row_cnt;        // token rows [row_lo, row_lo+row_cnt) are stored, as output rows 0.. (vocabulary projection)
    int orow_sel;               // several requests per pass: which table of out_row_tab() maps token rows to output rows
                                //   (1: the vocabulary projection keeps rows_out rows per request; 0: all rows kept)
    bool y_tiled;               // output goes to the chunk-major padded layout (it is a later phase's matmul input)
};

// Small per-launch tables in static shared memory, reached through functions so that no pointer to them has to
// stay in a register across the matmul loops (the kernel sits at its register limit).
__device__ __forceinline__ int* req_prefix_tab() {       // committed length of every request of the pass
    __shared__ int s_prefix[kMaxReq];
    return s_prefix;
}
__device__ __forceinline__ int* out_row_tab() {          // [2][32] output row of a token row, or -1 = not stored:
    __shared__ int s_orow[2 * 32];                       //   [0] every row kept, [1] the vocabulary projection's selection
    return s_orow;
}

struct Ctx {
    unsigned char* ring;
    uint64_t* full;
    uint64_t* empty;
    uint64_t* afull;              // attention geometry: one barrier pair per key-block slot
    uint64_t* aempty;
    unsigned char* scratch;
    const LayerPtrs* ltab;        // the layer pointer table, copied to shared memory at kernel start
    volatile int* abort_flag;
    volatile uint32_t* s_epoch;   // grid barriers this CTA has seen complete (written by thread 0)
    int* is_last;
    float* s_rstd;
    uint32_t pos;       // ring stages produced (producer warp) / consumed (consumer warps)
    uint32_t apos;      // attention key blocks produced / assigned so far
    uint32_t ause;      // key blocks this consumer warp has taken from its slot so far
    uint64_t* rbar;     // the producer warp has left the per-token 1/rms of the phase's input in s_rstd
    uint32_t ruse;      // phases that used rbar so far (both sides count)
    int ans;            // number of key-block slots (attention geometry)
    uint32_t epoch;     // barriers (device-wide or all-GPU) before the current phase
    uint32_t lbar;      // of those, the device-wide ones (the local counter's target is lbar * CTAs)
    uint32_t tpx;       // tensor-parallel exchanges done in this launch
    uint32_t tp_seq0;   // ... and by all earlier launches
    int lane, warp;
};

// Ring waits of this kernel: up to 2^20 polls of <= 1 us each (about a second) before giving up.
__device__ __forceinline__ bool fwd_wait(uint32_t bar, uint32_t parity) {
    return mbar_wait_timed(bar, parity, 1u << 20, 1000u);
}

__device__ __forceinline__ size_t xt_index(int tok, int n, int mp) {
    const int k = n & 127;
    return ((size_t)(n >> 7) * mp + tok) * kXRowH + ((((k >> 3) ^ ((tok & 1) << 2)) << 3) | (k & 7));
}

__device__ __forceinline__ void fence_proxy_async_all() { asm volatile("fence.proxy.async;\n" ::: "memory"); }

__device__ __forceinline__ int ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];\n" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;\n" : "=l"(t));
    return t;
}

// Profiling stamp k (2..7) of the phase in progress (thread 0 of the CTA, timeline enabled only).
__device__ __forceinline__ void stamp(const FwdParams& p, const Ctx& c, int k) {
    if (p.timeline != nullptr && threadIdx.x == 0 && (int)c.epoch < p.timeline_pitch)
        p.timeline[((size_t)blockIdx.x * p.timeline_pitch + c.epoch) * 8 + k] = clock64();   // SM cycles
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
    uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ int atom_add_acq_rel_gpu(int* addr, int v) {
    int old;
    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], %2;\n" : "=r"(old) : "l"(addr), "r"(v) : "memory");
    return old;
}

__device__ __forceinline__ void raise_error(const FwdParams& p, Ctx& c, int code) {
    *c.abort_flag = 1;
    atomicCAS(p.sync + kSyncErr, 0, code);
}

// Device-wide barrier.  Arrival: after the consumer warps of the CTA have met, one thread makes the CTA's
// writes visible and adds one to one of kBarLanes arrival counters (CTA b uses counter b % kBarLanes).
// Departure: warp 0 polls for the CTA (lanes 0..kBarLanes-1 read one counter each with an acquire load: one
// 32-byte sector per poll) and releases the other consumer warps through the CTA's named barrier; the producer
// warp polls the same counters itself when it first needs the previous phase's output, so the activation
// copies of the next phase are issued the moment the barrier opens, not after a relay through shared memory
// (measured: a 0.5B-shape pass of 120 barriers went from 929 to 835 us).  The counters only grow during a
// launch (counter j must reach barriers * CTAs that use j); the last CTA to leave the kernel resets them.
// Every poll loop is bounded.
__device__ __forceinline__ bool grid_poll(const FwdParams& p, uint32_t nbar, int lane, uint32_t limit, volatile int* abort_flag) {
    const int mine = lane < kBarLanes ? ((int)gridDim.x + kBarLanes - 1 - lane) / kBarLanes : 0;   // CTAs on counter `lane`
    const int target = (int)nbar * mine;
    const int* ctr = p.sync + kSyncBar + (lane < kBarLanes ? lane : 0);
    for (uint32_t i = 0; i < limit; i++) {
        const bool ok = lane >= kBarLanes || ld_acquire(ctr) >= target;
        if (__all_sync(0xffffffffu, ok)) return true;
        if ((i & 63u) == 63u && *abort_flag) return false;
    }
    return false;
}

__device__ void grid_barrier(const FwdParams& p, Ctx& c) {
    c.epoch++;
    c.lbar++;
    consumer_sync(kNCons);
    long long* tl = nullptr;
    if (threadIdx.x == 0 && !*c.abort_flag) {
        if (p.timeline != nullptr && (int)c.epoch <= p.timeline_pitch) {
            tl = p.timeline + ((size_t)blockIdx.x * p.timeline_pitch + (c.epoch - 1)) * 8;
            tl[0] = global_ns();
        }
        __threadfence();               // cumulative: covers the CTA's writes ordered before the bar.sync
        fence_proxy_async_all();
        atomicAdd(p.sync + kSyncBar + (blockIdx.x % kBarLanes), 1);
    }
    // warp 0 polls for the CTA (every warp polling for itself was measured slower: 9 x 148 pollers on one sector)
    if (c.warp == 0 && !*c.abort_flag) {
        if (!grid_poll(p, c.lbar, c.lane, p.grid_wait_limit, c.abort_flag) && c.lane == 0 && !*c.abort_flag) raise_error(p, c, 10);
    }
    consumer_sync(kNCons);
    if (tl != nullptr) {
        tl[1] = global_ns();
        tl[7] = clock64();             // same instant in SM cycles, the origin of the next phase's stamps
    }
}

// Producer side: the whole warp calls it before the first activation copy of a phase; it only
// observes the counters.  Returns false on timeout / abort.
__device__ bool producer_grid_wait(const FwdParams& p, Ctx& c, uint32_t need_lbar) {
    bool ok = true;
    if (need_lbar > 0) {
        ok = !*c.abort_flag && grid_poll(p, need_lbar, c.lane, p.grid_wait_limit << 4, c.abort_flag);
        if (!ok && c.lane == 0 && !*c.abort_flag) raise_error(p, c, 11);
        __syncwarp();
    }
    fence_proxy_async_all();       // activations were written through the generic proxy by other CTAs
    return ok;
}

// The ring memory has two geometries: NST matmul stages, or `ans` slots of one 64-key K/V block each
// (attention).  Producer side of a geometry switch: wait until the consumers have released
// everything issued so far in the other geometry.
template <int MT>
__device__ __forceinline__ bool drain_stages(const FwdParams& p, Ctx& c) {
    using G = Geo<MT>;
    bool ok = true;
    for (uint32_t s = c.pos > (uint32_t)G::NST ? c.pos - G::NST : 0; s < c.pos; s++)
        ok = ok && fwd_wait(smem_u32(c.empty + s % G::NST), (s / G::NST) & 1u);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok && c.lane == 0) raise_error(p, c, 8);
    return ok;
}
__device__ __forceinline__ bool drain_blocks(const FwdParams& p, Ctx& c) {
    const uint32_t ns = (uint32_t)c.ans;
    bool ok = true;
    for (uint32_t n = c.apos > ns ? c.apos - ns : 0; n < c.apos; n++)
        ok = ok && fwd_wait(smem_u32(c.aempty + n % ns), (n / ns) & 1u);
    ok = __all_sync(0xffffffffu, ok);
    if (!ok && c.lane == 0) raise_error(p, c, 9);
    return ok;
}

// ================================================================================ tensor parallelism
// This GPU's buffer of fp32 partial products for the exchange in progress (two buffers, used in turn, so
// that a GPU that is one exchange ahead never overwrites what a slower peer is still reading).
__device__ __forceinline__ float* tp_partial_of(const FwdParams& p, int rank, uint32_t x) {
    return reinterpret_cast<float*>(p.tp_peers[rank] + kTpHeader) + (size_t)(x & 1u) * 32 * p.H;
}
__device__ __forceinline__ float* tp_partial(const FwdParams& p, const Ctx& c) {
    return tp_partial_of(p, p.tp_rank, c.tp_seq0 + c.tpx);
}
// Push form: the buffer of GPU `dst` holds one slot of partial products per source rank (again two sets used in
// turn); a GPU stores its products into its slot on every GPU, so that after the all-GPU barrier each GPU adds up
// what lies in its own memory.
constexpr int kTpPushMinWorld = 2;      // groups of at least this many GPUs use the push form unless told otherwise
__device__ __forceinline__ size_t tp_push_base(const FwdParams& p) {
    return (size_t)kTpHeader + (size_t)2 * 32 * p.H * sizeof(float) + (size_t)2 * 32 * p.H * sizeof(__half);
}
__device__ __forceinline__ float* tp_push_of(const FwdParams& p, int dst, int src, uint32_t x) {
    return reinterpret_cast<float*>(p.tp_peers[dst] + tp_push_base(p)) + ((size_t)(x & 1u) * kMaxTp + src) * 32 * p.H;
}
// Where rank `r`'s partial products of exchange x are read from by this GPU.
__device__ __forceinline__ const float* tp_source_of(const FwdParams& p, int r, uint32_t x) {
    return p.tp_push ? tp_push_of(p, p.tp_rank, r, x) : tp_partial_of(p, r, x);
}
__device__ __forceinline__ float4 ld_sys_f4(const float* q) {
    float4 v;
    asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];\n"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(q) : "memory");
    return v;
}

// Barrier over all CTAs of all GPUs of the group.  Thread 0 of every CTA makes the CTA's writes visible
// system-wide; then, in the hierarchical form (always with the two-step exchange, on request with the one-step
// exchange), it takes a ticket on its own GPU's CTA counter, and the CTA that takes the last ticket adds one to the
// GPU-level arrival counter in every GPU's exchange buffer (its own included, release at system scope): ONE remote
// atomic per peer and barrier instead of one per CTA; otherwise every CTA adds one to every GPU's counter itself.  Every CTA then waits
// (bounded) until its own GPU's counter shows all arrivals.  `nbar` = all-GPU barriers completed since
// the buffers were last zeroed (the same on every GPU); counters only grow (compared modulo 2^32).
__device__ void tp_all_barrier(const FwdParams& p, Ctx& c, uint32_t nbar) {
    c.epoch++;
    consumer_sync(kNCons);
    if (threadIdx.x == 0 && !*c.abort_flag) {
        long long* tl = nullptr;
        if (p.timeline != nullptr && (int)c.epoch <= p.timeline_pitch) {
            tl = p.timeline + ((size_t)blockIdx.x * p.timeline_pitch + (c.epoch - 1)) * 8;
            tl[0] = global_ns();
        }
        __threadfence_system();
        fence_proxy_async_all();
        unsigned char* own = p.tp_peers[p.tp_rank];
        unsigned target;
        if (p.tp_hier) {
            // one remote atomic per GPU and barrier (the last CTA's), not one per CTA
            const unsigned ticket = atomicAdd(reinterpret_cast<unsigned*>(own + kTpFwdLocal), 1u);
            if (ticket + 1u == (nbar + 1u) * gridDim.x) {      // the last CTA of this GPU: tell every GPU
                __threadfence_system();                        // the other CTAs' writes, ordered before their tickets
                for (int r = 0; r < p.tp_world; r++) {
                    const int q = (p.tp_rank + r) % p.tp_world;    // own counter first
                    unsigned* cnt = reinterpret_cast<unsigned*>(p.tp_peers[q] + kTpFwdArrive);
                    asm volatile("red.release.sys.global.add.u32 [%0], 1;\n" ::"l"(cnt) : "memory");
                }
            }
            target = (nbar + 1u) * (unsigned)p.tp_world;
        } else {
            // every CTA adds one to every GPU's counter directly (one hop less on the critical path)
            for (int r = 0; r < p.tp_world; r++) {
                const int q = (p.tp_rank + r) % p.tp_world;
                unsigned* cnt = reinterpret_cast<unsigned*>(p.tp_peers[q] + kTpFwdArrive);
                asm volatile("red.relaxed.sys.global.add.u32 [%0], 1;\n" ::"l"(cnt) : "memory");   // ordered by the fence above
            }
            target = (nbar + 1u) * (unsigned)p.tp_world * gridDim.x;
        }
        const unsigned* mine = reinterpret_cast<const unsigned*>(own + kTpFwdArrive);
        bool ok = false;
        for (uint32_t i = 0; i < p.tp_wait_limit; i++) {
            if ((int)(ld_acquire_sys(mine) - target) >= 0) { ok = true; break; }
        }
        if (!ok) raise_error(p, c, 12);
        __threadfence();
        if (tl != nullptr) {
            tl[1] = global_ns();
            tl[7] = clock64();
        }
    }
    consumer_sync(kNCons);
}

// The all-reduce of a row-parallel layer, after the all-GPU barrier that follows the partial products: all
// consumer threads add the ranks' partial products in rank order (pull form: plain loads, the peers' over NVLink;
// push form: the slots the ranks stored into this GPU's buffer during the matmul phase), add
// the residual and write h, h*w and the sums of squares exactly like the single-GPU epilogue.
// (Not inlined: its registers, one pair of loads per rank, stay out of the matmul phases' allocation.)
__device__ __noinline__ void tp_reduce_rows(const FwdParams& p, const __half* wn, uint32_t xchg) {
    const int upt = p.H / 4;                           // 4-column units per token row: a warp reads 512 contiguous bytes
    const int units = p.M * upt;
    const int units32 = (units + 31) & ~31;
    const int stride = gridDim.x * kNCons;
    // two units per thread and trip, all ranks' loads of both in flight together (a peer's take microseconds)
    for (int i0 = blockIdx.x * kNCons + threadIdx.x; i0 < units32; i0 += 2 * stride) {
        float4 u[2][kMaxTp];
        int tok[2], n0[2];
        bool valid[2];
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int i = i0 + j * stride;
            valid[j] = i < units;
            tok[j] = valid[j] ? i / upt : 0;
            n0[j] = valid[j] ? (i - tok[j] * upt) * 4 : 0;
#pragma unroll
            for (int r = 0; r < kMaxTp; r++)
                if (r < p.tp_world && valid[j])
                    u[j][r] = ld_sys_f4(tp_source_of(p, r, xchg) + (size_t)tok[j] * p.H + n0[j]);
        }
#pragma unroll
        for (int j = 0; j < 2; j++) {
            if (i0 + j * stride >= units32) break;              // warp-uniform
            float ss = 0.f;
            if (valid[j]) {
                const uint2 rv = __ldcg(reinterpret_cast<const uint2*>(p.h + (size_t)tok[j] * p.H + n0[j]));
                const uint2 wv = *reinterpret_cast<const uint2*>(wn + n0[j]);
                float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int r = 0; r < kMaxTp; r++) {             // rank order: every GPU rounds identically
                    if (r < p.tp_world) { a[0] += u[j][r].x; a[1] += u[j][r].y; a[2] += u[j][r].z; a[3] += u[j][r].w; }
                }
                const __half* rh = reinterpret_cast<const __half*>(&rv);
                const __half* wh = reinterpret_cast<const __half*>(&wv);
                __align__(8) __half out[4], hw[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    out[e] = __hadd(rh[e], __float2half_rn(a[e]));
                    const float fv = __half2float(out[e]);
                    ss += fv * fv;
                    hw[e] = __hmul(out[e], wh[e]);
                }
                *reinterpret_cast<uint2*>(p.h + (size_t)tok[j] * p.H + n0[j]) = *reinterpret_cast<const uint2*>(out);
                *reinterpret_cast<uint2*>(p.hw + xt_index(tok[j], n0[j], p.mp)) = *reinterpret_cast<const uint2*>(hw);
            }
            ss += __shfl_xor_sync(0xffffffffu, ss, 1);          // the four 4-column quarters of a 16-column part
            ss += __shfl_xor_sync(0xffffffffu, ss, 2);
            if (valid[j] && (threadIdx.x & 3) == 0) p.ssq[(n0[j] >> 4) * kSsqPitch + tok[j]] = ss;
        }
    }
}

// Two-step variant, on request (the pull form makes every GPU read (N-1) whole partial buffers per exchange;
// measured on 4 GPUs the second all-GPU barrier of this form costs more than the reads it saves, so it is not the default).
// Shot one: GPU r adds, for ITS slice of H / N columns only, the partial products of all ranks (rank order) and
// the residual, and stores the fp16 result into the gather area of every GPU's exchange buffer (plain stores,
// the peers' over NVLink).  After another all-GPU barrier, shot two: every GPU turns the gathered rows into h,
// h*w and the sums of squares, exactly like the single-GPU epilogue; all GPUs hold bit-identical hidden states.
__device__ __forceinline__ __half* tp_gather_of(const FwdParams& p, int rank, uint32_t x) {
    return reinterpret_cast<__half*>(p.tp_peers[rank] + kTpHeader + (size_t)2 * 32 * p.H * sizeof(float)) + (size_t)(x & 1u) * 32 * p.H;
}

__device__ __noinline__ void tp_reduce_scatter(const FwdParams& p, uint32_t xchg) {
    const int W = p.H / p.tp_world;                    // columns this GPU reduces (a multiple of 16)
    const int upt = W / 4;
    const int units = p.M * upt;
    const int stride = gridDim.x * kNCons;
    for (int i = blockIdx.x * kNCons + threadIdx.x; i < units; i += stride) {
        const int tok = i / upt;
        const int n0 = p.tp_rank * W + (i - tok * upt) * 4;
        float4 u[kMaxTp];
#pragma unroll
        for (int r = 0; r < kMaxTp; r++)               // all ranks' loads in flight together
            if (r < p.tp_world) u[r] = ld_sys_f4(tp_partial_of(p, r, xchg) + (size_t)tok * p.H + n0);
        const uint2 rv = __ldcg(reinterpret_cast<const uint2*>(p.h + (size_t)tok * p.H + n0));
        float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < kMaxTp; r++) {             // rank order: the sum does not depend on who computes it
            if (r < p.tp_world) { a[0] += u[r].x; a[1] += u[r].y; a[2] += u[r].z; a[3] += u[r].w; }
        }
        const __half* rh = reinterpret_cast<const __half*>(&rv);
        __align__(8) __half out[4];
#pragma unroll
        for (int e = 0; e < 4; e++) out[e] = __hadd(rh[e], __float2half_rn(a[e]));
        const uint2 ov = *reinterpret_cast<const uint2*>(out);
#pragma unroll
        for (int r = 0; r < kMaxTp; r++) {
            if (r < p.tp_world) {
                uint2* dst = reinterpret_cast<uint2*>(tp_gather_of(p, r, xchg) + (size_t)tok * p.H + n0);
                asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};\n" ::"l"(dst), "r"(ov.x), "r"(ov.y) : "memory");
            }
        }
    }
}

__device__ __noinline__ void tp_finalize_rows(const FwdParams& p, const __half* wn, uint32_t xchg) {
    const int upt = p.H / 4;
    const int units = p.M * upt;
    const int units32 = (units + 31) & ~31;
    const int stride = gridDim.x * kNCons;
    const __half* gathered = tp_gather_of(p, p.tp_rank, xchg);
    for (int i = blockIdx.x * kNCons + threadIdx.x; i < units32; i += stride) {
        const bool valid = i < units;
        const int tok = valid ? i / upt : 0;
        const int n0 = valid ? (i - tok * upt) * 4 : 0;
        float ss = 0.f;
        if (valid) {
            uint2 hv;
            asm volatile("ld.relaxed.sys.global.v2.u32 {%0, %1}, [%2];\n" : "=r"(hv.x), "=r"(hv.y)
                         : "l"(gathered + (size_t)tok * p.H + n0) : "memory");
            const uint2 wv = *reinterpret_cast<const uint2*>(wn + n0);
            const __half* hh = reinterpret_cast<const __half*>(&hv);
            const __half* wh = reinterpret_cast<const __half*>(&wv);
            __align__(8) __half hw[4];
#pragma unroll
            for (int e = 0; e < 4; e++) {
                const float fv = __half2float(hh[e]);
                ss += fv * fv;
                hw[e] = __hmul(hh[e], wh[e]);
            }
            *reinterpret_cast<uint2*>(p.h + (size_t)tok * p.H + n0) = hv;
            *reinterpret_cast<uint2*>(p.hw + xt_index(tok, n0, p.mp)) = *reinterpret_cast<const uint2*>(hw);
        }
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);              // the four 4-column quarters of a 16-column part
        ss += __shfl_xor_sync(0xffffffffu, ss, 2);
        if (valid && (threadIdx.x & 3) == 0) p.ssq[(n0 >> 4) * kSsqPitch + tok] = ss;
    }
}

__device__ __forceinline__ void tp_reduce_phase(const FwdParams& p, Ctx& c, const __half* wn) {
    const uint32_t xchg = c.tp_seq0 + c.tpx;
    consumer_sync(kNCons);
    if (p.tp_two_shot) {
        if (!*c.abort_flag) tp_reduce_scatter(p, xchg);
        tp_all_barrier(p, c, xchg * 2u + 1u);
        if (!*c.abort_flag) tp_finalize_rows(p, wn, xchg);
    } else if (!*c.abort_flag) {
        tp_reduce_rows(p, wn, xchg);
    }
    c.tpx++;
}

// ================================================================================ QMM phases
// Item = (group of TPI = 8/kw 16-row tiles [tile pairs gate/up in dual mode], K range).  The eight
// consumer warps are arranged as TPI tiles x kw K-parts: warp (j, i) owns tile j of the item and, in
// every ring stage, the chunks i, i+kw, ... of that stage.  The K-parts of a tile are added in
// shared memory in part order, so small matrices need no split-K through global memory.  A stage
// holds CPS chunks (the planner takes as many as fit: narrow items leave most of the stage to the
// activations, so that a whole K of a few thousand is in flight when the barrier opens): for every chunk
// the TPI records of the item's tiles (contiguous in the streaming layout for TPI <= 4), then the same
// for up_proj in dual mode, then, right behind the weights, the activations of the stage's K range
// (one bulk copy: they are contiguous in the chunk-major layout).

// rstd[m] = rsqrt(mean(h[m]^2) + eps) from the per-16-column sums of squares the producer of h left in p.ssq, by
// the PRODUCER warp, once per phase, right after it has issued the phase's first activation copies: the loads
// (one 128-byte line per part) overlap the weight stream, and the consumers find the result in shared memory
// when they reach their first epilogue (they wait, bounded, on rbar).  Fixed summation order.
__device__ __forceinline__ void producer_rstd(const FwdParams& p, Ctx& c, int rows) {
    const int parts = p.H / 16;
    const int nq = rows <= 8 ? 2 : (rows <= 16 ? 4 : 8);         // token quads (float4 of a part's line)
    const int np = 32 / nq;                                       // parts read side by side
    const int tq = c.lane % nq, pq = c.lane / nq;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int base = 0; base < parts; base += 8 * np) {
        float4 v[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {                             // eight independent loads in flight per lane
            const int part = base + i * np + pq;
            v[i] = part < parts ? __ldcg(reinterpret_cast<const float4*>(p.ssq + part * kSsqPitch) + tq)
                                : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) { acc.x += v[i].x; acc.y += v[i].y; acc.z += v[i].z; acc.w += v[i].w; }
    }
    for (int o = nq; o < 32; o <<= 1) {
        acc.x += __shfl_xor_sync(0xffffffffu, acc.x, o);
        acc.y += __shfl_xor_sync(0xffffffffu, acc.y, o);
        acc.z += __shfl_xor_sync(0xffffffffu, acc.z, o);
        acc.w += __shfl_xor_sync(0xffffffffu, acc.w, o);
    }
    if (pq == 0) {
        const float hh = (float)p.H;
        const int m = tq * 4;
        if (m < rows) c.s_rstd[m] = rsqrtf(acc.x / hh + p.eps);
        if (m + 1 < rows) c.s_rstd[m + 1] = rsqrtf(acc.y / hh + p.eps);
        if (m + 2 < rows) c.s_rstd[m + 2] = rsqrtf(acc.z / hh + p.eps);
        if (m + 3 < rows) c.s_rstd[m + 3] = rsqrtf(acc.w / hh + p.eps);
    }
    __syncwarp();
    if (c.lane == 0) mbar_arrive(smem_u32(c.rbar));              // release: orders the stores above
}

// Streams the weight records (and activation rows) of this CTA's items into the ring.
// `need_epoch`: device-wide barriers that must have completed before the activations may be read.
template <int MT>
__device__ __forceinline__ void qmm_produce(const FwdParams& p, Ctx& c, const QDesc& d, uint32_t need_epoch,
                                            const bool dual, const bool need_rstd) {
    using G = Geo<MT>;
    const int lane = c.lane;
    const int kw = d.pl.kw;
    const int TPI = kWN / kw, CPS = d.pl.cps;
    const int chunk_bytes = TPI * kRec;
    const int up_off = CPS * chunk_bytes;
    const int x_off = (dual ? 2 : 1) * up_off;            // the activations follow the weights of the stage
    const int nchunks_total = d.K / kChunkK;
    const int nblocks = (d.N + 63) / 64;
    const int nitems = d.pl.row_items * d.pl.splits;
    if ((int)blockIdx.x >= nitems) return;
    if (c.apos > 0 && !drain_blocks(p, c)) return;        // key-block slots overlay the stages

    const uint64_t wpolicy = make_evict_first_policy();   // weights are read once per pass: do not let them crowd L2
    bool ready = false;
    int npend = 0;
    uint32_t pend_slot[G::NST];
    int pend_k0[G::NST], pend_recs[G::NST];

    // A bulk copy occupies the issuing warp for ~0.3 us whatever its size, but the lanes of ONE instruction issue
    // side by side: all copies of a stage (weights and activations) therefore go out in a single instruction.
    const uint64_t xpolicy = make_evict_normal_policy();
    auto x_src = [&](int k0) { return reinterpret_cast<const unsigned char*>(d.x + (size_t)(k0 >> 7) * G::MP * kXRowH); };
    auto flush = [&]() -> bool {
        if (!producer_grid_wait(p, c, need_epoch)) return false;
        uint32_t my_slot = 0;
        int my_k0 = 0, my_recs = 0;
#pragma unroll
        for (int i = 0; i < G::NST; i++)
            if (lane == i) { my_slot = pend_slot[i]; my_k0 = pend_k0[i]; my_recs = pend_recs[i]; }
        if (lane < npend)          // the activation runs of the stages queued before the barrier opened
            bulk_copy_g2s_hint(smem_u32(c.ring + my_slot * G::STAGE + x_off), x_src(my_k0), (uint32_t)(my_recs * G::MP * kXRow),
                               smem_u32(c.full + my_slot), xpolicy);
        npend = 0;
        ready = true;
        if (need_rstd) {
            producer_rstd(p, c, d.xrows);
            c.ruse++;
        }
        return true;
    };

    for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
        const int row_item = item % d.pl.row_items;
        const int split = item / d.pl.row_items;
        const int c_begin = split * d.pl.chunks_per_split;
        const int n = min(d.pl.chunks_per_split, nchunks_total - c_begin);
        const int nst = (n + CPS - 1) / CPS;
        const bool last_item = item + (int)gridDim.x >= nitems;
        const int t0 = row_item * TPI;                     // first 16-row tile of the item
        const int blk0 = min(t0 >> 2, nblocks - 1), blk1 = min((t0 >> 2) + 1, nblocks - 1);
        // the epilogue's per-column vectors (bias, next norm weight) are first touched there: pull them into L2 now
        if (lane < 2) {
            const __half* vec = lane == 0 ? d.bias : d.wn;
            const int col = t0 * 16 + 0;
            if (vec != nullptr && col < d.N) {
                asm volatile("prefetch.global.L2 [%0];\n" ::"l"(vec + col));
                if (TPI * 16 > 64 && col + 64 < d.N) asm volatile("prefetch.global.L2 [%0];\n" ::"l"(vec + col + 64));
            }
        }
        for (int st = 0; st < nst; st++, c.pos++) {
            const uint32_t slot = c.pos % G::NST, use = c.pos / G::NST;
            if (*c.abort_flag) return;
            if (use > 0 && !__all_sync(0xffffffffu, fwd_wait(smem_u32(c.empty + slot), (use - 1) & 1u))) {
                if (lane == 0) raise_error(p, c, 2);
                return;
            }
            const int recs = min(CPS, n - st * CPS);
            const uint32_t fbar = smem_u32(c.full + slot);
            const int nmat = dual ? 2 : 1;
            if (lane == 0) {
                fence_proxy_async();
                mbar_expect_tx(fbar, (uint32_t)(nmat * recs * chunk_bytes) + (uint32_t)(recs * G::MP * kXRow));
            }
            __syncwarp();
            unsigned char* stage = c.ring + slot * G::STAGE;
            const size_t ch0 = (size_t)(c_begin + st * CPS);
            const int k0 = (c_begin + st * CPS) * kChunkK;
            // lanes 0 .. ncw-1: the weight runs; lane ncw: the activation run (once the previous phase's output is visible)
            int ncw;
            uint32_t cdst = 0, cbytes = 0;
            const unsigned char* csrc = nullptr;
            if (TPI >= 4) {
                // whole 64-row blocks: the stage's chunks of a block are one contiguous run
                const int nb = TPI / 4;
                ncw = nb * nmat;
                if (lane < ncw) {
                    const int mtx = lane / nb, b = lane - mtx * nb;
                    const unsigned char* wbase = mtx ? d.w1 : d.w0;
                    cdst = smem_u32(stage + mtx * up_off + b * CPS * 4 * kRec);
                    csrc = wbase + ((size_t)(b ? blk1 : blk0) * nchunks_total + ch0) * 4 * kRec;
                    cbytes = (uint32_t)(recs * 4 * kRec);
                }
            } else {
                ncw = recs * nmat;                                        // part of a block: one copy per chunk (<= 16)
                if (lane < ncw) {
                    const int mtx = lane / recs, cc = lane - mtx * recs;
                    const unsigned char* wbase = mtx ? d.w1 : d.w0;
                    cdst = smem_u32(stage + mtx * up_off + cc * chunk_bytes);
                    csrc = wbase + (((size_t)blk0 * nchunks_total + ch0 + cc) * 4 + (t0 & 3)) * kRec;
                    cbytes = (uint32_t)chunk_bytes;
                }
            }
            const bool xlane = ready && lane == ncw;
            if (xlane) {
                cdst = smem_u32(stage + x_off);
                csrc = x_src(k0);
                cbytes = (uint32_t)(recs * G::MP * kXRow);
            }
            if (lane < ncw || xlane) bulk_copy_g2s_hint(cdst, csrc, cbytes, fbar, xlane ? xpolicy : wpolicy);
            if (!ready) {
#pragma unroll
                for (int i = 0; i < G::NST; i++)
                    if (i == npend) { pend_slot[i] = slot; pend_k0[i] = k0; pend_recs[i] = recs; }
                npend++;
                if (npend == G::NST || (last_item && st == nst - 1)) {
                    if (!flush()) return;
                }
            }
        }
    }
}

// Output row of token row `tok` in a row-major result, or -1 if the row is not stored.
template <bool BATCH>
__device__ __forceinline__ int out_row(const QDesc& d, int tok) {
    if (BATCH) return out_row_tab()[d.orow_sel * 32 + tok];
    return (tok >= d.row_lo && tok < d.row_lo + d.row_cnt) ? tok - d.row_lo : -1;
}

template <int MT, bool DUAL, bool TP, bool FAST, bool BATCH>
__device__ __forceinline__ void qmm_consume(const FwdParams& p, Ctx& c, const QDesc& d, const int EPI) {
    using G = Geo<MT>;
    constexpr int S = DUAL ? 2 : 1;
    constexpr int MP = MT * 8;
    const int lane = c.lane, warp = c.warp;
    const int g = lane >> 2, t = lane & 3;
    const int kw = d.pl.kw;
    const int TPI = kWN / kw, CPS = d.pl.cps;
    const int R = TPI * 16;                      // output rows (of each matrix) per item
    const int TW = S * R;
    const int chunk_bytes = TPI * kRec;
    const int up_off = CPS * chunk_bytes;
    const int x_off = S * up_off;
    const int tj = warp / kw, ki = warp - tj * kw;    // tile of the item, K-part
    // record of (chunk cc of the stage, tile tj): whole blocks arrive as [block][chunk][4 tiles], parts of a block as [chunk][tiles]
    const int rec_base = (TPI >= 4) ? ((tj >> 2) * CPS * 4 * kRec + (tj & 3) * kRec) : tj * kRec;
    const int rec_cstride = (TPI >= 4) ? 4 * kRec : chunk_bytes;
    const int nchunks_total = d.K / kChunkK;
    const int nitems = d.pl.row_items * d.pl.splits;
    const bool need_rstd = (EPI != EPI_RESID && !(TP && EPI == EPI_TP));
    constexpr bool fast = FAST;                   // every scale of the model is in the range of dequant_pack_fast
    stamp(p, c, 2);
    bool rstd_done = !need_rstd;

    for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
        const int row_item = item % d.pl.row_items;
        const int split = item / d.pl.row_items;
        const int c_begin = split * d.pl.chunks_per_split;
        const int n = min(d.pl.chunks_per_split, nchunks_total - c_begin);
        const int nst = (n + CPS - 1) / CPS;

        float acc[S][MT][4];
#pragma unroll
        for (int s = 0; s < S; s++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[s][mt][i] = 0.f;

        for (int st = 0; st < nst; st++, c.pos++) {
            const uint32_t slot = c.pos % G::NST;
            bool ok = !*c.abort_flag;
            if (ok && !fwd_wait(smem_u32(c.full + slot), (c.pos / G::NST) & 1u)) {
                ok = false;
                if (lane == 0) raise_error(p, c, 1);
            }
            ok = __all_sync(0xffffffffu, ok);      // warp-uniform: the MMA path below needs all lanes
            if (st == 0 && item == (int)blockIdx.x) stamp(p, c, 4);
            if (ok) {
                const unsigned char* stage = c.ring + slot * G::STAGE;
                const int nrec = min(CPS, n - st * CPS);
                // K-part ki owns the chunks of the ITEM whose index is ki modulo kw (stages need not hold a multiple of kw)
                const int first = (ki - st * CPS) & (kw - 1);       // kw is a power of two
                for (int cc = first; cc < nrec; cc += kw) {
                    const unsigned char* xrow = stage + x_off + (cc * MP + g) * kXRow + t * 16;
                    uint4 w[S][2];
                    uint2 sb[S][2];
#pragma unroll
                    for (int s = 0; s < S; s++) {
                        const unsigned char* rec = stage + s * up_off + cc * rec_cstride + rec_base;
                        w[s][0] = *reinterpret_cast<const uint4*>(rec + lane * 16);
                        w[s][1] = *reinterpret_cast<const uint4*>(rec + 512 + lane * 16);
                        sb[s][0] = *reinterpret_cast<const uint2*>(rec + 1024 + g * 8);
                        sb[s][1] = *reinterpret_cast<const uint2*>(rec + 1024 + (8 + g) * 8);
                    }
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        uint4 xb[MT];
#pragma unroll
                        for (int mt = 0; mt < MT; mt++)
                            xb[mt] = *reinterpret_cast<const uint4*>(xrow + mt * 8 * kXRow + ((j ^ (g & 1)) << 6));
#pragma unroll
                        for (int s = 0; s < S; s++) {
                            const __half2 p0 = u32_as_h2((j < 2) ? sb[s][0].x : sb[s][0].y);   // {scale, bias}
                            const __half2 p1 = u32_as_h2((j < 2) ? sb[s][1].x : sb[s][1].y);
                            uint32_t d0[4], d1[4];
                            if (fast) {
                                dequant_pack_fast(comp(w[s][0], j), scale_times_2_20(__low2half2(p0)), __high2half2(p0), d0);
                                dequant_pack_fast(comp(w[s][1], j), scale_times_2_20(__low2half2(p1)), __high2half2(p1), d1);
                            } else {
                                dequant_pack(comp(w[s][0], j), __low2half2(p0), __high2half2(p0), d0);
                                dequant_pack(comp(w[s][1], j), __low2half2(p1), __high2half2(p1), d1);
                            }
#pragma unroll
                            for (int mt = 0; mt < MT; mt++) {
                                mma_m16n8k16(acc[s][mt], d0[0], d1[0], d0[1], d1[1], xb[mt].x, xb[mt].y);
                                mma_m16n8k16(acc[s][mt], d0[2], d1[2], d0[3], d1[3], xb[mt].z, xb[mt].w);
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(c.empty + slot));
        }

        stamp(p, c, 5);
        if (!rstd_done) {             // the per-token 1/rms of the input (needed by the epilogue only): from the producer warp
            bool rok = !*c.abort_flag && fwd_wait(smem_u32(c.rbar), c.ruse & 1u);
            if (!__all_sync(0xffffffffu, rok) && lane == 0 && !*c.abort_flag) raise_error(p, c, 13);
            c.ruse++;
            rstd_done = true;
        }
        // ---- K-parts of a tile -> its first warp, through shared memory, in part order
        if (kw > 1) {
            float4* sc = reinterpret_cast<float4*>(c.scratch);
            if (ki != 0) {
#pragma unroll
                for (int s = 0; s < S; s++)
#pragma unroll
                    for (int mt = 0; mt < MT; mt++)
                        sc[((warp * S + s) * MT + mt) * 32 + lane] =
                            make_float4(acc[s][mt][0], acc[s][mt][1], acc[s][mt][2], acc[s][mt][3]);
            }
            consumer_sync(kNCons);
            if (ki == 0) {
                for (int i = 1; i < kw; i++) {
#pragma unroll
                    for (int s = 0; s < S; s++)
#pragma unroll
                        for (int mt = 0; mt < MT; mt++) {
                            const float4 v = sc[(((warp + i) * S + s) * MT + mt) * 32 + lane];
                            acc[s][mt][0] += v.x; acc[s][mt][1] += v.y; acc[s][mt][2] += v.z; acc[s][mt][3] += v.w;
                        }
                }
            }
            consumer_sync(kNCons);         // scratch is rewritten by the next item
        }
        const bool leader = (ki == 0);
        stamp(p, c, 6);

        // lane (g,t) of a tile's first warp holds, per matrix and token tile: rows g / g+8 x tokens 2t / 2t+1
        const int tile_global = row_item * TPI + tj;
        if (d.pl.splits > 1) {
            // ---- split-K across CTAs: partial sums through global memory, last CTA of the row item reduces
            float* mine = p.partial + ((size_t)split * d.pl.row_items + row_item) * MP * TW;
            if (leader) {
#pragma unroll
                for (int s = 0; s < S; s++) {
                    const int ri = s * R + tj * 16;
#pragma unroll
                    for (int mt = 0; mt < MT; mt++) {
                        const int tok = mt * 8 + 2 * t;
                        mine[(size_t)tok * TW + ri + g] = acc[s][mt][0];
                        mine[(size_t)(tok + 1) * TW + ri + g] = acc[s][mt][1];
                        mine[(size_t)tok * TW + ri + g + 8] = acc[s][mt][2];
                        mine[(size_t)(tok + 1) * TW + ri + g + 8] = acc[s][mt][3];
                    }
                }
            }
            consumer_sync(kNCons);
            if (threadIdx.x == 0) {
                // one acquire-release ticket: releases this CTA's partial sums (ordered before it by the bar.sync
                // above), and acquires the other splits' for the CTA that draws the last ticket
                const int old = atom_add_acq_rel_gpu(p.counter + row_item, 1);
                const int last = (old == d.pl.splits - 1);
                *c.is_last = last;
                if (last) p.counter[row_item] = 0;
            }
            consumer_sync(kNCons);
            if (*c.is_last) {
                const int UPT = R / 8;               // threads per token row
                const int units = d.xrows * UPT;
                const int units32 = (units + 31) & ~31;
                for (int i = threadIdx.x; i < units32; i += kNCons) {
                    const int tok = i / UPT;
                    const int c0 = (i - tok * UPT) * 8;
                    const int n0 = row_item * R + c0;
                    const bool valid = i < units && n0 < d.N;
                    float a0[8], a1[8];
#pragma unroll
                    for (int e = 0; e < 8; e++) a0[e] = a1[e] = 0.f;
                    // residual and norm weights of the epilogue: issued now, so that their latency runs with the
                    // partial sums' (h is read and written by this thread only)
                    uint4 rv = make_uint4(0, 0, 0, 0), wv = make_uint4(0, 0, 0, 0);
                    if (valid && EPI == EPI_RESID && !(TP && EPI == EPI_TP)) {
                        rv = __ldcg(reinterpret_cast<const uint4*>(p.h + (size_t)tok * d.N + n0));
                        wv = *reinterpret_cast<const uint4*>(d.wn + n0);
                    }
                    if (valid) {
                        // four splits' loads in flight at a time (a load from L2 takes the better part of a
                        // microsecond); added in split order, so the result does not depend on the batching
                        for (int sp0 = 0; sp0 < d.pl.splits; sp0 += 4) {
                            float4 u0[4], u1[4], v0[4], v1[4];
#pragma unroll
                            for (int j = 0; j < 4; j++) {          // past the last split: the last one again (weight 0 below)
                                const int sp = min(sp0 + j, d.pl.splits - 1);
                                const float* src = p.partial + ((size_t)sp * d.pl.row_items + row_item) * MP * TW + (size_t)tok * TW + c0;
                                u0[j] = __ldcg(reinterpret_cast<const float4*>(src));
                                u1[j] = __ldcg(reinterpret_cast<const float4*>(src) + 1);
                                if (DUAL) {
                                    v0[j] = __ldcg(reinterpret_cast<const float4*>(src + R));
                                    v1[j] = __ldcg(reinterpret_cast<const float4*>(src + R) + 1);
                                }
                            }
#pragma unroll
                            for (int j = 0; j < 4; j++) {
                                const float m = (sp0 + j < d.pl.splits) ? 1.f : 0.f;     // fma(1, x, a) == a + x
                                a0[0] = fmaf(m, u0[j].x, a0[0]); a0[1] = fmaf(m, u0[j].y, a0[1]);
                                a0[2] = fmaf(m, u0[j].z, a0[2]); a0[3] = fmaf(m, u0[j].w, a0[3]);
                                a0[4] = fmaf(m, u1[j].x, a0[4]); a0[5] = fmaf(m, u1[j].y, a0[5]);
                                a0[6] = fmaf(m, u1[j].z, a0[6]); a0[7] = fmaf(m, u1[j].w, a0[7]);
                                if (DUAL) {
                                    a1[0] = fmaf(m, v0[j].x, a1[0]); a1[1] = fmaf(m, v0[j].y, a1[1]);
                                    a1[2] = fmaf(m, v0[j].z, a1[2]); a1[3] = fmaf(m, v0[j].w, a1[3]);
                                    a1[4] = fmaf(m, v1[j].x, a1[4]); a1[5] = fmaf(m, v1[j].y, a1[5]);
                                    a1[6] = fmaf(m, v1[j].z, a1[6]); a1[7] = fmaf(m, v1[j].w, a1[7]);
                                }
                            }
                        }
                    }
                    __align__(16) __half out[8];
                    if (TP && EPI == EPI_TP) {
                        if (valid && p.tp_push) {
                            const size_t at = (size_t)tok * d.N + n0;
                            for (int r = 1; r <= p.tp_world; r++) {                   // the peers first, this GPU last
                                float* dst = tp_push_of(p, (p.tp_rank + r) % p.tp_world, p.tp_rank, c.tp_seq0 + c.tpx) + at;
                                *reinterpret_cast<float4*>(dst) = make_float4(a0[0], a0[1], a0[2], a0[3]);
                                *reinterpret_cast<float4*>(dst + 4) = make_float4(a0[4], a0[5], a0[6], a0[7]);
                            }
                        } else if (valid) {
                            float* dst = tp_partial(p, c) + (size_t)tok * d.N + n0;
                            *reinterpret_cast<float4*>(dst) = make_float4(a0[0], a0[1], a0[2], a0[3]);
                            *reinterpret_cast<float4*>(dst + 4) = make_float4(a0[4], a0[5], a0[6], a0[7]);
                        }
                    } else if (EPI == EPI_RESID) {
                        float ss = 0.f;
                        if (valid) {
                            const __half* rh = reinterpret_cast<const __half*>(&rv);
                            const __half* wh = reinterpret_cast<const __half*>(&wv);
                            __align__(16) __half hw[8];
#pragma unroll
                            for (int e = 0; e < 8; e++) {
                                out[e] = __hadd(rh[e], __float2half_rn(a0[e]));
                                const float f = __half2float(out[e]);
                                ss += f * f;
                                hw[e] = __hmul(out[e], wh[e]);
                            }
                            *reinterpret_cast<uint4*>(p.h + (size_t)tok * d.N + n0) = *reinterpret_cast<const uint4*>(out);
                            *reinterpret_cast<uint4*>(p.hw + xt_index(tok, n0, MP)) = *reinterpret_cast<const uint4*>(hw);
                        }
                        ss += __shfl_xor_sync(0xffffffffu, ss, 1);          // the two 8-column halves of a 16-row tile
                        if (valid && (lane & 1) == 0) p.ssq[(n0 >> 4) * kSsqPitch + tok] = ss;
                    } else if (valid) {
                        const float rs = c.s_rstd[tok];
                        if (DUAL) {
#pragma unroll
                            for (int e = 0; e < 8; e++) out[e] = __float2half_rn(silu_mul_f16(a0[e] * rs, a1[e] * rs));
                        } else {
#pragma unroll
                            for (int e = 0; e < 8; e++) out[e] = __float2half_rn(a0[e] * rs);
                            if (d.bias != nullptr) {
                                const uint4 bv = *reinterpret_cast<const uint4*>(d.bias + n0);
                                const __half* bh = reinterpret_cast<const __half*>(&bv);
#pragma unroll
                                for (int e = 0; e < 8; e++) out[e] = __hadd(out[e], bh[e]);
                            }
                        }
                        if (d.y_tiled) {
                            *reinterpret_cast<uint4*>(d.y + xt_index(tok, n0, MP)) = *reinterpret_cast<const uint4*>(out);
                        } else {
                            const int orow = out_row<BATCH>(d, tok);
                            if (orow >= 0) *reinterpret_cast<uint4*>(d.y + (size_t)orow * d.N + n0) = *reinterpret_cast<const uint4*>(out);
                        }
                    }
                }
            }
            consumer_sync(kNCons);     // is_last is rewritten by the next item
        } else if (leader) {
            // ---- direct epilogue from the registers of the tile's first warp
            const int nbase = tile_global * 16 + g;
            if (TP && EPI == EPI_TP) {
                const int ndst = p.tp_push ? p.tp_world : 1;
                for (int r = 1; r <= ndst; r++) {                                     // push form: the peers first, this GPU last
                    float* dst = p.tp_push ? tp_push_of(p, (p.tp_rank + r) % p.tp_world, p.tp_rank, c.tp_seq0 + c.tpx)
                                           : tp_partial(p, c);
#pragma unroll
                    for (int mt = 0; mt < MT; mt++) {
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const int tok = mt * 8 + 2 * t + (i & 1);
                            const int nn = nbase + ((i >> 1) ? 8 : 0);
                            if (tok < d.xrows && nn < d.N) dst[(size_t)tok * d.N + nn] = acc[0][mt][i];
                        }
                    }
                }
            } else if (EPI == EPI_RESID) {
                // residuals and norm weights first, all loads in flight together (h is read and written here)
                unsigned short res[MT][4];
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int tok = mt * 8 + 2 * t + (i & 1);
                        const int nn = nbase + ((i >> 1) ? 8 : 0);
                        res[mt][i] = (tok < d.xrows && nn < d.N)
                                         ? __ldcg(reinterpret_cast<const unsigned short*>(p.h) + (size_t)tok * d.N + nn) : (unsigned short)0;
                    }
                const __half wn0 = nbase < d.N ? d.wn[nbase] : __ushort_as_half(0);
                const __half wn8 = nbase + 8 < d.N ? d.wn[nbase + 8] : __ushort_as_half(0);
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    float ss0 = 0.f, ss1 = 0.f;            // tokens 2t, 2t+1 of this token tile
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int tok = mt * 8 + 2 * t + (i & 1);
                        const int nn = nbase + ((i >> 1) ? 8 : 0);
                        if (tok < d.xrows && nn < d.N) {
                            const __half r = __ushort_as_half(res[mt][i]);
                            const __half o = __hadd(r, __float2half_rn(acc[0][mt][i]));
                            const float f = __half2float(o);
                            if (i & 1) ss1 += f * f; else ss0 += f * f;
                            p.h[(size_t)tok * d.N + nn] = o;
                            p.hw[xt_index(tok, nn, MP)] = __hmul(o, (i >> 1) ? wn8 : wn0);
                        }
                    }
#pragma unroll
                    for (int o = 4; o < 32; o <<= 1) {
                        ss0 += __shfl_xor_sync(0xffffffffu, ss0, o);
                        ss1 += __shfl_xor_sync(0xffffffffu, ss1, o);
                    }
                    if (g == 0 && tile_global * 16 < d.N) {
                        const int tok = mt * 8 + 2 * t;
                        if (tok < d.xrows) p.ssq[tile_global * kSsqPitch + tok] = ss0;
                        if (tok + 1 < d.xrows) p.ssq[tile_global * kSsqPitch + tok + 1] = ss1;
                    }
                }
            } else {
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int tok = mt * 8 + 2 * t + (i & 1);
                        const int nn = nbase + ((i >> 1) ? 8 : 0);
                        if (tok >= d.xrows || nn >= d.N) continue;
                        const float rs = c.s_rstd[tok];
                        __half o;
                        if (DUAL) {
                            o = __float2half_rn(silu_mul_f16(acc[0][mt][i] * rs, acc[S - 1][mt][i] * rs));
                        } else {
                            o = __float2half_rn(acc[0][mt][i] * rs);
                            if (d.bias != nullptr) o = __hadd(o, d.bias[nn]);
                        }
                        if (d.y_tiled) {
                            d.y[xt_index(tok, nn, MP)] = o;
                        } else {
                            const int orow = out_row<BATCH>(d, tok);
                            if (orow >= 0) d.y[(size_t)orow * d.N + nn] = o;
                        }
                    }
                }
            }
        }
        stamp(p, c, 3);                // epilogue of the item issued
    }
}

// ================================================================================ phase 0
__device__ __forceinline__ void embed_phase(const FwdParams& p, Ctx& c) {
    const int lane = c.lane;
    const int NP = p.H / 128;
    const int units = p.M * NP;                         // (token, 128-column part), one half-warp each
    const int pairs = (units + 1) / 2;
    const __half* wn = c.ltab[0].norm_in;
    for (int pr = blockIdx.x * kWN + c.warp; pr < pairs; pr += gridDim.x * kWN) {
        const int u = pr * 2 + (lane >> 4);
        const bool valid = u < units;
        const int m = valid ? u / NP : 0, part = valid ? u - m * NP : 0;
        const int pack = part * 16 + (lane & 15);
        int tok = p.tokens[m];
        tok = min(max(tok, 0), p.V - 1);
        const uint32_t w = p.emb_wq[(size_t)tok * (p.H / 8) + pack];
        const int grp = pack >> 3;
        const __half s = p.emb_sc[(size_t)tok * (p.H / 64) + grp];
        const __half b = p.emb_bi[(size_t)tok * (p.H / 64) + grp];
        const uint4 wv = *reinterpret_cast<const uint4*>(wn + pack * 8);
        const __half* wh = reinterpret_cast<const __half*>(&wv);
        __align__(16) __half o[8], ow[8];
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < 8; j++) {
            o[j] = __hfma(__int2half_rn((int)((w >> (4 * j)) & 0xfu)), s, b);
            const float f = __half2float(o[j]);
            ss += f * f;
            ow[j] = __hmul(o[j], wh[j]);
        }
        if (valid) {
            *reinterpret_cast<uint4*>(p.h + (size_t)m * p.H + pack * 8) = *reinterpret_cast<const uint4*>(o);
            *reinterpret_cast<uint4*>(p.hw + xt_index(m, pack * 8, p.mp)) = *reinterpret_cast<const uint4*>(ow);
        } else {
            ss = 0.f;
        }
        ss += __shfl_xor_sync(0xffffffffu, ss, 1);          // two packs = one 16-column part
        if (valid && (lane & 1) == 0) p.ssq[(pack >> 1) * kSsqPitch + m] = ss;
    }
    // RoPE table: cs[m][i] = (cos, sin) of (scaling * inv_freq[i]) * pos[m]; one CTA per token, from the far end
    for (int m = (int)gridDim.x - 1 - (int)blockIdx.x; m < p.M; m += (int)gridDim.x) {
        for (int i = threadIdx.x; i < p.HD / 2; i += kNCons) {
            const float Lf = p.rope_scale * p.inv_freq[i];
            const float theta = Lf * (float)p.pos[m];
            float s, co;
            sincosf(theta, &s, &co);
            p.cs[m * kCsPitch + i] = make_float2(co, s);
        }
    }
}

// ================================================================================ attention
struct ADesc {
    __half* kc;
    __half* vc;
    int prefix, total, nact;
};

// 16-byte asynchronous copy global -> shared; bytes beyond src_bytes are written as zero.
__device__ __forceinline__ void cp_async16_zfill(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// Makes `bar` wait for every cp.async this thread has issued so far (pending count +1 now, -1 on completion).
__device__ __forceinline__ void cp_async_track(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
}

// One 64-key block of K and V, cache rows -> padded shared rows, by one warp: each lane owns one
// 16-byte column of the row and walks the rows (no divisions, two copies per step).
template <int HD>
__device__ __forceinline__ void kv_block_copy(uint32_t sk, uint32_t sv, const __half* kbase, const __half* vbase,
                                              int rows, int lane) {
    constexpr int KS = HD + 8;
    constexpr int VPR = HD / 8;                 // 16-byte vectors per row: 8 or 16
    constexpr int RPS = 32 / VPR;               // rows per step of the warp: 4 or 2
    const int cv = lane % VPR, r0 = lane / VPR;
    const __half* kp = kbase + cv * 8;
    const __half* vp = vbase + cv * 8;
    const uint32_t dk = sk + cv * 16, dv = sv + cv * 16;
#pragma unroll 4
    for (int r = r0; r < kKeyBlock; r += RPS) {
        const uint32_t nb = r < rows ? 16u : 0u;
        const int rs = r < rows ? r : 0;
        cp_async16_zfill(dk + r * (KS * 2), kp + (size_t)rs * HD, nb);
        cp_async16_zfill(dv + r * (KS * 2), vp + (size_t)rs * HD, nb);
    }
}

template <int MT, int HD>
__device__ __forceinline__ void attn_produce(const FwdParams& p, Ctx& c, const ADesc& a) {
    using G = Geo<MT>;
    constexpr int KS = HD + 8;
    static_assert(2 * kKeyBlock * KS * 2 <= kWArea, "K/V block must fit the weight area of a stage");
    const int lane = c.lane;
    const int nitems = p.Hkv * a.nact;
    if ((int)blockIdx.x < nitems && c.apos > 0 && !drain_blocks(p, c)) return;
    for (int item = blockIdx.x; item < nitems; item += gridDim.x, c.pos++) {
        const int hk = item / a.nact, kb = item - hk * a.nact;
        const int key0 = kb * kKeyBlock;
        const int rows = min(kKeyBlock, a.total - key0);
        const uint32_t slot = c.pos % G::NST, use = c.pos / G::NST;
        if (*c.abort_flag) return;
        if (use > 0 && !__all_sync(0xffffffffu, fwd_wait(smem_u32(c.empty + slot), (use - 1) & 1u))) {
            if (lane == 0) raise_error(p, c, 4);
            return;
        }
        const uint32_t fbar = smem_u32(c.full + slot);
        const uint32_t sk = smem_u32(c.ring + slot * G::STAGE);
        const __half* kbase = a.kc + ((size_t)hk * p.cap + key0) * HD;
        const __half* vbase = a.vc + ((size_t)hk * p.cap + key0) * HD;
        kv_block_copy<HD>(sk, sk + kKeyBlock * KS * 2, kbase, vbase, rows, lane);     // rows past the end become zero
        cp_async_track(fbar);
        __syncwarp();
        if (lane == 0) mbar_arrive(fbar);
    }
}

template <int MT, int HD>
__device__ __forceinline__ void attn_consume(const FwdParams& p, Ctx& c, const ADesc& a) {
    using G = Geo<MT>;
    constexpr int KS = HD + 8;
    constexpr int VPR = HD / 8;
    const int lane = c.lane, warp = c.warp;
    const int g = lane >> 2, t = lane & 3;
    const int nitems = p.Hkv * a.nact;
    const int Gq = p.Hq / p.Hkv;
    const int QR = p.M * Gq;
    const int ntiles = (QR + 15) / 16;
    const int prefix = a.prefix;

    for (int item = blockIdx.x; item < nitems; item += gridDim.x, c.pos++) {
        const int hk = item / a.nact, kb = item - hk * a.nact;
        const int key0 = kb * kKeyBlock;
        const uint32_t slot = c.pos % G::NST;
        bool ok = !*c.abort_flag;
        if (ok && !fwd_wait(smem_u32(c.full + slot), (c.pos / G::NST) & 1u)) {
            ok = false;
            if (lane == 0) raise_error(p, c, 5);
        }
        ok = __all_sync(0xffffffffu, ok);
        __half* sk = reinterpret_cast<__half*>(c.ring + slot * G::STAGE);
        __half* sv = sk + kKeyBlock * KS;
        if (ok) {
            // rows past the end -> zero; this pass's own rows -> from the qkv buffer (k rotated), and appended to the cache
            const int new0 = prefix + p.write_off;
            for (int idx = threadIdx.x; idx < kKeyBlock * VPR; idx += kNCons) {
                const int r = idx / VPR, cv = idx - r * VPR;
                const int key = key0 + r;
                if (key >= a.total) continue;                  // zero-filled by the producer
                const int m = key - new0;
                if (m < 0 || m >= p.M) continue;
                const __half* src = p.qkv + (size_t)m * p.NQKV;
                const uint4 vv = __ldcg(reinterpret_cast<const uint4*>(src + (size_t)(p.Hq + p.Hkv) * HD + (size_t)hk * HD + cv * 8));
                *reinterpret_cast<uint4*>(sv + r * KS + cv * 8) = vv;
                if (key < p.cap) *reinterpret_cast<uint4*>(a.vc + ((size_t)hk * p.cap + key) * HD + cv * 8) = vv;
                if (cv < VPR / 2) {
                    const __half* ksrc = src + (size_t)p.Hq * HD + (size_t)hk * HD;
                    const uint4 x1v = __ldcg(reinterpret_cast<const uint4*>(ksrc + cv * 8));
                    const uint4 x2v = __ldcg(reinterpret_cast<const uint4*>(ksrc + HD / 2 + cv * 8));
                    const __half* x1 = reinterpret_cast<const __half*>(&x1v);
                    const __half* x2 = reinterpret_cast<const __half*>(&x2v);
                    __align__(16) __half r1[8], r2[8];
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const float2 cs = __ldcg(p.cs + m * kCsPitch + cv * 8 + e);
                        const float a1 = __half2float(x1[e]), a2 = __half2float(x2[e]);
                        r1[e] = __float2half_rn(a1 * cs.x - a2 * cs.y);
                        r2[e] = __float2half_rn(a1 * cs.y + a2 * cs.x);
                    }
                    *reinterpret_cast<uint4*>(sk + r * KS + cv * 8) = *reinterpret_cast<const uint4*>(r1);
                    *reinterpret_cast<uint4*>(sk + r * KS + HD / 2 + cv * 8) = *reinterpret_cast<const uint4*>(r2);
                    if (key < p.cap) {
                        __half* kd = a.kc + ((size_t)hk * p.cap + key) * HD;
                        *reinterpret_cast<uint4*>(kd + cv * 8) = *reinterpret_cast<const uint4*>(r1);
                        *reinterpret_cast<uint4*>(kd + HD / 2 + cv * 8) = *reinterpret_cast<const uint4*>(r2);
                    }
                }
            }
            fence_proxy_async();       // the slot is refilled through the async proxy later
        }
        consumer_sync(kNCons);

        float* po = p.part_o + ((size_t)hk * p.nkb + kb) * p.qrp * HD;
        float* pml = p.part_ml + ((size_t)hk * p.nkb + kb) * p.qrp * 2;
        if (ok) {
            for (int rt = warp; rt < ntiles; rt += kWN) {
                const int r0 = rt * 16 + g, r1 = r0 + 8;
                const bool v0 = r0 < QR, v1 = r1 < QR;
                const int m0 = v0 ? r0 / Gq : 0, m1 = v1 ? r1 / Gq : 0;
                const __half* q0 = p.qkv + (size_t)m0 * p.NQKV + (size_t)(hk * Gq + (v0 ? r0 - m0 * Gq : 0)) * HD;
                const __half* q1 = p.qkv + (size_t)m1 * p.NQKV + (size_t)(hk * Gq + (v1 ? r1 - m1 * Gq : 0)) * HD;
                const unsigned long long mk0 = v0 ? p.mask[m0] : 0ull, mk1 = v1 ? p.mask[m1] : 0ull;

                uint32_t qa[HD / 16][4];
#pragma unroll
                for (int ks = 0; ks < HD / 16; ks++) {
                    qa[ks][0] = __ldcg(reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * t));
                    qa[ks][1] = __ldcg(reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * t));
                    qa[ks][2] = __ldcg(reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * t + 8));
                    qa[ks][3] = __ldcg(reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * t + 8));
                }
                // RoPE in registers: column i < HD/2 pairs with i + HD/2, i.e. fragment ks with ks + HD/32
#pragma unroll
                for (int ks = 0; ks < HD / 32; ks++) {
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        const int mm = (r & 1) ? m1 : m0;
                        const int i0 = ks * 16 + 2 * t + ((r >> 1) ? 8 : 0);
                        const float4 cs = __ldcg(reinterpret_cast<const float4*>(p.cs + mm * kCsPitch + i0));
                        const float2 lo = __half22float2(u32_as_h2(qa[ks][r]));
                        const float2 hi = __half22float2(u32_as_h2(qa[ks + HD / 32][r]));
                        const __half2 nlo = __halves2half2(__float2half_rn(lo.x * cs.x - hi.x * cs.y),
                                                           __float2half_rn(lo.y * cs.z - hi.y * cs.w));
                        const __half2 nhi = __halves2half2(__float2half_rn(lo.x * cs.y + hi.x * cs.x),
                                                           __float2half_rn(lo.y * cs.w + hi.y * cs.z));
                        qa[ks][r] = h2_as_u32(nlo);
                        qa[ks + HD / 32][r] = h2_as_u32(nhi);
                    }
                }

                float s[kKeyBlock / 8][4];
#pragma unroll
                for (int nt = 0; nt < kKeyBlock / 8; nt++) {
                    s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
                    const __half* krow = sk + (nt * 8 + g) * KS + 2 * t;
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ks++) {
                        const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + ks * 16);
                        const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + ks * 16 + 8);
                        mma_m16n8k16(s[nt], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
                    }
                }
                float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
                for (int nt = 0; nt < kKeyBlock / 8; nt++) {
#pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int key = key0 + nt * 8 + 2 * t + e;
                        const int j = key - prefix;
                        const bool in_prefix = key < prefix;
                        const bool in_tail = j >= 0 && j < p.tail;
                        const int js = in_tail ? j : 0;
                        const bool vis0 = v0 && (in_prefix || (in_tail && ((mk0 >> js) & 1ull)));
                        const bool vis1 = v1 && (in_prefix || (in_tail && ((mk1 >> js) & 1ull)));
                        s[nt][e] = vis0 ? s[nt][e] * p.scale_log2 : -INFINITY;
                        s[nt][2 + e] = vis1 ? s[nt][2 + e] * p.scale_log2 : -INFINITY;
                        mx0 = fmaxf(mx0, s[nt][e]);
                        mx1 = fmaxf(mx1, s[nt][2 + e]);
                    }
                }
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                const float base0 = (mx0 == -INFINITY) ? 0.f : mx0;
                const float base1 = (mx1 == -INFINITY) ? 0.f : mx1;
                float l0 = 0.f, l1 = 0.f;
                uint32_t pa[kKeyBlock / 8][2];
#pragma unroll
                for (int nt = 0; nt < kKeyBlock / 8; nt++) {
                    const float p00 = exp2f(s[nt][0] - base0), p01 = exp2f(s[nt][1] - base0);
                    const float p10 = exp2f(s[nt][2] - base1), p11 = exp2f(s[nt][3] - base1);
                    const __half2 h0 = __floats2half2_rn(p00, p01), h1 = __floats2half2_rn(p10, p11);
                    l0 += __low2float(h0) + __high2float(h0);
                    l1 += __low2float(h1) + __high2float(h1);
                    pa[nt][0] = h2_as_u32(h0);
                    pa[nt][1] = h2_as_u32(h1);
                }
                l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
                l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
                l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
                l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

                float o[HD / 8][4];
#pragma unroll
                for (int nd = 0; nd < HD / 8; nd++) o[nd][0] = o[nd][1] = o[nd][2] = o[nd][3] = 0.f;
#pragma unroll
                for (int kk = 0; kk < kKeyBlock / 16; kk++) {
#pragma unroll
                    for (int nd = 0; nd < HD / 8; nd += 2) {
                        uint32_t vb[4];
                        const __half* vp = sv + (kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * KS + (nd + (lane >> 4)) * 8;
                        ldmatrix_x4_trans(vb, vp);
                        mma_m16n8k16(o[nd], pa[2 * kk][0], pa[2 * kk][1], pa[2 * kk + 1][0], pa[2 * kk + 1][1], vb[0], vb[1]);
                        mma_m16n8k16(o[nd + 1], pa[2 * kk][0], pa[2 * kk][1], pa[2 * kk + 1][0], pa[2 * kk + 1][1], vb[2], vb[3]);
                    }
                }
                if (v0) {
                    if (t == 0) { pml[r0 * 2] = mx0; pml[r0 * 2 + 1] = l0; }
#pragma unroll
                    for (int nd = 0; nd < HD / 8; nd++)
                        *reinterpret_cast<float2*>(po + (size_t)r0 * HD + nd * 8 + 2 * t) = make_float2(o[nd][0], o[nd][1]);
                }
                if (v1) {
                    if (t == 0) { pml[r1 * 2] = mx1; pml[r1 * 2 + 1] = l1; }
#pragma unroll
                    for (int nd = 0; nd < HD / 8; nd++)
                        *reinterpret_cast<float2*>(po + (size_t)r1 * HD + nd * 8 + 2 * t) = make_float2(o[nd][2], o[nd][3]);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(c.empty + slot));
    }
}

// ---- block-parallel attention (the default) ---------------------------------------------------------
// One item is (kv head, 16-row query tile).  The ring memory is re-used as NS slots of one 64-key K/V
// block each (TMA tiles, 64 x 64 boxes, 128-byte swizzle: conflict-free fragment loads without
// padding); block n of the phase goes to slot n % NS and is scored by warp n % NS, so the key blocks
// of a tile are processed side by side, each warp keeping the running softmax state of its blocks
// in registers.  The warps then leave (max, sum, fp32 output) in their slots and all threads merge
// them in key-block order, normalise and store.  No partial sums in global memory, no merge phase.
// The slots overlay the matmul stages: the producer drains one geometry before it fills the other.
constexpr int kASlotsMax = 8;
constexpr int kBox = 64 * 128;                // bytes of one 64-row x 128-byte TMA box

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans_u(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
// 2-D tiled TMA load: box at (x = column in halves, y = row) of the tensor map -> shared memory.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];\n"
                 ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar) : "memory");
}
// Byte offset of 16-byte vector v (of HD/8) of row r inside a swizzled K or V block (boxes of 8 vectors side by side).
__device__ __forceinline__ uint32_t swz(int r, int v) {
    return (uint32_t)((v >> 3) * kBox + r * 128 + (((v & 7) ^ (r & 7)) << 4));
}

template <int MT, int HD>
struct AGeo {
    static constexpr int NBX = HD / 64;                      // boxes per K (and per V) block
    static constexpr int SLOT = 2 * NBX * kBox;              // 16 or 32 KB
    static constexpr int FIT = Geo<MT>::NST * Geo<MT>::STAGE / SLOT;
    static constexpr int NS = FIT < kASlotsMax ? FIT : kASlotsMax;
    static constexpr int OP = HD + 8;                        // pitch (floats) of a warp's partial output tile
    static_assert(16 * OP * 4 + 16 * 8 <= SLOT, "a warp's partial state must fit its slot");
};

// BATCH: the pass holds several requests (compiled separately, so that the one-request kernel is unchanged by it).
template <int MT, int HD, bool BATCH>
__device__ __forceinline__ void attn_bp_produce(const FwdParams& p, Ctx& c, const ADesc& a, int layer) {
    using A = AGeo<MT, HD>;
    const int lane = c.lane;
    const int Gq = p.Hq / p.Hkv;
    const int nreq = BATCH ? p.nreq : 1, mr = BATCH ? p.mr : p.M;
    const int ntiles = (mr * Gq + 15) / 16;
    const int nitems = nreq * p.Hkv * ntiles;             // item = (request, kv head, query tile)
    if ((int)blockIdx.x >= nitems) return;
    if (*c.abort_flag || !drain_stages<MT>(p, c)) return;
    for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
        const int req = BATCH ? item / (p.Hkv * ntiles) : 0;
        const int hk = BATCH ? (item / ntiles) % p.Hkv : item / ntiles;
        const int nact = BATCH ? min((req_prefix_tab()[req] + p.tail + kKeyBlock - 1) / kKeyBlock, p.nkb) : a.nact;
        const int krow0 = req * p.kv_req_rows + ((layer * 2 + 0) * p.Hkv + hk) * p.cap;   // row of the cache viewed as [rows][HD]
        const int vrow0 = req * p.kv_req_rows + ((layer * 2 + 1) * p.Hkv + hk) * p.cap;
        for (int kb = 0; kb < nact; kb++, c.apos++) {
            const uint32_t slot = c.apos % A::NS, use = c.apos / A::NS;
            if (*c.abort_flag) return;
            if (use > 0 && !__all_sync(0xffffffffu, fwd_wait(smem_u32(c.aempty + slot), (use - 1) & 1u))) {
                if (lane == 0) raise_error(p, c, 6);
                return;
            }
            const uint32_t fbar = smem_u32(c.afull + slot);
            const uint32_t sk = smem_u32(c.ring + slot * A::SLOT);
            if (lane == 0) {
                fence_proxy_async();
                mbar_expect_tx(fbar, A::SLOT);
            }
            __syncwarp();
            if (lane < 2 * A::NBX) {                  // K boxes, then V boxes
                const int isv = lane / A::NBX, bx = lane - isv * A::NBX;
                tma_load_2d(sk + lane * kBox, &p.kvmap, bx * 64, (isv ? vrow0 : krow0) + kb * kKeyBlock, fbar);
            }
        }
    }
}

template <int MT, int HD, bool BATCH>
__device__ __forceinline__ void attn_bp_consume(const FwdParams& p, Ctx& c, const ADesc& a) {
    using A = AGeo<MT, HD>;
    constexpr int NS = A::NS, NBX = A::NBX, OP = A::OP;
    constexpr int KS = HD + 8;                    // padded pitch of the query tile
    constexpr int VPR = HD / 8;
    static_assert(16 * KS * 2 <= kScratch, "the query tile must fit the scratch area");
    const int lane = c.lane, warp = c.warp;
    const int g = lane >> 2, t = lane & 3;
    const int Gq = p.Hq / p.Hkv;
    const int nreq = BATCH ? p.nreq : 1, mr = BATCH ? p.mr : p.M;
    const int QR = mr * Gq;                        // query rows (token, head of the group) of one request and kv head
    const int ntiles = (QR + 15) / 16;
    const int nitems = nreq * p.Hkv * ntiles;
    __half* sq = reinterpret_cast<__half*>(c.scratch);
    __half* nkv = sq + 16 * KS;                    // [2][M][HD]: rotated k rows, then v rows, of this pass
    static_assert(16 * KS * 2 + 2 * 32 * HD * 2 <= kScratch, "query tile and new K/V rows must fit the scratch area");
    unsigned char* myslot = c.ring + (warp < NS ? warp : 0) * A::SLOT;

    for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
        const int req = BATCH ? item / (p.Hkv * ntiles) : 0;
        const int hk = BATCH ? (item / ntiles) % p.Hkv : item / ntiles;
        const int rt = item - (req * p.Hkv + hk) * ntiles;
        const int prefix = BATCH ? req_prefix_tab()[req] : a.prefix;
        const int nact = BATCH ? min((prefix + p.tail + kKeyBlock - 1) / kKeyBlock, p.nkb) : a.nact;
        const int new0 = prefix + p.write_off;
        const int mbase = req * mr;                        // first token row of the request
        __half* const kc = a.kc + (size_t)req * p.kv_req_stride;
        __half* const vc = a.vc + (size_t)req * p.kv_req_stride;
        const uint32_t n0 = c.apos;                        // first block of this item in the phase's block sequence
        c.apos += nact;
        stamp(p, c, 2);
        // ---- rotated queries of the tile -> padded tile in shared memory, by all threads
        {
            constexpr int HV = VPR / 2;                       // vector pairs (i, i + HD/2) per row
            for (int pi = threadIdx.x; pi < 16 * HV; pi += kNCons) {
                const int row = pi / HV, cv = pi - row * HV;
                const int r = rt * 16 + row;
                uint4 o1 = make_uint4(0, 0, 0, 0), o2 = make_uint4(0, 0, 0, 0);
                if (r < QR) {
                    const int ml = r / Gq, hh = hk * Gq + (r - ml * Gq);
                    const int m = mbase + ml;
                    const __half* q = p.qkv + (size_t)m * p.NQKV + (size_t)hh * HD + cv * 8;
                    const uint4 x1v = __ldcg(reinterpret_cast<const uint4*>(q));
                    const uint4 x2v = __ldcg(reinterpret_cast<const uint4*>(q + HD / 2));
                    const float4* csp = reinterpret_cast<const float4*>(p.cs + m * kCsPitch + cv * 8);
                    float4 cs4[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) cs4[e] = __ldcg(csp + e);
                    const __half* x1 = reinterpret_cast<const __half*>(&x1v);
                    const __half* x2 = reinterpret_cast<const __half*>(&x2v);
                    __half* q1 = reinterpret_cast<__half*>(&o1);
                    __half* q2 = reinterpret_cast<__half*>(&o2);
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const float co = (e & 1) ? cs4[e >> 1].z : cs4[e >> 1].x;
                        const float si = (e & 1) ? cs4[e >> 1].w : cs4[e >> 1].y;
                        const float a1 = __half2float(x1[e]), a2 = __half2float(x2[e]);
                        q1[e] = __float2half_rn(a1 * co - a2 * si);
                        q2[e] = __float2half_rn(a1 * si + a2 * co);
                    }
                }
                *reinterpret_cast<uint4*>(sq + row * KS + cv * 8) = o1;
                *reinterpret_cast<uint4*>(sq + row * KS + HD / 2 + cv * 8) = o2;
            }
        }
        // ---- this pass's own K (rotated) and V rows of the head -> shared memory, by all threads; the first
        //      tile's item of each kv head also appends them to the cache
        {
            const bool writer = (rt == 0);
            for (int idx = threadIdx.x; idx < mr * VPR; idx += kNCons) {
                const int m = idx / VPR, cv = idx - m * VPR;          // m: row inside the request
                const int key = new0 + m;
                const __half* src = p.qkv + (size_t)(mbase + m) * p.NQKV;
                const uint4 vv = __ldcg(reinterpret_cast<const uint4*>(src + (size_t)(p.Hq + p.Hkv) * HD + (size_t)hk * HD + cv * 8));
                *reinterpret_cast<uint4*>(nkv + (mr + m) * HD + cv * 8) = vv;
                if (writer && key < p.cap) *reinterpret_cast<uint4*>(vc + ((size_t)hk * p.cap + key) * HD + cv * 8) = vv;
                if (cv < VPR / 2) {
                    const __half* ksrc = src + (size_t)p.Hq * HD + (size_t)hk * HD;
                    const uint4 x1v = __ldcg(reinterpret_cast<const uint4*>(ksrc + cv * 8));
                    const uint4 x2v = __ldcg(reinterpret_cast<const uint4*>(ksrc + HD / 2 + cv * 8));
                    const float4* csp = reinterpret_cast<const float4*>(p.cs + (mbase + m) * kCsPitch + cv * 8);
                    float4 cs4[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) cs4[e] = __ldcg(csp + e);
                    const __half* x1 = reinterpret_cast<const __half*>(&x1v);
                    const __half* x2 = reinterpret_cast<const __half*>(&x2v);
                    __align__(16) __half k1[8], k2[8];
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const float co = (e & 1) ? cs4[e >> 1].z : cs4[e >> 1].x;
                        const float si = (e & 1) ? cs4[e >> 1].w : cs4[e >> 1].y;
                        const float a1 = __half2float(x1[e]), a2 = __half2float(x2[e]);
                        k1[e] = __float2half_rn(a1 * co - a2 * si);
                        k2[e] = __float2half_rn(a1 * si + a2 * co);
                    }
                    *reinterpret_cast<uint4*>(nkv + m * HD + cv * 8) = *reinterpret_cast<const uint4*>(k1);
                    *reinterpret_cast<uint4*>(nkv + m * HD + HD / 2 + cv * 8) = *reinterpret_cast<const uint4*>(k2);
                    if (writer && key < p.cap) {
                        __half* kd = kc + ((size_t)hk * p.cap + key) * HD;
                        *reinterpret_cast<uint4*>(kd + cv * 8) = *reinterpret_cast<const uint4*>(k1);
                        *reinterpret_cast<uint4*>(kd + HD / 2 + cv * 8) = *reinterpret_cast<const uint4*>(k2);
                    }
                }
            }
        }
        consumer_sync(kNCons);
        stamp(p, c, 3);
        const uint32_t sq_frag = smem_u32(sq + ((lane & 7) + ((lane >> 3) & 1) * 8) * KS + (lane >> 4) * 8);

        const int r0 = rt * 16 + g, r1 = r0 + 8;
        const bool v0 = r0 < QR, v1 = r1 < QR;
        const int m0 = mbase + (v0 ? r0 / Gq : 0), m1 = mbase + (v1 ? r1 / Gq : 0);
        const unsigned long long mk0 = v0 ? p.mask[m0] : 0ull, mk1 = v1 ? p.mask[m1] : 0ull;

        float mrun0 = -INFINITY, mrun1 = -INFINITY, l0 = 0.f, l1 = 0.f;
        float o[HD / 8][4];
#pragma unroll
        for (int nd = 0; nd < HD / 8; nd++) o[nd][0] = o[nd][1] = o[nd][2] = o[nd][3] = 0.f;

        // ---- this warp's key blocks: those whose sequence number is congruent to the warp index
        bool ok = true;
        int nmine = 0;
        if (warp < NS) {
            const int kb_first = (int)((warp + NS - n0 % NS) % NS);
            for (int kb = kb_first; kb < nact; kb += NS, c.ause++, nmine++) {
                const int key0 = kb * kKeyBlock;
                if (nmine > 0) {                           // the previous block of this warp is done: give its slot back
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(c.aempty + warp));
                }
                ok = ok && !*c.abort_flag;
                if (ok && !fwd_wait(smem_u32(c.afull + warp), c.ause & 1u)) {
                    ok = false;
                    if (lane == 0) raise_error(p, c, 7);
                }
                ok = __all_sync(0xffffffffu, ok);
                if (kb == kb_first) stamp(p, c, 4);
                if (!ok) continue;
                const uint32_t sk = smem_u32(myslot), sv = sk + NBX * kBox;
                // this pass's own rows inside the block come from the rows prepared above
                if (key0 + kKeyBlock > new0 && key0 < new0 + mr) {
                    for (int idx = lane; idx < mr * VPR; idx += 32) {
                        const int m = idx / VPR, cv = idx - m * VPR;
                        const int r = new0 + m - key0;
                        if (r < 0 || r >= kKeyBlock) continue;
                        *reinterpret_cast<uint4*>(myslot + swz(r, cv)) = *reinterpret_cast<const uint4*>(nkv + m * HD + cv * 8);
                        *reinterpret_cast<uint4*>(myslot + NBX * kBox + swz(r, cv)) =
                            *reinterpret_cast<const uint4*>(nkv + (mr + m) * HD + cv * 8);
                    }
                    __syncwarp();
                }
                const bool all_visible = key0 + kKeyBlock <= prefix;      // committed rows: no mask needed
#pragma unroll
                for (int half = 0; half < 2; half++) {         // 32 keys at a time keeps the scores in 16 registers
                    float s[4][4];
#pragma unroll
                    for (int nt = 0; nt < 4; nt++) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
                    for (int ks = 0; ks < HD / 16; ks += 2) {
                        uint32_t qa0[4], qa1[4];
                        ldmatrix_x4(qa0, sq_frag + ks * 32);
                        ldmatrix_x4(qa1, sq_frag + ks * 32 + 32);
#pragma unroll
                        for (int nt = 0; nt < 4; nt++) {
                            uint32_t kf[4];
                            // matrices: (keys, hd ks*16..+8), (keys, +8), (keys, (ks+1)*16..+8), (keys, +8)
                            ldmatrix_x4(kf, sk + swz(half * 32 + nt * 8 + (lane & 7), ks * 2 + (lane >> 3)));
                            mma_m16n8k16(s[nt], qa0[0], qa0[1], qa0[2], qa0[3], kf[0], kf[1]);
                            mma_m16n8k16(s[nt], qa1[0], qa1[1], qa1[2], qa1[3], kf[2], kf[3]);
                        }
                    }
                    float mx0 = mrun0, mx1 = mrun1;
                    if (all_visible) {
#pragma unroll
                        for (int nt = 0; nt < 4; nt++) {
#pragma unroll
                            for (int e = 0; e < 2; e++) {
                                s[nt][e] = v0 ? s[nt][e] * p.scale_log2 : -INFINITY;
                                s[nt][2 + e] = v1 ? s[nt][2 + e] * p.scale_log2 : -INFINITY;
                                mx0 = fmaxf(mx0, s[nt][e]);
                                mx1 = fmaxf(mx1, s[nt][2 + e]);
                            }
                        }
                    } else {
#pragma unroll
                        for (int nt = 0; nt < 4; nt++) {
#pragma unroll
                            for (int e = 0; e < 2; e++) {
                                const int key = key0 + half * 32 + nt * 8 + 2 * t + e;
                                const int j = key - prefix;
                                const bool in_prefix = key < prefix;
                                const bool in_tail = j >= 0 && j < p.tail;
                                const int js = in_tail ? j : 0;
                                const bool vis0 = v0 && (in_prefix || (in_tail && ((mk0 >> js) & 1ull)));
                                const bool vis1 = v1 && (in_prefix || (in_tail && ((mk1 >> js) & 1ull)));
                                s[nt][e] = vis0 ? s[nt][e] * p.scale_log2 : -INFINITY;
                                s[nt][2 + e] = vis1 ? s[nt][2 + e] * p.scale_log2 : -INFINITY;
                                mx0 = fmaxf(mx0, s[nt][e]);
                                mx1 = fmaxf(mx1, s[nt][2 + e]);
                            }
                        }
                    }
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
                    const float base0 = (mx0 == -INFINITY) ? 0.f : mx0;
                    const float base1 = (mx1 == -INFINITY) ? 0.f : mx1;
                    if (mx0 != mrun0 || mx1 != mrun1) {        // the running maximum moved: rescale sums and outputs
                        const float al0 = (mrun0 == -INFINITY) ? 0.f : exp2f(mrun0 - base0);
                        const float al1 = (mrun1 == -INFINITY) ? 0.f : exp2f(mrun1 - base1);
                        mrun0 = mx0;
                        mrun1 = mx1;
                        l0 *= al0;
                        l1 *= al1;
#pragma unroll
                        for (int nd = 0; nd < HD / 8; nd++) {
                            o[nd][0] *= al0; o[nd][1] *= al0; o[nd][2] *= al1; o[nd][3] *= al1;
                        }
                    }
                    uint32_t pa[4][2];
#pragma unroll
                    for (int nt = 0; nt < 4; nt++) {
                        const float p00 = exp2f(s[nt][0] - base0), p01 = exp2f(s[nt][1] - base0);
                        const float p10 = exp2f(s[nt][2] - base1), p11 = exp2f(s[nt][3] - base1);
                        const __half2 hh0 = __floats2half2_rn(p00, p01), hh1 = __floats2half2_rn(p10, p11);
                        // the sum uses the rounded probabilities so that numerator and denominator agree
                        l0 += __low2float(hh0) + __high2float(hh0);
                        l1 += __low2float(hh1) + __high2float(hh1);
                        pa[nt][0] = h2_as_u32(hh0);
                        pa[nt][1] = h2_as_u32(hh1);
                    }
#pragma unroll
                    for (int kk = 0; kk < 2; kk++) {
#pragma unroll
                        for (int nd = 0; nd < HD / 8; nd += 2) {
                            uint32_t vb[4];
                            ldmatrix_x4_trans_u(vb, sv + swz(half * 32 + kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7), nd + (lane >> 4)));
                            mma_m16n8k16(o[nd], pa[2 * kk][0], pa[2 * kk][1], pa[2 * kk + 1][0], pa[2 * kk + 1][1], vb[0], vb[1]);
                            mma_m16n8k16(o[nd + 1], pa[2 * kk][0], pa[2 * kk][1], pa[2 * kk + 1][0], pa[2 * kk + 1][1], vb[2], vb[3]);
                        }
                    }
                }
            }
            // ---- leave the partial state in this warp's slot (its K/V block is no longer needed)
            if (nmine > 0) {
                l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
                l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
                l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
                l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
                __syncwarp();
                float* po = reinterpret_cast<float*>(myslot);
                float* pml = po + 16 * OP;
#pragma unroll
                for (int nd = 0; nd < HD / 8; nd++) {
                    *reinterpret_cast<float2*>(po + g * OP + nd * 8 + 2 * t) = make_float2(o[nd][0], o[nd][1]);
                    *reinterpret_cast<float2*>(po + (g + 8) * OP + nd * 8 + 2 * t) = make_float2(o[nd][2], o[nd][3]);
                }
                if (t == 0) {
                    *reinterpret_cast<float2*>(pml + g * 2) = make_float2(mrun0, l0);
                    *reinterpret_cast<float2*>(pml + (g + 8) * 2) = make_float2(mrun1, l1);
                }
            }
        }
        consumer_sync(kNCons);
        stamp(p, c, 5);

        // ---- merge in key-block order, normalise, store: thread = (row, HD/16 consecutive columns)
        {
            constexpr int CPT = HD / 16;
            const int row = threadIdx.x >> 4, c0 = (threadIdx.x & 15) * CPT;
            const int r = rt * 16 + row;
            const int nw = nact < NS ? nact : NS;
            if (r < QR) {
                float mstar = -INFINITY;
                for (int i = 0; i < nw; i++) {
                    const int w = (int)((n0 + i) % NS);
                    mstar = fmaxf(mstar, *reinterpret_cast<const float*>(c.ring + w * A::SLOT + (16 * OP + row * 2) * 4));
                }
                float acc[CPT];
#pragma unroll
                for (int e = 0; e < CPT; e++) acc[e] = 0.f;
                float denom = 0.f;
                for (int i = 0; i < nw; i++) {
                    const int w = (int)((n0 + i) % NS);
                    const float* base = reinterpret_cast<const float*>(c.ring + w * A::SLOT);
                    const float2 ml = *reinterpret_cast<const float2*>(base + 16 * OP + row * 2);
                    const float wgt = (ml.x == -INFINITY) ? 0.f : exp2f(ml.x - mstar);
                    denom += ml.y * wgt;
#pragma unroll
                    for (int e = 0; e < CPT; e += 4) {
                        const float4 v = *reinterpret_cast<const float4*>(base + row * OP + c0 + e);
                        acc[e] += wgt * v.x; acc[e + 1] += wgt * v.y; acc[e + 2] += wgt * v.z; acc[e + 3] += wgt * v.w;
                    }
                }
                const float inv = denom > 0.f ? 1.f / denom : 0.f;
                const int ml = r / Gq, hh = hk * Gq + (r - ml * Gq);
                const int m = mbase + ml;
                __align__(16) __half out[CPT];
#pragma unroll
                for (int e = 0; e < CPT; e++) out[e] = __float2half_rn(acc[e] * inv);
                __half* dst = p.attn + xt_index(m, hh * HD + c0, p.mp);       // a head's columns stay inside one 128-chunk
                if (CPT == 8) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(out);
                else *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(out);
            }
        }
        fence_proxy_async();           // the slots are refilled through the async proxy
        consumer_sync(kNCons);         // merge done: the last slots can go back, the query tile can be rewritten
        if (warp < NS && nmine > 0 && lane == 0) mbar_arrive(smem_u32(c.aempty + warp));
    }
}

// Merge of the key blocks: one warp per (token, query head), blocks added in block order.
template <int HD>
__device__ __forceinline__ void attn_merge(const FwdParams& p, Ctx& c, const ADesc& a) {
    const int lane = c.lane;
    const int Gq = p.Hq / p.Hkv;
    const int nrows = p.M * p.Hq;
    constexpr int CPT = HD / 32;
    for (int row = blockIdx.x * kWN + c.warp; row < nrows; row += gridDim.x * kWN) {
        const int m = row / p.Hq, head = row - m * p.Hq;
        const int hk = head / Gq, gq = head - hk * Gq;
        const int r = m * Gq + gq;
        const float* ho = p.part_o + (size_t)hk * p.nkb * p.qrp * HD;
        const float* hml = p.part_ml + (size_t)hk * p.nkb * p.qrp * 2;
        float mstar = -INFINITY;
        for (int b = lane; b < a.nact; b += 32) mstar = fmaxf(mstar, __ldcg(hml + ((size_t)b * p.qrp + r) * 2));
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mstar = fmaxf(mstar, __shfl_xor_sync(0xffffffffu, mstar, o));
        float denom = 0.f;
        float acc[CPT];
#pragma unroll
        for (int cc = 0; cc < CPT; cc++) acc[cc] = 0.f;
        for (int b0 = 0; b0 < a.nact; b0 += 32) {
            const int b = b0 + lane;
            float wl = 0.f, ll = 0.f;
            if (b < a.nact) {
                const float mb = __ldcg(hml + ((size_t)b * p.qrp + r) * 2);
                ll = __ldcg(hml + ((size_t)b * p.qrp + r) * 2 + 1);
                wl = (mb == -INFINITY) ? 0.f : exp2f(mb - mstar);
            }
            const int cnt = min(32, a.nact - b0);
            for (int i = 0; i < cnt; i++) {
                const float w = __shfl_sync(0xffffffffu, wl, i);
                denom += __shfl_sync(0xffffffffu, ll, i) * w;
                const float* src = ho + ((size_t)(b0 + i) * p.qrp + r) * HD + lane;
#pragma unroll
                for (int cc = 0; cc < CPT; cc++) acc[cc] += w * __ldcg(src + 32 * cc);
            }
        }
        const float inv = denom > 0.f ? 1.f / denom : 0.f;
#pragma unroll
        for (int cc = 0; cc < CPT; cc++) p.attn[xt_index(m, head * HD + lane + 32 * cc, p.mp)] = __float2half_rn(acc[cc] * inv);
    }
}

// ================================================================================ the kernel
template <int MT, int HD, bool TP, bool BATCH>
__global__ void __launch_bounds__(kFwdThreads, 1) forward_kernel(const __grid_constant__ FwdParams p) {
    using G = Geo<MT>;
    extern __shared__ __align__(1024) unsigned char smem[];      // swizzled TMA boxes want 1024-byte aligned stages
    __shared__ int s_abort, s_is_last;
    __shared__ uint32_t s_epoch;
    __shared__ float s_rstd[32];

    Ctx c;
    c.ring = smem;
    c.full = reinterpret_cast<uint64_t*>(smem + G::NST * G::STAGE);
    c.empty = c.full + G::NST;
    c.afull = c.empty + G::NST;
    c.aempty = c.afull + kASlotsMax;
    c.rbar = c.aempty + kASlotsMax;
    c.ruse = 0;
    c.apos = 0;
    c.ause = 0;
    c.ans = AGeo<MT, HD>::NS;
    c.scratch = smem + G::NST * G::STAGE + 256;
    {
        // every phase needs its layer's pointers the moment a barrier opens: keep the table on chip
        uint4* dst = reinterpret_cast<uint4*>(c.scratch + kScratch);
        const uint4* src = reinterpret_cast<const uint4*>(p.layers);
        for (int i = threadIdx.x; i < p.L * 4; i += kFwdThreads) dst[i] = src[i];
        c.ltab = reinterpret_cast<const LayerPtrs*>(dst);
    }
    c.abort_flag = &s_abort;
    c.s_epoch = &s_epoch;
    c.is_last = &s_is_last;
    c.s_rstd = s_rstd;

    c.pos = 0;
    c.epoch = 0;
    c.lbar = 0;
    c.tpx = 0;
    c.tp_seq0 = TP ? *reinterpret_cast<const volatile unsigned*>(p.tp_peers[p.tp_rank] + kTpFwdCount) : 0u;
    c.lane = threadIdx.x & 31;
    c.warp = threadIdx.x >> 5;

    if (BATCH && (int)threadIdx.x < p.nreq) req_prefix_tab()[threadIdx.x] = p.prefix[threadIdx.x];
    if (BATCH && threadIdx.x < 32) {
        // the head keeps rows [row_index[q], +rows_out) of request q (of mr rows) as output rows q * rows_out ..
        const int mr = BATCH ? p.mr : p.M;
        const int tok = threadIdx.x, q = BATCH ? tok / mr : 0;
        const int rel = tok - q * mr - ((p.row_index && tok < p.M) ? p.row_index[q] : 0);
        out_row_tab()[tok] = tok < p.M ? tok : -1;
        out_row_tab()[32 + tok] = (tok < p.M && rel >= 0 && rel < p.rows_out) ? q * p.rows_out + rel : -1;
    }
    if (threadIdx.x == 0) {
        s_abort = 0;
        s_epoch = 0;
#pragma unroll
        for (int s = 0; s < G::NST; s++) {
            mbar_init(smem_u32(c.full + s), 1);
            mbar_init(smem_u32(c.empty + s), kWN);
        }
#pragma unroll
        for (int s = 0; s < kASlotsMax; s++) {
            mbar_init(smem_u32(c.afull + s), 1);
            mbar_init(smem_u32(c.aempty + s), 1);
        }
        mbar_init(smem_u32(c.rbar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    const bool producer = c.warp == kWN;
    const int prefix = p.prefix[0];
    const int row_off = p.row_index ? p.row_index[0] : 0;
    ADesc ad;
    ad.prefix = prefix;
    ad.total = prefix + p.tail;
    ad.nact = min((ad.total + kKeyBlock - 1) / kKeyBlock, p.nkb);
    ad.kc = ad.vc = nullptr;
    const bool attn_fused = ad.nact <= p.attn_fused_max;

    // Phases in order: 0 = embedding, then per layer A, B1, B2, C, D, E, last = vocabulary projection.
    // One code path per kind (the four single-matrix products share one), a device-wide barrier after
    // every executed phase but the last.  phase_mask (one bit per kind) selects kinds for profiling.
    const int nph = 6 * p.L + 2;
    for (int ph = 0; ph < nph; ph++) {
        int kind = K_HEAD, l = 0;
        if (ph == 0) {
            kind = K_EMBED;
        } else if (ph < nph - 1) {
            l = (ph - 1) / 6;
            kind = K_A + (ph - 1) - 6 * l;
        }
        if (!((p.phase_mask >> kind) & 1u)) continue;
        const __half* tp_wn = nullptr;
        if (kind == K_EMBED) {
            if (!producer) embed_phase(p, c);
        } else if (kind == K_B1) {
            ad.kc = p.kv + (size_t)l * p.kv_layer_stride;
            ad.vc = ad.kc + p.kv_half_stride;
            if (attn_fused) {
                if (producer) attn_bp_produce<MT, HD, BATCH>(p, c, ad, l);
                else attn_bp_consume<MT, HD, BATCH>(p, c, ad);
            } else {
                if (producer) attn_produce<MT, HD>(p, c, ad);
                else attn_consume<MT, HD>(p, c, ad);
            }
        } else if (kind == K_B2) {
            if (attn_fused) continue;                      // no merge phase and no barrier in single-phase mode
            if (!producer) attn_merge<HD>(p, c, ad);
        } else {
            const LayerPtrs lp = c.ltab[l];
            QDesc d;
            d.xrows = p.M;
            d.row_lo = 0; d.row_cnt = p.M;
            d.orow_sel = 0;
            d.y_tiled = false;
            d.w1 = nullptr; d.bias = nullptr; d.wn = nullptr;
            int epi = TP ? EPI_TP : EPI_RESID;
            if (kind == K_A) {
                d.x = p.hw; d.w0 = lp.qkv_w; d.bias = lp.qkv_bias; d.y = p.qkv;
                d.N = p.NQKV; d.K = p.H; d.pl = p.plan[PLAN_A]; epi = EPI_QKV;
            } else if (kind == K_C) {
                d.x = p.attn; d.w0 = lp.o_w; d.wn = lp.norm_post; d.y = p.h;
                d.N = p.H; d.K = p.Hq * p.HD; d.pl = p.plan[PLAN_C];
            } else if (kind == K_D) {
                d.x = p.hw; d.w0 = lp.gate_w; d.w1 = lp.up_w; d.y = p.act; d.y_tiled = true;
                d.N = p.I; d.K = p.H; d.pl = p.plan[PLAN_D]; epi = EPI_SILU;
            } else if (kind == K_E) {
                d.x = p.act; d.w0 = lp.down_w;
                d.wn = (l + 1 < p.L) ? c.ltab[l + 1].norm_in : p.final_norm; d.y = p.h;
                d.N = p.H; d.K = p.I; d.pl = p.plan[PLAN_E];
            } else {                                   // K_HEAD, on the selected rows
                d.row_lo = row_off; d.row_cnt = p.rows_out;       // all rows are multiplied, the selected ones stored
                d.orow_sel = 1;
                d.x = p.hw; d.w0 = p.head_w; d.y = p.logits;
                d.N = p.head_rows; d.K = p.H; d.pl = p.plan[PLAN_HEAD]; epi = EPI_HEAD;
            }
            tp_wn = d.wn;
            if (producer) {
                qmm_produce<MT>(p, c, d, c.lbar, kind == K_D, epi != EPI_RESID && epi != EPI_TP);
            } else if (p.fast_scales) {          // uniform: chosen once per launch by the host
                if (kind == K_D) qmm_consume<MT, true, false, true, BATCH>(p, c, d, EPI_SILU);
                else qmm_consume<MT, false, TP, true, BATCH>(p, c, d, epi);
            } else {
                if (kind == K_D) qmm_consume<MT, true, false, false, BATCH>(p, c, d, EPI_SILU);
                else qmm_consume<MT, false, TP, false, BATCH>(p, c, d, epi);
            }
        }
        const bool exchange = TP && (kind == K_C || kind == K_E);
        if (kind != K_HEAD) {
            if (producer) { c.epoch++; if (!exchange) c.lbar++; }
            else if (exchange) tp_all_barrier(p, c, (c.tp_seq0 + c.tpx) * (p.tp_two_shot ? 2u : 1u));
            else grid_barrier(p, c);
        }
        if (exchange) {
            // the partial products of all GPUs -> h, h*w, sums of squares (every GPU computes all of it)
            if (producer) {
                c.epoch += p.tp_two_shot ? 2 : 1;
                c.lbar++;
            } else {
                tp_reduce_phase(p, c, tp_wn);
                grid_barrier(p, c);
            }
        }
    }

    if (threadIdx.x == 0 && p.timeline != nullptr && (int)c.epoch < p.timeline_pitch)
        p.timeline[((size_t)blockIdx.x * p.timeline_pitch + c.epoch) * 8] = global_ns();
    // ---- leave: the last CTA out resets the barrier words for the next launch (not after an error)
    __syncthreads();
    if (threadIdx.x == 0 && !s_abort) {
        __threadfence();
        const int old = atomicAdd(p.sync + kSyncExit, 1);
        if (old == (int)gridDim.x - 1) {
            for (int j = 0; j < kBarLanes; j++) p.sync[kSyncBar + j] = 0;
            p.sync[kSyncExit] = 0;
            if (TP)                        // every CTA read the old count before its first barrier
                *reinterpret_cast<volatile unsigned*>(p.tp_peers[p.tp_rank] + kTpFwdCount) = c.tp_seq0 + c.tpx;
        }
    }
}

// Chooses, for one matmul phase, how the eight consumer warps split an item (kw K-parts x 8/kw
// tiles) and whether K is also split across CTAs, with a small cost model in microseconds: a warp
// spends about half a microsecond per record while all warps of an SM stream, a shared-memory
// K reduction costs a few tenths, a split through global memory four to five (partial sums out,
// ticket, partial sums back in).
// Tuning hook (b200_forward_plan_hint, or the environment variable B200_FWD_PLAN read at the first launch):
// "A=kw:cps:splits,D=..." (phases A C D E, H = vocabulary projection) replaces the planner's choice for a
// phase wherever the values are feasible for the shape.  For measuring plans on the GPU, not an interface of the model.
struct PlanOverride { int kw, cps, splits; };
PlanOverride g_plan_override[5];
bool g_plan_override_init = false;
void parse_plan_hint(const char* e) {
    for (auto& o : g_plan_override) o = PlanOverride{0, 0, 0};
    g_plan_override_init = true;
    if (e == nullptr) return;
    const char* names = "ACDEH";
    while (*e) {
        const char* f = std::strchr(names, *e);
        int kw = 0, cps = 0, sp = 0;
        if (f && e[1] == '=' && std::sscanf(e + 2, "%d:%d:%d", &kw, &cps, &sp) == 3) g_plan_override[f - names] = PlanOverride{kw, cps, sp};
        const char* nx = std::strchr(e, ',');
        if (!nx) break;
        e = nx + 1;
    }
}
const PlanOverride* plan_override(int which) {
    if (!g_plan_override_init) parse_plan_hint(std::getenv("B200_FWD_PLAN"));
    return g_plan_override[which].kw > 0 ? &g_plan_override[which] : nullptr;
}

// Chooses, per phase, the K-parts inside a CTA (kw), the chunks of K per ring stage (cps) and the split of K
// across CTAs.  A stage holds cps x (the item's records [x2 in dual mode] + the activations of a chunk); narrow
// items (few tiles) therefore take many chunks per stage, and a K of a few thousand is wholly in flight when
// the barrier before the phase opens.  The cost model is in microseconds, fitted to phase timelines on B200:
// a record costs a warp ~0.19 us (two warps per scheduler), the first stage lands ~1.1 us after the barrier,
// every further generation of the three-stage ring adds ~0.5 us that the arithmetic does not hide, adding the
// K-parts through shared memory 0.4 us, a split through global memory (partial sums out, ticket, partial sums
// in) 1.4 to 4 us on the last CTA, growing with the partial slab (token rows x tiles) and the splits; an SM takes ~45 KB per
// us through its ring (weights from HBM and activations from L2 together), which is what keeps wide-K phases on
// split-K: without it every CTA re-reads all of x.
constexpr double kRingBytesPerUs = 45e3;
PhasePlan make_plan(int N, int K, int grid, int mt, bool dual, int which, bool hinted = true) {
    const int nchunks = K / kChunkK;
    const int tiles = (N + 15) / 16;
    const int nmat = dual ? 2 : 1;
    const int stage_bytes = kStageBytes;
    const double t_rec = 0.19 * (mt == 1 ? 0.85 : (mt == 2 ? 1.0 : (mt == 3 ? 1.3 : 1.6)));
    PhasePlan best{};
    double best_cost = 1e30;
    const PlanOverride* ov = hinted ? plan_override(which) : nullptr;
    for (int kw = 1; kw <= 8; kw *= 2) {
        if (kw > nchunks) continue;
        if (dual && mt >= 3 && kw > 1) continue;        // the K-part scratch holds 8 warps x 2 matrices x 2 token tiles
        if (ov && kw != ov->kw) continue;
        const int tpi = kWN / kw;
        const int row_items = (tiles + tpi - 1) / tpi;
        int fit = stage_bytes / (nmat * tpi * kRec + mt * 8 * kXRow);
        if (tpi < 4) fit = std::min(fit, 31 / nmat);     // parts of a block: one bulk copy per chunk and matrix, <= 31 lanes
        if (fit < kw) continue;                          // every K-part needs a chunk of the stage
        const int max_splits = row_items < kMaxCounters ? (nchunks + 3) / 4 : 1;
        for (int splits = 1; splits <= max_splits; splits++) {
            if (ov && splits != ov->splits) continue;
            const int per_split = (nchunks + splits - 1) / splits;
            const int eff = (nchunks + per_split - 1) / per_split;
            if (eff != splits) continue;
            const long long items = (long long)row_items * splits;
            const long long rounds = (items + grid - 1) / grid;
            int stages = (per_split + fit - 1) / fit;
            int cps = (per_split + stages - 1) / stages;                     // even stages
            if (ov && ov->cps >= kw && ov->cps <= fit) { cps = ov->cps; stages = (per_split + cps - 1) / cps; }
            const int rec_per_warp = ((per_split + kw - 1) / kw) * nmat;
            const double compute = rec_per_warp * t_rec;
            const double refill = ((stages + 2) / 3 - 1) * 1.0;
            const double stream = (double)per_split * (nmat * tpi * kRec + mt * 8 * kXRow) / kRingBytesPerUs;
            const double cost = rounds * (1.1 + std::max(compute, stream) + 0.5 * refill + 0.02 * stages + (kw > 1 ? 0.4 : 0.0) +
                                          (splits > 1 ? 1.0 + 0.08 * mt * tpi + 0.12 * splits : 0.0) + 0.8);
            if (cost < best_cost - 1e-9) {
                best_cost = cost;
                best.row_items = row_items; best.splits = splits; best.chunks_per_split = per_split; best.kw = kw; best.cps = cps;
            }
            if (items >= 4LL * grid) break;             // more splits cannot help any more
        }
    }
    if (ov && best_cost > 1e29) return make_plan(N, K, grid, mt, dual, which, false);    // the hint does not fit this shape
    return best;
}

size_t partial_bytes(const PhasePlan& pl, int mp, bool dual) {
    if (pl.splits <= 1) return 0;
    return (size_t)pl.splits * pl.row_items * mp * (dual ? 2 : 1) * (kWN / pl.kw) * 16 * sizeof(float);
}

struct WsLayout {
    size_t sync, counter, ssq, cs, part_ml, part_o, partial, total;
    int nkb, qrp;
};

// CTAs of a launch: one per SM of the current device, or the descriptor's smaller request.
int fwd_grid(const b200_forward_desc* d) {
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
        n = 148;
    if (d->grid_ctas > 0 && d->grid_ctas < n) n = d->grid_ctas;
    return n;
}


bool fwd_shape_ok(const b200_forward_desc* d) {
    if (!d) return false;
    if (d->M < 1 || d->M > 32 || d->rows_out < 1 || d->rows_out > d->M) return false;
    if (d->hidden < 128 || (d->hidden % 128) != 0 || d->hidden / 16 > kMaxSsqParts) return false;
    if (d->intermediate < 128 || (d->intermediate % 128) != 0) return false;
    if (d->head_dim != 64 && d->head_dim != 128) return false;
    if (d->n_heads < 1 || d->n_kv_heads < 1 || (d->n_heads % d->n_kv_heads) != 0) return false;
    if (((d->n_heads * d->head_dim) % 128) != 0) return false;
    if (d->vocab < 8 || (d->vocab % 8) != 0 || d->n_layers < 1 || d->n_layers > kMaxLayers) return false;
    if (d->tail < 1 || d->tail > 64 || d->write_off < 0) return false;
    if (d->requests <= 1 && d->write_off + d->M > d->tail) return false;      // (several requests: checked below, per request)
    if (d->cache_rows < d->tail) return false;
    if (d->head_rows < 0 || (d->head_rows % 8) != 0 || d->head_rows > d->vocab) return false;
    if (d->tp_world > 1) {
        if (d->tp_world > kMaxTp || d->tp_rank < 0 || d->tp_rank >= d->tp_world) return false;
    } else if (d->tp_world < 0) {
        return false;
    }
    if (d->grid_ctas < 0) return false;
    if (d->requests > 1) {
        // several requests per pass: equal row groups, single-phase attention only (the cache must be short enough
        // for it whatever the committed lengths are), no tensor-parallel shard
        if (d->requests > kMaxReq || (d->M % d->requests) != 0 || d->tp_world > 1) return false;
        if (d->write_off + d->M / d->requests > d->tail) return false;
        const int fused_max = d->attn_split_blocks > 0 ? d->attn_split_blocks - 1 : (d->attn_split_blocks < 0 ? 0 : 32);
        if ((d->cache_rows + kKeyBlock - 1) / kKeyBlock > fused_max) return false;
        if (d->rows_out > d->M / d->requests) return false;
    } else if (d->requests < 0) {
        return false;
    }
    return true;
}

WsLayout fwd_layout(const b200_forward_desc* d, PhasePlan (&plan)[5], int* grid_out = nullptr) {
    const int grid = fwd_grid(d);
    if (grid_out) *grid_out = grid;
    const int mp = ((d->M + 7) / 8) * 8;
    const int nqkv = (d->n_heads + 2 * d->n_kv_heads) * d->head_dim;
    const int mt = mp / 8;
    plan[PLAN_A] = make_plan(nqkv, d->hidden, grid, mt, false, PLAN_A);
    plan[PLAN_C] = make_plan(d->hidden, d->n_heads * d->head_dim, grid, mt, false, PLAN_C);
    plan[PLAN_D] = make_plan(d->intermediate, d->hidden, grid, mt, true, PLAN_D);
    plan[PLAN_E] = make_plan(d->hidden, d->intermediate, grid, mt, false, PLAN_E);
    const int head_rows = d->head_rows > 0 ? d->head_rows : d->vocab;
    plan[PLAN_HEAD] = make_plan(head_rows, d->hidden, grid, mt, false, PLAN_HEAD);
    // split-K scratch: sized for any row count up to 32, so one workspace serves every pass shape
    size_t pb = 0;
    for (int m = 1; m <= 4; m++) {
        PhasePlan q[5] = {make_plan(nqkv, d->hidden, grid, m, false, PLAN_A),
                          make_plan(d->hidden, d->n_heads * d->head_dim, grid, m, false, PLAN_C),
                          make_plan(d->intermediate, d->hidden, grid, m, true, PLAN_D),
                          make_plan(d->hidden, d->intermediate, grid, m, false, PLAN_E),
                          make_plan(head_rows, d->hidden, grid, m, false, PLAN_HEAD)};
        for (int i = 0; i < 5; i++) pb = std::max(pb, partial_bytes(q[i], m * 8, i == PLAN_D));
    }
    WsLayout w{};
    const int G = d->n_heads / d->n_kv_heads;
    w.qrp = ((32 * G + 15) / 16) * 16;
    w.nkb = (d->cache_rows + kKeyBlock - 1) / kKeyBlock;
    size_t off = 0;
    w.sync = off; off += 256;
    w.counter = off; off += kCounterBytes;
    w.ssq = off; off += (size_t)kMaxSsqParts * kSsqPitch * sizeof(float);
    w.cs = off; off += (size_t)32 * kCsPitch * sizeof(float2);
    w.part_ml = off; off += (size_t)d->n_kv_heads * w.nkb * w.qrp * 2 * sizeof(float);
    off = (off + 255) & ~(size_t)255;
    w.part_o = off; off += (size_t)d->n_kv_heads * w.nkb * w.qrp * d->head_dim * sizeof(float);
    off = (off + 255) & ~(size_t)255;
    w.partial = off; off += pb;
    w.total = off;
    return w;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup (no link against libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode_tiled = nullptr;

int make_kv_map(CUtensorMap* map, void* cache, int layers, int hkv, int cap, int hd) {
    if (g_encode_tiled == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess || fn == nullptr)
            return check_launch() == B200_OK ? B200_ECUDA : B200_ECUDA;
        g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
    }
    const cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)layers * 2 * hkv * cap};
    const cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
    const cuuint32_t box[2] = {64, 64};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = g_encode_tiled(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, cache, dims, strides, box, estr,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda_error = (int)r;
        return B200_ECUDA;
    }
    return B200_OK;
}

template <int MT, int HD, bool TP, bool BATCH>
int launch_forward(const FwdParams& p, int grid, cudaStream_t stream) {
    auto kern = forward_kernel<MT, HD, TP, BATCH>;
    bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Geo<MT>::SMEM) != cudaSuccess)
            return check_launch();
        attr_set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(kFwdThreads);
    cfg.dynamicSmemBytes = Geo<MT>::SMEM;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaLaunchKernelEx(&cfg, kern, p);
    return check_launch();
}

template <int MT>
int launch_forward_hd(const FwdParams& p, int grid, cudaStream_t stream) {
    if (p.tp_world > 1)         // a shard: the variant with the exchange phases
        return p.HD == 128 ? launch_forward<MT, 128, true, false>(p, grid, stream) : launch_forward<MT, 64, true, false>(p, grid, stream);
    if (p.nreq > 1)             // several requests in the pass
        return p.HD == 128 ? launch_forward<MT, 128, false, true>(p, grid, stream) : launch_forward<MT, 64, false, true>(p, grid, stream);
    return p.HD == 128 ? launch_forward<MT, 128, false, false>(p, grid, stream) : launch_forward<MT, 64, false, false>(p, grid, stream);
}

}  // namespace
}  // namespace b200

extern "C" {

using namespace b200;

size_t b200_forward_tp_buffer_bytes(int hidden) {
    if (hidden < 128 || (hidden % 128) != 0) return 0;
    return (size_t)kTpHeader + (size_t)2 * 32 * hidden * sizeof(float) + (size_t)2 * 32 * hidden * sizeof(__half) +
           (size_t)2 * kMaxTp * 32 * hidden * sizeof(float);       // partial products, gather area, push slots
}

void b200_forward_plan_hint(const char* spec) { parse_plan_hint(spec); }

size_t b200_forward_workspace_bytes(const b200_forward_desc* d) {
    if (!fwd_shape_ok(d)) return 0;
    PhasePlan plan[5];
    return fwd_layout(d, plan).total;
}

int b200_forward(const b200_forward_desc* d, void* stream) {
    if (!fwd_shape_ok(d)) return B200_EINVAL;
    const void* need[] = {d->tokens, d->pos, d->mask, d->prefix, d->inv_freq, d->embed_wq, d->embed_scales,
                          d->embed_biases, d->final_norm, d->lm_head_tiled, d->layer_table, d->h, d->hw, d->qkv,
                          d->attn, d->act, d->logits, d->kv_cache, d->workspace};
    for (const void* q : need)
        if (!q) return B200_EINVAL;
    const void* al[] = {d->lm_head_tiled, d->h, d->hw, d->qkv, d->attn, d->act, d->logits, d->kv_cache, d->workspace,
                        d->final_norm};
    for (const void* q : al)
        if (!aligned16(q)) return B200_EALIGN;
    FwdParams p{};
    int grid = 0;
    const WsLayout w = fwd_layout(d, p.plan, &grid);
    if (d->workspace_bytes < w.total) return B200_EWORKSPACE;
    p.M = d->M; p.mp = ((d->M + 7) / 8) * 8; p.rows_out = d->rows_out; p.H = d->hidden; p.I = d->intermediate; p.Hq = d->n_heads;
    p.Hkv = d->n_kv_heads; p.HD = d->head_dim; p.V = d->vocab; p.L = d->n_layers;
    p.NQKV = (d->n_heads + 2 * d->n_kv_heads) * d->head_dim;
    p.eps = d->rms_eps; p.rope_scale = d->rope_scaling; p.scale_log2 = d->attn_scale * kLog2e;
    p.tokens = d->tokens; p.pos = d->pos; p.mask = d->mask; p.prefix = d->prefix; p.row_index = d->row_index;
    p.inv_freq = d->inv_freq;
    p.emb_wq = d->embed_wq;
    p.emb_sc = static_cast<const __half*>(d->embed_scales);
    p.emb_bi = static_cast<const __half*>(d->embed_biases);
    p.final_norm = static_cast<const __half*>(d->final_norm);
    p.head_w = static_cast<const unsigned char*>(d->lm_head_tiled);
    p.layers = static_cast<const LayerPtrs*>(d->layer_table);
    p.h = static_cast<__half*>(d->h); p.hw = static_cast<__half*>(d->hw); p.qkv = static_cast<__half*>(d->qkv);
    p.attn = static_cast<__half*>(d->attn); p.act = static_cast<__half*>(d->act);
    p.logits = static_cast<__half*>(d->logits);
    p.kv = static_cast<__half*>(d->kv_cache);
    p.kv_half_stride = (size_t)d->n_kv_heads * d->cache_rows * d->head_dim;
    p.kv_layer_stride = 2 * p.kv_half_stride;
    p.cap = d->cache_rows; p.write_off = d->write_off; p.tail = d->tail;
    p.nreq = d->requests > 1 ? d->requests : 1;
    p.mr = d->M / p.nreq;
    p.kv_req_stride = (size_t)d->n_layers * p.kv_layer_stride;
    p.kv_req_rows = d->n_layers * 2 * d->n_kv_heads * d->cache_rows;
    char* ws = static_cast<char*>(d->workspace);
    p.sync = reinterpret_cast<int*>(ws + w.sync);
    p.counter = reinterpret_cast<int*>(ws + w.counter);
    p.ssq = reinterpret_cast<float*>(ws + w.ssq);
    p.cs = reinterpret_cast<float2*>(ws + w.cs);
    p.part_ml = reinterpret_cast<float*>(ws + w.part_ml);
    p.part_o = reinterpret_cast<float*>(ws + w.part_o);
    p.partial = reinterpret_cast<float*>(ws + w.partial);
    p.nkb = w.nkb; p.qrp = w.qrp;
    {
        const int rc = make_kv_map(&p.kvmap, d->kv_cache, d->n_layers * p.nreq, d->n_kv_heads, d->cache_rows, d->head_dim);
        if (rc != B200_OK) return rc;
    }
    p.head_rows = d->head_rows > 0 ? d->head_rows : d->vocab;
    p.tp_world = d->tp_world > 1 ? d->tp_world : 1;
    p.tp_rank = d->tp_world > 1 ? d->tp_rank : 0;
    p.tp_two_shot = (p.tp_world > 1 && (p.H % (16 * p.tp_world)) == 0 &&
                     d->tp_two_shot == 1) ? 1 : 0;
    p.tp_hier = (p.tp_world > 1 && (p.tp_two_shot || d->tp_two_shot == 2)) ? 1 : 0;
    p.tp_push = (p.tp_world > 1 && (d->tp_two_shot == 3 || (d->tp_two_shot == 0 && p.tp_world >= kTpPushMinWorld))) ? 1 : 0;
    if (p.tp_world > 1) {
        for (int r = 0; r < p.tp_world; r++) {
            if (!d->tp_peers[r]) return B200_EINVAL;
            if (!aligned16(d->tp_peers[r])) return B200_EALIGN;
            p.tp_peers[r] = static_cast<unsigned char*>(d->tp_peers[r]);
        }
    }
    p.phase_mask = d->phase_mask ? (unsigned)d->phase_mask : 0xffu;
    p.grid_wait_limit = g_wait_limit ? (g_wait_limit < (1u << 27) ? g_wait_limit : (1u << 27)) : kGridWaitLimit;
    p.tp_wait_limit = g_wait_limit ? g_wait_limit : kTpWaitLimit;
    p.fast_scales = d->scales_in_fast_range ? 1 : 0;
    p.attn_fused_max = d->attn_split_blocks > 0 ? d->attn_split_blocks - 1 : (d->attn_split_blocks < 0 ? 0 : 32);
    p.timeline = static_cast<long long*>(d->timeline);
    p.timeline_pitch = d->timeline ? d->timeline_pitch : 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch ((d->M + 7) / 8) {
        case 1: return launch_forward_hd<1>(p, grid, st);
        case 2: return launch_forward_hd<2>(p, grid, st);
        case 3: return launch_forward_hd<3>(p, grid, st);
        default: return launch_forward_hd<4>(p, grid, st);
    }
}

}  // extern "C"
