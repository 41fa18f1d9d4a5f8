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
#include "pipeline.cuh"
#include "qmm_common.cuh"

namespace b200 {
namespace {

constexpr int kWN = 8;                        // consumer warps per CTA
constexpr int kNCons = kWN * 32;
constexpr int kFwdThreads = kNCons + 32;      // + one producer warp
constexpr int kRec = 1152;                    // bytes per 16-row x 128-k weight record
constexpr int kWArea = 8 * 4 * kRec;          // weight bytes of a ring stage: 8 (block, chunk) cells of 4 records
constexpr int kXPitch = 4 * kChunkK * 2 + 64; // activation row pitch in a stage (up to 4 chunks)
constexpr int kKeyBlock = 64;
constexpr float kLog2e = 1.4426950408889634f;
constexpr uint32_t kGridWaitLimit = 1u << 22;
constexpr int kSsqPitch = 32;                 // ssq[part][token]
constexpr int kMaxSsqParts = 64;
constexpr int kCsPitch = 64;                  // cos/sin table: cs[token][i], i < head_dim/2 <= 64

// sync words (ints) at the head of the workspace
constexpr int kSyncBar = 0, kSyncExit = 1, kSyncErr = 2;

enum { EPI_QKV = 0, EPI_SILU = 1, EPI_RESID = 2, EPI_HEAD = 3 };
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
    int row_tiles, splits, chunks_per_split;
};

struct FwdParams {
    int M, rows_out, H, I, Hq, Hkv, HD, V, L, NQKV;
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
    int* sync;
    int* counter;
    float* ssq;
    float2* cs;
    float* part_ml;
    float* part_o;
    float* partial;
    int nkb, qrp;
    PhasePlan plan[5];
    long long* timeline;           // optional [CTAs][timeline_pitch][2] globaltimer stamps (arrive, leave) per barrier
    int timeline_pitch;
};

template <int MT>
struct Geo {
    static constexpr int MP = MT * 8;
    static constexpr int STAGE = kWArea + MP * kXPitch;
    static constexpr int NST = MT <= 2 ? 4 : 3;
    static constexpr int SMEM = NST * STAGE + 128;
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
    int xrows;
    int rstd_off;               // token row of x row 0 (selects the ssq column)
    int ssq_parts;
};

struct Ctx {
    unsigned char* ring;
    uint64_t* full;
    uint64_t* empty;
    uint64_t* rstd_bar;
    volatile int* abort_flag;
    int* is_last;
    float* s_rstd;
    uint32_t pos;       // ring stages produced (producer warp) / consumed (consumer warps)
    uint32_t epoch;     // grid barriers before the current phase
    uint32_t rstd_n;    // rstd hand-overs consumed
    int lane, warp;
};

// Ring waits of this kernel: up to 2^20 polls of <= 1 us each (about a second) before giving up.
__device__ __forceinline__ bool fwd_wait(uint32_t bar, uint32_t parity) {
    return mbar_wait_timed(bar, parity, 1u << 20, 1000u);
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

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
    uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void raise_error(const FwdParams& p, Ctx& c, int code) {
    *c.abort_flag = 1;
    atomicCAS(p.sync + kSyncErr, 0, code);
}

// Device-wide barrier, consumer side: every consumer thread calls it; thread 0 arrives for the CTA
// and polls.  The counter only grows during a launch (target = epoch * CTAs); the last CTA to
// leave the kernel resets it.
__device__ void grid_barrier(const FwdParams& p, Ctx& c) {
    c.epoch++;
    consumer_sync(kNCons);
    if (threadIdx.x == 0 && !*c.abort_flag) {
        long long* tl = nullptr;
        if (p.timeline != nullptr && (int)c.epoch <= p.timeline_pitch) {
            tl = p.timeline + ((size_t)blockIdx.x * p.timeline_pitch + (c.epoch - 1)) * 2;
            tl[0] = global_ns();
        }
        __threadfence();               // cumulative: covers the CTA's writes ordered before the bar.sync
        fence_proxy_async_all();
        atomicAdd(p.sync + kSyncBar, 1);
        const int target = (int)(c.epoch * gridDim.x);
        bool ok = false;
        for (uint32_t i = 0; i < kGridWaitLimit; i++) {
            if (ld_acquire(p.sync + kSyncBar) >= target) { ok = true; break; }
        }
        if (!ok) raise_error(p, c, 10);
        __threadfence();
        if (tl != nullptr) tl[1] = global_ns();
    }
    consumer_sync(kNCons);
}

// Producer side: the whole warp calls it before the first activation copy of a phase; it only
// observes the counter.  Returns false on timeout / abort.
__device__ bool producer_grid_wait(const FwdParams& p, Ctx& c, uint32_t need_epoch) {
    int ok = 1;
    if (need_epoch > 0 && c.lane == 0) {
        ok = 0;
        const int target = (int)(need_epoch * gridDim.x);
        for (uint32_t i = 0; i < kGridWaitLimit && !*c.abort_flag; i++) {
            if (ld_acquire(p.sync + kSyncBar) >= target) { ok = 1; break; }
        }
        if (!ok && !*c.abort_flag) raise_error(p, c, 11);
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    fence_proxy_async_all();       // activations were written through the generic proxy by other CTAs
    return ok != 0;
}

// ================================================================================ QMM, producer
// Streams the weight records (and activation rows) of this CTA's items of one matmul phase into the
// ring.  `need_epoch`: grid barriers that must have completed before the activations may be read.
template <int MT, bool DUAL>
__device__ void qmm_produce(const FwdParams& p, Ctx& c, const QDesc& d, uint32_t need_epoch, bool need_rstd) {
    using G = Geo<MT>;
    constexpr int NB = DUAL ? 4 : 2;            // 64-row block cells per stage
    constexpr int CPS = 8 / NB;                 // chunks per stage
    constexpr int CELL = CPS * 4 * kRec;        // bytes of one block cell
    constexpr int R = 128;
    const int lane = c.lane;
    const int nchunks_total = d.K / kChunkK;
    const int nblocks = (d.N + 63) / 64;
    const int nitems = d.pl.row_tiles * d.pl.splits;
    if ((int)blockIdx.x >= nitems) return;
    (void)R;

    bool ready = false;
    int npend = 0;
    uint32_t pend_slot[G::NST];
    int pend_k0[G::NST], pend_recs[G::NST];

    auto issue_x = [&](uint32_t slot, int k0, int recs) {
        if (lane < d.xrows)
            bulk_copy_g2s(smem_u32(c.ring + slot * G::STAGE + kWArea + lane * kXPitch),
                          d.x + (size_t)lane * d.K + k0, (uint32_t)(recs * kChunkK * 2), smem_u32(c.full + slot));
    };
    auto flush = [&]() -> bool {
        if (!producer_grid_wait(p, c, need_epoch)) return false;
#pragma unroll
        for (int i = 0; i < G::NST; i++)
            if (i < npend) issue_x(pend_slot[i], pend_k0[i], pend_recs[i]);
        npend = 0;
        ready = true;
        if (need_rstd) {
            float ss = 0.f;
            if (lane < d.xrows) {
#pragma unroll 8
                for (int part = 0; part < d.ssq_parts; part++)
                    ss += __ldcg(p.ssq + part * kSsqPitch + d.rstd_off + lane);
            }
            c.s_rstd[lane] = (lane < d.xrows) ? rsqrtf(ss / (float)p.H + p.eps) : 0.f;
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(c.rstd_bar));
        }
        return true;
    };

    for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
        const int row_tile = item % d.pl.row_tiles;
        const int split = item / d.pl.row_tiles;
        const int c_begin = split * d.pl.chunks_per_split;
        const int n = min(d.pl.chunks_per_split, nchunks_total - c_begin);
        const int nst = (n + CPS - 1) / CPS;
        const bool last_item = item + (int)gridDim.x >= nitems;
        const unsigned char* src[NB];
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const int blk = min(row_tile * 2 + (b & 1), nblocks - 1);
            const unsigned char* base = (DUAL && b >= 2) ? d.w1 : d.w0;
            src[b] = base + ((size_t)blk * nchunks_total + c_begin) * 4 * kRec;
        }
        for (int st = 0; st < nst; st++, c.pos++) {
            const uint32_t slot = c.pos % G::NST, use = c.pos / G::NST;
            if (*c.abort_flag) return;
            if (use > 0 && !__all_sync(0xffffffffu, fwd_wait(smem_u32(c.empty + slot), (use - 1) & 1u))) {
                if (lane == 0) raise_error(p, c, 2);
                return;
            }
            const int recs = min(CPS, n - st * CPS);
            if (lane == 0) {
                const uint32_t fbar = smem_u32(c.full + slot);
                const uint32_t bytes = (uint32_t)(recs * 4 * kRec);
                fence_proxy_async();
                mbar_expect_tx(fbar, NB * bytes + (uint32_t)d.xrows * (uint32_t)(recs * kChunkK * 2));
#pragma unroll
                for (int b = 0; b < NB; b++)
                    bulk_copy_g2s(smem_u32(c.ring + slot * G::STAGE + b * CELL), src[b] + (size_t)st * CELL, bytes, fbar);
            }
            __syncwarp();
            const int k0 = (c_begin + st * CPS) * kChunkK;
            if (ready) {
                issue_x(slot, k0, recs);
            } else {
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

// ================================================================================ QMM, consumers
template <int MT, bool DUAL, int EPI>
__device__ void qmm_consume(const FwdParams& p, Ctx& c, const QDesc& d) {
    using G = Geo<MT>;
    constexpr int NB = DUAL ? 4 : 2;
    constexpr int CPS = 8 / NB;
    constexpr int CELL = CPS * 4 * kRec;
    constexpr int S = DUAL ? 2 : 1;
    constexpr int R = 128;                       // output rows (of each matrix) per item
    constexpr int MP = MT * 8;
    constexpr int TW = DUAL ? 2 * R : R;
    constexpr bool NEED_RSTD = (EPI != EPI_RESID);
    const int lane = c.lane, warp = c.warp;
    const int g = lane >> 2, t = lane & 3;
    const int nchunks_total = d.K / kChunkK;
    const int nitems = d.pl.row_tiles * d.pl.splits;
    bool rstd_ready = false;

    int rec_off[S];
#pragma unroll
    for (int s = 0; s < S; s++) rec_off[s] = ((DUAL ? 2 * s : 0) + warp / 4) * CELL + (warp % 4) * kRec;

    for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
        const int row_tile = item % d.pl.row_tiles;
        const int split = item / d.pl.row_tiles;
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
            if (ok) {
                const unsigned char* stage = c.ring + slot * G::STAGE;
#pragma unroll
                for (int cc = 0; cc < CPS; cc++) {
                    if (st * CPS + cc < n) {
                        const unsigned char* xrow = stage + kWArea + g * kXPitch + cc * (kChunkK * 2) + t * 16;
                        uint4 w[S][2];
                        uint2 sb[S][2];
#pragma unroll
                        for (int s = 0; s < S; s++) {
                            const unsigned char* rec = stage + rec_off[s] + cc * 4 * kRec;
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
                                xb[mt] = *reinterpret_cast<const uint4*>(xrow + mt * 8 * kXPitch + j * 64);
#pragma unroll
                            for (int s = 0; s < S; s++) {
                                const __half2 p0 = u32_as_h2((j < 2) ? sb[s][0].x : sb[s][0].y);   // {scale, bias}
                                const __half2 p1 = u32_as_h2((j < 2) ? sb[s][1].x : sb[s][1].y);
                                uint32_t d0[4], d1[4];
                                dequant_pack(comp(w[s][0], j), __low2half2(p0), __high2half2(p0), d0);
                                dequant_pack(comp(w[s][1], j), __low2half2(p1), __high2half2(p1), d1);
#pragma unroll
                                for (int mt = 0; mt < MT; mt++) {
                                    mma_m16n8k16(acc[s][mt], d0[0], d1[0], d0[1], d1[1], xb[mt].x, xb[mt].y);
                                    mma_m16n8k16(acc[s][mt], d0[2], d1[2], d0[3], d1[3], xb[mt].z, xb[mt].w);
                                }
                            }
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(c.empty + slot));
        }

        if (NEED_RSTD && !rstd_ready) {
            if (!*c.abort_flag && !fwd_wait(smem_u32(c.rstd_bar), c.rstd_n & 1u)) {
                if (lane == 0) raise_error(p, c, 3);
            }
            c.rstd_n++;
            rstd_ready = true;
        }

        // lane (g,t) holds, per sub-tile and token tile: rows g / g+8 x tokens 2t / 2t+1
        const bool via_partials = (EPI == EPI_RESID) || d.pl.splits > 1;
        if (via_partials) {
            float* mine = p.partial + ((size_t)split * d.pl.row_tiles + row_tile) * MP * TW;
#pragma unroll
            for (int s = 0; s < S; s++) {
                const int ri = s * R + warp * 16;
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    const int tok = mt * 8 + 2 * t;
                    mine[(size_t)tok * TW + ri + g] = acc[s][mt][0];
                    mine[(size_t)(tok + 1) * TW + ri + g] = acc[s][mt][1];
                    mine[(size_t)tok * TW + ri + g + 8] = acc[s][mt][2];
                    mine[(size_t)(tok + 1) * TW + ri + g + 8] = acc[s][mt][3];
                }
            }
            __threadfence();
            consumer_sync(kNCons);
            if (threadIdx.x == 0) {
                const int old = atomicAdd(p.counter + row_tile, 1);
                const int last = (old == d.pl.splits - 1);
                *c.is_last = last;
                if (last) p.counter[row_tile] = 0;
            }
            consumer_sync(kNCons);
            if (*c.is_last) {
                __threadfence();
                // last CTA of the row tile: add the splits in split order, 8 outputs per thread step
                constexpr int UPT = R / 8;           // 16 threads per token row
                const int units = d.xrows * UPT;
                const int units32 = (units + 31) & ~31;
                for (int i = threadIdx.x; i < units32; i += kNCons) {
                    const int tok = i / UPT;
                    const int c0 = (i - tok * UPT) * 8;
                    const int n0 = row_tile * R + c0;
                    const bool valid = i < units && n0 < d.N;
                    float a0[8], a1[8];
#pragma unroll
                    for (int e = 0; e < 8; e++) a0[e] = a1[e] = 0.f;
                    if (valid) {
                        for (int sp = 0; sp < d.pl.splits; sp++) {
                            const float* src = p.partial + ((size_t)sp * d.pl.row_tiles + row_tile) * MP * TW + (size_t)tok * TW + c0;
                            const float4 u0 = __ldcg(reinterpret_cast<const float4*>(src));
                            const float4 u1 = __ldcg(reinterpret_cast<const float4*>(src) + 1);
                            a0[0] += u0.x; a0[1] += u0.y; a0[2] += u0.z; a0[3] += u0.w;
                            a0[4] += u1.x; a0[5] += u1.y; a0[6] += u1.z; a0[7] += u1.w;
                            if (DUAL) {
                                const float4 v0 = __ldcg(reinterpret_cast<const float4*>(src + R));
                                const float4 v1 = __ldcg(reinterpret_cast<const float4*>(src + R) + 1);
                                a1[0] += v0.x; a1[1] += v0.y; a1[2] += v0.z; a1[3] += v0.w;
                                a1[4] += v1.x; a1[5] += v1.y; a1[6] += v1.z; a1[7] += v1.w;
                            }
                        }
                    }
                    __align__(16) __half out[8];
                    if (EPI == EPI_RESID) {
                        float ss = 0.f;
                        if (valid) {
                            const uint4 rv = __ldcg(reinterpret_cast<const uint4*>(p.h + (size_t)tok * d.N + n0));
                            const uint4 wv = *reinterpret_cast<const uint4*>(d.wn + n0);
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
                            *reinterpret_cast<uint4*>(p.hw + (size_t)tok * d.N + n0) = *reinterpret_cast<const uint4*>(hw);
                        }
#pragma unroll
                        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                        if (valid && (lane & 15) == 0) p.ssq[row_tile * kSsqPitch + tok] = ss;
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
                        *reinterpret_cast<uint4*>(d.y + (size_t)tok * d.N + n0) = *reinterpret_cast<const uint4*>(out);
                    }
                }
            }
            consumer_sync(kNCons);     // is_last is rewritten by the next item
        } else {
            // direct epilogue from registers (QKV / SILU / HEAD without split-K)
            const int nbase = row_tile * R + warp * 16 + g;
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
                    d.y[(size_t)tok * d.N + nn] = o;
                }
            }
        }
    }
}

// ================================================================================ phase 0
__device__ void embed_phase(const FwdParams& p, Ctx& c) {
    const int lane = c.lane;
    const int NP = p.H / 128;
    const int units = p.M * NP;                         // (token, 128-column part), one half-warp each
    const int pairs = (units + 1) / 2;
    const __half* wn = p.layers[0].norm_in;
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
            *reinterpret_cast<uint4*>(p.hw + (size_t)m * p.H + pack * 8) = *reinterpret_cast<const uint4*>(ow);
        } else {
            ss = 0.f;
        }
#pragma unroll
        for (int o2 = 8; o2 > 0; o2 >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o2);
        if (valid && (lane & 15) == 0) p.ssq[part * kSsqPitch + m] = ss;
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

template <int MT, int HD>
__device__ void attn_produce(const FwdParams& p, Ctx& c, const ADesc& a) {
    using G = Geo<MT>;
    constexpr int KS = HD + 8;
    static_assert(2 * kKeyBlock * KS * 2 <= kWArea, "K/V block must fit the weight area of a stage");
    const int lane = c.lane;
    const int nitems = p.Hkv * a.nact;
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
        if (lane == 0) {
            fence_proxy_async();
            mbar_expect_tx(fbar, (uint32_t)rows * HD * 2 * 2);
        }
        __syncwarp();
        unsigned char* stage = c.ring + slot * G::STAGE;
        const __half* kbase = a.kc + ((size_t)hk * p.cap + key0) * HD;
        const __half* vbase = a.vc + ((size_t)hk * p.cap + key0) * HD;
        for (int r = lane; r < rows; r += 32) {
            bulk_copy_g2s(smem_u32(stage + r * KS * 2), kbase + (size_t)r * HD, HD * 2, fbar);
            bulk_copy_g2s(smem_u32(stage + (kKeyBlock + r) * KS * 2), vbase + (size_t)r * HD, HD * 2, fbar);
        }
    }
}

template <int MT, int HD>
__device__ void attn_consume(const FwdParams& p, Ctx& c, const ADesc& a) {
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
                if (key >= a.total) {
                    *reinterpret_cast<uint4*>(sk + r * KS + cv * 8) = make_uint4(0, 0, 0, 0);
                    *reinterpret_cast<uint4*>(sv + r * KS + cv * 8) = make_uint4(0, 0, 0, 0);
                    continue;
                }
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

// Merge of the key blocks: one warp per (token, query head), blocks added in block order.
template <int HD>
__device__ void attn_merge(const FwdParams& p, Ctx& c, const ADesc& a) {
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
        __half* orow = p.attn + (size_t)m * p.Hq * HD + (size_t)head * HD;
#pragma unroll
        for (int cc = 0; cc < CPT; cc++) orow[lane + 32 * cc] = __float2half_rn(acc[cc] * inv);
    }
}

// ================================================================================ the kernel
template <int MT, int HD>
__global__ void __launch_bounds__(kFwdThreads, 1) forward_kernel(const __grid_constant__ FwdParams p) {
    using G = Geo<MT>;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_abort, s_is_last;
    __shared__ float s_rstd[32];
    Ctx c;
    c.ring = smem;
    c.full = reinterpret_cast<uint64_t*>(smem + G::NST * G::STAGE);
    c.empty = c.full + G::NST;
    c.rstd_bar = c.empty + G::NST;
    c.abort_flag = &s_abort;
    c.is_last = &s_is_last;
    c.s_rstd = s_rstd;
    c.pos = 0;
    c.epoch = 0;
    c.rstd_n = 0;
    c.lane = threadIdx.x & 31;
    c.warp = threadIdx.x >> 5;

    if (threadIdx.x == 0) {
        s_abort = 0;
#pragma unroll
        for (int s = 0; s < G::NST; s++) {
            mbar_init(smem_u32(c.full + s), 1);
            mbar_init(smem_u32(c.empty + s), kWN);
        }
        mbar_init(smem_u32(c.rstd_bar), 1);
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
    const int ssq_parts = p.H / 128;

    // ---- phase 0
    if (!producer) {
        embed_phase(p, c);
        grid_barrier(p, c);
    } else {
        c.epoch++;
    }

    for (int l = 0; l < p.L; l++) {
        const LayerPtrs lp = p.layers[l];
        ad.kc = p.kv + (size_t)l * p.kv_layer_stride;
        ad.vc = ad.kc + p.kv_half_stride;
        QDesc d;
        d.xrows = p.M;
        d.rstd_off = 0;
        d.ssq_parts = ssq_parts;
        // ---- A: q|k|v
        d.x = p.hw; d.w0 = lp.qkv_w; d.w1 = nullptr; d.bias = lp.qkv_bias; d.wn = nullptr; d.y = p.qkv;
        d.N = p.NQKV; d.K = p.H; d.pl = p.plan[PLAN_A];
        if (producer) { qmm_produce<MT, false>(p, c, d, c.epoch, true); c.epoch++; }
        else { qmm_consume<MT, false, EPI_QKV>(p, c, d); grid_barrier(p, c); }
        // ---- B1: attention partials (K/V blocks do not depend on this pass: no barrier for the producer)
        if (producer) { attn_produce<MT, HD>(p, c, ad); c.epoch++; }
        else { attn_consume<MT, HD>(p, c, ad); grid_barrier(p, c); }
        // ---- B2: merge
        if (producer) { c.epoch++; }
        else { attn_merge<HD>(p, c, ad); grid_barrier(p, c); }
        // ---- C: h += attn . Wo^T
        d.x = p.attn; d.w0 = lp.o_w; d.bias = nullptr; d.wn = lp.norm_post; d.y = p.h;
        d.N = p.H; d.K = p.Hq * p.HD; d.pl = p.plan[PLAN_C];
        if (producer) { qmm_produce<MT, false>(p, c, d, c.epoch, false); c.epoch++; }
        else { qmm_consume<MT, false, EPI_RESID>(p, c, d); grid_barrier(p, c); }
        // ---- D: act = silu(gate) * up
        d.x = p.hw; d.w0 = lp.gate_w; d.w1 = lp.up_w; d.wn = nullptr; d.y = p.act;
        d.N = p.I; d.K = p.H; d.pl = p.plan[PLAN_D];
        if (producer) { qmm_produce<MT, true>(p, c, d, c.epoch, true); c.epoch++; }
        else { qmm_consume<MT, true, EPI_SILU>(p, c, d); grid_barrier(p, c); }
        // ---- E: h += act . Wdown^T
        d.x = p.act; d.w0 = lp.down_w; d.w1 = nullptr;
        d.wn = (l + 1 < p.L) ? p.layers[l + 1].norm_in : p.final_norm; d.y = p.h;
        d.N = p.H; d.K = p.I; d.pl = p.plan[PLAN_E];
        if (producer) { qmm_produce<MT, false>(p, c, d, c.epoch, false); c.epoch++; }
        else { qmm_consume<MT, false, EPI_RESID>(p, c, d); grid_barrier(p, c); }
    }

    // ---- vocabulary projection on the selected rows
    {
        QDesc d;
        d.xrows = p.rows_out;
        d.rstd_off = row_off;
        d.ssq_parts = ssq_parts;
        d.x = p.hw + (size_t)row_off * p.H; d.w0 = p.head_w; d.w1 = nullptr; d.bias = nullptr; d.wn = nullptr;
        d.y = p.logits; d.N = p.V; d.K = p.H; d.pl = p.plan[PLAN_HEAD];
        if (producer) qmm_produce<MT, false>(p, c, d, c.epoch, true);
        else qmm_consume<MT, false, EPI_HEAD>(p, c, d);
    }

    if (threadIdx.x == 0 && p.timeline != nullptr && (int)c.epoch < p.timeline_pitch)
        p.timeline[((size_t)blockIdx.x * p.timeline_pitch + c.epoch) * 2] = global_ns();
    // ---- leave: the last CTA out resets the barrier words for the next launch (not after an error)
    __syncthreads();
    if (threadIdx.x == 0 && !s_abort) {
        __threadfence();
        const int old = atomicAdd(p.sync + kSyncExit, 1);
        if (old == (int)gridDim.x - 1) {
            p.sync[kSyncBar] = 0;
            p.sync[kSyncExit] = 0;
        }
    }
}

PhasePlan make_plan(int N, int K, int grid, bool allow_split) {
    PhasePlan pl{};
    pl.row_tiles = (N + 127) / 128;
    const int nchunks = K / kChunkK;
    int splits = 1;
    if (allow_split && pl.row_tiles < grid && pl.row_tiles < kMaxCounters) {
        splits = grid / pl.row_tiles;
        const int max_splits = (nchunks + 3) / 4;
        if (splits > max_splits) splits = max_splits;
        if (splits < 1) splits = 1;
    }
    pl.chunks_per_split = (nchunks + splits - 1) / splits;
    pl.splits = (nchunks + pl.chunks_per_split - 1) / pl.chunks_per_split;
    return pl;
}

size_t partial_bytes(const PhasePlan& pl, int mp, bool dual, bool always) {
    if (pl.splits <= 1 && !always) return 0;
    return (size_t)pl.splits * pl.row_tiles * mp * (dual ? 256 : 128) * sizeof(float);
}

struct WsLayout {
    size_t sync, counter, ssq, cs, part_ml, part_o, partial, total;
    int nkb, qrp;
};

int g_fwd_grid = 0;
int fwd_grid() {
    if (g_fwd_grid == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        g_fwd_grid = n;
    }
    return g_fwd_grid;
}


bool fwd_shape_ok(const b200_forward_desc* d) {
    if (!d) return false;
    if (d->M < 1 || d->M > 32 || d->rows_out < 1 || d->rows_out > d->M) return false;
    if (d->hidden < 128 || (d->hidden % 128) != 0 || d->hidden / 128 > kMaxSsqParts) return false;
    if (d->intermediate < 128 || (d->intermediate % 128) != 0) return false;
    if (d->head_dim != 64 && d->head_dim != 128) return false;
    if (d->n_heads < 1 || d->n_kv_heads < 1 || (d->n_heads % d->n_kv_heads) != 0) return false;
    if (((d->n_heads * d->head_dim) % 128) != 0) return false;
    if (d->vocab < 8 || (d->vocab % 8) != 0 || d->n_layers < 1) return false;
    if (d->tail < 1 || d->tail > 64 || d->write_off < 0 || d->write_off + d->M > d->tail) return false;
    if (d->cache_rows < d->tail) return false;
    return true;
}

WsLayout fwd_layout(const b200_forward_desc* d, PhasePlan (&plan)[5]) {
    const int grid = fwd_grid();
    const int mp = ((d->M + 7) / 8) * 8;
    const int nqkv = (d->n_heads + 2 * d->n_kv_heads) * d->head_dim;
    plan[PLAN_A] = make_plan(nqkv, d->hidden, grid, true);
    plan[PLAN_C] = make_plan(d->hidden, d->n_heads * d->head_dim, grid, true);
    plan[PLAN_D] = make_plan(d->intermediate, d->hidden, grid, true);
    plan[PLAN_E] = make_plan(d->hidden, d->intermediate, grid, true);
    plan[PLAN_HEAD] = make_plan(d->vocab, d->hidden, grid, true);
    size_t pb = 0;
    pb = std::max(pb, partial_bytes(plan[PLAN_A], mp, false, false));
    pb = std::max(pb, partial_bytes(plan[PLAN_C], mp, false, true));
    pb = std::max(pb, partial_bytes(plan[PLAN_D], mp, true, false));
    pb = std::max(pb, partial_bytes(plan[PLAN_E], mp, false, true));
    pb = std::max(pb, partial_bytes(plan[PLAN_HEAD], mp, false, false));
    WsLayout w{};
    const int G = d->n_heads / d->n_kv_heads;
    w.qrp = ((d->M * G + 15) / 16) * 16;
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

template <int MT, int HD>
int launch_forward(const FwdParams& p, cudaStream_t stream) {
    auto kern = forward_kernel<MT, HD>;
    bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Geo<MT>::SMEM) != cudaSuccess)
            return check_launch();
        attr_set = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(fwd_grid());
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
int launch_forward_hd(const FwdParams& p, cudaStream_t stream) {
    return p.HD == 128 ? launch_forward<MT, 128>(p, stream) : launch_forward<MT, 64>(p, stream);
}

}  // namespace
}  // namespace b200

extern "C" {

using namespace b200;

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
    const WsLayout w = fwd_layout(d, p.plan);
    if (d->workspace_bytes < w.total) return B200_EWORKSPACE;
    p.M = d->M; p.rows_out = d->rows_out; p.H = d->hidden; p.I = d->intermediate; p.Hq = d->n_heads;
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
    char* ws = static_cast<char*>(d->workspace);
    p.sync = reinterpret_cast<int*>(ws + w.sync);
    p.counter = reinterpret_cast<int*>(ws + w.counter);
    p.ssq = reinterpret_cast<float*>(ws + w.ssq);
    p.cs = reinterpret_cast<float2*>(ws + w.cs);
    p.part_ml = reinterpret_cast<float*>(ws + w.part_ml);
    p.part_o = reinterpret_cast<float*>(ws + w.part_o);
    p.partial = reinterpret_cast<float*>(ws + w.partial);
    p.nkb = w.nkb; p.qrp = w.qrp;
    p.timeline = static_cast<long long*>(d->timeline);
    p.timeline_pitch = d->timeline ? d->timeline_pitch : 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch ((d->M + 7) / 8) {
        case 1: return launch_forward_hd<1>(p, st);
        case 2: return launch_forward_hd<2>(p, st);
        case 3: return launch_forward_hd<3>(p, st);
        default: return launch_forward_hd<4>(p, st);
    }
}

}  // extern "C"
