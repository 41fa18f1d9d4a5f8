// Quantised matmul on weights re-laid-out for streaming ("tiled" layout), sm_100a.
//
// Offline re-layout (the analogue of the reference's swizzle.py / kernels/swizzle.metal): the matrix
// is cut into records of 16 rows x 128 k.  A record is 1152 contiguous bytes: 1024 bytes of packs
// in exactly the order the 32 lanes of a warp consume them (lane (g,t) owns 16 bytes of row g and
// 16 bytes of row g+8: the packs of k-blocks t, 4+t, 8+t, 12+t), then 128 bytes of {scale, bias}
// pairs (row-major, two 64-k groups per row).  Inside a pack the nibbles are re-ordered so that
// the mask pairs 0x000f000f, 0x00f000f0 (and the same after >> 8) yield ADJACENT k pairs
// (k0,k1) (k2,k3) (k4,k5) (k6,k7): the activations can then stay in their natural order.  Records are ordered [64-row block][k chunk][16-row
// tile of the block], so everything a CTA needs for one k chunk of a 64-row block is one
// contiguous 4.5 KiB run, and consecutive chunks follow each other.
//
// Kernel: persistent CTAs (two per SM) loop over (row block, K split) items.  One extra producer
// warp streams the weights with bulk asynchronous copies (cp.async.bulk global -> shared, completion
// counted on an mbarrier) into a ring of stages shared by the CTA and runs ahead across item
// boundaries, so the stream never drains; the consumer warps wait on a stage's "full" barrier
// (bounded), read their own record conflict-free, expand nibbles and feed mma.sync m16n8k16
// (weights = A operand, tokens = B operand, fp32 accumulate) exactly as the row-major kernel does,
// then release the stage on its "empty" barrier.  Split-K partial sums,
// deterministic last-arriver reduction and the fused epilogues are shared with the row-major
// kernel.  The activations of a stage's k range travel in the same stage (one bulk copy per token
// row, issued by one producer lane each, counted on the same barrier), so consumers never synchronise
// block-wide while streaming; results leave through registers.  Every wait is bounded: on a timeout the CTA raises an error flag in the workspace and
// skips the remaining work instead of hanging.  No load in this file uses cluster multicast.
#include "pipeline.cuh"
#include "qmm_common.cuh"

namespace b200 {
namespace {

constexpr int kRec = 1152;            // bytes per 16-row x 128-k record
constexpr int kCPS = 2;               // records (chunks) per ring stage and sub-tile
constexpr int kErrWord = kMaxCounters - 1;   // workspace counter slot used as an error flag
constexpr int kBlockRows = 64;       // rows per layout block (4 records per chunk)

struct TiledParams {
    const __half* x;
    const unsigned char* wt[2];       // tiled weights (gate / up in dual mode)
    const __half* bias;
    const __half* extra;
    __half* y;
    float* partial;
    int* counter;
    int M, N, K;
    int chunks_per_split, splits, row_tiles, epilogue;
};

template <int MT, int S, int WN, bool DUAL>
__global__ void __launch_bounds__((WN + 1) * 32, 2) qmm_tiled_kernel(const TiledParams p) {
    constexpr int RW = DUAL ? 16 : S * 16;
    constexpr int R = WN * RW;
    constexpr int NB = DUAL ? 2 : R / kBlockRows;               // 64-row blocks a stage holds
    constexpr int MP = MT * 8;
    constexpr int TW = DUAL ? 2 * R : R;
    constexpr int BLOCK_STAGE = kCPS * 4 * kRec;                // weight bytes of one block in a stage
    constexpr int XPITCH = kCPS * kChunkK * 2 + 64;             // activation row pitch in a stage
    constexpr int XOFF = NB * BLOCK_STAGE;
    constexpr int STAGE_BYTES = XOFF + MP * XPITCH;
    constexpr int kNST = (NB == 4) ? 2 : ((MT <= 2 && S == 1) ? 4 : 3);   // ring stages
    constexpr int NCONS = WN * 32;
    static_assert(!DUAL || (S == 2 && WN == 4), "dual mode: two sub-tiles, four consumer warps");
    static_assert(DUAL || R % kBlockRows == 0, "CTA rows must be whole layout blocks");

    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_is_last;
    __shared__ int s_abort;
    unsigned char* ring = smem;
    uint64_t* full = reinterpret_cast<uint64_t*>(smem + kNST * STAGE_BYTES);
    uint64_t* empty = full + kNST;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int nchunks_total = p.K / kChunkK;
    const int nblocks = (p.N + kBlockRows - 1) / kBlockRows;
    const int nitems = p.row_tiles * p.splits;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        s_abort = 0;
#pragma unroll
        for (int s = 0; s < kNST; s++) {
            mbar_init(smem_u32(full + s), 1);      // lane 0's expect_tx arrive; bytes counted by the copies
            mbar_init(smem_u32(empty + s), WN);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();
    volatile int* abort_flag = &s_abort;

    if (warp == WN) {
        // ------------------------------------------------------------------ producer warp
        // Weights do not depend on the kernel before this one, activations do: the first stages'
        // weight copies are issued before the programmatic-dependency wait, so the stream starts
        // while the previous kernel is still draining.
        uint32_t ps = 0;
        bool dep_waited = false;
        for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
            const int row_tile = item % p.row_tiles;
            const int split = item / p.row_tiles;
            const int c_begin = split * p.chunks_per_split;
            const int n = min(p.chunks_per_split, nchunks_total - c_begin);
            const int nst = (n + kCPS - 1) / kCPS;
            const unsigned char* src[NB];
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const int blk = min(DUAL ? row_tile : row_tile * NB + b, nblocks - 1);
                src[b] = p.wt[DUAL ? b : 0] + ((size_t)blk * nchunks_total + c_begin) * 4 * kRec;
            }
            const int xrows = min(p.M, MP);
            auto issue_weights = [&](int st, uint32_t slot) {
                const int recs = min(kCPS, n - st * kCPS);
                const uint32_t fbar = smem_u32(full + slot);
                if (lane == 0) {
                    const uint32_t bytes = (uint32_t)(recs * 4 * kRec);
                    fence_proxy_async();
                    mbar_expect_tx(fbar, NB * bytes + (uint32_t)xrows * (uint32_t)(recs * kChunkK * 2));
#pragma unroll
                    for (int b = 0; b < NB; b++)
                        bulk_copy_g2s(smem_u32(ring + slot * STAGE_BYTES + b * BLOCK_STAGE),
                                      src[b] + (size_t)st * kCPS * 4 * kRec, bytes, fbar);
                }
                __syncwarp();
            };
            // activations of a stage's k range: one bulk copy per token row, one lane per row
            // (rows >= M are never written: their accumulator columns are discarded)
            auto issue_x = [&](int st, uint32_t slot) {
                const int recs = min(kCPS, n - st * kCPS);
                if (lane < xrows)
                    bulk_copy_g2s(smem_u32(ring + slot * STAGE_BYTES + XOFF + lane * XPITCH),
                                  p.x + (size_t)lane * p.K + (size_t)(c_begin + st * kCPS) * kChunkK,
                                  (uint32_t)(recs * kChunkK * 2), smem_u32(full + slot));
            };
            int st0 = 0;
            if (!dep_waited) {
                const int pre = min((int)kNST, nst);          // ring is empty: no "empty" waits needed
                for (int st = 0; st < pre; st++) issue_weights(st, (uint32_t)st);
                pdl_wait();
                dep_waited = true;
                for (int st = 0; st < pre; st++) issue_x(st, (uint32_t)st);
                ps = (uint32_t)pre;
                st0 = pre;
            }
            for (int st = st0; st < nst; st++, ps++) {
                const uint32_t slot = ps % kNST, use = ps / kNST;
                bool ok = !*abort_flag;
                if (ok && use > 0 && !mbar_wait_bounded(smem_u32(empty + slot), (use - 1) & 1u)) {
                    ok = false;
                    *abort_flag = 1;
                    if (lane == 0) atomicExch(p.counter + kErrWord, 2);
                }
                if (!ok) return;
                issue_weights(st, slot);
                issue_x(st, slot);
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumers
    pdl_wait();
    uint32_t cs = 0;
    int rec_off[S];
#pragma unroll
    for (int s = 0; s < S; s++) {
        const int tile_in_cta = DUAL ? warp : warp * S + s;
        const int b = DUAL ? s : tile_in_cta / 4;
        const int tib = DUAL ? warp : tile_in_cta % 4;
        rec_off[s] = b * BLOCK_STAGE + tib * kRec;
    }

    for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
        const int row_tile = item % p.row_tiles;
        const int split = item / p.row_tiles;
        const int c_begin = split * p.chunks_per_split;
        const int n = min(p.chunks_per_split, nchunks_total - c_begin);
        const int nst = (n + kCPS - 1) / kCPS;

        float acc[S][MT][4];
#pragma unroll
        for (int s = 0; s < S; s++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[s][mt][i] = 0.f;

        for (int st = 0; st < nst; st++, cs++) {
            const uint32_t slot = cs % kNST;
            bool ok = !*abort_flag;
            if (ok && !mbar_wait_bounded(smem_u32(full + slot), (cs / kNST) & 1u)) {
                ok = false;
                *abort_flag = 1;
                if (lane == 0) atomicExch(p.counter + kErrWord, 1);
            }
            if (ok) {
                const unsigned char* stage = ring + slot * STAGE_BYTES;
#pragma unroll
                for (int cc = 0; cc < kCPS; cc++) {
                    if (st * kCPS + cc < n) {
                        const unsigned char* xrow = stage + XOFF + g * XPITCH + cc * (kChunkK * 2) + t * 16;
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
                                xb[mt] = *reinterpret_cast<const uint4*>(xrow + mt * 8 * XPITCH + j * 64);
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
            if (lane == 0) mbar_arrive(smem_u32(empty + slot));     // stage free for the producer
        }

        // ---- results leave through registers -------------------------------------------------
        // lane (g,t) holds, per sub-tile and token tile: rows g / g+8 x tokens 2t / 2t+1
        if (p.splits > 1) {
            float* mine = p.partial + ((size_t)split * p.row_tiles + row_tile) * MP * TW;
#pragma unroll
            for (int s = 0; s < S; s++) {
                const int ri = DUAL ? (s * R + warp * 16) : (warp * RW + s * 16);
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
            consumer_sync(NCONS);
            if (threadIdx.x == 0) {
                const int old = atomicAdd(p.counter + row_tile, 1);
                s_is_last = (old == p.splits - 1);
                if (s_is_last) p.counter[row_tile] = 0;
            }
            consumer_sync(NCONS);
            if (s_is_last) {
                __threadfence();
                // last CTA of the row tile: add the splits in split order, 8 outputs per thread step
                const int units_per_tok = R / 8;
                for (int i = threadIdx.x; i < p.M * units_per_tok; i += NCONS) {
                    const int tok = i / units_per_tok;
                    const int c0 = (i - tok * units_per_tok) * 8;
                    const int n0 = row_tile * R + c0;
                    if (n0 >= p.N) continue;
                    float a0[8], a1[8];
#pragma unroll
                    for (int e = 0; e < 8; e++) a0[e] = a1[e] = 0.f;
                    for (int sp = 0; sp < p.splits; sp++) {
                        const float* src = p.partial + ((size_t)sp * p.row_tiles + row_tile) * MP * TW + (size_t)tok * TW + c0;
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
                    __align__(16) __half out[8];
                    if (!DUAL && p.epilogue == B200_EPI_F32) {          // partial sums for a tensor-parallel all-reduce
                        float* yf = reinterpret_cast<float*>(p.y) + (size_t)tok * p.N + n0;
                        *reinterpret_cast<float4*>(yf) = make_float4(a0[0], a0[1], a0[2], a0[3]);
                        *reinterpret_cast<float4*>(yf + 4) = make_float4(a0[4], a0[5], a0[6], a0[7]);
                        continue;
                    }
                    if (DUAL) {
#pragma unroll
                        for (int e = 0; e < 8; e++) out[e] = __float2half_rn(silu_mul_f16(a0[e], a1[e]));
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; e++) out[e] = __float2half_rn(a0[e]);
                        if (p.bias != nullptr) {
                            uint4 bv = *reinterpret_cast<const uint4*>(p.bias + n0);
                            const __half* bh = reinterpret_cast<const __half*>(&bv);
#pragma unroll
                            for (int e = 0; e < 8; e++) out[e] = __hadd(out[e], bh[e]);
                        }
                        if (p.epilogue == B200_EPI_RESIDUAL) {
                            uint4 rv = __ldcg(reinterpret_cast<const uint4*>(p.extra + (size_t)tok * p.N + n0));
                            const __half* rh = reinterpret_cast<const __half*>(&rv);
#pragma unroll
                            for (int e = 0; e < 8; e++) out[e] = __hadd(rh[e], out[e]);
                        }
                    }
                    *reinterpret_cast<uint4*>(p.y + (size_t)tok * p.N + n0) = *reinterpret_cast<const uint4*>(out);
                }
            }
            consumer_sync(NCONS);     // s_is_last is rewritten by the next item
        } else {
            constexpr int SS = DUAL ? 1 : S;
#pragma unroll
            for (int s = 0; s < SS; s++) {
                const int nbase = row_tile * R + (DUAL ? warp * 16 : warp * RW + s * 16) + g;
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        const int tok = mt * 8 + 2 * t + (i & 1);
                        const int nn = nbase + ((i >> 1) ? 8 : 0);
                        if (tok >= p.M || nn >= p.N) continue;
                        if (!DUAL && p.epilogue == B200_EPI_F32) {
                            reinterpret_cast<float*>(p.y)[(size_t)tok * p.N + nn] = acc[s][mt][i];
                            continue;
                        }
                        __half o;
                        if (DUAL) {
                            o = __float2half_rn(silu_mul_f16(acc[0][mt][i], acc[S - 1][mt][i]));
                        } else {
                            o = __float2half_rn(acc[s][mt][i]);
                            if (p.bias != nullptr) o = __hadd(o, p.bias[nn]);
                            if (p.epilogue == B200_EPI_RESIDUAL)
                                o = __hadd(__ushort_as_half(__ldcg(reinterpret_cast<const unsigned short*>(p.extra) + (size_t)tok * p.N + nn)), o);
                        }
                        p.y[(size_t)tok * p.N + nn] = o;
                    }
                }
            }
        }
    }
}

// ---- re-layout -------------------------------------------------------------------------------
__global__ void relayout_kernel(const uint32_t* __restrict__ wq, const __half* __restrict__ scales,
                                const __half* __restrict__ biases, uint32_t* __restrict__ out, int N, int K) {
    const int nchunks = K / kChunkK;
    const int rec = blockIdx.x;                 // (block64 * nchunks + c) * 4 + tile in block
    const int tib = rec & 3, bc = rec >> 2;
    const int blk = bc / nchunks, c = bc - blk * nchunks;
    const int t16 = blk * 4 + tib;
    const int i = threadIdx.x;                  // 0..287: u32 index inside the record
    pdl_wait();
    uint32_t v = 0;
    if (i < 256) {
        const int hh = i >> 7, lane = (i >> 2) & 31, j = i & 3;
        const int row = t16 * 16 + (lane >> 2) + 8 * hh;
        if (row < N) {
            const uint32_t w = wq[(size_t)row * (K / 8) + c * 16 + j * 4 + (lane & 3)];
            // element e (bits 4e..4e+3 in the MLX pack) moves to nibble (e >> 1) + 4 * (e & 1)
#pragma unroll
            for (int e = 0; e < 8; e++) v |= ((w >> (4 * e)) & 0xfu) << (4 * ((e >> 1) + 4 * (e & 1)));
        }
    } else {
        const int q = i - 256, row = t16 * 16 + (q >> 1), grp = q & 1;
        if (row < N) {
            const unsigned short s = __half_as_ushort(scales[(size_t)row * (K / 64) + 2 * c + grp]);
            const unsigned short b = __half_as_ushort(biases[(size_t)row * (K / 64) + 2 * c + grp]);
            v = (uint32_t)s | ((uint32_t)b << 16);
        }
    }
    out[(size_t)rec * (kRec / 4) + i] = v;
}

struct TPlan {
    int mt, wn, s, splits, chunks_per_split, row_tiles, rows_per_cta, tile_width, grid;
    size_t smem_bytes, partial_bytes;
};

int g_sms = 0;
int sms() {
    if (g_sms == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        g_sms = n;
    }
    return g_sms;
}

TPlan make_tplan(int M, int N, int K, bool dual, long long ws_bytes) {
    TPlan pl{};
    pl.mt = (M + 7) / 8;
    const int slots0 = 2 * sms();
    // 9..16 rows: two sub-tiles per warp halve the activation traffic from shared memory; worth it
    // when 256-row blocks alone give every SM work (the vocabulary projection)
    const bool wide16 = !dual && pl.mt == 2 && (N + 255) / 256 >= slots0 / 2;
    const int S = dual ? 2 : ((pl.mt >= 3 || wide16) ? 2 : 1);
    const int rw = dual ? 16 : S * 16;
    const int slots = 2 * sms();                       // resident CTAs: one wave of the persistent grid
    const int nchunks = K / kChunkK;
    // two 16-row sub-tiles per warp need twice the ring: four warps then; otherwise eight warps when
    // that alone gives every SM a row block
    pl.wn = (S == 1 && (N + 8 * rw - 1) / (8 * rw) >= slots / 2) ? 8 : 4;
    if (wide16) pl.wn = 8;
    pl.s = S;
    pl.rows_per_cta = pl.wn * rw;
    pl.tile_width = dual ? 2 * pl.rows_per_cta : pl.rows_per_cta;
    pl.row_tiles = (N + pl.rows_per_cta - 1) / pl.rows_per_cta;
    // Split K so that the items fill the resident CTAs about evenly; keep >= 4 chunks per split.
    int splits = 1;
    if (pl.row_tiles < slots && pl.row_tiles < kErrWord) {
        splits = slots / pl.row_tiles;
        const int max_splits = (nchunks + 3) / 4;
        if (splits > max_splits) splits = max_splits;
        if (splits < 1) splits = 1;
    }
    auto pbytes = [&](int sp) {
        return sp > 1 ? (size_t)sp * pl.row_tiles * pl.mt * 8 * pl.tile_width * sizeof(float) : (size_t)0;
    };
    if (ws_bytes >= 0)
        while (splits > 1 && (long long)(kCounterBytes + pbytes(splits)) > ws_bytes) splits--;
    pl.chunks_per_split = (nchunks + splits - 1) / splits;
    pl.splits = (nchunks + pl.chunks_per_split - 1) / pl.chunks_per_split;
    pl.partial_bytes = pbytes(pl.splits);
    const int nb = dual ? 2 : pl.rows_per_cta / kBlockRows;
    const int nst = nb == 4 ? 2 : ((pl.mt <= 2 && S == 1) ? 4 : 3);
    pl.smem_bytes = (size_t)nst * ((size_t)nb * kCPS * 4 * kRec + (size_t)pl.mt * 8 * (kCPS * kChunkK * 2 + 64)) +
                    (size_t)nst * 16;
    const int items = pl.row_tiles * pl.splits;
    pl.grid = items < slots ? items : slots;
    return pl;
}

template <int MT, int S, int WN, bool DUAL>
int launch_t(const TiledParams& p, const TPlan& pl, cudaStream_t stream) {
    auto kern = qmm_tiled_kernel<MT, S, WN, DUAL>;
    // per launch: the attribute belongs to the current device, and a process may drive several
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 111 * 1024) != cudaSuccess)
        return check_launch();
    launch_kernel(kern, dim3(pl.grid), dim3((WN + 1) * 32), pl.smem_bytes, stream, p);
    return check_launch();
}

template <int MT>
int launch_tmt(const TiledParams& p, const TPlan& pl, bool dual, cudaStream_t stream) {
    constexpr int S = (MT >= 3) ? 2 : 1;
    if (dual) return launch_t<MT, 2, 4, true>(p, pl, stream);
    if constexpr (MT == 2) {
        if (pl.s == 2) return pl.wn == 8 ? launch_t<2, 2, 8, false>(p, pl, stream) : launch_t<2, 2, 4, false>(p, pl, stream);
    }
    if constexpr (S == 2) {
        return launch_t<MT, S, 4, false>(p, pl, stream);
    } else {
        return pl.wn == 8 ? launch_t<MT, S, 8, false>(p, pl, stream) : launch_t<MT, S, 4, false>(p, pl, stream);
    }
}

}  // namespace
}  // namespace b200

extern "C" {

size_t b200_qmm_tiled_bytes(int N, int K) {
    if (N < 1 || K < b200::kChunkK || (K % b200::kChunkK) != 0) return 0;
    return (size_t)((N + b200::kBlockRows - 1) / b200::kBlockRows) * (K / b200::kChunkK) * 4 * b200::kRec;
}

int b200_qmm_relayout(const uint32_t* wq, const void* scales, const void* biases, void* out, int N, int K,
                      void* stream) {
    if (!wq || !scales || !biases || !out || N < 1 || K < b200::kChunkK || (K % b200::kChunkK) != 0) return B200_EINVAL;
    if (!b200::aligned16(out)) return B200_EALIGN;
    const int recs = ((N + b200::kBlockRows - 1) / b200::kBlockRows) * (K / b200::kChunkK) * 4;
    b200::launch_kernel(b200::relayout_kernel, dim3(recs), dim3(b200::kRec / 4), 0, static_cast<cudaStream_t>(stream),
                        wq, static_cast<const __half*>(scales), static_cast<const __half*>(biases),
                        static_cast<uint32_t*>(out), N, K);
    return b200::check_launch();
}

size_t b200_qmm_tiled_workspace_bytes(int M, int N, int K) {
    if (M < 1 || N < 8 || K < b200::kChunkK || (K % b200::kChunkK) != 0) return 0;
    if (M > 32) M = 32;
    size_t need = b200::kCounterBytes;
    for (int dual = 0; dual < 2; dual++) {
        b200::TPlan pl = b200::make_tplan(M, N, K, dual != 0, -1);
        const size_t b = b200::kCounterBytes + pl.partial_bytes;
        if (b > need) need = b;
    }
    return need;
}

int b200_qmm_tiled(const void* x, const void* wt, const void* wt2, const void* bias, const void* extra, void* y,
                   int M, int N, int K, int epilogue, void* workspace, size_t workspace_bytes, void* stream) {
    if (M < 1 || M > 32 || N < 8 || (N % 8) != 0 || K < b200::kChunkK || (K % b200::kChunkK) != 0) return B200_EINVAL;
    if (epilogue < B200_EPI_NONE || epilogue > B200_EPI_F32) return B200_EINVAL;
    if (epilogue == B200_EPI_F32 && bias) return B200_EINVAL;
    const bool dual = epilogue == B200_EPI_SILU_MUL;
    if (!x || !wt || !y || !workspace || (dual && (!wt2 || bias)) || (epilogue == B200_EPI_RESIDUAL && !extra))
        return B200_EINVAL;
    if (!b200::aligned16(x) || !b200::aligned16(wt) || !b200::aligned16(wt2) || !b200::aligned16(y) ||
        !b200::aligned16(bias) || !b200::aligned16(extra) || !b200::aligned16(workspace))
        return B200_EALIGN;
    if (workspace_bytes < (size_t)b200::kCounterBytes) return B200_EWORKSPACE;
    b200::TPlan pl = b200::make_tplan(M, N, K, dual, (long long)workspace_bytes);
    if (pl.splits > 1 && (size_t)b200::kCounterBytes + pl.partial_bytes > workspace_bytes) return B200_EWORKSPACE;
    b200::TiledParams p{};
    p.x = static_cast<const __half*>(x);
    p.wt[0] = static_cast<const unsigned char*>(wt);
    p.wt[1] = static_cast<const unsigned char*>(dual ? wt2 : wt);
    p.bias = static_cast<const __half*>(bias);
    p.extra = static_cast<const __half*>(extra);
    p.y = static_cast<__half*>(y);
    p.counter = static_cast<int*>(workspace);
    p.partial = reinterpret_cast<float*>(static_cast<char*>(workspace) + b200::kCounterBytes);
    p.M = M; p.N = N; p.K = K;
    p.chunks_per_split = pl.chunks_per_split; p.splits = pl.splits; p.row_tiles = pl.row_tiles; p.epilogue = epilogue;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (pl.mt) {
        case 1: return b200::launch_tmt<1>(p, pl, dual, st);
        case 2: return b200::launch_tmt<2>(p, pl, dual, st);
        case 3: return b200::launch_tmt<3>(p, pl, dual, st);
        default: return b200::launch_tmt<4>(p, pl, dual, st);
    }
}

}  // extern "C"
