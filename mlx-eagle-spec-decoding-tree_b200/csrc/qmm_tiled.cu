// Quantised matmul on weights re-laid-out for streaming ("tiled" layout), sm_100a.
//
// Offline re-layout (the analogue of the reference's swizzle.py / kernels/swizzle.metal): the matrix
// is cut into records of 16 rows x 128 k.  A record is 1152 contiguous bytes: 1024 bytes of packs
// in exactly the order the 32 lanes of a warp consume them (lane (g,t) owns 16 bytes of row g and
// 16 bytes of row g+8: the packs of k-blocks t, 4+t, 8+t, 12+t), then 128 bytes of {scale, bias}
// pairs (row-major, two 64-k groups per row).  Records of one 16-row tile are consecutive along K,
// so a warp streams one contiguous region.
//
// Kernel: persistent CTAs (at most two per SM) loop over (row block, K split) items.  Every warp
// owns a private ring of shared-memory stages filled by bulk asynchronous copies
// (cp.async.bulk global -> shared, completion counted on an mbarrier): lane 0 keeps 3-4 stages of
// 2 records in flight, all lanes wait on the stage's barrier (bounded), read their 16-byte pieces
// conflict-free, expand nibbles and feed mma.sync m16n8k16 (weights = A operand, tokens = B
// operand, fp32 accumulate) exactly as the row-major kernel does.  No block-wide barrier sits
// inside the stream of an item; activations are staged once per item in shared memory.
// Split-K partial sums, deterministic last-arriver reduction and the fused epilogues are shared
// with the row-major kernel.  No load in this file uses cluster multicast.
#include "qmm_common.cuh"

namespace b200 {
namespace {

constexpr int kRec = 1152;            // bytes per 16-row x 128-k record
constexpr int kCPS = 2;               // records (chunks) per ring stage and sub-tile
constexpr int kErrWord = kMaxCounters - 1;   // workspace counter slot used as an error flag
constexpr uint32_t kWaitLimit = 1u << 22;

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

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: returns false if the barrier did not complete within the iteration limit.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kWaitLimit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }

template <int MT, int S, int WN, bool DUAL>
__global__ void __launch_bounds__(WN * 32, 2) qmm_tiled_kernel(const TiledParams p) {
    constexpr int KS = (MT == 1) ? 16 : (MT == 2 ? 8 : 4);      // chunks of x resident in smem
    constexpr int kNST = (S == 1) ? 4 : 3;                      // ring stages per warp
    constexpr int RW = DUAL ? 16 : S * 16;
    constexpr int R = WN * RW;
    constexpr int TW = DUAL ? 2 * R : R;
    constexpr int XSTRIDE = KS * kChunkK * 2 + 64;
    constexpr int XBYTES = MT * 8 * XSTRIDE;
    constexpr int STAGE_BYTES = S * kCPS * kRec;
    constexpr int RING_BYTES = kNST * STAGE_BYTES;
    constexpr int TSTRIDE = TW + 1;
    static_assert(!DUAL || S == 2, "dual mode needs two sub-tiles");
    static_assert(MT * 8 * TSTRIDE * 4 <= XBYTES, "epilogue tile must fit in the activation slice");
    static_assert(KS % kCPS == 0, "slice must hold whole stages");

    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_is_last;
    unsigned char* xs = smem;
    unsigned char* ring = smem + XBYTES + (threadIdx.x >> 5) * RING_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + XBYTES + WN * RING_BYTES) + (threadIdx.x >> 5) * kNST;

    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int nchunks_total = p.K / kChunkK;
    const int tiles16 = (p.N + 15) / 16;
    const int nitems = p.row_tiles * p.splits;

    if (lane == 0) {
#pragma unroll
        for (int s = 0; s < kNST; s++) mbar_init(smem_u32(bars + s), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    uint32_t gstage = 0;     // stages issued == stages consumed at item boundaries (per warp)
    const int MP = MT * 8;
    float* tile = reinterpret_cast<float*>(xs);

    for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
        const int row_tile = item % p.row_tiles;
        const int split = item / p.row_tiles;
        const int c_begin = split * p.chunks_per_split;
        const int n = min(p.chunks_per_split, nchunks_total - c_begin);
        const int nst = (n + kCPS - 1) / kCPS;

        const unsigned char* src[S];
#pragma unroll
        for (int s = 0; s < S; s++) {
            int t16 = (row_tile * R + warp * RW) / 16 + (DUAL ? 0 : s);
            t16 = min(t16, tiles16 - 1);
            src[s] = p.wt[DUAL ? s : 0] + ((size_t)t16 * nchunks_total + c_begin) * kRec;
        }
        auto issue = [&](int st) {          // lane 0 only
            const uint32_t slot = (gstage + st) % kNST;
            const int recs = min(kCPS, n - st * kCPS);
            const uint32_t bar = smem_u32(bars + slot);
            mbar_expect_tx(bar, (uint32_t)(S * recs * kRec));
#pragma unroll
            for (int s = 0; s < S; s++)
                bulk_copy_g2s(smem_u32(ring + slot * STAGE_BYTES + s * kCPS * kRec),
                              src[s] + (size_t)st * kCPS * kRec, (uint32_t)(recs * kRec), bar);
        };
        if (lane == 0) {
            fence_proxy_async();
            for (int st = 0; st < min(kNST, nst); st++) issue(st);
        }

        float acc[S][MT][4];
#pragma unroll
        for (int s = 0; s < S; s++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[s][mt][i] = 0.f;

        bool failed = false;
        for (int st = 0; st < nst; st++) {
            if ((st * kCPS) % KS == 0) {
                // activation slice for chunks [st*CPS, +KS) of this item: natural k order, halves of
                // every 8-block reordered to (0,4,1,5,2,6,3,7) to match the nibble pairs of a pack
                if (st > 0) __syncthreads();
                const int c0 = st * kCPS;
                const int slice_chunks = min(KS, n - c0);
                const int blocks_per_row = slice_chunks * 16;
                const int total = MP * blocks_per_row;
                const __half* xbase = p.x + (size_t)(c_begin + c0) * kChunkK;
                for (int i = threadIdx.x; i < total; i += WN * 32) {
                    const int m = i / blocks_per_row;
                    const int bb = i - m * blocks_per_row;
                    uint4 v = make_uint4(0u, 0u, 0u, 0u);
                    if (m < p.M) v = *reinterpret_cast<const uint4*>(xbase + (size_t)m * p.K + bb * 8);
                    uint4 o;
                    o.x = __byte_perm(v.x, v.z, 0x5410);
                    o.y = __byte_perm(v.x, v.z, 0x7632);
                    o.z = __byte_perm(v.y, v.w, 0x5410);
                    o.w = __byte_perm(v.y, v.w, 0x7632);
                    *reinterpret_cast<uint4*>(xs + (size_t)m * XSTRIDE + bb * 16) = o;
                }
                __syncthreads();
            }
            const uint32_t gs = gstage + st;
            const uint32_t slot = gs % kNST;
            if (!failed && !mbar_wait_bounded(smem_u32(bars + slot), (gs / kNST) & 1u)) {
                failed = true;
                if (lane == 0) atomicExch(p.counter + kErrWord, 1);
            }
            if (!failed) {
                const unsigned char* stage = ring + slot * STAGE_BYTES;
#pragma unroll
                for (int cc = 0; cc < kCPS; cc++) {
                    if (st * kCPS + cc < n) {
                        const int cslice = (st * kCPS + cc) % KS;
                        const unsigned char* xrow = xs + (size_t)g * XSTRIDE + cslice * (kChunkK * 2) + t * 16;
                        uint4 w[S][2];
                        uint2 sb[S][2];
#pragma unroll
                        for (int s = 0; s < S; s++) {
                            const unsigned char* rec = stage + (s * kCPS + cc) * kRec;
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
                                xb[mt] = *reinterpret_cast<const uint4*>(xrow + (size_t)mt * 8 * XSTRIDE + j * 64);
#pragma unroll
                            for (int s = 0; s < S; s++) {
                                const uint32_t p0 = (j < 2) ? sb[s][0].x : sb[s][0].y;
                                const uint32_t p1 = (j < 2) ? sb[s][1].x : sb[s][1].y;
                                uint32_t d0[4], d1[4];
                                dequant_pack(comp(w[s][0], j), u32_as_h2(__byte_perm(p0, p0, 0x1010)),
                                             u32_as_h2(__byte_perm(p0, p0, 0x3232)), d0);
                                dequant_pack(comp(w[s][1], j), u32_as_h2(__byte_perm(p1, p1, 0x1010)),
                                             u32_as_h2(__byte_perm(p1, p1, 0x3232)), d1);
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
            if (lane == 0 && !failed && st + kNST < nst) {
                fence_proxy_async();
                issue(st + kNST);
            }
        }
        if (failed && lane == 0) {
            // give copies still in flight a (bounded) chance to land before this warp moves on
            for (int st = 0; st < kNST; st++) mbar_wait_bounded(smem_u32(bars + st), ((gstage + nst) / kNST) & 1u);
        }
        gstage += (uint32_t)nst;

        // ---- split-K reduction and epilogue (tile overlays the activation slice) --------------
        __syncthreads();
        bool do_epilogue = true;
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
            __syncthreads();
            if (threadIdx.x == 0) {
                const int old = atomicAdd(p.counter + row_tile, 1);
                s_is_last = (old == p.splits - 1);
                if (s_is_last) p.counter[row_tile] = 0;
            }
            __syncthreads();
            do_epilogue = s_is_last;
            if (do_epilogue) {
                __threadfence();
                for (int i = threadIdx.x; i < MP * TW; i += WN * 32) {
                    const int tok = i / TW, ri = i - tok * TW;
                    float sum = 0.f;
                    for (int sp = 0; sp < p.splits; sp++)
                        sum += __ldcg(p.partial + ((size_t)sp * p.row_tiles + row_tile) * MP * TW + i);
                    tile[tok * TSTRIDE + ri] = sum;
                }
            }
        } else {
#pragma unroll
            for (int s = 0; s < S; s++) {
                const int ri = DUAL ? (s * R + warp * 16) : (warp * RW + s * 16);
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    const int tok = mt * 8 + 2 * t;
                    tile[tok * TSTRIDE + ri + g] = acc[s][mt][0];
                    tile[(tok + 1) * TSTRIDE + ri + g] = acc[s][mt][1];
                    tile[tok * TSTRIDE + ri + g + 8] = acc[s][mt][2];
                    tile[(tok + 1) * TSTRIDE + ri + g + 8] = acc[s][mt][3];
                }
            }
        }
        if (do_epilogue) {
            __syncthreads();
            const int units_per_tok = R / 8;
            for (int i = threadIdx.x; i < p.M * units_per_tok; i += WN * 32) {
                const int tok = i / units_per_tok;
                const int c0 = (i - tok * units_per_tok) * 8;
                const int n0 = row_tile * R + c0;
                if (n0 >= p.N) continue;
                __align__(16) __half out[8];
                if (DUAL) {
#pragma unroll
                    for (int e = 0; e < 8; e++)
                        out[e] = __float2half_rn(silu_mul_f16(tile[tok * TSTRIDE + c0 + e], tile[tok * TSTRIDE + R + c0 + e]));
                } else {
#pragma unroll
                    for (int e = 0; e < 8; e++) out[e] = __float2half_rn(tile[tok * TSTRIDE + c0 + e]);
                    if (p.bias != nullptr) {
                        uint4 bv = *reinterpret_cast<const uint4*>(p.bias + n0);
                        const __half* bh = reinterpret_cast<const __half*>(&bv);
#pragma unroll
                        for (int e = 0; e < 8; e++) out[e] = __hadd(out[e], bh[e]);
                    }
                    if (p.epilogue == B200_EPI_RESIDUAL) {
                        uint4 rv = *reinterpret_cast<const uint4*>(p.extra + (size_t)tok * p.N + n0);
                        const __half* rh = reinterpret_cast<const __half*>(&rv);
#pragma unroll
                        for (int e = 0; e < 8; e++) out[e] = __hadd(rh[e], out[e]);
                    }
                }
                *reinterpret_cast<uint4*>(p.y + (size_t)tok * p.N + n0) = *reinterpret_cast<const uint4*>(out);
            }
        }
        __syncthreads();      // tile / activation slice free for the next item
    }
}

// ---- re-layout -------------------------------------------------------------------------------
__global__ void relayout_kernel(const uint32_t* __restrict__ wq, const __half* __restrict__ scales,
                                const __half* __restrict__ biases, uint32_t* __restrict__ out, int N, int K) {
    const int nchunks = K / kChunkK;
    const int rec = blockIdx.x;                 // t16 * nchunks + c
    const int t16 = rec / nchunks, c = rec - t16 * nchunks;
    const int i = threadIdx.x;                  // 0..287: u32 index inside the record
    uint32_t v = 0;
    if (i < 256) {
        const int hh = i >> 7, lane = (i >> 2) & 31, j = i & 3;
        const int row = t16 * 16 + (lane >> 2) + 8 * hh;
        if (row < N) v = wq[(size_t)row * (K / 8) + c * 16 + j * 4 + (lane & 3)];
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
    int mt, wn, splits, chunks_per_split, row_tiles, rows_per_cta, tile_width, grid;
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
    const int S = dual ? 2 : (pl.mt >= 3 ? 2 : 1);
    const int rw = dual ? 16 : S * 16;
    const int slots = 2 * sms();                       // resident CTAs: one wave of the persistent grid
    const int nchunks = K / kChunkK;
    // two 16-row sub-tiles per warp need twice the ring: four warps then; otherwise eight warps when
    // that alone gives every SM a row block
    pl.wn = (S == 1 && (N + 8 * rw - 1) / (8 * rw) >= slots / 2) ? 8 : 4;
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
    const int ks = pl.mt == 1 ? 16 : (pl.mt == 2 ? 8 : 4);
    const int nst = S == 1 ? 4 : 3;
    pl.smem_bytes = (size_t)pl.mt * 8 * (ks * kChunkK * 2 + 64) + (size_t)pl.wn * nst * S * kCPS * kRec +
                    (size_t)pl.wn * nst * 8;
    const int items = pl.row_tiles * pl.splits;
    pl.grid = items < slots ? items : slots;
    return pl;
}

template <int MT, int S, int WN, bool DUAL>
int launch_t(const TiledParams& p, const TPlan& pl, cudaStream_t stream) {
    auto kern = qmm_tiled_kernel<MT, S, WN, DUAL>;
    static bool attr_set = false;
    if (!attr_set) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 112 * 1024) != cudaSuccess)
            return check_launch();
        attr_set = true;
    }
    kern<<<pl.grid, WN * 32, pl.smem_bytes, stream>>>(p);
    return check_launch();
}

template <int MT>
int launch_tmt(const TiledParams& p, const TPlan& pl, bool dual, cudaStream_t stream) {
    constexpr int S = (MT >= 3) ? 2 : 1;
    if (dual) return pl.wn == 8 ? launch_t<MT, 2, 8, true>(p, pl, stream) : launch_t<MT, 2, 4, true>(p, pl, stream);
    return pl.wn == 8 ? launch_t<MT, S, 8, false>(p, pl, stream) : launch_t<MT, S, 4, false>(p, pl, stream);
}

}  // namespace
}  // namespace b200

extern "C" {

size_t b200_qmm_tiled_bytes(int N, int K) {
    if (N < 1 || K < b200::kChunkK || (K % b200::kChunkK) != 0) return 0;
    return (size_t)((N + 15) / 16) * (K / b200::kChunkK) * b200::kRec;
}

int b200_qmm_relayout(const uint32_t* wq, const void* scales, const void* biases, void* out, int N, int K,
                      void* stream) {
    if (!wq || !scales || !biases || !out || N < 1 || K < b200::kChunkK || (K % b200::kChunkK) != 0) return B200_EINVAL;
    if (!b200::aligned16(out)) return B200_EALIGN;
    const int recs = ((N + 15) / 16) * (K / b200::kChunkK);
    b200::relayout_kernel<<<recs, b200::kRec / 4, 0, static_cast<cudaStream_t>(stream)>>>(
        wq, static_cast<const __half*>(scales), static_cast<const __half*>(biases), static_cast<uint32_t*>(out), N, K);
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
    if (epilogue < B200_EPI_NONE || epilogue > B200_EPI_SILU_MUL) return B200_EINVAL;
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
