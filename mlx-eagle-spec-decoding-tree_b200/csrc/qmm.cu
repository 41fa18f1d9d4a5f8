// Batched 4-bit affine quantised matmul for 1..32 rows ("tree tokens") on sm_100a.
//
//   y[M,N] = x[M,K] . dequant(W[N,K])^T        W packed 8 x 4 bit per uint32 (element j in bits
//                                               4j..4j+3), one fp16 scale and bias per 64 k.
//
// The op is HBM-bound (0.5625 byte per weight, every weight used once), so the kernel is a
// weight streamer:
//   * each lane keeps a ring of 128-bit weight loads in flight straight from global memory
//     (non-coherent, no L1 allocation); a warp owns 16 (or 32) weight rows and walks K in chunks
//     of 128, a quad of lanes covering 64 contiguous bytes of a row per load;
//   * nibbles are expanded to fp16 in registers with the 0x6400 exponent trick and the exact
//     value q is dequantised with one HFMA2 (q*s+b, single rounding - the reference shader's
//     `half2(q) * s0 + b0`, simd_no_swizzle_cast.metal:83);
//   * the products go through mma.sync m16n8k16 with the WEIGHTS as the 16-row A operand and
//     the tokens as the 8-wide B operand, fp32 accumulation.  Which k lands in which fragment
//     slot is free as long as both operands agree, so the natural nibble pairs (e0,e4), (e1,e5),
//     (e2,e6), (e3,e7) of a pack are used as they come and the activations are stored in shared
//     memory in the matching order once per CTA;
//   * small-N layers are split along K across CTAs; partial sums go to a caller-provided
//     workspace and the last CTA of a row tile adds them in split order (deterministic) and runs
//     the epilogue (bias / residual add / SiLU-gate multiply).
#include "qmm_common.cuh"

namespace b200 {
namespace {

template <int S>
struct Stage {
    uint4 w[S][2];
    unsigned short s[S][2];
    unsigned short b[S][2];
};

// MT: token tiles of 8 (M <= 8*MT).  S: 16-row sub-tiles per warp.  WN: warps per CTA, all along
// the rows.  DUAL: sub-tile 0 reads weight set 0 (gate), sub-tile 1 weight set 1 (up), same rows.
template <int MT, int S, int WN, bool DUAL>
__global__ void __launch_bounds__(WN * 32)
qmm_kernel(const QmmParams p) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int PF = (S == 1) ? 4 : 2;                       // weight chunks in flight per lane
    constexpr int KS = (MT == 1) ? 32 : (MT == 2 ? 16 : 8);    // chunks of x resident in smem
    constexpr int RW = DUAL ? 16 : S * 16;                      // output rows per warp
    constexpr int R = WN * RW;                                  // output rows per CTA
    constexpr int TW = DUAL ? 2 * R : R;                        // accumulator rows per CTA
    constexpr int XSTRIDE = KS * kChunkK * 2 + 64;              // bytes per token row in smem
    static_assert(!DUAL || S == 2, "dual mode needs two sub-tiles");

    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int s_is_last;

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;
    const int g = lane >> 2;
    const int t = lane & 3;
    const int row_tile = blockIdx.x;
    const int split = blockIdx.y;
    const int nchunks_total = p.K / kChunkK;
    const int c_begin = split * p.chunks_per_split;
    const int n = min(p.chunks_per_split, nchunks_total - c_begin);

    const int row_words = p.K / 8;
    const int row_groups = p.K / 64;

    const uint4* wptr[S][2];
    const unsigned short* sptr[S][2];
    const unsigned short* bptr[S][2];
#pragma unroll
    for (int s = 0; s < S; s++) {
        const int set = DUAL ? s : 0;
        const int base = row_tile * R + warp * RW + (DUAL ? 0 : s * 16);
#pragma unroll
        for (int hh = 0; hh < 2; hh++) {
            const int r = min(base + g + 8 * hh, p.N - 1);
            wptr[s][hh] = reinterpret_cast<const uint4*>(p.wq[set] + (size_t)r * row_words) + t;
            sptr[s][hh] = reinterpret_cast<const unsigned short*>(p.sc[set]) +
                          (size_t)r * row_groups + (t >> 1);
            bptr[s][hh] = reinterpret_cast<const unsigned short*>(p.bi[set]) +
                          (size_t)r * row_groups + (t >> 1);
        }
    }

    Stage<S> st[PF];
    auto load_stage = [&](Stage<S>& dst, int c) {
#pragma unroll
        for (int s = 0; s < S; s++)
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                dst.w[s][hh] = ldg_nc_v4(wptr[s][hh] + c * 4);
                dst.s[s][hh] = __ldg(sptr[s][hh] + c * 2);
                dst.b[s][hh] = __ldg(bptr[s][hh] + c * 2);
            }
    };

    float acc[S][MT][4];
#pragma unroll
    for (int s = 0; s < S; s++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[s][mt][i] = 0.f;

#pragma unroll
    for (int u = 0; u < PF; u++)
        if (u < n) load_stage(st[u], c_begin + u);

    auto consume = [&](const Stage<S>& cur, int cc) {
        const unsigned char* xrow = smem + (size_t)g * XSTRIDE + cc * (kChunkK * 2) + t * 16;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            uint4 xb[MT];
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
                xb[mt] = *reinterpret_cast<const uint4*>(xrow + (size_t)mt * 8 * XSTRIDE + j * 64);
#pragma unroll
            for (int s = 0; s < S; s++) {
                uint32_t d0[4], d1[4];
                dequant_pack(comp(cur.w[s][0], j), dup_half(cur.s[s][0]), dup_half(cur.b[s][0]), d0);
                dequant_pack(comp(cur.w[s][1], j), dup_half(cur.s[s][1]), dup_half(cur.b[s][1]), d1);
#pragma unroll
                for (int mt = 0; mt < MT; mt++) {
                    mma_m16n8k16(acc[s][mt], d0[0], d1[0], d0[1], d1[1], xb[mt].x, xb[mt].y);
                    mma_m16n8k16(acc[s][mt], d0[2], d1[2], d0[3], d1[3], xb[mt].z, xb[mt].w);
                }
            }
        }
    };

    for (int c = 0; c < n; c += PF) {
        if (c % KS == 0) {
            // (Re)stage the activation slice for chunks [c, c+KS) of this CTA's K range, in the
            // fragment order the lanes read it: 16-byte block (t*4+j) of a 128-k segment goes to
            // slot (j*4+t), halves of a block reordered to (0,4,1,5,2,6,3,7).
            __syncthreads();
            const int slice_chunks = min(KS, n - c);
            const int blocks_per_row = slice_chunks * 16;
            const int total = MT * 8 * blocks_per_row;
            const __half* xbase = p.x + (size_t)(c_begin + c) * kChunkK;
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
                const int seg = bb >> 4, b16 = bb & 15;
                const int slot = ((b16 & 3) << 2) | (b16 >> 2);
                *reinterpret_cast<uint4*>(smem + (size_t)m * XSTRIDE + seg * (kChunkK * 2) + slot * 16) = o;
            }
            __syncthreads();
        }
#pragma unroll
        for (int u = 0; u < PF; u++) {
            if (c + u < n) {
                consume(st[u], (c + u) % KS);
                if (c + u + PF < n) load_stage(st[u], c_begin + c + u + PF);
            }
        }
    }

    // ---- reduction across K splits (if any) and epilogue --------------------------------------
    const int MP = MT * 8;
    float* tile = reinterpret_cast<float*>(smem);   // [MP][TW + 1] fp32, reuses the x slice
    constexpr int TSTRIDE = TW + 1;
    bool do_epilogue = true;
    __syncthreads();
    if (p.splits > 1) {
        float* mine = p.partial + ((size_t)split * gridDim.x + row_tile) * MP * TW;
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
            int old = atomicAdd(p.counter + row_tile, 1);
            s_is_last = (old == p.splits - 1);
            if (s_is_last) p.counter[row_tile] = 0;   // ready for the next launch
        }
        __syncthreads();
        do_epilogue = s_is_last;
        if (do_epilogue) {
            __threadfence();
            for (int i = threadIdx.x; i < MP * TW; i += WN * 32) {
                const int tok = i / TW, ri = i - tok * TW;
                float sum = 0.f;
                for (int sp = 0; sp < p.splits; sp++)
                    sum += __ldcg(p.partial + ((size_t)sp * gridDim.x + row_tile) * MP * TW + i);
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
    if (!do_epilogue) return;
    __syncthreads();

    // One unit = 8 consecutive output columns of one token (a 16-byte store).
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
                out[e] = __float2half_rn(silu_mul_f16(tile[tok * TSTRIDE + c0 + e],
                                                      tile[tok * TSTRIDE + R + c0 + e]));
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

struct Plan {
    int mt, wn, splits, chunks_per_split, row_tiles, rows_per_cta, tile_width;
    size_t smem_bytes, partial_bytes;
};

int g_num_sms = 0;

int num_sms() {
    if (g_num_sms == 0) {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        g_num_sms = n;
    }
    return g_num_sms;
}

// Decide tile shape and K split for a problem.  `ws_bytes` < 0 means "assume any workspace".
Plan make_plan(int M, int N, int K, bool dual, long long ws_bytes) {
    Plan pl{};
    pl.mt = (M + 7) / 8;
    const int S = dual ? 2 : (pl.mt >= 3 ? 2 : 1);
    const int rw = dual ? 16 : S * 16;
    const int target = 2 * num_sms();
    const int nchunks = K / kChunkK;
    // Prefer the wide CTA (8 warps) when it alone fills the GPU twice over.
    pl.wn = ((N + 8 * rw - 1) / (8 * rw) >= target) ? 8 : 4;
    pl.rows_per_cta = pl.wn * rw;
    pl.tile_width = dual ? 2 * pl.rows_per_cta : pl.rows_per_cta;
    pl.row_tiles = (N + pl.rows_per_cta - 1) / pl.rows_per_cta;
    int splits = 1;
    if (pl.row_tiles < target && pl.row_tiles <= kMaxCounters) {
        splits = (target + pl.row_tiles - 1) / pl.row_tiles;
        const int max_splits = (nchunks + 3) / 4;           // keep >= 4 chunks per split
        if (splits > max_splits) splits = max_splits;
        if (splits < 1) splits = 1;
    }
    auto partial_bytes = [&](int sp) {
        return sp > 1 ? (size_t)sp * pl.row_tiles * pl.mt * 8 * pl.tile_width * sizeof(float) : (size_t)0;
    };
    if (ws_bytes >= 0) {
        while (splits > 1 && (long long)(kCounterBytes + partial_bytes(splits)) > ws_bytes) splits--;
    }
    pl.chunks_per_split = (nchunks + splits - 1) / splits;
    pl.splits = (nchunks + pl.chunks_per_split - 1) / pl.chunks_per_split;
    pl.partial_bytes = partial_bytes(pl.splits);
    const int ks = pl.mt == 1 ? 32 : (pl.mt == 2 ? 16 : 8);
    const size_t xs = (size_t)pl.mt * 8 * (ks * kChunkK * 2 + 64);
    const size_t ts = (size_t)pl.mt * 8 * (pl.tile_width + 1) * sizeof(float);
    pl.smem_bytes = xs > ts ? xs : ts;
    return pl;
}

template <int MT, int S, int WN, bool DUAL>
int launch_one(const QmmParams& p, const Plan& pl, cudaStream_t stream) {
    auto kern = qmm_kernel<MT, S, WN, DUAL>;
    // the attribute is per device: set it on every launch (a process may drive several GPUs)
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024) != cudaSuccess)
        return check_launch();
    dim3 grid(pl.row_tiles, pl.splits, 1);
    launch_kernel(kern, dim3(grid), dim3(WN * 32), pl.smem_bytes, stream, p);
    return check_launch();
}

template <int MT>
int launch_mt(const QmmParams& p, const Plan& pl, bool dual, cudaStream_t stream) {
    constexpr int S = (MT >= 3) ? 2 : 1;
    if (dual) {
        return pl.wn == 8 ? launch_one<MT, 2, 8, true>(p, pl, stream)
                          : launch_one<MT, 2, 4, true>(p, pl, stream);
    }
    return pl.wn == 8 ? launch_one<MT, S, 8, false>(p, pl, stream)
                      : launch_one<MT, S, 4, false>(p, pl, stream);
}

int qmm_launch(const void* x, const uint32_t* wq, const void* scales, const void* biases,
               const uint32_t* wq2, const void* scales2, const void* biases2, const void* bias,
               const void* extra, void* y, int M, int N, int K, int group_size, int dtype,
               int epilogue, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    if (dtype != B200_DTYPE_F16 || group_size != 64) return B200_EUNSUPPORTED;
    if (M < 1 || M > 32 || N < 8 || (N % 8) != 0 || K < kChunkK || (K % kChunkK) != 0) return B200_EINVAL;
    if (epilogue < B200_EPI_NONE || epilogue > B200_EPI_SILU_MUL) return B200_EINVAL;
    const bool dual = epilogue == B200_EPI_SILU_MUL;
    if (!x || !wq || !scales || !biases || !y) return B200_EINVAL;
    if (dual && (!wq2 || !scales2 || !biases2 || bias)) return B200_EINVAL;
    if (epilogue == B200_EPI_RESIDUAL && !extra) return B200_EINVAL;
    if (!aligned16(x) || !aligned16(wq) || !aligned16(y) || !aligned16(bias) || !aligned16(extra) ||
        !aligned16(wq2) || !aligned16(workspace))
        return B200_EALIGN;
    const long long ws = workspace ? (long long)workspace_bytes : 0;
    Plan pl = make_plan(M, N, K, dual, ws);
    if (pl.splits > 1 && (size_t)kCounterBytes + pl.partial_bytes > workspace_bytes) return B200_EWORKSPACE;

    QmmParams p{};
    p.x = static_cast<const __half*>(x);
    p.wq[0] = wq;
    p.sc[0] = static_cast<const __half*>(scales);
    p.bi[0] = static_cast<const __half*>(biases);
    p.wq[1] = dual ? wq2 : wq;
    p.sc[1] = static_cast<const __half*>(dual ? scales2 : scales);
    p.bi[1] = static_cast<const __half*>(dual ? biases2 : biases);
    p.bias = static_cast<const __half*>(bias);
    p.extra = static_cast<const __half*>(extra);
    p.y = static_cast<__half*>(y);
    p.counter = static_cast<int*>(workspace);
    p.partial = workspace ? reinterpret_cast<float*>(static_cast<char*>(workspace) + kCounterBytes) : nullptr;
    p.M = M;
    p.N = N;
    p.K = K;
    p.chunks_per_split = pl.chunks_per_split;
    p.splits = pl.splits;
    p.epilogue = epilogue;
    switch (pl.mt) {
        case 1: return launch_mt<1>(p, pl, dual, stream);
        case 2: return launch_mt<2>(p, pl, dual, stream);
        case 3: return launch_mt<3>(p, pl, dual, stream);
        default: return launch_mt<4>(p, pl, dual, stream);
    }
}

// Scratch of the allocation-free entry point: lives in the library image, one copy per GPU that
// loads the library, held until the process exits.
constexpr size_t kStaticScratchBytes = 4u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
constexpr int kMaxDevices = 64;
void* g_static_scratch_ptr[kMaxDevices] = {};

// Device address of the static scratch on the CURRENT device.  The array's name is only a host-side
// handle; the address a kernel may use has to be asked from the runtime, once per device.
int static_scratch_address(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        g_last_cuda_error = (int)e;
        return B200_ECUDA;
    }
    if (dev < 0 || dev >= kMaxDevices) return B200_EINVAL;
    if (g_static_scratch_ptr[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            g_last_cuda_error = (int)e;
            return B200_ECUDA;
        }
        g_static_scratch_ptr[dev] = ptr;
    }
    *out = g_static_scratch_ptr[dev];
    return B200_OK;
}

}  // namespace
}  // namespace b200

extern "C" {

size_t b200_qmm_workspace_bytes(int M, int N, int K) {
    if (M < 1 || N < 8 || K < b200::kChunkK || (K % b200::kChunkK) != 0) return 0;
    if (M > 32) M = 32;
    size_t need = 0;
    for (int dual = 0; dual < 2; dual++) {
        b200::Plan pl = b200::make_plan(M, N, K, dual != 0, -1);
        size_t b = pl.splits > 1 ? b200::kCounterBytes + pl.partial_bytes : 0;
        if (b > need) need = b;
    }
    return need;
}

int b200_qmm(const void* x, const uint32_t* wq, const void* scales, const void* biases,
             const void* bias, void* y, int M, int N, int K, int group_size, int dtype,
             void* workspace, size_t workspace_bytes, void* stream) {
    if (M < 1) return B200_EINVAL;
    // Rows beyond 32 (prompt ingestion) are processed in passes of 32; each pass streams W again.
    for (int m0 = 0; m0 < M; m0 += 32) {
        const int mb = (M - m0 < 32) ? (M - m0) : 32;
        const char* xp = static_cast<const char*>(x) + (size_t)m0 * K * 2;
        char* yp = static_cast<char*>(y) + (size_t)m0 * N * 2;
        int rc = b200::qmm_launch(xp, wq, scales, biases, nullptr, nullptr, nullptr, bias, nullptr, yp,
                                  mb, N, K, group_size, dtype, B200_EPI_NONE, workspace,
                                  workspace_bytes, static_cast<cudaStream_t>(stream));
        if (rc != B200_OK) return rc;
    }
    return B200_OK;
}

int b200_qmm_fused(const void* x, const uint32_t* wq, const void* scales, const void* biases,
                   const uint32_t* wq2, const void* scales2, const void* biases2,
                   const void* bias, const void* extra, void* y, int M, int N, int K,
                   int group_size, int dtype, int epilogue,
                   void* workspace, size_t workspace_bytes, void* stream) {
    return b200::qmm_launch(x, wq, scales, biases, wq2, scales2, biases2, bias, extra, y, M, N, K,
                            group_size, dtype, epilogue, workspace, workspace_bytes,
                            static_cast<cudaStream_t>(stream));
}

size_t b200_qmm_noalloc_max_scratch_bytes(void) { return b200::kStaticScratchBytes; }

int b200_qmm_noalloc(const void* x, const uint32_t* wq, const void* scales, const void* biases,
                     const void* bias, void* y, int M, int N, int K, int group_size, int dtype, void* stream) {
    if (M < 1 || M > 32) return B200_EINVAL;
    // The problem must fit the fixed scratch with the split it would normally use; no silent downgrade.
    // (Only the plain epilogue runs here, so only its plan counts, not the gate/up pair's.)
    if (N < 8 || K < b200::kChunkK || (K % b200::kChunkK) != 0) return B200_EINVAL;
    const b200::Plan plain = b200::make_plan(M, N, K, false, -1);
    const size_t need = plain.splits > 1 ? b200::kCounterBytes + plain.partial_bytes : 0;
    if (need > b200::kStaticScratchBytes) return B200_ELIMIT;
    void* scratch = nullptr;
    int rc = b200::static_scratch_address(&scratch);
    if (rc != B200_OK) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the previous call left; the tile counters at its head must start at zero.
    cudaError_t e = cudaMemsetAsync(scratch, 0, b200::kCounterBytes, st);
    if (e != cudaSuccess) {
        b200::g_last_cuda_error = (int)e;
        return B200_ECUDA;
    }
    return b200::qmm_launch(x, wq, scales, biases, nullptr, nullptr, nullptr, bias, nullptr, y, M, N, K,
                            group_size, dtype, B200_EPI_NONE, scratch, b200::kStaticScratchBytes, st);
}

}  // extern "C"
