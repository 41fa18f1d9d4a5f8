// 4-bit affine quantised matmul for <= 128 token rows on the fifth-generation tensor cores (tcgen05, TMEM).
//
//   y[M][N] = x[M][K] . dequant(W)[N][K]^T     (+ bias), fp16 in, fp32 accumulate, fp16 out
//
// W is in the streaming layout of b200_qmm_relayout (records of 16 rows x 128 k, 1152 bytes, ordered
// [64-row block][k chunk][4 records]).  One CTA owns items of 128 weight rows (the M of one tcgen05.mma):
//
//   producer warp    bulk-copies, per k chunk, the two 4608-byte record runs of the item and the chunk's
//                    activations into a ring of packed stages (one lane per copy);
//   16 dequant warps in two groups of 8 that take the chunks in turn.  Thread = weight row: a row's 16 packs
//                    of a chunk are 64 contiguous bytes of its record; the thread expands its half of them
//                    (exact q*s+b, rounded once to fp16, like every other kernel of this library) and writes
//                    the fp16 pairs with tcgen05.st into its own lane of a 128-lane x 64-column tile in tensor
//                    memory (lane = weight row, column = two k values): the A operand never touches shared
//                    memory;
//   MMA warp         one thread issues 8 tcgen05.mma (128 x N x 16, N = 16 .. 128 tokens; A from tensor memory,
//                    B = the chunk's activations, read in place from the packed stage) per chunk into a TMEM
//                    accumulator and commits to the mbarriers that free the tile, free the packed stage (together
//                    with the eight warps that read its packs) and publish the accumulator;
//   epilogue         the dequant warps read the accumulator (tcgen05.ld, one weight row per thread) and store fp16.
//
// The activations come in the tensor cores' canonical K-major layout without swizzle ([chunk][token group of 8]
// [k group of 8][8 tokens][8 halves]: a core matrix is 8 rows x 16 bytes; k groups 160 bytes apart, token rows
// padded with zeros to 16, 32, 64 or 128), written by a small relayout kernel into the caller's workspace.
// Tensor memory: all 512 columns of the SM (4 tiles of 64 columns, then 2 accumulators of up to 128).
// Every wait is bounded; a wait that gives up sets the error word in the workspace and the CTA runs to its end
// (TMEM is always freed).  No copy uses cluster multicast.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "b200_eagle.h"
#include "common.cuh"
#include "pipeline.cuh"
#include "qmm_common.cuh"

namespace b200 {
namespace {

constexpr int kRecBytes = 1152;
constexpr int kRunBytes = 4 * kRecBytes;        // the four records of a 64-row block for one chunk
constexpr int kItemRows = 128;
constexpr int kGroupWarps = 8;                   // warps that expand one chunk together (one 16-row record each)
constexpr int kDeqWarps = 2 * kGroupWarps;       // two such groups take the chunks in turn
constexpr int kUThreads = (kDeqWarps + 2) * 32;  // + producer warp + MMA warp
// Core matrices (8 rows x 16 bytes = 128 bytes) of the activation tile are spaced 160 bytes apart along K (any
// multiple of 16 is allowed): stores of one row's neighbouring k groups then fall into different banks.
constexpr int kLBO = 160;                        // bytes between core matrices along K
constexpr int kSBO = (kChunkK / 8) * kLBO;       // bytes between 8-row groups of a 128-k tile
constexpr int kAStages = 4;                      // dequantised weight tiles in tensor memory
constexpr int kAColumns = kChunkK / 2;           // 64 columns of 32 bits: 128 fp16 k values per weight row
constexpr int kAccColumn = kAStages * kAColumns; // the two accumulators follow the tiles
// (the CTA allocates all 512 columns of the SM's tensor memory: 4 x 64 for tiles, 2 x 32 for accumulators)
constexpr uint32_t kUmmaWaitPolls = 1u << 24;    // x <= 32 ns each (short suspensions: the handshakes are on the critical path)

template <int NT>                                // token columns of the MMA: 16 or 32
struct UGeo {
    static constexpr int XBYTES = (NT / 8) * kSBO;                   // activations of one chunk, same layout
    static constexpr int PSTAGE = 2 * kRunBytes + XBYTES;            // packed stage: two record runs + the chunk's activations
    static constexpr int NP = NT <= 32 ? 8 : (NT == 64 ? 6 : 4);      // packed stages (the MMAs read the activations in place)
    static constexpr int NTS = NT <= 64 ? kAStages : 2;              // tile stages (tensor-memory tiles)
    static constexpr int ACC = NT < 32 ? 32 : NT;                    // columns of one accumulator
    static constexpr int BAR_OFF = NP * PSTAGE;
    static constexpr int SMEM = BAR_OFF + 256 + 1024;                // + barriers, + alignment slack
};

struct UParams {
    const unsigned char* w;     // streaming layout
    const __half* xc;           // activations, canonical layout [chunk][NT/8 token groups][16 k groups, 160 bytes apart][8][8]
    const __half* bias;
    __half* y;                  // [M][N]
    int* err;
    int M, N, K;
};

__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    // shared-memory matrix descriptor, no swizzle: start >> 4 | LBO >> 4 at bit 16 | SBO >> 4 at bit 32 | version 1 at bit 46
    return (uint64_t)((saddr & 0x3ffffu) >> 4) | ((uint64_t)(kLBO >> 4) << 16) | ((uint64_t)(kSBO >> 4) << 32) |
           ((uint64_t)1 << 46);
}

__device__ __forceinline__ bool uwait(uint32_t bar, uint32_t parity) {
    return mbar_wait_timed(bar, parity, kUmmaWaitPolls, 32u);
}

__global__ void x_canonical_kernel(const __half* __restrict__ x, __half* __restrict__ xc, int M, int K, int NT) {
    pdl_wait();
    pdl_launch_dependents();
    // one 16-byte unit (token, k group of 8) per thread
    const int units = NT * (K / 8);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < units; i += gridDim.x * blockDim.x) {
        const int tok = i / (K / 8), kg_all = i - tok * (K / 8);
        const int c = kg_all >> 4, kg = kg_all & 15;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (tok < M) v = *reinterpret_cast<const uint4*>(x + (size_t)tok * K + kg_all * 8);
        *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(xc) + ((size_t)c * (NT / 8) + tok / 8) * kSBO + kg * kLBO +
                                  (tok & 7) * 16) = v;
    }
}

template <int NT>
__global__ void __launch_bounds__(kUThreads, 1) qmm_umma_kernel(const __grid_constant__ UParams p) {
    using G = UGeo<NT>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* packed = smem;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + G::BAR_OFF);
    uint64_t* pfull = bars;                          // packed stage landed            (producer -> dequant warps)
    uint64_t* pempty = pfull + G::NP;        // packed stage read              (8 dequant warps -> producer)
    uint64_t* tready = pempty + G::NP;       // tile written                   (8 dequant warps -> MMA warp)
    uint64_t* tfree = tready + G::NTS;          // tile's MMAs complete           (tcgen05.commit -> dequant warps)
    uint64_t* accfull = tfree + G::NTS;         // item's accumulator complete    (tcgen05.commit -> epilogue)
    uint64_t* accempty = accfull + 2;                // accumulator read               (8 warps -> MMA warp)
    __shared__ uint32_t s_tmem;
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nchunks = p.K / kChunkK;
    const int nitems = p.N / kItemRows;
    const size_t block_stride = (size_t)nchunks * kRunBytes;        // bytes of one 64-row block

    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int s = 0; s < G::NP; s++) {
            mbar_init(smem_u32(pfull + s), 1);
            mbar_init(smem_u32(pempty + s), kGroupWarps + 1);   // the eight warps that read the packs + the MMAs that read the activations
        }
        for (int s = 0; s < G::NTS; s++) {
            mbar_init(smem_u32(tready + s), kGroupWarps);
            mbar_init(smem_u32(tfree + s), 1);
        }
        for (int s = 0; s < 2; s++) {
            mbar_init(smem_u32(accfull + s), 1);
            mbar_init(smem_u32(accempty + s), kDeqWarps);
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == kDeqWarps + 1) {                     // the MMA warp owns the tensor memory: 64 columns = two accumulators
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;\n" ::"r"(smem_u32(&s_tmem)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = s_tmem;
    volatile int* abort_flag = &s_abort;
    pdl_wait();
    pdl_launch_dependents();

    if (warp == kDeqWarps) {
        // ------------------------------------------------------------------ producer
        const uint64_t pol = make_evict_first_policy();
        uint32_t n = 0;
        for (int item = blockIdx.x; item < nitems; item += gridDim.x) {
            const unsigned char* w0 = p.w + (size_t)(2 * item) * block_stride;
            for (int c = 0; c < nchunks; c++, n++) {
                const uint32_t s = n % G::NP, use = n / G::NP;
                if (*abort_flag) break;
                if (use > 0 && !__all_sync(0xffffffffu, uwait(smem_u32(pempty + s), (use - 1) & 1u))) {
                    if (lane == 0) { *abort_flag = 1; atomicCAS(p.err, 0, 1); }
                    break;
                }
                // one lane per copy (a bulk copy costs ~150 cycles to issue from a single lane, whatever its size)
                const uint32_t bar = smem_u32(pfull + s);
                const uint32_t dst = smem_u32(packed + s * G::PSTAGE);
                if (lane == 0) mbar_expect_tx(bar, G::PSTAGE);
                __syncwarp();
                if (lane < 2)
                    bulk_copy_g2s_hint(dst + lane * kRunBytes, w0 + lane * block_stride + (size_t)c * kRunBytes, kRunBytes, bar, pol);
                else if (lane == 2)
                    bulk_copy_g2s(dst + 2 * kRunBytes, reinterpret_cast<const unsigned char*>(p.xc) + (size_t)c * G::XBYTES,
                                  G::XBYTES, bar);
                __syncwarp();
            }
        }
    } else if (warp == kDeqWarps + 1) {
        // ------------------------------------------------------------------ MMA issuer (one thread)
        if (lane == 0) {
            const uint32_t idesc = (1u << 4) | ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(kItemRows >> 4) << 24);
            uint32_t n = 0, it = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < nitems && ok; item += gridDim.x, it++) {
                const uint32_t ab = it & 1u;
                if (it >= 2) ok = uwait(smem_u32(accempty + ab), ((it >> 1) - 1) & 1u);     // epilogue of item it-2 done
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                for (int c = 0; c < nchunks && ok; c++, n++) {
                    const uint32_t ts = n % G::NTS, use = n / G::NTS;
                    ok = !*abort_flag && uwait(smem_u32(tready + ts), use & 1u);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t a0 = tmem + ts * kAColumns;        // the tile: lane = weight row, column = two k values
                    const uint32_t ps = n % G::NP;                    // the chunk's packed stage still holds its activations
                    ok = uwait(smem_u32(pfull + ps), (n / G::NP) & 1u);   // (observed here too: the MMAs read what the copy wrote)
                    if (!ok) break;
                    const uint32_t b0 = smem_u32(packed + ps * G::PSTAGE + 2 * kRunBytes);
#pragma unroll
                    for (int ks = 0; ks < kChunkK / 16; ks++) {
                        const uint64_t db = umma_desc(b0 + ks * 2 * kLBO);
                        const uint32_t accumulate = (c > 0 || ks > 0) ? 1u : 0u;
                        asm volatile(
                            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                            "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(tmem + kAccColumn + ab * G::ACC),
                            "r"(a0 + ks * 8), "l"(db), "r"(idesc), "r"(accumulate)
                            : "memory");
                    }
                    // the tile and the stage's activations may be rewritten once these MMAs have read them
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(
                                     smem_u32(tfree + ts))
                                 : "memory");
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(
                                     smem_u32(pempty + ps))
                                 : "memory");
                }
                if (ok)
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(
                                     smem_u32(accfull + ab))
                                 : "memory");
            }
            if (!ok && !*abort_flag) { *abort_flag = 1; atomicCAS(p.err, 0, 2); }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------------ dequant warps + epilogue
        const uint32_t grp = warp / kGroupWarps;     // this warp's group takes the chunks with n % 2 == grp
        const int wl = warp % kGroupWarps;
        uint32_t n = 0, it = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < nitems && ok; item += gridDim.x, it++) {
            for (int c = 0; c < nchunks && ok; c++, n++) {
                if ((n & 1u) != grp) continue;
                const uint32_t ps = n % G::NP, ts = n % G::NTS, tuse = n / G::NTS;
                ok = !*abort_flag && uwait(smem_u32(pfull + ps), (n / G::NP) & 1u);
                if (ok && tuse > 0) ok = uwait(smem_u32(tfree + ts), (tuse - 1) & 1u);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                const unsigned char* stage = packed + ps * G::PSTAGE;
                // Thread = weight row 32 * (wl % 4) + lane of the item (the tensor-memory lane this warp may write);
                // warps 0-3 of the group take the k groups 4j+0, 4j+1, warps 4-7 the k groups 4j+2, 4j+3.  A row's 16
                // packs are 64 contiguous bytes of its record: pack j of k group 4j+t at byte 16 t + 4 j.
                const int q = wl & 3, kh = wl >> 2;
                const int tile_i = 2 * q + (lane >> 4), r = lane & 15;
                const unsigned char* rec = stage + (tile_i >> 2) * kRunBytes + (tile_i & 3) * kRecBytes;
                const unsigned char* rowp = rec + (r >> 3) * 512 + (r & 7) * 64 + kh * 32;
                const uint4 u0 = *reinterpret_cast<const uint4*>(rowp);
                const uint4 u1 = *reinterpret_cast<const uint4*>(rowp + 16);
                const uint2 sb = *reinterpret_cast<const uint2*>(rec + 1024 + r * 8);
                const uint32_t trow = tmem + ts * kAColumns + ((uint32_t)(q * 32) << 16);
#pragma unroll
                for (int tt = 0; tt < 2; tt++) {
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const __half2 sbj = u32_as_h2((j < 2) ? sb.x : sb.y);      // {scale, bias} of the k group of 64
                        uint32_t d[4];
                        dequant_pack(comp(tt == 0 ? u0 : u1, j), __low2half2(sbj), __high2half2(sbj), d);
                        // k group 4 j + t = columns 16 j + 4 t .. + 3 (two k values per column)
                        asm volatile("tcgen05.st.sync.aligned.32x32b.x4.b32 [%0], {%1,%2,%3,%4};\n" ::"r"(
                                         trow + 16 * j + 4 * (2 * kh + tt)),
                                     "r"(d[0]), "r"(d[1]), "r"(d[2]), "r"(d[3])
                                     : "memory");
                    }
                }
                asm volatile("tcgen05.wait::st.sync.aligned;\n" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(smem_u32(pempty + ps));
                    mbar_arrive(smem_u32(tready + ts));
                }
            }
            if (!ok) break;
            // ---- epilogue: thread = weight row 32 * (warp % 4) + lane of the item, a quarter of the token columns
            const uint32_t ab = it & 1u;
            ok = __all_sync(0xffffffffu, !*abort_flag && uwait(smem_u32(accfull + ab), (it >> 1) & 1u));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            constexpr int CH = NT / 4;                // columns per warp: 4 .. 32
            const int col0 = (warp >> 2) * CH;
            const uint32_t taddr = tmem + kAccColumn + ab * G::ACC + col0 + ((uint32_t)((warp & 3) * 32) << 16);
            uint32_t r[CH];
#pragma unroll
            for (int c4 = 0; c4 < CH; c4 += 4)        // four columns per load
                asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];\n"
                             : "=r"(r[c4]), "=r"(r[c4 + 1]), "=r"(r[c4 + 2]), "=r"(r[c4 + 3])
                             : "r"(taddr + c4)
                             : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(accempty + ab));
            const int row = item * kItemRows + (warp & 3) * 32 + lane;
            const __half bv = p.bias != nullptr ? p.bias[row] : __ushort_as_half(0);
#pragma unroll
            for (int i = 0; i < CH; i++) {
                const int tok = col0 + i;
                if (tok < p.M) {
                    __half o = __float2half_rn(__uint_as_float(r[i]));
                    if (p.bias != nullptr) o = __hadd(o, bv);
                    p.y[(size_t)tok * p.N + row] = o;
                }
            }
        }
        if (!ok && lane == 0 && !*abort_flag) { *abort_flag = 1; atomicCAS(p.err, 0, 3); }
    }

    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == kDeqWarps + 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;\n" ::"r"(tmem) : "memory");
}

template <int NT>
int launch_umma(const UParams& p, cudaStream_t stream) {
    auto kern = qmm_umma_kernel<NT>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, UGeo<NT>::SMEM) != cudaSuccess)
        return check_launch();
    int dev = 0, sms = 148;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int nitems = p.N / kItemRows;
    launch_kernel(kern, dim3(nitems < sms ? nitems : sms), dim3(kUThreads), (size_t)UGeo<NT>::SMEM, stream, p);
    return check_launch();
}

}  // namespace
}  // namespace b200

extern "C" {

using namespace b200;

size_t b200_qmm_umma_workspace_bytes(int M, int K) {
    if (M < 1 || M > 128 || K < kChunkK || (K % kChunkK) != 0) return 0;
    const int nt = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
    return 256 + (size_t)(K / kChunkK) * (nt / 8) * kSBO;
}

int b200_qmm_umma(const void* x, const void* w_tiled, const void* bias, void* y, int M, int N, int K, void* workspace,
                  size_t workspace_bytes, void* stream) {
    if (!x || !w_tiled || !y || !workspace || M < 1 || M > 128 || N < kItemRows || K < kChunkK) return B200_EINVAL;
    if ((N % kItemRows) != 0 || (K % kChunkK) != 0) return B200_EUNSUPPORTED;
    if (!aligned16(x) || !aligned16(w_tiled) || !aligned16(y) || !aligned16(workspace)) return B200_EALIGN;
    if (workspace_bytes < b200_qmm_umma_workspace_bytes(M, K)) return B200_EWORKSPACE;
    const int nt = M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    __half* xc = reinterpret_cast<__half*>(static_cast<char*>(workspace) + 256);
    const int units = nt * (K / 8);
    launch_kernel(x_canonical_kernel, dim3((units + 255) / 256), dim3(256), 0, st, static_cast<const __half*>(x), xc, M, K, nt);
    if (check_launch() != B200_OK) return B200_ECUDA;
    UParams p{};
    p.w = static_cast<const unsigned char*>(w_tiled);
    p.xc = xc;
    p.bias = static_cast<const __half*>(bias);
    p.y = static_cast<__half*>(y);
    p.err = static_cast<int*>(workspace);
    p.M = M; p.N = N; p.K = K;
    switch (nt) {
        case 16: return launch_umma<16>(p, st);
        case 32: return launch_umma<32>(p, st);
        case 64: return launch_umma<64>(p, st);
        default: return launch_umma<128>(p, st);
    }
}

}  // extern "C"
