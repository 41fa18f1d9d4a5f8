// Tree-masked attention of <= 32 query tokens against the KV cache (one layer), GQA aware.
//
// Visible keys of query m: every committed cache row (< prefix), plus tail row j (cache row
// prefix + j, j < tail <= 64) iff bit j of mask[m] is set.  That one rule covers the verify pass
// (ancestor mask), the draft tree levels (one ancestor per earlier level + self), the 8-token
// catch-up pass and prompt ingestion (causal masks).  The reference builds the same thing as an
// additive 0/-inf matrix (mlx_eagle.py:143-146,171,336-338) for mx.fast.scaled_dot_product_attention
// (mlx_llama.py:185-192).
//
// Work split: grid (key blocks of 64, kv heads).  A CTA loads its K/V block once into shared
// memory and serves all query heads of the group (M*G query rows, tiles of 16 rows per warp) with
// mma.sync m16n8k16: S = Q K^T (fp32), masked softmax statistics in fp32, P rounded to fp16,
// O = P V (fp32).  Partial (max, sum, O) go to a workspace; a second small kernel (one warp per
// token and query head) merges the key blocks in block order and writes fp16.  Key blocks past the current length exit at once, so
// one launch shape serves a growing cache (CUDA-graph friendly: the length is read on the device).
#include "common.cuh"

namespace b200 {
namespace {

constexpr int kKeyBlock = 64;
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
    uint32_t addr = (uint32_t)__cvta_generic_to_shared(smem_ptr);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

struct AttnParams {
    const __half* q;       // rotated queries inside the qkv activation buffer
    int q_stride;          // halves between consecutive tokens
    const __half* kcache;  // [Hkv][cap][HD]
    const __half* vcache;
    const unsigned long long* mask;   // [M]
    const int* prefix;
    __half* out;           // [M][Hq*HD]
    float* part_o;         // [Hkv][nkb][QRP][HD]
    float* part_ml;        // [Hkv][nkb][QRP][2]
    int* counter;          // [Hkv]
    int M, Hq, Hkv, cap, tail, nkb, qrp;
    float scale_log2;      // head_dim^-0.5 * log2(e)
};

template <int HD>
__global__ void __launch_bounds__(128) tree_attention_kernel(const AttnParams p) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int KS = HD + 8;                       // padded smem row (halves)
    __shared__ __align__(16) __half sk[kKeyBlock * KS];
    __shared__ __align__(16) __half sv[kKeyBlock * KS];
    const int kb = blockIdx.x;
    const int hk = blockIdx.y;
    const int prefix = p.prefix[0];
    const int total = prefix + p.tail;
    const int key0 = kb * kKeyBlock;
    if (key0 >= total) return;
    const int G = p.Hq / p.Hkv;
    const int QR = p.M * G;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t = lane & 3;

    // K/V block -> shared memory (rows past the end are zero)
    {
        const __half* kbase = p.kcache + ((size_t)hk * p.cap + key0) * HD;
        const __half* vbase = p.vcache + ((size_t)hk * p.cap + key0) * HD;
        constexpr int VPR = HD / 8;                 // 16-byte vectors per row
        for (int i = threadIdx.x; i < kKeyBlock * VPR; i += 128) {
            const int r = i / VPR, c = i - r * VPR;
            uint4 kv = make_uint4(0, 0, 0, 0), vv = make_uint4(0, 0, 0, 0);
            if (key0 + r < total) {
                kv = *reinterpret_cast<const uint4*>(kbase + (size_t)r * HD + c * 8);
                vv = *reinterpret_cast<const uint4*>(vbase + (size_t)r * HD + c * 8);
            }
            *reinterpret_cast<uint4*>(sk + r * KS + c * 8) = kv;
            *reinterpret_cast<uint4*>(sv + r * KS + c * 8) = vv;
        }
    }
    __syncthreads();

    const int ntiles = (QR + 15) / 16;
    float* po = p.part_o + ((size_t)hk * p.nkb + kb) * p.qrp * HD;
    float* pml = p.part_ml + ((size_t)hk * p.nkb + kb) * p.qrp * 2;

    for (int rt = warp; rt < ntiles; rt += 4) {
        const int r0 = rt * 16 + g, r1 = r0 + 8;
        const bool v0 = r0 < QR, v1 = r1 < QR;
        const int m0 = v0 ? r0 / G : 0, m1 = v1 ? r1 / G : 0;
        const __half* q0 = p.q + (size_t)m0 * p.q_stride + (size_t)(hk * G + (v0 ? r0 - m0 * G : 0)) * HD;
        const __half* q1 = p.q + (size_t)m1 * p.q_stride + (size_t)(hk * G + (v1 ? r1 - m1 * G : 0)) * HD;
        const unsigned long long mk0 = v0 ? p.mask[m0] : 0ull, mk1 = v1 ? p.mask[m1] : 0ull;

        uint32_t qa[HD / 16][4];
#pragma unroll
        for (int ks = 0; ks < HD / 16; ks++) {
            qa[ks][0] = *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * t);
            qa[ks][1] = *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * t);
            qa[ks][2] = *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * t + 8);
            qa[ks][3] = *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * t + 8);
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

        // scale, mask, block-local softmax statistics (base-2 domain)
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
            // the sum uses the rounded probabilities so that numerator and denominator agree
            l0 += __low2float(h0) + __high2float(h0);
            l1 += __low2float(h1) + __high2float(h1);
            pa[nt][0] = h2_as_u32(h0);
            pa[nt][1] = h2_as_u32(h1);
        }
        l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
        l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);

        // O = P V
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

// Merge of the key blocks: one warp per (token, query head) row.  Lanes first share the per-block
// (max, sum) pairs to get the softmax weights of the blocks, then add the partial outputs in block
// order and write fp16.
template <int HD>
__global__ void __launch_bounds__(128) tree_attention_merge_kernel(const AttnParams p) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int row_global = blockIdx.x * 4 + (threadIdx.x >> 5);       // m * Hq + head
    if (row_global >= p.M * p.Hq) return;
    const int G = p.Hq / p.Hkv;
    const int m = row_global / p.Hq, head = row_global - m * p.Hq;
    const int hk = head / G, gq = head - hk * G;
    const int r = m * G + gq;
    const int total = p.prefix[0] + p.tail;
    const int nact = (total + kKeyBlock - 1) / kKeyBlock;
    const float* ho = p.part_o + (size_t)hk * p.nkb * p.qrp * HD;
    const float* hml = p.part_ml + (size_t)hk * p.nkb * p.qrp * 2;
    constexpr int CPT = HD / 32;
    float mstar = -INFINITY;
    for (int b = lane; b < nact; b += 32) mstar = fmaxf(mstar, __ldcg(hml + ((size_t)b * p.qrp + r) * 2));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mstar = fmaxf(mstar, __shfl_xor_sync(0xffffffffu, mstar, o));
    float denom = 0.f;
    float acc[CPT];
#pragma unroll
    for (int c = 0; c < CPT; c++) acc[c] = 0.f;
    for (int b0 = 0; b0 < nact; b0 += 32) {
        const int b = b0 + lane;
        float wl = 0.f, ll = 0.f;
        if (b < nact) {
            const float mb = __ldcg(hml + ((size_t)b * p.qrp + r) * 2);
            ll = __ldcg(hml + ((size_t)b * p.qrp + r) * 2 + 1);
            wl = (mb == -INFINITY) ? 0.f : exp2f(mb - mstar);
        }
        const int cnt = min(32, nact - b0);
        for (int i = 0; i < cnt; i++) {
            const float w = __shfl_sync(0xffffffffu, wl, i);
            denom += __shfl_sync(0xffffffffu, ll, i) * w;
            const float* src = ho + ((size_t)(b0 + i) * p.qrp + r) * HD + lane;
#pragma unroll
            for (int c = 0; c < CPT; c++) acc[c] += w * __ldcg(src + 32 * c);
        }
    }
    const float inv = denom > 0.f ? 1.f / denom : 0.f;
    __half* orow = p.out + (size_t)m * p.Hq * HD + (size_t)head * HD;
#pragma unroll
    for (int c = 0; c < CPT; c++) orow[lane + 32 * c] = __float2half_rn(acc[c] * inv);
}

}  // namespace
}  // namespace b200

extern "C" {

// Scratch needed for a launch whose cache may hold up to max_kv rows (committed + tail).
size_t b200_tree_attention_workspace_bytes(int M, int Hq, int Hkv, int hd, int max_kv) {
    if (M < 1 || Hq < 1 || Hkv < 1 || Hq % Hkv || max_kv < 1) return 0;
    const int G = Hq / Hkv;
    const size_t qrp = (size_t)((M * G + 15) / 16) * 16;
    const size_t nkb = (size_t)(max_kv + b200::kKeyBlock - 1) / b200::kKeyBlock;
    return 256 + (size_t)Hkv * nkb * qrp * ((size_t)hd + 2) * sizeof(float);
}

int b200_tree_attention(const void* q, int q_stride, const void* kcache, const void* vcache,
                        const unsigned long long* mask, const int* prefix, int tail, void* out,
                        int M, int Hq, int Hkv, int hd, int cache_rows, int max_kv, float scale,
                        void* workspace, size_t workspace_bytes, void* stream) {
    if (!q || !kcache || !vcache || !mask || !prefix || !out || !workspace) return B200_EINVAL;
    if (M < 1 || M > 32 || Hq < 1 || Hkv < 1 || Hq % Hkv || Hkv > 64 || tail < 1 || tail > 64 ||
        max_kv < tail || max_kv > cache_rows || (q_stride % 8) != 0)
        return B200_EINVAL;
    if (hd != 64 && hd != 128) return B200_EUNSUPPORTED;
    if (!b200::aligned16(q) || !b200::aligned16(kcache) || !b200::aligned16(vcache) || !b200::aligned16(workspace))
        return B200_EALIGN;
    if (workspace_bytes < b200_tree_attention_workspace_bytes(M, Hq, Hkv, hd, max_kv)) return B200_EWORKSPACE;
    b200::AttnParams p{};
    const int G = Hq / Hkv;
    p.q = static_cast<const __half*>(q);
    p.q_stride = q_stride;
    p.kcache = static_cast<const __half*>(kcache);
    p.vcache = static_cast<const __half*>(vcache);
    p.mask = mask;
    p.prefix = prefix;
    p.out = static_cast<__half*>(out);
    p.M = M; p.Hq = Hq; p.Hkv = Hkv; p.cap = cache_rows; p.tail = tail;
    p.nkb = (max_kv + b200::kKeyBlock - 1) / b200::kKeyBlock;
    p.qrp = ((M * G + 15) / 16) * 16;
    p.counter = static_cast<int*>(workspace);
    p.part_ml = reinterpret_cast<float*>(static_cast<char*>(workspace) + 256);
    p.part_o = p.part_ml + (size_t)Hkv * p.nkb * p.qrp * 2;
    p.scale_log2 = scale * b200::kLog2e;
    dim3 grid(p.nkb, Hkv);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int merge_blocks = (M * Hq + 3) / 4;
    if (hd == 128) {
    b200::launch_kernel(b200::tree_attention_kernel<128>, dim3(grid), dim3(128), 0, st, p);
    b200::launch_kernel(b200::tree_attention_merge_kernel<128>, dim3(merge_blocks), dim3(128), 0, st, p);
    } else {
    b200::launch_kernel(b200::tree_attention_kernel<64>, dim3(grid), dim3(128), 0, st, p);
    b200::launch_kernel(b200::tree_attention_merge_kernel<64>, dim3(merge_blocks), dim3(128), 0, st, p);
    }
    return b200::check_launch();
}

}  // extern "C"
