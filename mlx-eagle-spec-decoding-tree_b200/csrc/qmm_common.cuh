// Pieces shared by the two quantised-matmul kernels (row-major weights / tiled weights): problem
// description, nibble expansion, and the rounding points of the fused epilogues.
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int kChunkK = 128;          // k values one warp iteration covers
constexpr int kCounterBytes = 4096;   // head of the workspace: one int per row tile
constexpr int kMaxCounters = kCounterBytes / 4;

struct QmmParams {
    const __half* x;
    const uint32_t* wq[2];
    const __half* sc[2];
    const __half* bi[2];
    const __half* bias;
    const __half* extra;
    __half* y;
    float* partial;
    int* counter;
    int M, N, K;
    int chunks_per_split;
    int splits;
    int epilogue;
};

__device__ __forceinline__ __half2 dup_half(unsigned short bits) {
    uint32_t u = (uint32_t)bits | ((uint32_t)bits << 16);
    return u32_as_h2(u);
}

// 8 nibbles of one pack -> 4 half2 {e0,e4} {e1,e5} {e2,e6} {e3,e7}, each q*s+b rounded once.
__device__ __forceinline__ void dequant_pack(uint32_t w, __half2 s2, __half2 b2, uint32_t (&d)[4]) {
    constexpr uint32_t kMagic = 0x64006400u;  // fp16 1024.0 in both halves
    const __half2 k1024 = u32_as_h2(0x64006400u);
    const __half2 kSixteenth = u32_as_h2(0x2c002c00u);  // 1/16
    const __half2 kNeg64 = u32_as_h2(0xd400d400u);      // -64
    uint32_t w8 = w >> 8;
    __half2 q04 = __hsub2(u32_as_h2((w & 0x000f000fu) | kMagic), k1024);
    __half2 q15 = __hfma2(u32_as_h2((w & 0x00f000f0u) | kMagic), kSixteenth, kNeg64);
    __half2 q26 = __hsub2(u32_as_h2((w8 & 0x000f000fu) | kMagic), k1024);
    __half2 q37 = __hfma2(u32_as_h2((w8 & 0x00f000f0u) | kMagic), kSixteenth, kNeg64);
    d[0] = h2_as_u32(__hfma2(q04, s2, b2));
    d[1] = h2_as_u32(__hfma2(q15, s2, b2));
    d[2] = h2_as_u32(__hfma2(q26, s2, b2));
    d[3] = h2_as_u32(__hfma2(q37, s2, b2));
}

// Same result, bit for bit, for scales whose fp16 exponent field lies in 1..10 (2^-14 <= |s| < 2^-4; the caller
// checks this once per matrix when the weights are re-laid-out).  A nibble moved to bits 4..7 of a half IS the
// fp16 subnormal q * 2^-20, so q * s + b is one HFMA2 with s20 = s * 2^20 (exact: the product of the two is q * s,
// rounded once together with b), and s20 is the bits of s plus 20 in the exponent field.  7 integer ops + 4 HFMA2
// per pack instead of 5 + 8: on this GPU a half2 arithmetic instruction occupies its scheduler for two cycles, so
// the fp16 ops are what bounds the expansion.
__device__ __forceinline__ void dequant_pack_fast(uint32_t w, __half2 s20, __half2 b2, uint32_t (&d)[4]) {
    constexpr uint32_t kNib = 0x00f000f0u;
    d[0] = h2_as_u32(__hfma2(u32_as_h2((w << 4) & kNib), s20, b2));
    d[1] = h2_as_u32(__hfma2(u32_as_h2(w & kNib), s20, b2));
    d[2] = h2_as_u32(__hfma2(u32_as_h2((w >> 4) & kNib), s20, b2));
    d[3] = h2_as_u32(__hfma2(u32_as_h2((w >> 8) & kNib), s20, b2));
}
__device__ __forceinline__ __half2 scale_times_2_20(__half2 s2) { return u32_as_h2(h2_as_u32(s2) + 0x50005000u); }

__device__ __forceinline__ uint32_t comp(const uint4& v, int j) {
    return j == 0 ? v.x : (j == 1 ? v.y : (j == 2 ? v.z : v.w));
}

__device__ __forceinline__ float silu_mul_f16(float gate, float up) {
    // Rounding points of the unfused reference graph (mlx_llama.py:215): every op result is fp16.
    __half g = __float2half_rn(gate);
    __half u = __float2half_rn(up);
    float gf = __half2float(g);
    __half sig = __float2half_rn(1.0f / (1.0f + expf(-gf)));
    __half t = __hmul(g, sig);
    return __half2float(__hmul(t, u));
}


}  // namespace b200
