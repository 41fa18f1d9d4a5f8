// Small per-token kernels of one decoder layer: quantised embedding gather, RMSNorm, and
// tree-position RoPE fused with the KV-cache append.  All are tiny (<= 32 tokens), HBM/launch
// bound; they exist so that a whole forward pass stays on the device with no host decisions.
#include "common.cuh"

namespace b200 {
namespace {

// ---- embedding: h[m,:] = dequant(E[tokens[m], :]) --------------------------------------------
// One thread per uint32 pack (8 weights).  Same dequantisation as the matmul (q*s+b rounded once).
__global__ void embed_gather_kernel(const int* __restrict__ tokens, const uint32_t* __restrict__ wq,
                                    const __half* __restrict__ scales, const __half* __restrict__ biases,
                                    __half* __restrict__ out, int M, int H, int V) {
    pdl_wait();
    pdl_launch_dependents();
    const int m = blockIdx.y;
    const int pack = blockIdx.x * blockDim.x + threadIdx.x;
    if (pack >= H / 8) return;
    int tok = tokens[m];
    tok = min(max(tok, 0), V - 1);
    const uint32_t w = wq[(size_t)tok * (H / 8) + pack];
    const int grp = pack >> 3;
    const __half s = scales[(size_t)tok * (H / 64) + grp];
    const __half b = biases[(size_t)tok * (H / 64) + grp];
    __align__(16) __half o[8];
#pragma unroll
    for (int j = 0; j < 8; j++) o[j] = __hfma(__int2half_rn((int)((w >> (4 * j)) & 0xfu)), s, b);
    *reinterpret_cast<uint4*>(out + (size_t)m * H + pack * 8) = *reinterpret_cast<const uint4*>(o);
}

// ---- RMSNorm: y = fp16( (x * rsqrt(mean(x^2) + eps)) * w ), fp32 math --------------------------
// One CTA per output row; `row_index` (optional, device) selects the source row of output row 0.
__global__ void rms_norm_kernel(const __half* __restrict__ x, const __half* __restrict__ w,
                                __half* __restrict__ y, const int* __restrict__ row_index, int H, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float red[32];
    const int out_row = blockIdx.x;
    const int src_row = row_index ? (row_index[0] + out_row) : out_row;
    const __half2* xr = reinterpret_cast<const __half2*>(x + (size_t)src_row * H);
    float ss = 0.f;
    for (int i = threadIdx.x; i < H / 2; i += blockDim.x) {
        float2 v = __half22float2(xr[i]);
        ss += v.x * v.x + v.y * v.y;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (threadIdx.x == 0) red[0] = v;
    }
    __syncthreads();
    const float inv = rsqrtf(red[0] / (float)H + eps);
    const __half2* wr = reinterpret_cast<const __half2*>(w);
    __half2* yr = reinterpret_cast<__half2*>(y + (size_t)out_row * H);
    for (int i = threadIdx.x; i < H / 2; i += blockDim.x) {
        float2 v = __half22float2(xr[i]);
        float2 g = __half22float2(wr[i]);
        yr[i] = __floats2half2_rn((v.x * inv) * g.x, (v.y * inv) * g.y);
    }
}

// ---- RoPE at per-token positions + KV append ----------------------------------------------------
// qkv: [M, (Hq + 2*Hkv) * hd] (q heads, then k heads, then v heads), already biased.
// q is rotated in place; k is rotated and stored, v stored, at cache row  prefix + write_off + m.
// Rotation (non-traditional / half-split layout), fp32 math:
//   theta = (scaling * inv_freq[i]) * pos ;  (x[i], x[i+hd/2]) -> (x1 cos - x2 sin, x1 sin + x2 cos)
__global__ void rope_kv_append_kernel(__half* __restrict__ qkv, const int* __restrict__ pos,
                                      const float* __restrict__ inv_freq, float scaling,
                                      __half* __restrict__ kcache, __half* __restrict__ vcache,
                                      const int* __restrict__ prefix, int write_off, int Hq, int Hkv,
                                      int hd, int cap) {
    pdl_wait();
    pdl_launch_dependents();
    const int m = blockIdx.y;
    const int head = blockIdx.x;              // 0..Hq-1 q, Hq..Hq+Hkv-1 k, then v
    const int i = threadIdx.x;                // 0..hd/2-1
    const int row = prefix[0] + write_off + m;
    __half* src = qkv + (size_t)m * (Hq + 2 * Hkv) * hd + (size_t)head * hd;
    if (head >= Hq + Hkv) {                   // v: plain copy
        if (row < cap) {
            __half* dst = vcache + ((size_t)(head - Hq - Hkv) * cap + row) * hd;
            dst[i] = src[i];
            dst[i + hd / 2] = src[i + hd / 2];
        }
        return;
    }
    const float L = scaling * inv_freq[i];
    const float theta = L * (float)pos[m];
    float s, c;
    sincosf(theta, &s, &c);
    const float x1 = __half2float(src[i]);
    const float x2 = __half2float(src[i + hd / 2]);
    const __half r1 = __float2half_rn(x1 * c - x2 * s);
    const __half r2 = __float2half_rn(x1 * s + x2 * c);
    if (head < Hq) {
        src[i] = r1;
        src[i + hd / 2] = r2;
    } else if (row < cap) {
        __half* dst = kcache + ((size_t)(head - Hq) * cap + row) * hd;
        dst[i] = r1;
        dst[i + hd / 2] = r2;
    }
}

// ---- tensor-parallel epilogue: h = fp16(h + fp16(sum)) where `sum` holds the all-reduced fp32 partial
// products of a row-parallel linear layer (the rounding points of the unsharded residual epilogue).
__global__ void residual_add_f32_kernel(__half* __restrict__ h, const float* __restrict__ sum, int n) {
    pdl_wait();
    pdl_launch_dependents();
    const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i >= n) return;
    const float4 s = *reinterpret_cast<const float4*>(sum + i);
    __half2* hp = reinterpret_cast<__half2*>(h + i);
    hp[0] = __hadd2(hp[0], __floats2half2_rn(s.x, s.y));
    hp[1] = __hadd2(hp[1], __floats2half2_rn(s.z, s.w));
}

// ---- element-wise halves of the fused matmul epilogues, for prompt ingestion through the large-M matmul (whose own
// epilogue is plain): the same rounding points as B200_EPI_RESIDUAL and B200_EPI_SILU_MUL.
__global__ void add_f16_kernel(__half* __restrict__ h, const __half* __restrict__ y, size_t n) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= n) return;
    uint4 a = *reinterpret_cast<const uint4*>(h + i);
    const uint4 b = *reinterpret_cast<const uint4*>(y + i);
    __half2* ah = reinterpret_cast<__half2*>(&a);
    const __half2* bh = reinterpret_cast<const __half2*>(&b);
#pragma unroll
    for (int e = 0; e < 4; e++) ah[e] = __hadd2(ah[e], bh[e]);
    *reinterpret_cast<uint4*>(h + i) = a;
}

__global__ void silu_mul_f16_kernel(const __half* __restrict__ gate, const __half* __restrict__ up, __half* __restrict__ out,
                                    size_t n) {
    pdl_wait();
    pdl_launch_dependents();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i >= n) return;
    const uint4 g4 = *reinterpret_cast<const uint4*>(gate + i);
    const uint4 u4 = *reinterpret_cast<const uint4*>(up + i);
    const __half* g = reinterpret_cast<const __half*>(&g4);
    const __half* u = reinterpret_cast<const __half*>(&u4);
    __align__(16) __half o[8];
#pragma unroll
    for (int e = 0; e < 8; e++) {                 // every op result fp16, as in the fused epilogue (mlx_llama.py:215)
        const float gf = __half2float(g[e]);
        const __half sig = __float2half_rn(1.0f / (1.0f + expf(-gf)));
        o[e] = __hmul(__hmul(g[e], sig), u[e]);
    }
    *reinterpret_cast<uint4*>(out + i) = *reinterpret_cast<const uint4*>(o);
}

// Stand-alone operator with the reference's tensor layout: in/out (B, H, L, D), offsets (B, L).
__global__ void rope_positions_kernel(const __half* __restrict__ in, const int* __restrict__ offsets,
                                      const float* __restrict__ inv_freq, float scaling,
                                      __half* __restrict__ out, int H, int Lq, int D) {
    pdl_wait();
    pdl_launch_dependents();
    const int l = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int i = threadIdx.x;
    const size_t base = (((size_t)b * H + h) * Lq + l) * D;
    const float theta = (scaling * inv_freq[i]) * (float)offsets[(size_t)b * Lq + l];
    float s, c;
    sincosf(theta, &s, &c);
    const float x1 = __half2float(in[base + i]);
    const float x2 = __half2float(in[base + i + D / 2]);
    out[base + i] = __float2half_rn(x1 * c - x2 * s);
    out[base + i + D / 2] = __float2half_rn(x1 * s + x2 * c);
}

}  // namespace
}  // namespace b200

extern "C" {

int b200_embed_gather(const int* tokens, const uint32_t* wq, const void* scales, const void* biases,
                      void* out, int M, int H, int V, void* stream) {
    if (!tokens || !wq || !scales || !biases || !out) return B200_EINVAL;
    if (M < 1 || H < 64 || (H % 64) != 0 || V < 1) return B200_EINVAL;
    if (!b200::aligned16(out)) return B200_EALIGN;
    dim3 grid((H / 8 + 127) / 128, M);
    b200::launch_kernel(b200::embed_gather_kernel, dim3(grid), dim3(128), 0, static_cast<cudaStream_t>(stream), tokens, wq, static_cast<const __half*>(scales), static_cast<const __half*>(biases),
        static_cast<__half*>(out), M, H, V);
    return b200::check_launch();
}

int b200_rms_norm(const void* x, const void* w, void* y, const int* row_index, int M, int H, float eps,
                  void* stream) {
    if (!x || !w || !y || M < 1 || H < 2 || (H % 2) != 0) return B200_EINVAL;
    b200::launch_kernel(b200::rms_norm_kernel, dim3(M), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const __half*>(x), static_cast<const __half*>(w), static_cast<__half*>(y), row_index, H, eps);
    return b200::check_launch();
}

int b200_rope_kv_append(void* qkv, const int* pos, const float* inv_freq, float scaling, void* kcache,
                        void* vcache, const int* prefix, int write_off, int M, int Hq, int Hkv, int hd,
                        int cache_rows, void* stream) {
    if (!qkv || !pos || !inv_freq || !kcache || !vcache || !prefix) return B200_EINVAL;
    if (M < 1 || Hq < 1 || Hkv < 1 || hd < 2 || (hd % 2) != 0 || hd > 2048 || write_off < 0 || cache_rows < 1)
        return B200_EINVAL;
    dim3 grid(Hq + 2 * Hkv, M);
    b200::launch_kernel(b200::rope_kv_append_kernel, dim3(grid), dim3(hd / 2), 0, static_cast<cudaStream_t>(stream), static_cast<__half*>(qkv), pos, inv_freq, scaling, static_cast<__half*>(kcache),
        static_cast<__half*>(vcache), prefix, write_off, Hq, Hkv, hd, cache_rows);
    return b200::check_launch();
}

int b200_residual_add_f32(void* h, const float* sum, int M, int N, void* stream) {
    if (!h || !sum || M < 1 || N < 4 || (N % 4) != 0) return B200_EINVAL;
    if (!b200::aligned16(h) || !b200::aligned16(sum)) return B200_EALIGN;
    const int n = M * N;
    b200::launch_kernel(b200::residual_add_f32_kernel, dim3((n / 4 + 255) / 256), dim3(256), 0,
                        static_cast<cudaStream_t>(stream), static_cast<__half*>(h), sum, n);
    return b200::check_launch();
}

int b200_add_f16(void* h, const void* y, size_t n, void* stream) {
    if (!h || !y || n < 8 || (n % 8) != 0) return B200_EINVAL;
    if (!b200::aligned16(h) || !b200::aligned16(y)) return B200_EALIGN;
    b200::launch_kernel(b200::add_f16_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                        static_cast<__half*>(h), static_cast<const __half*>(y), n);
    return b200::check_launch();
}

int b200_silu_mul_f16(const void* gate, const void* up, void* out, size_t n, void* stream) {
    if (!gate || !up || !out || n < 8 || (n % 8) != 0) return B200_EINVAL;
    if (!b200::aligned16(gate) || !b200::aligned16(up) || !b200::aligned16(out)) return B200_EALIGN;
    b200::launch_kernel(b200::silu_mul_f16_kernel, dim3((unsigned)((n / 8 + 255) / 256)), dim3(256), 0,
                        static_cast<cudaStream_t>(stream), static_cast<const __half*>(gate), static_cast<const __half*>(up),
                        static_cast<__half*>(out), n);
    return b200::check_launch();
}

int b200_rope_positions(const void* in, const int* offsets, const float* inv_freqs, float scaling_factor,
                        void* out, int B, int H, int L, int D, void* stream) {
    if (!in || !offsets || !inv_freqs || !out) return B200_EINVAL;
    if (B < 1 || H < 1 || L < 1 || D < 2 || (D % 2) != 0 || D > 2048 || H > 65535 || B > 65535) return B200_EINVAL;
    dim3 grid(L, H, B);
    b200::launch_kernel(b200::rope_positions_kernel, dim3(grid), dim3(D / 2), 0, static_cast<cudaStream_t>(stream), static_cast<const __half*>(in), offsets, inv_freqs, scaling_factor, static_cast<__half*>(out), H, L, D);
    return b200::check_launch();
}

}  // extern "C"
