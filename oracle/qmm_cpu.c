/*
 * CPU restatement (plain C + OpenMP) of the reference's batched 4-bit affine
 * quantised matmul, used as the checker for the CUDA path and as the timed
 * CPU baseline.  TEST INFRASTRUCTURE: the shipped library never links this.
 *
 * Follows kernels/progression/simd_no_swizzle_cast.metal:
 *   :82,96,110,124  element j of a uint32 pack sits in bits 4j..4j+3
 *   :63-64,76-77    one fp16 scale / bias per 64 consecutive k of a row
 *   :83             dequantisation in half precision, half(q)*s + b
 *   :66-68,93       fp16 x fp16 products accumulated in fp32
 *   :236-241        result cast to fp16, stored as result[batch_row][n]
 * and mlx_model_fwd_bench.py:69-71 (linear bias added after the kernel, in
 * fp16).  The dequantised weight is the exact value q*s+b rounded once to
 * fp16.  Summation order: 16 interleaved fp32 partial sums over k, then the
 * partial sums added lane 0..15 (the shader's own order is a different
 * permutation of K; only fp32 rounding differs).
 *
 * MLX itself (mx.quantized_matmul) cannot be run here, so parity with MLX is
 * unpinned; see oracle/__init__.py.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define VW 16
#define MB 8

static float g_h2f[65536];
static int g_h2f_ready = 0;

static float half_bits_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h >> 15) << 31;
    uint32_t exp = (h >> 10) & 0x1f;
    uint32_t man = h & 0x3ff;
    float out;
    if (exp == 0) {
        out = ldexpf((float)man, -24);
        if (sign) out = -out;
        return out;
    }
    if (exp == 31) {
        uint32_t bits = sign | 0x7f800000u | (man << 13);
        memcpy(&out, &bits, 4);
        return out;
    }
    uint32_t bits = sign | ((exp + 112) << 23) | (man << 13);
    memcpy(&out, &bits, 4);
    return out;
}

static void init_tables(void) {
    if (g_h2f_ready) return;
    for (int i = 0; i < 65536; i++) g_h2f[i] = half_bits_to_float((uint16_t)i);
    g_h2f_ready = 1;
}

/* Round a double to the nearest fp16 (ties to even), returned as its bit pattern.  Integer
 * arithmetic on the double's bits: the 53-bit significand is shifted down to 11 bits (fewer for
 * fp16 subnormals) and rounded on the discarded part. */
uint16_t oracle_f64_to_f16(double d) {
    uint64_t bits;
    memcpy(&bits, &d, 8);
    uint16_t sign = (uint16_t)((bits >> 48) & 0x8000u);
    int bexp = (int)((bits >> 52) & 0x7ff);
    uint64_t frac = bits & 0xfffffffffffffULL;
    if (bexp == 0x7ff) return frac ? 0x7e00 : (uint16_t)(sign | 0x7c00);
    if (bexp == 0) return sign;                       /* double zero / subnormal: far below fp16 range */
    int e = bexp - 1023;
    if (e >= 16) return sign | 0x7c00;
    uint64_t mant = frac | (1ULL << 52);
    int shift = 42;                                   /* keep 11 significant bits */
    int hexp = e + 15;                                /* biased fp16 exponent */
    if (e < -14) {                                    /* fp16 subnormal: fewer bits survive */
        shift += -14 - e;
        hexp = 0;
        if (shift > 54) return sign;                  /* below half of the smallest subnormal */
    }
    uint64_t q = mant >> shift;
    uint64_t rem = mant & ((1ULL << shift) - 1);
    uint64_t half = 1ULL << (shift - 1);
    if (rem > half || (rem == half && (q & 1))) q++;
    uint32_t out = (hexp > 0) ? (uint32_t)(((uint32_t)hexp << 10) + (uint32_t)(q - 1024)) : (uint32_t)q;
    if (out >= 0x7c00) out = 0x7c00;
    return sign | (uint16_t)out;
}

float oracle_f16_to_f32(uint16_t h) {
    init_tables();
    return g_h2f[h];
}

/* Dequantise one weight row into fp16-rounded floats. */
static void dequant_row(const uint32_t* wq_row, const uint16_t* s_row, const uint16_t* b_row,
                        int K, int group_size, float* out) {
    float lut[16];
    for (int g = 0; g < K / group_size; g++) {
        double s = (double)g_h2f[s_row[g]];
        double b = (double)g_h2f[b_row[g]];
        for (int q = 0; q < 16; q++) lut[q] = g_h2f[oracle_f64_to_f16((double)q * s + b)];
        const uint32_t* packs = wq_row + g * (group_size / 8);
        float* o = out + g * group_size;
        for (int p = 0; p < group_size / 8; p++) {
            uint32_t w = packs[p];
            for (int j = 0; j < 8; j++) o[p * 8 + j] = lut[(w >> (4 * j)) & 0xf];
        }
    }
}

__attribute__((target_clones("avx512f", "avx2", "default")))
static void row_dots(const float* xf, const float* wrow, int M, int K, float* out) {
    for (int m0 = 0; m0 < M; m0 += MB) {
        int mb = (M - m0 < MB) ? (M - m0) : MB;
        float acc[MB][VW];
        memset(acc, 0, sizeof(acc));
        for (int k = 0; k < K; k += VW) {
            for (int m = 0; m < mb; m++) {
                const float* xr = xf + (size_t)(m0 + m) * K + k;
                for (int v = 0; v < VW; v++) acc[m][v] += xr[v] * wrow[k + v];
            }
        }
        for (int m = 0; m < mb; m++) {
            float s = 0.f;
            for (int v = 0; v < VW; v++) s += acc[m][v];
            out[m0 + m] = s;
        }
    }
}

/*
 * y[M,N] (fp16 bits) = x[M,K] (fp16 bits) . dequant(W[N,K])^T ; optional fp16 bias[N] added after
 * the fp16 rounding of the product.  K must be a multiple of 16 and of group_size.
 * nthreads <= 0 uses the OpenMP default.  Returns 0, or -1 on a bad shape.
 */
int oracle_qmm_f16(const uint16_t* x, const uint32_t* wq, const uint16_t* scales,
                   const uint16_t* biases, const uint16_t* bias, uint16_t* y,
                   int M, int N, int K, int group_size, int nthreads) {
    if (M <= 0 || N <= 0 || K <= 0 || group_size <= 0 || K % group_size || K % VW || group_size % 8)
        return -1;
    init_tables();
    float* xf = (float*)malloc((size_t)M * K * sizeof(float));
    if (!xf) return -2;
    for (size_t i = 0; i < (size_t)M * K; i++) xf[i] = g_h2f[x[i]];
    int groups = K / group_size;
#ifdef _OPENMP
    if (nthreads > 0) omp_set_num_threads(nthreads);
#endif
#pragma omp parallel
    {
        float* wrow = (float*)malloc((size_t)K * sizeof(float));
        float* out = (float*)malloc((size_t)M * sizeof(float));
#pragma omp for schedule(static)
        for (int n = 0; n < N; n++) {
            dequant_row(wq + (size_t)n * (K / 8), scales + (size_t)n * groups,
                        biases + (size_t)n * groups, K, group_size, wrow);
            row_dots(xf, wrow, M, K, out);
            for (int m = 0; m < M; m++) {
                uint16_t h = oracle_f64_to_f16((double)out[m]);
                if (bias) h = oracle_f64_to_f16((double)g_h2f[h] + (double)g_h2f[bias[n]]);
                y[(size_t)m * N + n] = h;
            }
        }
        free(wrow);
        free(out);
    }
    free(xf);
    return 0;
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Thread count of later calls, whatever OMP_NUM_THREADS said at start-up (launchers such as
 * torch.distributed.run set it to 1 for every rank). */
void oracle_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}
