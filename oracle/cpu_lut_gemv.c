/*
 * CPU restatement of the reference's bit-serial LUT GEMV for HLQ weights.
 *
 * TEST INFRASTRUCTURE ONLY: this file is the checker and the timed CPU baseline.
 * Nothing in the shipped library links or calls it.
 *
 * The reference's runtime (ELUTQ, directory C++/) is written with ARM NEON
 * intrinsics throughout and does not compile on x86-64, so this file restates
 * the same algorithm, in the same order of fp16 operations, with x86 AVX2 + F16C:
 *
 *   worker:      C++/ops/src/arm/arm_gemm.cpp:248-308
 *   N split:     C++/ops/src/arm/arm_gemm.cpp:312-360
 *   GEMM loop:   C++/ops/src/arm/arm_gemm.cpp:362-387
 *   LUT build:   C++/ops/src/arm/arm_t_mac_kernal.cpp:95-138
 *   plane pass:  C++/ops/src/arm/arm_t_mac_kernal.cpp:364-469
 *   re-layout:   C++/ops/src/arm/arm_t_mac_kernal.cpp:472-552
 *
 * Every arithmetic result is rounded to fp16 before it is used again, as the
 * reference's float16 vectors do; products and sums are rounded separately.
 * The table lookup uses a byte shuffle on the split low/high bytes of the
 * 16 fp16 table entries, the x86 counterpart of the reference's vqtbl1q_u8 use.
 *
 * Parity pin: checked in tests against the NumPy restatement of the same
 * operation order and against float64 products of weights dequantized by the
 * reference's own Python code (fixtures under tests/golden/).
 */
#include <immintrin.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <omp.h>

typedef uint16_t f16;

static inline float h2f(f16 h) { return _cvtsh_ss(h); }
static inline f16 f2h(float f) { return _cvtss_sh(f, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC); }
static inline f16 h_add(f16 a, f16 b) { return f2h(h2f(a) + h2f(b)); }

/* round 8 floats to fp16 precision and widen again */
static inline __m256 round16(__m256 v) {
    return _mm256_cvtph_ps(_mm256_cvtps_ph(v, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
}

/* 16 partial sums per 4 activations; entry e adds x[b] for every set bit b of e,
 * in the order b = 0,1,2,3 (arm_t_mac_kernal.cpp:107-123).  32 bytes per chunk. */
static void build_lut(int k, const f16 *x, f16 *lut) {
    for (int i = 0; i < k; i += 4) {
        f16 *t = lut + (i / 4) * 16;
        for (int e = 0; e < 16; ++e) {
            f16 acc = 0;
            for (int b = 0; b < 4; ++b)
                if (e >> b & 1) acc = h_add(acc, x[i + b]);
            t[e] = acc;
        }
    }
}

/* One bit-plane over n rows (n % 32 == 0) of a re-laid-out chunk
 * (arm_t_mac_kernal.cpp:390-467).  weight: [n/32][k/8][32] bytes;
 * scale: [n/32][k/g][32] fp16; lut_lo/lut_hi: per 4-activation chunk the low and
 * high bytes of its 16 entries (the de-interleaved copy of :379-384). */
static void plane_pass(f16 *out, const uint8_t *weight, int k, int n, const uint8_t *lut_lo,
                       const uint8_t *lut_hi, const f16 *scale, int g) {
    const __m256i nib = _mm256_set1_epi8(0x0f);
    for (int i = 0; i < n; i += 32) {
        __m256 c0 = _mm256_setzero_ps(), c1 = c0, c2 = c0, c3 = c0;
        for (int j = 0; j < k; j += g) {
            __m256 a0 = _mm256_setzero_ps(), a1 = a0, a2 = a0, a3 = a0;
            for (int l = 0; l < g; l += 8) {
                const uint8_t *wp = weight + ((size_t)i * k) / 8 + (size_t)(j + l) * 4;
                __m256i w = _mm256_loadu_si256((const __m256i *)wp);
                __m256i bot = _mm256_and_si256(w, nib);
                __m256i top = _mm256_and_si256(_mm256_srli_epi16(w, 4), nib);
                int c = (j + l) / 4;
                for (int half = 0; half < 2; ++half) {
                    __m256i idx = half ? top : bot;
                    __m256i tl = _mm256_broadcastsi128_si256(
                        _mm_loadu_si128((const __m128i *)(lut_lo + (size_t)(c + half) * 16)));
                    __m256i th = _mm256_broadcastsi128_si256(
                        _mm_loadu_si128((const __m128i *)(lut_hi + (size_t)(c + half) * 16)));
                    __m256i vl = _mm256_shuffle_epi8(tl, idx);
                    __m256i vh = _mm256_shuffle_epi8(th, idx);
                    __m256i r_a = _mm256_unpacklo_epi8(vl, vh); /* rows 0-7 | 16-23 */
                    __m256i r_b = _mm256_unpackhi_epi8(vl, vh); /* rows 8-15 | 24-31 */
                    a0 = round16(_mm256_add_ps(a0, _mm256_cvtph_ps(_mm256_castsi256_si128(r_a))));
                    a1 = round16(_mm256_add_ps(a1, _mm256_cvtph_ps(_mm256_castsi256_si128(r_b))));
                    a2 = round16(_mm256_add_ps(a2, _mm256_cvtph_ps(_mm256_extracti128_si256(r_a, 1))));
                    a3 = round16(_mm256_add_ps(a3, _mm256_cvtph_ps(_mm256_extracti128_si256(r_b, 1))));
                }
            }
            const f16 *sp = scale + ((size_t)i * k) / g + (size_t)32 * (j / g);
            __m256 s0 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *)(sp + 0)));
            __m256 s1 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *)(sp + 8)));
            __m256 s2 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *)(sp + 16)));
            __m256 s3 = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *)(sp + 24)));
            __m256 p0 = round16(_mm256_mul_ps(a0, s0)), p1 = round16(_mm256_mul_ps(a1, s1));
            __m256 p2 = round16(_mm256_mul_ps(a2, s2)), p3 = round16(_mm256_mul_ps(a3, s3));
            if (j == 0) {
                c0 = p0; c1 = p1; c2 = p2; c3 = p3;
            } else {
                c0 = round16(_mm256_add_ps(c0, p0));
                c1 = round16(_mm256_add_ps(c1, p1));
                c2 = round16(_mm256_add_ps(c2, p2));
                c3 = round16(_mm256_add_ps(c3, p3));
            }
        }
        __m256 cs[4] = {c0, c1, c2, c3};
        for (int v = 0; v < 4; ++v) {
            __m128i *op = (__m128i *)(out + i + 8 * v);
            __m256 cur = _mm256_cvtph_ps(_mm_loadu_si128(op));
            _mm_storeu_si128(op, _mm256_cvtps_ph(_mm256_add_ps(cur, cs[v]),
                                                 _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
        }
    }
}

/* The work of one thread on its slice of output rows (arm_gemm.cpp:248-308). */
static void worker(int k, int n, const f16 *x, const uint8_t *weight, const f16 *scale,
                   const f16 *zero, const f16 *bias, f16 *out, int g, int bits, f16 *xsum,
                   f16 *lut, uint8_t *lut_lo, uint8_t *lut_hi) {
    int ng = k / g;
    for (int gi = 0; gi < ng; ++gi) {
        f16 acc = 0;
        for (int j = 0; j < g; ++j) acc = h_add(acc, x[gi * g + j]);
        xsum[gi] = acc;
    }
    for (int i = 0; i < n; i += 32) {
        __m256 o[4] = {_mm256_setzero_ps(), _mm256_setzero_ps(), _mm256_setzero_ps(),
                       _mm256_setzero_ps()};
        for (int gi = 0; gi < ng; ++gi) {
            __m256 xs = _mm256_set1_ps(h2f(xsum[gi]));
            const f16 *zp = zero + ((size_t)i * k) / g + (size_t)32 * gi;
            for (int v = 0; v < 4; ++v) {
                __m256 zv = _mm256_cvtph_ps(_mm_loadu_si128((const __m128i *)(zp + 8 * v)));
                o[v] = round16(_mm256_add_ps(o[v], round16(_mm256_mul_ps(xs, zv))));
            }
        }
        for (int v = 0; v < 4; ++v)
            _mm_storeu_si128((__m128i *)(out + i + 8 * v),
                             _mm256_cvtps_ph(o[v], _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
    }
    build_lut(k, x, lut);
    for (int c = 0; c < k / 4; ++c)
        for (int e = 0; e < 16; ++e) {
            lut_lo[c * 16 + e] = (uint8_t)(lut[c * 16 + e] & 0xff);
            lut_hi[c * 16 + e] = (uint8_t)(lut[c * 16 + e] >> 8);
        }
    for (int p = 0; p < bits; ++p)
        plane_pass(out, weight + (size_t)p * k * n / 8, k, n, lut_lo, lut_hi,
                   scale + (size_t)p * k * n / g, g);
    if (bias)
        for (int j = 0; j < n; ++j) out[j] = h_add(out[j], bias[j]);
}

/* bytes of scratch one call needs: per thread group sums, table and split table */
size_t hlq_cpu_workspace_bytes(int k, int g, int threads) {
    size_t per = (size_t)(k / g) * 2 + (size_t)k * 8 + (size_t)k * 8 + 256;
    return per * (size_t)threads;
}

/*
 * y[m, n] = x[m, k] . W_hat^T + bias over buffers already re-laid-out for `threads`
 * thread chunks.  Rows are split into ceil(n/threads) per thread with the pointer
 * offsets of arm_gemm.cpp:336-349; m > 1 repeats the GEMV per row of x
 * (arm_gemm.cpp:380-385).  Returns 0, or -1 when a chunk is not a multiple of 32 rows.
 */
int hlq_cpu_gemm(int m, int k, int n, const f16 *x, f16 *y, const uint8_t *weight,
                 const f16 *scale, const f16 *zero, const f16 *bias, int g, int bits,
                 int threads, void *workspace) {
    int chunk = (n + threads - 1) / threads;
    if (chunk % 32 || n % 32 || k % g || g % 8) return -1;
    size_t per = hlq_cpu_workspace_bytes(k, g, 1);
    for (int row = 0; row < m; ++row) {
#pragma omp parallel for num_threads(threads) schedule(static, 1)
        for (int t = 0; t < threads; ++t) {
            int start = chunk * t;
            int end = start + chunk < n ? start + chunk : n;
            if (end <= start) continue;
            uint8_t *ws = (uint8_t *)workspace + per * (size_t)t;
            f16 *xsum = (f16 *)ws;
            f16 *lut = (f16 *)(ws + (((size_t)(k / g) * 2 + 63) & ~(size_t)63));
            uint8_t *lut_lo = (uint8_t *)lut + (size_t)k * 8;
            uint8_t *lut_hi = lut_lo + (size_t)k * 4;
            worker(k, end - start, x + (size_t)row * k,
                   weight + (size_t)bits * start * k / 8,
                   scale + (size_t)bits * start * k / g, zero + (size_t)start * k / g,
                   bias ? bias + start : NULL, y + (size_t)row * n + start, g, bits, xsum, lut,
                   lut_lo, lut_hi);
        }
    }
    return 0;
}

/*
 * Export layout -> the runtime layout above (arm_t_mac_kernal.cpp:472-552):
 * bits [q][N][K/8] -> [thread][q][rows/32][K/8][32]; scales [q][N][G] ->
 * [thread][q][rows/32][G][32]; zeros [N][G] -> [N/32][G][32].
 */
int hlq_cpu_relayout(int n, int k, int g, int bits, int threads, const uint8_t *w_quant,
                     const f16 *w_scale, const f16 *w_zero, uint8_t *out_quant, f16 *out_scale,
                     f16 *out_zero) {
    int chunk = (n + threads - 1) / threads;
    int kb = k / 8, ng = k / g;
    if (chunk % 32 || n % 32) return -1;
    size_t iq = 0, is = 0, iz = 0;
    for (int t = 0; t < threads; ++t) {
        int start = t * chunk, end = start + chunk < n ? start + chunk : n;
        for (int p = 0; p < bits; ++p) {
            const uint8_t *wp = w_quant + (size_t)p * n * kb;
            const f16 *sp = w_scale + (size_t)p * n * ng;
            for (int i = start; i < end; i += 32) {
                for (int j = 0; j < kb; ++j)
                    for (int r = 0; r < 32; ++r) out_quant[iq++] = wp[(size_t)(i + r) * kb + j];
            }
            for (int i = start; i < end; i += 32) {
                for (int j = 0; j < ng; ++j)
                    for (int r = 0; r < 32; ++r) out_scale[is++] = sp[(size_t)(i + r) * ng + j];
            }
        }
    }
    for (int i = 0; i < n; i += 32)
        for (int j = 0; j < ng; ++j)
            for (int r = 0; r < 32; ++r) out_zero[iz++] = w_zero[(size_t)(i + r) * ng + j];
    return (iq == (size_t)bits * n * kb && is == (size_t)bits * n * ng) ? 0 : -2;
}

int hlq_cpu_max_threads(void) { return omp_get_max_threads(); }
