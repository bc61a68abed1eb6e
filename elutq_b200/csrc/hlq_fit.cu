// Fit of the HLQ parameters of one group of weights (q plane scales and one offset) by
// alternating between the assignment of every weight to the nearest of the 2^q values
// sum_j s_j b_j + c and a least-squares solve for (s, c) under that assignment.
//
// Replaces the reference quantizer's
//   find_optimal_params_alternating        GPTQ/quant.py:118-153
//   optimize_s_batch_with_constant         GPTQ/quant.py:104-116   (batched (q+1) x (q+1) normal equations, pinv)
//   generate_augmented_bit_combinations    GPTQ/quant.py:95-102    (value i has bit j = (i >> j) & 1, then the constant)
// One warp owns one group: its weights stay in shared memory for all iterations, the sums of
// the normal equations (counts of bit pairs, sums of the weights per bit) are warp reductions,
// and every lane solves the same small symmetric system in double precision through its
// eigen-decomposition (Jacobi), inverting only eigenvalues above max(q+1) * eps_f32 * largest as
// torch.linalg.pinv does for float32, so that a bit-plane no weight uses gets scale 0.
#include <cuda_runtime.h>
#include <math.h>

#include "hlq_internal.h"

namespace hlq {
namespace {

constexpr int kFitWarps = 4;
constexpr int kFitMaxG = 1024;

// pinv(A) * r for a symmetric positive semi-definite A of order n <= 5, in place: x = result
template <int N>
__device__ void solve_pinv(double (&A)[N][N], const double (&r)[N], double (&x)[N], double rtol) {
    double V[N][N];
#pragma unroll
    for (int i = 0; i < N; ++i)
#pragma unroll
        for (int j = 0; j < N; ++j) V[i][j] = i == j ? 1.0 : 0.0;
    for (int sweep = 0; sweep < 12; ++sweep) {
        double off = 0.0;
#pragma unroll
        for (int p = 0; p < N; ++p)
#pragma unroll
            for (int q = p + 1; q < N; ++q) off += A[p][q] * A[p][q];
        if (off < 1e-26) break;
#pragma unroll
        for (int p = 0; p < N; ++p) {
#pragma unroll
            for (int q = p + 1; q < N; ++q) {
                const double apq = A[p][q];
                if (fabs(apq) < 1e-300) continue;
                const double theta = (A[q][q] - A[p][p]) / (2.0 * apq);
                const double t = (theta >= 0 ? 1.0 : -1.0) / (fabs(theta) + sqrt(theta * theta + 1.0));
                const double c = 1.0 / sqrt(t * t + 1.0), s = t * c;
#pragma unroll
                for (int k = 0; k < N; ++k) {          // A <- A J
                    const double akp = A[k][p], akq = A[k][q];
                    A[k][p] = c * akp - s * akq;
                    A[k][q] = s * akp + c * akq;
                }
#pragma unroll
                for (int k = 0; k < N; ++k) {          // A <- J^T A
                    const double apk = A[p][k], aqk = A[q][k];
                    A[p][k] = c * apk - s * aqk;
                    A[q][k] = s * apk + c * aqk;
                }
#pragma unroll
                for (int k = 0; k < N; ++k) {
                    const double vkp = V[k][p], vkq = V[k][q];
                    V[k][p] = c * vkp - s * vkq;
                    V[k][q] = s * vkp + c * vkq;
                }
            }
        }
    }
    double lmax = 0.0;
#pragma unroll
    for (int i = 0; i < N; ++i) lmax = fmax(lmax, fabs(A[i][i]));
#pragma unroll
    for (int i = 0; i < N; ++i) x[i] = 0.0;
#pragma unroll
    for (int e = 0; e < N; ++e) {
        const double lam = A[e][e];
        if (fabs(lam) <= rtol * lmax) continue;
        double proj = 0.0;
#pragma unroll
        for (int k = 0; k < N; ++k) proj += V[k][e] * r[k];
        proj /= lam;
#pragma unroll
        for (int k = 0; k < N; ++k) x[k] += V[k][e] * proj;
    }
}

template <int Q>
__global__ void __launch_bounds__(kFitWarps * 32) fit_alternating_kernel(const float *__restrict__ w,
                                                                         float *__restrict__ scales,
                                                                         float *__restrict__ zeros, int64_t blocks,
                                                                         int g, int iters) {
    __shared__ float ys[kFitWarps][kFitMaxG];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t b = (int64_t)blockIdx.x * kFitWarps + warp;
    if (b >= blocks) return;
    float *y = ys[warp];
    float lo = INFINITY, hi = -INFINITY;
    for (int e = lane; e < g; e += 32) {
        const float v = w[b * g + e];
        y[e] = v;
        lo = fminf(lo, v);
        hi = fmaxf(hi, v);
    }
#pragma unroll
    for (int d = 16; d; d >>= 1) {
        lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, d));
        hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, d));
    }
    __syncwarp();
    // start: plane j gets range / (2^q - 1) * 2^j, the constant the minimum (quant.py:128-134)
    float s[Q + 1];
    const float step = (hi - lo) / (float)((1 << Q) - 1);
#pragma unroll
    for (int j = 0; j < Q; ++j) s[j] = step * (float)(1 << j);
    s[Q] = lo;
    for (int it = 0; it < iters; ++it) {
        float comb[1 << Q];
#pragma unroll
        for (int v = 0; v < (1 << Q); ++v) {
            float t = 0.f;
#pragma unroll
            for (int j = 0; j < Q; ++j)
                if ((v >> j) & 1) t += s[j];
            comb[v] = t + s[Q];
        }
        // sums of the normal equations over this lane's weights
        constexpr int NP = Q * (Q + 1) / 2;      // pairs i <= j < Q
        float cnt[NP], sy[Q + 1];
#pragma unroll
        for (int i = 0; i < NP; ++i) cnt[i] = 0.f;
#pragma unroll
        for (int i = 0; i <= Q; ++i) sy[i] = 0.f;
        for (int e = lane; e < g; e += 32) {
            const float v = y[e];
            float best = INFINITY;
            int arg = 0;
#pragma unroll
            for (int c = 0; c < (1 << Q); ++c) {
                const float dist = fabsf(v - comb[c]);
                if (dist < best) {               // first minimum, as torch.argmin
                    best = dist;
                    arg = c;
                }
            }
            int idx = 0;
#pragma unroll
            for (int i = 0; i < Q; ++i) {
#pragma unroll
                for (int j = i; j < Q; ++j) {
                    if (((arg >> i) & 1) && ((arg >> j) & 1)) cnt[idx] += 1.f;
                    ++idx;
                }
                if ((arg >> i) & 1) sy[i] += v;
            }
            sy[Q] += v;
        }
#pragma unroll
        for (int d = 16; d; d >>= 1) {
#pragma unroll
            for (int i = 0; i < NP; ++i) cnt[i] += __shfl_xor_sync(0xffffffffu, cnt[i], d);
#pragma unroll
            for (int i = 0; i <= Q; ++i) sy[i] += __shfl_xor_sync(0xffffffffu, sy[i], d);
        }
        double A[Q + 1][Q + 1], r[Q + 1], x[Q + 1];
        int idx = 0;
#pragma unroll
        for (int i = 0; i < Q; ++i) {
#pragma unroll
            for (int j = i; j < Q; ++j) {
                A[i][j] = A[j][i] = (double)cnt[idx];
                ++idx;
            }
        }
        idx = 0;
#pragma unroll
        for (int i = 0; i < Q; ++i) {
            A[i][Q] = A[Q][i] = (double)cnt[idx];      // sum of b_i = count of (i, i)
            idx += Q - i;
            r[i] = (double)sy[i];
        }
        A[Q][Q] = (double)g;
        r[Q] = (double)sy[Q];
        solve_pinv<Q + 1>(A, r, x, (double)(Q + 1) * 1.1920928955078125e-7);
#pragma unroll
        for (int i = 0; i <= Q; ++i) s[i] = (float)x[i];
    }
    if (lane == 0) {
#pragma unroll
        for (int j = 0; j < Q; ++j) scales[b * Q + j] = s[j];
        zeros[b] = s[Q];
    }
}

}  // namespace
}  // namespace hlq

using namespace hlq;

extern "C" int hlq_fit_alternating_device(const float *d_w, float *d_scales, float *d_zeros, int64_t blocks, int g,
                                          int q, int iters, void *stream) {
    if (blocks < 0 || g <= 0 || iters < 0) return HLQ_ERR_INVALID_ARGUMENT;
    if (q < 1 || q > 4) return HLQ_ERR_SHAPE;
    if (g > kFitMaxG) return HLQ_ERR_UNSUPPORTED;
    if (blocks == 0) return HLQ_OK;
    if (!d_w || !d_scales || !d_zeros) return HLQ_ERR_INVALID_ARGUMENT;
    const unsigned grid = (unsigned)((blocks + kFitWarps - 1) / kFitWarps);
    cudaStream_t st = (cudaStream_t)stream;
    switch (q) {
        case 1: fit_alternating_kernel<1><<<grid, kFitWarps * 32, 0, st>>>(d_w, d_scales, d_zeros, blocks, g, iters); break;
        case 2: fit_alternating_kernel<2><<<grid, kFitWarps * 32, 0, st>>>(d_w, d_scales, d_zeros, blocks, g, iters); break;
        case 3: fit_alternating_kernel<3><<<grid, kFitWarps * 32, 0, st>>>(d_w, d_scales, d_zeros, blocks, g, iters); break;
        default: fit_alternating_kernel<4><<<grid, kFitWarps * 32, 0, st>>>(d_w, d_scales, d_zeros, blocks, g, iters); break;
    }
    count_launch();
    return note_cuda(cudaGetLastError());
}
