/*
 * CPU restatement (C + OpenMP) of the MLX affine INT4 projection path.
 * TEST INFRASTRUCTURE ONLY: used by the tests as a second checker and by the benchmark
 * as the timed CPU baseline ("port").  Nothing in the shipped library links it.
 *
 * The reference project's ground truth for this path is MLX's CPU quantized_matmul,
 * a third-party dependency absent from the reference tree (mlx>=0.31,
 * pyproject.toml:24-30).  PARITY UNPINNED against MLX's internal accumulation order;
 * pinned against the packed layout and formulas in the reference's own sources:
 *   - word / element / group indexing and w = scale*q + bias, fp32 accumulation:
 *     kernels/affine_qmv.py:25-53
 *   - residual added to the un-rounded sum: kernels/affine_qmv.py:124-131
 *   - SwiGLU on un-rounded sums g/(1+exp(-g))*u: kernels/affine_qmv.py:204-208
 *   - MLP = down(swiglu(x)) + residual with bf16 hidden:
 *     metile/backends/mlx_quantized.py:1798,1829-1830
 *   - add + RMSNorm: kernels/add_rmsnorm.py:7-25
 *
 * bf16 values are passed as uint16_t bit patterns.  Accumulation is fp32 in ascending k.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static inline float bf16_to_f32(uint16_t v) {
    uint32_t bits = (uint32_t)v << 16;
    float out;
    memcpy(&out, &bits, 4);
    return out;
}

static inline uint16_t f32_to_bf16(float v) {
    uint32_t bits;
    memcpy(&bits, &v, 4);
    if ((bits & 0x7F800000u) == 0x7F800000u && (bits & 0x007FFFFFu)) return (uint16_t)((bits >> 16) | 0x40);
    bits += 0x7FFFu + ((bits >> 16) & 1u);
    return (uint16_t)(bits >> 16);
}

/* Sets the OpenMP thread count (launchers such as torchrun export OMP_NUM_THREADS=1). */
void oracle_set_threads(int threads) {
#ifdef _OPENMP
    if (threads > 0) omp_set_num_threads(threads);
#else
    (void)threads;
#endif
}

int oracle_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* acc[m] = sum_k x[m,k] * (s*q + b) for one output row n; xf is fp32 [M,K]. */
static void row_dot(const float* xf, const uint32_t* wrow, const uint16_t* srow, const uint16_t* brow,
                    int M, int K, float* acc) {
    for (int m = 0; m < M; ++m) acc[m] = 0.0f;
    const int groups = K / 64;
    for (int g = 0; g < groups; ++g) {
        const float scale = bf16_to_f32(srow[g]);
        const float bias = bf16_to_f32(brow[g]);
        float wf[64];
        for (int j = 0; j < 8; ++j) {
            const uint32_t packed = wrow[g * 8 + j];
            for (int e = 0; e < 8; ++e) wf[j * 8 + e] = (float)((packed >> (4 * e)) & 15u) * scale + bias;
        }
        for (int m = 0; m < M; ++m) {
            const float* xr = xf + (size_t)m * K + g * 64;
            float sum = acc[m];
            for (int k = 0; k < 64; ++k) sum += xr[k] * wf[k];
            acc[m] = sum;
        }
    }
}

static float* to_f32(const uint16_t* x, size_t count) {
    float* out = (float*)malloc(count * sizeof(float));
    for (size_t i = 0; i < count; ++i) out[i] = bf16_to_f32(x[i]);
    return out;
}

/* out[m,n] = bf16( sum + residual[m,n] ) ; residual may be NULL. */
int oracle_qmm_bf16(const uint16_t* x, const uint32_t* w, const uint16_t* scales, const uint16_t* biases,
                    const uint16_t* residual, uint16_t* out, int M, int K, int N) {
    if (K % 64 || M < 1 || M > 1024) return -1;
    float* xf = to_f32(x, (size_t)M * K);
#pragma omp parallel
    {
        float* acc = (float*)malloc(sizeof(float) * M);
#pragma omp for schedule(static)
        for (int n = 0; n < N; ++n) {
            row_dot(xf, w + (size_t)n * (K / 8), scales + (size_t)n * (K / 64), biases + (size_t)n * (K / 64), M, K, acc);
            for (int m = 0; m < M; ++m) {
                float v = acc[m];
                if (residual) v += bf16_to_f32(residual[(size_t)m * N + n]);
                out[(size_t)m * N + n] = f32_to_bf16(v);
            }
        }
        free(acc);
    }
    free(xf);
    return 0;
}

/* out[m,n] = bf16( g/(1+exp(-g)) * u ) with g,u un-rounded fp32 sums. */
int oracle_swiglu_bf16(const uint16_t* x, const uint32_t* gw, const uint16_t* gs, const uint16_t* gb,
                       const uint32_t* uw, const uint16_t* us, const uint16_t* ub, uint16_t* out, int M, int K,
                       int N) {
    if (K % 64 || M < 1 || M > 1024) return -1;
    float* xf = to_f32(x, (size_t)M * K);
#pragma omp parallel
    {
        float* g = (float*)malloc(sizeof(float) * M);
        float* u = (float*)malloc(sizeof(float) * M);
#pragma omp for schedule(static)
        for (int n = 0; n < N; ++n) {
            row_dot(xf, gw + (size_t)n * (K / 8), gs + (size_t)n * (K / 64), gb + (size_t)n * (K / 64), M, K, g);
            row_dot(xf, uw + (size_t)n * (K / 8), us + (size_t)n * (K / 64), ub + (size_t)n * (K / 64), M, K, u);
            for (int m = 0; m < M; ++m) out[(size_t)m * N + n] = f32_to_bf16(g[m] / (1.0f + expf(-g[m])) * u[m]);
        }
        free(g);
        free(u);
    }
    free(xf);
    return 0;
}

/* y = down(swiglu(x)) + residual ; hidden [M, I] is caller-provided bf16 scratch. */
int oracle_mlp_bf16(const uint16_t* x, const uint32_t* gw, const uint16_t* gs, const uint16_t* gb,
                    const uint32_t* uw, const uint16_t* us, const uint16_t* ub, const uint32_t* dw,
                    const uint16_t* ds, const uint16_t* db, const uint16_t* residual, uint16_t* hidden,
                    uint16_t* out, int M, int H, int I) {
    int rc = oracle_swiglu_bf16(x, gw, gs, gb, uw, us, ub, hidden, M, H, I);
    if (rc) return rc;
    return oracle_qmm_bf16(hidden, dw, ds, db, residual, out, M, I, H);
}

/* Sum = bf16(x+res); Out = bf16(f32(Sum) * rsqrt(mean((x+res)^2)+eps) * w). */
int oracle_add_rmsnorm_bf16(const uint16_t* x, const uint16_t* residual, const uint16_t* weight, uint16_t* sum_out,
                            uint16_t* norm_out, int rows, int H, float eps) {
#pragma omp parallel for schedule(static)
    for (int r = 0; r < rows; ++r) {
        float ss = 0.0f;
        for (int c = 0; c < H; ++c) {
            float v = bf16_to_f32(x[(size_t)r * H + c]);
            if (residual) v += bf16_to_f32(residual[(size_t)r * H + c]);
            if (sum_out) sum_out[(size_t)r * H + c] = f32_to_bf16(v);
            ss += v * v;
        }
        const float inv = 1.0f / sqrtf(ss / (float)H + eps);
        for (int c = 0; c < H; ++c) {
            float v = bf16_to_f32(x[(size_t)r * H + c]);
            if (residual) v = bf16_to_f32(f32_to_bf16(v + bf16_to_f32(residual[(size_t)r * H + c])));
            norm_out[(size_t)r * H + c] = f32_to_bf16(v * inv * bf16_to_f32(weight[c]));
        }
    }
    return 0;
}
