// Dense bf16 small-batch projection: rows of a batch share every weight load, and each row's
// result is bit-identical to running that row alone.
//
// Follows the arithmetic order of the reference's generated small-batch kernels
// (metile/compiler/dense.py:193-381, emitted by metile/codegen/msl_emitter.py:1067-1120 and
// :1218-1251): lane l of a 32-lane group owns k = 128*b + 4*l .. +3, accumulates in fp32 in
// ascending (b, component) order with fused multiply-adds, lanes are combined by a shuffle-down
// tree with offsets 16, 8, 4, 2, 1, lane 0 rounds to bf16, then the typed epilogue runs:
//   residual : bf16(bf16(acc) + residual)
//   SwiGLU   : l = bf16(gate), r = bf16(up), y = 1/(1+exp(|l|)), sig = bf16(l<0 ? y : 1-y),
//              out = bf16(bf16(l*sig) * r)
// One warp produces kOut outputs for all rows of a pass; up to 16 rows share one pass over the matrix.
#pragma once

#include "common.cuh"

namespace mt {

__device__ __forceinline__ uint2 ldg_stream_u2(const uint2* p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

__device__ __forceinline__ float round_bf16(float v) { return bf16_bits_to_f32(f32_to_bf16_bits(v)); }

enum class DenseEpilogue { kPlain, kSwiglu };

// kM: activation rows of the launch's template (rows past `rows` are computed on row `rows - 1`'s
// activations and not stored); kOut: outputs per warp; kAhead: 128-column blocks whose weights are
// requested together (bytes in flight per lane = kAhead * kOut * kStreams * 8).
template <int kM, int kOut, int kAhead, DenseEpilogue kEp>
__global__ void __launch_bounds__(256)
dense_rows_kernel(const uint16_t* __restrict__ x, const uint16_t* __restrict__ w0, const uint16_t* __restrict__ w1,
                  const uint16_t* __restrict__ residual, uint16_t* __restrict__ out, int rows, int K, int N) {
    constexpr int kStreams = kEp == DenseEpilogue::kSwiglu ? 2 : 1;
    const int lane = threadIdx.x & 31;
    const int warp_global = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int warps_total = gridDim.x * (blockDim.x >> 5);
    const int blocks = K >> 7;

    for (int out_base = warp_global * kOut; out_base < N; out_base += warps_total * kOut) {
        float acc[kStreams][kOut][kM];
#pragma unroll
        for (int s = 0; s < kStreams; ++s)
#pragma unroll
            for (int o = 0; o < kOut; ++o)
#pragma unroll
                for (int m = 0; m < kM; ++m) acc[s][o][m] = 0.0f;
        size_t row_offset[kOut];
#pragma unroll
        for (int o = 0; o < kOut; ++o) row_offset[o] = (size_t)min(out_base + o, N - 1) * K;

        for (int b0 = 0; b0 < blocks; b0 += kAhead) {
            // Request the weights of kAhead blocks before any of them is used: the kernel streams the
            // matrix once, so what matters is how many bytes each warp keeps in flight.
            uint2 wv[kAhead][kStreams][kOut];
#pragma unroll
            for (int a = 0; a < kAhead; ++a) {
                const int k = (min(b0 + a, blocks - 1) << 7) + (lane << 2);
#pragma unroll
                for (int s = 0; s < kStreams; ++s)
#pragma unroll
                    for (int o = 0; o < kOut; ++o)
                        wv[a][s][o] = ldg_stream_u2(reinterpret_cast<const uint2*>((s == 0 ? w0 : w1) + row_offset[o] + k));
            }
#pragma unroll
            for (int a = 0; a < kAhead; ++a) {
                if (b0 + a >= blocks) break;  // ascending block order, whatever kAhead is
                const int k = ((b0 + a) << 7) + (lane << 2);
                float wf[kStreams][kOut][4];
#pragma unroll
                for (int s = 0; s < kStreams; ++s)
#pragma unroll
                    for (int o = 0; o < kOut; ++o) {
                        wf[s][o][0] = bf16_lo(wv[a][s][o].x); wf[s][o][1] = bf16_hi(wv[a][s][o].x);
                        wf[s][o][2] = bf16_lo(wv[a][s][o].y); wf[s][o][3] = bf16_hi(wv[a][s][o].y);
                    }
#pragma unroll
                for (int m = 0; m < kM; ++m) {
                    const int row = kM <= 8 ? m : min(m, rows - 1);
                    const uint2 xv = __ldg(reinterpret_cast<const uint2*>(x + (size_t)row * K + k));
                    const float xf[4] = {bf16_lo(xv.x), bf16_hi(xv.x), bf16_lo(xv.y), bf16_hi(xv.y)};
#pragma unroll
                    for (int s = 0; s < kStreams; ++s)
#pragma unroll
                        for (int o = 0; o < kOut; ++o)
#pragma unroll
                            for (int c = 0; c < 4; ++c) acc[s][o][m] = fmaf(wf[s][o][c], xf[c], acc[s][o][m]);
                }
            }
        }

#pragma unroll
        for (int s = 0; s < kStreams; ++s)
#pragma unroll
            for (int o = 0; o < kOut; ++o)
#pragma unroll
                for (int m = 0; m < kM; ++m) {
                    float v = acc[s][o][m];
#pragma unroll
                    for (int offset = 16; offset >= 1; offset >>= 1) v += __shfl_down_sync(0xFFFFFFFFu, v, offset);
                    acc[s][o][m] = v;
                }

        if (lane == 0) {
#pragma unroll
            for (int o = 0; o < kOut; ++o) {
                const int n = out_base + o;
                if (n >= N) continue;
#pragma unroll
                for (int m = 0; m < kM; ++m) {
                    if (m >= rows) break;
                    float v;
                    if constexpr (kEp == DenseEpilogue::kSwiglu) {
                        const float left = round_bf16(acc[0][o][m]);
                        const float right = round_bf16(acc[1][o][m]);
                        const float y = 1.0f / (1.0f + expf(fabsf(left)));
                        const float sigmoid = round_bf16(left < 0.0f ? y : 1.0f - y);
                        v = round_bf16(left * sigmoid) * right;
                    } else {
                        v = round_bf16(acc[0][o][m]);
                        if (residual) v += bf16_bits_to_f32(residual[(size_t)m * N + n]);
                    }
                    out[(size_t)m * N + n] = f32_to_bf16_bits(v);
                }
            }
        }
    }
}

template <int kM, DenseEpilogue kEp>
inline int launch_dense_m(const uint16_t* x, const uint16_t* w0, const uint16_t* w1, const uint16_t* residual,
                          uint16_t* out, int rows, int K, int N, int sm_count, cudaStream_t stream) {
    constexpr int kStreams = kEp == DenseEpilogue::kSwiglu ? 2 : 1;
    // The fp32 order of an output is fixed (one warp, ascending blocks), so parallelism comes from the
    // outputs.  Two outputs per warp share every activation load and conversion (measured at 8 rows:
    // 17.3 us against 20.2 us with one output per warp); 32 rows x two outputs would not fit the registers.
    constexpr int kOut = (kM * kStreams <= 16) ? 2 : 1;
    constexpr int kAhead = kM * kStreams <= 4 ? 3 : 2;
    const int warps_needed = (N + kOut - 1) / kOut;
    int grid = (warps_needed + 7) / 8;
    const int cap = sm_count * 8;
    if (grid > cap) grid = cap;
    dense_rows_kernel<kM, kOut, kAhead, kEp><<<grid, 256, 0, stream>>>(x, w0, w1, residual, out, rows, K, N);
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_LAUNCH;
}

template <DenseEpilogue kEp>
inline int launch_dense(const void* x, const void* w0, const void* w1, const void* residual, void* out, int M, int K,
                        int N, int sm_count, cudaStream_t stream) {
    if (M < 1 || K < 128 || K % 128 || N < 1) return MT_ERR_SHAPE;
    if (!aligned_to(x, 8) || !aligned_to(w0, 8) || (w1 && !aligned_to(w1, 8))) return MT_ERR_ALIGN;
    const uint16_t* xp = static_cast<const uint16_t*>(x);
    const uint16_t* ap = static_cast<const uint16_t*>(w0);
    const uint16_t* bp = static_cast<const uint16_t*>(w1);
    const uint16_t* rp = static_cast<const uint16_t*>(residual);
    uint16_t* op = static_cast<uint16_t*>(out);
    // Up to 16 rows share one pass over the weights; larger batches run as chunks of 16, whose
    // re-reads of the matrix come from L2 when it fits there (measured at K = 1536, N = 8960: 26 us per
    // 16-row pass against 92 us for a 32-row pass, whose 32 accumulators per output leave the FMA pipe
    // waiting on activation loads).  A row's result is the same in any chunking: its fp32 order depends
    // on (K, lane) only.
    constexpr int kChunk = 16;
    for (int m0 = 0; m0 < M; m0 += kChunk) {
        const int rows = M - m0 < kChunk ? M - m0 : kChunk;
        const uint16_t* xc = xp + (size_t)m0 * K;
        const uint16_t* rc = rp ? rp + (size_t)m0 * N : nullptr;
        uint16_t* oc = op + (size_t)m0 * N;
        int rc_code;
        switch (rows) {
            case 1: rc_code = launch_dense_m<1, kEp>(xc, ap, bp, rc, oc, rows, K, N, sm_count, stream); break;
            case 2: rc_code = launch_dense_m<2, kEp>(xc, ap, bp, rc, oc, rows, K, N, sm_count, stream); break;
            case 3: rc_code = launch_dense_m<3, kEp>(xc, ap, bp, rc, oc, rows, K, N, sm_count, stream); break;
            case 4: rc_code = launch_dense_m<4, kEp>(xc, ap, bp, rc, oc, rows, K, N, sm_count, stream); break;
            case 5: rc_code = launch_dense_m<5, kEp>(xc, ap, bp, rc, oc, rows, K, N, sm_count, stream); break;
            case 6: rc_code = launch_dense_m<6, kEp>(xc, ap, bp, rc, oc, rows, K, N, sm_count, stream); break;
            case 7: rc_code = launch_dense_m<7, kEp>(xc, ap, bp, rc, oc, rows, K, N, sm_count, stream); break;
            case 8: rc_code = launch_dense_m<8, kEp>(xc, ap, bp, rc, oc, rows, K, N, sm_count, stream); break;
            default:
                rc_code = launch_dense_m<16, kEp>(xc, ap, bp, rc, oc, rows, K, N, sm_count, stream);
                break;
        }
        if (rc_code != MT_OK) return rc_code;
    }
    return MT_OK;
}

}  // namespace mt
