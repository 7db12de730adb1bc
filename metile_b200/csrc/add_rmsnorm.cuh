// Residual add + RMSNorm (two outputs) and plain RMSNorm, bf16 in / bf16 out, fp32 math.
//
// Semantics follow the reference's kernels/add_rmsnorm.py:7-25 and kernels/rmsnorm.py:5-26:
//   Sum = bf16(f32(x) + f32(res));  ss = sum over the row of the UN-rounded f32 sums squared;
//   Out = bf16(f32(Sum) * rsqrt(ss / H + eps) * f32(w)).
// One CTA per row.  The CTA width depends on H only, so a row's result does not depend on how
// many rows are in the batch.  HBM-bound: 2 reads + 2 writes of a row (+ the weight vector).
#pragma once

#include "common.cuh"

namespace mt {

constexpr int kNormMaxVecPerThread = 4;  // 8 bf16 per vector; rows up to 8*1024*4 = 32768 wide

template <bool kHasResidual, bool kVector>
__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(const uint16_t* __restrict__ x,
                                                           const uint16_t* __restrict__ residual,
                                                           const uint16_t* __restrict__ weight,
                                                           uint16_t* __restrict__ sum_out,
                                                           uint16_t* __restrict__ norm_out, int H, float eps) {
    __shared__ float warp_partial[32];
    __shared__ float inverse_rms_shared;
    const size_t row_base = (size_t)blockIdx.x * H;
    float ss = 0.0f;

    // Rounded sums kept in registers as bf16 pairs so pass two does not touch memory again.
    uint4 kept[kNormMaxVecPerThread];
    const int vectors = kVector ? H / 8 : 0;

    if constexpr (kVector) {
#pragma unroll
        for (int i = 0; i < kNormMaxVecPerThread; ++i) {
            const int v = threadIdx.x + i * blockDim.x;
            if (v < vectors) {
                uint4 xv = *reinterpret_cast<const uint4*>(x + row_base + (size_t)v * 8);
                uint32_t xs[4] = {xv.x, xv.y, xv.z, xv.w};
                uint32_t rs[4] = {0, 0, 0, 0};
                if constexpr (kHasResidual) {
                    uint4 rv = *reinterpret_cast<const uint4*>(residual + row_base + (size_t)v * 8);
                    rs[0] = rv.x; rs[1] = rv.y; rs[2] = rv.z; rs[3] = rv.w;
                }
                uint32_t packed[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float lo = bf16_lo(xs[j]) + (kHasResidual ? bf16_lo(rs[j]) : 0.0f);
                    float hi = bf16_hi(xs[j]) + (kHasResidual ? bf16_hi(rs[j]) : 0.0f);
                    ss = fmaf(lo, lo, ss);
                    ss = fmaf(hi, hi, ss);
                    packed[j] = kHasResidual ? pack_bf16x2(lo, hi) : xs[j];
                }
                kept[i] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                if constexpr (kHasResidual) {
                    if (sum_out) *reinterpret_cast<uint4*>(sum_out + row_base + (size_t)v * 8) = kept[i];
                }
            }
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            float v = bf16_bits_to_f32(x[row_base + c]);
            if constexpr (kHasResidual) {
                v += bf16_bits_to_f32(residual[row_base + c]);
                if (sum_out) sum_out[row_base + c] = f32_to_bf16_bits(v);
            }
            ss = fmaf(v, v, ss);
        }
    }

    ss = warp_sum_xor(ss);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) warp_partial[warp] = ss;
    __syncthreads();
    if (warp == 0) {
        const int warps = (blockDim.x + 31) >> 5;
        float v = lane < warps ? warp_partial[lane] : 0.0f;
        v = warp_sum_xor(v);
        if (lane == 0) inverse_rms_shared = 1.0f / sqrtf(v / (float)H + eps);
    }
    __syncthreads();
    const float inverse_rms = inverse_rms_shared;

    if constexpr (kVector) {
#pragma unroll
        for (int i = 0; i < kNormMaxVecPerThread; ++i) {
            const int v = threadIdx.x + i * blockDim.x;
            if (v < vectors) {
                uint4 wv = *reinterpret_cast<const uint4*>(weight + (size_t)v * 8);
                uint32_t ws[4] = {wv.x, wv.y, wv.z, wv.w};
                uint32_t ks[4] = {kept[i].x, kept[i].y, kept[i].z, kept[i].w};
                uint32_t outp[4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    outp[j] = pack_bf16x2(bf16_lo(ks[j]) * inverse_rms * bf16_lo(ws[j]),
                                          bf16_hi(ks[j]) * inverse_rms * bf16_hi(ws[j]));
                *reinterpret_cast<uint4*>(norm_out + row_base + (size_t)v * 8) =
                    make_uint4(outp[0], outp[1], outp[2], outp[3]);
            }
        }
    } else {
        for (int c = threadIdx.x; c < H; c += blockDim.x) {
            float v = bf16_bits_to_f32(x[row_base + c]);
            if constexpr (kHasResidual)
                v = bf16_bits_to_f32(f32_to_bf16_bits(v + bf16_bits_to_f32(residual[row_base + c])));
            norm_out[row_base + c] = f32_to_bf16_bits(v * inverse_rms * bf16_bits_to_f32(weight[c]));
        }
    }
}

inline int launch_add_rmsnorm(const void* x, const void* residual, const void* weight, void* sum_out,
                              void* norm_out, int rows, int H, float eps, cudaStream_t stream) {
    if (!x || !weight || !norm_out) return MT_ERR_NULL;
    if (rows < 0 || H < 1) return MT_ERR_SHAPE;
    if (rows == 0) return MT_OK;
    const bool has_residual = residual != nullptr;
    bool vector = (H % 8 == 0) && aligned_to(x, 16) && aligned_to(weight, 16) && aligned_to(norm_out, 16) &&
                  (!residual || aligned_to(residual, 16)) && (!sum_out || aligned_to(sum_out, 16));
    int threads;
    if (vector) {
        const int vectors = H / 8;
        threads = ((vectors + 31) / 32) * 32;
        if (threads > 1024) threads = 1024;
        // Keep at least two vectors per thread for wide rows so fewer warps take part in the reduce.
        if (vectors > 1024 * kNormMaxVecPerThread) vector = false;
    }
    if (!vector) threads = H >= 1024 ? 1024 : ((H + 31) / 32) * 32;
    const uint16_t* xp = static_cast<const uint16_t*>(x);
    const uint16_t* rp = static_cast<const uint16_t*>(residual);
    const uint16_t* wp = static_cast<const uint16_t*>(weight);
    uint16_t* sp = static_cast<uint16_t*>(sum_out);
    uint16_t* np_ = static_cast<uint16_t*>(norm_out);
    if (has_residual) {
        if (vector) add_rmsnorm_kernel<true, true><<<rows, threads, 0, stream>>>(xp, rp, wp, sp, np_, H, eps);
        else add_rmsnorm_kernel<true, false><<<rows, threads, 0, stream>>>(xp, rp, wp, sp, np_, H, eps);
    } else {
        if (vector) add_rmsnorm_kernel<false, true><<<rows, threads, 0, stream>>>(xp, rp, wp, sp, np_, H, eps);
        else add_rmsnorm_kernel<false, false><<<rows, threads, 0, stream>>>(xp, rp, wp, sp, np_, H, eps);
    }
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_LAUNCH;
}

}  // namespace mt
