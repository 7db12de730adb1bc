// Shared device/host helpers for the affine INT4 projection kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// ---- status codes returned by every extern "C" entry point -------------------------------
#define MT_OK 0
#define MT_ERR_SHAPE (-1)        // shape outside what the kernels accept
#define MT_ERR_ALIGN (-2)        // pointer not aligned for the vector width the kernel uses
#define MT_ERR_FORMAT (-3)       // quantisation format other than 4-bit, group 64
#define MT_ERR_LAUNCH (-4)       // CUDA reported a launch / API error
#define MT_ERR_DEVICE (-5)       // current device is not compute capability 10.x
#define MT_ERR_NULL (-6)         // required pointer is null
#define MT_ERR_WORKSPACE (-7)    // workspace missing or too small
#define MT_ERR_DEVICE_WAIT (-8)  // a bounded device-side wait gave up (see mt_device_status)

// ---- flags word ---------------------------------------------------------------------------
#define MT_FLAG_FORCE_GEMV 0x1u   // CUDA-core GEMV regardless of row count (rows <= 8 only)
#define MT_FLAG_FORCE_UMMA 0x2u   // tcgen05 path regardless of row count
#define MT_FLAG_MLP_FUSED_MMA 0x80u  // mt_affine_mlp: insist on the warp-MMA single-launch kernel (M <= 8)
#define MT_FLAG_HOST_PAIR 0x40u    // mt_affine_mlp_host: activations and residual share one host allocation
#define MT_FLAG_MLP_FUSED 0x20u    // mt_affine_mlp: insist on the single-launch kernel (error if it does not apply)
#define MT_FLAG_GELU 0x10u        // dense activation: x/(1+exp(-1.702x)) instead of SiLU

namespace mt {

// Device-side record of a bounded wait that gave up: word 0 = code, 1 = block, 2 = detail.
// Written with atomicCAS so the first failure wins; zero means every wait completed.
// The library is one translation unit, so the definition lives here.
__device__ unsigned int g_device_status[4] = {0, 0, 0, 0};

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits16) { return __uint_as_float(bits16 << 16); }
__device__ __forceinline__ float bf16_lo(uint32_t pair) { return __uint_as_float(pair << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t pair) { return __uint_as_float(pair & 0xFFFF0000u); }

__device__ __forceinline__ uint16_t f32_to_bf16_bits(float v) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    return (uint32_t)f32_to_bf16_bits(lo) | ((uint32_t)f32_to_bf16_bits(hi) << 16);
}

// One packed word (8 nibbles e0..e7) -> four bf16 pairs (128+e_i, 128+e_{i+4}), i = 0..3: the nibble
// lands in the low mantissa bits of the bf16 value 128.0 (0x4300), so every value is exact.
// (x & mask) | magic as ONE lop3 (truth table 0xEA) with both constants in registers.
__device__ __forceinline__ void unpack_word_offset128(uint32_t w, uint32_t* out) {
#pragma unroll
    for (int i = 0; i < 4; ++i)
        asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(out[i]) : "r"(w >> (4 * i)), "r"(0x000F000Fu), "r"(0x43004300u));
}

// The eight nibbles of a word as the floats 128+e0 .. 128+e7 (natural order).
__device__ __forceinline__ void unpack_word_f32_offset128(uint32_t w, float (&q)[8]) {
    const uint32_t even = w & 0x0F0F0F0Fu, odd = (w >> 4) & 0x0F0F0F0Fu;
    constexpr uint32_t kMagic = 0x43000000u;  // 128.0f
    q[0] = __uint_as_float(__byte_perm(even, kMagic, 0x7044));
    q[1] = __uint_as_float(__byte_perm(odd, kMagic, 0x7044));
    q[2] = __uint_as_float(__byte_perm(even, kMagic, 0x7144));
    q[3] = __uint_as_float(__byte_perm(odd, kMagic, 0x7144));
    q[4] = __uint_as_float(__byte_perm(even, kMagic, 0x7244));
    q[5] = __uint_as_float(__byte_perm(odd, kMagic, 0x7244));
    q[6] = __uint_as_float(__byte_perm(even, kMagic, 0x7344));
    q[7] = __uint_as_float(__byte_perm(odd, kMagic, 0x7344));
}

__device__ __forceinline__ float warp_sum_xor(float v) {
#pragma unroll
    for (int offset = 16; offset >= 1; offset >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, offset);
    return v;
}

// g/(1+exp(-g)) * u on un-rounded fp32 sums.
__device__ __forceinline__ float swiglu_f32(float gate, float up) { return gate / (1.0f + __expf(-gate)) * up; }

inline bool aligned_to(const void* p, size_t bytes) { return (reinterpret_cast<uintptr_t>(p) % bytes) == 0; }

}  // namespace mt
