// INT4 affine dequant-GEMV on the CUDA cores, for 1..8 activation rows served from ONE read of
// the packed weights.
//
// Computes what the reference's kernels/affine_qmv.py:4-54 computes (word / element / group
// indexing, w = scale*q + bias, fp32 accumulation, one rounding at the store) with the residual
// epilogue of :124-131 and the SwiGLU epilogue of :204-208.  Unlike the reference's kernel, which
// re-reads the weights once per activation row (flattened output index, :22-24), every row of the
// batch shares the same weight registers here.
//
// Mapping: half a warp (16 lanes) owns one output row; lane l reads the 128-bit word group
// j = l + 16*t of that row (32 nibbles = half a scale group), t = 0, 1, ...  A warp pass covers
// 2*kRows output rows.  When N is small the K range of a row is cut into `ksplit` contiguous
// parts handled by different warps of the CTA (more bytes in flight); the parts are summed
// through shared memory in part order.  ksplit is a function of (N, K) only.
//
// Arithmetic.  The kernel is bound by instruction issue, not by HBM (the logic pipe runs at half
// the FMA pipe's rate), so a nibble costs two instructions: one byte-permute puts it into the
// mantissa of 128.0f, giving the float 128+q exactly, and one FMA multiplies it with the
// activation.  Per 32-nibble slot:  dot = sum_e (128+q_e) * x_e  in ascending e, then
//     acc = fma(scale, dot, fma(bias - 128*scale, xsum, acc)),   xsum = ((x_0 + x_1) + ...) + x_31,
// which equals scale*sum(q*x) + bias*sum(x) up to fp32 rounding.  Weights are never rounded.
// With one activation row the activations are converted to fp32 once per CTA and kept in shared
// memory in the order the lanes read them (16-byte chunks of consecutive lanes adjacent: no bank
// conflicts), together with the per-slot sums; with more rows they are converted on the fly.
// The order of every fp32 operation for one (row, output) pair depends on K only -- not on the
// number of rows, the grid, N or where the activations are staged -- so results are bit-identical
// for a row run alone or inside a batch of up to 8.
#pragma once

#include "common.cuh"
#include "ptx.cuh"

namespace mt {

__device__ __forceinline__ uint4 ldg_stream_u4(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

struct GemvWeights {
    const uint32_t* w;
    const uint16_t* scales;
    const uint16_t* biases;
};

enum GemvStage : int {
    kStageNone = 0,  // activations read from global memory
    kStageBf16 = 1,  // copied to shared memory as they are
    kStageF32 = 2,   // one row: converted to fp32, lane-interleaved, plus per-slot sums
};

// Shared-memory bytes of the kStageF32 layout: ceil(K/512) steps x 8 chunks x 16 lanes x 16 B, then
// one fp32 sum per 32-column slot.
inline int gemv_f32_stage_bytes(int K) {
    const int steps = ((K >> 5) + 15) >> 4;
    return steps * 8 * 16 * 16 + (K >> 5) * 4;
}

// kM rows of activations; kRows output rows per half-warp per pass; kDual = gate|up with SwiGLU.
//
// The (pass, slot) iteration space is flattened and software-pipelined: the packed words, scale and
// bias of iteration i+1 are requested before iteration i is computed.  With programmatic dependent
// launch the first request goes out before the kernel waits for its predecessor (nobody writes
// weights); the activations -- the predecessor's output -- are read only after that wait, with
// coherent loads.
template <int kM, int kRows, bool kDual, int kStage>
__global__ void __launch_bounds__(256)
affine_gemv_kernel(const uint16_t* x, GemvWeights first, GemvWeights second, const uint16_t* residual,
                   uint16_t* __restrict__ out, int K, int N, int ksplit) {
    static_assert(kStage != kStageF32 || kM == 1, "the fp32 stage holds one activation row");
    constexpr int kStreams = kDual ? 2 : 1;
    constexpr int kWarps = 8;
    extern __shared__ uint4 x_shared[];  // kStageBf16: [kM][K/8] vectors of 8 bf16; kStageF32: see above
    __shared__ float partial[kWarps][2][kStreams * kRows * kM];
    const int lane = threadIdx.x & 31;
    const int half = lane >> 4;
    const int l16 = lane & 15;
    const int warp = threadIdx.x >> 5;
    const int part = warp % ksplit;          // which K part this warp sums
    const int team = warp / ksplit;          // which row group of the CTA it belongs to
    const int teams_per_cta = kWarps / ksplit;
    const int slots_per_row = K >> 5;  // 128-bit word groups per weight row
    const int words_per_row = K >> 3;
    const int groups_per_row = K >> 6;
    const int rows_per_pass = 2 * kRows;
    const int slots_per_part = (slots_per_row + ksplit - 1) / ksplit;
    const int slot_begin = part * slots_per_part;
    const int slot_end = min(slot_begin + slots_per_part, slots_per_row);
    const int team_global = blockIdx.x * teams_per_cta + team;
    const int teams_total = gridDim.x * teams_per_cta;
    // A CTA's row blocks (rows_per_pass rows per team) are blockIdx.x, blockIdx.x + gridDim.x, ...: it
    // runs as many passes as it has blocks that start below N -- not the grid-wide maximum, which at
    // N = 8192 made most CTAs spend a second pass on clamped rows whose results nobody stores, in a
    // kernel bound by instruction issue.  Every warp of a CTA runs the same number of iterations (the
    // bounds depend on blockIdx only), so the __syncthreads below are reached by all of them.
    const int row_blocks = (N + teams_per_cta * rows_per_pass - 1) / (teams_per_cta * rows_per_pass);
    const int passes = (int)((unsigned int)(row_blocks - 1 - (int)blockIdx.x) / gridDim.x) + 1;  // the grid has at most row_blocks CTAs
    const int steps = (slots_per_part + 15) >> 4;  // slot iterations per pass (some lanes idle in the last)

    struct Weights {
        uint4 packed[kStreams][kRows];
        uint32_t scale[kStreams][kRows], bias[kStreams][kRows];
    };
    auto request = [&](int pass, int step, Weights& w) {
        const int slot = slot_begin + l16 + (step << 4);
        if (pass >= passes || slot >= slot_end) return;
        const int row_base = (pass * teams_total + team_global) * rows_per_pass;
#pragma unroll
        for (int s = 0; s < kStreams; ++s) {
            const GemvWeights& wt = s == 0 ? first : second;
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                const int n = min(row_base + half * kRows + r, N - 1);  // clamp loads; the store is guarded
                w.packed[s][r] = ldg_stream_u4(reinterpret_cast<const uint4*>(wt.w + (size_t)n * words_per_row) + slot);
                const size_t g = (size_t)n * groups_per_row + (slot >> 1);
                w.scale[s][r] = __ldg(wt.scales + g);
                w.bias[s][r] = __ldg(wt.biases + g);
            }
        }
    };

    ptx::griddep_launch_dependents();
    Weights next;
    request(0, 0, next);
    ptx::griddep_wait();  // activations and residual are the preceding kernel's output
    if constexpr (kStage == kStageBf16) {
        const int vectors = kM * (K >> 3);
        for (int v = threadIdx.x; v < vectors; v += blockDim.x) x_shared[v] = ptx::ld_global_dependent_u4(x + (size_t)v * 8);
        __syncthreads();
    }
    if constexpr (kStage == kStageF32) {
        float4* xq = reinterpret_cast<float4*>(x_shared);
        const int steps_all = (slots_per_row + 15) >> 4;
        float* slot_sum = reinterpret_cast<float*>(xq + steps_all * 128);
        // Eight bf16 = chunks 2c and 2c+1 of their slot; chunk i of slot j lives at ((j/16)*8 + i)*16 + j%16.
        for (int v = threadIdx.x; v < (K >> 3); v += blockDim.x) {
            const uint4 raw = ptx::ld_global_dependent_u4(x + (size_t)v * 8);
            const int slot = v >> 2, chunk = (v & 3) << 1;
            float4* dst = xq + (((slot >> 4) << 3) + chunk) * 16 + (slot & 15);
            dst[0] = make_float4(bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y));
            dst[16] = make_float4(bf16_lo(raw.z), bf16_hi(raw.z), bf16_lo(raw.w), bf16_hi(raw.w));
        }
        __syncthreads();
        for (int slot = threadIdx.x; slot < slots_per_row; slot += blockDim.x) {
            const float4* src = xq + ((slot >> 4) << 3) * 16 + (slot & 15);
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float4 c = src[i * 16];
                sum += c.x; sum += c.y; sum += c.z; sum += c.w;
            }
            slot_sum[slot] = sum;
        }
        __syncthreads();
    }

    float acc[kStreams][kRows][kM];
    int next_pass = 0, next_step = 0;
    for (int pass = 0; pass < passes; ++pass) {
        const int row_base = (pass * teams_total + team_global) * rows_per_pass;
#pragma unroll
        for (int s = 0; s < kStreams; ++s)
#pragma unroll
            for (int r = 0; r < kRows; ++r)
#pragma unroll
                for (int m = 0; m < kM; ++m) acc[s][r][m] = 0.0f;

        for (int step = 0; step < steps; ++step) {
            const int slot = slot_begin + l16 + (step << 4);
            const Weights cur = next;
            if (++next_step == steps) {
                next_step = 0;
                ++next_pass;
            }
            request(next_pass, next_step, next);
            if (slot >= slot_end) continue;

            float dot[kStreams][kRows][kM];
            float xsum[kM];
#pragma unroll
            for (int m = 0; m < kM; ++m) {
                xsum[m] = 0.0f;
#pragma unroll
                for (int s = 0; s < kStreams; ++s)
#pragma unroll
                    for (int r = 0; r < kRows; ++r) dot[s][r][m] = 0.0f;
            }
#pragma unroll
            for (int wi = 0; wi < 4; ++wi) {
                float xv[kM][8];
                if constexpr (kStage == kStageF32) {
                    const float4* src = reinterpret_cast<const float4*>(x_shared) + (((slot >> 4) << 3) + 2 * wi) * 16 + (slot & 15);
                    const float4 a = src[0], b = src[16];
                    xv[0][0] = a.x; xv[0][1] = a.y; xv[0][2] = a.z; xv[0][3] = a.w;
                    xv[0][4] = b.x; xv[0][5] = b.y; xv[0][6] = b.z; xv[0][7] = b.w;
                } else {
#pragma unroll
                    for (int m = 0; m < kM; ++m) {
                        uint4 raw;
                        if constexpr (kStage == kStageBf16) raw = x_shared[m * (K >> 3) + slot * 4 + wi];
                        else raw = ptx::ld_global_dependent_u4(x + (size_t)m * K + (size_t)slot * 32 + wi * 8);
                        xv[m][0] = bf16_lo(raw.x); xv[m][1] = bf16_hi(raw.x);
                        xv[m][2] = bf16_lo(raw.y); xv[m][3] = bf16_hi(raw.y);
                        xv[m][4] = bf16_lo(raw.z); xv[m][5] = bf16_hi(raw.z);
                        xv[m][6] = bf16_lo(raw.w); xv[m][7] = bf16_hi(raw.w);
#pragma unroll
                        for (int e = 0; e < 8; ++e) xsum[m] += xv[m][e];
                    }
                }
#pragma unroll
                for (int s = 0; s < kStreams; ++s)
#pragma unroll
                    for (int r = 0; r < kRows; ++r) {
                        const uint32_t word = wi == 0 ? cur.packed[s][r].x
                                            : wi == 1 ? cur.packed[s][r].y
                                            : wi == 2 ? cur.packed[s][r].z
                                                      : cur.packed[s][r].w;
                        float q[8];
                        unpack_word_f32_offset128(word, q);
#pragma unroll
                        for (int m = 0; m < kM; ++m)
#pragma unroll
                            for (int e = 0; e < 8; ++e) dot[s][r][m] = fmaf(q[e], xv[m][e], dot[s][r][m]);
                    }
            }
            if constexpr (kStage == kStageF32) {
                const float4* base = reinterpret_cast<const float4*>(x_shared);
                xsum[0] = reinterpret_cast<const float*>(base + ((slots_per_row + 15) >> 4) * 128)[slot];
            }
#pragma unroll
            for (int s = 0; s < kStreams; ++s)
#pragma unroll
                for (int r = 0; r < kRows; ++r) {
                    const float scale = bf16_bits_to_f32(cur.scale[s][r]), bias = bf16_bits_to_f32(cur.bias[s][r]);
                    const float shifted = fmaf(-128.0f, scale, bias);  // the weights were decoded as 128+q
#pragma unroll
                    for (int m = 0; m < kM; ++m)
                        acc[s][r][m] = fmaf(scale, dot[s][r][m], fmaf(shifted, xsum[m], acc[s][r][m]));
                }
        }

        // ---- end of a pass: 16-lane butterfly inside each half-warp, then the K parts in order
#pragma unroll
        for (int s = 0; s < kStreams; ++s)
#pragma unroll
            for (int r = 0; r < kRows; ++r)
#pragma unroll
                for (int m = 0; m < kM; ++m) {
                    float v = acc[s][r][m];
#pragma unroll
                    for (int offset = 8; offset >= 1; offset >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, offset);
                    acc[s][r][m] = v;
                }
        if (ksplit > 1) {
            if (l16 == 0) {
#pragma unroll
                for (int s = 0; s < kStreams; ++s)
#pragma unroll
                    for (int r = 0; r < kRows; ++r)
#pragma unroll
                        for (int m = 0; m < kM; ++m) partial[warp][half][(s * kRows + r) * kM + m] = acc[s][r][m];
            }
            __syncthreads();
            if (part == 0 && l16 == 0) {
#pragma unroll
                for (int s = 0; s < kStreams; ++s)
#pragma unroll
                    for (int r = 0; r < kRows; ++r)
#pragma unroll
                        for (int m = 0; m < kM; ++m) {
                            float v = acc[s][r][m];
                            for (int p = 1; p < ksplit; ++p) v += partial[warp + p][half][(s * kRows + r) * kM + m];
                            acc[s][r][m] = v;
                        }
            }
            __syncthreads();
        }
        if (part == 0 && l16 == 0) {
#pragma unroll
            for (int r = 0; r < kRows; ++r) {
                const int n = row_base + half * kRows + r;
                if (n < N) {
#pragma unroll
                    for (int m = 0; m < kM; ++m) {
                        float v;
                        if constexpr (kDual) v = swiglu_f32(acc[0][r][m], acc[kStreams - 1][r][m]);
                        else v = acc[0][r][m];
                        if (residual) v += bf16_bits_to_f32(ptx::ld_global_dependent_u16(residual + (size_t)m * N + n));
                        out[(size_t)m * N + n] = f32_to_bf16_bits(v);
                    }
                }
            }
        }
    }
}

constexpr int kGemvStageLimit = 104 * 1024;

// K parts per row: enough warps to keep the memory system busy when N is small.  Depends on
// (N, K) only, never on the number of activation rows.
inline int gemv_ksplit(int K, int N) {
    int ksplit = 1;
    const int slots = K >> 5;
    while (ksplit < 8 && (long)N * ksplit < 16384 && slots / (ksplit * 2) >= 16) ksplit *= 2;
    return ksplit;
}

template <int kM, bool kDual, int kStage>
inline int launch_gemv_instance(const uint16_t* x, GemvWeights a, GemvWeights b, const uint16_t* residual,
                                uint16_t* out, int K, int N, int sm_count, cudaStream_t stream) {
    constexpr int kRows = kDual ? (kM <= 2 ? 2 : 1) : (kM <= 2 ? 4 : (kM <= 4 ? 2 : 1));
    constexpr int kWarps = 8;
    auto kernel = affine_gemv_kernel<kM, kRows, kDual, kStage>;
    const int smem = kStage == kStageF32 ? gemv_f32_stage_bytes(K) : kStage == kStageBf16 ? kM * K * 2 : 0;
    if (smem > 32 * 1024) {  // the static partial-sum array counts toward the 48 KB default limit too
        static bool configured[64] = {};
        int device = 0;
        cudaGetDevice(&device);
        if (device >= 64 || !configured[device]) {
            if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemvStageLimit) != cudaSuccess)
                return MT_ERR_LAUNCH;
            if (device < 64) configured[device] = true;
        }
    }
    const int ksplit = gemv_ksplit(K, N);
    const int rows_per_cta = (kWarps / ksplit) * 2 * kRows;
    int grid = (N + rows_per_cta - 1) / rows_per_cta;
    // Resident CTAs per SM (each loops over its share of the rows): three when registers (80 x 256
    // threads) and the staged activations allow, else two.  The kernel waits on HBM latency with one
    // request in flight per lane and stream, so more resident warps mean more bytes in flight.
    const int cap = sm_count * (kM == 1 && smem <= 72 * 1024 ? 3 : 2);
    if (grid > cap) grid = cap;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid, 1, 1);
    config.blockDim = dim3(kWarps * 32, 1, 1);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attrs;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, x, a, b, residual, out, K, N, ksplit) == cudaSuccess ? MT_OK
                                                                                                     : MT_ERR_LAUNCH;
}

// Activations are staged in shared memory when they fit kGemvStageLimit, which leaves room for two
// CTAs per SM (one row as fp32: K up to 24576; more rows as bf16); larger problems read them from
// global memory.
template <int kM, bool kDual>
inline int launch_gemv_m(const uint16_t* x, GemvWeights a, GemvWeights b, const uint16_t* residual, uint16_t* out,
                         int K, int N, int sm_count, cudaStream_t stream) {
    if constexpr (kM == 1) {
        if (gemv_f32_stage_bytes(K) <= kGemvStageLimit)
            return launch_gemv_instance<kM, kDual, kStageF32>(x, a, b, residual, out, K, N, sm_count, stream);
    }
    if ((long)kM * K * 2 <= kGemvStageLimit)
        return launch_gemv_instance<kM, kDual, kStageBf16>(x, a, b, residual, out, K, N, sm_count, stream);
    return launch_gemv_instance<kM, kDual, kStageNone>(x, a, b, residual, out, K, N, sm_count, stream);
}

template <bool kDual>
inline int launch_gemv(const void* x, GemvWeights a, GemvWeights b, const void* residual, void* out, int M, int K,
                       int N, int sm_count, cudaStream_t stream) {
    const uint16_t* xp = static_cast<const uint16_t*>(x);
    const uint16_t* rp = static_cast<const uint16_t*>(residual);
    uint16_t* op = static_cast<uint16_t*>(out);
    switch (M) {
        case 1: return launch_gemv_m<1, kDual>(xp, a, b, rp, op, K, N, sm_count, stream);
        case 2: return launch_gemv_m<2, kDual>(xp, a, b, rp, op, K, N, sm_count, stream);
        case 3: return launch_gemv_m<3, kDual>(xp, a, b, rp, op, K, N, sm_count, stream);
        case 4: return launch_gemv_m<4, kDual>(xp, a, b, rp, op, K, N, sm_count, stream);
        case 5: return launch_gemv_m<5, kDual>(xp, a, b, rp, op, K, N, sm_count, stream);
        case 6: return launch_gemv_m<6, kDual>(xp, a, b, rp, op, K, N, sm_count, stream);
        case 7: return launch_gemv_m<7, kDual>(xp, a, b, rp, op, K, N, sm_count, stream);
        case 8: return launch_gemv_m<8, kDual>(xp, a, b, rp, op, K, N, sm_count, stream);
        default: return MT_ERR_SHAPE;
    }
}

}  // namespace mt
