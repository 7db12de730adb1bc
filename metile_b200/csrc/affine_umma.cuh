// INT4 affine dequant-MMA on the 5th-generation tensor cores (tcgen05 + TMEM), 1..128 activation
// rows per launch, packed weights read from HBM exactly once.
//
// Computes Y[M,N] = X[M,K] * dequant(W)[N,K]^T with the MLX layout the reference consumes
// (kernels/affine_qmv.py:25-51; shapes metile/backends/mlx_quantized.py:478-480), optionally
// fused gate|up with the SwiGLU epilogue g/(1+exp(-g))*u on un-rounded sums
// (kernels/affine_qmv.py:204-208) or the residual epilogue (:124-131).  It plays the role of the
// reference's multi-row matrix-unit path (metile/compiler/affine_quantized.py:7-99), which, like
// this kernel, rounds each dequantised weight to the 16-bit input type before the MMA
// (metile/codegen/msl_emitter.py:1413-1418) and accumulates in fp32.
//
// Shape of the computation ("swap-AB"): the 128 weight rows of a tile are the MMA's M dimension
// (128 TMEM lanes), the activation rows (padded to 16/32/64/128) are its N dimension, K advances
// 16 elements per instruction, 64 (one quantisation group) per pipeline step.
//
//   producer lane  : TMA (cp.async.bulk.tensor, no multicast) packed weight tile(s) 128x32 B and
//                    the activation tile kMPad x 128 B into a shared-memory ring
//   dequant warps  : one thread per weight row; nibbles -> bf16x2 with the 0x4300 exponent trick
//                    ((w>>4i)&0x000F000F | 0x43004300 = 128+q), q = v-128, w = fma(q, scale, bias)
//                    (one rounding: RN_bf16(scale*q+bias)); result either stored to TMEM as the A
//                    operand (kTmemA) or to 128B-swizzled shared memory; also copies the activation
//                    tile into the swizzled B tile with the same within-8 element order the unpack
//                    produces (e0,e4,e1,e5,e2,e6,e3,e7) -- a K permutation applied to both operands
//                    leaves the contraction unchanged
//   MMA lane       : tcgen05.mma kind::f16 (bf16 x bf16 -> fp32 in TMEM), tcgen05.commit
//   epilogue       : tcgen05.ld -> fp32 partial tile in shared memory; when the K range is split
//                    over a thread-block cluster the partials are summed over DSMEM in rank order;
//                    then SwiGLU / residual, bf16 store (coalesced along N)
//
// Determinism: the K split (cluster size) is a function of (N, K, tile kind) only; each output is
// produced by one accumulator chain in ascending k plus an ordered sum of cluster partials, so a
// row's result does not depend on how many other rows are in the batch.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "ptx.cuh"

namespace mt {

constexpr int kUmmaTileRows = 128;
constexpr int kUmmaBlockK = 64;

constexpr int pow2_at_least(int v) {
    int p = 32;
    while (p < v) p *= 2;
    return p;
}

template <int kT, int kMPad, bool kTmemA>
struct UmmaConfig {
    static constexpr int kDequantWarps = 4 * kT;
    static constexpr int kProducerWarp = kDequantWarps;
    static constexpr int kMmaWarp = kDequantWarps + 1;
    static constexpr int kThreads = (kDequantWarps + 2) * 32;
    static constexpr int kWTileBytes = kUmmaTileRows * 32;          // one packed tile, one k-block
    static constexpr int kWBytes = kT * kWTileBytes;
    static constexpr int kXBytes = kMPad * 128;
    static constexpr int kStageBytes = kWBytes + kXBytes;
    static constexpr int kATileBytes = kUmmaTileRows * 128;         // one dequantised bf16 tile
    static constexpr int kABytes = kTmemA ? 0 : kT * kATileBytes;
    static constexpr int kBBytes = kMPad * 128;
    static constexpr int kAbBytes = kABytes + kBBytes;
    static constexpr int kAbStages = kTmemA ? 3 : 2;
    static constexpr int kAccCols = kT * kMPad;
    static constexpr int kATmemCols = kTmemA ? kAbStages * kT * 32 : 0;
    static constexpr int kTmemCols = pow2_at_least(kAccCols + kATmemCols);
    // Shared-memory target: two CTAs per SM while their TMEM fits twice, else one.
    static constexpr int kRingTarget = (kTmemCols <= 256 ? 106 : 196) * 1024 - kAbStages * kAbBytes;
    static constexpr int kStagesRaw = kRingTarget / kStageBytes;
    static constexpr int kStages = kStagesRaw < 2 ? 2 : (kStagesRaw > 8 ? 8 : kStagesRaw);
    static constexpr int kRingBytes = kStages * kStageBytes;
    static constexpr int kStagingBytes = kT * kMPad * kUmmaTileRows * 4;
    static constexpr int kDataBytesRaw = kRingBytes + kAbStages * kAbBytes;
    static constexpr int kDataBytes = kDataBytesRaw > kStagingBytes ? kDataBytesRaw : kStagingBytes;
    static constexpr int kBarrierBytes = 8 * (2 * kStages + 2 * kAbStages + 1) + 16;
    static constexpr int kSmemBytes = 1024 + kDataBytes + kBarrierBytes;
    // TMEM columns x resident CTAs must stay within 512, or tcgen05.alloc of a later CTA would
    // wait for an earlier one to finish.  Shared memory bounds the residency.
    static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
    static_assert(kStageBytes % 1024 == 0 && kWBytes % 1024 == 0 && kAbBytes % 1024 == 0, "1024 B alignment");
    static_assert((227 * 1024 / kSmemBytes) * kTmemCols <= 512, "TMEM over-subscription");
};

struct UmmaParams {
    CUtensorMap w_map[2];  // packed weights, uint32 [N, K/8], box {8, 128}
    CUtensorMap x_map;     // activations, bf16 [M, K], box {64, kMPad}
    const uint16_t* scales[2];
    const uint16_t* biases[2];
    const uint16_t* residual;
    uint16_t* out;
    int M, K, N, ksplit;
};

enum : unsigned int {
    kWaitRingEmpty = 0x101,
    kWaitRingFull = 0x102,
    kWaitAbEmpty = 0x103,
    kWaitAbFull = 0x104,
    kWaitAccFull = 0x105,
    kWaitDrain = 0x106,
};

__device__ __forceinline__ uint32_t bf162_bits(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }
__device__ __forceinline__ __nv_bfloat162 bits_bf162(uint32_t v) { return *reinterpret_cast<__nv_bfloat162*>(&v); }

// One packed word (8 nibbles) -> 8 bf16 weights in the order e0,e4,e1,e5,e2,e6,e3,e7.
__device__ __forceinline__ void dequant_word_bf16(uint32_t w, __nv_bfloat162 scale2, __nv_bfloat162 bias2,
                                                  uint32_t* out) {
    const __nv_bfloat162 k128 = bits_bf162(0x43004300u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t v = ((w >> (4 * i)) & 0x000F000Fu) | 0x43004300u;  // bf16 pair (128+q_i, 128+q_{i+4})
        const __nv_bfloat162 q = __hsub2(bits_bf162(v), k128);            // exact: integers 0..15
        out[i] = bf162_bits(__hfma2(q, scale2, bias2));                   // RN_bf16(scale*q + bias)
    }
}

template <int kT, int kMPad, bool kTmemA, bool kSwiglu>
__global__ void __launch_bounds__(UmmaConfig<kT, kMPad, kTmemA>::kThreads, 1)
affine_umma_kernel(const __grid_constant__ UmmaParams p) {
    using Cfg = UmmaConfig<kT, kMPad, kTmemA>;
    static_assert(!kSwiglu || kT == 2, "SwiGLU pairs a gate tile with an up tile");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* ring = smem;
    uint8_t* ab = smem + Cfg::kRingBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kDataBytes);
    uint64_t* ring_full = bars;
    uint64_t* ring_empty = ring_full + Cfg::kStages;
    uint64_t* ab_full = ring_empty + Cfg::kStages;
    uint64_t* ab_empty = ab_full + Cfg::kAbStages;
    uint64_t* acc_full = ab_empty + Cfg::kAbStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int ksplit = p.ksplit;
    const int rank = blockIdx.x % ksplit;  // equals the CTA's rank in its cluster
    const int tile = blockIdx.x / ksplit;
    const int n0 = tile * kUmmaTileRows;
    const int kblocks = p.K / kUmmaBlockK;
    const int kb_begin = (int)(((long long)kblocks * rank) / ksplit);
    const int kb_end = (int)(((long long)kblocks * (rank + 1)) / ksplit);
    const int nkb = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        for (int i = 0; i < Cfg::kStages; ++i) {
            ptx::mbar_init(&ring_full[i], 1);
            ptx::mbar_init(&ring_empty[i], Cfg::kDequantWarps);
        }
        for (int i = 0; i < Cfg::kAbStages; ++i) {
            ptx::mbar_init(&ab_full[i], Cfg::kDequantWarps);
            ptx::mbar_init(&ab_empty[i], 1);
        }
        ptx::mbar_init(acc_full, 1);
        *abort_flag = 0;
        ptx::mbar_fence_init();
    }
    if (warp == Cfg::kMmaWarp) {
        ptx::tmem_alloc(tmem_slot, Cfg::kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == Cfg::kProducerWarp) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            ptx::prefetch_tensor_map(&p.w_map[0]);
            if (kT == 2) ptx::prefetch_tensor_map(&p.w_map[1]);
            ptx::prefetch_tensor_map(&p.x_map);
            int issued = 0;
            for (int i = 0; i < nkb; ++i) {
                const int s = i % Cfg::kStages;
                const uint32_t phase = (i / Cfg::kStages) & 1;
                if (!ptx::mbar_wait(&ring_empty[s], phase ^ 1, abort_flag, kWaitRingEmpty)) break;
                ptx::mbar_expect_tx(&ring_full[s], Cfg::kStageBytes);
                uint8_t* stage = ring + s * Cfg::kStageBytes;
                const int kb = kb_begin + i;
#pragma unroll
                for (int t = 0; t < kT; ++t)
                    ptx::tma_load_2d(stage + t * Cfg::kWTileBytes, &p.w_map[t], kb * 8, n0, &ring_full[s]);
                ptx::tma_load_2d(stage + Cfg::kWBytes, &p.x_map, kb * kUmmaBlockK, 0, &ring_full[s]);
                ++issued;
            }
            if (*abort_flag) {
                // Let copies already in flight land before the CTA may exit.
                const int first = issued > Cfg::kStages ? issued - Cfg::kStages : 0;
                for (int i = first; i < issued; ++i)
                    ptx::mbar_wait(&ring_full[i % Cfg::kStages], (i / Cfg::kStages) & 1, abort_flag, kWaitDrain);
            }
        }
    } else if (warp == Cfg::kMmaWarp) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::umma_idesc_bf16(kUmmaTileRows, kMPad);
            for (int i = 0; i < nkb; ++i) {
                const int a = i % Cfg::kAbStages;
                const uint32_t phase = (i / Cfg::kAbStages) & 1;
                if (!ptx::mbar_wait(&ab_full[a], phase, abort_flag, kWaitAbFull)) break;
                ptx::tc_fence_after_sync();
                const uint32_t b_addr = ptx::smem_u32(ab + a * Cfg::kAbBytes + Cfg::kABytes);
#pragma unroll
                for (int t = 0; t < kT; ++t) {
#pragma unroll
                    for (int ks = 0; ks < kUmmaBlockK / 16; ++ks) {
                        const uint32_t d_tmem = tmem_base + t * kMPad;
                        const uint64_t b_desc = ptx::smem_desc_k_major_sw128(b_addr + ks * 32);
                        const uint32_t accumulate = (i > 0 || ks > 0) ? 1u : 0u;
                        if constexpr (kTmemA) {
                            const uint32_t a_tmem = tmem_base + Cfg::kAccCols + (a * kT + t) * 32 + ks * 8;
                            ptx::umma_ts(d_tmem, a_tmem, b_desc, idesc, accumulate);
                        } else {
                            const uint32_t a_addr = ptx::smem_u32(ab + a * Cfg::kAbBytes + t * Cfg::kATileBytes);
                            ptx::umma_ss(d_tmem, ptx::smem_desc_k_major_sw128(a_addr + ks * 32), b_desc, idesc,
                                         accumulate);
                        }
                    }
                }
                ptx::umma_commit(&ab_empty[a]);
            }
            ptx::umma_commit(acc_full);
        }
    } else {
        // ------------------------------------------------------------------ dequant warps
        const int t = warp >> 2;                       // which tile (gate / up) this warp feeds
        const int r = ((warp & 3) << 5) | lane;        // weight row inside the tile == TMEM lane
        const int n = min(n0 + r, p.N - 1);            // rows past N were zero-filled by TMA
        const uint16_t* scale_row = p.scales[t] + (size_t)n * kblocks;
        const uint16_t* bias_row = p.biases[t] + (size_t)n * kblocks;
        const int tid = threadIdx.x;                   // 0 .. 128*kT-1
        uint32_t scale_next = 0, bias_next = 0;
        if (nkb > 0) {
            scale_next = __ldg(scale_row + kb_begin);
            bias_next = __ldg(bias_row + kb_begin);
        }
        for (int i = 0; i < nkb; ++i) {
            const int s = i % Cfg::kStages;
            const uint32_t phase = (i / Cfg::kStages) & 1;
            const uint32_t scale_bits = scale_next, bias_bits = bias_next;
            if (i + 1 < nkb) {
                scale_next = __ldg(scale_row + kb_begin + i + 1);
                bias_next = __ldg(bias_row + kb_begin + i + 1);
            }
            if (!ptx::mbar_wait(&ring_full[s], phase, abort_flag, kWaitRingFull)) break;
            __syncwarp();
            const uint8_t* stage = ring + s * Cfg::kStageBytes;
            const uint4* wsrc = reinterpret_cast<const uint4*>(stage + t * Cfg::kWTileBytes + r * 32);
            const uint4 w_lo = wsrc[0], w_hi = wsrc[1];
            // Activation tile: each thread moves kXTasks 16-byte chunks (8 consecutive k of one row).
            constexpr int kXTasks = (kMPad * 8 + Cfg::kDequantWarps * 32 - 1) / (Cfg::kDequantWarps * 32);
            uint4 xv[kXTasks];
#pragma unroll
            for (int j = 0; j < kXTasks; ++j) {
                const int task = tid + j * Cfg::kDequantWarps * 32;
                if (task < kMPad * 8)
                    xv[j] = *reinterpret_cast<const uint4*>(stage + Cfg::kWBytes + task * 16);
            }
            // The slot is about to be overwritten by TMA (async proxy) while it was just read with
            // ordinary loads (generic proxy): without this cross-proxy fence the refill was observed
            // to overtake the reads when the ring is only two slots deep.
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&ring_empty[s]);  // ring slot may be refilled

            const int a = i % Cfg::kAbStages;
            const uint32_t aphase = (i / Cfg::kAbStages) & 1;
            if (!ptx::mbar_wait(&ab_empty[a], aphase ^ 1, abort_flag, kWaitAbEmpty)) break;
            __syncwarp();  // the .sync.aligned tcgen05 instructions below need a converged warp
            ptx::tc_fence_after_sync();

            const __nv_bfloat162 scale2 = bits_bf162(scale_bits | (scale_bits << 16));
            const __nv_bfloat162 bias2 = bits_bf162(bias_bits | (bias_bits << 16));
            uint32_t wq[32];
            const uint32_t words[8] = {w_lo.x, w_lo.y, w_lo.z, w_lo.w, w_hi.x, w_hi.y, w_hi.z, w_hi.w};
#pragma unroll
            for (int c = 0; c < 8; ++c) dequant_word_bf16(words[c], scale2, bias2, &wq[4 * c]);

            uint8_t* ab_stage = ab + a * Cfg::kAbBytes;
            if constexpr (kTmemA) {
                const uint32_t a_tmem = tmem_base + ((uint32_t)((warp & 3) << 5) << 16) + Cfg::kAccCols +
                                        (a * kT + t) * 32;
                ptx::tmem_st16(a_tmem, &wq[0]);
                ptx::tmem_st16(a_tmem + 16, &wq[16]);
            } else {
                uint8_t* a_row = ab_stage + t * Cfg::kATileBytes + r * 128;
#pragma unroll
                for (int c = 0; c < 8; ++c)
                    *reinterpret_cast<uint4*>(a_row + ((c ^ (r & 7)) << 4)) =
                        make_uint4(wq[4 * c], wq[4 * c + 1], wq[4 * c + 2], wq[4 * c + 3]);
            }
            uint8_t* b_tile = ab_stage + Cfg::kABytes;
#pragma unroll
            for (int j = 0; j < kXTasks; ++j) {
                const int task = tid + j * Cfg::kDequantWarps * 32;
                if (task < kMPad * 8) {
                    const int row = task >> 3, c = task & 7;
                    uint4 o;
                    o.x = __byte_perm(xv[j].x, xv[j].z, 0x5410);  // (x0, x4)
                    o.y = __byte_perm(xv[j].x, xv[j].z, 0x7632);  // (x1, x5)
                    o.z = __byte_perm(xv[j].y, xv[j].w, 0x5410);  // (x2, x6)
                    o.w = __byte_perm(xv[j].y, xv[j].w, 0x7632);  // (x3, x7)
                    *reinterpret_cast<uint4*>(b_tile + row * 128 + ((c ^ (row & 7)) << 4)) = o;
                }
            }
            ptx::fence_proxy_async_smem();
            if constexpr (kTmemA) {
                ptx::tc_wait_st();
                ptx::tc_fence_before_sync();
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&ab_full[a]);
        }

        // -------------------------------------------------------------- accumulators -> smem
        // Lanes can leave a polling loop, or the lane-0 arrive above, at different times; the
        // aligned TMEM loads need every lane of the warp together, with one verdict.
        __syncwarp();
        const bool ok = __all_sync(0xFFFFFFFFu, nkb > 0 && ptx::mbar_wait(acc_full, 0, abort_flag, kWaitAccFull));
        ptx::tc_fence_after_sync();
        float* staging = reinterpret_cast<float*>(smem);
#pragma unroll
        for (int c0 = 0; c0 < kMPad; c0 += 16) {
            uint32_t v[16];
            if (ok) {
                ptx::tmem_ld16(tmem_base + ((uint32_t)((warp & 3) << 5) << 16) + t * kMPad + c0, v);
                ptx::tc_wait_ld();
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = 0u;
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) staging[(t * kMPad + c0 + j) * kUmmaTileRows + r] = __uint_as_float(v[j]);
        }
    }

    // ---------------------------------------------------------------------- reduce + store
    __syncwarp();
    ptx::tc_fence_before_sync();
    if (ksplit > 1) {
        ptx::cluster_arrive();
        ptx::cluster_wait();
    } else {
        __syncthreads();
    }
    if (warp < Cfg::kDequantWarps) {
        const int r = threadIdx.x & 127;
        const int group = threadIdx.x >> 7;        // kT groups of 128 threads
        const int n = n0 + r;
        const uint32_t staging_addr = ptx::smem_u32(smem);
        for (int m = rank + ksplit * group; m < p.M; m += ksplit * kT) {
            float first = 0.0f, second = 0.0f;
            if (ksplit > 1) {
                for (int j = 0; j < ksplit; ++j) {
                    const uint32_t peer = ptx::map_to_cta(staging_addr, (uint32_t)j);
                    first += ptx::ld_cluster_f32(peer + 4u * (uint32_t)(m * kUmmaTileRows + r));
                    if constexpr (kSwiglu)
                        second += ptx::ld_cluster_f32(peer + 4u * (uint32_t)((kMPad + m) * kUmmaTileRows + r));
                }
            } else {
                const float* staging = reinterpret_cast<const float*>(smem);
                first = staging[m * kUmmaTileRows + r];
                if constexpr (kSwiglu) second = staging[(kMPad + m) * kUmmaTileRows + r];
            }
            if (n < p.N) {
                float v = kSwiglu ? swiglu_f32(first, second) : first;
                if (!kSwiglu && p.residual) v += bf16_bits_to_f32(p.residual[(size_t)m * p.N + n]);
                p.out[(size_t)m * p.N + n] = f32_to_bf16_bits(v);
            }
        }
    }
    __syncwarp();
    if (ksplit > 1) {
        ptx::cluster_arrive();
        ptx::cluster_wait();
    } else {
        __syncthreads();
    }
    if (warp == Cfg::kMmaWarp) {
        __syncwarp();
        ptx::tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// ------------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult result;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) != cudaSuccess ||
            result != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(ptr);
    }();
    return fn;
}

inline bool encode_2d(CUtensorMap* map, CUtensorMapDataType type, int elem_bytes, const void* base, uint64_t inner,
                      uint64_t outer, uint64_t row_bytes, uint32_t box_inner, uint32_t box_outer) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t elem_strides[2] = {1, 1};
    (void)elem_bytes;
    return fn(map, type, 2, const_cast<void*>(base), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Cluster size along K: fill the SMs when there are few 128-row tiles.  Function of the tile
// count and K only.
inline int umma_ksplit(int tiles, int kblocks, int sm_count) {
    int best = 1;
    double best_score = -1.0;
    for (int s = 1; s <= 8; s *= 2) {
        if (s > 1 && kblocks / s < 4) break;
        const long ctas = (long)tiles * s;
        const long waves = (ctas + sm_count - 1) / sm_count;
        const double score = (double)ctas / (double)(waves * sm_count) - 0.01 * (s - 1);
        if (score > best_score + 1e-9) {
            best_score = score;
            best = s;
        }
    }
    return best;
}

template <int kT, int kMPad, bool kTmemA, bool kSwiglu>
inline int launch_umma_instance(const UmmaParams& params, int tiles, cudaStream_t stream) {
    using Cfg = UmmaConfig<kT, kMPad, kTmemA>;
    auto kernel = affine_umma_kernel<kT, kMPad, kTmemA, kSwiglu>;
    static bool configured[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (device < 64 && !configured[device]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess)
            return MT_ERR_LAUNCH;
        configured[device] = true;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(tiles * params.ksplit, 1, 1);
    config.blockDim = dim3(Cfg::kThreads, 1, 1);
    config.dynamicSmemBytes = Cfg::kSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = params.ksplit;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    config.attrs = attrs;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, kernel, params) == cudaSuccess ? MT_OK : MT_ERR_LAUNCH;
}

template <int kT, bool kTmemA, bool kSwiglu>
inline int launch_umma_mpad(const UmmaParams& params, int tiles, int mpad, cudaStream_t stream) {
    switch (mpad) {
        case 16: return launch_umma_instance<kT, 16, kTmemA, kSwiglu>(params, tiles, stream);
        case 32: return launch_umma_instance<kT, 32, kTmemA, kSwiglu>(params, tiles, stream);
        case 64: return launch_umma_instance<kT, 64, kTmemA, kSwiglu>(params, tiles, stream);
        case 128: return launch_umma_instance<kT, 128, kTmemA, kSwiglu>(params, tiles, stream);
        default: return MT_ERR_SHAPE;
    }
}

struct AffineWeights {
    const uint32_t* w;
    const uint16_t* scales;
    const uint16_t* biases;
};

// x [M,K] bf16 (M <= 128), one weight triple (plain / residual) or two (gate, up -> SwiGLU).
inline int launch_umma(const void* x, const AffineWeights* first, const AffineWeights* second, const void* residual,
                       void* out, int M, int K, int N, bool tmem_a, int sm_count, cudaStream_t stream) {
    if (M < 1 || M > 128 || K % kUmmaBlockK || K < kUmmaBlockK || N < 1) return MT_ERR_SHAPE;
    if (!aligned_to(x, 16) || !aligned_to(first->w, 16) || (second && !aligned_to(second->w, 16))) return MT_ERR_ALIGN;
    const bool swiglu = second != nullptr;
    const int mpad = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
    const int tiles = (N + kUmmaTileRows - 1) / kUmmaTileRows;
    UmmaParams params;
    params.scales[0] = first->scales;
    params.biases[0] = first->biases;
    params.scales[1] = swiglu ? second->scales : first->scales;
    params.biases[1] = swiglu ? second->biases : first->biases;
    params.residual = static_cast<const uint16_t*>(residual);
    params.out = static_cast<uint16_t*>(out);
    params.M = M;
    params.K = K;
    params.N = N;
    params.ksplit = umma_ksplit(tiles, K / kUmmaBlockK, sm_count);
    const uint64_t row_bytes = (uint64_t)K / 2;
    if (!encode_2d(&params.w_map[0], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, first->w, (uint64_t)K / 8, (uint64_t)N,
                   row_bytes, 8, kUmmaTileRows))
        return MT_ERR_LAUNCH;
    if (!encode_2d(&params.w_map[1], CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, swiglu ? second->w : first->w,
                   (uint64_t)K / 8, (uint64_t)N, row_bytes, 8, kUmmaTileRows))
        return MT_ERR_LAUNCH;
    if (!encode_2d(&params.x_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, x, (uint64_t)K, (uint64_t)M, (uint64_t)K * 2,
                   kUmmaBlockK, (uint32_t)mpad))
        return MT_ERR_LAUNCH;
    if (swiglu) {
        return tmem_a ? launch_umma_mpad<2, true, true>(params, tiles, mpad, stream)
                      : launch_umma_mpad<2, false, true>(params, tiles, mpad, stream);
    }
    return tmem_a ? launch_umma_mpad<1, true, false>(params, tiles, mpad, stream)
                  : launch_umma_mpad<1, false, false>(params, tiles, mpad, stream);
}

}  // namespace mt
