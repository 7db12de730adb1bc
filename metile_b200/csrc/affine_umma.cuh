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
//   producer lane  : TMA (per-CTA tiled load, 128B swizzle) packed weight tile(s) of
//                    128 rows x 128 B = four k-blocks per ring slot; boxes with a 32-byte inner
//                    extent were measured to be limited by the TMA request rate, not by HBM
//   dequant warps  : 16 warps in groups of four (one group = the 128 rows of one tile); with kT
//                    tiles per CTA there are kDepth = 4/kT groups per tile and group d handles the
//                    k-blocks i = d, d+kDepth, ... so several k-blocks are in flight per SM.
//                    One thread per weight row; nibbles -> bf16x2 in NATURAL element order (pairs
//                    (e0,e1), (e2,e3), ...: two masks, one byte-permute and one or-with-0x4300 per
//                    pair = 128+q), q = v-128, w = fma(q, scale, bias) (one rounding:
//                    RN_bf16(scale*q+bias)); result stored to tensor memory as the A operand
//   x lane         : the activation tile of each k-block ([kMPad rows] x 64 columns, rows past M
//                    zero-filled) arrives by TMA straight into the swizzled B tile: no thread touches
//                    the activations, whose handling cost as many instructions as the dequantisation
//                    at 128 rows when every dequant thread did a share of it
//   MMA lanes      : two threads issue tcgen05.mma kind::f16 (bf16 x bf16 -> fp32 in TMEM) and
//                    tcgen05.commit, one per tile (gate / up) or per k-block parity (single tile)
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
constexpr int kUmmaBlockK = 64;      // one quantisation group per MMA pipeline step
constexpr int kUmmaKBlocksPerSlot = 4;  // a ring slot holds 4 k-blocks: 128 B of packed nibbles per row

constexpr int pow2_at_least(int v) {
    int p = 32;
    while (p < v) p *= 2;
    return p;
}

template <int kT, int kMPad>
struct UmmaConfig {
    // One footprint: 16 dequant warps, one CTA per SM.  A lighter variant (8 dequant warps, two
    // CTAs per SM so that consecutive kernels chained by programmatic dependent launch overlap)
    // was measured and was slower (16.2 vs 12.7 us for the 2048->8192 gate|up projection at one
    // row): what limits a CTA is the latency of one warp's dequant iteration, so halving the
    // warps per CTA doubled it and the overlap did not pay that back.  Staging the dequantised A
    // tile in shared memory instead of tensor memory was measured too and never won.
    static constexpr int kDequantWarps = 16;                        // 4 warps x kT tiles x kDepth
    static constexpr int kDepth = kDequantWarps / (4 * kT);         // dequant groups per tile
    static constexpr int kWarpsPerKBlock = 4 * kT;                  // warps that serve one k-block
    static constexpr int kProducerWarp = kDequantWarps;
    static constexpr int kMmaWarp = kDequantWarps + 1;
    static constexpr int kXWarp = kDequantWarps + 2;
    static constexpr int kMmaWarp2 = kDequantWarps + 3;
    static constexpr int kThreads = (kDequantWarps + 4) * 32;
    static constexpr int kWTileBytes = kUmmaTileRows * 128;         // one packed tile, four k-blocks
    static constexpr int kSlotBytes = kT * kWTileBytes;
    static constexpr int kBBytes = kMPad * 128;                     // activation tile of one k-block
    // A hand-off between the dequant warps and the MMA issuers covers kPair k-blocks: the waits,
    // fences and arrivals of a hand-off cost about as many instructions as dequantising one k-block, so
    // sharing them between two k-blocks shortens the instruction stream that bounds the kernel.
    static constexpr int kPair = 2;
    static constexpr int kPairsPerSlot = kUmmaKBlocksPerSlot / kPair;
    static constexpr int kAbBytes = kPair * kBBytes;                // activation bytes per stage in shared memory (A lives in tensor memory)
    // One operand stage per depth group.  A ring of activation tiles of its own, eight k-blocks ahead
    // of the A stages, was measured and was slower (617 against 559 cycles per k-block at 16 rows): the
    // extra wait and commit per k-block in the issuing threads cost more than the earlier request saved.
    static constexpr int kAbStages = kDepth;
    static constexpr int kRingReaders = kT == 2 ? kDequantWarps : kDequantWarps / 2;  // warps that read one ring slot
    // Two threads (in two warps) issue the MMAs.  One issuer's loop per k-block -- poll the operand
    // barrier (~140 cycles even when it is already complete), four MMAs whose issue blocks while the
    // pipe is busy, commit -- measured 566 cycles per k-block at 16 rows, more than twice what the
    // tensor pipe needs for the four MMAs (45-67 cycles each), so the issuers alternate.  With two
    // tiles per CTA each issuer owns one tile (gate / up) and its accumulator; with one tile the
    // issuers take the even and the odd k-blocks and accumulate into two accumulators that the
    // epilogue adds (even + odd), an order that depends on K only.
    static constexpr int kAcc = kT == 1 ? 2 : 1;
    static constexpr int kAccCols = kT * kAcc * kMPad;
    static constexpr int kATmemCols = kAbStages * kT * kPair * 32;
    static constexpr int kTmemCols = pow2_at_least(kAccCols + kATmemCols);
    // The ring takes what shared memory the footprint leaves, up to 8 slots.
    static constexpr int kBudgetBytes = 196 * 1024;
    static constexpr int kRingTarget = kBudgetBytes - kAbStages * kAbBytes;
    static constexpr int kStagesRaw = kRingTarget / kSlotBytes;
    static constexpr int kStages = kStagesRaw < 2 ? 2 : (kStagesRaw > 8 ? 8 : kStagesRaw);
    static constexpr int kRingBytes = kStages * kSlotBytes;
    static constexpr int kStagingBytes = kT * kMPad * kUmmaTileRows * 4;
    static constexpr int kDataBytesRaw = kRingBytes + kAbStages * kAbBytes;
    static constexpr int kDataBytesMin = kDataBytesRaw > kStagingBytes ? kDataBytesRaw : kStagingBytes;
    // TMEM columns x resident CTAs must never exceed 512: a later CTA's tcgen05.alloc would wait
    // for an earlier CTA to finish.  Shared memory bounds residency, so every CTA asks for more
    // than 1/(allowed+1) of an SM's shared memory.
    static constexpr int kAllowedPerSm = 1;
    static constexpr int kFloorBytes = (227 * 1024) / (kAllowedPerSm + 1) + 2048;
    static constexpr int kDataBytes = kDataBytesMin < kFloorBytes ? kFloorBytes : kDataBytesMin;
    static constexpr int kBarrierBytes = 8 * (2 * kStages + 2 * kAbStages + 1) + 16;
    static constexpr int kSmemBytes = 1024 + kDataBytes + kBarrierBytes;
    static_assert(kTmemCols <= 512, "tensor memory budget");
    static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
    static_assert(kSlotBytes % 1024 == 0 && kAbBytes % 1024 == 0, "1024 B alignment");
    static_assert((kAllowedPerSm + 1) * kSmemBytes > 227 * 1024, "one CTA too many would fit on an SM");
    static_assert(kAllowedPerSm * (kSmemBytes + 1024) <= 227 * 1024, "the intended residency does not fit");
    static_assert(kAllowedPerSm * kTmemCols <= 512, "tensor memory over-subscribed");
    static_assert(kAbStages == kDepth, "each depth group owns one operand stage");
    static_assert(kDepth % kPairsPerSlot == 0, "a group sees the same pair of k-blocks in every slot it reads");
};

struct UmmaParams {
    CUtensorMap w_map[2];  // packed weights, uint32 [N, K/8], box {32, 128}, 128B swizzle
    CUtensorMap x_map;     // activations, bf16 [M, K], box {64, padded rows}, 128B swizzle (the B tile of a k-block)
    const uint16_t* x;     // activations, bf16 [M, K]
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

// One packed word (8 nibbles) -> 8 bf16 weights in natural order: out[i] = (w_{2i}, w_{2i+1}).
__device__ __forceinline__ void dequant_word_bf16(uint32_t w, __nv_bfloat162 scale2, __nv_bfloat162 bias2,
                                                  uint32_t* out) {
    const __nv_bfloat162 k128 = bits_bf162(0x43004300u);
    const uint32_t even = w & 0x0F0F0F0Fu;         // bytes e0, e2, e4, e6
    const uint32_t odd = (w >> 4) & 0x0F0F0F0Fu;   // bytes e1, e3, e5, e7
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        // bytes (e_2i, ., e_2i+1, .), then (x & 0x00FF00FF) | 0x43004300 as ONE lop3 (truth table 0xEA):
        // the bf16 pair (128 + e_2i, 128 + e_2i+1).
        const uint32_t pair = __byte_perm(even, odd, (uint32_t)(i | (i << 4) | ((4 + i) << 8) | ((4 + i) << 12)));
        uint32_t v;
        asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v) : "r"(pair), "r"(0x00FF00FFu), "r"(0x43004300u));
        const __nv_bfloat162 q = __hsub2(bits_bf162(v), k128);            // exact: integers 0..15
        out[i] = bf162_bits(__hfma2(q, scale2, bias2));                   // RN_bf16(scale*q + bias)
    }
}

// volatile: a plain __ldg may be sunk by the compiler to its first use, which would turn the
// one-iteration-ahead prefetch of scales and biases into a load on the critical path.
__device__ __forceinline__ uint32_t ldg_nc_u16(const uint16_t* p) {
    uint16_t v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ uint4 ldg_nc_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// The loop of one of the two MMA-issuing threads.  kIssuer picks the tile (two tiles per CTA) or the
// parity of the k-blocks (one tile).  The thread's loop is kept to a few instructions per MMA: the
// operand descriptor of byte 0 of the operand area is built once and every other descriptor is that
// value plus a compile-time offset (the start-address field counts 16-byte units and never carries
// out of its 14 bits), and the loop over k-blocks is unrolled by the number of operand stages so that
// stage indices are constants.
template <int kT, int kMPad, int kIssuer>
__device__ __forceinline__ void umma_issue(uint32_t tmem_base, const uint8_t* ab, uint64_t* ab_full, uint64_t* ab_empty,
                                           uint64_t* acc_full, volatile int* abort_flag, int nkb) {
    using Cfg = UmmaConfig<kT, kMPad>;
    constexpr uint32_t idesc = ptx::umma_idesc_bf16(kUmmaTileRows, kMPad);
    constexpr int t = kT == 2 ? kIssuer : 0;          // the tile this thread accumulates
    constexpr int chain = kT == 2 ? 0 : kIssuer;      // its accumulator within the tile
    const uint32_t d_tmem = tmem_base + (t * Cfg::kAcc + chain) * kMPad;
    const uint64_t desc0 = ptx::smem_desc_k_major_sw128(ptx::smem_u32(ab));
    const int npairs = (nkb + Cfg::kPair - 1) / Cfg::kPair;
    for (int p0 = 0; p0 < npairs; p0 += Cfg::kAbStages) {
        const uint32_t phase = (p0 / Cfg::kAbStages) & 1;
        const uint32_t later = p0 > 0 ? 1u : 0u;
#pragma unroll
        for (int a = 0; a < Cfg::kAbStages; ++a) {
            if (kT == 1 && (a & 1) != kIssuer) continue;
            const int pair = p0 + a;
            if (pair >= npairs) break;
            if (!ptx::mbar_wait_spin(&ab_full[a], phase, abort_flag, kWaitAbFull)) { p0 = npairs; break; }
            ptx::tc_fence_after_sync();
            const int valid = nkb - pair * Cfg::kPair;  // k-blocks of this pair in range: 1 only at a ragged end
#pragma unroll
            for (int kb = 0; kb < Cfg::kPair; ++kb) {
                if (kb >= valid) break;
#pragma unroll
                for (int ks = 0; ks < kUmmaBlockK / 16; ++ks) {
                    const uint64_t b_desc = desc0 + (uint64_t)((a * Cfg::kAbBytes + kb * Cfg::kBBytes + ks * 32) >> 4);
                    // The first MMA into an accumulator overwrites it.
                    const uint32_t accumulate = (kb > 0 || ks > 0 || a > (kT == 1 ? kIssuer : 0)) ? 1u : later;
                    const uint32_t a_tmem = tmem_base + Cfg::kAccCols + ((a * kT + t) * Cfg::kPair + kb) * 32 + ks * 8;
                    ptx::umma_ts(d_tmem, a_tmem, b_desc, idesc, accumulate);
                }
            }
            ptx::umma_commit(&ab_empty[a]);
        }
    }
    ptx::umma_commit(acc_full);
}

template <int kT, int kMPad, bool kSwiglu>
__global__ void __launch_bounds__(UmmaConfig<kT, kMPad>::kThreads, UmmaConfig<kT, kMPad>::kAllowedPerSm)
affine_umma_kernel(const __grid_constant__ UmmaParams p) {
    using Cfg = UmmaConfig<kT, kMPad>;
    static_assert(!kSwiglu || kT == 2, "SwiGLU pairs a gate tile with an up tile");
    extern __shared__ uint8_t smem_raw[];
    // Aligned by offsetting the array itself (not by rounding a generic address), so that the compiler
    // still knows these are shared-memory addresses and emits shared loads and stores.
    uint8_t* smem = smem_raw + ((1024u - (ptx::smem_u32(smem_raw) & 1023u)) & 1023u);
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
    // The K range is cut between the CTAs of a cluster in whole ring slots (4 k-blocks).
    const int slots_total = (kblocks + kUmmaKBlocksPerSlot - 1) / kUmmaKBlocksPerSlot;
    const int slot_begin = (int)(((long long)slots_total * rank) / ksplit);
    const int slot_end = (int)(((long long)slots_total * (rank + 1)) / ksplit);
    const int nslots = slot_end - slot_begin;
    const int kb_begin = slot_begin * kUmmaKBlocksPerSlot;
    const int kb_end = min(slot_end * kUmmaKBlocksPerSlot, kblocks);
    const int nkb = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        for (int i = 0; i < Cfg::kStages; ++i) {
            ptx::mbar_init(&ring_full[i], 1);
            ptx::mbar_init(&ring_empty[i], Cfg::kRingReaders);
        }
        for (int i = 0; i < Cfg::kAbStages; ++i) {
            ptx::mbar_init(&ab_full[i], Cfg::kWarpsPerKBlock + 1);  // dequant warps + the activation tile's copy
            ptx::mbar_init(&ab_empty[i], kT == 2 ? 2 : 1);  // two tiles: both issuers read the stage
        }
        ptx::mbar_init(acc_full, 2);
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
    // Programmatic dependent launch: the next kernel of the stream may begin its own set-up and
    // weight prefetch while this one is still running.  Only the weights (which no kernel writes)
    // are touched before griddep_wait(); activations, residual and outputs come after it.
    ptx::griddep_launch_dependents();

    if (warp == Cfg::kProducerWarp) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            ptx::prefetch_tensor_map(&p.w_map[0]);
            if (kT == 2) ptx::prefetch_tensor_map(&p.w_map[1]);
            int issued = 0;
            for (int st = 0; st < nslots; ++st) {
                const int s = st % Cfg::kStages;
                const uint32_t phase = (st / Cfg::kStages) & 1;
                if (!ptx::mbar_wait(&ring_empty[s], phase ^ 1, abort_flag, kWaitRingEmpty)) break;
                ptx::mbar_expect_tx(&ring_full[s], Cfg::kSlotBytes);
                uint8_t* slot = ring + s * Cfg::kSlotBytes;
#pragma unroll
                for (int t = 0; t < kT; ++t)
                    ptx::tma_load_2d(slot + t * Cfg::kWTileBytes, &p.w_map[t], (slot_begin + st) * 32, n0,
                                     &ring_full[s]);
                ++issued;
            }
            if (*abort_flag) {
                // Let copies already in flight land before the CTA may exit.
                const int first = issued > Cfg::kStages ? issued - Cfg::kStages : 0;
                for (int st = first; st < issued; ++st)
                    ptx::mbar_wait(&ring_full[st % Cfg::kStages], (st / Cfg::kStages) & 1, abort_flag, kWaitDrain);
            }
        }
    } else if (warp == Cfg::kXWarp) {
        // ------------------------------------------------------------------ activation tiles by TMA
        if (lane == 0) {
            ptx::prefetch_tensor_map(&p.x_map);
            ptx::griddep_wait();  // the activations are the preceding kernel's output
            int issued = 0;
            const int npairs = (nkb + Cfg::kPair - 1) / Cfg::kPair;
            for (int pair = 0; pair < npairs; ++pair) {
                const int a = pair % Cfg::kAbStages;
                const uint32_t phase = (uint32_t)(pair / Cfg::kAbStages) & 1u;
                if (!ptx::mbar_wait(&ab_empty[a], phase ^ 1u, abort_flag, kWaitAbEmpty)) break;
                const int valid = min(Cfg::kPair, nkb - pair * Cfg::kPair);
                ptx::mbar_expect_tx(&ab_full[a], (uint32_t)valid * Cfg::kBBytes);
                for (int kb = 0; kb < valid; ++kb)
                    ptx::tma_load_2d(ab + a * Cfg::kAbBytes + kb * Cfg::kBBytes, &p.x_map,
                                     (kb_begin + pair * Cfg::kPair + kb) * kUmmaBlockK, 0, &ab_full[a]);
                ++issued;
            }
            if (*abort_flag) {
                // Copies in flight complete their barrier's transaction count; nothing else waits for
                // them, so let them land before the CTA may exit.
                const unsigned long long start = ptx::global_timer_ns();
                while (issued > 0 && ptx::global_timer_ns() - start < 200000ull) {}
            }
        }
    } else if (warp == Cfg::kMmaWarp) {
        // ------------------------------------------------------------------ MMA issuers
        if (lane == 0) umma_issue<kT, kMPad, 0>(tmem_base, ab, ab_full, ab_empty, acc_full, abort_flag, nkb);
    } else if (warp == Cfg::kMmaWarp2) {
        if (lane == 0) umma_issue<kT, kMPad, 1>(tmem_base, ab, ab_full, ab_empty, acc_full, abort_flag, nkb);
    } else {
        // ------------------------------------------------------------------ dequant warps
        const int group = warp >> 2;                   // four warps = one group = 128 rows
        const int t = kT == 2 ? (group & 1) : 0;       // which tile (gate / up) this group feeds
        const int depth = kT == 2 ? (group >> 1) : group;  // which k-blocks: i = depth, depth+kDepth, ...
        const int r = ((warp & 3) << 5) | lane;        // weight row inside the tile == TMEM lane
        const int n = min(n0 + r, p.N - 1);            // rows past N were zero-filled by TMA
        const uint16_t* scale_row = p.scales[t] + (size_t)n * kblocks + kb_begin;
        const uint16_t* bias_row = p.biases[t] + (size_t)n * kblocks + kb_begin;
        // This group's share: pair `pair_in_slot` of every `slot_step`-th ring slot, always into operand
        // stage `depth`; its n-th hand-off uses phase n & 1 of that stage's barriers.
        constexpr int kSlotStep = Cfg::kDepth / Cfg::kPairsPerSlot;
        const int pair_in_slot = depth % Cfg::kPairsPerSlot;
        const int slot_first = depth / Cfg::kPairsPerSlot;
        const int a = depth;
        uint32_t scale_next[Cfg::kPair], bias_next[Cfg::kPair];
#pragma unroll
        for (int kb = 0; kb < Cfg::kPair; ++kb) {
            const int i = slot_first * kUmmaKBlocksPerSlot + pair_in_slot * Cfg::kPair + kb;
            scale_next[kb] = i < nkb ? ldg_nc_u16(scale_row + i) : 0u;
            bias_next[kb] = i < nkb ? ldg_nc_u16(bias_row + i) : 0u;
        }
        uint32_t use = 0;
        for (int st = slot_first; st < nslots; st += kSlotStep, ++use) {
            const int s = st % Cfg::kStages;
            const uint32_t phase = (st / Cfg::kStages) & 1;
            const uint8_t* slot = ring + s * Cfg::kSlotBytes;
            const int i0 = st * kUmmaKBlocksPerSlot + pair_in_slot * Cfg::kPair;  // first k-block of the pair
            uint32_t scale_bits[Cfg::kPair], bias_bits[Cfg::kPair];
#pragma unroll
            for (int kb = 0; kb < Cfg::kPair; ++kb) {
                scale_bits[kb] = scale_next[kb];
                bias_bits[kb] = bias_next[kb];
                const int following = i0 + kSlotStep * kUmmaKBlocksPerSlot + kb;
                if (following < nkb) {
                    scale_next[kb] = ldg_nc_u16(scale_row + following);
                    bias_next[kb] = ldg_nc_u16(bias_row + following);
                }
            }
            if (!ptx::mbar_wait(&ring_full[s], phase, abort_flag, kWaitRingFull)) break;
            if (i0 < nkb) {
                if (!ptx::mbar_wait(&ab_empty[a], (use & 1u) ^ 1u, abort_flag, kWaitAbEmpty)) break;
                __syncwarp();  // the .sync.aligned tcgen05 instructions below need a converged warp
                ptx::tc_fence_after_sync();
                const uint8_t* wrow = slot + t * Cfg::kWTileBytes + r * 128;
#pragma unroll
                for (int kb = 0; kb < Cfg::kPair; ++kb) {
                    if (i0 + kb >= nkb) break;  // ragged end: the pair holds one k-block
                    // 32 B of this row for k-block j: 16-byte chunks 2j and 2j+1, XOR-swizzled by the row.
                    const int j = pair_in_slot * Cfg::kPair + kb;
                    const uint4 w_lo = *reinterpret_cast<const uint4*>(wrow + (((2 * j) ^ (r & 7)) << 4));
                    const uint4 w_hi = *reinterpret_cast<const uint4*>(wrow + (((2 * j + 1) ^ (r & 7)) << 4));
                    const __nv_bfloat162 scale2 = bits_bf162(scale_bits[kb] | (scale_bits[kb] << 16));
                    const __nv_bfloat162 bias2 = bits_bf162(bias_bits[kb] | (bias_bits[kb] << 16));
                    uint32_t wq[32];
                    const uint32_t words[8] = {w_lo.x, w_lo.y, w_lo.z, w_lo.w, w_hi.x, w_hi.y, w_hi.z, w_hi.w};
#pragma unroll
                    for (int c = 0; c < 8; ++c) dequant_word_bf16(words[c], scale2, bias2, &wq[4 * c]);
                    const uint32_t a_tmem = tmem_base + ((uint32_t)((warp & 3) << 5) << 16) + Cfg::kAccCols +
                                            ((a * kT + t) * Cfg::kPair + kb) * 32;
                    ptx::tmem_st16(a_tmem, &wq[0]);
                    ptx::tmem_st16(a_tmem + 16, &wq[16]);
                }
                // The ring slot read above with ordinary loads may later be overwritten by TMA (async
                // proxy): order the two.  Releasing a slot without such a fence was observed to let the
                // refill overtake the reads.
                ptx::fence_proxy_async_smem();
                ptx::tc_wait_st();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&ab_full[a]);
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&ring_empty[s]);
        }

        // -------------------------------------------------------------- accumulators -> smem
        // Lanes can leave a polling loop, or a lane-0 arrive above, at different times; the
        // aligned TMEM loads need every lane of the warp together, with one verdict.
        __syncwarp();
        if (depth == 0) {
            const bool ok =
                __all_sync(0xFFFFFFFFu, nkb > 0 && ptx::mbar_wait(acc_full, 0, abort_flag, kWaitAccFull));
            ptx::tc_fence_after_sync();
            float* staging = reinterpret_cast<float*>(smem);
#pragma unroll
            for (int c0 = 0; c0 < kMPad; c0 += 16) {
                float v[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] = 0.0f;
                if (ok) {
#pragma unroll
                    for (int chain = 0; chain < Cfg::kAcc; ++chain) {
                        if (chain > 0 && nkb <= Cfg::kPair) break;  // the odd pairs' accumulator was never written
                        uint32_t part[16];
                        ptx::tmem_ld16(tmem_base + ((uint32_t)((warp & 3) << 5) << 16) +
                                           (t * Cfg::kAcc + chain) * kMPad + c0, part);
                        ptx::tc_wait_ld();
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            v[j] = chain == 0 ? __uint_as_float(part[j]) : v[j] + __uint_as_float(part[j]);
                    }
                }
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    if (c0 + j < p.M) staging[(t * kMPad + c0 + j) * kUmmaTileRows + r] = v[j];
            }
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
        const int part = threadIdx.x >> 7;         // groups of 128 threads share the rows
        constexpr int kParts = Cfg::kDequantWarps / 4;
        const int n = n0 + r;
        const uint32_t staging_addr = ptx::smem_u32(smem);
        // Four rows per trip so that the remote loads of a trip are all in flight together; the
        // partials of one output are still added in rank order.
        constexpr int kUnroll = 4;
        const int stride = ksplit * kParts;
        for (int m0 = rank + ksplit * part; m0 < p.M; m0 += stride * kUnroll) {
            float first[kUnroll], second[kUnroll], extra[kUnroll];
#pragma unroll
            for (int u = 0; u < kUnroll; ++u) {
                first[u] = 0.0f;
                second[u] = 0.0f;
                extra[u] = 0.0f;
            }
            if (ksplit > 1) {
                for (int j = 0; j < ksplit; ++j) {
                    const uint32_t peer = ptx::map_to_cta(staging_addr, (uint32_t)j);
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) {
                        const int m = m0 + u * stride;
                        if (m < p.M) {
                            first[u] += ptx::ld_cluster_f32(peer + 4u * (uint32_t)(m * kUmmaTileRows + r));
                            if constexpr (kSwiglu)
                                second[u] += ptx::ld_cluster_f32(peer + 4u * (uint32_t)((kMPad + m) * kUmmaTileRows + r));
                        }
                    }
                }
            } else {
                const float* staging = reinterpret_cast<const float*>(smem);
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    const int m = m0 + u * stride;
                    if (m < p.M) {
                        first[u] = staging[m * kUmmaTileRows + r];
                        if constexpr (kSwiglu) second[u] = staging[(kMPad + m) * kUmmaTileRows + r];
                    }
                }
            }
            if (n < p.N) {
                if (!kSwiglu && p.residual) {
#pragma unroll
                    for (int u = 0; u < kUnroll; ++u) {
                        const int m = m0 + u * stride;
                        if (m < p.M)
                            extra[u] = bf16_bits_to_f32(ptx::ld_global_dependent_u16(p.residual + (size_t)m * p.N + n));
                    }
                }
#pragma unroll
                for (int u = 0; u < kUnroll; ++u) {
                    const int m = m0 + u * stride;
                    if (m < p.M) {
                        const float v = kSwiglu ? swiglu_f32(first[u], second[u]) : first[u] + extra[u];
                        p.out[(size_t)m * p.N + n] = f32_to_bf16_bits(v);
                    }
                }
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

// Packed weights as a 2-D uint32 tensor [N, K/8]; box = 32 words (128 B, four k-blocks) x 128 rows,
// 128-byte swizzle so that a thread reading "its" row's 32 bytes hits distinct banks.
// Activations as a 2-D bf16 tensor [M, K]; box = 64 columns (128 B, one k-block) x the padded row
// count, 128-byte swizzle: the box is the B tile of one k-block, rows past M read as zero.
// A tensor map is a pure function of (address, extents, box): encoding one costs a microsecond or
// two of host time and a two-kernel MLP needs five, so each host thread remembers the last few it built
// (weights never move, executors reuse their activation buffers).  Direct-mapped, 64 entries.
struct TensorMapKey {
    const void* base;
    int a, b, box_rows, kind;
    bool operator==(const TensorMapKey& o) const {
        return base == o.base && a == o.a && b == o.b && box_rows == o.box_rows && kind == o.kind;
    }
};
struct TensorMapSlot {
    TensorMapKey key;
    CUtensorMap map;
    bool valid;
};
inline TensorMapSlot& tensor_map_slot(const TensorMapKey& key) {
    thread_local TensorMapSlot slots[64] = {};
    const uintptr_t bits = reinterpret_cast<uintptr_t>(key.base) >> 8;
    const size_t index = (size_t)((bits ^ (bits >> 7) ^ (uintptr_t)(key.a * 31 + key.b * 7 + key.box_rows + key.kind * 13)) & 63u);
    return slots[index];
}

inline bool encode_activation_map_uncached(CUtensorMap* map, const void* base, int M, int K, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    cuuint32_t box[2] = {(cuuint32_t)kUmmaBlockK, (cuuint32_t)box_rows};
    cuuint32_t elem_strides[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

inline bool encode_weight_map_uncached(CUtensorMap* map, const void* base, int K, int N, int box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K / 8, (cuuint64_t)N};
    cuuint64_t strides[1] = {(cuuint64_t)K / 2};
    cuuint32_t box[2] = {32, (cuuint32_t)box_rows};
    cuuint32_t elem_strides[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, elem_strides,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

inline bool encode_activation_map(CUtensorMap* map, const void* base, int M, int K, int box_rows) {
    const TensorMapKey key{base, M, K, box_rows, 1};
    TensorMapSlot& slot = tensor_map_slot(key);
    if (!(slot.valid && slot.key == key)) {
        if (!encode_activation_map_uncached(&slot.map, base, M, K, box_rows)) {
            slot.valid = false;
            return false;
        }
        slot.key = key;
        slot.valid = true;
    }
    *map = slot.map;
    return true;
}

inline bool encode_weight_map(CUtensorMap* map, const void* base, int K, int N, int box_rows = kUmmaTileRows) {
    const TensorMapKey key{base, K, N, box_rows, 2};
    TensorMapSlot& slot = tensor_map_slot(key);
    if (!(slot.valid && slot.key == key)) {
        if (!encode_weight_map_uncached(&slot.map, base, K, N, box_rows)) {
            slot.valid = false;
            return false;
        }
        slot.key = key;
        slot.valid = true;
    }
    *map = slot.map;
    return true;
}

template <int kT, int kMPad, bool kSwiglu>
inline cudaError_t configure_umma_instance() {
    using Cfg = UmmaConfig<kT, kMPad>;
    static bool configured[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (device < 64 && configured[device]) return cudaSuccess;
    const cudaError_t rc = cudaFuncSetAttribute(affine_umma_kernel<kT, kMPad, kSwiglu>,
                                                cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (rc == cudaSuccess && device < 64) configured[device] = true;
    return rc;
}

// How many clusters of `size` CTAs of the 128-row instance can be resident at once.  Measured on
// the largest instance of the family so that the answer, and with it the K split, does not depend
// on the number of activation rows.
template <int kT, bool kSwiglu>
inline int umma_active_clusters(int size) {
    static int cached[64][9] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (device < 64 && cached[device][size]) return cached[device][size];
    using Cfg = UmmaConfig<kT, 128>;
    if (configure_umma_instance<kT, 128, kSwiglu>() != cudaSuccess) return 0;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(size * 64, 1, 1);
    config.blockDim = dim3(Cfg::kThreads, 1, 1);
    config.dynamicSmemBytes = Cfg::kSmemBytes;
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = size;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    config.attrs = attrs;
    config.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, affine_umma_kernel<kT, 128, kSwiglu>, &config) !=
        cudaSuccess)
        clusters = 0;
    if (device < 64) cached[device][size] = clusters > 0 ? clusters : -1;
    return clusters;
}

// Cluster size along K.  A function of (tile count, K, kernel family, device) only -- never of the
// number of activation rows.  cost = waves x (ring slots per CTA + a fixed prologue/epilogue term).
template <int kT, bool kSwiglu>
inline int umma_ksplit(int tiles, int slots_total) {
    int best = 1;
    long best_cost = -1;
    for (int s = 1; s <= 8; ++s) {
        if (s > slots_total) break;
        const int active = umma_active_clusters<kT, kSwiglu>(s);
        if (active <= 0) continue;
        const long waves = (tiles + active - 1) / active;
        const long per_cta = (slots_total + s - 1) / s;
        const long cost = waves * (per_cta * 4 + 6);
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best = s;
        }
    }
    return best;
}

template <int kT, int kMPad, bool kSwiglu>
inline int launch_umma_instance(const UmmaParams& params, int tiles, cudaStream_t stream) {
    using Cfg = UmmaConfig<kT, kMPad>;
    if (configure_umma_instance<kT, kMPad, kSwiglu>() != cudaSuccess) return MT_ERR_LAUNCH;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(tiles * params.ksplit, 1, 1);
    config.blockDim = dim3(Cfg::kThreads, 1, 1);
    config.dynamicSmemBytes = Cfg::kSmemBytes;
    config.stream = stream;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = params.ksplit;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attrs;
    config.numAttrs = 2;
    return cudaLaunchKernelEx(&config, affine_umma_kernel<kT, kMPad, kSwiglu>, params) == cudaSuccess
               ? MT_OK
               : MT_ERR_LAUNCH;
}

template <int kT, bool kSwiglu>
inline int launch_umma_family(UmmaParams& params, int tiles, int mpad, cudaStream_t stream) {
    const int kblocks = params.K / kUmmaBlockK;
    params.ksplit = umma_ksplit<kT, kSwiglu>(tiles, (kblocks + kUmmaKBlocksPerSlot - 1) / kUmmaKBlocksPerSlot);
    switch (mpad) {
        case 16: return launch_umma_instance<kT, 16, kSwiglu>(params, tiles, stream);
        case 32: return launch_umma_instance<kT, 32, kSwiglu>(params, tiles, stream);
        case 64: return launch_umma_instance<kT, 64, kSwiglu>(params, tiles, stream);
        case 128: return launch_umma_instance<kT, 128, kSwiglu>(params, tiles, stream);
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
                       void* out, int M, int K, int N, cudaStream_t stream) {
    if (M < 1 || M > 128 || K % kUmmaBlockK || K < kUmmaBlockK || N < 1) return MT_ERR_SHAPE;
    if (!aligned_to(x, 16) || !aligned_to(first->w, 16) || (second && !aligned_to(second->w, 16))) return MT_ERR_ALIGN;
    const bool swiglu = second != nullptr;
    const int mpad = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
    const int tiles = (N + kUmmaTileRows - 1) / kUmmaTileRows;
    UmmaParams params;
    params.x = static_cast<const uint16_t*>(x);
    params.scales[0] = first->scales;
    params.biases[0] = first->biases;
    params.scales[1] = swiglu ? second->scales : first->scales;
    params.biases[1] = swiglu ? second->biases : first->biases;
    params.residual = static_cast<const uint16_t*>(residual);
    params.out = static_cast<uint16_t*>(out);
    params.M = M;
    params.K = K;
    params.N = N;
    params.ksplit = 1;
    if (!encode_weight_map(&params.w_map[0], first->w, K, N)) return MT_ERR_LAUNCH;
    if (!encode_weight_map(&params.w_map[1], swiglu ? second->w : first->w, K, N)) return MT_ERR_LAUNCH;
    if (!encode_activation_map(&params.x_map, x, M, K, mpad)) return MT_ERR_LAUNCH;
    return swiglu ? launch_umma_family<2, true>(params, tiles, mpad, stream)
                  : launch_umma_family<1, false>(params, tiles, mpad, stream);
}

}  // namespace mt
