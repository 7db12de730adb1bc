// INT4 affine projection on tcgen05 with EXACT weights, 1..32 activation rows per launch, in a
// footprint of half an SM so that consecutive launches of a stream overlap.
//
// Computes Y[M,N] = X[M,K] * dequant(W)[N,K]^T for the MLX layout the reference consumes
// (kernels/affine_qmv.py:25-51; shapes metile/backends/mlx_quantized.py:478-480), with the residual
// epilogue of kernels/affine_qmv.py:124-131 or, for a gate|up pair, the SwiGLU epilogue
// g/(1+exp(-g))*u on un-rounded sums of :204-208.
//
// Arithmetic.  For one quantisation group g (64 columns, one k-block) of one weight row
//     sum_k x_k (s q_k + b)  =  s * P + (b - 128 s) * X,
//     P = sum_k x_k (128 + q_k)   on the tensor core (fp32 accumulate),
//     X = sum_k x_k               once per CTA in fp32.
// The A operand is the bf16 pair (128+q_i, 128+q_{i+4}) straight out of the mask-or-magic unpack
// (integers up to 143 are exact in bf16), so nothing is rounded before the MMA and the result is
// compared with the exact-weight oracle.  Per output the fp32 order is: k-blocks of one dequant
// group ascending, dequant groups in order, cluster ranks in order -- a function of (K, N, device)
// only, so a row's bits do not depend on how many rows share the launch.
//
// Instruction diet.  A dequant thread owns one weight row of the tile.  Per k-block (64 weights)
// it issues two 128-bit shared loads, 56 integer instructions of unpack, two tcgen05.st, one
// tcgen05.ld and 2 FMAs per activation row; scales and biases arrive four groups per 64-bit load;
// the activation tile and the group sums X are prepared by ONE warp per CTA, not by every thread.
//
// Footprint.  352 threads, <= 88 registers, 108 KB of shared memory and 256 columns of tensor
// memory for up to 16 rows: two CTAs fit on an SM.  A launch has at most one CTA per SM, so with
// programmatic dependent launch the NEXT kernel of the stream becomes resident beside it, fills its
// own ring with packed weights (which nobody writes) and has them in shared memory when its
// predecessor's results arrive: the weight stream from HBM does not stop between kernels.
//
//   producer lane : TMA boxes of 128 rows x 128 B (four k-blocks of one tile), 128B swizzle, ring
//                   of five boxes
//   dequant warps : 8 = two groups of four warps (128 rows).  gate|up: group t feeds tile t.
//                   Single projection: group d takes the k-blocks i = d (mod 2).
//   x warp        : activation chunks (L2-resident, cp.async) -> ring of swizzled B tiles in the
//                   element order the unpack produces (e0,e4,e1,e5,e2,e6,e3,e7); group sums X -> shared
//                   table; runs ahead of the weight pipeline, two k-blocks per hand-over
//   MMA lane      : four tcgen05.mma (M=128, K=16) per k-block and tile into that stage's OWN
//                   partial accumulator, tcgen05.commit
//   fold          : the dequant thread that refills a stage first reads the stage's finished
//                   partial tile (tcgen05.ld) and folds it with the group's scale and bias
//   epilogue      : fp32 accumulators -> shared memory; K split over a thread-block cluster is
//                   summed over DSMEM in rank order; SwiGLU / residual; bf16 store
#pragma once

#include <cuda.h>

#include "affine_umma.cuh"
#include "common.cuh"
#include "ptx.cuh"

namespace mt {

template <int kT, int kNPad>
struct StreamConfig {
    static constexpr int kDequantWarps = 8;
    static constexpr int kDepth = kDequantWarps / (4 * kT);   // dequant groups per tile
    static constexpr int kQueue = 2;                           // stages (pending partial tiles) per thread
    static constexpr int kStages = kDepth * kQueue;            // k-block stages: A, B, partial tile, X sums
    static constexpr int kPerSlot = kUmmaKBlocksPerSlot / kDepth;  // k-blocks of one box a thread handles
    static constexpr int kProducerWarp = kDequantWarps;
    static constexpr int kMmaWarp = kDequantWarps + 1;
    static constexpr int kXWarp = kDequantWarps + 2;
    static constexpr int kThreads = (kDequantWarps + 3) * 32;
    static constexpr int kBoxBytes = kUmmaTileRows * 128;      // one tile, four k-blocks
    static constexpr int kRingBoxes = 5;
    static constexpr int kRingBytes = kRingBoxes * kBoxBytes;
    static constexpr int kBBytes = kNPad * 128;
    static constexpr int kBSlots = 4;                          // ring of activation (B) tiles, indexed by k-block
    static constexpr int kXBatch = 2;                          // k-blocks the x warp prepares per iteration
    static constexpr int kXDepth = 2;                          // batches of raw activation chunks in flight (cp.async)
    static constexpr int kXsumEntries = 16;                    // ring of group-sum rows, indexed by k-block
    static constexpr int kXStageBytes = kXDepth * kXBatch * kNPad * 128;
    static constexpr int kXsumBytes = kXsumEntries * kNPad * 4;
    static constexpr int kACols = kStages * kT * 32;
    static constexpr int kPCols = kStages * kT * kNPad;
    static constexpr int kTmemCols = pow2_at_least(kACols + kPCols);
    static constexpr int kStagingBytes = kDepth * kT * kNPad * kUmmaTileRows * 4;
    static constexpr int kDataBytes = kRingBytes + kBSlots * kBBytes + kXStageBytes + kXsumBytes;
    static constexpr int kBarrierBytes = 8 * (2 * kRingBoxes + 2 * kStages + 2 * kBSlots) + 16;
    static constexpr int kSmemBytes = 1024 + kDataBytes + kBarrierBytes;
    static constexpr int kPerSm = kNPad <= 16 ? 2 : 1;         // CTAs (of consecutive launches) per SM
    static constexpr int kFullArrivals = kDequantWarps / kDepth;      // warps that fill one A stage
    static_assert(kT == 1 || kT == 2, "one tile, or a gate tile and an up tile");
    static_assert(kNPad == 16 || kNPad == 32, "activation rows are padded to 16 or 32");
    static_assert(kPerSm * kTmemCols <= 512, "tensor memory budget");
    static_assert(kPerSm * (kSmemBytes + 1024) <= 227 * 1024, "shared memory budget");
    static_assert(kStagingBytes <= kRingBytes, "the epilogue reuses the ring");
    static_assert(kBSlots % kStages == 0 && kBSlots % kXBatch == 0, "static stage and slot indices in the MMA loop");
    static_assert(kXsumEntries > kBSlots + kStages && (kXsumEntries & (kXsumEntries - 1)) == 0, "group sums outlive their fold");
};

enum : unsigned int {
    kWaitStreamRingEmpty = 0x301,
    kWaitStreamRingFull = 0x302,
    kWaitStreamStageFree = 0x303,
    kWaitStreamStageFull = 0x304,
    kWaitStreamDrain = 0x305,
};

// Four consecutive bf16 table entries (scales or biases of one weight row) as one 64-bit load when
// they are 8-byte aligned, else entry by entry; entries from `count` on are not read.  volatile: the
// loads stay where they are written, one box ahead of their use.
__device__ __forceinline__ uint2 stream_load_entries(const uint16_t* p, int count, bool aligned8) {
    uint2 v = make_uint2(0u, 0u);
    if (aligned8 && count >= 4) {
        asm volatile("ld.global.nc.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    } else {
        uint32_t e[4] = {0u, 0u, 0u, 0u};
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if (i < count) e[i] = ldg_nc_u16(p + i);
        v.x = e[0] | (e[1] << 16);
        v.y = e[2] | (e[3] << 16);
    }
    return v;
}

__device__ __forceinline__ float stream_entry_f32(uint2 four, int i) {
    const uint32_t word = i < 2 ? four.x : four.y;
    return __uint_as_float((i & 1) ? (word & 0xFFFF0000u) : (word << 16));
}

template <int kT, int kNPad, bool kSwiglu>
__global__ void __launch_bounds__(StreamConfig<kT, kNPad>::kThreads, StreamConfig<kT, kNPad>::kPerSm)
affine_stream_kernel(const __grid_constant__ UmmaParams p) {
    using Cfg = StreamConfig<kT, kNPad>;
    static_assert(!kSwiglu || kT == 2, "SwiGLU pairs a gate tile with an up tile");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* ring = smem;
    uint8_t* b_tiles = smem + Cfg::kRingBytes;
    uint8_t* x_stage = b_tiles + Cfg::kBSlots * Cfg::kBBytes;                       // [batch % depth][task] x 16 B
    float* xsum = reinterpret_cast<float*>(x_stage + Cfg::kXStageBytes);            // [k-block % entries][kNPad]
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + Cfg::kDataBytes);
    uint64_t* ring_full = bars;
    uint64_t* ring_empty = ring_full + Cfg::kRingBoxes;
    uint64_t* st_full = ring_empty + Cfg::kRingBoxes;   // A stage filled: dequant warps -> MMA lane
    uint64_t* st_done = st_full + Cfg::kStages;         // A stage and its partial tile consumed: MMA commit -> dequant warps
    uint64_t* b_full = st_done + Cfg::kStages;          // B tile and group sums written: x warp -> MMA lane, dequant warps
    uint64_t* b_free = b_full + Cfg::kBSlots;           // B tile consumed: MMA commit -> x warp
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(b_free + Cfg::kBSlots);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int ksplit = p.ksplit;
    const int rank = blockIdx.x % ksplit;  // equals the CTA's rank in its cluster
    const int tile = blockIdx.x / ksplit;
    const int n0 = tile * kUmmaTileRows;
    const int kblocks = p.K / kUmmaBlockK;
    // The K range is cut between the CTAs of a cluster in whole boxes (4 k-blocks).
    const int slots_total = (kblocks + kUmmaKBlocksPerSlot - 1) / kUmmaKBlocksPerSlot;
    const int slot_begin = (int)(((long long)slots_total * rank) / ksplit);
    const int slot_end = (int)(((long long)slots_total * (rank + 1)) / ksplit);
    const int nslots = slot_end - slot_begin;
    const int kb_begin = slot_begin * kUmmaKBlocksPerSlot;
    const int kb_end = min(slot_end * kUmmaKBlocksPerSlot, kblocks);
    const int nkb = kb_end - kb_begin;

    if (threadIdx.x == 0) {
        for (int i = 0; i < Cfg::kRingBoxes; ++i) {
            ptx::mbar_init(&ring_full[i], 1);
            ptx::mbar_init(&ring_empty[i], Cfg::kDequantWarps / kT);
        }
        for (int i = 0; i < Cfg::kStages; ++i) {
            ptx::mbar_init(&st_full[i], Cfg::kFullArrivals);
            ptx::mbar_init(&st_done[i], 1);
        }
        for (int i = 0; i < Cfg::kBSlots; ++i) {
            ptx::mbar_init(&b_full[i], 1);
            ptx::mbar_init(&b_free[i], 1);
        }
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
    // The next kernel of the stream may become resident now.  Only the packed weights, scales and
    // biases (which no kernel writes) are touched before griddep_wait().
    ptx::griddep_launch_dependents();

    float acc[kNPad];
#pragma unroll
    for (int m = 0; m < kNPad; ++m) acc[m] = 0.0f;
    int t = 0, depth = 0, r = 0;
    bool acc_ok = true;

    if (warp == Cfg::kProducerWarp) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            ptx::prefetch_tensor_map(&p.w_map[0]);
            if (kT == 2) ptx::prefetch_tensor_map(&p.w_map[1]);
            const int boxes = nslots * kT;
            int issued = 0;
            for (int b = 0; b < boxes; ++b) {
                const int s = b % Cfg::kRingBoxes;
                const uint32_t use = (uint32_t)(b / Cfg::kRingBoxes);
                if (!ptx::mbar_wait(&ring_empty[s], (use & 1u) ^ 1u, abort_flag, kWaitStreamRingEmpty)) break;
                ptx::mbar_expect_tx(&ring_full[s], Cfg::kBoxBytes);
                ptx::tma_load_2d(ring + s * Cfg::kBoxBytes, &p.w_map[b % kT], (slot_begin + b / kT) * 32, n0,
                                 &ring_full[s]);
                ++issued;
            }
            if (*abort_flag) {
                // Let copies already in flight land before the CTA may exit.
                const int first = issued > Cfg::kRingBoxes ? issued - Cfg::kRingBoxes : 0;
                for (int b = first; b < issued; ++b)
                    ptx::mbar_wait(&ring_full[b % Cfg::kRingBoxes], (uint32_t)(b / Cfg::kRingBoxes) & 1u, abort_flag,
                                   kWaitStreamDrain);
            }
        }
    } else if (warp == Cfg::kMmaWarp) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::umma_idesc_bf16(kUmmaTileRows, kNPad);
            const uint64_t desc0 = ptx::smem_desc_k_major_sw128(ptx::smem_u32(b_tiles));
            for (int i0 = 0; i0 < nkb; i0 += Cfg::kBSlots) {
                const uint32_t b_phase = (uint32_t)(i0 / Cfg::kBSlots) & 1u;
#pragma unroll
                for (int u = 0; u < Cfg::kBSlots; ++u) {
                    const int i = i0 + u;
                    if (i >= nkb) break;
                    constexpr int kUsesPerRound = Cfg::kBSlots / Cfg::kStages;  // uses of an A stage per round of B slots
                    const int a = u % Cfg::kStages;
                    const uint32_t a_phase = (uint32_t)((i0 / Cfg::kBSlots) * kUsesPerRound + u / Cfg::kStages) & 1u;
                    if (!ptx::mbar_wait(&b_full[u], b_phase, abort_flag, kWaitStreamStageFull) ||
                        !ptx::mbar_wait(&st_full[a], a_phase, abort_flag, kWaitStreamStageFull)) { i0 = nkb; break; }
                    ptx::tc_fence_after_sync();
#pragma unroll
                    for (int ks = 0; ks < kUmmaBlockK / 16; ++ks) {
#pragma unroll
                        for (int tt = 0; tt < kT; ++tt) {
                            const uint32_t d_tmem = tmem_base + Cfg::kACols + (a * kT + tt) * kNPad;
                            const uint32_t a_tmem = tmem_base + (a * kT + tt) * 32 + ks * 8;
                            const uint64_t b_desc = desc0 + (uint64_t)((u * Cfg::kBBytes + ks * 32) >> 4);
                            ptx::umma_ts(d_tmem, a_tmem, b_desc, idesc, ks > 0 ? 1u : 0u);
                        }
                    }
                    ptx::umma_commit(&st_done[a]);
                    ptx::umma_commit(&b_free[u]);
                }
            }
        }
    } else if (warp == Cfg::kXWarp) {
        // ------------------------------------------------------------------ activation tiles + group sums
        // Task = (k-block of the batch, activation row, 16-byte chunk of the k-block's 64 columns); lane l
        // takes the tasks l, l + 32, ...  The eight chunks of one (k-block, row) are eight neighbouring
        // tasks, hence eight neighbouring lanes, whose sums meet in a fixed butterfly: a group sum does
        // not depend on how many rows there are.  kXBatch k-blocks are prepared per iteration so that the
        // cross-proxy fence and the hand-over are paid once per batch.
        ptx::griddep_wait();  // the activations are the preceding kernel's output
        const int tasks_per_kb = p.M * 8;
        const int tasks = Cfg::kXBatch * tasks_per_kb;
        const int trips = (tasks + 31) >> 5;
        const uint16_t* x_base = p.x + (size_t)kb_begin * kUmmaBlockK;
        constexpr int kBatchChunks = Cfg::kXBatch * kNPad * 8;  // 16-byte chunks of one staging slot
        // The chunks come from L2 (several hundred cycles away), so kXDepth batches are kept in flight
        // with cp.async into a small ring; a lane reads back only the chunks it copied itself.  One
        // group is committed per batch, empty or not, so that the group count stays uniform.
        auto issue_x = [&](int batch) {
            const int kb0 = batch * Cfg::kXBatch;
            if (kb0 < nkb) {
                for (int trip = 0; trip < trips; ++trip) {
                    const int task = trip * 32 + lane;
                    const int kbl = task >= tasks_per_kb ? 1 : 0;
                    const int rem = task - kbl * tasks_per_kb;
                    if (task < tasks && kb0 + kbl < nkb)
                        ptx::cp_async_16(ptx::smem_u32(x_stage) + (uint32_t)(((batch % Cfg::kXDepth) * kBatchChunks + task) * 16),
                                         x_base + (size_t)(rem >> 3) * p.K + (size_t)(kb0 + kbl) * kUmmaBlockK + (rem & 7) * 8);
                }
            }
            ptx::cp_async_commit();
        };
        static_assert(Cfg::kXBatch == 2, "the task decoding above assumes two k-blocks per batch");
        const int batches = (nkb + Cfg::kXBatch - 1) / Cfg::kXBatch;
#pragma unroll
        for (int d = 0; d < Cfg::kXDepth; ++d) issue_x(d);
        for (int batch = 0; batch < batches; ++batch) {
            const int kb0 = batch * Cfg::kXBatch;
            ptx::cp_async_wait_group<Cfg::kXDepth - 1>();
            bool ok = true;
#pragma unroll
            for (int kbl = 0; kbl < Cfg::kXBatch; ++kbl) {
                const int kb = kb0 + kbl;
                if (kb < nkb)
                    ok = ok && ptx::mbar_wait(&b_free[kb % Cfg::kBSlots], ((uint32_t)(kb / Cfg::kBSlots) & 1u) ^ 1u, abort_flag,
                                              kWaitStreamStageFree);
            }
            if (!__all_sync(0xFFFFFFFFu, ok)) break;
            for (int trip = 0; trip < trips; ++trip) {
                const int task = trip * 32 + lane;
                const int kbl = task >= tasks_per_kb ? 1 : 0;
                const int rem = task - kbl * tasks_per_kb;
                const int row = rem >> 3, c = rem & 7, kb = kb0 + kbl;
                const bool active = task < tasks && kb < nkb;
                float part = 0.0f;
                if (active) {
                    const uint4 v = *reinterpret_cast<const uint4*>(x_stage + ((batch % Cfg::kXDepth) * kBatchChunks + task) * 16);
                    uint4 o;
                    o.x = __byte_perm(v.x, v.z, 0x5410);  // (x0, x4)
                    o.y = __byte_perm(v.x, v.z, 0x7632);  // (x1, x5)
                    o.z = __byte_perm(v.y, v.w, 0x5410);  // (x2, x6)
                    o.w = __byte_perm(v.y, v.w, 0x7632);  // (x3, x7)
                    *reinterpret_cast<uint4*>(b_tiles + (kb % Cfg::kBSlots) * Cfg::kBBytes + row * 128 + ((c ^ (row & 7)) << 4)) = o;
                    part = ((bf16_lo(v.x) + bf16_hi(v.x)) + (bf16_lo(v.y) + bf16_hi(v.y))) +
                           ((bf16_lo(v.z) + bf16_hi(v.z)) + (bf16_lo(v.w) + bf16_hi(v.w)));
                }
                part += __shfl_xor_sync(0xFFFFFFFFu, part, 1);
                part += __shfl_xor_sync(0xFFFFFFFFu, part, 2);
                part += __shfl_xor_sync(0xFFFFFFFFu, part, 4);
                if (active && c == 0) xsum[(kb & (Cfg::kXsumEntries - 1)) * kNPad + row] = part;
            }
            issue_x(batch + Cfg::kXDepth);  // reuses the staging slot that was just read
            // The B tiles are read by the tensor core (async proxy).
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
#pragma unroll
                for (int kbl = 0; kbl < Cfg::kXBatch; ++kbl)
                    if (kb0 + kbl < nkb) ptx::mbar_arrive(&b_full[(kb0 + kbl) % Cfg::kBSlots]);
            }
        }
        ptx::cp_async_wait_group<0>();  // nothing of this thread's is in flight when the CTA ends
    } else {
        // ------------------------------------------------------------------ dequant + fold warps
        const int group = warp >> 2;                       // four warps = 128 rows
        t = kT == 2 ? group : 0;                           // which tile (gate / up) this group feeds
        depth = kT == 2 ? 0 : group;                       // which k-blocks: i = depth (mod kDepth)
        r = ((warp & 3) << 5) | lane;                      // weight row inside the tile == TMEM lane
        const int n = min(n0 + r, p.N - 1);                // rows past N were zero-filled by TMA
        const uint16_t* scale_row = p.scales[t] + (size_t)n * kblocks + kb_begin;
        const uint16_t* bias_row = p.biases[t] + (size_t)n * kblocks + kb_begin;
        const bool aligned8 = (kblocks & 3) == 0 && ((reinterpret_cast<uintptr_t>(p.scales[t]) |
                                                       reinterpret_cast<uintptr_t>(p.biases[t])) & 7) == 0;
        const uint32_t lane_field = (uint32_t)((warp & 3) << 5) << 16;
        uint2 scales_next = make_uint2(0u, 0u), biases_next = make_uint2(0u, 0u);
        if (nslots > 0) {
            scales_next = stream_load_entries(scale_row, nkb, aligned8);
            biases_next = stream_load_entries(bias_row, nkb, aligned8);
        }
        float pend_scale[Cfg::kQueue], pend_offset[Cfg::kQueue];
#pragma unroll
        for (int q = 0; q < Cfg::kQueue; ++q) { pend_scale[q] = 0.0f; pend_offset[q] = 0.0f; }
        int count = 0;  // k-blocks this thread has handed to the MMA so far

        // Fold one finished partial tile (columns c0 .. c0+15 already in registers).
        auto fold16 = [&](const uint32_t (&part)[16], int c0, float scale, float offset, const float* sums) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                if (c0 + g * 4 < p.M) {
                    const float4 v = *reinterpret_cast<const float4*>(sums + c0 + 4 * g);  // same address warp-wide
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const float xs = e == 0 ? v.x : e == 1 ? v.y : e == 2 ? v.z : v.w;
                        acc[c0 + 4 * g + e] =
                            fmaf(scale, __uint_as_float(part[4 * g + e]), fmaf(offset, xs, acc[c0 + 4 * g + e]));
                    }
                }
            }
        };

        bool alive = true;
        for (int st = 0; st < nslots && alive; ++st) {
            const int b = st * kT + t;
            const int s = b % Cfg::kRingBoxes;
            const uint32_t ring_phase = (uint32_t)(b / Cfg::kRingBoxes) & 1u;
            const uint8_t* wrow = ring + s * Cfg::kBoxBytes + r * 128;
            const uint2 scales4 = scales_next, biases4 = biases_next;
            if (st + 1 < nslots) {
                const int left = nkb - (st + 1) * kUmmaKBlocksPerSlot;
                scales_next = stream_load_entries(scale_row + (st + 1) * kUmmaKBlocksPerSlot, left, aligned8);
                biases_next = stream_load_entries(bias_row + (st + 1) * kUmmaKBlocksPerSlot, left, aligned8);
            }
            const bool landed = ptx::mbar_wait(&ring_full[s], ring_phase, abort_flag, kWaitStreamRingFull);
            if (!__all_sync(0xFFFFFFFFu, landed)) { alive = false; break; }
#pragma unroll
            for (int jj = 0; jj < Cfg::kPerSlot; ++jj) {
                const int j = depth + jj * Cfg::kDepth;          // k-block inside the box
                const int i = st * kUmmaKBlocksPerSlot + j;      // k-block inside this CTA's range
                if (i >= nkb) break;
                const int a = i % Cfg::kStages;
                const uint32_t use = (uint32_t)(i / Cfg::kStages);
                const int q_slot = jj % Cfg::kQueue;             // == count % kQueue (kPerSlot is even)
                // The stage is free once the MMAs of its previous k-block -- handed over by this same
                // thread kQueue iterations ago -- are complete: start reading that partial tile back
                // now, wait for it before the stage is handed over again, fold it after the hand-over.
                const bool freed = ptx::mbar_wait(&st_done[a], (use & 1u) ^ 1u, abort_flag, kWaitStreamStageFree);
                if (!__all_sync(0xFFFFFFFFu, freed)) { alive = false; break; }  // also reconverges the warp
                ptx::tc_fence_after_sync();
                const bool folding = count >= Cfg::kQueue;
                const uint32_t p_tmem = tmem_base + lane_field + Cfg::kACols + (a * kT + t) * kNPad;
                const bool wide = kNPad > 16 && p.M > 16;
                uint32_t part[16], part_hi[kNPad > 16 ? 16 : 1];
                if (folding) {
                    ptx::tmem_ld16(p_tmem, part);
                    if constexpr (kNPad > 16) {
                        if (wide) ptx::tmem_ld16(p_tmem + 16, part_hi);
                    }
                }

                // 32 B of this row for k-block j: 16-byte chunks 2j and 2j+1, XOR-swizzled by the row.
                const uint4 w_lo = *reinterpret_cast<const uint4*>(wrow + (((2 * j) ^ (r & 7)) << 4));
                const uint4 w_hi = *reinterpret_cast<const uint4*>(wrow + (((2 * j + 1) ^ (r & 7)) << 4));
                const uint32_t a_tmem = tmem_base + lane_field + (a * kT + t) * 32;
                uint32_t wq[16];
                unpack_word_offset128(w_lo.x, &wq[0]);
                unpack_word_offset128(w_lo.y, &wq[4]);
                unpack_word_offset128(w_lo.z, &wq[8]);
                unpack_word_offset128(w_lo.w, &wq[12]);
                ptx::tmem_st16(a_tmem, wq);
                unpack_word_offset128(w_hi.x, &wq[0]);
                unpack_word_offset128(w_hi.y, &wq[4]);
                unpack_word_offset128(w_hi.z, &wq[8]);
                unpack_word_offset128(w_hi.w, &wq[12]);
                ptx::tmem_st16(a_tmem + 16, wq);

                if (folding) {
                    ptx::tc_wait_ld16(part);
                    if constexpr (kNPad > 16) {
                        if (wide) ptx::tc_wait_ld16(part_hi);
                    }
                }
                ptx::tc_wait_st();
                ptx::tc_fence_before_sync();
                // The group sums of k-block i are read when its partial tile is folded, kQueue iterations
                // from now.  Observing the x warp's hand-over of that k-block here -- before this warp's own
                // hand-over, without which the k-block's MMAs cannot run and its B slot cannot be reused --
                // is what orders those reads after the x warp's writes.
                const bool sums_ready = ptx::mbar_wait(&b_full[i % Cfg::kBSlots], (uint32_t)(i / Cfg::kBSlots) & 1u, abort_flag,
                                                       kWaitStreamStageFull);
                if (!__all_sync(0xFFFFFFFFu, sums_ready)) { alive = false; break; }
                if (lane == 0) ptx::mbar_arrive(&st_full[a]);

                // The group sums of the folded k-block are still there: the x warp reuses a table row
                // kXsumEntries k-blocks later, which needs hand-overs this thread has not made yet.
                if (folding) {
                    const float* sums = xsum + ((i - Cfg::kStages) & (Cfg::kXsumEntries - 1)) * kNPad;
                    fold16(part, 0, pend_scale[q_slot], pend_offset[q_slot], sums);
                    if constexpr (kNPad > 16) {
                        if (wide) fold16(part_hi, 16, pend_scale[q_slot], pend_offset[q_slot], sums);
                    }
                }
                const float scale = stream_entry_f32(scales4, j);
                pend_scale[q_slot] = scale;
                pend_offset[q_slot] = fmaf(-128.0f, scale, stream_entry_f32(biases4, j));  // b - 128 s
                ++count;
            }
            if (!alive) break;
            // The box was read with ordinary loads and will be overwritten by TMA (async proxy).
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&ring_empty[s]);
        }

        // -------------------------------------------------------------- drain the pending partial tiles
        __syncwarp();
        alive = __all_sync(0xFFFFFFFFu, alive);
        if (alive) {
            const int pending = count < Cfg::kQueue ? count : Cfg::kQueue;
#pragma unroll
            for (int step = 0; step < Cfg::kQueue; ++step) {
                if (step < pending) {
                    const int seq = count - pending + step;                 // this thread's seq-th k-block
                    const int i = (seq / Cfg::kPerSlot) * kUmmaKBlocksPerSlot + depth + (seq % Cfg::kPerSlot) * Cfg::kDepth;
                    const int a = i % Cfg::kStages;
                    const uint32_t use = (uint32_t)(i / Cfg::kStages);
                    const bool ok = __all_sync(0xFFFFFFFFu, ptx::mbar_wait(&st_done[a], use & 1u, abort_flag, kWaitStreamStageFree));
                    ptx::tc_fence_after_sync();
                    if (!ok) { alive = false; break; }
                    const uint32_t p_tmem = tmem_base + lane_field + Cfg::kACols + (a * kT + t) * kNPad;
                    const float* sums = xsum + (i & (Cfg::kXsumEntries - 1)) * kNPad;
                    const float scale = (seq % Cfg::kQueue) == 0 ? pend_scale[0] : pend_scale[1];
                    const float offset = (seq % Cfg::kQueue) == 0 ? pend_offset[0] : pend_offset[1];
                    uint32_t part[16];
                    ptx::tmem_ld16(p_tmem, part);
                    ptx::tc_wait_ld16(part);
                    fold16(part, 0, scale, offset, sums);
                    if constexpr (kNPad > 16) {
                        if (p.M > 16) {
                            ptx::tmem_ld16(p_tmem + 16, part);
                            ptx::tc_wait_ld16(part);
                            fold16(part, 16, scale, offset, sums);
                        }
                    }
                }
            }
        }
        acc_ok = alive;
        // Every dequant warp has consumed its boxes: the ring becomes the staging area.
        asm volatile("bar.sync 1, %0;" ::"r"(Cfg::kDequantWarps * 32) : "memory");
        float* staging = reinterpret_cast<float*>(smem);
#pragma unroll
        for (int m = 0; m < kNPad; ++m)
            if (m < p.M) staging[((depth * kT + t) * kNPad + m) * kUmmaTileRows + r] = acc_ok ? acc[m] : 0.0f;
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
        ptx::griddep_wait();  // the residual is read and the output written only after the preceding kernel
        const int row = threadIdx.x & 127;
        const int part = threadIdx.x >> 7;
        constexpr int kParts = Cfg::kDequantWarps / 4;
        const int n = n0 + row;
        const uint32_t staging_addr = ptx::smem_u32(smem);
        for (int m = rank + ksplit * part; m < p.M; m += ksplit * kParts) {
            float first = 0.0f, second = 0.0f;
            for (int j = 0; j < ksplit; ++j) {
                const uint32_t peer = ksplit > 1 ? ptx::map_to_cta(staging_addr, (uint32_t)j) : staging_addr;
#pragma unroll
                for (int d = 0; d < Cfg::kDepth; ++d) {
                    const int index = ((d * kT) * kNPad + m) * kUmmaTileRows + row;
                    if (ksplit > 1) {
                        first += ptx::ld_cluster_f32(peer + 4u * (uint32_t)index);
                        if constexpr (kSwiglu)
                            second += ptx::ld_cluster_f32(peer + 4u * (uint32_t)(index + kNPad * kUmmaTileRows));
                    } else {
                        const float* local = reinterpret_cast<const float*>(smem);
                        first += local[index];
                        if constexpr (kSwiglu) second += local[index + kNPad * kUmmaTileRows];
                    }
                }
            }
            if (n < p.N) {
                float v = kSwiglu ? swiglu_f32(first, second) : first;
                if (!kSwiglu && p.residual)
                    v += bf16_bits_to_f32(ptx::ld_global_dependent_u16(p.residual + (size_t)m * p.N + n));
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
template <int kT, int kNPad, bool kSwiglu>
inline cudaError_t configure_stream_instance() {
    using Cfg = StreamConfig<kT, kNPad>;
    static bool configured[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (device < 64 && configured[device]) return cudaSuccess;
    auto kernel = affine_stream_kernel<kT, kNPad, kSwiglu>;
    cudaError_t rc = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (rc == cudaSuccess)
        rc = cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (rc == cudaSuccess && device < 64) configured[device] = true;
    return rc;
}

// Cluster size along K: the largest split that still leaves at most one CTA per SM (so that the next
// kernel of the stream finds room beside this one), at most 8, at most one box per CTA.  A function
// of (tile count, K, device) only -- never of the number of activation rows.
inline int stream_ksplit(int tiles, int slots_total, int sm_count) {
    int s = sm_count / (tiles > 0 ? tiles : 1);
    if (s > 8) s = 8;
    if (s > slots_total) s = slots_total;
    return s < 1 ? 1 : s;
}

template <int kT, int kNPad, bool kSwiglu>
inline int launch_stream_instance(const UmmaParams& params, int tiles, cudaStream_t stream) {
    using Cfg = StreamConfig<kT, kNPad>;
    if (configure_stream_instance<kT, kNPad, kSwiglu>() != cudaSuccess) return MT_ERR_LAUNCH;
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
    return cudaLaunchKernelEx(&config, affine_stream_kernel<kT, kNPad, kSwiglu>, params) == cudaSuccess ? MT_OK
                                                                                                         : MT_ERR_LAUNCH;
}

constexpr int kStreamMaxRows = 32;

// x [M,K] bf16 with M <= 32, one weight triple (plain / residual) or two (gate, up -> SwiGLU).
inline int launch_stream(const void* x, const AffineWeights* first, const AffineWeights* second, const void* residual,
                         void* out, int M, int K, int N, int sm_count, cudaStream_t stream) {
    if (M < 1 || M > kStreamMaxRows || K % kUmmaBlockK || K < kUmmaBlockK || N < 1) return MT_ERR_SHAPE;
    if (!aligned_to(x, 16) || !aligned_to(first->w, 16) || (second && !aligned_to(second->w, 16))) return MT_ERR_ALIGN;
    const bool swiglu = second != nullptr;
    const int tiles = (N + kUmmaTileRows - 1) / kUmmaTileRows;
    const int kblocks = K / kUmmaBlockK;
    const int slots_total = (kblocks + kUmmaKBlocksPerSlot - 1) / kUmmaKBlocksPerSlot;
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
    params.ksplit = stream_ksplit(tiles, slots_total, sm_count);
    if (!encode_weight_map(&params.w_map[0], first->w, K, N)) return MT_ERR_LAUNCH;
    if (!encode_weight_map(&params.w_map[1], swiglu ? second->w : first->w, K, N)) return MT_ERR_LAUNCH;
    if (M <= 16) {
        return swiglu ? launch_stream_instance<2, 16, true>(params, tiles, stream)
                      : launch_stream_instance<1, 16, false>(params, tiles, stream);
    }
    return swiglu ? launch_stream_instance<2, 32, true>(params, tiles, stream)
                  : launch_stream_instance<1, 32, false>(params, tiles, stream);
}

}  // namespace mt
