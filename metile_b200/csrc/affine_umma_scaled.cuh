// INT4 affine projection on tcgen05 for up to 16 activation rows with EXACT weights: the scale and
// bias of a quantisation group are applied to the group's partial sums in fp32, not to the weights.
//
//   sum_k x_k (s_g q_k + b_g)  =  s_g * P_g + (b_g - 128 s_g) * X_g,
//   P_g = sum_{k in g} x_k (128 + q_k)   (one k-block = one group, computed by the tensor core),
//   X_g = sum_{k in g} x_k               (computed once per CTA in fp32).
//
// The A operand is the bf16 pair (128+q_i, 128+q_{i+4}) straight out of the mask-or-magic unpack
// -- integers up to 143, exact in bf16 -- so the dequant warps do no arithmetic on the weights at
// all (the unpack is 7 instructions per 8 weights), and nothing is rounded before the MMA: results
// match the exact-weight oracle like the CUDA-core GEMV does.  The price is that every k-block's
// 128 x 16 partial tile is read back from TMEM (tcgen05.ld) and folded into per-thread fp32
// accumulators with 2 FMAs per activation row, which is cheaper than dequantising only while the
// batch is small; above 16 rows the bf16-dequant kernel in affine_umma.cuh takes over.
//
// Same skeleton as affine_umma.cuh (TMA ring of 4-k-block slots, 16 dequant warps in depth groups,
// one MMA-issuing thread, cluster split-K over DSMEM, programmatic dependent launch).  Each
// operand stage owns its own 16-column accumulator: the MMA of k-block i overwrites it
// (accumulate off at the first K step), and the thread that refills the stage for k-block
// i + kStages reads it first.  Per output the fp32 order is: k-blocks of one depth group ascending,
// depth groups in order, cluster ranks in order -- a function of (K, N, device) only.
#pragma once

#include "affine_umma.cuh"

namespace mt {

template <int kT>
struct UmmaScaledConfig {
    static constexpr int kMPad = 16;
    static constexpr int kDequantWarps = 16;
    static constexpr int kDepth = kDequantWarps / (4 * kT);
    static constexpr int kWarpsPerKBlock = 4 * kT;
    static constexpr int kProducerWarp = kDequantWarps;
    static constexpr int kMmaWarp = kDequantWarps + 1;
    static constexpr int kThreads = (kDequantWarps + 2) * 32;
    static constexpr int kWTileBytes = kUmmaTileRows * 128;
    static constexpr int kSlotBytes = kT * kWTileBytes;
    static constexpr int kBBytes = kMPad * 128;
    static constexpr int kAbStages = 4;
    static constexpr int kAccCols = kAbStages * kT * kMPad;          // one partial tile per stage and tile
    static constexpr int kATmemCols = kAbStages * kT * 32;
    static constexpr int kTmemCols = pow2_at_least(kAccCols + kATmemCols);
    static constexpr int kStages = (kT == 2) ? 5 : 8;                // ring slots (160 KB / 128 KB)
    static constexpr int kRingBytes = kStages * kSlotBytes;
    static constexpr int kMaxKBlocks = 256;                          // per CTA: K range up to 16384
    static constexpr int kXsumBytes = kMaxKBlocks * kMPad * 4;       // X_g per k-block and row
    static constexpr int kStagingBytes = kDepth * kT * kMPad * kUmmaTileRows * 4;
    static constexpr int kDataBytes = kRingBytes + kAbStages * kBBytes + kXsumBytes;
    static constexpr int kBarrierBytes = 8 * (2 * kStages + 2 * kAbStages + 1) + 16;
    static constexpr int kSmemBytes = 1024 + kDataBytes + kBarrierBytes;
    static_assert(kTmemCols <= 512, "tensor memory budget");
    static_assert(kSmemBytes <= 227 * 1024 && 2 * kSmemBytes > 227 * 1024, "one CTA per SM");
    static_assert(kStagingBytes <= kRingBytes, "the epilogue reuses the ring");
    static_assert(kAbStages % kDepth == 0 && kUmmaKBlocksPerSlot % kDepth == 0, "depth groups");
};

template <int kT, bool kSwiglu>
__global__ void __launch_bounds__(UmmaScaledConfig<kT>::kThreads, 1)
affine_umma_scaled_kernel(const __grid_constant__ UmmaParams p) {
    using Cfg = UmmaScaledConfig<kT>;
    constexpr int kMPad = Cfg::kMPad;
    static_assert(!kSwiglu || kT == 2, "SwiGLU pairs a gate tile with an up tile");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* ring = smem;
    uint8_t* b_tiles = smem + Cfg::kRingBytes;
    float* xsum = reinterpret_cast<float*>(b_tiles + Cfg::kAbStages * Cfg::kBBytes);  // [k-block][16]
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
    const int rank = blockIdx.x % ksplit;
    const int tile = blockIdx.x / ksplit;
    const int n0 = tile * kUmmaTileRows;
    const int kblocks = p.K / kUmmaBlockK;
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
            ptx::mbar_init(&ring_empty[i], Cfg::kDequantWarps);
        }
        for (int i = 0; i < Cfg::kAbStages; ++i) {
            ptx::mbar_init(&ab_full[i], Cfg::kWarpsPerKBlock);
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
    ptx::griddep_launch_dependents();

    // Per-thread fp32 accumulators of the dequant warps (one weight row, up to 16 activation rows).
    float acc[kMPad];
#pragma unroll
    for (int m = 0; m < kMPad; ++m) acc[m] = 0.0f;
    int t = 0, depth = 0, r = 0;

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
                for (int tt = 0; tt < kT; ++tt)
                    ptx::tma_load_2d(slot + tt * Cfg::kWTileBytes, &p.w_map[tt], (slot_begin + st) * 32, n0,
                                     &ring_full[s]);
                ++issued;
            }
            if (*abort_flag) {
                const int first = issued > Cfg::kStages ? issued - Cfg::kStages : 0;
                for (int st = first; st < issued; ++st)
                    ptx::mbar_wait(&ring_full[st % Cfg::kStages], (st / Cfg::kStages) & 1, abort_flag, kWaitDrain);
            }
        }
    } else if (warp == Cfg::kMmaWarp) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = ptx::umma_idesc_bf16(kUmmaTileRows, kMPad);
            const uint64_t desc0 = ptx::smem_desc_k_major_sw128(ptx::smem_u32(b_tiles));
            for (int i0 = 0; i0 < nkb; i0 += Cfg::kAbStages) {
                const uint32_t phase = (i0 / Cfg::kAbStages) & 1;
#pragma unroll
                for (int a = 0; a < Cfg::kAbStages; ++a) {
                    if (i0 + a >= nkb) break;
                    if (!ptx::mbar_wait(&ab_full[a], phase, abort_flag, kWaitAbFull)) { i0 = nkb; break; }
                    ptx::tc_fence_after_sync();
#pragma unroll
                    for (int ks = 0; ks < kUmmaBlockK / 16; ++ks) {
#pragma unroll
                        for (int tt = 0; tt < kT; ++tt) {
                            const uint32_t d_tmem = tmem_base + (a * kT + tt) * kMPad;  // this stage's partial tile
                            const uint32_t a_tmem = tmem_base + Cfg::kAccCols + (a * kT + tt) * 32 + ks * 8;
                            const uint64_t b_desc = desc0 + (uint64_t)((a * Cfg::kBBytes + ks * 32) >> 4);
                            ptx::umma_ts(d_tmem, a_tmem, b_desc, idesc, ks > 0 ? 1u : 0u);
                        }
                    }
                    ptx::umma_commit(&ab_empty[a]);
                }
            }
            ptx::umma_commit(acc_full);
        }
    } else {
        // ------------------------------------------------------------------ dequant warps
        const int group = warp >> 2;
        t = kT == 2 ? (group & 1) : 0;
        depth = kT == 2 ? (group >> 1) : group;
        r = ((warp & 3) << 5) | lane;
        const int n = min(n0 + r, p.N - 1);
        const uint16_t* scale_row = p.scales[t] + (size_t)n * kblocks + kb_begin;
        const uint16_t* bias_row = p.biases[t] + (size_t)n * kblocks + kb_begin;
        const int tid = t * 128 + r;
        constexpr int kKBlockThreads = Cfg::kWarpsPerKBlock * 32;
        constexpr int kXTasks = (kMPad * 8 + kKBlockThreads - 1) / kKBlockThreads;
        constexpr int kQueue = Cfg::kAbStages / Cfg::kDepth;  // stages (= pending partial tiles) per group
        const int x_tasks = p.M * 8;
        const uint16_t* x_base = p.x + (size_t)kb_begin * kUmmaBlockK;
        const uint32_t lane_field = (uint32_t)((warp & 3) << 5) << 16;
        uint32_t scale_next = 0, bias_next = 0;
        if (depth < nkb) {
            scale_next = ldg_nc_u16(scale_row + depth);
            bias_next = ldg_nc_u16(bias_row + depth);
        }
        ptx::griddep_wait();  // everything below may read what the preceding kernel wrote

        uint4 xv_next[kXTasks];
        auto load_x = [&](int kblock) {
#pragma unroll
            for (int q = 0; q < kXTasks; ++q) {
                const int task = tid + q * kKBlockThreads;
                if (task < x_tasks)
                    xv_next[q] = ptx::ld_global_dependent_u4(x_base + (size_t)(task >> 3) * p.K +
                                                             (size_t)kblock * kUmmaBlockK + (task & 7) * 8);
            }
        };
        if (depth < nkb) load_x(depth);

        // X_g for every k-block of this CTA and every real row, fp32, ascending k.  The table is
        // first read when a partial tile is folded, kQueue iterations into the loop, so the barrier
        // that publishes it is taken there (exactly once per warp) and not here.
        for (int pair = threadIdx.x; pair < nkb * p.M; pair += Cfg::kDequantWarps * 32) {
            const int kb = pair / p.M, m = pair - kb * p.M;
            const uint16_t* src = x_base + (size_t)m * p.K + (size_t)kb * kUmmaBlockK;
            uint4 v[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) v[c] = ptx::ld_global_dependent_u4(src + c * 8);
            float total = 0.0f;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                total += bf16_lo(v[c].x); total += bf16_hi(v[c].x); total += bf16_lo(v[c].y); total += bf16_hi(v[c].y);
                total += bf16_lo(v[c].z); total += bf16_hi(v[c].z); total += bf16_lo(v[c].w); total += bf16_hi(v[c].w);
            }
            xsum[kb * kMPad + m] = total;
        }
        bool table_published = false;
        auto publish_table = [&]() {
            if (!table_published) {
                asm volatile("bar.sync 1, %0;" ::"r"(Cfg::kDequantWarps * 32) : "memory");
                table_published = true;
            }
        };

        // Fold a finished partial tile (k-block `kb`, already in registers) into the accumulators.
        auto fold = [&](const uint32_t (&part)[16], float scale, float offset, int kb) {
            const float4* xs = reinterpret_cast<const float4*>(xsum + kb * kMPad);  // same address warp-wide
#pragma unroll
            for (int g = 0; g < kMPad / 4; ++g) {
                if (g * 4 < p.M) {
                    const float4 v = xs[g];
                    acc[4 * g + 0] = fmaf(scale, __uint_as_float(part[4 * g + 0]), fmaf(offset, v.x, acc[4 * g + 0]));
                    acc[4 * g + 1] = fmaf(scale, __uint_as_float(part[4 * g + 1]), fmaf(offset, v.y, acc[4 * g + 1]));
                    acc[4 * g + 2] = fmaf(scale, __uint_as_float(part[4 * g + 2]), fmaf(offset, v.z, acc[4 * g + 2]));
                    acc[4 * g + 3] = fmaf(scale, __uint_as_float(part[4 * g + 3]), fmaf(offset, v.w, acc[4 * g + 3]));
                }
            }
        };
        float pend_scale[kQueue], pend_offset[kQueue];
        int pend_kb[kQueue], pend_stage[kQueue];
#pragma unroll
        for (int q = 0; q < kQueue; ++q) { pend_scale[q] = 0.0f; pend_offset[q] = 0.0f; pend_kb[q] = 0; pend_stage[q] = 0; }
        int count = 0;  // k-blocks this thread has handed to the MMA so far

        bool alive = true;
        for (int st = 0; st < nslots && alive; ++st) {
            const int s = st % Cfg::kStages;
            const uint32_t phase = (st / Cfg::kStages) & 1;
            const uint8_t* slot = ring + s * Cfg::kSlotBytes;
            bool waited = false;
#pragma unroll
            for (int jj = 0; jj < kUmmaKBlocksPerSlot / Cfg::kDepth; ++jj) {
                const int j = depth + jj * Cfg::kDepth;
                const int i = st * kUmmaKBlocksPerSlot + j;
                if (i >= nkb) break;
                const int a = i % Cfg::kAbStages;
                const uint32_t aphase = (i / Cfg::kAbStages) & 1;
                const uint32_t scale_bits = scale_next, bias_bits = bias_next;
                if (i + Cfg::kDepth < nkb) {
                    scale_next = ldg_nc_u16(scale_row + i + Cfg::kDepth);
                    bias_next = ldg_nc_u16(bias_row + i + Cfg::kDepth);
                }
                uint4 xv[kXTasks];
#pragma unroll
                for (int q = 0; q < kXTasks; ++q) xv[q] = xv_next[q];
                if (i + Cfg::kDepth < nkb) load_x(i + Cfg::kDepth);
                if (!waited) {
                    if (!ptx::mbar_wait(&ring_full[s], phase, abort_flag, kWaitRingFull)) { alive = false; break; }
                    waited = true;
                }
                if (!ptx::mbar_wait(&ab_empty[a], aphase ^ 1, abort_flag, kWaitAbEmpty)) { alive = false; break; }
                __syncwarp();
                ptx::tc_fence_after_sync();

                // The stage is free, so the MMA of its previous k-block (handled by this same thread
                // kQueue iterations ago) is complete: start reading that partial tile back now, wait
                // for it only before the stage is handed over again, and fold it after the hand-over.
                const int q_slot = count % kQueue;
                const bool folding = count >= kQueue;
                uint32_t part[16];
                if (folding) ptx::tmem_ld16(tmem_base + lane_field + (a * kT + t) * kMPad, part);

                const uint8_t* wrow = slot + t * Cfg::kWTileBytes + r * 128;
                const uint4 w_lo = *reinterpret_cast<const uint4*>(wrow + (((2 * j) ^ (r & 7)) << 4));
                const uint4 w_hi = *reinterpret_cast<const uint4*>(wrow + (((2 * j + 1) ^ (r & 7)) << 4));
                uint32_t wq[32];
                const uint32_t words[8] = {w_lo.x, w_lo.y, w_lo.z, w_lo.w, w_hi.x, w_hi.y, w_hi.z, w_hi.w};
#pragma unroll
                for (int c = 0; c < 8; ++c) unpack_word_offset128(words[c], &wq[4 * c]);
                const uint32_t a_tmem = tmem_base + lane_field + Cfg::kAccCols + (a * kT + t) * 32;
                ptx::tmem_st16(a_tmem, &wq[0]);
                ptx::tmem_st16(a_tmem + 16, &wq[16]);

                uint8_t* b_tile = b_tiles + a * Cfg::kBBytes;
#pragma unroll
                for (int q = 0; q < kXTasks; ++q) {
                    const int task = tid + q * kKBlockThreads;
                    if (task < x_tasks) {
                        const int row = task >> 3, c = task & 7;
                        uint4 o;
                        o.x = __byte_perm(xv[q].x, xv[q].z, 0x5410);
                        o.y = __byte_perm(xv[q].x, xv[q].z, 0x7632);
                        o.z = __byte_perm(xv[q].y, xv[q].w, 0x5410);
                        o.w = __byte_perm(xv[q].y, xv[q].w, 0x7632);
                        *reinterpret_cast<uint4*>(b_tile + row * 128 + ((c ^ (row & 7)) << 4)) = o;
                    }
                }
                ptx::fence_proxy_async_smem();
                if (folding) ptx::tc_wait_ld16(part);
                ptx::tc_wait_st();
                ptx::tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&ab_full[a]);

                if (folding) {
                    publish_table();
#pragma unroll
                    for (int q = 0; q < kQueue; ++q)
                        if (q == q_slot) fold(part, pend_scale[q], pend_offset[q], pend_kb[q]);
                }
                const float scale = bf16_bits_to_f32(scale_bits), bias = bf16_bits_to_f32(bias_bits);
#pragma unroll
                for (int q = 0; q < kQueue; ++q)
                    if (q == q_slot) {
                        pend_scale[q] = scale;
                        pend_offset[q] = fmaf(-128.0f, scale, bias);  // b - 128 s: undoes the 128 in 128+q
                        pend_kb[q] = i;
                        pend_stage[q] = a;
                    }
                ++count;
            }
            if (!alive) break;
            if (!waited) {
                if (!ptx::mbar_wait(&ring_full[s], phase, abort_flag, kWaitRingFull)) break;
            }
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&ring_empty[s]);
        }

        // -------------------------------------------------------------- drain, accumulators -> smem
        __syncwarp();
        publish_table();  // warps that never folded inside the loop take the barrier here
        const bool ok = __all_sync(0xFFFFFFFFu, nkb > 0 && ptx::mbar_wait(acc_full, 0, abort_flag, kWaitAccFull));
        ptx::tc_fence_after_sync();
        if (ok) {
            const int pending = count < kQueue ? count : kQueue;
#pragma unroll
            for (int step = 0; step < kQueue; ++step) {
                if (step < pending) {
                    const int q_slot = (count - pending + step) % kQueue;  // oldest first
#pragma unroll
                    for (int q = 0; q < kQueue; ++q)
                        if (q == q_slot) {
                            uint32_t part[16];
                            ptx::tmem_ld16(tmem_base + lane_field + (pend_stage[q] * kT + t) * kMPad, part);
                            ptx::tc_wait_ld16(part);
                            fold(part, pend_scale[q], pend_offset[q], pend_kb[q]);
                        }
                }
            }
        }
        float* staging = reinterpret_cast<float*>(smem);
#pragma unroll
        for (int m = 0; m < kMPad; ++m)
            if (m < p.M) staging[((depth * kT + t) * kMPad + m) * kUmmaTileRows + r] = ok ? acc[m] : 0.0f;
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
        const int row = threadIdx.x & 127;
        const int part = threadIdx.x >> 7;
        const int n = n0 + row;
        const uint32_t staging_addr = ptx::smem_u32(smem);
        for (int m = rank + ksplit * part; m < p.M; m += ksplit * 4) {
            float first = 0.0f, second = 0.0f;
            for (int j = 0; j < ksplit; ++j) {
                const uint32_t peer = ksplit > 1 ? ptx::map_to_cta(staging_addr, (uint32_t)j) : staging_addr;
#pragma unroll
                for (int d = 0; d < Cfg::kDepth; ++d) {
                    const uint32_t base = 4u * (uint32_t)(((d * kT) * kMPad + m) * kUmmaTileRows + row);
                    if (ksplit > 1) {
                        first += ptx::ld_cluster_f32(peer + base);
                        if constexpr (kSwiglu) second += ptx::ld_cluster_f32(peer + base + 4u * kMPad * kUmmaTileRows);
                    } else {
                        const float* local = reinterpret_cast<const float*>(smem);
                        first += local[((d * kT) * kMPad + m) * kUmmaTileRows + row];
                        if constexpr (kSwiglu) second += local[((d * kT + 1) * kMPad + m) * kUmmaTileRows + row];
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

template <int kT, bool kSwiglu>
inline int launch_umma_scaled(UmmaParams& params, int tiles, cudaStream_t stream) {
    using Cfg = UmmaScaledConfig<kT>;
    auto kernel = affine_umma_scaled_kernel<kT, kSwiglu>;
    static bool configured[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (device >= 64 || !configured[device]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes) != cudaSuccess)
            return MT_ERR_LAUNCH;
        if (device < 64) configured[device] = true;
    }
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
    return cudaLaunchKernelEx(&config, kernel, params) == cudaSuccess ? MT_OK : MT_ERR_LAUNCH;
}

// x [M,K] bf16 with M <= 16.  The K split is the one the bf16-dequant family would use, so the two
// families cut the K range identically.
inline int launch_umma_scaled_any(const void* x, const AffineWeights* first, const AffineWeights* second,
                                  const void* residual, void* out, int M, int K, int N, cudaStream_t stream) {
    if (M < 1 || M > 16 || K % kUmmaBlockK || K < kUmmaBlockK || N < 1) return MT_ERR_SHAPE;
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
    params.ksplit = swiglu ? umma_ksplit<2, true, true>(tiles, slots_total) : umma_ksplit<1, true, false>(tiles, slots_total);
    const int per_cta = ((slots_total + params.ksplit - 1) / params.ksplit) * kUmmaKBlocksPerSlot;
    if (per_cta > UmmaScaledConfig<1>::kMaxKBlocks) return MT_ERR_SHAPE;
    if (!encode_weight_map(&params.w_map[0], first->w, K, N)) return MT_ERR_LAUNCH;
    if (!encode_weight_map(&params.w_map[1], swiglu ? second->w : first->w, K, N)) return MT_ERR_LAUNCH;
    return swiglu ? launch_umma_scaled<2, true>(params, tiles, stream) : launch_umma_scaled<1, false>(params, tiles, stream);
}

}  // namespace mt
