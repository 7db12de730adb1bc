// The whole INT4 affine MLP  out = down(silu(x Wg^T) * (x Wu^T)) + residual  for a single
// activation row as ONE cooperative launch, one CTA per SM.
//
// Why one launch.  At one row the MLP is a pure stream of packed weights (28 MB at the
// Llama-3.2-1B shape: 4.4 us at the measured HBM rate), and two dependent kernels spend more time
// starting, ramping up their loads and draining than moving those bytes.  Here a CTA streams its rows
// of gate and up, then its rows of down, through ONE ring of shared-memory slots fed by bulk copies.
// At the Llama-3.2-1B shape the ring holds the CTA's whole share (6 items of 36 KB), so every
// weight byte of the MLP is requested in the first microsecond and HBM stays busy while the
// arithmetic runs behind the copies; larger shapes reuse slots.  The two projections are separated
// by a grid-wide barrier (every hidden activation must exist before any down row can be summed);
// the down rows are already in the ring when the barrier opens.
//
// Work split.  CTA c owns gate/up rows [c*I/grid, (c+1)*I/grid) and down rows [c*H/grid,
// (c+1)*H/grid).  A weight row of K columns is cut into K/1024 sets of 1024 columns (32 lanes x 32
// nibbles): warp w of the compute warps serves set w % sets and, in every ring item, the rows
// w / sets + (warps / sets) * j.  Its activations (32 per lane, fp32 in registers) therefore never
// change during a projection.  Per-set partial sums of a row meet in shared memory and are added
// in set order, so the fp32 order depends on (H, I, grid) only.
//
// Arithmetic.  A lane turns 16 bytes of a weight row into the floats 128+q with one byte-permute
// each (the nibble becomes mantissa bits 16..19 of 0x43000000 = 128.0f) and multiplies them with
// its 32 activations by plain FMAs, four weight-row shares at a time so that their dependency
// chains overlap.  Scale and bias are folded per lane:  s * dot + (b - 128 s) * (sum of the lane's
// activations);  a butterfly adds the 32 lanes.  Weights are never rounded.
//
// Ring items (all the same size): gate|up item = 16 rows of gate, 16 rows of up and their four
// 16-row blocks of scales and biases (18*H bytes); down item = 32*H/I rows of down with their
// scales and biases.
//
// What bounds it (measured on B200).  One weight-row share costs about 76 instructions per warp
// (32 byte-permutes, 32 FMAs, masks, scale fold, butterfly) and the SM sub-partition sustains about
// 0.7 of them per cycle, so the MLP's 50 M weights take about 5 us of instruction issue per SM --
// more than the 4.4 us the bytes take.  Eight compute warps with 146 registers beat sixteen with 96.
// Also measured and dropped: a warp-level MMA variant (mma.sync m16n8k16 issues about once per 32
// cycles per SM sub-partition), the packed fma.rn.f32x2 (the compiler moves every unpacked weight
// into a register pair first, two extra instructions per weight), a bf16-pair unpack (same
// instruction count as the byte-permutes), and a half-SM variant meant to let two launches overlap
// (a cooperative launch does not start before its predecessor has drained, so nothing overlapped).
#pragma once

#include <cstdlib>

#include "common.cuh"
#include "ptx.cuh"

namespace mt {

#ifndef MT_FUSED_WARPS
#define MT_FUSED_WARPS 8
#endif
#ifndef MT_FUSED_ITEM_ROWS
#define MT_FUSED_ITEM_ROWS 16
#endif
constexpr int kFusedComputeWarps = MT_FUSED_WARPS;
constexpr int kFusedComputeThreads = kFusedComputeWarps * 32;
constexpr int kFusedThreads = kFusedComputeThreads + 32;  // + the producer warp
constexpr int kFusedMaxRows = 4;       // activation rows (each lane keeps 32 fp32 activations per row in registers)
constexpr int kFusedDefaultRows = 3;   // rows served by default (measured faster than the two-kernel path up to
                                       // three rows); four rows only when asked with MT_FLAG_MLP_FUSED
constexpr int kFusedMaxSlots = 12;
constexpr int kFusedItemRows = MT_FUSED_ITEM_ROWS;  // gate/up rows per ring item
constexpr int kFusedSmemBudget = 226 * 1024;  // one CTA per SM
constexpr int kFusedBarrierSlots = 64;

enum FusedWaitCode : unsigned int {
    kWaitFusedFull = 0x201,
    kWaitFusedEmpty = 0x202,
    kWaitFusedGrid = 0x203,
};

// Grid-barrier counters, one slot per launch in flight (launch n uses slot n % 64).  Every launch
// adds exactly gridDim.x to its slot, so a slot is always a multiple of the grid size between uses.
__device__ unsigned long long g_fused_barrier[kFusedBarrierSlots];

struct FusedMlpParams {
    const uint16_t* x;         // [1, H] bf16
    const uint32_t* gate_w;    // [I, H/8]
    const uint32_t* up_w;      // [I, H/8]
    const uint32_t* down_w;    // [H, I/8]
    const uint16_t* gate_s;    // [I, H/64]
    const uint16_t* gate_b;
    const uint16_t* up_s;
    const uint16_t* up_b;
    const uint16_t* down_s;    // [H, I/64]
    const uint16_t* down_b;
    const uint16_t* residual;  // [1, H] or null
    uint16_t* hidden;          // [1, I] bf16, written then read
    uint16_t* out;             // [1, H]
    unsigned long long* barrier;
    long long* timeline;       // diagnostic phase stamps of CTA 0 (only in MT_TIMELINE builds), else null
    int M, H, I;
};

#ifdef MT_TIMELINE
#define MT_FUSED_STAMP(slot)                                                                         \
    do {                                                                                             \
        if (p.timeline != nullptr && blockIdx.x == 0 && threadIdx.x == 0) p.timeline[slot] = clock64(); \
    } while (0)
#else
#define MT_FUSED_STAMP(slot) do { } while (0)
#endif

struct FusedMlpLayout {
    int rows1_max, rows2_max;  // most rows any CTA owns in each projection
    int sets1, sets2;          // 1024-column sets per weight row
    int item_bytes, slots;     // ring geometry
    int down_rows;             // down rows per ring item
    int ring, scratch, bars, total;  // byte offsets
};

__host__ __device__ inline int fused_round16(int v) { return (v + 15) & ~15; }

__host__ __device__ inline FusedMlpLayout fused_mlp_layout(int M, int H, int I, int grid) {
    FusedMlpLayout l;
    l.rows1_max = (I + grid - 1) / grid;
    l.rows2_max = (H + grid - 1) / grid;
    l.sets1 = H / 1024;
    l.sets2 = I / 1024;
    l.item_bytes = kFusedItemRows * (H + H / 8);  // rows x (H/2 gate + H/2 up) + rows x 4 x H/32
    int down = (2 * kFusedItemRows * H) / I;      // rows r with r * (I/2 + 2 * I/32) <= item_bytes
    if (down > 2 * kFusedItemRows) down = 2 * kFusedItemRows;
    l.down_rows = down;
    const int floats1 = l.rows1_max * 2 * l.sets1 * M, floats2 = l.rows2_max * l.sets2 * M;
    const int scratch_bytes = fused_round16(4 * (floats1 > floats2 ? floats1 : floats2));
    const int bars_bytes = 8 * (2 * kFusedMaxSlots) + 16;
    const int fixed = scratch_bytes + bars_bytes + 128;
    int slots = (kFusedSmemBudget - fixed) / l.item_bytes;
    if (slots > kFusedMaxSlots) slots = kFusedMaxSlots;
    l.slots = slots;
    l.ring = 0;
    l.scratch = l.ring + slots * l.item_bytes;
    l.bars = l.scratch + scratch_bytes;
    l.total = l.bars + bars_bytes;
    return l;
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

// Barrier among the compute warps only (the producer warp keeps feeding the ring).
__device__ __forceinline__ void fused_compute_sync() {
    asm volatile("bar.sync 1, %0;" ::"r"(kFusedComputeThreads) : "memory");
}

// The lane's 32 consecutive activations starting at column k0 of each of kM rows, as fp32 in
// registers, and their sums.
template <int kM>
struct LaneActivations {
    float value[kM][32];
    float sum[kM];
};

template <int kM, bool kFromL2>
__device__ __forceinline__ void load_lane_activations(const uint16_t* src, int width, int k0, LaneActivations<kM>& x) {
#pragma unroll
    for (int m = 0; m < kM; ++m) {
        const uint16_t* from = src + (size_t)m * width + k0;
        uint4 v[4];
#pragma unroll
        for (int c = 0; c < 4; ++c) v[c] = kFromL2 ? ptx::ld_global_l2_u4(from + c * 8) : ptx::ld_global_dependent_u4(from + c * 8);
        float total = 0.0f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const uint32_t words[4] = {v[c].x, v[c].y, v[c].z, v[c].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                x.value[m][8 * c + 2 * i] = bf16_lo(words[i]);
                x.value[m][8 * c + 2 * i + 1] = bf16_hi(words[i]);
                total += bf16_lo(words[i]);
                total += bf16_hi(words[i]);
            }
        }
        x.sum[m] = total;
    }
}

// kN weight-row shares (32 nibbles each, same columns) against the lane's activations, interleaved so
// that their dependency chains overlap.  out[i][m] = s_i * sum x_m (128+q_i) + (b_i - 128 s_i) * sum x_m,
// added over the 32 lanes by a butterfly.  The unpacked weights are shared by the kM activation rows.
template <int kN, int kM>
__device__ __forceinline__ void fma_shares(const uint4 (&pk)[kN], const uint32_t (&scale_bits)[kN],
                                           const uint32_t (&bias_bits)[kN], const LaneActivations<kM>& x,
                                           float (&out)[kN][kM]) {
    constexpr int kChains = 4;  // independent accumulators per (share, row); the same for every kM, so a
                                // row's fp32 order does not depend on how many rows share the launch
    float a[kN][kM][kChains];
#pragma unroll
    for (int i = 0; i < kN; ++i)
#pragma unroll
        for (int m = 0; m < kM; ++m)
#pragma unroll
            for (int c = 0; c < kChains; ++c) a[i][m][c] = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
#pragma unroll
        for (int i = 0; i < kN; ++i) {
            const uint32_t word = j == 0 ? pk[i].x : j == 1 ? pk[i].y : j == 2 ? pk[i].z : pk[i].w;
            float q[8];
            unpack_word_f32_offset128(word, q);
#pragma unroll
            for (int e = 0; e < 8; ++e)
#pragma unroll
                for (int m = 0; m < kM; ++m)
                    a[i][m][e % kChains] = fmaf(q[e], x.value[m][8 * j + e], a[i][m][e % kChains]);
        }
    }
#pragma unroll
    for (int i = 0; i < kN; ++i) {
        const float scale = bf16_bits_to_f32(scale_bits[i]);
        const float offset = fmaf(-128.0f, scale, bf16_bits_to_f32(bias_bits[i]));
#pragma unroll
        for (int m = 0; m < kM; ++m) {
            const float dot = (a[i][m][0] + a[i][m][1]) + (a[i][m][2] + a[i][m][3]);
            out[i][m] = fmaf(scale, dot, offset * x.sum[m]);
        }
    }
#pragma unroll
    for (int offset = 16; offset >= 1; offset >>= 1)
#pragma unroll
        for (int i = 0; i < kN; ++i)
#pragma unroll
            for (int m = 0; m < kM; ++m) out[i][m] += __shfl_xor_sync(0xFFFFFFFFu, out[i][m], offset);
}

// The grid-wide barrier, called by the compute warps: every CTA arrives once; the slot grows by
// gridDim.x per launch.
__device__ __forceinline__ void fused_grid_barrier(unsigned long long* slot, int grid, volatile int* abort_flag) {
    fused_compute_sync();  // orders this CTA's stores before thread 0's release
    if (threadIdx.x == 0) {
        // Release: this CTA's stores are visible to whoever acquires the counter afterwards; the
        // acquire loads below pair with the other CTAs' releases.
        const unsigned long long arrived = ptx::atom_add_release_gpu_u64(slot, 1ull);
        const unsigned long long target = (arrived / (unsigned long long)grid + 1ull) * (unsigned long long)grid;
        const unsigned long long start = ptx::global_timer_ns();
        while (ptx::ld_acquire_gpu_u64(slot) < target) {
            if (ptx::global_timer_ns() - start > ptx::kWaitLimitNs) {
                if (atomicCAS(&g_device_status[0], 0u, (unsigned int)kWaitFusedGrid) == 0u) {
                    g_device_status[1] = blockIdx.x;
                    g_device_status[2] = threadIdx.x;
                    g_device_status[3] = 0;
                }
                *abort_flag = 1;
                break;
            }
        }
    }
    fused_compute_sync();
}

template <int kM>
__global__ void __launch_bounds__(kFusedThreads, 1)
affine_mlp_fused_kernel(const __grid_constant__ FusedMlpParams p) {
    constexpr int kShares = kM == 1 ? 4 : 2;  // weight-row shares in flight per warp
    extern __shared__ uint8_t fused_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fused_smem_raw) + 127) & ~(uintptr_t)127);
    const int grid = gridDim.x, cta = blockIdx.x;
    const int H = p.H, I = p.I;
    const FusedMlpLayout lay = fused_mlp_layout(kM, H, I, grid);
    uint8_t* ring = smem + lay.ring;
    float* scratch = reinterpret_cast<float*>(smem + lay.scratch);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + lay.bars);
    uint64_t* empty_bar = full_bar + kFusedMaxSlots;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kFusedMaxSlots);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    MT_FUSED_STAMP(0);

    const int row1 = (int)((unsigned)I * (unsigned)cta / (unsigned)grid);
    const int n1 = (int)((unsigned)I * (unsigned)(cta + 1) / (unsigned)grid) - row1;
    const int row2 = (int)((unsigned)H * (unsigned)cta / (unsigned)grid);
    const int n2 = (int)((unsigned)H * (unsigned)(cta + 1) / (unsigned)grid) - row2;
    const int items1 = (n1 + kFusedItemRows - 1) / kFusedItemRows;
    const int items2 = (n2 + lay.down_rows - 1) / lay.down_rows;
    const int rb1 = H >> 1, rb2 = I >> 1;  // bytes of a packed weight row
    const int sb1 = H >> 5, sb2 = I >> 5;  // bytes of a row of scales (or biases)
    const int slots = lay.slots;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kFusedMaxSlots; ++i) {
            ptx::mbar_init(&full_bar[i], 1);
            ptx::mbar_init(&empty_bar[i], kFusedComputeWarps);
        }
        *abort_flag = 0;
        ptx::mbar_fence_init();
    }
    __syncthreads();
    MT_FUSED_STAMP(1);
    ptx::griddep_launch_dependents();

    if (warp == kFusedComputeWarps) {
        // ------------------------------------------------------------------ producer warp
        // Weights do not depend on the preceding kernel, so nothing here waits for it.  Lanes 0..5
        // each issue one copy of an item.
        for (int it = 0; it < items1 + items2; ++it) {
            const int slot = it % slots, use = it / slots;
            if (use > 0 && !ptx::mbar_wait(&empty_bar[slot], (uint32_t)(use - 1) & 1u, abort_flag, kWaitFusedEmpty)) break;
            __syncwarp();
            uint8_t* dst = ring + (size_t)slot * lay.item_bytes;
#ifdef MT_TIMELINE
            if (p.timeline != nullptr && blockIdx.x == 0 && lane == 0 && it < 12) p.timeline[30 + it] = clock64();
#endif
            if (it < items1) {
                const int rows = min(kFusedItemRows, n1 - kFusedItemRows * it);
                const size_t r0 = (size_t)(row1 + kFusedItemRows * it);
                if (lane == 0) ptx::mbar_expect_tx(&full_bar[slot], (uint32_t)rows * (uint32_t)(2 * rb1 + 4 * sb1));
                __syncwarp();
                if (lane < 2) {
                    const uint32_t* src = (lane ? p.up_w : p.gate_w) + r0 * (size_t)(H >> 3);
                    ptx::bulk_load(dst + lane * kFusedItemRows * rb1, src, (uint32_t)rows * rb1, &full_bar[slot]);
                } else if (lane < 6) {
                    const uint16_t* base = lane == 2 ? p.gate_s : lane == 3 ? p.gate_b : lane == 4 ? p.up_s : p.up_b;
                    ptx::bulk_load(dst + 2 * kFusedItemRows * rb1 + (lane - 2) * kFusedItemRows * sb1,
                                   base + r0 * (size_t)(H >> 6), (uint32_t)rows * sb1, &full_bar[slot]);
                }
            } else {
                const int j = it - items1;
                const int rows = min(lay.down_rows, n2 - lay.down_rows * j);
                const size_t r0 = (size_t)(row2 + lay.down_rows * j);
                if (lane == 0) ptx::mbar_expect_tx(&full_bar[slot], (uint32_t)rows * (uint32_t)(rb2 + 2 * sb2));
                __syncwarp();
                if (lane == 0) {
                    ptx::bulk_load(dst, p.down_w + r0 * (size_t)(I >> 3), (uint32_t)rows * rb2, &full_bar[slot]);
                } else if (lane < 3) {
                    const uint16_t* base = lane == 1 ? p.down_s : p.down_b;
                    ptx::bulk_load(dst + lay.down_rows * rb2 + (lane - 1) * lay.down_rows * sb2,
                                   base + r0 * (size_t)(I >> 6), (uint32_t)rows * sb2, &full_bar[slot]);
                }
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- compute warps
    ptx::griddep_wait();  // the activations and the residual are the preceding kernel's output
    MT_FUSED_STAMP(3);
    float residual_value = 0.0f;  // fetched now, used at the very end
    if ((int)threadIdx.x < n2 * kM && p.residual) {
        const int row = threadIdx.x / kM, m = threadIdx.x - row * kM;
        residual_value = bf16_bits_to_f32(ptx::ld_global_dependent_u16(p.residual + (size_t)m * H + row2 + row));
    }
    bool alive = true;
    {
        // ------------------------------------------------------------------ gate | up
        // A step of a warp = kShares of the item's 2 * rows share-rows (share-row 2 r + matrix).
        const int sets = lay.sets1, step = kFusedComputeWarps / sets;
        const int set = warp % sets, first = warp / sets;
        const int chunk = (set * 32 + lane) * 16;        // byte offset of the lane's 32 nibbles in a row
        const int group = (set * 16 + (lane >> 1)) * 2;  // byte offset of their scale in a row of scales
        LaneActivations<kM> x;
        load_lane_activations<kM, false>(p.x, H, set * 1024 + lane * 32, x);
        MT_FUSED_STAMP(4);
        for (int it = 0; it < items1 && alive; ++it) {
            const int slot = it % slots, use = it / slots;
            if (!ptx::mbar_wait(&full_bar[slot], (uint32_t)use & 1u, abort_flag, kWaitFusedFull)) { alive = false; break; }
            __syncwarp();
            if (it < 4) MT_FUSED_STAMP(5 + it);
            const uint8_t* item = ring + (size_t)slot * lay.item_bytes;
            const uint8_t* tables = item + 2 * kFusedItemRows * rb1;
            const int share_rows = 2 * min(kFusedItemRows, n1 - kFusedItemRows * it);
            for (int base = first; base < share_rows; base += kShares * step) {
                uint4 pk[kShares];
                uint32_t scale_bits[kShares], bias_bits[kShares];
                int where[kShares];  // share-row, or the first one again past the end (computed, discarded)
#pragma unroll
                for (int i = 0; i < kShares; ++i) {
                    where[i] = base + i * step < share_rows ? base + i * step : base;
                    const int row = where[i] >> 1, matrix = where[i] & 1;
                    pk[i] = *reinterpret_cast<const uint4*>(item + (matrix * kFusedItemRows + row) * rb1 + chunk);
                    scale_bits[i] = *reinterpret_cast<const uint16_t*>(tables + ((2 * matrix) * kFusedItemRows + row) * sb1 + group);
                    bias_bits[i] = *reinterpret_cast<const uint16_t*>(tables + ((2 * matrix + 1) * kFusedItemRows + row) * sb1 + group);
                }
                float part[kShares][kM];
                fma_shares<kShares, kM>(pk, scale_bits, bias_bits, x, part);
                if (lane == 0) {
#pragma unroll
                    for (int i = 0; i < kShares; ++i)
                        if (base + i * step < share_rows) {
#pragma unroll
                            for (int m = 0; m < kM; ++m)
                                scratch[((2 * kFusedItemRows * it + where[i]) * sets + set) * kM + m] = part[i][m];
                        }
                }
            }
            if (it < 8) MT_FUSED_STAMP(20 + it);
            // The slot was read with ordinary loads; if the copy engine will overwrite it, order the two.
            if (it + slots < items1 + items2) {
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&empty_bar[slot]);
            }
        }
        MT_FUSED_STAMP(9);
        fused_compute_sync();
        MT_FUSED_STAMP(10);
        for (int idx = threadIdx.x; idx < n1 * kM; idx += kFusedComputeThreads) {
            const int row = idx / kM, m = idx - row * kM;
            float gate = 0.0f, up = 0.0f;
            for (int s = 0; s < sets; ++s) {
                gate += scratch[((2 * row + 0) * sets + s) * kM + m];
                up += scratch[((2 * row + 1) * sets + s) * kM + m];
            }
            p.hidden[(size_t)m * I + row1 + row] = f32_to_bf16_bits(swiglu_f32(gate, up));
        }
    }
    MT_FUSED_STAMP(11);
    fused_grid_barrier(p.barrier, grid, abort_flag);
    MT_FUSED_STAMP(12);
    {
        // ------------------------------------------------------------------ down
        const int sets = lay.sets2, step = kFusedComputeWarps / sets;
        const int set = warp % sets, first = warp / sets;
        const int chunk = (set * 32 + lane) * 16;
        const int group = (set * 16 + (lane >> 1)) * 2;
        LaneActivations<kM> x;
        load_lane_activations<kM, true>(p.hidden, I, set * 1024 + lane * 32, x);
        MT_FUSED_STAMP(13);
        for (int j = 0; j < items2 && alive; ++j) {
            const int it = items1 + j;
            const int slot = it % slots, use = it / slots;
            if (!ptx::mbar_wait(&full_bar[slot], (uint32_t)use & 1u, abort_flag, kWaitFusedFull)) { alive = false; break; }
            __syncwarp();
            if (j == 0) MT_FUSED_STAMP(14);
            const uint8_t* item = ring + (size_t)slot * lay.item_bytes;
            const uint8_t* tables = item + lay.down_rows * rb2;
            const int rows_here = min(lay.down_rows, n2 - lay.down_rows * j);
            for (int base = first; base < rows_here; base += kShares * step) {
                uint4 pk[kShares];
                uint32_t scale_bits[kShares], bias_bits[kShares];
                int rows[kShares];
#pragma unroll
                for (int i = 0; i < kShares; ++i) {
                    rows[i] = base + i * step < rows_here ? base + i * step : base;  // past the end: recompute, discard
                    pk[i] = *reinterpret_cast<const uint4*>(item + rows[i] * rb2 + chunk);
                    scale_bits[i] = *reinterpret_cast<const uint16_t*>(tables + rows[i] * sb2 + group);
                    bias_bits[i] = *reinterpret_cast<const uint16_t*>(tables + (lay.down_rows + rows[i]) * sb2 + group);
                }
                float part[kShares][kM];
                fma_shares<kShares, kM>(pk, scale_bits, bias_bits, x, part);
                if (lane == 0) {
#pragma unroll
                    for (int i = 0; i < kShares; ++i)
                        if (base + i * step < rows_here) {
#pragma unroll
                            for (int m = 0; m < kM; ++m)
                                scratch[((lay.down_rows * j + rows[i]) * sets + set) * kM + m] = part[i][m];
                        }
                }
            }
            if (it + slots < items1 + items2) {
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&empty_bar[slot]);
            }
        }
        MT_FUSED_STAMP(15);
        fused_compute_sync();
        if ((int)threadIdx.x < n2 * kM) {
            const int row = threadIdx.x / kM, m = threadIdx.x - row * kM;
            float v = 0.0f;
            for (int s = 0; s < sets; ++s) v += scratch[(row * sets + s) * kM + m];
            p.out[(size_t)m * H + row2 + row] = f32_to_bf16_bits(v + residual_value);
        }
    }
    MT_FUSED_STAMP(16);
}

// Whether the fused kernel serves this problem on a device with `sm_count` SMs.
inline bool fused_mlp_applicable(const FusedMlpParams& p, int sm_count) {
    if (p.M < 1 || p.M > kFusedMaxRows || sm_count < 1) return false;
    auto supported = [](int v) {  // a whole number of 1024-column sets that divides the compute warps
        return v >= 1024 && v % 1024 == 0 && kFusedComputeWarps % (v / 1024) == 0;
    };
    if (!supported(p.H) || !supported(p.I)) return false;
    const FusedMlpLayout lay = fused_mlp_layout(p.M, p.H, p.I, sm_count);
    if (lay.slots < 2 || lay.down_rows < 1) return false;
    if (lay.rows2_max * p.M > kFusedComputeThreads) return false;
    if (lay.total + 128 > kFusedSmemBudget) return false;
    const void* pointers[] = {p.x, p.gate_w, p.up_w, p.down_w, p.gate_s, p.gate_b, p.up_s, p.up_b, p.down_s, p.down_b,
                              p.hidden};
    for (const void* ptr : pointers)
        if (!aligned_to(ptr, 16)) return false;
    return true;
}

// 0 = untried, 1 = programmatic dependent launch accepted together with a cooperative launch, -1 = refused.
static int g_fused_pdl_state[64] = {};

template <int kM>
inline int launch_mlp_fused_rows(const FusedMlpParams& params, int sm_count, int device, cudaStream_t stream) {
    static bool configured[64] = {};
    auto kernel = affine_mlp_fused_kernel<kM>;
    const int smem = fused_mlp_layout(kM, params.H, params.I, sm_count).total + 128;
    if (!configured[device]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFusedSmemBudget) != cudaSuccess)
            return MT_ERR_LAUNCH;
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        int resident = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, kFusedThreads, smem) != cudaSuccess || resident < 1)
            return MT_ERR_LAUNCH;
        configured[device] = true;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(sm_count, 1, 1);
    config.blockDim = dim3(kFusedThreads, 1, 1);
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeCooperative;  // all CTAs resident together: they meet at a grid barrier
    attrs[0].val.cooperative = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attrs;
    // Whether the two attributes combine is decided by one trial launch outside stream capture (a
    // refused launch would invalidate a capture); until then captures use the cooperative attribute alone.
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(stream, &capturing);
    if (g_fused_pdl_state[device] == 0 && capturing == cudaStreamCaptureStatusNone) {
        config.numAttrs = 2;
        if (cudaLaunchKernelEx(&config, kernel, params) == cudaSuccess) {
            g_fused_pdl_state[device] = 1;
            return MT_OK;
        }
        cudaGetLastError();
        g_fused_pdl_state[device] = -1;
    }
    config.numAttrs = g_fused_pdl_state[device] == 1 ? 2 : 1;
    return cudaLaunchKernelEx(&config, kernel, params) == cudaSuccess ? MT_OK : MT_ERR_LAUNCH;
}

// Caller has checked fused_mlp_applicable().
inline int launch_mlp_fused(FusedMlpParams params, int sm_count, cudaStream_t stream) {
    static unsigned long long* slots[64] = {};
    static unsigned int launches = 0;
    int device = 0;
    cudaGetDevice(&device);
    if (device >= 64) return MT_ERR_DEVICE;
    if (!slots[device]) {
        if (getenv("MT_FUSED_NO_PDL")) g_fused_pdl_state[device] = -1;  // diagnostic switch
        void* address = nullptr;
        if (cudaGetSymbolAddress(&address, g_fused_barrier) != cudaSuccess) return MT_ERR_LAUNCH;
        slots[device] = static_cast<unsigned long long*>(address);
    }
    params.barrier = slots[device] + (__atomic_fetch_add(&launches, 1u, __ATOMIC_RELAXED) % kFusedBarrierSlots);
    switch (params.M) {
        case 1: return launch_mlp_fused_rows<1>(params, sm_count, device, stream);
        case 2: return launch_mlp_fused_rows<2>(params, sm_count, device, stream);
        case 3: return launch_mlp_fused_rows<3>(params, sm_count, device, stream);
        case 4: return launch_mlp_fused_rows<4>(params, sm_count, device, stream);
        default: return MT_ERR_SHAPE;
    }
}

}  // namespace mt
