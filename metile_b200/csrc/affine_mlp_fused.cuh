// The whole INT4 affine MLP  out = down(silu(x Wg^T) * (x Wu^T)) + residual  for a handful of
// activation rows as ONE cooperative launch, one CTA per SM.  Two kernels share the launch structure:
// the FMA kernel described first (one to four rows, default for one) and the warp-MMA kernel
// further down (up to eight rows, default from two).
//
// Why one launch.  At a few rows the MLP is a pure stream of packed weights (28 MB at the
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
// nibbles): warp w of the compute warps serves set w % sets and, in every ring item, the share-rows
// w / sets + (warps / sets) * j.  Its activations (32 per lane and row, fp32 in registers) therefore
// never change during a projection.  Per-set partial sums of a row meet in shared memory and are added
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
// Each further activation row adds 32 FMAs per share, which is why the warp-MMA kernel takes over
// at two rows.  Also measured and dropped: the packed fma.rn.f32x2 (the compiler moves every
// unpacked weight into a register pair first, two extra instructions per weight), a bf16-pair
// unpack (same instruction count as the byte-permutes), and a half-SM variant meant to let two
// launches overlap (a cooperative launch does not start before its predecessor has drained, so
// nothing overlapped).
#pragma once

#include <cuda.h>

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
constexpr int kFusedDefaultRows = 1;   // rows the FMA kernel serves by default (measured: 16.2 / 20.1 / 22.4 us at
                                       // 1 / 2 / 3 rows against 19.3 us for the warp-MMA kernel); two to four
                                       // rows only when asked with MT_FLAG_MLP_FUSED
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
// adds exactly gridDim.x to its slot, so a slot is always a multiple of the grid size between uses --
// unless a bounded wait gave up and left its slot short; mt_device_status(reset) zeroes the slots again.
__device__ unsigned long long g_fused_barrier[kFusedBarrierSlots];

struct FusedMlpParams {
    CUtensorMap gate_map;      // warp-MMA kernel only: gate_w / up_w as [I, H/8] uint32 tensors, boxes of
    CUtensorMap up_map;        // 32 words x 16 rows with the 128-byte swizzle
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
    int M, H, I;
};

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
    if (down > 8) down -= down % 8;  // whole 8-row halves of a 16-row fragment (the warp-MMA variant needs it)
    l.down_rows = down;
    const int floats1 = l.rows1_max * 2 * l.sets1 * M, floats2 = l.rows2_max * l.sets2 * M;
    int scratch_floats = floats1 > floats2 ? floats1 : floats2;
    const int mma_floats = kFusedComputeWarps * 2 * 16 * 8;  // per-item partial tiles of the warp-MMA variant
    if (M > kFusedMaxRows && scratch_floats < mma_floats) scratch_floats = mma_floats;
    const int scratch_bytes = fused_round16(4 * scratch_floats);
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
__device__ __forceinline__ void fused_grid_barrier(unsigned long long* slot, int grid, volatile int* abort_flag,
                                                   unsigned long long limit_ns = ptx::kWaitLimitNs) {
    fused_compute_sync();  // orders this CTA's stores before thread 0's release
    if (threadIdx.x == 0) {
        // Release: this CTA's stores are visible to whoever acquires the counter afterwards; the
        // acquire loads below pair with the other CTAs' releases.
        const unsigned long long arrived = ptx::atom_add_release_gpu_u64(slot, 1ull);
        const unsigned long long target = (arrived / (unsigned long long)grid + 1ull) * (unsigned long long)grid;
        const unsigned long long start = ptx::global_timer_ns();
        while (ptx::ld_acquire_gpu_u64(slot) < target) {
            if (ptx::global_timer_ns() - start > limit_ns) {
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

// The producer warp of both kernel variants: streams the CTA's items through the ring.  Weights do
// not depend on the preceding kernel, so nothing here waits for it.  Lanes 0..5 each issue one copy.
// kTiled: the gate|up rows of an item arrive as 128-byte-wide tensor-map boxes (32 words x 16 rows, 128-byte
// swizzle; layout [matrix][H/256 column blocks][16 rows][128 B]) instead of dense rows -- what the warp-MMA
// kernel's fragment loads need to stay free of bank conflicts.  A box is always 16 rows: rows past the
// CTA's share (or past the tensor, zero-filled) are simply not used.
template <bool kTiled>
__device__ __forceinline__ void fused_producer(const FusedMlpParams& p, const FusedMlpLayout& lay, uint8_t* ring,
                                               uint64_t* full_bar, uint64_t* empty_bar, volatile int* abort_flag,
                                               int lane, int row1, int n1, int row2, int n2) {
    const int H = p.H, I = p.I;
    const int items1 = (n1 + kFusedItemRows - 1) / kFusedItemRows;
    const int items2 = (n2 + lay.down_rows - 1) / lay.down_rows;
    const int rb1 = H >> 1, rb2 = I >> 1, sb1 = H >> 5, sb2 = I >> 5;
    const int slots = lay.slots;
    for (int it = 0; it < items1 + items2; ++it) {
        const int slot = it % slots, use = it / slots;
        if (use > 0 && !ptx::mbar_wait(&empty_bar[slot], (uint32_t)(use - 1) & 1u, abort_flag, kWaitFusedEmpty)) break;
        __syncwarp();
        uint8_t* dst = ring + (size_t)slot * lay.item_bytes;
        if (it < items1) {
            const int rows = min(kFusedItemRows, n1 - kFusedItemRows * it);
            const size_t r0 = (size_t)(row1 + kFusedItemRows * it);
            if constexpr (kTiled) {
                const int blocks = H >> 8;  // 256 columns = 128 packed bytes per box
                if (lane == 0)
                    ptx::mbar_expect_tx(&full_bar[slot], (uint32_t)(2 * kFusedItemRows * rb1) + (uint32_t)rows * (uint32_t)(4 * sb1));
                __syncwarp();
                for (int box = lane; box < 2 * blocks; box += 32) {
                    const int matrix = box / blocks, block = box - matrix * blocks;
                    ptx::tma_load_2d(dst + (size_t)box * (kFusedItemRows * 128), matrix ? &p.up_map : &p.gate_map, block * 32,
                                     (int)r0, &full_bar[slot]);
                }
                if (lane >= 28) {
                    const int which = lane - 28;
                    const uint16_t* base = which == 0 ? p.gate_s : which == 1 ? p.gate_b : which == 2 ? p.up_s : p.up_b;
                    ptx::bulk_load(dst + 2 * kFusedItemRows * rb1 + which * kFusedItemRows * sb1,
                                   base + r0 * (size_t)(H >> 6), (uint32_t)rows * sb1, &full_bar[slot]);
                }
            } else {
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
}

template <int kM>
__global__ void __launch_bounds__(kFusedThreads, 1)
affine_mlp_fused_kernel(const __grid_constant__ FusedMlpParams p) {
    constexpr int kShares = kM == 1 ? 4 : 2;  // weight-row shares in flight per warp
    extern __shared__ uint8_t fused_smem_raw[];
    uint8_t* smem = fused_smem_raw + ((128u - (ptx::smem_u32(fused_smem_raw) & 127u)) & 127u);  // stays a shared-memory address
    const int grid = gridDim.x, cta = blockIdx.x;
    const int H = p.H, I = p.I;
    const FusedMlpLayout lay = fused_mlp_layout(kM, H, I, grid);
    uint8_t* ring = smem + lay.ring;
    float* scratch = reinterpret_cast<float*>(smem + lay.scratch);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + lay.bars);
    uint64_t* empty_bar = full_bar + kFusedMaxSlots;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kFusedMaxSlots);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

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
    ptx::griddep_launch_dependents();

    if (warp == kFusedComputeWarps) {
        fused_producer<false>(p, lay, ring, full_bar, empty_bar, abort_flag, lane, row1, n1, row2, n2);
        return;
    }

    // ---------------------------------------------------------------------- compute warps
    ptx::griddep_wait();  // the activations and the residual are the preceding kernel's output
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
        for (int it = 0; it < items1 && alive; ++it) {
            const int slot = it % slots, use = it / slots;
            if (!ptx::mbar_wait(&full_bar[slot], (uint32_t)use & 1u, abort_flag, kWaitFusedFull)) { alive = false; break; }
            __syncwarp();
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
            // The slot was read with ordinary loads; if the copy engine will overwrite it, order the two.
            if (it + slots < items1 + items2) {
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&empty_bar[slot]);
            }
        }
        fused_compute_sync();
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
    fused_grid_barrier(p.barrier, grid, abort_flag);
    {
        // ------------------------------------------------------------------ down
        const int sets = lay.sets2, step = kFusedComputeWarps / sets;
        const int set = warp % sets, first = warp / sets;
        const int chunk = (set * 32 + lane) * 16;
        const int group = (set * 16 + (lane >> 1)) * 2;
        LaneActivations<kM> x;
        load_lane_activations<kM, true>(p.hidden, I, set * 1024 + lane * 32, x);
        for (int j = 0; j < items2 && alive; ++j) {
            const int it = items1 + j;
            const int slot = it % slots, use = it / slots;
            if (!ptx::mbar_wait(&full_bar[slot], (uint32_t)use & 1u, abort_flag, kWaitFusedFull)) { alive = false; break; }
            __syncwarp();
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
        fused_compute_sync();
        if ((int)threadIdx.x < n2 * kM) {
            const int row = threadIdx.x / kM, m = threadIdx.x - row * kM;
            float v = 0.0f;
            for (int s = 0; s < sets; ++s) v += scratch[(row * sets + s) * kM + m];
            p.out[(size_t)m * H + row2 + row] = f32_to_bf16_bits(v + residual_value);
        }
    }
}

// ===================================================================================================
// Warp-MMA variant for four to eight activation rows.
//
// The FMA kernel above costs one FMA per weight per row, so it loses to the tensor-core path from four
// rows on.  Here the multiply runs on mma.sync (m16n8k16, bf16 in, fp32 out): the A fragment is exactly
// what the nibble unpack produces -- bf16 pairs (128+q_i, 128+q_{i+4}), 7 integer instructions per
// packed word -- and up to eight activation rows ride in the B fragment for free.  Four MMAs cover one
// quantisation group (64 k) of 16 weight rows; the group's partial sums P are folded as
// acc += s * P + (b - 128 s) * X, X = the group's activation sum, so weights stay exact.  mma.sync issues
// about once per 32 cycles per SM sub-partition on this part, which bounds the kernel near the FMA
// kernel's one-row time, independent of the row count.  The four MMAs of a group are a dependent chain,
// so four (block, group) pairs are issued round-robin; with one chain at a time the kernel took 25 us.
// The fragment loads are 64 bits per lane from four weight rows at a time; in a dense row layout those
// rows share their banks (4-way conflicts, 1.5 M extra wavefronts per launch), so the gate|up rows arrive
// as 128-byte-swizzled tensor-map boxes and fragment row g is given weight row 2 (g % 4) + g / 4, which
// makes the four rows' swizzles differ; scales and biases are read four groups per load (their rows lie
// 64 or 256 bytes apart, again in the same banks).  Measured at the Llama-3.2-1B shape: 19.2-19.5 us for
// 1-8 rows (22 us with dense rows, 20.3 us before the wide table loads) against 25.4-25.9 us on the
// two-kernel tensor-core path, so it is the default for two to eight rows.
//
// Same producer, ring and grid barrier.  The K range is cut into one slice per compute warp; every
// warp walks all rows of an item for its slice; the warps' partial 16 x 8 tiles meet in shared memory
// and are added in warp order.  Activation fragments hold element pairs in the order the unpack emits
// them: (e0,e4), (e1,e5), (e2,e6), (e3,e7).

constexpr int kFusedMmaMaxRows = 8;
constexpr int kFusedMmaMaxGroups1 = 4;  // quantisation groups of H per warp that fit in registers

__device__ __forceinline__ uint4 permute_for_fragment(uint4 v) {
    uint4 o;
    o.x = __byte_perm(v.x, v.z, 0x5410);
    o.y = __byte_perm(v.x, v.z, 0x7632);
    o.z = __byte_perm(v.y, v.w, 0x5410);
    o.w = __byte_perm(v.y, v.w, 0x7632);
    return o;
}

// Lane (g, t) loads column g's 16 activations k = 64 group + 16 t .. +15 as two fragment registers
// sets, and returns the group's sums of columns 2t and 2t+1 (x0, x1) gathered by shuffles.
template <bool kFromL2>
__device__ __forceinline__ void load_group_fragments(const uint16_t* column, bool active, int group, int t, uint4& bx0,
                                                     uint4& bx1, float& x0, float& x1) {
    uint4 v0 = make_uint4(0, 0, 0, 0), v1 = make_uint4(0, 0, 0, 0);
    if (active) {
        const uint16_t* from = column + group * 64 + t * 16;
        v0 = kFromL2 ? ptx::ld_global_l2_u4(from) : ptx::ld_global_dependent_u4(from);
        v1 = kFromL2 ? ptx::ld_global_l2_u4(from + 8) : ptx::ld_global_dependent_u4(from + 8);
    }
    bx0 = permute_for_fragment(v0);
    bx1 = permute_for_fragment(v1);
    const uint32_t words[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    float partial = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        partial += bf16_lo(words[i]);
        partial += bf16_hi(words[i]);
    }
    partial += __shfl_xor_sync(0xFFFFFFFFu, partial, 1);
    partial += __shfl_xor_sync(0xFFFFFFFFu, partial, 2);  // every lane of fragment row g holds column g's sum
    x0 = __shfl_sync(0xFFFFFFFFu, partial, 8 * t);        // lane 4 * (2t)
    x1 = __shfl_sync(0xFFFFFFFFu, partial, 8 * t + 4);    // lane 4 * (2t + 1)
}

// kN independent (16-row block, quantisation group) pairs at once: rows g (lower) and g+8 (upper) of
// each fragment.  The four MMAs of a pair form a dependent chain (they accumulate one group's partial
// sums), so the pairs' MMAs are issued round-robin to keep the tensor pipe fed.
// Four consecutive bf16 table entries (scales or biases of groups group..group+3 of one row) as one
// 64-bit load when they are 8-byte aligned, else entry by entry; entries past `count` are not read.
__device__ __forceinline__ uint2 load_four_entries(const uint8_t* row, int group, int count) {
    if (((group & 3) == 0) && count >= 4) return *reinterpret_cast<const uint2*>(row + group * 2);
    uint32_t e[4] = {0, 0, 0, 0};
#pragma unroll
    for (int i = 0; i < 4; ++i)
        if (i < count) e[i] = *reinterpret_cast<const uint16_t*>(row + (group + i) * 2);
    return make_uint2(e[0] | (e[1] << 16), e[2] | (e[3] << 16));
}
__device__ __forceinline__ uint32_t entry_of(uint2 four, int i) {
    const uint32_t word = i < 2 ? four.x : four.y;
    return (i & 1) ? word >> 16 : word & 0xFFFFu;
}

struct MmaOperand {
    const uint8_t* lower;   // this lane's 8 packed bytes of row g for the group
    const uint8_t* upper;   // ... of row g+8 (ignored without kUpper)
    uint32_t scale_lo, bias_lo, scale_hi, bias_hi;  // bf16 bits
};

template <int kN, bool kUpper>
__device__ __forceinline__ void mma_groups(const MmaOperand (&op)[kN], const uint4 (&bx0)[kN], const uint4 (&bx1)[kN],
                                           const float (&x0)[kN], const float (&x1)[kN], float* const (&acc)[kN]) {
    uint32_t lo[kN][8], hi[kN][8];
#pragma unroll
    for (int i = 0; i < kN; ++i) {
        const uint2 l = *reinterpret_cast<const uint2*>(op[i].lower);
        unpack_word_offset128(l.x, &lo[i][0]);
        unpack_word_offset128(l.y, &lo[i][4]);
        if constexpr (kUpper) {
            const uint2 h = *reinterpret_cast<const uint2*>(op[i].upper);
            unpack_word_offset128(h.x, &hi[i][0]);
            unpack_word_offset128(h.y, &hi[i][4]);
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) hi[i][k] = 0u;
        }
    }
    float d[kN][4];
#pragma unroll
    for (int i = 0; i < kN; ++i) d[i][0] = d[i][1] = d[i][2] = d[i][3] = 0.0f;
#pragma unroll
    for (int i = 0; i < kN; ++i) ptx::mma_bf16_m16n8k16(d[i], lo[i][0], hi[i][0], lo[i][1], hi[i][1], bx0[i].x, bx0[i].y);
#pragma unroll
    for (int i = 0; i < kN; ++i) ptx::mma_bf16_m16n8k16(d[i], lo[i][2], hi[i][2], lo[i][3], hi[i][3], bx0[i].z, bx0[i].w);
#pragma unroll
    for (int i = 0; i < kN; ++i) ptx::mma_bf16_m16n8k16(d[i], lo[i][4], hi[i][4], lo[i][5], hi[i][5], bx1[i].x, bx1[i].y);
#pragma unroll
    for (int i = 0; i < kN; ++i) ptx::mma_bf16_m16n8k16(d[i], lo[i][6], hi[i][6], lo[i][7], hi[i][7], bx1[i].z, bx1[i].w);
#pragma unroll
    for (int i = 0; i < kN; ++i) {
        const float s_lo = bf16_bits_to_f32(op[i].scale_lo);
        const float o_lo = fmaf(-128.0f, s_lo, bf16_bits_to_f32(op[i].bias_lo));  // undoes the 128 in 128+q
        acc[i][0] = fmaf(s_lo, d[i][0], fmaf(o_lo, x0[i], acc[i][0]));
        acc[i][1] = fmaf(s_lo, d[i][1], fmaf(o_lo, x1[i], acc[i][1]));
        if constexpr (kUpper) {
            const float s_hi = bf16_bits_to_f32(op[i].scale_hi);
            const float o_hi = fmaf(-128.0f, s_hi, bf16_bits_to_f32(op[i].bias_hi));
            acc[i][2] = fmaf(s_hi, d[i][2], fmaf(o_hi, x0[i], acc[i][2]));
            acc[i][3] = fmaf(s_hi, d[i][3], fmaf(o_hi, x1[i], acc[i][3]));
        }
    }
}

__global__ void __launch_bounds__(kFusedThreads, 1)
affine_mlp_fused_mma_kernel(const __grid_constant__ FusedMlpParams p) {
    extern __shared__ uint8_t fused_smem_raw[];
    // 1024-byte alignment: the swizzle pattern of the tensor-map boxes repeats every 1024 bytes.
    uint8_t* smem = fused_smem_raw + ((1024u - (ptx::smem_u32(fused_smem_raw) & 1023u)) & 1023u);  // stays a shared-memory address
    const int grid = gridDim.x, cta = blockIdx.x;
    const int M = p.M, H = p.H, I = p.I;
    const FusedMlpLayout lay = fused_mlp_layout(kFusedMmaMaxRows, H, I, grid);
    uint8_t* ring = smem + lay.ring;
    float* scratch = reinterpret_cast<float*>(smem + lay.scratch);
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + lay.bars);
    uint64_t* empty_bar = full_bar + kFusedMaxSlots;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + kFusedMaxSlots);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    const int row1 = (int)((unsigned)I * (unsigned)cta / (unsigned)grid);
    const int n1 = (int)((unsigned)I * (unsigned)(cta + 1) / (unsigned)grid) - row1;
    const int row2 = (int)((unsigned)H * (unsigned)cta / (unsigned)grid);
    const int n2 = (int)((unsigned)H * (unsigned)(cta + 1) / (unsigned)grid) - row2;
    const int items1 = (n1 + kFusedItemRows - 1) / kFusedItemRows;
    const int items2 = (n2 + lay.down_rows - 1) / lay.down_rows;
    const int rb1 = H >> 1, rb2 = I >> 1, sb1 = H >> 5, sb2 = I >> 5;
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
    ptx::griddep_launch_dependents();
    if (warp == kFusedComputeWarps) {
        if (lane == 0) {
            ptx::prefetch_tensor_map(&p.gate_map);
            ptx::prefetch_tensor_map(&p.up_map);
        }
        fused_producer<true>(p, lay, ring, full_bar, empty_bar, abort_flag, lane, row1, n1, row2, n2);
        return;
    }

    // ---------------------------------------------------------------------- compute warps
    ptx::griddep_wait();  // the activations and the residual are the preceding kernel's output
    float residual_value = 0.0f;
    if ((int)threadIdx.x < n2 * M && p.residual) {
        const int row = threadIdx.x / M, m = threadIdx.x - row * M;
        residual_value = bf16_bits_to_f32(ptx::ld_global_dependent_u16(p.residual + (size_t)m * H + row2 + row));
    }
    const bool active = g < M;  // fragment column g carries activation row g
    bool alive = true;
    {
        // ------------------------------------------------------------------ gate | up
        const int groups = (H >> 6) / kFusedComputeWarps;  // quantisation groups in this warp's K slice (<= 4)
        const int group0 = warp * groups;
        // Fragment row g carries weight row 2 (g % 4) + g / 4 of each 8-row half: the four rows a half-warp
        // loads at once then differ in their swizzle by 0, 2, 4, 6 and hit disjoint banks.
        const int wrow = ((g & 3) << 1) | (g >> 2);
        uint4 bx0[kFusedMmaMaxGroups1], bx1[kFusedMmaMaxGroups1];
        float x0[kFusedMmaMaxGroups1], x1[kFusedMmaMaxGroups1];
#pragma unroll
        for (int gi = 0; gi < kFusedMmaMaxGroups1; ++gi)
            if (gi < groups) load_group_fragments<false>(p.x + (size_t)(active ? g : 0) * H, active, group0 + gi, t, bx0[gi], bx1[gi], x0[gi], x1[gi]);
        for (int it = 0; it < items1; ++it) {
            const int slot = it % slots, use = it / slots;
            if (alive && !ptx::mbar_wait(&full_bar[slot], (uint32_t)use & 1u, abort_flag, kWaitFusedFull)) alive = false;
            alive = __all_sync(0xFFFFFFFFu, alive);  // the MMAs and shuffles below need the whole warp or none of it
            const uint8_t* item = ring + (size_t)slot * lay.item_bytes;
            const uint8_t* tables = item + 2 * kFusedItemRows * rb1;
            const int rows_here = min(kFusedItemRows, n1 - kFusedItemRows * it);
            const bool upper = rows_here > 8;
            float acc[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
            if (alive) {
                // This warp's scales and biases of the item: rows wrow and wrow + 8, gate and up, four groups each.
                uint2 sc4[2][2], bi4[2][2];  // [matrix][lower / upper]
#pragma unroll
                for (int matrix = 0; matrix < 2; ++matrix)
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        const int row = wrow + 8 * half;
                        const bool present = half == 0 || upper;
                        sc4[matrix][half] = present ? load_four_entries(tables + ((2 * matrix) * kFusedItemRows + row) * sb1, group0, groups)
                                                    : make_uint2(0, 0);
                        bi4[matrix][half] = present ? load_four_entries(tables + ((2 * matrix + 1) * kFusedItemRows + row) * sb1, group0, groups)
                                                    : make_uint2(0, 0);
                    }
                // Two groups x (gate, up) = four independent MMA chains per step.  A second group past
                // the slice's end repeats the first one into a discarded accumulator.
#pragma unroll
                for (int gi = 0; gi < kFusedMmaMaxGroups1; gi += 2) {
                    if (gi < groups) {
                        const bool second = gi + 1 < groups;
                        float discard[4];
                        MmaOperand op[4];
                        uint4 fx0[4], fx1[4];
                        float fs0[4], fs1[4];
                        float* into[4];
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            const int matrix = c & 1, which = (c >> 1) && second ? gi + 1 : gi;
                            const int group = group0 + which;
                            // Box (matrix, group / 4), row `wrow`, 16-byte chunk (group % 4) * 2 + t / 2 XOR-swizzled
                            // by the row; rows wrow and wrow + 8 share the swizzle.
                            const int chunk = (((group & 3) << 1) | (t >> 1)) ^ (wrow & 7);
                            op[c].lower = item + (size_t)((matrix * (H >> 8) + (group >> 2)) * kFusedItemRows + wrow) * 128 +
                                          (chunk << 4) + (t & 1) * 8;
                            op[c].upper = op[c].lower + 8 * 128;
                            op[c].scale_lo = entry_of(sc4[matrix][0], which);
                            op[c].bias_lo = entry_of(bi4[matrix][0], which);
                            op[c].scale_hi = entry_of(sc4[matrix][1], which);
                            op[c].bias_hi = entry_of(bi4[matrix][1], which);
                            fx0[c] = (c >> 1) && second ? bx0[(gi + 1) % kFusedMmaMaxGroups1] : bx0[gi];
                            fx1[c] = (c >> 1) && second ? bx1[(gi + 1) % kFusedMmaMaxGroups1] : bx1[gi];
                            fs0[c] = (c >> 1) && second ? x0[(gi + 1) % kFusedMmaMaxGroups1] : x0[gi];
                            fs1[c] = (c >> 1) && second ? x1[(gi + 1) % kFusedMmaMaxGroups1] : x1[gi];
                            into[c] = (c >> 1) && !second ? discard : acc[matrix];
                        }
                        // The two chains of one matrix add into the same accumulators: fold the second
                        // group's pair after the first by giving it its own accumulators.
                        float later[2][4] = {{0.0f, 0.0f, 0.0f, 0.0f}, {0.0f, 0.0f, 0.0f, 0.0f}};
                        if (second) { into[2] = later[0]; into[3] = later[1]; }
                        if (upper) mma_groups<4, true>(op, fx0, fx1, fs0, fs1, into);
                        else mma_groups<4, false>(op, fx0, fx1, fs0, fs1, into);
                        if (second) {
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                acc[0][k] += later[0][k];
                                acc[1][k] += later[1][k];
                            }
                        }
                    }
                }
            }
            if (it + slots < items1 + items2) {
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&empty_bar[slot]);
            }
            // scratch[((warp * 2 + matrix) * 16 + row) * 8 + column]
#pragma unroll
            for (int matrix = 0; matrix < 2; ++matrix) {
                float* tile = scratch + (size_t)((warp * 2 + matrix) * 16) * 8;
                *reinterpret_cast<float2*>(tile + wrow * 8 + 2 * t) = make_float2(acc[matrix][0], acc[matrix][1]);
                *reinterpret_cast<float2*>(tile + (wrow + 8) * 8 + 2 * t) = make_float2(acc[matrix][2], acc[matrix][3]);
            }
            fused_compute_sync();
            for (int idx = threadIdx.x; idx < rows_here * M; idx += kFusedComputeThreads) {
                const int row = idx / M, m = idx - row * M;
                float gate = 0.0f, up = 0.0f;
                for (int w = 0; w < kFusedComputeWarps; ++w) {
                    gate += scratch[((w * 2 + 0) * 16 + row) * 8 + m];
                    up += scratch[((w * 2 + 1) * 16 + row) * 8 + m];
                }
                p.hidden[(size_t)m * I + row1 + kFusedItemRows * it + row] = f32_to_bf16_bits(swiglu_f32(gate, up));
            }
            fused_compute_sync();
        }
    }
    fused_grid_barrier(p.barrier, grid, abort_flag);
    {
        // ------------------------------------------------------------------ down
        const int groups = (I >> 6) / kFusedComputeWarps;
        const int group0 = warp * groups;
        const uint16_t* column = p.hidden + (size_t)(active ? g : 0) * I;
        const int tiles = (n2 + 15) >> 4;
        int released = 0;  // down items handed back to the producer so far
        for (int tile = 0; tile < tiles; ++tile) {
            // Rows 16 tile + g (lower) and 16 tile + 8 + g (upper) of this CTA's down rows, wherever
            // their items sit in the ring.
            const int r_lo = 16 * tile, r_hi = 16 * tile + 8;
            const bool upper = r_hi < n2;
            const int j_lo = r_lo / lay.down_rows, j_hi = upper ? r_hi / lay.down_rows : j_lo;
            for (int j = j_lo; j <= j_hi; ++j) {
                const int it = items1 + j;
                if (alive && !ptx::mbar_wait(&full_bar[it % slots], (uint32_t)(it / slots) & 1u, abort_flag, kWaitFusedFull))
                    alive = false;
            }
            alive = __all_sync(0xFFFFFFFFu, alive);
            const uint8_t* item_lo = ring + (size_t)((items1 + j_lo) % slots) * lay.item_bytes;
            const uint8_t* item_hi = ring + (size_t)((items1 + j_hi) % slots) * lay.item_bytes;
            const int local_lo = r_lo - j_lo * lay.down_rows + g, local_hi = r_hi - j_hi * lay.down_rows + g;
            const uint8_t* lower = item_lo + local_lo * rb2 + t * 8;
            const uint8_t* upper_row = item_hi + local_hi * rb2 + t * 8;
            const uint8_t* sc_lo = item_lo + lay.down_rows * rb2 + local_lo * sb2;
            const uint8_t* sc_hi = item_hi + lay.down_rows * rb2 + local_hi * sb2;
            const int table = lay.down_rows * sb2;  // biases follow the scales
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (alive) {
                // Four groups = four independent MMA chains per step; their activation fragments come
                // from L2 one step ahead.  Chains past the slice's end repeat the step's first group
                // into a discarded accumulator.
                uint4 bx0[4], bx1[4], nx0[4], nx1[4];
                float x0[4], x1[4], y0[4], y1[4];
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    load_group_fragments<true>(column, active, group0 + (c < groups ? c : 0), t, bx0[c], bx1[c], x0[c], x1[c]);
                for (int gi = 0; gi < groups; gi += 4) {
                    if (gi + 4 < groups) {
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            load_group_fragments<true>(column, active, group0 + (gi + 4 + c < groups ? gi + 4 + c : gi + 4), t,
                                                       nx0[c], nx1[c], y0[c], y1[c]);
                    }
                    MmaOperand op[4];
                    float part[4][4];
                    float* into[4];
                    const int step_groups = min(4, groups - gi);
                    const uint2 s_lo4 = load_four_entries(sc_lo, group0 + gi, step_groups);
                    const uint2 b_lo4 = load_four_entries(sc_lo + table, group0 + gi, step_groups);
                    const uint2 s_hi4 = upper ? load_four_entries(sc_hi, group0 + gi, step_groups) : make_uint2(0, 0);
                    const uint2 b_hi4 = upper ? load_four_entries(sc_hi + table, group0 + gi, step_groups) : make_uint2(0, 0);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int within = gi + c < groups ? c : 0;
                        const int group = group0 + gi + within;
                        op[c].lower = lower + group * 32;
                        op[c].upper = upper_row + group * 32;
                        op[c].scale_lo = entry_of(s_lo4, within);
                        op[c].bias_lo = entry_of(b_lo4, within);
                        op[c].scale_hi = entry_of(s_hi4, within);
                        op[c].bias_hi = entry_of(b_hi4, within);
                        part[c][0] = part[c][1] = part[c][2] = part[c][3] = 0.0f;
                        into[c] = part[c];
                    }
                    if (upper) mma_groups<4, true>(op, bx0, bx1, x0, x1, into);
                    else mma_groups<4, false>(op, bx0, bx1, x0, x1, into);
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        if (gi + c < groups) {
#pragma unroll
                            for (int k = 0; k < 4; ++k) acc[k] += part[c][k];
                        }
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        bx0[c] = nx0[c]; bx1[c] = nx1[c]; x0[c] = y0[c]; x1[c] = y1[c];
                    }
                }
            }
            // Hand back the items that end inside this tile.
            while (released < items2 && (released + 1) * lay.down_rows <= 16 * (tile + 1)) {
                const int it = items1 + released;
                if (it + slots < items1 + items2) {
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(&empty_bar[it % slots]);
                }
                ++released;
            }
            float* part = scratch + (size_t)(warp * 16) * 8;  // scratch[(warp * 16 + row) * 8 + column]
            *reinterpret_cast<float2*>(part + g * 8 + 2 * t) = make_float2(acc[0], acc[1]);
            *reinterpret_cast<float2*>(part + (g + 8) * 8 + 2 * t) = make_float2(acc[2], acc[3]);
            fused_compute_sync();
            const int rows_here = min(16, n2 - 16 * tile);
            for (int idx = threadIdx.x; idx < rows_here * M; idx += kFusedComputeThreads) {
                const int row = idx / M, m = idx - row * M;
                float v = 0.0f;
                for (int w = 0; w < kFusedComputeWarps; ++w) v += scratch[(w * 16 + row) * 8 + m];
                // The residual was fetched by thread (16 tile + row) * M + m, which is this one only in the
                // first tile; later tiles read it here.
                const size_t at = (size_t)m * H + row2 + 16 * tile + row;
                float extra = residual_value;
                if (tile > 0) extra = p.residual ? bf16_bits_to_f32(ptx::ld_global_dependent_u16(p.residual + at)) : 0.0f;
                p.out[at] = f32_to_bf16_bits(v + extra);
            }
            fused_compute_sync();
        }
    }
}

// Whether the warp-MMA variant serves this problem.
inline bool fused_mlp_mma_applicable(const FusedMlpParams& p, int sm_count) {
    if (p.M < 1 || p.M > kFusedMmaMaxRows || sm_count < 1) return false;
    if (p.H < 512 || p.H % (64 * kFusedComputeWarps) || (p.H >> 6) / kFusedComputeWarps > kFusedMmaMaxGroups1) return false;
    if (p.I < 512 || p.I % (64 * kFusedComputeWarps)) return false;
    const FusedMlpLayout lay = fused_mlp_layout(kFusedMmaMaxRows, p.H, p.I, sm_count);
    if (lay.slots < 2 || lay.down_rows < 8 || lay.down_rows % 8) return false;
    if (16 * p.M > kFusedComputeThreads) return false;
    if (p.H % 256 || lay.item_bytes % 1024) return false;  // whole tensor-map boxes, swizzle-aligned items
    if (lay.total + 1024 > kFusedSmemBudget) return false;
    const void* pointers[] = {p.x, p.gate_w, p.up_w, p.down_w, p.gate_s, p.gate_b, p.up_s, p.up_b, p.down_s, p.down_b,
                              p.hidden};
    for (const void* ptr : pointers)
        if (!aligned_to(ptr, 16)) return false;
    return true;
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

// `kKind` only separates the per-kernel static state (1..4 = FMA kernel rows, 0 = warp-MMA kernel).
template <int kKind>
inline int launch_mlp_fused_kernel(void (*kernel)(const FusedMlpParams), int smem, const FusedMlpParams& params,
                                   int sm_count, int device, cudaStream_t stream) {
    static bool configured[64] = {};
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

template <int kM>
inline int launch_mlp_fused_rows(const FusedMlpParams& params, int sm_count, int device, cudaStream_t stream) {
    const int smem = fused_mlp_layout(kM, params.H, params.I, sm_count).total + 128;
    return launch_mlp_fused_kernel<kM>(affine_mlp_fused_kernel<kM>, smem, params, sm_count, device, stream);
}

// The barrier slot of the next launch on the current device (slots rotate, one per launch in flight).
inline unsigned long long* next_fused_barrier_slot() {
    static unsigned long long* slots[64] = {};
    static unsigned int launches = 0;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return nullptr;
    if (!slots[device]) {
        void* address = nullptr;
        if (cudaGetSymbolAddress(&address, g_fused_barrier) != cudaSuccess) return nullptr;
        slots[device] = static_cast<unsigned long long*>(address);
    }
    return slots[device] + (__atomic_fetch_add(&launches, 1u, __ATOMIC_RELAXED) % kFusedBarrierSlots);
}

// Caller has checked fused_mlp_applicable(), or fused_mlp_mma_applicable() when `mma` is set.
inline int launch_mlp_fused(FusedMlpParams params, int sm_count, bool mma, cudaStream_t stream) {
    int device = 0;
    cudaGetDevice(&device);
    if (device >= 64) return MT_ERR_DEVICE;
    params.barrier = next_fused_barrier_slot();
    if (!params.barrier) return MT_ERR_LAUNCH;
    if (mma) {
        if (!encode_weight_map(&params.gate_map, params.gate_w, params.H, params.I, kFusedItemRows) ||
            !encode_weight_map(&params.up_map, params.up_w, params.H, params.I, kFusedItemRows))
            return MT_ERR_LAUNCH;
        const int smem = fused_mlp_layout(kFusedMmaMaxRows, params.H, params.I, sm_count).total + 1024;
        return launch_mlp_fused_kernel<0>(affine_mlp_fused_mma_kernel, smem, params, sm_count, device, stream);
    }
    switch (params.M) {
        case 1: return launch_mlp_fused_rows<1>(params, sm_count, device, stream);
        case 2: return launch_mlp_fused_rows<2>(params, sm_count, device, stream);
        case 3: return launch_mlp_fused_rows<3>(params, sm_count, device, stream);
        case 4: return launch_mlp_fused_rows<4>(params, sm_count, device, stream);
        default: return MT_ERR_SHAPE;
    }
}

}  // namespace mt
