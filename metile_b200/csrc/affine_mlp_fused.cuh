// The whole INT4 affine MLP  out = down(silu(x Wg^T) * (x Wu^T)) + residual  for a single
// activation row as ONE cooperative launch that occupies HALF of every SM.
//
// Why one launch.  At one row the MLP is a pure stream of packed weights (28 MB at the
// Llama-3.2-1B shape: 4.4 us at the measured HBM rate), and two dependent kernels spend more time
// starting, ramping up their loads and draining than moving those bytes.  Here a CTA streams its rows
// of gate and up, then its rows of down, through ONE ring of shared-memory slots fed by bulk copies;
// the two projections are separated by a grid-wide barrier (every hidden activation must exist
// before any down row can be summed) and the copy engine keeps running across it, so the down rows
// are already in the ring when the barrier opens.
//
// Why half an SM.  A CTA takes 544 threads, at most 56 registers per thread and under 113 KB of
// shared memory, so the CTAs of TWO consecutive launches fit on an SM together.  With programmatic
// dependent launch the next MLP's producer warp starts as soon as this one has started, fills its
// ring (weights do not depend on the predecessor) and only its compute warps wait for this launch
// to finish.  In a chain of launches HBM is therefore busy during each launch's barrier and tail.
//
// Work split.  CTA c owns gate/up rows [c*I/grid, (c+1)*I/grid) and down rows [c*H/grid,
// (c+1)*H/grid).  A weight row of K columns is cut into K/1024 sets of 1024 columns (32 lanes x 32
// nibbles): warp w of the 16 compute warps serves set w % sets and, in every ring item, the rows
// w / sets + (16 / sets) * j.  Per-set partial sums of a row meet in shared memory and are added in
// set order, so the fp32 order depends on (H, I, grid) only.
//
// Arithmetic.  The activations sit in shared memory as fp32, transposed so that a lane reads the
// four values it needs with one conflict-free 128-bit load.  A lane turns 16 bytes of a weight row
// into the floats 128+q with one byte-permute each (the nibble becomes mantissa bits 16..19 of
// 0x43000000 = 128.0f) and multiplies them with its 32 activations by plain FMAs, two weight rows
// at a time.  Scale and bias are folded per lane:  s * dot + (b - 128 s) * (sum of the lane's
// activations);  a butterfly adds the 32 lanes.  Weights are never rounded.
//
// Ring items (all the same size, 9*H bytes): gate|up item = 8 rows of gate, 8 rows of up and their
// four 8-row blocks of scales and biases; down item = 16*H/I rows of down with their scales and
// biases.
//
// Measured and dropped on B200: a warp-level MMA variant (mma.sync m16n8k16 issues about once per
// 32 cycles per SM sub-partition, more than the FMAs cost) and the packed fma.rn.f32x2 (the
// compiler moves every unpacked weight into a register pair first, two extra instructions per weight).
#pragma once

#include <cstdlib>

#include "common.cuh"
#include "ptx.cuh"

namespace mt {

constexpr int kFusedComputeWarps = 16;
constexpr int kFusedComputeThreads = kFusedComputeWarps * 32;
constexpr int kFusedThreads = kFusedComputeThreads + 32;  // + the producer warp
constexpr int kFusedMaxRows = 1;       // activation rows
constexpr int kFusedMaxSlots = 12;
constexpr int kFusedItemRows = 8;      // gate/up rows per ring item
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
    int ring, acts, sums, scratch, bars, total;  // byte offsets
};

__host__ __device__ inline int fused_round16(int v) { return (v + 15) & ~15; }

__host__ __device__ inline FusedMlpLayout fused_mlp_layout(int H, int I, int grid) {
    FusedMlpLayout l;
    l.rows1_max = (I + grid - 1) / grid;
    l.rows2_max = (H + grid - 1) / grid;
    l.sets1 = H / 1024;
    l.sets2 = I / 1024;
    l.item_bytes = 9 * H;  // 8 rows x (H/2 gate + H/2 up) + 8 rows x 4 x H/32
    int down = (16 * H) / I;  // rows r with r * (I/2 + 2 * I/32) <= 9 * H
    if (down > 16) down = 16;
    l.down_rows = down;
    const int widest = H > I ? H : I;
    const int acts_bytes = widest * 4;         // fp32 activations of the wider projection
    const int sums_bytes = (widest / 32) * 4;  // one sum per (set, lane)
    const int floats1 = l.rows1_max * 2 * l.sets1, floats2 = l.rows2_max * l.sets2;
    const int scratch_bytes = fused_round16(4 * (floats1 > floats2 ? floats1 : floats2));
    const int bars_bytes = 8 * (2 * kFusedMaxSlots) + 16;
    const int fixed = acts_bytes + sums_bytes + scratch_bytes + bars_bytes + 128;
    int slots = (kFusedSmemBudget - fixed) / l.item_bytes;
    if (slots > kFusedMaxSlots) slots = kFusedMaxSlots;
    l.slots = slots;
    l.ring = 0;
    l.acts = l.ring + slots * l.item_bytes;
    l.sums = l.acts + acts_bytes;
    l.scratch = l.sums + sums_bytes;
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

// One activation row of `width` bf16 -> fp32 in shared memory, transposed for the compute warps:
// the four floats k = 1024 s + 32 lane + 8 j + 4 h + (0..3) live at float4 index ((4 s + j) * 2 + h) * 32 + lane,
// and sums[32 s + lane] is the sum of that lane's 32 values.  Called by all compute threads.
template <bool kFromL2>
__device__ __forceinline__ void stage_activations(const uint16_t* src, int width, float4* acts, float* sums) {
    for (int c = threadIdx.x; c < (width >> 3); c += kFusedComputeThreads) {  // 16-byte chunk = 8 values
        const uint4 v = kFromL2 ? ptx::ld_global_l2_u4(src + c * 8) : ptx::ld_global_dependent_u4(src + c * 8);
        const int s = c >> 7, lane_of = (c >> 2) & 31, j = c & 3;
        const float4 a = make_float4(bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y));
        const float4 b = make_float4(bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w));
        acts[((4 * s + j) * 2 + 0) * 32 + lane_of] = a;
        acts[((4 * s + j) * 2 + 1) * 32 + lane_of] = b;
        // Four consecutive threads hold the four words of one lane's 32 values.
        float total = ((a.x + a.y) + (a.z + a.w)) + ((b.x + b.y) + (b.z + b.w));
        total += __shfl_xor_sync(0xFFFFFFFFu, total, 1);
        total += __shfl_xor_sync(0xFFFFFFFFu, total, 2);
        if (j == 0) sums[c >> 2] = total;
    }
}

// Two weight-row shares (the 32 nibbles in pk0 and pk1, same columns) against the lane's activations.
// Returns s * sum x (128+q) + (b - 128 s) * sum x for each, still to be added over the 32 lanes.
__device__ __forceinline__ void fma_two_shares(const uint4& pk0, const uint4& pk1, uint32_t scale0, uint32_t bias0,
                                               uint32_t scale1, uint32_t bias1, const float4* acts_of_set, int lane,
                                               float lane_sum, float& out0, float& out1) {
    const uint32_t w0[4] = {pk0.x, pk0.y, pk0.z, pk0.w};
    const uint32_t w1[4] = {pk1.x, pk1.y, pk1.z, pk1.w};
    float a0[4] = {0.0f, 0.0f, 0.0f, 0.0f}, a1[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float4 xa = acts_of_set[(j * 2 + 0) * 32 + lane];
        const float4 xb = acts_of_set[(j * 2 + 1) * 32 + lane];
        const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
        float q0[8], q1[8];
        unpack_word_f32_offset128(w0[j], q0);
        unpack_word_f32_offset128(w1[j], q1);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            a0[e & 3] = fmaf(q0[e], xv[e], a0[e & 3]);
            a1[e & 3] = fmaf(q1[e], xv[e], a1[e & 3]);
        }
    }
    const float s0 = bf16_bits_to_f32(scale0), s1 = bf16_bits_to_f32(scale1);
    const float o0 = fmaf(-128.0f, s0, bf16_bits_to_f32(bias0)), o1 = fmaf(-128.0f, s1, bf16_bits_to_f32(bias1));
    out0 = fmaf(s0, (a0[0] + a0[1]) + (a0[2] + a0[3]), o0 * lane_sum);
    out1 = fmaf(s1, (a1[0] + a1[1]) + (a1[2] + a1[3]), o1 * lane_sum);
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

__global__ void __launch_bounds__(kFusedThreads, 1)
affine_mlp_fused_kernel(const __grid_constant__ FusedMlpParams p) {
    extern __shared__ uint8_t fused_smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(fused_smem_raw) + 127) & ~(uintptr_t)127);
    const int grid = gridDim.x, cta = blockIdx.x;
    const int H = p.H, I = p.I;
    const FusedMlpLayout lay = fused_mlp_layout(H, I, grid);
    uint8_t* ring = smem + lay.ring;
    float4* acts = reinterpret_cast<float4*>(smem + lay.acts);
    float* sums = reinterpret_cast<float*>(smem + lay.sums);
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
            if (use > 0 && !ptx::mbar_wait_spin(&empty_bar[slot], (uint32_t)(use - 1) & 1u, abort_flag, kWaitFusedEmpty)) break;
            __syncwarp();
            uint8_t* dst = ring + (size_t)slot * lay.item_bytes;
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
    if ((int)threadIdx.x < n2 && p.residual)
        residual_value = bf16_bits_to_f32(ptx::ld_global_dependent_u16(p.residual + row2 + threadIdx.x));
    stage_activations<false>(p.x, H, acts, sums);
    fused_compute_sync();
    MT_FUSED_STAMP(4);
    bool alive = true;
    {
        // ------------------------------------------------------------------ gate | up
        const int sets = lay.sets1, step = kFusedComputeWarps / sets;
        const int set = warp % sets, first = warp / sets;
        const int chunk = (set * 32 + lane) * 16;        // byte offset of the lane's 32 nibbles in a row
        const int group = (set * 16 + (lane >> 1)) * 2;  // byte offset of their scale in a row of scales
        const float4* acts_of_set = acts + set * 256;
        const float lane_sum = sums[set * 32 + lane];
        for (int it = 0; it < items1 && alive; ++it) {
            const int slot = it % slots, use = it / slots;
            if (!ptx::mbar_wait_spin(&full_bar[slot], (uint32_t)use & 1u, abort_flag, kWaitFusedFull)) { alive = false; break; }
            __syncwarp();
            if (it < 4) MT_FUSED_STAMP(5 + it);
            const uint8_t* item = ring + (size_t)slot * lay.item_bytes;
            const uint8_t* tables = item + 2 * kFusedItemRows * rb1;
            const int rows_here = min(kFusedItemRows, n1 - kFusedItemRows * it);
            for (int row = first; row < rows_here; row += step) {
                const uint4 pk_gate = *reinterpret_cast<const uint4*>(item + row * rb1 + chunk);
                const uint4 pk_up = *reinterpret_cast<const uint4*>(item + (kFusedItemRows + row) * rb1 + chunk);
                const uint32_t gate_s = *reinterpret_cast<const uint16_t*>(tables + (0 * kFusedItemRows + row) * sb1 + group);
                const uint32_t gate_b = *reinterpret_cast<const uint16_t*>(tables + (1 * kFusedItemRows + row) * sb1 + group);
                const uint32_t up_s = *reinterpret_cast<const uint16_t*>(tables + (2 * kFusedItemRows + row) * sb1 + group);
                const uint32_t up_b = *reinterpret_cast<const uint16_t*>(tables + (3 * kFusedItemRows + row) * sb1 + group);
                float gate, up;
                fma_two_shares(pk_gate, pk_up, gate_s, gate_b, up_s, up_b, acts_of_set, lane, lane_sum, gate, up);
#pragma unroll
                for (int offset = 16; offset >= 1; offset >>= 1) {
                    gate += __shfl_xor_sync(0xFFFFFFFFu, gate, offset);
                    up += __shfl_xor_sync(0xFFFFFFFFu, up, offset);
                }
                if (lane == 0) {
                    float* at = scratch + ((kFusedItemRows * it + row) * 2) * sets + set;
                    at[0] = gate;
                    at[sets] = up;
                }
            }
            // The slot was read with ordinary loads and will be overwritten by the copy engine.
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&empty_bar[slot]);
        }
        MT_FUSED_STAMP(9);
        fused_compute_sync();
        MT_FUSED_STAMP(10);
        for (int row = threadIdx.x; row < n1; row += kFusedComputeThreads) {
            float gate = 0.0f, up = 0.0f;
            for (int s = 0; s < sets; ++s) {
                gate += scratch[(row * 2 + 0) * sets + s];
                up += scratch[(row * 2 + 1) * sets + s];
            }
            p.hidden[row1 + row] = f32_to_bf16_bits(swiglu_f32(gate, up));
        }
    }
    MT_FUSED_STAMP(11);
    fused_grid_barrier(p.barrier, grid, abort_flag);
    MT_FUSED_STAMP(12);
    stage_activations<true>(p.hidden, I, acts, sums);
    fused_compute_sync();
    MT_FUSED_STAMP(13);
    {
        // ------------------------------------------------------------------ down
        const int sets = lay.sets2, step = kFusedComputeWarps / sets;
        const int set = warp % sets, first = warp / sets;
        const int chunk = (set * 32 + lane) * 16;
        const int group = (set * 16 + (lane >> 1)) * 2;
        const float4* acts_of_set = acts + set * 256;
        const float lane_sum = sums[set * 32 + lane];
        for (int j = 0; j < items2 && alive; ++j) {
            const int it = items1 + j;
            const int slot = it % slots, use = it / slots;
            if (!ptx::mbar_wait_spin(&full_bar[slot], (uint32_t)use & 1u, abort_flag, kWaitFusedFull)) { alive = false; break; }
            __syncwarp();
            if (j == 0) MT_FUSED_STAMP(14);
            const uint8_t* item = ring + (size_t)slot * lay.item_bytes;
            const uint8_t* tables = item + lay.down_rows * rb2;
            const int rows_here = min(lay.down_rows, n2 - lay.down_rows * j);
            for (int base = first; base < rows_here; base += 2 * step) {
                const bool pair = base + step < rows_here;
                const int other = pair ? base + step : base;  // no second row: recompute the first, discard
                const uint4 pk0 = *reinterpret_cast<const uint4*>(item + base * rb2 + chunk);
                const uint4 pk1 = *reinterpret_cast<const uint4*>(item + other * rb2 + chunk);
                const uint32_t s0 = *reinterpret_cast<const uint16_t*>(tables + base * sb2 + group);
                const uint32_t b0 = *reinterpret_cast<const uint16_t*>(tables + (lay.down_rows + base) * sb2 + group);
                const uint32_t s1 = *reinterpret_cast<const uint16_t*>(tables + other * sb2 + group);
                const uint32_t b1 = *reinterpret_cast<const uint16_t*>(tables + (lay.down_rows + other) * sb2 + group);
                float v0, v1;
                fma_two_shares(pk0, pk1, s0, b0, s1, b1, acts_of_set, lane, lane_sum, v0, v1);
#pragma unroll
                for (int offset = 16; offset >= 1; offset >>= 1) {
                    v0 += __shfl_xor_sync(0xFFFFFFFFu, v0, offset);
                    v1 += __shfl_xor_sync(0xFFFFFFFFu, v1, offset);
                }
                if (lane == 0) {
                    scratch[(lay.down_rows * j + base) * sets + set] = v0;
                    if (pair) scratch[(lay.down_rows * j + other) * sets + set] = v1;
                }
            }
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&empty_bar[slot]);
        }
        MT_FUSED_STAMP(15);
        fused_compute_sync();
        if ((int)threadIdx.x < n2) {
            const int row = threadIdx.x;
            float v = 0.0f;
            for (int s = 0; s < sets; ++s) v += scratch[row * sets + s];
            p.out[row2 + row] = f32_to_bf16_bits(v + residual_value);
        }
    }
    MT_FUSED_STAMP(16);
}

// Whether the fused kernel serves this problem on a device with `sm_count` SMs.
inline bool fused_mlp_applicable(const FusedMlpParams& p, int sm_count) {
    if (p.M != 1 || sm_count < 1) return false;
    auto supported = [](int v) { return v == 1024 || v == 2048 || v == 4096 || v == 8192 || v == 16384; };  // sets divide 16
    if (!supported(p.H) || !supported(p.I)) return false;
    const FusedMlpLayout lay = fused_mlp_layout(p.H, p.I, sm_count);
    if (lay.slots < 2 || lay.down_rows < 1) return false;
    if (lay.rows2_max > kFusedComputeThreads) return false;
    if (lay.total + 128 > kFusedSmemBudget) return false;
    const void* pointers[] = {p.x, p.gate_w, p.up_w, p.down_w, p.gate_s, p.gate_b, p.up_s, p.up_b, p.down_s, p.down_b,
                              p.hidden};
    for (const void* ptr : pointers)
        if (!aligned_to(ptr, 16)) return false;
    return true;
}

// 0 = untried, 1 = programmatic dependent launch accepted together with a cooperative launch, -1 = refused.
static int g_fused_pdl_state[64] = {};

// Caller has checked fused_mlp_applicable().
inline int launch_mlp_fused(FusedMlpParams params, int sm_count, cudaStream_t stream) {
    static unsigned long long* slots[64] = {};
    static bool configured[64] = {};
    static unsigned int launches = 0;
    auto kernel = affine_mlp_fused_kernel;
    int device = 0;
    cudaGetDevice(&device);
    if (device >= 64) return MT_ERR_DEVICE;
    const int smem = fused_mlp_layout(params.H, params.I, sm_count).total + 128;
    if (!configured[device]) {
        if (getenv("MT_FUSED_NO_PDL")) g_fused_pdl_state[device] = -1;  // diagnostic switch
        void* address = nullptr;
        if (cudaGetSymbolAddress(&address, g_fused_barrier) != cudaSuccess) return MT_ERR_LAUNCH;
        slots[device] = static_cast<unsigned long long*>(address);
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kFusedSmemBudget) != cudaSuccess)
            return MT_ERR_LAUNCH;
        cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
        int resident = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&resident, kernel, kFusedThreads, smem) != cudaSuccess || resident < 1)
            return MT_ERR_LAUNCH;
        configured[device] = true;
    }
    params.barrier = slots[device] + (__atomic_fetch_add(&launches, 1u, __ATOMIC_RELAXED) % kFusedBarrierSlots);
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

}  // namespace mt
