// Decode attention (one query row per sequence and head) over an in-place KV cache, grouped-query
// aware, plus the rotary embedding + cache append that precedes it in a decoder block.
//
// Computes what the reference's kernels/attention.py:27-143 computes -- softmax(q.k * scale) @ v per
// (batch, query head), query head h reading KV head h / (Hq / Hkv) (:41-44), every load cast to fp32
// before it is multiplied (:58-62), fp32 accumulation, one rounding at the store -- behind the
// admission rule of metile/integrations/mlx_lm.py:3558-3573 (query length one, no mask, equal K/V
// shapes, head dim a multiple of 32).  The reference launches one threadgroup per (batch, QUERY head),
// so a KV head's keys and values are streamed once per query head of its group; here one CTA serves
// every query head of a KV head, so each cache byte is read once.
//
// Split over the KV range ("flash decoding"): CTA (s, b*Hkv + h) takes tokens [128 s, 128 s + 128) of
// one (sequence, KV head).  Its key and value tiles (35 KB each at head dim 128, rows padded by 16
// bytes) are copied to shared memory by 16-byte asynchronous copies issued before anything else, so
// the whole tile pair is in flight at once; the arithmetic runs on the tensor cores (see the kernel):
// scores K . Q^T with the KV head's query-head group as the N dimension, softmax on the score
// fragments in registers, values P . V with the probabilities split into two bf16 numbers; the CTA's
// partial (max, sum, O) goes to the caller's scratch and a second kernel merges the splits in split
// order.  The reference multiplies fp32 casts of the same bf16 inputs (:58-62); the products are
// exact either way, the sums are fp32, and the scale multiplies the fp32 score instead of the query.
// The split size is a constant, so a (sequence, head)'s bits depend on its own KV length only -- not
// on how many sequences share the launch.
//
// Bytes: K and V rows of the tokens in use, 2 * B * Hkv * N * D * 2; everything else is noise.
#pragma once

#include "common.cuh"
#include "ptx.cuh"

namespace mt {

constexpr int kAttnSplitTokens = 128;  // tokens per CTA: four groups of 32 lanes
constexpr int kAttnMaxGroup = 8;       // query heads per KV head

struct AttentionParams {
    const uint16_t* q;        // [B, Hq, D] bf16
    const uint16_t* k;        // [B, Hkv, capacity, D] bf16
    const uint16_t* v;
    const int* lengths;       // [B] tokens in use per sequence, or null: `tokens` for all
    float* partial;           // [B*Hkv, splits, G, D + 2] fp32 (caller scratch); unused when splits == 1
    uint16_t* out;            // [B, Hq, D] bf16
    int q_heads, kv_heads, capacity, tokens, splits;
    float scale;
};

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* global_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(ptx::smem_u32(smem_dst)), "l"(global_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(kPending) : "memory");
}

constexpr int kAttnThreads = 256;
constexpr int kAttnRowPad = 8;  // bf16 elements: a tile row in shared memory is 16 bytes longer than in the cache

template <int kD>
constexpr int attention_smem_bytes() {
    return 2 * kAttnSplitTokens * (kD + kAttnRowPad) * 2;  // key tile + value tile
}

// Four 8x8 b16 matrices from shared memory into the fragment layout of mma.sync (lane l supplies the
// address of row l % 8 of matrix l / 8); `trans` delivers each matrix transposed.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(ptx::smem_u32(row)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(ptx::smem_u32(row)));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t (&r)[2], const void* row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];"
                 : "=r"(r[0]), "=r"(r[1]) : "r"(ptx::smem_u32(row)));
}
// D += A (16x16, row) * B (16x8, col), bf16 inputs, fp32 accumulate.
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The arithmetic runs on the tensor cores (mma.sync m16n8k16, bf16 x bf16 -> fp32):
//   scores : S[16 tokens x 8 heads] = K[16 x D] . Q^T[D x 8]  -- the query-head group of a KV head (up to 8
//            heads) is the N dimension; warp w owns tokens [16 w, 16 w + 16); keys and queries enter as the
//            bf16 numbers they are and the scale multiplies the fp32 sums;
//   softmax: one warp per head over the split's 128 scores (shared memory), fp32; the probabilities are
//            written as TWO bf16 numbers hi + lo (relative error 2^-17), so that the second product runs
//            on the tensor cores without giving up the fp32 probabilities of the reference;
//   values : O[8 heads x D] = P[8 x 128 tokens] . V[128 x D]  -- warp w owns D / 8 head-dim columns, the value
//            tile is read with transposing matrix loads, hi and lo are two MMAs into one accumulator.
// Measured against the CUDA-core form of the same kernel (one token per lane, FMAs against the queries in
// shared memory), which spent two thirds of its instructions on converts and shared-memory reads.
template <int kD, int kG>
__global__ void __launch_bounds__(kAttnThreads) attention_decode_split_kernel(const AttentionParams p) {
    constexpr int kRow = kD + kAttnRowPad;   // elements; the 16 bytes of padding keep matrix loads conflict-free
    constexpr int kSlices = kD / 16;         // k-steps of the score product
    constexpr int kColsPerWarp = kD / 8;     // head-dim columns a warp owns in the value product (16 or 8)
    constexpr int kNTiles = kColsPerWarp / 8;
    constexpr int kProbRow = kAttnSplitTokens + 8;
    extern __shared__ __align__(16) uint16_t tiles[];
    uint16_t* key_tile = tiles;                                // [128][kRow]
    uint16_t* value_tile = tiles + kAttnSplitTokens * kRow;    // [128][kRow]
    __shared__ __align__(16) uint16_t prob_hi[8][kProbRow], prob_lo[8][kProbRow];
    __shared__ float warp_max[8][8], warp_sum[8][8];           // [warp][head]

    const int split = blockIdx.x;
    const int bh = blockIdx.y;                     // b * Hkv + h
    const int b = bh / p.kv_heads, h = bh - b * p.kv_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;         // fragment coordinates
    ptx::griddep_launch_dependents();
    ptx::griddep_wait();                           // q and the newest cache row are the preceding kernels' output
    const int n = p.lengths ? p.lengths[b] : p.tokens;
    const size_t cache_row0 = ((size_t)bh * p.capacity) * kD;
    const int split_first = split * kAttnSplitTokens;
    const int rows = min(kAttnSplitTokens, n - split_first);  // tokens of this split in use (<= 0: none)
    // A split past the sequence's end has nothing to do and the merge never reads its partial (callers
    // pass whole caches with the lengths on the device, so most splits of a short sequence are such).
    if (rows <= 0 && p.splits > 1) return;

    // Both tiles are requested at once, 16 bytes per copy: every byte this CTA will read is in flight
    // before any arithmetic starts.  Two groups, so the score phase can begin when the keys are in.
    constexpr int kChunks = kD / 8;
    for (int c = threadIdx.x; c < rows * kChunks; c += kAttnThreads) {
        const int row = c / kChunks, chunk = c - row * kChunks;
        cp_async_16(key_tile + row * kRow + chunk * 8, p.k + cache_row0 + (size_t)(split_first + row) * kD + chunk * 8);
    }
    cp_async_commit();
    for (int c = threadIdx.x; c < rows * kChunks; c += kAttnThreads) {
        const int row = c / kChunks, chunk = c - row * kChunks;
        cp_async_16(value_tile + row * kRow + chunk * 8, p.v + cache_row0 + (size_t)(split_first + row) * kD + chunk * 8);
    }
    cp_async_commit();
    // Rows past the sequence's end enter the value product with probability zero; their bytes must
    // still be numbers (0 x NaN is NaN).  Key rows past the end only produce scores that are masked.
    const int first_unused = max(rows, 0);
    for (int c = threadIdx.x; c < (kAttnSplitTokens - first_unused) * kChunks; c += kAttnThreads) {
        const int row = first_unused + c / kChunks, chunk = c % kChunks;
        *reinterpret_cast<uint4*>(value_tile + row * kRow + chunk * 8) = make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(key_tile + row * kRow + chunk * 8) = make_uint4(0u, 0u, 0u, 0u);
    }

    // Query fragments (the B operand of the score product): head g, dims 16 s + 2 t (+1) and + 8.
    uint32_t qf[kSlices][2];
    {
        const uint16_t* qrow = p.q + ((size_t)b * p.q_heads + (size_t)h * kG + min(g, kG - 1)) * kD;
#pragma unroll
        for (int s = 0; s < kSlices; ++s) {
            uint32_t lo, hi;
            asm volatile("ld.global.u32 %0, [%1];" : "=r"(lo) : "l"(qrow + 16 * s + 2 * t));
            asm volatile("ld.global.u32 %0, [%1];" : "=r"(hi) : "l"(qrow + 16 * s + 2 * t + 8));
            qf[s][0] = g < kG ? lo : 0u;
            qf[s][1] = g < kG ? hi : 0u;
        }
    }
    cp_async_wait<1>();
    __syncthreads();

    // ---------------------------------------------------------------- scores: 16 tokens per warp
    // c0, c1: token 16 w + g, heads 2 t and 2 t + 1; c2, c3: token 16 w + g + 8.  The scores stay in
    // these registers through the softmax; only the per-warp maxima and sums meet in shared memory.
    float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    {
        const uint16_t* a_row = key_tile + (16 * warp + (lane & 15)) * kRow + 8 * (lane >> 4);
#pragma unroll
        for (int s = 0; s < kSlices; ++s) {
            uint32_t a[4];
            ldmatrix_x4(a, a_row + 16 * s);
            mma_bf16_16816(c, a, qf[s][0], qf[s][1]);
        }
    }
    const int token0 = 16 * warp + g, token1 = token0 + 8;
    c[0] = token0 < rows ? c[0] * p.scale : -INFINITY;
    c[1] = token0 < rows ? c[1] * p.scale : -INFINITY;
    c[2] = token1 < rows ? c[2] * p.scale : -INFINITY;
    c[3] = token1 < rows ? c[3] * p.scale : -INFINITY;
    {
        float even = fmaxf(c[0], c[2]), odd = fmaxf(c[1], c[3]);   // heads 2 t and 2 t + 1 over this lane's tokens
#pragma unroll
        for (int offset = 4; offset <= 16; offset <<= 1) {        // over g: the warp's 16 tokens
            even = fmaxf(even, __shfl_xor_sync(0xFFFFFFFFu, even, offset));
            odd = fmaxf(odd, __shfl_xor_sync(0xFFFFFFFFu, odd, offset));
        }
        if (g == 0) {
            warp_max[warp][2 * t] = even;
            warp_max[warp][2 * t + 1] = odd;
        }
    }
    __syncthreads();
    // ---------------------------------------------------------------- softmax over the split's 128 tokens
    {
        float m_even = warp_max[0][2 * t], m_odd = warp_max[0][2 * t + 1];
#pragma unroll
        for (int w = 1; w < 8; ++w) {
            m_even = fmaxf(m_even, warp_max[w][2 * t]);
            m_odd = fmaxf(m_odd, warp_max[w][2 * t + 1]);
        }
        // Masked tokens: exp(-inf - m) = 0; a split with no token at all has m = -inf and contributes 0.
        const float e0 = m_even == -INFINITY ? 0.0f : __expf(c[0] - m_even);
        const float e1 = m_odd == -INFINITY ? 0.0f : __expf(c[1] - m_odd);
        const float e2 = m_even == -INFINITY ? 0.0f : __expf(c[2] - m_even);
        const float e3 = m_odd == -INFINITY ? 0.0f : __expf(c[3] - m_odd);
        float even = e0 + e2, odd = e1 + e3;
#pragma unroll
        for (int offset = 4; offset <= 16; offset <<= 1) {
            even += __shfl_xor_sync(0xFFFFFFFFu, even, offset);
            odd += __shfl_xor_sync(0xFFFFFFFFu, odd, offset);
        }
        if (g == 0) {
            warp_sum[warp][2 * t] = even;
            warp_sum[warp][2 * t + 1] = odd;
        }
        // The probabilities as hi + lo (two bf16 numbers each), [head][token]; heads past the group get
        // zeros (their queries were zero, so e = exp(0 - 0) = 1 must not reach the padded rows).
        const float e[4] = {e0, e1, e2, e3};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int head = 2 * t + (i & 1), token = i < 2 ? token0 : token1;
            const float value = head < kG ? e[i] : 0.0f;
            const uint16_t hi = f32_to_bf16_bits(value);
            prob_hi[head][token] = hi;
            prob_lo[head][token] = f32_to_bf16_bits(value - bf16_bits_to_f32(hi));
        }
    }
    cp_async_wait<0>();
    __syncthreads();  // values have landed and every probability is written
    // ---------------------------------------------------------------- values: D / 8 columns per warp
    float acc[kNTiles][4];
#pragma unroll
    for (int nt = 0; nt < kNTiles; ++nt)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[nt][i] = 0.0f;
    const int dim0 = warp * kColsPerWarp;
#pragma unroll
    for (int ks = 0; ks < kAttnSplitTokens / 16; ++ks) {
        if (16 * ks >= rows) break;  // whole k-steps past the end contribute nothing
        // A operand: P[head g][tokens 16 ks + 2 t (+1)] and + 8; rows 8..15 of the 16-row tile are zero.
        uint32_t a_hi[4], a_lo[4];
        a_hi[0] = *reinterpret_cast<const uint32_t*>(&prob_hi[g][16 * ks + 2 * t]);
        a_hi[2] = *reinterpret_cast<const uint32_t*>(&prob_hi[g][16 * ks + 2 * t + 8]);
        a_lo[0] = *reinterpret_cast<const uint32_t*>(&prob_lo[g][16 * ks + 2 * t]);
        a_lo[2] = *reinterpret_cast<const uint32_t*>(&prob_lo[g][16 * ks + 2 * t + 8]);
        a_hi[1] = a_hi[3] = a_lo[1] = a_lo[3] = 0u;
        if constexpr (kNTiles == 2) {
            uint32_t bfrag[4];
            ldmatrix_x4_trans(bfrag, value_tile + (16 * ks + (lane & 7) + ((lane >> 3) & 1) * 8) * kRow + dim0 + 8 * (lane >> 4));
            mma_bf16_16816(acc[0], a_hi, bfrag[0], bfrag[1]);
            mma_bf16_16816(acc[0], a_lo, bfrag[0], bfrag[1]);
            mma_bf16_16816(acc[1], a_hi, bfrag[2], bfrag[3]);
            mma_bf16_16816(acc[1], a_lo, bfrag[2], bfrag[3]);
        } else {
            uint32_t bfrag[2];
            ldmatrix_x2_trans(bfrag, value_tile + (16 * ks + (lane & 7) + ((lane >> 3) & 1) * 8) * kRow + dim0);
            mma_bf16_16816(acc[0], a_hi, bfrag[0], bfrag[1]);
            mma_bf16_16816(acc[0], a_lo, bfrag[0], bfrag[1]);
        }
    }
    // acc[nt][0], [1]: head g, dims dim0 + 8 nt + 2 t (+1); [2], [3] belong to the padded heads.
    if (g < kG) {
        float m = warp_max[0][g], total = warp_sum[0][g];
#pragma unroll
        for (int w = 1; w < 8; ++w) {   // the eight warps' sums in warp order
            m = fmaxf(m, warp_max[w][g]);
            total += warp_sum[w][g];
        }
#pragma unroll
        for (int nt = 0; nt < kNTiles; ++nt) {
            const int d = dim0 + 8 * nt + 2 * t;
            if (p.splits == 1) {
                const size_t at = ((size_t)b * p.q_heads + (size_t)h * kG + g) * kD + d;
                const uint32_t pair = pack_bf16x2(acc[nt][0] / total, acc[nt][1] / total);
                *reinterpret_cast<uint32_t*>(p.out + at) = pair;
            } else {
                float* row = p.partial + (((size_t)bh * p.splits + split) * kG + g) * (kD + 2);
                row[d] = acc[nt][0];
                row[d + 1] = acc[nt][1];
                if (d == 0) {
                    row[kD] = m;
                    row[kD + 1] = total;
                }
            }
        }
    }
}

// Merges the splits of one (sequence, query head) in split order.
template <int kD>
__global__ void __launch_bounds__(kD) attention_decode_merge_kernel(const AttentionParams p, int group) {
    const int bq = blockIdx.x;                      // b * Hq + query head
    const int b = bq / p.q_heads, qh = bq - b * p.q_heads;
    const int h = qh / group, g = qh - h * group;
    const int d = threadIdx.x;
    ptx::griddep_launch_dependents();
    ptx::griddep_wait();
    const int n = p.lengths ? p.lengths[b] : p.tokens;
    const int used = min(p.splits, (n + kAttnSplitTokens - 1) / kAttnSplitTokens);
    const float* base = p.partial + (((size_t)(b * p.kv_heads + h) * p.splits) * group + g) * (kD + 2);
    const size_t stride = (size_t)group * (kD + 2);
    float m = -INFINITY;
    for (int s = 0; s < used; ++s) m = fmaxf(m, base[s * stride + kD]);
    float total = 0.0f, value = 0.0f;
    for (int s = 0; s < used; ++s) {
        const float factor = __expf(base[s * stride + kD] - m);
        total = fmaf(base[s * stride + kD + 1], factor, total);
        value = fmaf(base[s * stride + d], factor, value);
    }
    p.out[(size_t)bq * kD + d] = f32_to_bf16_bits(value / total);
}

inline int attention_splits(int tokens) { return tokens <= 0 ? 1 : (tokens + kAttnSplitTokens - 1) / kAttnSplitTokens; }

inline size_t attention_workspace_bytes(int batch, int q_heads, int tokens, int head_dim) {
    const int splits = attention_splits(tokens);
    if (splits <= 1) return 0;
    return (size_t)batch * q_heads * splits * (head_dim + 2) * sizeof(float);
}

template <int kD, int kG>
inline int launch_attention_instance(const AttentionParams& params, int batch, cudaStream_t stream) {
    static bool configured[64] = {};
    int device = 0;
    cudaGetDevice(&device);
    if (device >= 64 || !configured[device]) {
        if (cudaFuncSetAttribute(attention_decode_split_kernel<kD, kG>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 attention_smem_bytes<kD>()) != cudaSuccess)
            return MT_ERR_LAUNCH;
        if (device < 64) configured[device] = true;
    }
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(params.splits, batch * params.kv_heads, 1);
    config.blockDim = dim3(kAttnThreads, 1, 1);
    config.dynamicSmemBytes = attention_smem_bytes<kD>();
    config.stream = stream;
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attrs;
    config.numAttrs = 1;
    if (cudaLaunchKernelEx(&config, attention_decode_split_kernel<kD, kG>, params) != cudaSuccess) return MT_ERR_LAUNCH;
    if (params.splits > 1) {
        config.gridDim = dim3(batch * params.q_heads, 1, 1);
        config.blockDim = dim3(kD, 1, 1);
        config.dynamicSmemBytes = 0;
        if (cudaLaunchKernelEx(&config, attention_decode_merge_kernel<kD>, params, kG) != cudaSuccess)
            return MT_ERR_LAUNCH;
    }
    return MT_OK;
}

template <int kD>
inline int launch_attention_dim(const AttentionParams& params, int batch, int group, cudaStream_t stream) {
    switch (group) {
        case 1: return launch_attention_instance<kD, 1>(params, batch, stream);
        case 2: return launch_attention_instance<kD, 2>(params, batch, stream);
        case 3: return launch_attention_instance<kD, 3>(params, batch, stream);
        case 4: return launch_attention_instance<kD, 4>(params, batch, stream);
        case 5: return launch_attention_instance<kD, 5>(params, batch, stream);
        case 6: return launch_attention_instance<kD, 6>(params, batch, stream);
        case 7: return launch_attention_instance<kD, 7>(params, batch, stream);
        case 8: return launch_attention_instance<kD, 8>(params, batch, stream);
        default: return MT_ERR_SHAPE;
    }
}

// ---------------------------------------------------------------------------------------------
// Rotary embedding (half-split pairs (i, i + D/2), angle = position * theta^(-2i/D)) of the new
// query and key rows, and the append of the rotated key and of the value at `position` of each
// sequence's cache.  One CTA per (sequence, head) over Hq + 2 Hkv heads; thread i owns pair i.
struct RopeAppendParams {
    const uint16_t* q;        // [B, Hq, D], consecutive sequences `row_stride` elements apart
    const uint16_t* k;        // [B, Hkv, D], same stride
    const uint16_t* v;        // [B, Hkv, D], same stride
    const int* positions;     // [B]
    uint16_t* q_out;          // [B, Hq, D]
    uint16_t* k_cache;        // [B, Hkv, capacity, D]
    uint16_t* v_cache;
    int q_heads, kv_heads, capacity, head_dim;
    long long row_stride;     // elements between sequences in q, k and v (one fused q|k|v row, or dense)
    float log2_theta;
};

__global__ void rope_kv_append_kernel(const RopeAppendParams p) {
    const int heads = p.q_heads + 2 * p.kv_heads;
    const int b = blockIdx.x / heads, slot = blockIdx.x - b * heads;
    const int dim = p.head_dim, half = dim >> 1;
    ptx::griddep_launch_dependents();
    ptx::griddep_wait();
    const int position = p.positions[b];
    if (slot >= p.q_heads + p.kv_heads) {  // value row: a plain copy into the cache
        const int h = slot - p.q_heads - p.kv_heads;
        const uint16_t* from = p.v + (size_t)b * p.row_stride + (size_t)h * dim;
        uint16_t* to = p.v_cache + (((size_t)b * p.kv_heads + h) * p.capacity + position) * dim;
        for (int d = threadIdx.x; d < dim; d += blockDim.x) to[d] = ptx::ld_global_dependent_u16(from + d);
        return;
    }
    const bool is_query = slot < p.q_heads;
    const int h = is_query ? slot : slot - p.q_heads;
    const uint16_t* from = (is_query ? p.q : p.k) + (size_t)b * p.row_stride + (size_t)h * dim;
    uint16_t* to = is_query ? p.q_out + ((size_t)b * p.q_heads + h) * dim
                            : p.k_cache + (((size_t)b * p.kv_heads + h) * p.capacity + position) * dim;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        // theta^(-2i/D) = 2^(-(2i/D) log2 theta); sincosf on position * that, in fp32.
        const float inverse = exp2f(-(2.0f * (float)i / (float)dim) * p.log2_theta);
        float s, c;
        sincosf((float)position * inverse, &s, &c);
        const float first = bf16_bits_to_f32(ptx::ld_global_dependent_u16(from + i));
        const float second = bf16_bits_to_f32(ptx::ld_global_dependent_u16(from + i + half));
        to[i] = f32_to_bf16_bits(first * c - second * s);
        to[i + half] = f32_to_bf16_bits(second * c + first * s);
    }
}

}  // namespace mt
