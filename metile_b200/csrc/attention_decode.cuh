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
// one (sequence, KV head).  Its key and value tiles (32 KB each at head dim 128) are copied to
// shared memory by 16-byte asynchronous copies issued before anything else, so the whole 64 KB is in
// flight at once; a warp takes 32 tokens, one token per lane, and half of the group's query heads.
//   scores : the lane reads ITS token's key row from shared memory (rows padded by 16 bytes: no bank
//            conflicts) and multiplies it with the scaled query rows, which sit in shared memory as
//            fp32 (broadcast reads).  No shuffles.
//   softmax: per query head, maximum and sum over the warp's 32 tokens by butterfly; probabilities
//            go to shared memory.
//   values : lanes now own head-dim slices (coalesced 256-byte rows) and accumulate
//            O[g][d] += p[token][g] * V[token][d] over the warp's tokens.
//   merge  : the four warps' (max, sum, O) are merged in warp order, the CTA's partial goes to the
//            caller's scratch, and a second kernel merges the splits in split order.
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
constexpr int kAttnKeyPad = 8;  // bf16 elements: a key row in shared memory is 16 bytes longer than in the cache

template <int kD>
constexpr int attention_smem_bytes() {
    return kAttnSplitTokens * (kD + kAttnKeyPad) * 2 + kAttnSplitTokens * kD * 2;
}

// Eight warps: warp w works on tokens [32 (w % 4), +32) of the split and on the query heads of half
// w / 4 of the group (the first (G+1)/2 heads or the rest), so a tile in shared memory is read by two
// warps and the FMAs of a token are shared between them.
template <int kD, int kG>
__global__ void __launch_bounds__(kAttnThreads) attention_decode_split_kernel(const AttentionParams p) {
    constexpr int kPerLane = kD / 32;  // head-dim elements a lane owns in the value phase (2 or 4)
    constexpr int kGPad = 8;
    constexpr int kFirstHalf = (kG + 1) / 2;
    constexpr int kKeyRow = kD + kAttnKeyPad;  // elements; 16 bytes of padding make lane-per-token reads conflict-free
    extern __shared__ __align__(16) uint16_t tiles[];
    uint16_t* key_tile = tiles;                               // [128][kD + 8]
    uint16_t* value_tile = tiles + kAttnSplitTokens * kKeyRow;  // [128][kD]
    __shared__ __align__(16) float q_shared[kG][kD];
    __shared__ __align__(16) float prob[4][32][kGPad];
    __shared__ float warp_max[4][kG], warp_sum[4][kG];
    // The four token groups' outputs reuse the key tile once every warp is done with it.
    float* warp_out = reinterpret_cast<float*>(key_tile);     // [4][kG][kD]
    static_assert(4 * kG * kD * 4 <= kAttnSplitTokens * kKeyRow * 2, "warp outputs fit the key tile");

    const int split = blockIdx.x;
    const int bh = blockIdx.y;                     // b * Hkv + h
    const int b = bh / p.kv_heads, h = bh - b * p.kv_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int group = warp & 3, half = warp >> 2;
    const int g_begin = half == 0 ? 0 : kFirstHalf;
    const int g_end = half == 0 ? kFirstHalf : kG;
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
        cp_async_16(key_tile + row * kKeyRow + chunk * 8, p.k + cache_row0 + (size_t)(split_first + row) * kD + chunk * 8);
    }
    cp_async_commit();
    for (int c = threadIdx.x; c < rows * kChunks; c += kAttnThreads) {
        const int row = c / kChunks, chunk = c - row * kChunks;
        cp_async_16(value_tile + row * kD + chunk * 8, p.v + cache_row0 + (size_t)(split_first + row) * kD + chunk * 8);
    }
    cp_async_commit();

    // Scaled queries of this KV head's group, fp32 (the cast comes before the scale multiplies).
    for (int idx = threadIdx.x; idx < kG * kD; idx += kAttnThreads) {
        const int g = idx / kD, d = idx - g * kD;
        const size_t at = ((size_t)b * p.q_heads + (size_t)h * kG + g) * kD + d;
        q_shared[g][d] = bf16_bits_to_f32(ptx::ld_global_dependent_u16(p.q + at)) * p.scale;
    }
    cp_async_wait<1>();
    __syncthreads();

    const int local = group * 32 + lane;           // this lane's token inside the split
    const bool valid = local < rows;
    const int first = group * 32;
    const int count = min(32, rows - first);       // tokens of this warp in use (<= 0: none)

    // ---------------------------------------------------------------- scores: one token per lane
    float score[kFirstHalf];
#pragma unroll
    for (int j = 0; j < kFirstHalf; ++j) score[j] = 0.0f;
    if (valid) {
        const uint16_t* key = key_tile + local * kKeyRow;
#pragma unroll 4
        for (int d0 = 0; d0 < kD; d0 += 8) {
            const uint4 raw = *reinterpret_cast<const uint4*>(key + d0);
            const float kf[8] = {bf16_lo(raw.x), bf16_hi(raw.x), bf16_lo(raw.y), bf16_hi(raw.y),
                                 bf16_lo(raw.z), bf16_hi(raw.z), bf16_lo(raw.w), bf16_hi(raw.w)};
#pragma unroll
            for (int j = 0; j < kFirstHalf; ++j) {
                const int g = g_begin + j;
                if (g >= g_end) break;
                const float4 qa = *reinterpret_cast<const float4*>(&q_shared[g][d0]);
                const float4 qb = *reinterpret_cast<const float4*>(&q_shared[g][d0 + 4]);
                float s = score[j];
                s = fmaf(qa.x, kf[0], s); s = fmaf(qa.y, kf[1], s); s = fmaf(qa.z, kf[2], s); s = fmaf(qa.w, kf[3], s);
                s = fmaf(qb.x, kf[4], s); s = fmaf(qb.y, kf[5], s); s = fmaf(qb.z, kf[6], s); s = fmaf(qb.w, kf[7], s);
                score[j] = s;
            }
        }
    }
    // ---------------------------------------------------------------- softmax over the warp's tokens
    float block_max[kFirstHalf], block_sum[kFirstHalf];
#pragma unroll
    for (int j = 0; j < kFirstHalf; ++j) {
        const int g = g_begin + j;
        if (g >= g_end) break;
        float m = valid ? score[j] : -INFINITY;
#pragma unroll
        for (int offset = 16; offset >= 1; offset >>= 1) m = fmaxf(m, __shfl_xor_sync(0xFFFFFFFFu, m, offset));
        const float e = valid ? __expf(score[j] - m) : 0.0f;
        prob[group][lane][g] = e;
        block_max[j] = m;
        block_sum[j] = warp_sum_xor(e);
    }
    cp_async_wait<0>();
    __syncthreads();  // values have landed; every warp is done with the key tile and has written its probabilities
    // ---------------------------------------------------------------- values: lanes own head-dim slices
    float acc[kFirstHalf][kPerLane];
#pragma unroll
    for (int j = 0; j < kFirstHalf; ++j)
#pragma unroll
        for (int e = 0; e < kPerLane; ++e) acc[j][e] = 0.0f;
    if (count > 0) {
        const uint16_t* value = value_tile + first * kD + lane * kPerLane;
#pragma unroll 4
        for (int t = 0; t < count; ++t) {
            float vf[kPerLane];
            if constexpr (kPerLane == 4) {
                const uint2 raw = *reinterpret_cast<const uint2*>(value + t * kD);
                vf[0] = bf16_lo(raw.x); vf[1] = bf16_hi(raw.x); vf[2] = bf16_lo(raw.y); vf[3] = bf16_hi(raw.y);
            } else {
                const uint32_t raw = *reinterpret_cast<const uint32_t*>(value + t * kD);
                vf[0] = bf16_lo(raw); vf[1] = bf16_hi(raw);
            }
            const float4 pa = *reinterpret_cast<const float4*>(&prob[group][t][0]);
            const float4 pb = *reinterpret_cast<const float4*>(&prob[group][t][4]);
            const float pg[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
#pragma unroll
            for (int j = 0; j < kFirstHalf; ++j) {
                const int g = half == 0 ? j : kFirstHalf + j;   // a compile-time index in each branch of `half`
                if (g >= g_end) break;
#pragma unroll
                for (int e = 0; e < kPerLane; ++e) acc[j][e] = fmaf(half == 0 ? pg[j] : pg[(kFirstHalf + j) & 7], vf[e], acc[j][e]);
            }
        }
    }
    // ---------------------------------------------------------------- merge the four token groups, in order
#pragma unroll
    for (int j = 0; j < kFirstHalf; ++j) {
        const int g = g_begin + j;
        if (g >= g_end) break;
        if (lane == 0) {
            warp_max[group][g] = block_max[j];
            warp_sum[group][g] = block_sum[j];
        }
#pragma unroll
        for (int e = 0; e < kPerLane; ++e) warp_out[(group * kG + g) * kD + lane * kPerLane + e] = acc[j][e];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < kG * kD; idx += kAttnThreads) {
        const int g = idx / kD, d = idx - g * kD;
        float m = warp_max[0][g];
#pragma unroll
        for (int w = 1; w < 4; ++w) m = fmaxf(m, warp_max[w][g]);
        float total = 0.0f, value = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float factor = warp_max[w][g] == -INFINITY ? 0.0f : __expf(warp_max[w][g] - m);
            total = fmaf(warp_sum[w][g], factor, total);
            value = fmaf(warp_out[(w * kG + g) * kD + d], factor, value);
        }
        if (p.splits == 1) {
            const size_t at = ((size_t)b * p.q_heads + (size_t)h * kG + g) * kD + d;
            p.out[at] = f32_to_bf16_bits(value / total);
        } else {
            float* row = p.partial + (((size_t)bh * p.splits + split) * kG + g) * (kD + 2);
            row[d] = value;
            if (d == 0) {
                row[kD] = m;
                row[kD + 1] = total;
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
