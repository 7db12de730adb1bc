/*
 * C ABI of libmetile_b200.so: the MLX-format affine INT4 projection path for NVIDIA B200
 * (sm_100a).  Plain pointers and sizes only; every pointer is DEVICE memory owned by the
 * caller (the *_host arguments of mt_affine_mlp_host excepted); the library allocates no device
 * memory (mt_peer_group_create excepted: the receive buffer of the tensor-parallel sum), keeps no
 * caller pointer after a call returns, and every call is asynchronous on `stream` (a cudaStream_t
 * passed as void*; NULL = default stream).
 * Every pointer and the stream must belong to the CURRENT device: the library takes its SM count, its
 * per-device caches and its launches from it.  What the library does hold on each device is a few
 * hundred bytes of status words and barrier counters, and the 4 MiB array of mt_affine_mlp_static.
 *
 * Data layout (identical to what the reference project consumes, so packed MLX weights drop
 * in unchanged -- metile/backends/mlx_quantized.py:478-480, kernels/affine_qmv.py:25-51):
 *   x        bf16  [M, K]        row-major activations
 *   w        u32   [N, K/8]      8 nibbles per word, element 8j+e in bits [4e, 4e+4)
 *   scales   bf16  [N, K/64]     one per group of 64 along K
 *   biases   bf16  [N, K/64]     w[n,k] = scales[n,k/64] * q[n,k] + biases[n,k/64]
 *   out      bf16  [M, N]        y = x @ w^T, fp32 accumulation, one rounding at the store
 *
 * Return value: 0 (MT_OK) or a negative code; mt_status_string() names it.  Codes:
 *   -1 shape, -2 alignment, -3 quantisation format, -4 CUDA launch error, -5 wrong device,
 *   -6 null pointer, -7 workspace, -8 a bounded device-side wait gave up.
 * Argument errors (codes -1, -2, -3, -5, -6, -7) are detected before any GPU work is queued; -4 is
 * what the CUDA runtime reported for a launch.  There is no CPU fallback.
 *
 * `flags`: 0 selects the kernel by row count.  A single projection (mt_affine_qmv, mt_affine_swiglu):
 * the CUDA-core GEMV for M = 1, the tcgen05 kernel above.  mt_affine_mlp: one cooperative launch for
 * the whole MLP when the shape allows it -- on CUDA cores for M = 1 (H and I in {1024, 2048, 4096,
 * 8192}), on mma.sync for M = 2 ... 8 (H in {512, 1024, 1536, 2048}, I a multiple of 512) -- else two
 * kernels (gate|up SwiGLU, then down) of the families above.
 *   MT_FLAG_FORCE_GEMV (1)   CUDA-core GEMV (M <= 8)
 *   MT_FLAG_FORCE_UMMA (2)   tcgen05 kernel for any M (one accumulation order for every M: use it
 *                            when rows must be bit-identical across batch sizes 1..128)
 *   MT_FLAG_GELU (16)        mt_dense_act: x/(1+exp(-1.702x)) instead of SiLU
 *   MT_FLAG_MLP_FUSED (32)   mt_affine_mlp: insist on the single-launch CUDA-core kernel (M <= 4); -1
 *                            when it does not apply.  With flags = 0 the default dispatch falls back
 *                            to the two-kernel path if the driver refuses the cooperative launch.
 *   MT_FLAG_HOST_PAIR (64)   mt_affine_mlp_host: see there
 *   MT_FLAG_MLP_FUSED_MMA (128) mt_affine_mlp: insist on the mma.sync single-launch kernel (M <= 8);
 *                            -1 when it does not apply.
 */
#ifndef METILE_B200_H
#define METILE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MT_FLAG_FORCE_GEMV 0x1u
#define MT_FLAG_FORCE_UMMA 0x2u
#define MT_FLAG_GELU 0x10u
#define MT_FLAG_MLP_FUSED 0x20u
#define MT_FLAG_HOST_PAIR 0x40u
#define MT_FLAG_MLP_FUSED_MMA 0x80u

/* Library version (major*10000 + minor*100 + patch). */
int mt_version(void);

/* Human-readable name of a status code. */
const char* mt_status_string(int status);

/* 0 when the current CUDA device is compute capability 10.x, else MT_ERR_DEVICE. */
int mt_device_check(void);

/* Reads (and with reset != 0 clears) the device-side record of a bounded wait that gave up:
 * words[0] = wait code (0 = none), [1] = block, [2] = thread, [3] = parity.  Synchronises the
 * device.  Returns 0, or -8 when words[0] != 0. */
int mt_device_status(unsigned int words[4], int reset);

/* Self-test of the bounded device-side waits: queues a tiny kernel whose wait can never be satisfied
 * (which = 0: an mbarrier nobody arrives at; which = 1: the single-launch MLP's grid barrier with an
 * unreachable target) and gives up after limit_us microseconds (1 ... 100000).  Nothing faults or
 * hangs: the kernel records the wait code and returns, the next mt_device_status() reports -8 and,
 * with reset != 0, clears the record and the grid-barrier counters.  Production kernels run the same
 * wait code with a 2 s limit.  No counterpart in the reference project. */
int mt_selftest_bounded_wait(int which, unsigned int limit_us, void* stream);

/* y = x @ dequant(w)^T (+ residual, added to the un-rounded sum).
 * Replaces: metile/backends/mlx_quantized.py:691 (mlx_affine_qmv), :1538
 * (mlx_affine_residual_qmv), kernels/affine_qmv.py:57,94 and, for M > 1,
 * metile/backends/mlx_affine.py:359 (mlx_affine_matmul).  residual may be NULL. */
int mt_affine_qmv(const void* x, const uint32_t* w, const void* scales, const void* biases,
                  const void* residual, void* out, int M, int K, int N, int group_size, int bits,
                  unsigned int flags, void* stream);

/* out = silu(x @ Wg^T) * (x @ Wu^T) on un-rounded fp32 sums.
 * Replaces: metile/backends/mlx_quantized.py:717 (mlx_affine_swiglu_qmv), :1645
 * (mlx_affine_swiglu), kernels/affine_qmv.py:135,217. */
int mt_affine_swiglu(const void* x, const uint32_t* gate_w, const void* gate_scales,
                     const void* gate_biases, const uint32_t* up_w, const void* up_scales,
                     const void* up_biases, void* out, int M, int K, int N, int group_size, int bits,
                     unsigned int flags, void* stream);

/* Bytes of device workspace mt_affine_mlp needs (the bf16 hidden activations [M, I]). */
size_t mt_affine_mlp_workspace_bytes(int M, int H, int I);

/* out[M,H] = down(swiglu(x)) + residual: gate/up [I, H/8], down [H, I/8].  `workspace` is
 * caller-owned device memory of at least mt_affine_mlp_workspace_bytes() bytes, 16-byte
 * aligned; its contents after the call are the bf16 hidden activations.
 * Replaces: metile/backends/mlx_quantized.py:1770 (mlx_affine_mlp_executor) and the call in
 * metile/integrations/mlx_lm.py:3837 (_execute_quantized_mlp).  residual may be NULL. */
int mt_affine_mlp(const void* x, const uint32_t* gate_w, const void* gate_scales,
                  const void* gate_biases, const uint32_t* up_w, const void* up_scales,
                  const void* up_biases, const uint32_t* down_w, const void* down_scales,
                  const void* down_biases, const void* residual, void* workspace,
                  size_t workspace_bytes, void* out, int M, int H, int I, int group_size, int bits,
                  unsigned int flags, void* stream);

/* mt_affine_mlp for activations that live in HOST memory: queues, in order on `stream`, the copy of
 * x (and of residual, unless residual_host is NULL) from the host buffers into the caller's device
 * staging buffers, mt_affine_mlp on those, and the copy of the result into out_host.  The host
 * buffers should be page-locked (cudaHostAlloc / cudaHostRegister) so the copies are asynchronous;
 * out_host is valid once the stream has been synchronised.  Page-locked, mapped buffers of up to
 * 512 KB per copy are read and written by small kernels chained to the MLP kernels (a copy engine's
 * turn between two kernels costs more than such a copy); pageable memory and larger copies go
 * through cudaMemcpyAsync -- the library asks the runtime what kind of memory each host pointer is.  Staging buffers hold M*H bf16 each and
 * `workspace` is as for mt_affine_mlp; nothing is allocated here.  With MT_FLAG_HOST_PAIR the caller
 * states that residual_host directly follows x_host inside ONE host allocation; if residual_device
 * also directly follows x_device, one copy moves both (small copies cost their latency, not their
 * bytes).  The flag has no other effect.
 * Replaces, for a host whose activations are not on the GPU, the same call sites as mt_affine_mlp;
 * the reference has no such split because Apple GPUs share memory with the host. */
int mt_affine_mlp_host(const void* x_host, const void* residual_host, void* out_host, void* x_device,
                       void* residual_device, void* out_device, const uint32_t* gate_w,
                       const void* gate_scales, const void* gate_biases, const uint32_t* up_w,
                       const void* up_scales, const void* up_biases, const uint32_t* down_w,
                       const void* down_scales, const void* down_biases, void* workspace,
                       size_t workspace_bytes, int M, int H, int I, int group_size, int bits,
                       unsigned int flags, void* stream);

/* How many kernels mt_affine_mlp queues for this problem on the current device with 16-byte
 * aligned operands: 1 when a single-launch kernel serves it (one row on CUDA cores, up to four with
 * MT_FLAG_MLP_FUSED, H and I in {1024, 2048, 4096, 8192}; two to eight rows on mma.sync, H <= 2048),
 * else 2 (gate|up
 * SwiGLU, then down); 0 for M <= 0.  No counterpart in the reference project; used for launch
 * accounting. */
int mt_affine_mlp_launches(int M, int H, int I, unsigned int flags);

/* The fused MLP of mt_affine_mlp for callers that may not allocate device memory.
 * No counterpart in the reference project.
 * Some hosts of this library cannot call cudaMalloc on the path that runs the MLP: a serving loop
 * that forbids allocation after start-up because cudaMalloc synchronises the whole device, or a
 * plugin that was handed a fixed arena and nothing else.  For them the bf16 hidden activations [M, I] live
 * in an array compiled into the library (mt_affine_mlp_static_max_bytes() bytes, 4 MiB, held by
 * every GPU that loads the library until the process exits) instead of a caller workspace.  Inputs
 * and the output are still the caller's.  The call makes no cudaMalloc / cudaFree and uses no
 * allocating library routine.
 *   - Limit: M * I * 2 bytes must not exceed mt_affine_mlp_static_max_bytes(); larger problems are
 *     refused with -7 before anything is queued.  Use mt_affine_mlp with your own workspace then.
 *   - The first call on a device looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current) and keeps it.
 *   - All calls share the one array and it keeps the last call's contents.  Nothing needs clearing:
 *     each call overwrites every element it later reads.  Two calls that overlap on the GPU (two
 *     streams, two host threads) race on the array; serialise them.
 * Results are bit-identical to mt_affine_mlp with the same arguments. */
size_t mt_affine_mlp_static_max_bytes(void);
int mt_affine_mlp_static(const void* x, const uint32_t* gate_w, const void* gate_scales,
                         const void* gate_biases, const uint32_t* up_w, const void* up_scales,
                         const void* up_biases, const uint32_t* down_w, const void* down_scales,
                         const void* down_biases, const void* residual, void* out, int M, int H, int I,
                         int group_size, int bits, unsigned int flags, void* stream);

/* sum_out = bf16(x + residual); norm_out = bf16(sum_out * rsqrt(mean((x+residual)^2) + eps) * w).
 * Replaces: metile/backends/mlx.py:786 (mlx_add_rms_norm), kernels/add_rmsnorm.py:5.
 * sum_out may be NULL. */
int mt_add_rmsnorm(const void* x, const void* residual, const void* weight, void* sum_out,
                   void* norm_out, int rows, int H, float eps, void* stream);

/* out = bf16(x * rsqrt(mean(x^2) + eps) * w).
 * Replaces: metile/backends/mlx.py:748 (mlx_rms_norm), kernels/rmsnorm.py:5. */
int mt_rmsnorm(const void* x, const void* weight, void* out, int rows, int H, float eps,
               void* stream);

/* Decode attention: one query row per sequence and head over a KV cache,
 *   out[b, h, :] = softmax(scale * q[b, h, :] . K[b, h / (Hq/Hkv), 0:n, :]) @ V[b, h / (Hq/Hkv), 0:n, :],
 * fp32 accumulation, one rounding at the store.  q, out: bf16 [batch, q_heads, head_dim]; k_cache,
 * v_cache: bf16 [batch, kv_heads, capacity, head_dim] (the [B, H, N, D] layout of the reference's
 * decode kernel with room for `capacity` tokens per head); n = lengths[b] when `lengths` (int32
 * [batch], device) is given, else `tokens`, which must also bound every lengths[b].  head_dim 64 or
 * 128, q_heads a multiple of kv_heads, at most 8 query heads per KV head.  `workspace`: device scratch
 * of mt_attention_decode_workspace_bytes() bytes (0 when tokens <= 128), 16-byte aligned.
 * Replaces: kernels/attention.py:27 (attention_decode_kernel), metile/backends/mlx.py:718
 * (mlx_attention_decode), behind the admission rule of metile/integrations/mlx_lm.py:3558. */
size_t mt_attention_decode_workspace_bytes(int batch, int q_heads, int tokens, int head_dim);
int mt_attention_decode(const void* q, const void* k_cache, const void* v_cache, const int* lengths,
                        void* out, void* workspace, size_t workspace_bytes, int batch, int q_heads,
                        int kv_heads, int tokens, int capacity, int head_dim, float scale, void* stream);

/* Rotary embedding of the new query and key rows (half-split pairs (i, i + D/2), angle =
 * positions[b] * theta^(-2i/D)) and the in-place append of the rotated key and of the value at
 * row positions[b] of each sequence's cache.  q: bf16 [batch, q_heads, head_dim], k, v: bf16 [batch,
 * kv_heads, head_dim], consecutive sequences `row_stride` elements apart in all three (q_heads *
 * head_dim etc. for dense arrays; the width of a fused q|k|v projection row when q, k and v point
 * into one); q_out: dense bf16 [batch, q_heads, head_dim]; caches as for mt_attention_decode;
 * positions: int32 [batch] on the device, each < capacity.  The reference leaves both steps to MLX-LM (nn.RoPE,
 * KVCache.update_and_fetch); they are here so that a decode step needs no framework op between the
 * projections and the attention kernel. */
int mt_rope_kv_append(const void* q, const void* k, const void* v, long long row_stride,
                      const int* positions, void* q_out, void* k_cache, void* v_cache, int batch,
                      int q_heads, int kv_heads, int capacity, int head_dim, float theta, void* stream);

/* Sum of bf16 partial results over the GPUs of one node (one process per GPU), for the
 * tensor-parallel form of the fused MLP: the down projection of a K-sharded MLP leaves a partial
 * [M, H] result on every rank.  NO COUNTERPART IN THE REFERENCE, which is single-device.
 *
 * One kernel per rank stores the partial into every peer's receive buffer over NVLink (very large
 * messages among many ranks: only the segment each peer reduces, then the reduced segment to
 * everyone), signals, waits
 * (bounded by limit_ms, 1..2000; on expiry nothing is written to `out` and mt_device_status reports
 * code 0x9E0 with the peer that did not arrive) and adds the partials in rank order in fp32, so every
 * rank obtains the same bits whatever the message size.
 *
 * mt_peer_group_create allocates this rank's receive buffer (the only allocation; `slot_bytes` =
 * largest message in bytes, a multiple of 16, at most 64 MiB) and writes its 64-byte CUDA IPC handle to
 * ipc_handle_out.  The caller exchanges the handles between the processes by any host means and passes
 * all `world` of them, in rank order, to mt_peer_group_connect.  Every rank must call
 * mt_peer_all_reduce the same number of times with the same `elements` (bf16 elements, a multiple
 * of 8); `partial` and `out` may be the same buffer.  The call number lives on the device (the
 * kernel advances it), so a CUDA graph that contains the call can be replayed, every rank the same
 * number of times.  Two calls on one group must never overlap on a GPU: issue them on one stream,
 * or order the streams.  Ranks that fall out of step (one launches more calls than another) wait
 * out the limit on every later call, or read a slot before it is rewritten: count the launches.
 * Before mt_peer_group_destroy the caller makes sure (a host barrier) that no peer has a call in
 * flight. */
int mt_peer_group_create(int rank, int world, size_t slot_bytes, void** group_out,
                         void* ipc_handle_out);
int mt_peer_group_connect(void* group, const void* ipc_handles);
/* mode 0 (default): one shot, or two shots (reduce-scatter then all-gather, both by peer stores) where
 * one shot would store more than 4 MB per rank among six or more ranks; 1: always one shot; 2: always
 * two shots.  Every rank must choose the same. */
int mt_peer_group_set_mode(void* group, int mode);
int mt_peer_all_reduce(void* group, const void* partial, void* out, size_t elements,
                       unsigned int limit_ms, void* stream);
int mt_peer_group_destroy(void* group);

/* Dense bf16 small-batch projection, w [N, K] bf16: out = bf16(bf16(x @ w^T) + residual).
 * Every row is bit-identical to running it alone.  K % 128 == 0.  residual may be NULL.
 * Replaces: metile/compiler/dense.py:302 (lower_dense_residual_qmv) and its backend entry
 * metile/backends/mlx_dense_residual.py. */
int mt_dense_rows(const void* x, const void* w, const void* residual, void* out, int M, int K,
                  int N, void* stream);

/* Dense bf16 small-batch SwiGLU with the typed epilogue of the reference's exact path.
 * Replaces: metile/compiler/dense.py:193 (lower_dense_swiglu_qmv),
 * metile/backends/mlx_dense_swiglu.py. */
int mt_dense_swiglu(const void* x, const void* gate_w, const void* up_w, void* out, int M, int K,
                    int N, void* stream);

/* C[M,N] = act(A[M,K] @ B[K,N]), bf16, fp32 accumulate, M <= 128; act = SiLU, or the
 * x/(1+exp(-1.702x)) GELU form with MT_FLAG_GELU.
 * Replaces: kernels/mlp.py:34 (matmul_silu) and :7 (matmul_gelu). */
int mt_dense_act(const void* a, const void* b, void* c, int M, int N, int K, unsigned int flags,
                 void* stream);

#ifdef __cplusplus
}
#endif
#endif /* METILE_B200_H */
