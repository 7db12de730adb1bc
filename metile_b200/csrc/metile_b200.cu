// extern "C" entry points of libmetile_b200.so (declared in include/metile_b200.h).
// One translation unit: the kernels live in the .cuh files included below.
#include "../../include/metile_b200.h"

#include "add_rmsnorm.cuh"
#include "attention_decode.cuh"
#include "peer_reduce.cuh"
#include "affine_gemv.cuh"
#include "affine_umma.cuh"
#include "affine_mlp_fused.cuh"
#include <string.h>

#include "common.cuh"
#include "dense_rows.cuh"

namespace mt {

static int device_sm_count() {
    static int cached[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 0;
    if (device < 64 && cached[device]) return cached[device];
    int count = 0;
    if (cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device) != cudaSuccess) return 0;
    if (device < 64) cached[device] = count;
    return count;
}

static int device_is_sm100() {
    static int cached[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 0;
    if (device < 64 && cached[device]) return cached[device] > 0;
    int major = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device) != cudaSuccess) return 0;
    if (device < 64) cached[device] = major == 10 ? 1 : -1;
    return major == 10;
}

static int check_format(int K, int N, int group_size, int bits) {
    if (group_size != 64 || bits != 4) return MT_ERR_FORMAT;
    if (K < 64 || K % 64 || N < 1) return MT_ERR_SHAPE;
    return MT_OK;
}

static int check_affine_ptrs(const void* x, const uint32_t* w, const void* s, const void* b, const void* out) {
    if (!x || !w || !s || !b || !out) return MT_ERR_NULL;
    if (!aligned_to(x, 16) || !aligned_to(w, 16) || !aligned_to(s, 2) || !aligned_to(b, 2) || !aligned_to(out, 2))
        return MT_ERR_ALIGN;
    return MT_OK;
}

// Row-count split: the CUDA-core GEMV issues one FMA per weight per row on top of the unpack, so
// it is instruction-bound already at one row; measured, it wins at one row only (fused MLP at the
// Llama-3.2-1B shape: 18.7 us vs 24.6 us) and loses from two rows on (26.1 us vs 24.7 us).
static bool use_gemv(int M, unsigned int flags) {
    if (flags & MT_FLAG_FORCE_GEMV) return true;
    if (flags & MT_FLAG_FORCE_UMMA) return false;
    return M <= 1;
}

static int run_projection(const void* x, const AffineWeights& first, const AffineWeights* second, const void* residual,
                          void* out, int M, int K, int N, unsigned int flags, cudaStream_t stream) {
    const int sms = device_sm_count();
    if (sms <= 0) return MT_ERR_DEVICE;
    if (M == 0) return MT_OK;
    if (use_gemv(M, flags)) {
        if (M > 8) return MT_ERR_SHAPE;
        GemvWeights a{first.w, first.scales, first.biases};
        GemvWeights b = second ? GemvWeights{second->w, second->scales, second->biases} : a;
        return second ? launch_gemv<true>(x, a, b, residual, out, M, K, N, sms, stream)
                      : launch_gemv<false>(x, a, b, residual, out, M, K, N, sms, stream);
    }
    const uint16_t* xp = static_cast<const uint16_t*>(x);
    const uint16_t* rp = static_cast<const uint16_t*>(residual);
    uint16_t* op = static_cast<uint16_t*>(out);
    for (int m0 = 0; m0 < M; m0 += 128) {
        const int rows = M - m0 < 128 ? M - m0 : 128;
        const int rc = launch_umma(xp + (size_t)m0 * K, &first, second, rp ? rp + (size_t)m0 * N : nullptr,
                                   op + (size_t)m0 * N, rows, K, N, stream);
        if (rc != MT_OK) return rc;
    }
    return MT_OK;
}

// C[M,N] = act(A[M,K] @ B[K,N]); a thread owns two adjacent output columns of kRows rows.
template <int kRows>
__global__ void __launch_bounds__(128)
dense_act_kernel(const uint16_t* __restrict__ a, const uint16_t* __restrict__ b, uint16_t* __restrict__ c, int M,
                 int N, int K, int gelu) {
    const int col = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
    const int m0 = blockIdx.y * kRows;
    if (col >= N) return;
    float acc[kRows][2];
#pragma unroll
    for (int r = 0; r < kRows; ++r) acc[r][0] = acc[r][1] = 0.0f;
    const bool pair = col + 1 < N && (N % 2 == 0);
    for (int k = 0; k < K; ++k) {
        float b0, b1 = 0.0f;
        if (pair) {
            const uint32_t bv = __ldg(reinterpret_cast<const uint32_t*>(b + (size_t)k * N + col));
            b0 = bf16_lo(bv);
            b1 = bf16_hi(bv);
        } else {
            b0 = bf16_bits_to_f32(b[(size_t)k * N + col]);
            if (col + 1 < N) b1 = bf16_bits_to_f32(b[(size_t)k * N + col + 1]);
        }
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
            const int m = m0 + r < M ? m0 + r : M - 1;
            const float av = bf16_bits_to_f32(__ldg(a + (size_t)m * K + k));
            acc[r][0] = fmaf(av, b0, acc[r][0]);
            acc[r][1] = fmaf(av, b1, acc[r][1]);
        }
    }
    const float slope = gelu ? 1.702f : 1.0f;
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
        if (m0 + r >= M) break;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            if (col + j >= N) break;
            const float v = acc[r][j];
            c[(size_t)(m0 + r) * N + col + j] = f32_to_bf16_bits(v / (1.0f + __expf(-slope * v)));
        }
    }
}

// Scratch for mt_affine_mlp_static: the bf16 hidden activations [M, I] of one fused MLP call.
// It lives in the library's device image, so every GPU that loads the library holds these bytes
// until the process exits.  In host code this name is only a handle for cudaGetSymbolAddress; the
// device address is looked up once per device (static_hidden_address below).
constexpr size_t kStaticHiddenBytes = 4u << 20;
static __device__ __align__(256) unsigned char g_static_hidden[kStaticHiddenBytes];

// Device address of g_static_hidden on the current device, resolved on first use per device.
static int static_hidden_address(void** out) {
    static void* cached[64] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return MT_ERR_DEVICE;
    if (device >= 0 && device < 64 && cached[device]) {
        *out = cached[device];
        return MT_OK;
    }
    void* address = nullptr;
    if (cudaGetSymbolAddress(&address, g_static_hidden) != cudaSuccess || address == nullptr) return MT_ERR_LAUNCH;
    if (device >= 0 && device < 64) cached[device] = address;
    *out = address;
    return MT_OK;
}

// ---- staging between page-locked host memory and the device with a kernel instead of a copy engine ----
// A copy engine's turn between two kernels of a stream costs several microseconds of hand-over on
// each side; a small kernel that reads (writes) the mapped host buffer itself is chained to its
// neighbours by programmatic dependent launch like any other kernel.  Used for up to kStageKernelBytes
// per copy; larger copies keep the copy engine, whose bandwidth then matters more than its latency.
constexpr size_t kStageKernelBytes = 512u << 10;

__global__ void __launch_bounds__(256) stage_copy_kernel(const uint4* src, uint4* dst, unsigned int vectors) {
    ptx::griddep_launch_dependents();
    ptx::griddep_wait();  // the destination may still be read, the source still be written, by the kernel before
    const unsigned int base = blockIdx.x * 1024u + threadIdx.x;
    uint4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const unsigned int i = base + 256u * j;
        if (i < vectors)
            asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(v[j].x), "=r"(v[j].y), "=r"(v[j].z), "=r"(v[j].w)
                         : "l"(src + i));
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const unsigned int i = base + 256u * j;
        if (i < vectors) dst[i] = v[j];
    }
}

// The device's address of a page-locked, mapped host buffer, or null when `host` is anything else
// (pageable memory must never be handed to a kernel).
static void* device_view_of_host(const void* host) {
    cudaPointerAttributes attributes;
    if (cudaPointerGetAttributes(&attributes, host) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    if (attributes.type != cudaMemoryTypeHost) return nullptr;
    return attributes.devicePointer;
}

// Copies `bytes` (a multiple of 16, both ends 16-byte aligned) with the kernel; false = not queued.
static bool stage_with_kernel(const void* src, void* dst, size_t bytes, cudaStream_t stream) {
    if (bytes == 0 || bytes % 16 || bytes > kStageKernelBytes || !aligned_to(src, 16) || !aligned_to(dst, 16)) return false;
    const unsigned int vectors = (unsigned int)(bytes / 16);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3((vectors + 1023) / 1024);
    config.blockDim = dim3(256);
    config.stream = stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, stage_copy_kernel, static_cast<const uint4*>(src), static_cast<uint4*>(dst),
                              vectors) == cudaSuccess;
}

// ---- self-test kernels: make a bounded device-side wait run out, on purpose and harmlessly ----------
constexpr unsigned int kWaitSelfTest = 0x7E1;

// One CTA waits on an mbarrier nobody arrives at; the wait gives up after `limit_ns` and returns.
__global__ void selftest_mbarrier_wait_kernel(unsigned long long limit_ns) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar, 1);
        abort_flag = 0;
        ptx::mbar_fence_init();
    }
    __syncthreads();
    ptx::mbar_wait(&bar, 0, &abort_flag, kWaitSelfTest, limit_ns);
}

// Two CTAs meet at the single-launch MLP's grid barrier with a target no arrival count can reach.
__global__ void __launch_bounds__(kFusedComputeThreads)
selftest_grid_barrier_kernel(unsigned long long* slot, unsigned long long limit_ns) {
    __shared__ int abort_flag;
    if (threadIdx.x == 0) abort_flag = 0;
    __syncthreads();
    fused_grid_barrier(slot, (int)gridDim.x + 1, &abort_flag, limit_ns);
}

}  // namespace mt

using namespace mt;

extern "C" {

int mt_version(void) { return 100; }

const char* mt_status_string(int status) {
    switch (status) {
        case MT_OK: return "ok";
        case MT_ERR_SHAPE: return "unsupported shape";
        case MT_ERR_ALIGN: return "misaligned pointer";
        case MT_ERR_FORMAT: return "unsupported quantisation format (need 4 bits, group size 64)";
        case MT_ERR_LAUNCH: return "CUDA launch error";
        case MT_ERR_DEVICE: return "current device is not compute capability 10.x";
        case MT_ERR_NULL: return "null pointer";
        case MT_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
        case MT_ERR_DEVICE_WAIT: return "a bounded device-side wait gave up";
        default: return "unknown status";
    }
}

int mt_device_check(void) { return device_is_sm100() ? MT_OK : MT_ERR_DEVICE; }

int mt_device_status(unsigned int words[4], int reset) {
    if (!words) return MT_ERR_NULL;
    if (cudaDeviceSynchronize() != cudaSuccess) return MT_ERR_LAUNCH;
    if (cudaMemcpyFromSymbol(words, g_device_status, sizeof(unsigned int) * 4) != cudaSuccess) return MT_ERR_LAUNCH;
    if (reset) {
        const unsigned int zeros[4] = {0, 0, 0, 0};
        if (cudaMemcpyToSymbol(g_device_status, zeros, sizeof(zeros)) != cudaSuccess) return MT_ERR_LAUNCH;
        // A wait that gave up at the single-launch MLP's grid barrier leaves its counter short of a
        // multiple of the grid size; the device is idle here, so every counter can start over.
        static const unsigned long long no_arrivals[kFusedBarrierSlots] = {};
        if (words[0] && cudaMemcpyToSymbol(g_fused_barrier, no_arrivals, sizeof(no_arrivals)) != cudaSuccess)
            return MT_ERR_LAUNCH;
    }
    return words[0] ? MT_ERR_DEVICE_WAIT : MT_OK;
}

int mt_selftest_bounded_wait(int which, unsigned int limit_us, void* stream) {
    if (!device_is_sm100()) return MT_ERR_DEVICE;
    if (limit_us < 1 || limit_us > 100000) return MT_ERR_SHAPE;  // 1 us ... 100 ms
    const unsigned long long limit_ns = 1000ull * limit_us;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (which == 0) {
        selftest_mbarrier_wait_kernel<<<1, 64, 0, s>>>(limit_ns);
    } else if (which == 1) {
        unsigned long long* slot = next_fused_barrier_slot();
        if (!slot) return MT_ERR_LAUNCH;
        selftest_grid_barrier_kernel<<<2, kFusedComputeThreads, 0, s>>>(slot, limit_ns);
    } else {
        return MT_ERR_SHAPE;
    }
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_LAUNCH;
}

int mt_affine_qmv(const void* x, const uint32_t* w, const void* scales, const void* biases, const void* residual,
                  void* out, int M, int K, int N, int group_size, int bits, unsigned int flags, void* stream) {
    int rc = check_format(K, N, group_size, bits);
    if (rc != MT_OK) return rc;
    if (M < 0) return MT_ERR_SHAPE;
    if (M == 0) return MT_OK;
    rc = check_affine_ptrs(x, w, scales, biases, out);
    if (rc != MT_OK) return rc;
    if (!device_is_sm100()) return MT_ERR_DEVICE;
    AffineWeights first{w, static_cast<const uint16_t*>(scales), static_cast<const uint16_t*>(biases)};
    return run_projection(x, first, nullptr, residual, out, M, K, N, flags, static_cast<cudaStream_t>(stream));
}

int mt_affine_swiglu(const void* x, const uint32_t* gate_w, const void* gate_scales, const void* gate_biases,
                     const uint32_t* up_w, const void* up_scales, const void* up_biases, void* out, int M, int K,
                     int N, int group_size, int bits, unsigned int flags, void* stream) {
    int rc = check_format(K, N, group_size, bits);
    if (rc != MT_OK) return rc;
    if (M < 0) return MT_ERR_SHAPE;
    if (M == 0) return MT_OK;
    rc = check_affine_ptrs(x, gate_w, gate_scales, gate_biases, out);
    if (rc != MT_OK) return rc;
    rc = check_affine_ptrs(x, up_w, up_scales, up_biases, out);
    if (rc != MT_OK) return rc;
    if (!device_is_sm100()) return MT_ERR_DEVICE;
    AffineWeights gate{gate_w, static_cast<const uint16_t*>(gate_scales), static_cast<const uint16_t*>(gate_biases)};
    AffineWeights up{up_w, static_cast<const uint16_t*>(up_scales), static_cast<const uint16_t*>(up_biases)};
    return run_projection(x, gate, &up, nullptr, out, M, K, N, flags, static_cast<cudaStream_t>(stream));
}

size_t mt_affine_mlp_workspace_bytes(int M, int H, int I) {
    (void)H;
    if (M <= 0 || I <= 0) return 0;
    return (size_t)M * (size_t)I * 2;
}

int mt_affine_mlp(const void* x, const uint32_t* gate_w, const void* gate_scales, const void* gate_biases,
                  const uint32_t* up_w, const void* up_scales, const void* up_biases, const uint32_t* down_w,
                  const void* down_scales, const void* down_biases, const void* residual, void* workspace,
                  size_t workspace_bytes, void* out, int M, int H, int I, int group_size, int bits,
                  unsigned int flags, void* stream) {
    int rc = check_format(H, I, group_size, bits);
    if (rc != MT_OK) return rc;
    rc = check_format(I, H, group_size, bits);
    if (rc != MT_OK) return rc;
    if (M < 0) return MT_ERR_SHAPE;
    if (M == 0) return MT_OK;
    if (!workspace || !aligned_to(workspace, 16) || workspace_bytes < mt_affine_mlp_workspace_bytes(M, H, I))
        return MT_ERR_WORKSPACE;
    // Every operand of all three projections is checked before the first kernel is queued: a bad
    // down operand must not leave the gate|up kernel running and the workspace half written.
    rc = check_affine_ptrs(x, gate_w, gate_scales, gate_biases, out);
    if (rc == MT_OK) rc = check_affine_ptrs(x, up_w, up_scales, up_biases, out);
    if (rc == MT_OK) rc = check_affine_ptrs(workspace, down_w, down_scales, down_biases, out);
    if (rc != MT_OK) return rc;
    if ((flags & MT_FLAG_FORCE_GEMV) && M > 8) return MT_ERR_SHAPE;
    if (!device_is_sm100()) return MT_ERR_DEVICE;
    // A handful of rows: the whole MLP as one cooperative launch when the shape fits it.  Any flag
    // that pins a kernel family keeps the two-kernel path; MT_FLAG_MLP_FUSED insists on this one.
    if (flags == 0 || (flags & (MT_FLAG_MLP_FUSED | MT_FLAG_MLP_FUSED_MMA))) {
        if (!x || !gate_w || !gate_scales || !gate_biases || !up_w || !up_scales || !up_biases || !down_w ||
            !down_scales || !down_biases || !out)
            return MT_ERR_NULL;
        if (!device_is_sm100()) return MT_ERR_DEVICE;
        FusedMlpParams params;
        params.x = static_cast<const uint16_t*>(x);
        params.gate_w = gate_w;
        params.up_w = up_w;
        params.down_w = down_w;
        params.gate_s = static_cast<const uint16_t*>(gate_scales);
        params.gate_b = static_cast<const uint16_t*>(gate_biases);
        params.up_s = static_cast<const uint16_t*>(up_scales);
        params.up_b = static_cast<const uint16_t*>(up_biases);
        params.down_s = static_cast<const uint16_t*>(down_scales);
        params.down_b = static_cast<const uint16_t*>(down_biases);
        params.residual = static_cast<const uint16_t*>(residual);
        params.hidden = static_cast<uint16_t*>(workspace);
        params.out = static_cast<uint16_t*>(out);
        params.barrier = nullptr;
        params.M = M;
        params.H = H;
        params.I = I;
        const int sms = device_sm_count();
        // Up to kFusedDefaultRows rows: the FMA kernel.  Above, to eight rows: the warp-MMA kernel.
        const bool want_mma = (flags & MT_FLAG_MLP_FUSED_MMA) != 0;
        const bool fma = !want_mma && (flags || M <= kFusedDefaultRows) && fused_mlp_applicable(params, sms);
        const bool mma = !fma && (want_mma || (!flags && M > kFusedDefaultRows)) && fused_mlp_mma_applicable(params, sms);
        if (fma || mma) {
            const int fused_rc = launch_mlp_fused(params, sms, mma, static_cast<cudaStream_t>(stream));
            // A cooperative launch is refused when the whole grid cannot be resident (a GPU shared with
            // another context, a carve-out that leaves too little shared memory).  Nothing was queued:
            // the default dispatch then takes the two-kernel path; an explicit request reports it.
            if (fused_rc != MT_ERR_LAUNCH || flags) return fused_rc;
            cudaGetLastError();
        }
        if (flags) return MT_ERR_SHAPE;
    }
    rc = mt_affine_swiglu(x, gate_w, gate_scales, gate_biases, up_w, up_scales, up_biases, workspace, M, H, I,
                          group_size, bits, flags, stream);
    if (rc != MT_OK) return rc;
    return mt_affine_qmv(workspace, down_w, down_scales, down_biases, residual, out, M, I, H, group_size, bits, flags,
                         stream);
}

int mt_affine_mlp_host(const void* x_host, const void* residual_host, void* out_host, void* x_device,
                       void* residual_device, void* out_device, const uint32_t* gate_w, const void* gate_scales,
                       const void* gate_biases, const uint32_t* up_w, const void* up_scales, const void* up_biases,
                       const uint32_t* down_w, const void* down_scales, const void* down_biases, void* workspace,
                       size_t workspace_bytes, int M, int H, int I, int group_size, int bits, unsigned int flags,
                       void* stream) {
    if (M < 0 || H < 1) return MT_ERR_SHAPE;
    if (M == 0) return MT_OK;
    if (!x_host || !out_host || !x_device || !out_device || (residual_host && !residual_device)) return MT_ERR_NULL;
    // The MLP's own checks, made here before the first copy is queued.
    int rc_early = check_format(H, I, group_size, bits);
    if (rc_early == MT_OK) rc_early = check_format(I, H, group_size, bits);
    if (rc_early != MT_OK) return rc_early;
    if (!workspace || !aligned_to(workspace, 16) || workspace_bytes < mt_affine_mlp_workspace_bytes(M, H, I))
        return MT_ERR_WORKSPACE;
    rc_early = check_affine_ptrs(x_device, gate_w, gate_scales, gate_biases, out_device);
    if (rc_early == MT_OK) rc_early = check_affine_ptrs(x_device, up_w, up_scales, up_biases, out_device);
    if (rc_early == MT_OK) rc_early = check_affine_ptrs(workspace, down_w, down_scales, down_biases, out_device);
    if (rc_early != MT_OK) return rc_early;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t bytes = (size_t)M * (size_t)H * 2;
    // Small copies cost their fixed latency, not their bytes: when the residual follows the activations
    // directly in host memory and the two staging buffers are adjacent as well, one copy moves both.
    // The caller vouches with MT_FLAG_HOST_PAIR that both lie in ONE host allocation (a copy may not span two).
    const bool adjacent = residual_host && (flags & MT_FLAG_HOST_PAIR) &&
                          static_cast<const char*>(residual_host) == static_cast<const char*>(x_host) + bytes &&
                          static_cast<char*>(residual_device) == static_cast<char*>(x_device) + bytes;
    // Page-locked, mapped host buffers are read and written by small kernels (see stage_copy_kernel);
    // anything else, and large copies, go through the copy engine.
    const size_t in_bytes = adjacent ? 2 * bytes : bytes;
    const void* x_view = in_bytes <= kStageKernelBytes ? device_view_of_host(x_host) : nullptr;
    if (!(x_view && stage_with_kernel(x_view, x_device, in_bytes, s)) &&
        cudaMemcpyAsync(x_device, x_host, in_bytes, cudaMemcpyHostToDevice, s) != cudaSuccess)
        return MT_ERR_LAUNCH;
    if (residual_host && !adjacent) {
        const void* r_view = bytes <= kStageKernelBytes ? device_view_of_host(residual_host) : nullptr;
        if (!(r_view && stage_with_kernel(r_view, residual_device, bytes, s)) &&
            cudaMemcpyAsync(residual_device, residual_host, bytes, cudaMemcpyHostToDevice, s) != cudaSuccess)
            return MT_ERR_LAUNCH;
    }
    const int rc = mt_affine_mlp(x_device, gate_w, gate_scales, gate_biases, up_w, up_scales, up_biases, down_w,
                                 down_scales, down_biases, residual_host ? residual_device : nullptr, workspace,
                                 workspace_bytes, out_device, M, H, I, group_size, bits, flags & ~MT_FLAG_HOST_PAIR,
                                 stream);
    if (rc != MT_OK) return rc;
    void* out_view = bytes <= kStageKernelBytes ? device_view_of_host(out_host) : nullptr;
    if (out_view && stage_with_kernel(out_device, out_view, bytes, s)) return MT_OK;
    return cudaMemcpyAsync(out_host, out_device, bytes, cudaMemcpyDeviceToHost, s) == cudaSuccess ? MT_OK : MT_ERR_LAUNCH;
}

int mt_affine_mlp_launches(int M, int H, int I, unsigned int flags) {
    if (M <= 0) return 0;
    if (flags != 0 && !(flags & (MT_FLAG_MLP_FUSED | MT_FLAG_MLP_FUSED_MMA))) return 2;
    FusedMlpParams params = {};
    params.M = M;
    params.H = H;
    params.I = I;
    const int sms = device_sm_count();
    if (sms <= 0) return 2;
    const bool want_mma = (flags & MT_FLAG_MLP_FUSED_MMA) != 0;
    if (!want_mma && (flags || M <= kFusedDefaultRows) && fused_mlp_applicable(params, sms)) return 1;  // null pointers count as aligned
    return (want_mma || (!flags && M > kFusedDefaultRows)) && fused_mlp_mma_applicable(params, sms) ? 1 : 2;
}

size_t mt_affine_mlp_static_max_bytes(void) { return kStaticHiddenBytes; }

int mt_affine_mlp_static(const void* x, const uint32_t* gate_w, const void* gate_scales, const void* gate_biases,
                         const uint32_t* up_w, const void* up_scales, const void* up_biases, const uint32_t* down_w,
                         const void* down_scales, const void* down_biases, const void* residual, void* out, int M,
                         int H, int I, int group_size, int bits, unsigned int flags, void* stream) {
    if (M < 0 || H < 1 || I < 1) return MT_ERR_SHAPE;
    if (M == 0) return MT_OK;
    const size_t needed = (size_t)M * (size_t)I * 2;
    if (needed > kStaticHiddenBytes) return MT_ERR_WORKSPACE;  // the hidden activations do not fit the array
    void* scratch = nullptr;
    const int rc = static_hidden_address(&scratch);
    if (rc != MT_OK) return rc;
    // Every element of hidden[0:M, 0:I] is written by the gate|up kernel before the down kernel
    // reads it, so nothing left over from an earlier call is ever consumed and nothing is cleared.
    return mt_affine_mlp(x, gate_w, gate_scales, gate_biases, up_w, up_scales, up_biases, down_w, down_scales,
                         down_biases, residual, scratch, kStaticHiddenBytes, out, M, H, I, group_size, bits, flags,
                         stream);
}

int mt_add_rmsnorm(const void* x, const void* residual, const void* weight, void* sum_out, void* norm_out, int rows,
                   int H, float eps, void* stream) {
    if (rows == 0) return MT_OK;
    if (!residual) return MT_ERR_NULL;
    if (!device_is_sm100()) return MT_ERR_DEVICE;
    return launch_add_rmsnorm(x, residual, weight, sum_out, norm_out, rows, H, eps, static_cast<cudaStream_t>(stream));
}

int mt_rmsnorm(const void* x, const void* weight, void* out, int rows, int H, float eps, void* stream) {
    if (rows == 0) return MT_OK;
    if (!device_is_sm100()) return MT_ERR_DEVICE;
    return launch_add_rmsnorm(x, nullptr, weight, nullptr, out, rows, H, eps, static_cast<cudaStream_t>(stream));
}

size_t mt_attention_decode_workspace_bytes(int batch, int q_heads, int tokens, int head_dim) {
    if (batch <= 0 || q_heads <= 0 || tokens <= 0 || head_dim <= 0) return 0;
    return attention_workspace_bytes(batch, q_heads, tokens, head_dim);
}

int mt_attention_decode(const void* q, const void* k_cache, const void* v_cache, const int* lengths, void* out,
                        void* workspace, size_t workspace_bytes, int batch, int q_heads, int kv_heads, int tokens,
                        int capacity, int head_dim, float scale, void* stream) {
    if (batch < 0 || q_heads < 1 || kv_heads < 1 || q_heads % kv_heads || q_heads / kv_heads > kAttnMaxGroup)
        return MT_ERR_SHAPE;
    if (head_dim != 64 && head_dim != 128) return MT_ERR_SHAPE;
    if (tokens < 1 || capacity < tokens) return MT_ERR_SHAPE;
    if (batch == 0) return MT_OK;
    if (!q || !k_cache || !v_cache || !out) return MT_ERR_NULL;
    if (!aligned_to(q, 16) || !aligned_to(k_cache, 16) || !aligned_to(v_cache, 16) || !aligned_to(out, 2))
        return MT_ERR_ALIGN;
    const int splits = attention_splits(tokens);
    if (splits > 1 && (!workspace || !aligned_to(workspace, 16) ||
                       workspace_bytes < attention_workspace_bytes(batch, q_heads, tokens, head_dim)))
        return MT_ERR_WORKSPACE;
    if (!device_is_sm100()) return MT_ERR_DEVICE;
    AttentionParams params;
    params.q = static_cast<const uint16_t*>(q);
    params.k = static_cast<const uint16_t*>(k_cache);
    params.v = static_cast<const uint16_t*>(v_cache);
    params.lengths = lengths;
    params.partial = static_cast<float*>(workspace);
    params.out = static_cast<uint16_t*>(out);
    params.q_heads = q_heads;
    params.kv_heads = kv_heads;
    params.capacity = capacity;
    params.tokens = tokens;
    params.splits = splits;
    params.scale = scale;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return head_dim == 128 ? launch_attention_dim<128>(params, batch, q_heads / kv_heads, s)
                           : launch_attention_dim<64>(params, batch, q_heads / kv_heads, s);
}

int mt_rope_kv_append(const void* q, const void* k, const void* v, long long row_stride, const int* positions,
                      void* q_out, void* k_cache, void* v_cache, int batch, int q_heads, int kv_heads, int capacity,
                      int head_dim, float theta, void* stream) {
    if (batch < 0 || q_heads < 1 || kv_heads < 1 || capacity < 1 || head_dim < 2 || head_dim % 2 || theta <= 0.0f)
        return MT_ERR_SHAPE;
    if (row_stride < (long long)kv_heads * head_dim) return MT_ERR_SHAPE;
    if (batch == 0) return MT_OK;
    if (!q || !k || !v || !positions || !q_out || !k_cache || !v_cache) return MT_ERR_NULL;
    if (!device_is_sm100()) return MT_ERR_DEVICE;
    RopeAppendParams params;
    params.q = static_cast<const uint16_t*>(q);
    params.k = static_cast<const uint16_t*>(k);
    params.v = static_cast<const uint16_t*>(v);
    params.positions = positions;
    params.q_out = static_cast<uint16_t*>(q_out);
    params.k_cache = static_cast<uint16_t*>(k_cache);
    params.v_cache = static_cast<uint16_t*>(v_cache);
    params.q_heads = q_heads;
    params.kv_heads = kv_heads;
    params.capacity = capacity;
    params.head_dim = head_dim;
    params.row_stride = row_stride;
    params.log2_theta = log2f(theta);
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(batch * (q_heads + 2 * kv_heads), 1, 1);
    config.blockDim = dim3(64, 1, 1);
    config.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attrs;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, rope_kv_append_kernel, params) == cudaSuccess ? MT_OK : MT_ERR_LAUNCH;
}

int mt_dense_rows(const void* x, const void* w, const void* residual, void* out, int M, int K, int N, void* stream) {
    if (!x || !w || !out) return MT_ERR_NULL;
    if (M == 0) return MT_OK;
    if (!device_is_sm100()) return MT_ERR_DEVICE;
    return launch_dense<DenseEpilogue::kPlain>(x, w, nullptr, residual, out, M, K, N, device_sm_count(),
                                               static_cast<cudaStream_t>(stream));
}

int mt_dense_swiglu(const void* x, const void* gate_w, const void* up_w, void* out, int M, int K, int N,
                    void* stream) {
    if (!x || !gate_w || !up_w || !out) return MT_ERR_NULL;
    if (M == 0) return MT_OK;
    if (!device_is_sm100()) return MT_ERR_DEVICE;
    return launch_dense<DenseEpilogue::kSwiglu>(x, gate_w, up_w, nullptr, out, M, K, N, device_sm_count(),
                                                static_cast<cudaStream_t>(stream));
}

int mt_dense_act(const void* a, const void* b, void* c, int M, int N, int K, unsigned int flags, void* stream) {
    if (!a || !b || !c) return MT_ERR_NULL;
    if (M < 0 || M > 128 || N < 1 || K < 1) return MT_ERR_SHAPE;
    if (M == 0) return MT_OK;
    if (!aligned_to(b, 4)) return MT_ERR_ALIGN;
    if (!device_is_sm100()) return MT_ERR_DEVICE;
    constexpr int kRows = 8;
    dim3 grid(((N + 1) / 2 + 127) / 128, (M + kRows - 1) / kRows);
    dense_act_kernel<kRows><<<grid, 128, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint16_t*>(a), static_cast<const uint16_t*>(b), static_cast<uint16_t*>(c), M, N, K,
        (flags & MT_FLAG_GELU) ? 1 : 0);
    return cudaGetLastError() == cudaSuccess ? MT_OK : MT_ERR_LAUNCH;
}

// ---- tensor-parallel sum over the GPUs of one node (peer stores over NVLink) --------------------------

int mt_peer_group_create(int rank, int world, size_t slot_bytes, void** group_out, void* ipc_handle_out) {
    if (!group_out || !ipc_handle_out) return MT_ERR_NULL;
    if (world < 1 || world > kPeerMaxWorld || rank < 0 || rank >= world) return MT_ERR_SHAPE;
    if (slot_bytes == 0 || slot_bytes % 16 || slot_bytes > (64u << 20)) return MT_ERR_SHAPE;
    if (!device_is_sm100()) return MT_ERR_DEVICE;
    PeerGroup* group = new PeerGroup();
    group->rank = rank;
    group->world = world;
    group->slot_bytes = slot_bytes;
    group->flags_offset = 2 * (size_t)world * slot_bytes;
    void* memory = nullptr;
    const size_t bytes = peer_group_bytes(world, slot_bytes);
    if (cudaGetDevice(&group->device) != cudaSuccess || cudaMalloc(&memory, bytes) != cudaSuccess) {
        delete group;
        return MT_ERR_LAUNCH;
    }
    cudaIpcMemHandle_t handle;
    if (cudaMemset(memory, 0, bytes) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess ||
        cudaIpcGetMemHandle(&handle, memory) != cudaSuccess) {
        cudaFree(memory);
        delete group;
        return MT_ERR_LAUNCH;
    }
    group->peers[rank] = static_cast<unsigned char*>(memory);
    static_assert(sizeof(handle) == 64, "CUDA IPC handles are 64 bytes");
    memcpy(ipc_handle_out, &handle, sizeof(handle));
    *group_out = group;
    return MT_OK;
}

int mt_peer_group_connect(void* group_pointer, const void* ipc_handles) {
    if (!group_pointer || !ipc_handles) return MT_ERR_NULL;
    PeerGroup* group = static_cast<PeerGroup*>(group_pointer);
    if (group->connected) return MT_OK;
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device != group->device) return MT_ERR_DEVICE;
    for (int peer = 0; peer < group->world; ++peer) {
        if (peer == group->rank) continue;
        cudaIpcMemHandle_t handle;
        memcpy(&handle, static_cast<const unsigned char*>(ipc_handles) + 64 * (size_t)peer, sizeof(handle));
        void* mapped = nullptr;
        if (cudaIpcOpenMemHandle(&mapped, handle, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
            cudaGetLastError();
            return MT_ERR_LAUNCH;
        }
        group->peers[peer] = static_cast<unsigned char*>(mapped);
        group->opened[peer] = true;
    }
    group->connected = true;
    return MT_OK;
}

int mt_peer_all_reduce(void* group_pointer, const void* partial, void* out, size_t elements, unsigned int limit_ms,
                       void* stream) {
    if (!group_pointer || !partial || !out) return MT_ERR_NULL;
    PeerGroup* group = static_cast<PeerGroup*>(group_pointer);
    if (!group->connected && group->world > 1) return MT_ERR_WORKSPACE;
    int device = -1;
    if (cudaGetDevice(&device) != cudaSuccess || device != group->device) return MT_ERR_DEVICE;
    if (limit_ms < 1 || limit_ms > 2000) return MT_ERR_SHAPE;
    return launch_peer_reduce(group, partial, out, elements, 1000000ull * limit_ms, static_cast<cudaStream_t>(stream));
}

int mt_peer_group_set_mode(void* group_pointer, int mode) {
    if (!group_pointer) return MT_ERR_NULL;
    if (mode < 0 || mode > 2) return MT_ERR_SHAPE;
    static_cast<PeerGroup*>(group_pointer)->mode = mode;
    return MT_OK;
}

int mt_peer_group_destroy(void* group_pointer) {
    if (!group_pointer) return MT_OK;
    PeerGroup* group = static_cast<PeerGroup*>(group_pointer);
    int rc = MT_OK;
    if (cudaDeviceSynchronize() != cudaSuccess) rc = MT_ERR_LAUNCH;
    for (int peer = 0; peer < group->world; ++peer)
        if (group->opened[peer] && cudaIpcCloseMemHandle(group->peers[peer]) != cudaSuccess) rc = MT_ERR_LAUNCH;
    if (group->peers[group->rank] && cudaFree(group->peers[group->rank]) != cudaSuccess) rc = MT_ERR_LAUNCH;
    delete group;
    return rc;
}

}  // extern "C"
