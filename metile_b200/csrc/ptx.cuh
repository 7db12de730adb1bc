// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA (plain per-CTA tiled loads),
// tcgen05 (TMEM alloc / mma / commit / ld / st) and cluster helpers.
//
// Every wait on an mbarrier is BOUNDED: after a time limit the waiter records a code in
// mt::g_device_status, raises the CTA's abort flag in shared memory and returns false.  Callers
// leave their pipeline loops when a wait fails, still pass every CTA / cluster barrier, and free
// their TMEM, so a logic error ends as a status code instead of a hung device.
#pragma once

#include "common.cuh"

namespace mt {
namespace ptx {

constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // 2 s

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---- mbarrier ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// try_wait with a suspend-time hint: the hardware may park the thread for up to `hint_ns` until the
// phase completes, instead of returning at once.  A parked warp takes no issue slots away from the
// warps that are working, which matters here: eighteen warps share four schedulers.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
        : "memory");
    return done != 0;
}

// Bounded wait.  `abort_flag` lives in shared memory and is shared by the whole CTA.  The kernels use
// the 2 s limit; only the library's self-test passes a shorter one, through the same code.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned int code, unsigned long long limit_ns = kWaitLimitNs) {
    if (mbar_try_wait(bar, parity)) return true;
    for (int spin = 0; spin < 64; ++spin)
        if (mbar_try_wait_hint(bar, parity, 100000u)) return true;
    const unsigned long long start = global_timer_ns();
    while (true) {
        if (mbar_try_wait_hint(bar, parity, 100000u)) return true;
        if (*abort_flag) return false;
        if (global_timer_ns() - start > limit_ns) {
            if (atomicCAS(&g_device_status[0], 0u, code) == 0u) {
                g_device_status[1] = blockIdx.x;
                g_device_status[2] = threadIdx.x;
                g_device_status[3] = parity;
            }
            *abort_flag = 1;
            return false;
        }
    }
}

// Bounded wait without a suspend-time hint: the waiter keeps polling, so it resumes within a few
// cycles of the phase completing.  For waits on the critical path of a short pipeline stage.
__device__ __forceinline__ bool mbar_wait_spin(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                               unsigned int code) {
    for (int spin = 0; spin < 4096; ++spin)
        if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long start = global_timer_ns();
    while (true) {
        for (int spin = 0; spin < 256; ++spin)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_timer_ns() - start > kWaitLimitNs) {
            if (atomicCAS(&g_device_status[0], 0u, code) == 0u) {
                g_device_status[1] = blockIdx.x;
                g_device_status[2] = threadIdx.x;
                g_device_status[3] = parity;
            }
            *abort_flag = 1;
            return false;
        }
    }
}

// ---- proxies / fences --------------------------------------------------------------------
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- TMA: 2-D tiled load, global -> this CTA's shared memory, completion on an mbarrier --
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const void* tensor_map, int c0, int c1, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(smem_dst)), "l"(tensor_map), "r"(c0), "r"(c1), "r"(smem_u32(bar))
        : "memory");
}

// ---- bulk copy: contiguous global bytes -> this CTA's shared memory, completion on an mbarrier.
// Both addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void prefetch_tensor_map(const void* tensor_map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tensor_map) : "memory");
}

// ---- tcgen05 -----------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_result)),
                 "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Waits for this thread's tcgen05.ld and names the 16 destination registers as in/out operands, so
// that no arithmetic on them can be scheduled above the wait.
__device__ __forceinline__ void tc_wait_ld16(uint32_t (&v)[16]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;"
                 : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
                   "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]),
                   "+r"(v[15])
                 :
                 : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// D[tmem] (+)= A[tmem] * B[smem desc], bf16 inputs, fp32 accumulate.
__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// Arrive on an mbarrier of this CTA once every tcgen05.mma issued so far by this thread is done.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns; thread i of the warp reads lane (base lane + i).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}

// 32 lanes x 16 consecutive 32-bit columns; thread i of the warp writes lane (base lane + i).
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, rows of 64 bf16 (128 B),
// groups of 8 rows 1024 B apart.  Field layout: start address >> 4 in bits [0,14), leading byte
// offset >> 4 in [16,30), stride byte offset >> 4 in [32,46), descriptor version 1 in [46,48),
// swizzle mode 2 (128 B) in [61,64).
__device__ __forceinline__ uint64_t smem_desc_k_major_sw128(uint32_t smem_addr) {
    uint64_t desc = 0;
    desc |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    desc |= (uint64_t)1 << 16;                 // leading byte offset: unused for swizzled K-major
    desc |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset: 8 rows x 128 B
    desc |= (uint64_t)1 << 46;                 // descriptor version (Blackwell)
    desc |= (uint64_t)2 << 61;                 // 128-byte swizzle
    return desc;
}

// Instruction descriptor for kind::f16: bf16 x bf16 -> fp32, both operands K-major.
// c_format (bits 4-5) = 1 (f32); a_format (7-9) = b_format (10-12) = 1 (bf16);
// N >> 3 in bits 17-22; M >> 4 in bits 24-28.
__host__ __device__ constexpr uint32_t umma_idesc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ---- programmatic dependent launch ----------------------------------------------------------
// launch_dependents: the next kernel in the stream (if launched with the programmatic-serialization
// attribute) may start once every CTA of this grid has executed this or exited.
// wait: blocks until the preceding grid has completed and its memory is visible.
__device__ __forceinline__ void griddep_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Coherent 128-bit global load for data the PRECEDING kernel may still have been writing when this
// kernel started (programmatic dependent launch): never the non-coherent (.nc / __ldg) path, and
// volatile (volatile asm statements keep their order) so the compiler keeps it after griddep_wait().
__device__ __forceinline__ uint4 ld_global_dependent_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_global_dependent_u16(const uint16_t* p) {
    uint16_t v;
    asm volatile("ld.global.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}

// 128-bit load served from L2, for data other CTAs of the SAME grid wrote before a grid-wide barrier.
__device__ __forceinline__ uint4 ld_global_l2_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ unsigned long long ld_acquire_gpu_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ unsigned long long atom_add_release_gpu_u64(unsigned long long* p, unsigned long long v) {
    unsigned long long old;
    asm volatile("atom.add.release.gpu.global.u64 %0, [%1], %2;" : "=l"(old) : "l"(p), "l"(v) : "memory");
    return old;
}

// ---- warp-level MMA: D[16x8] += A[16x16] * B[16x8], bf16 inputs, fp32 accumulate --------------
// Fragments (g = lane / 4, t = lane % 4): a0 = A[g][2t, 2t+1], a1 = A[g+8][2t, 2t+1],
// a2 = A[g][2t+8, 2t+9], a3 = A[g+8][2t+8, 2t+9]; b0 = B[2t, 2t+1][g], b1 = B[2t+8, 2t+9][g];
// d0, d1 = D[g][2t, 2t+1], d2, d3 = D[g+8][2t, 2t+1].
__device__ __forceinline__ void mma_bf16_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                  uint32_t b0, uint32_t b1) {
    // Not volatile: a pure function of its operands, so independent chains may be interleaved.
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- cluster -----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_arrive() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
}
__device__ __forceinline__ void cluster_wait() {
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of `smem_addr` (a shared::cta address of this CTA) as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_addr), "r"(rank));
    return out;
}
__device__ __forceinline__ float ld_cluster_f32(uint32_t cluster_addr) {
    float v;
    // volatile without a memory clobber: stays after the (volatile) cluster barrier, yet several of
    // these can be in flight at once.
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(cluster_addr));
    return v;
}

}  // namespace ptx
}  // namespace mt
