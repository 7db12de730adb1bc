// Sum of bf16 partial results over the GPUs of one node, through the peers' memory (NVLink).
//
// The tensor-parallel MLP ends with every rank holding a partial [M, H] result of a few KB to about
// a megabyte.  At that size a collective is latency, not bandwidth, so this is a ONE-SHOT exchange in
// one kernel per rank: every rank stores its partial into a slot of every peer's receive buffer
// (plain 16-byte stores over NVLink), raises one flag per (peer, CTA) with a system-scope release,
// waits for the flags its peers raised here, and adds the `world` slots in RANK ORDER in fp32.  Every
// rank therefore computes the same sum in the same order: the result is identical on all ranks and
// does not depend on message size, which a library all-reduce does not promise.
//
// Memory: each rank owns [2][world][slot_bytes] of receive slots plus [world][kPeerMaxCtas] flags,
// allocated by mt_peer_group_create and opened by the peers through CUDA IPC handles.  Calls alternate
// between the two slot sets: a rank can only be two calls ahead of a peer after that peer has launched
// the call in between, which in stream order means the peer finished reading the older set.
// Flags hold the call number (monotonic), so nothing is ever reset.  The call number itself lives on
// the device: every CTA reads it after the wait for the preceding kernel, and the last CTA to finish
// advances it, so a launch carries no per-call argument and a captured CUDA graph of it can be
// replayed (every rank must replay the same number of launches, as it must make the same calls).
//
// No multicast objects and no TMA are involved: ordinary stores to peer addresses and ordinary loads
// from local memory.  Every wait is bounded; a rank whose peer never arrives records the peer in
// g_device_status and returns without writing its output.
#pragma once

#include "common.cuh"
#include "ptx.cuh"

namespace mt {

constexpr int kPeerMaxWorld = 8;
constexpr int kPeerMaxCtas = 64;
constexpr int kPeerThreads = 512;
constexpr unsigned int kPeerWaitCode = 0x9E0;

struct PeerGroup {
    int rank;
    int world;
    int device;
    size_t slot_bytes;
    size_t flags_offset;
    unsigned char* peers[kPeerMaxWorld];  // every rank's allocation as mapped in this process
    bool opened[kPeerMaxWorld];
    bool connected;
};

struct PeerReduceParams {
    const uint4* partial;
    uint4* out;
    unsigned char* peers[kPeerMaxWorld];
    unsigned char* local;  // == peers[rank]
    int rank;
    int world;
    unsigned int vectors;  // 16-byte units of the message
    size_t slot_bytes;
    size_t flags_offset;   // [world][kPeerMaxCtas] flags, then the call counter and the exit tickets
    unsigned long long limit_ns;
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void accumulate_bf16x8(float* acc, const uint4& v) {
    acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x);
    acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
    acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z);
    acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
}

__global__ void __launch_bounds__(kPeerThreads) peer_reduce_kernel(const PeerReduceParams p) {
    __shared__ int gave_up;
    __shared__ unsigned int call_shared;
    __shared__ unsigned char* peers[kPeerMaxWorld];  // indexed at run time: kept out of the parameter space
    const unsigned int per_cta = (p.vectors + gridDim.x - 1) / gridDim.x;
    const unsigned int begin = blockIdx.x * per_cta;
    const unsigned int end = min(begin + per_cta, p.vectors);
    if (threadIdx.x == 0) gave_up = 0;
    if (threadIdx.x < kPeerMaxWorld) {
#pragma unroll
        for (int i = 0; i < kPeerMaxWorld; ++i)
            if (i == threadIdx.x) peers[i] = p.peers[i];
    }
    // The partial is the output of the kernel before this one in the stream; the call counter was
    // advanced by the previous launch of this kernel.
    ptx::griddep_wait();
    unsigned int* counter = reinterpret_cast<unsigned int*>(p.local + p.flags_offset) + kPeerMaxWorld * kPeerMaxCtas;
    if (threadIdx.x == 0) call_shared = __ldcg(counter) + 1u;
    __syncthreads();
    const unsigned int call = call_shared;
    const unsigned int set = call & 1u;

    // 1. push this CTA's part of the partial into slot `rank` of every peer
    const size_t mine = ((size_t)set * p.world + p.rank) * p.slot_bytes;
    for (unsigned int i = begin + threadIdx.x; i < end; i += blockDim.x) {
        const uint4 v = p.partial[i];
        for (int peer = 0; peer < p.world; ++peer)
            if (peer != p.rank) reinterpret_cast<uint4*>(peers[peer] + mine)[i] = v;
    }
    __threadfence_system();
    __syncthreads();
    const int peer = threadIdx.x;
    if (peer < p.world && peer != p.rank) {
        unsigned int* theirs =
            reinterpret_cast<unsigned int*>(peers[peer] + p.flags_offset) + p.rank * kPeerMaxCtas + blockIdx.x;
        st_release_sys(theirs, call);

        // 2. wait until that peer's CTA of the same index has pushed its part here
        const unsigned int* here =
            reinterpret_cast<const unsigned int*>(peers[p.rank] + p.flags_offset) + peer * kPeerMaxCtas + blockIdx.x;
        const unsigned long long start = ptx::global_timer_ns();
        while ((int)(ld_acquire_sys(here) - call) < 0) {
            if (ptx::global_timer_ns() - start > p.limit_ns) {
                if (atomicCAS(&g_device_status[0], 0u, kPeerWaitCode) == 0u) {
                    g_device_status[1] = blockIdx.x;
                    g_device_status[2] = (unsigned int)peer;
                    g_device_status[3] = call;
                }
                gave_up = 1;
                break;
            }
        }
    }
    __syncthreads();

    // 3. add the slots in rank order (this rank's own partial takes its place in the order)
    if (!gave_up) {
        const unsigned char* slots = peers[p.rank] + (size_t)set * p.world * p.slot_bytes;
        for (unsigned int i = begin + threadIdx.x; i < end; i += blockDim.x) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (int source = 0; source < p.world; ++source) {
                const uint4 v = source == p.rank
                                    ? p.partial[i]
                                    : __ldcg(reinterpret_cast<const uint4*>(slots + (size_t)source * p.slot_bytes) + i);
                accumulate_bf16x8(acc, v);
            }
            uint4 r;
            r.x = pack_bf16x2(acc[0], acc[1]);
            r.y = pack_bf16x2(acc[2], acc[3]);
            r.z = pack_bf16x2(acc[4], acc[5]);
            r.w = pack_bf16x2(acc[6], acc[7]);
            p.out[i] = r;
        }
    }

    // 4. the last CTA out advances the call counter (also after a wait that gave up: the peers count
    //    launches, not successes)
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned int* tickets = counter + 1;
        if (atomicAdd(tickets, 1u) == gridDim.x - 1) {
            *tickets = 0u;
            *counter = call;
            __threadfence();
        }
    }
}

inline size_t peer_group_bytes(int world, size_t slot_bytes) {
    return 2 * (size_t)world * slot_bytes + ((size_t)kPeerMaxWorld * kPeerMaxCtas + 4) * sizeof(unsigned int);
}

inline int launch_peer_reduce(PeerGroup* group, const void* partial, void* out, size_t elements,
                              unsigned long long limit_ns, cudaStream_t stream) {
    if (elements == 0) return MT_OK;
    if (elements % 8) return MT_ERR_SHAPE;
    if (elements * 2 > group->slot_bytes) return MT_ERR_WORKSPACE;
    if (!aligned_to(partial, 16) || !aligned_to(out, 16)) return MT_ERR_ALIGN;
    PeerReduceParams p;
    p.partial = static_cast<const uint4*>(partial);
    p.out = static_cast<uint4*>(out);
    for (int i = 0; i < kPeerMaxWorld; ++i) p.peers[i] = group->peers[i];
    p.local = group->peers[group->rank];
    p.rank = group->rank;
    p.world = group->world;
    p.vectors = (unsigned int)(elements / 8);
    p.slot_bytes = group->slot_bytes;
    p.flags_offset = group->flags_offset;
    p.limit_ns = limit_ns;
    // The grid depends on the message size only, so CTA c of every rank covers the same part.
    int grid = (int)((p.vectors + 2 * kPeerThreads - 1) / (2 * kPeerThreads));
    grid = grid < 1 ? 1 : grid > kPeerMaxCtas ? kPeerMaxCtas : grid;
    cudaLaunchConfig_t config = {};
    config.gridDim = dim3(grid);
    config.blockDim = dim3(kPeerThreads);
    config.stream = stream;
    cudaLaunchAttribute attribute;
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute.val.programmaticStreamSerializationAllowed = 1;
    config.attrs = &attribute;
    config.numAttrs = 1;
    return cudaLaunchKernelEx(&config, peer_reduce_kernel, p) == cudaSuccess ? MT_OK : MT_ERR_LAUNCH;
}

}  // namespace mt
