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
// Memory: each rank owns [2][world][slot_bytes] of receive slots plus two arrays of per-CTA flags,
// allocated by mt_peer_group_create and opened by the peers through CUDA IPC handles.  Calls alternate
// between the two slot sets: a rank can only be two calls ahead of a peer after that peer has launched
// the call in between, which in stream order means the peer finished reading the older set.
// Flags hold the call number (monotonic), so nothing is ever reset.  The call number itself lives on
// the device: every CTA reads it after the wait for the preceding kernel, and the last CTA to finish
// advances it, so a launch carries no per-call argument and a captured CUDA graph of it can be
// replayed (every rank must replay the same number of launches, as it must make the same calls).
//
// Very large messages among many ranks take TWO shots instead (peer_reduce_two_shot_kernel): every
// rank first sends each peer only the segment that peer will reduce, reduces its own segment in rank
// order, then sends the reduced segment to everyone -- 2 (world-1)/world messages' worth of stores
// per rank instead of world-1, for a second round of flags.  Both phases write into the same slots:
// peer j's slot of rank r holds rank r's partial in segment j (first shot) and rank r's reduced
// values in segment r (second shot), which never overlap.
//
// No multicast objects and no TMA are involved: ordinary stores to peer addresses and ordinary loads
// from local memory.  Every wait is bounded; a rank whose peer never arrives records the peer in
// g_device_status and returns without writing its output.
#pragma once

#include "common.cuh"
#include "ptx.cuh"

namespace mt {

constexpr int kPeerMaxWorld = 8;
constexpr int kPeerMaxCtas = 128;
constexpr int kPeerThreads = 512;
constexpr unsigned int kPeerWaitCode = 0x9E0;

struct PeerGroup {
    int rank;
    int world;
    int device;
    size_t slot_bytes;
    size_t flags_offset;
    unsigned char* peers[kPeerMaxWorld];  // every rank's allocation as mapped in this process
    int mode;                             // 0 = by size and rank count, 1 = always one shot, 2 = always two shots
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
    size_t flags_offset;   // first shot's flags [kPeerMaxWorld][kPeerMaxCtas], call counter, exit tickets, second shot's flags
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

// Raises this CTA's flag for `call` on every peer (flag array `which`: 0 = first shot, 1 = second) and
// waits, bounded, for the peers' flags here.  Called by all threads after their stores: the CTA
// barrier orders those stores before the signalling threads, whose system-scope fence and release
// store then publish them (one fence per signalling thread instead of one per thread of the CTA: a
// system fence waits for every store the SM has in flight).  Returns after a __syncthreads() with
// *gave_up set if a peer never arrived.
__device__ __forceinline__ void peer_signal_and_wait(unsigned char* const* peers, const PeerReduceParams& p, int which,
                                                     unsigned int call, int* gave_up) {
    __syncthreads();
    const int peer = threadIdx.x;
    if (peer < p.world && peer != p.rank) {
        const size_t flags = p.flags_offset + (size_t)which * (kPeerMaxWorld * kPeerMaxCtas + 4) * sizeof(unsigned int);
        unsigned int* theirs = reinterpret_cast<unsigned int*>(peers[peer] + flags) + p.rank * kPeerMaxCtas + blockIdx.x;
        __threadfence_system();
        st_release_sys(theirs, call);
        const unsigned int* here =
            reinterpret_cast<const unsigned int*>(peers[p.rank] + flags) + peer * kPeerMaxCtas + blockIdx.x;
        const unsigned long long start = ptx::global_timer_ns();
        while ((int)(ld_acquire_sys(here) - call) < 0) {
            if (ptx::global_timer_ns() - start > p.limit_ns) {
                if (atomicCAS(&g_device_status[0], 0u, kPeerWaitCode) == 0u) {
                    g_device_status[1] = blockIdx.x;
                    g_device_status[2] = (unsigned int)peer;
                    g_device_status[3] = call;
                }
                *gave_up = 1;
                break;
            }
        }
    }
    __syncthreads();
}

// The last CTA out advances the call counter (also after a wait that gave up: the peers count
// launches, not successes).
__device__ __forceinline__ void peer_finish_call(unsigned int* counter, unsigned int call) {
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

__device__ __forceinline__ uint4 sum_in_rank_order(const PeerReduceParams& p, const unsigned char* slots, unsigned int i) {
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
    return r;
}

__global__ void __launch_bounds__(kPeerThreads) peer_reduce_two_shot_kernel(const PeerReduceParams p) {
    __shared__ int gave_up;
    __shared__ unsigned int call_shared;
    __shared__ unsigned char* peers[kPeerMaxWorld];
    if (threadIdx.x == 0) gave_up = 0;
    if (threadIdx.x < kPeerMaxWorld) {
#pragma unroll
        for (int i = 0; i < kPeerMaxWorld; ++i)
            if (i == threadIdx.x) peers[i] = p.peers[i];
    }
    ptx::griddep_wait();
    unsigned int* counter = reinterpret_cast<unsigned int*>(p.local + p.flags_offset) + kPeerMaxWorld * kPeerMaxCtas;
    if (threadIdx.x == 0) call_shared = __ldcg(counter) + 1u;
    __syncthreads();
    const unsigned int call = call_shared;
    const unsigned int set = call & 1u;
    // Segment j = the part of the message rank j reduces; CTA c covers chunk c of every segment.
    const unsigned int longest = (p.vectors + p.world - 1) / p.world;
    const unsigned int per_cta = (longest + gridDim.x - 1) / gridDim.x;
    auto chunk_of = [&](int j, unsigned int& begin, unsigned int& end) {
        const unsigned int first = (unsigned int)(((unsigned long long)p.vectors * j) / p.world);
        const unsigned int last = (unsigned int)(((unsigned long long)p.vectors * (j + 1)) / p.world);
        begin = min(first + blockIdx.x * per_cta, last);
        end = min(begin + per_cta, last);
    };
    const size_t mine = ((size_t)set * p.world + p.rank) * p.slot_bytes;
    const unsigned char* slots = peers[p.rank] + (size_t)set * p.world * p.slot_bytes;

    // first shot: to every peer, the chunk of ITS segment
    for (int j = 0; j < p.world; ++j) {
        if (j == p.rank) continue;
        unsigned int begin, end;
        chunk_of(j, begin, end);
        uint4* theirs = reinterpret_cast<uint4*>(peers[j] + mine);
        for (unsigned int i = begin + threadIdx.x; i < end; i += blockDim.x) theirs[i] = p.partial[i];
    }
    peer_signal_and_wait(peers, p, 0, call, &gave_up);
    if (!gave_up) {
        // this rank's segment: add in rank order, keep the result and send it to everyone
        unsigned int begin, end;
        chunk_of(p.rank, begin, end);
        for (unsigned int i = begin + threadIdx.x; i < end; i += blockDim.x) {
            const uint4 r = sum_in_rank_order(p, slots, i);
            p.out[i] = r;
            for (int j = 0; j < p.world; ++j)
                if (j != p.rank) reinterpret_cast<uint4*>(peers[j] + mine)[i] = r;
        }
    }
    peer_signal_and_wait(peers, p, 1, call, &gave_up);
    if (!gave_up) {
        // second shot landed: the peers' reduced segments
        for (int j = 0; j < p.world; ++j) {
            if (j == p.rank) continue;
            unsigned int begin, end;
            chunk_of(j, begin, end);
            const uint4* theirs = reinterpret_cast<const uint4*>(slots + (size_t)j * p.slot_bytes);
            for (unsigned int i = begin + threadIdx.x; i < end; i += blockDim.x) p.out[i] = __ldcg(theirs + i);
        }
    }
    peer_finish_call(counter, call);
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
    // 2. signal every peer, wait until each peer's CTA of the same index has pushed its part here
    peer_signal_and_wait(peers, p, 0, call, &gave_up);

    // 3. add the slots in rank order (this rank's own partial takes its place in the order)
    if (!gave_up) {
        const unsigned char* slots = peers[p.rank] + (size_t)set * p.world * p.slot_bytes;
        for (unsigned int i = begin + threadIdx.x; i < end; i += blockDim.x) p.out[i] = sum_in_rank_order(p, slots, i);
    }
    peer_finish_call(counter, call);
}

inline size_t peer_group_bytes(int world, size_t slot_bytes) {
    // two slot sets, then per shot a flag array [kPeerMaxWorld][kPeerMaxCtas] followed by four words
    // (the first shot's hold the call counter and the exit tickets)
    return 2 * (size_t)world * slot_bytes + 2 * ((size_t)kPeerMaxWorld * kPeerMaxCtas + 4) * sizeof(unsigned int);
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
    // The grid and the choice between one and two shots depend on the message size and the rank count
    // only, so every rank launches the same kernel with the same grid.  Two shots send
    // 2 (world-1)/world messages instead of world-1 but pay a second round of stores, system fence and
    // flags (about 10 us): measured on four GPUs at 1.3 MB, 34.7 us against 25.6 us for one shot, so the
    // default takes two shots only where one shot would store more than 4 MB per rank among six or more
    // ranks (eight GPUs, 1.3 MB messages, 9.2 MB of stores: 34 us, level with the library all-reduce).
    const bool two_shot = group->world >= 2 &&
                          (group->mode == 2 || (group->mode == 0 && group->world >= 6 &&
                                                elements * 2 * (size_t)(group->world - 1) >= (4u << 20)));
    const unsigned int units = two_shot ? (p.vectors + group->world - 1) / group->world : p.vectors;
    int grid = (int)((units + kPeerThreads - 1) / kPeerThreads);
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
    const cudaError_t rc = two_shot ? cudaLaunchKernelEx(&config, peer_reduce_two_shot_kernel, p)
                                    : cudaLaunchKernelEx(&config, peer_reduce_kernel, p);
    return rc == cudaSuccess ? MT_OK : MT_ERR_LAUNCH;
}

}  // namespace mt
