// Expert parallelism inside one NVLink box: every GPU holds a contiguous block of the experts and a contiguous
// block of the request's tokens. Nothing is packed, sent and unpacked: the dispatch is the permutation kernel reading
// token rows from their owners' memory, the return is the FC2 epilogue writing each route's row into the owner's
// buffer, both through peer mappings. What remains between the GPUs is two rendezvous per step (rows ready, results
// complete) and one small pull of everybody's routes.
//
// Window of a rank (one allocation, mapped by every peer):
//   EpHeader | ids [cap][8] i32 | weights [cap][8] f32 | xq [cap][4096] | xs [cap][128] | y [cap][8][4096] f32
// `cap` is the largest token block of any rank.
#pragma once
#include "ffn_kernels.cuh"

namespace m26b {

struct EpHeader {
    uint32_t flags[2][8];      // flags[b][r] = last step for which rank r reached rendezvous b
    uint32_t error;            // bit (8 b + r): gave up waiting for rank r at rendezvous b
    uint32_t pad[47];
};
static_assert(sizeof(EpHeader) == 256, "window header is 256 bytes");

struct EpLayout {
    uint32_t cap;
    __host__ __device__ size_t ids_off() const { return sizeof(EpHeader); }
    __host__ __device__ size_t w_off() const { return ids_off() + size_t(cap) * kTopK * 4; }
    __host__ __device__ size_t xq_off() const { return w_off() + size_t(cap) * kTopK * 4; }
    __host__ __device__ size_t xs_off() const { return xq_off() + size_t(cap) * kHidden; }
    __host__ __device__ size_t y_off() const { return (xs_off() + size_t(cap) * (kHidden / kBlockK) + 255) & ~size_t(255); }
    __host__ __device__ size_t bytes() const { return y_off() + size_t(cap) * kTopK * kHidden * 4; }
};

struct EpPeers {
    uint8_t* window[8];
};

// Rendezvous `which` of step `step`: tell every peer, then wait (bounded) until every peer has told this rank.
// One CTA; thread r handles peer r. Everything this GPU wrote in earlier kernels of the stream is visible to a
// peer that has seen the flag; everything the peers wrote before their flags is visible to the kernels after this one.
__global__ void __launch_bounds__(32) ep_rendezvous_kernel(EpPeers peers, int rank, int world, int which, uint32_t step,
                                                           long long wait_cycles) {
    EpHeader* mine = reinterpret_cast<EpHeader*>(peers.window[rank]);
    const int r = int(threadIdx.x);
    if (r < world && r != rank) {
        __threadfence_system();
        st_release_sys(&reinterpret_cast<EpHeader*>(peers.window[r])->flags[which][rank], step);
        const long long t0 = clock64();
        while (int32_t(ld_acquire_sys(&mine->flags[which][r]) - step) < 0) {
            if (clock64() - t0 > wait_cycles) { atomicOr(&mine->error, 1u << (8 * which + r)); break; }
        }
    }
}

// Pull every rank's routes (ids, weights) into one local array in request order.
__global__ void __launch_bounds__(256) ep_gather_routes_kernel(EpPeers peers, EpLayout lay, int world, TokenSources shards,
                                                               int32_t* __restrict__ ids, float* __restrict__ w) {
    const uint32_t total = shards.lo[world] * kTopK;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const uint32_t token = i / kTopK;
        uint32_t k = 0;
#pragma unroll
        for (uint32_t j = 1; j < 8; ++j)
            if (j < uint32_t(world) && token >= shards.lo[j]) k = j;
        const uint32_t local = i - shards.lo[k] * kTopK;
        ids[i] = __ldcv(reinterpret_cast<const int32_t*>(peers.window[k] + lay.ids_off()) + local);
        w[i] = __ldcv(reinterpret_cast<const float*>(peers.window[k] + lay.w_off()) + local);
    }
}

}  // namespace m26b
