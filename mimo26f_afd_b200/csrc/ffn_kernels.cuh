// The bandwidth-bound kernels around the two grouped GEMMs: activation
// quantisers, the stable route planner, the token-to-expert permutation, the
// ordered top-k weighted combine, the cross-rank sum and the weight repack.
// All are plain coalesced/vectorised CUDA; none reshapes its work into a GEMM.
#pragma once
#include <cuda_runtime.h>
#include "layout.cuh"
#include "codec.cuh"
#include "sm100_ptx.cuh"

namespace m26b {

// ---------------------------------------------------------------- quantisers
// One K32 block = two threads of sixteen elements (2 x 16-byte loads for BF16, 4 x 16 bytes for FP32, one 16-byte
// store); the block maximum crosses the two lanes by shuffle.
// CODEC 0: wire codec (scale byte 0 for a zero block, ties away from zero).
// CODEC 1: quant_v1 (floor 1e-4, ties to even, faults instead of clipping; a
// faulting block writes nothing), crates/mimo26-expert/kernels/b1/quant_v1.cu:34-59.
// Sixteen consecutive elements starting at element 16 g (half a K32 block; the other half is lane ^ 1's): the packed
// payload, the block's scale byte and whether the block may be written; faults are ORed into `bad`. Every lane of the
// warp must call it (the halves meet by shuffle); `live` = this lane's elements exist.
template <int CODEC, typename IN>
__device__ __forceinline__ bool quant16(const IN* __restrict__ x, uint64_t g, bool live, uint4& out, uint32_t& sbyte, uint32_t& bad) {
    uint32_t bits[16];
    if (live) {
        if constexpr (sizeof(IN) == 2) {
            const uint4 a = reinterpret_cast<const uint4*>(x)[2 * g], b = reinterpret_cast<const uint4*>(x)[2 * g + 1];
            const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 8; ++i) { bits[2 * i] = w[i] << 16; bits[2 * i + 1] = w[i] & 0xffff0000u; }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint4 a = reinterpret_cast<const uint4*>(x)[4 * g + i];
                bits[4 * i] = a.x; bits[4 * i + 1] = a.y; bits[4 * i + 2] = a.z; bits[4 * i + 3] = a.w;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 16; ++i) bits[i] = 0;
    }
    uint32_t amax = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        uint32_t m = bits[i] & 0x7fffffffu;
        if (CODEC == 0 && m > 0x7f800000u) m = 0;   // the wire codec's maximum skips NaN
        amax = m > amax ? m : amax;
    }
    const uint32_t o = __shfl_xor_sync(0xffffffffu, amax, 1);
    amax = o > amax ? o : amax;
    uint32_t code[16];
    bool write = live;
    if constexpr (CODEC == 0) {
        sbyte = wire_scale_byte(amax);
#pragma unroll
        for (int i = 0; i < 16; ++i) code[i] = wire_payload(bits[i], sbyte);
    } else {
        bool over = false;
        if (amax >= 0x7f800000u) {
            if (live) bad |= kFaultQuantNonfinite;
            write = false;
            sbyte = 0;
#pragma unroll
            for (int i = 0; i < 16; ++i) code[i] = 0;
        } else {
            const int k = quant_v1_scale_exp(amax);
            sbyte = uint32_t(k + 127);
#pragma unroll
            for (int i = 0; i < 16; ++i) { code[i] = quant_v1_payload(bits[i], k); over |= !quant_v1_finite(code[i], k); }
        }
        uint32_t ov = over ? 1u : 0u;
        ov |= __shfl_xor_sync(0xffffffffu, ov, 1);
        if (ov) { if (live) bad |= kFaultQuantOverflow; write = false; }
    }
    out.x = code[0] | (code[1] << 8) | (code[2] << 16) | (code[3] << 24);
    out.y = code[4] | (code[5] << 8) | (code[6] << 16) | (code[7] << 24);
    out.z = code[8] | (code[9] << 8) | (code[10] << 16) | (code[11] << 24);
    out.w = code[12] | (code[13] << 8) | (code[14] << 16) | (code[15] << 24);
    return write;
}
template <int CODEC, typename IN>
__device__ __forceinline__ void quantize_span(const IN* __restrict__ x, uint64_t n_elems, uint8_t* __restrict__ payload,
                                              uint8_t* __restrict__ scales, uint32_t* __restrict__ fault, uint64_t first,
                                              uint64_t stride) {
    const uint64_t n16 = n_elems / 16;
    uint32_t bad = 0;
    // the bound is rounded up to a whole warp so every lane reaches the shuffles
    for (uint64_t g = first; g < ((n16 + 31) & ~uint64_t(31)); g += stride) {
        uint4 out;
        uint32_t sbyte;
        if (quant16<CODEC, IN>(x, g, g < n16, out, sbyte, bad)) {
            reinterpret_cast<uint4*>(payload)[g] = out;
            if ((g & 1) == 0) scales[g >> 1] = uint8_t(sbyte);
        }
    }
    if (bad) atomicOr(fault, bad);
}
template <int CODEC, typename IN>
__global__ void __launch_bounds__(256) quantize_rows_kernel(const IN* __restrict__ x, uint64_t n_elems,
                                                            uint8_t* __restrict__ payload,
                                                            uint8_t* __restrict__ scales,
                                                            uint32_t* __restrict__ fault) {
    quantize_span<CODEC, IN>(x, n_elems, payload, scales, fault, uint64_t(blockIdx.x) * blockDim.x + threadIdx.x,
                             uint64_t(gridDim.x) * blockDim.x);
}

// ---------------------------------------------------------------- router (the caller's step before the plan)
// crates/mimo26-coordinator/src/router.rs:42-80 and kernels/glue.cu:72-126: FP64 sigmoid of the FP32 logits, the
// top 8 of 256 experts by score + bias (descending, a tie to the lower expert id), weights = unbiased scores over
// their sum taken in selection order, all in FP64, stored as FP32. One warp per token: lane l holds experts
// l, l + 32, ..., l + 224, so a lane's candidates are in ascending id order and a strict comparison keeps the lower id.
__device__ __forceinline__ void router_topk_warp(const float* __restrict__ logits, const float* __restrict__ bias,
                                                 uint32_t lane, int32_t* __restrict__ ids_out, float* __restrict__ w_out) {
    double score[8], sel[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = int(lane) + 32 * i;
        score[i] = 1.0 / (1.0 + exp(-double(logits[e])));
        sel[i] = score[i] + (bias ? double(bias[e]) : 0.0);
    }
    uint32_t taken = 0;
    double wsum = 0.0, mine_score = 0.0;
    int32_t mine_id = 0;
#pragma unroll 1
    for (int k = 0; k < kTopK; ++k) {
        double bv = 0.0;
        int bi = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (!((taken >> i) & 1u) && (bi == 0x7fffffff || sel[i] > bv)) { bv = sel[i]; bi = int(lane) + 32 * i; }
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) {
            const double ov = __shfl_xor_sync(0xffffffffu, bv, d);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, d);
            if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
        }
        double sc = 0.0;
        if ((uint32_t(bi) & 31u) == lane) {
            const int slot = bi >> 5;
            taken |= 1u << slot;
#pragma unroll
            for (int i = 0; i < 8; ++i)
                if (i == slot) sc = score[i];
        }
        sc = __shfl_sync(0xffffffffu, sc, bi & 31);
        wsum += sc;
        if (int(lane) == k) { mine_id = bi; mine_score = sc; }
    }
    if (lane < uint32_t(kTopK)) {
        ids_out[lane] = mine_id;
        w_out[lane] = float(mine_score / wsum);
    }
}

// The caller's two steps in front of the path in one launch: the first `router_ctas` CTAs route (8 tokens each, one
// warp per token), the others quantise the hidden rows. n_elems = 0: routing only.
template <int CODEC, typename IN>
__global__ void __launch_bounds__(256) produce_kernel(const float* __restrict__ logits, const float* __restrict__ bias,
                                                      uint32_t rows, uint32_t router_ctas, int32_t* __restrict__ ids_out,
                                                      float* __restrict__ w_out, const IN* __restrict__ x, uint64_t n_elems,
                                                      uint8_t* __restrict__ payload, uint8_t* __restrict__ scales,
                                                      uint32_t* __restrict__ fault) {
    if (blockIdx.x < router_ctas) {
        const uint32_t token = blockIdx.x * 8u + (threadIdx.x >> 5);
        if (token < rows)
            router_topk_warp(logits + size_t(token) * kExperts, bias, threadIdx.x & 31u, ids_out + size_t(token) * kTopK,
                             w_out + size_t(token) * kTopK);
        return;
    }
    if (n_elems)
        quantize_span<CODEC, IN>(x, n_elems, payload, scales, fault, uint64_t(blockIdx.x - router_ctas) * blockDim.x + threadIdx.x,
                                 uint64_t(gridDim.x - router_ctas) * blockDim.x);
}

// ---------------------------------------------------------------- route plan
struct ExpertPlan {
    int32_t count, rbase, tile_start, width;
};
struct PlanOut {
    int32_t* inverse;          // original route -> grouped route
    int32_t* original_routes;  // grouped route -> original route
    float* grouped_weights;
    ExpertPlan* experts;       // [256]
    TokenTile* tiles;
    WorkItem* items_fc1;
    WorkItem* items_fc2;
    PlanMeta* meta;
};

// One CTA of 32 warps. Validates the routes, counts per expert, then places
// routes in expert-major order, stable inside an expert (identical to a stable
// sort by expert id: crates/mimo26-expert/kernels/b1/group_plan.cu:32-79), and
// cuts each expert's run into token tiles of at most `max_n` rows.
// Rejection rules as the reference planner (b1_serve.cu:46-59): id in
// [0,256), expert resident, 0 <= weight <= FLT_MAX, no expert twice in a row.
//
// Each warp owns one contiguous segment of the routes. It counts its segment
// per expert, a 256-thread pass turns the counts into per-(warp, expert) start
// offsets, and each warp then walks its segment again in route order, 32 routes
// at a time, ranking equal experts inside the group with match.any. Between
// the two block-wide barriers no warp waits for another.
__device__ __forceinline__ uint32_t warp_inclusive_scan(uint32_t v, uint32_t lane) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint32_t o = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= uint32_t(d)) v += o;
    }
    return v;
}
// Work items: for every token tile, weight tile pairs 0, m_step, 2 m_step ... of each GEMM (m_step1 for FC1, m_step2 for FC2:
// 2 when a CTA pair takes two
// neighbouring weight tile pairs per item).
//
// skip_foreign (expert parallelism: this GPU holds a subset of the experts and sees every route of the request): a
// route this rank does not serve (slot_serves: an expert it does not hold, or a replicated expert and somebody else's
// token) is left out of the plan (inverse = -1) instead of rejecting the request; the other rules still apply to every
// route. `slots` is the layer's expert table, [own_lo, own_hi) the tokens of the pass this rank owns.
struct PlanScope {
    const int16_t* slots;
    uint32_t own_lo, own_hi;
    int skip_foreign;
};
__global__ void __launch_bounds__(1024) plan_kernel(const int32_t* __restrict__ ids, const float* __restrict__ w,
                                                    uint32_t rows, PlanScope sc, int max_n,
                                                    int mt_fc1, int mt_fc2, int m_step1, int m_step2, PlanOut o) {
    const int skip_foreign = sc.skip_foreign;
    const int16_t* __restrict__ slots = sc.slots;
    mt_fc1 /= m_step1;
    mt_fc2 /= m_step2;
    __shared__ uint32_t cnt[kExperts], rbase[kExperts], tstart[kExperts], width[kExperts], ntl[kExperts];
    __shared__ uint32_t i1base[kExperts], i2base[kExperts];
    __shared__ uint32_t wcnt[32][kExperts];
    __shared__ uint32_t wsum[4][8];
    __shared__ uint32_t bad, max_count;
    const uint32_t tid = threadIdx.x, routes = rows * kTopK;
    const uint32_t lane = tid & 31u, warp = tid >> 5;
    const uint32_t seg = (((routes + 31u) / 32u) + 31u) & ~31u;          // routes per warp, a multiple of 32
    const uint32_t lo = warp * seg < routes ? warp * seg : routes;
    const uint32_t hi = lo + seg < routes ? lo + seg : routes;
    for (uint32_t i = tid; i < 32 * kExperts; i += 1024) (&wcnt[0][0])[i] = 0;
    if (tid == 0) { bad = 0; max_count = 0; }
    __syncthreads();
    uint32_t my_bad = 0;
    for (uint32_t r0 = lo; r0 < hi; r0 += 32) {
        const uint32_t r = r0 + lane;
        const bool live = r < hi;
        int32_t e = -1;
        bool ok = false;
        if (live) {
            e = ids[r];
            const float wt = w[r];
            ok = e >= 0 && e < kExperts && wt >= 0.0f && wt <= 3.402823466e+38f;
            if (ok)
                for (uint32_t k = (r / kTopK) * kTopK; k < r; ++k) ok = ok && ids[k] != e;
            const bool here = ok && slot_serves(sc.slots[e], r / kTopK, sc.own_lo, sc.own_hi);
            if (skip_foreign ? !ok : !here) my_bad = 1;
            ok = here;
        }
        const uint32_t peers = __match_any_sync(0xffffffffu, ok ? e : -1 - int32_t(lane));
        if (ok && (peers & ((1u << lane) - 1u)) == 0u) wcnt[warp][e] += __popc(peers);
        __syncwarp();
    }
    if (my_bad) atomicOr(&bad, 1u);
    __syncthreads();
    if (bad) {
        if (tid == 0) { PlanMeta m{}; m.fault = kFaultPlan; *o.meta = m; }
        return;
    }
    uint32_t c = 0, n = 0;
    if (tid < kExperts) {
        for (int wi = 0; wi < 32; ++wi) { const uint32_t t = wcnt[wi][tid]; wcnt[wi][tid] = c; c += t; }
        n = c ? (c + max_n - 1) / max_n : 0;
        const uint32_t per = n ? (c + n - 1) / n : 0;
        cnt[tid] = c; ntl[tid] = n; width[tid] = (per + 15u) & ~15u;
        atomicMax(&max_count, c);
        // exclusive scans over experts of routes, tiles, FC1 items, FC2 items
        const uint32_t v[4] = {c, n, n * uint32_t(mt_fc1), n * uint32_t(mt_fc2)};
        uint32_t inc[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) { inc[k] = warp_inclusive_scan(v[k], lane); if (lane == 31) wsum[k][warp] = inc[k]; }
        rbase[tid] = inc[0] - v[0]; tstart[tid] = inc[1] - v[1]; i1base[tid] = inc[2] - v[2]; i2base[tid] = inc[3] - v[3];
    }
    const uint32_t active = __syncthreads_count(tid < kExperts && c > 0);
    if (tid < kExperts) {
        uint32_t add[4] = {0, 0, 0, 0};
        for (uint32_t wi = 0; wi < warp; ++wi)
#pragma unroll
            for (int k = 0; k < 4; ++k) add[k] += wsum[k][wi];
        rbase[tid] += add[0]; tstart[tid] += add[1]; i1base[tid] += add[2]; i2base[tid] += add[3];
        if (tid == kExperts - 1) {
            PlanMeta m{};
            m.fault = 0; m.n_tiles = tstart[tid] + n; m.n_items_fc1 = i1base[tid] + n * mt_fc1;
            m.n_items_fc2 = i2base[tid] + n * mt_fc2; m.active_experts = active; m.max_count = max_count;
            *o.meta = m;
        }
    }
    __syncthreads();
    // stable placement: this warp's segment in route order, 32 routes at a time
    for (uint32_t r0 = lo; r0 < hi; r0 += 32) {
        const uint32_t r = r0 + lane;
        const bool in = r < hi;
        int32_t e = in ? ids[r] : -1;
        const bool live = in && (!skip_foreign || slot_serves(sc.slots[e], r / kTopK, sc.own_lo, sc.own_hi));
        if (!live) e = -1 - int32_t(lane);
        const uint32_t peers = __match_any_sync(0xffffffffu, e);
        const uint32_t rank = __popc(peers & ((1u << lane) - 1u));
        uint32_t g = 0;
        if (live) g = rbase[e] + wcnt[warp][e] + rank;
        __syncwarp();
        if (live && rank == 0) wcnt[warp][e] += __popc(peers);
        __syncwarp();
        if (live) {
            o.inverse[r] = int32_t(g);
            o.original_routes[g] = int32_t(r);
            o.grouped_weights[g] = w[r];
        } else if (in) {
            o.inverse[r] = -1;
        }
    }
    // tiles and work items: one warp per expert, lanes over (weight tile pair, token tile)
    for (uint32_t e = warp; e < kExperts; e += 32) {
        const uint32_t ce = cnt[e], ne = ntl[e], wd = width[e];
        if (lane == 0) o.experts[e] = ExpertPlan{int32_t(ce), int32_t(rbase[e]), int32_t(tstart[e]), int32_t(wd)};
        for (uint32_t j = lane; j < ne; j += 32) {
            const uint32_t nv = ce - j * wd < wd ? ce - j * wd : wd;
            o.tiles[tstart[e] + j] = TokenTile{int32_t(slots[e]) & kSlotMask, int32_t(rbase[e] + j * wd), int32_t(nv), int32_t((nv + 15u) & ~15u)};
        }
        for (uint32_t i = lane; i < ne * mt_fc1; i += 32)
            o.items_fc1[i1base[e] + i] = WorkItem{int32_t(tstart[e] + i % ne), int32_t(i / ne) * m_step1};
        for (uint32_t i = lane; i < ne * mt_fc2; i += 32)
            o.items_fc2[i2base[e] + i] = WorkItem{int32_t(tstart[e] + i % ne), int32_t(i / ne) * m_step2};
    }
}

// ---- the same plan in three launches, for requests too large for one CTA ----
// CTA c owns routes [c S, (c+1) S). (1) count per (CTA, expert) and validate;
// (2) one CTA turns the counts into per-(CTA, expert) start offsets, tiles the
// experts and writes tiles / work items / metadata; (3) every CTA places its
// routes: global offset of its (CTA, expert) pair + the per-warp offset inside
// the CTA + the rank inside the 32-route group. Stable by construction.
__device__ __forceinline__ void plan_warp_counts(const int32_t* __restrict__ ids, const float* __restrict__ w,
                                                 const PlanScope& sc, uint32_t lo, uint32_t hi,
                                                 uint32_t lane, uint32_t* __restrict__ wrow, bool validate, uint32_t& bad) {
    const int skip_foreign = sc.skip_foreign;
    for (uint32_t r0 = lo; r0 < hi; r0 += 32) {
        const uint32_t r = r0 + lane;
        const bool live = r < hi;
        int32_t e = -1;
        bool ok = false;
        if (live) {
            e = ids[r];
            ok = true;
            if (validate) {
                const float wt = w[r];
                ok = e >= 0 && e < kExperts && wt >= 0.0f && wt <= 3.402823466e+38f;
                if (ok)
                    for (uint32_t k = (r / kTopK) * kTopK; k < r; ++k) ok = ok && ids[k] != e;
                const bool here = ok && slot_serves(sc.slots[e], r / kTopK, sc.own_lo, sc.own_hi);
                if (skip_foreign ? !ok : !here) bad = 1;
                ok = here;
            } else if (skip_foreign) {
                ok = slot_serves(sc.slots[e], r / kTopK, sc.own_lo, sc.own_hi);      // validated by the counting launch
            }
        }
        const uint32_t peers = __match_any_sync(0xffffffffu, ok ? e : -1 - int32_t(lane));
        if (ok && (peers & ((1u << lane) - 1u)) == 0u) wrow[e] += __popc(peers);
        __syncwarp();
    }
}
__global__ void __launch_bounds__(1024) plan_count_kernel(const int32_t* __restrict__ ids, const float* __restrict__ w,
                                                          uint32_t rows, PlanScope sc,
                                                          uint32_t cta_routes, uint32_t* __restrict__ cta_cnt,
                                                          PlanMeta* __restrict__ meta) {
    __shared__ uint32_t wcnt[32][kExperts];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, routes = rows * kTopK;
    const uint32_t seg = cta_routes / 32u, base = blockIdx.x * cta_routes;
    const uint32_t lo = base + warp * seg < routes ? base + warp * seg : routes;
    const uint32_t hi = lo + seg < routes ? lo + seg : routes;
    for (uint32_t i = tid; i < 32 * kExperts; i += 1024) (&wcnt[0][0])[i] = 0;
    __syncthreads();
    uint32_t bad = 0;
    plan_warp_counts(ids, w, sc, lo, hi, lane, wcnt[warp], true, bad);
    if (bad) atomicOr(&meta->fault, uint32_t(kFaultPlan));
    __syncthreads();
    if (tid < kExperts) {
        uint32_t c = 0;
        for (int wi = 0; wi < 32; ++wi) c += wcnt[wi][tid];
        cta_cnt[blockIdx.x * kExperts + tid] = c;
    }
}
__global__ void __launch_bounds__(1024) plan_scan_kernel(uint32_t n_cta, uint32_t* __restrict__ cta_cnt, int max_n,
                                                         int mt_fc1, int mt_fc2, int m_step1, int m_step2, const int16_t* __restrict__ slots,
                                                         PlanOut o) {
    mt_fc1 /= m_step1;
    mt_fc2 /= m_step2;
    __shared__ uint32_t cnt[kExperts], rbase[kExperts], tstart[kExperts], width[kExperts], ntl[kExperts];
    __shared__ uint32_t i1base[kExperts], i2base[kExperts];
    __shared__ uint32_t wsum[4][8];
    __shared__ uint32_t part_sum[4][kExperts];
    __shared__ uint32_t max_count;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    if (o.meta->fault) {   // uniform: written by the previous launch
        if (tid == 0) { PlanMeta m{}; m.fault = kFaultPlan; *o.meta = m; }
        return;
    }
    if (tid == 0) max_count = 0;
    __syncthreads();
    // per-(CTA, expert) counts -> exclusive offsets over the CTAs: thread (expert, quarter) scans a quarter of the CTAs
    // from registers (all its loads in flight at once), the quarters meet in shared memory
    {
        const uint32_t e = tid & (kExperts - 1u), part = tid >> 8;
        const uint32_t per = (n_cta + 3u) / 4u, k0 = part * per;
        uint32_t v[32];
#pragma unroll
        for (uint32_t i = 0; i < 32; ++i) v[i] = (i < per && k0 + i < n_cta) ? cta_cnt[(k0 + i) * kExperts + e] : 0u;
        uint32_t sum = 0;
#pragma unroll
        for (uint32_t i = 0; i < 32; ++i) sum += v[i];
        part_sum[part][e] = sum;
        __syncthreads();
        uint32_t run = 0;
        for (uint32_t q = 0; q < part; ++q) run += part_sum[q][e];
#pragma unroll
        for (uint32_t i = 0; i < 32; ++i)
            if (i < per && k0 + i < n_cta) { cta_cnt[(k0 + i) * kExperts + e] = run; run += v[i]; }
    }
    uint32_t c = 0, n = 0;
    if (tid < kExperts) {
        c = part_sum[0][tid] + part_sum[1][tid] + part_sum[2][tid] + part_sum[3][tid];
        n = c ? (c + max_n - 1) / max_n : 0;
        const uint32_t per = n ? (c + n - 1) / n : 0;
        cnt[tid] = c; ntl[tid] = n; width[tid] = (per + 15u) & ~15u;
        atomicMax(&max_count, c);
        const uint32_t v[4] = {c, n, n * uint32_t(mt_fc1), n * uint32_t(mt_fc2)};
        uint32_t inc[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) { inc[k] = warp_inclusive_scan(v[k], lane); if (lane == 31) wsum[k][warp] = inc[k]; }
        rbase[tid] = inc[0] - v[0]; tstart[tid] = inc[1] - v[1]; i1base[tid] = inc[2] - v[2]; i2base[tid] = inc[3] - v[3];
    }
    const uint32_t active = __syncthreads_count(tid < kExperts && c > 0);
    if (tid < kExperts) {
        uint32_t add[4] = {0, 0, 0, 0};
        for (uint32_t wi = 0; wi < warp; ++wi)
#pragma unroll
            for (int k = 0; k < 4; ++k) add[k] += wsum[k][wi];
        rbase[tid] += add[0]; tstart[tid] += add[1]; i1base[tid] += add[2]; i2base[tid] += add[3];
        if (tid == kExperts - 1) {
            PlanMeta m{};
            m.fault = 0; m.n_tiles = tstart[tid] + n; m.n_items_fc1 = i1base[tid] + n * mt_fc1;
            m.n_items_fc2 = i2base[tid] + n * mt_fc2; m.active_experts = active; m.max_count = max_count;
            *o.meta = m;
        }
    }
    __syncthreads();
    for (uint32_t e = warp; e < kExperts; e += 32) {
        const uint32_t ce = cnt[e], ne = ntl[e], wd = width[e];
        if (lane == 0) o.experts[e] = ExpertPlan{int32_t(ce), int32_t(rbase[e]), int32_t(tstart[e]), int32_t(wd)};
        for (uint32_t j = lane; j < ne; j += 32) {
            const uint32_t nv = ce - j * wd < wd ? ce - j * wd : wd;
            o.tiles[tstart[e] + j] = TokenTile{int32_t(slots[e]) & kSlotMask, int32_t(rbase[e] + j * wd), int32_t(nv), int32_t((nv + 15u) & ~15u)};
        }
        for (uint32_t i = lane; i < ne * mt_fc1; i += 32)
            o.items_fc1[i1base[e] + i] = WorkItem{int32_t(tstart[e] + i % ne), int32_t(i / ne) * m_step1};
        for (uint32_t i = lane; i < ne * mt_fc2; i += 32)
            o.items_fc2[i2base[e] + i] = WorkItem{int32_t(tstart[e] + i % ne), int32_t(i / ne) * m_step2};
    }
}
__global__ void __launch_bounds__(1024) plan_place_kernel(const int32_t* __restrict__ ids, const float* __restrict__ w,
                                                          uint32_t rows, uint32_t cta_routes,
                                                          const uint32_t* __restrict__ cta_off, PlanOut o, PlanScope sc) {
    const int skip_foreign = sc.skip_foreign;
    __shared__ uint32_t wcnt[32][kExperts];
    if (o.meta->fault) return;
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, routes = rows * kTopK;
    const uint32_t seg = cta_routes / 32u, base = blockIdx.x * cta_routes;
    const uint32_t lo = base + warp * seg < routes ? base + warp * seg : routes;
    const uint32_t hi = lo + seg < routes ? lo + seg : routes;
    for (uint32_t i = tid; i < 32 * kExperts; i += 1024) (&wcnt[0][0])[i] = 0;
    __syncthreads();
    uint32_t bad = 0;
    plan_warp_counts(ids, w, sc, lo, hi, lane, wcnt[warp], false, bad);
    __syncthreads();
    if (tid < kExperts) {   // per-warp exclusive offsets, on top of this CTA's global start for the expert
        uint32_t run = uint32_t(o.experts[tid].rbase) + cta_off[blockIdx.x * kExperts + tid];
        for (int wi = 0; wi < 32; ++wi) { const uint32_t t = wcnt[wi][tid]; wcnt[wi][tid] = run; run += t; }
    }
    __syncthreads();
    for (uint32_t r0 = lo; r0 < hi; r0 += 32) {
        const uint32_t r = r0 + lane;
        const bool in = r < hi;
        int32_t e = in ? ids[r] : -1;
        const bool live = in && (!skip_foreign || slot_serves(sc.slots[e], r / kTopK, sc.own_lo, sc.own_hi));
        if (!live) e = -1 - int32_t(lane);
        const uint32_t peers = __match_any_sync(0xffffffffu, e);
        const uint32_t rank = __popc(peers & ((1u << lane) - 1u));
        uint32_t g = 0;
        if (live) g = wcnt[warp][e] + rank;
        __syncwarp();
        if (live && rank == 0) wcnt[warp][e] += __popc(peers);
        __syncwarp();
        if (live) {
            o.inverse[r] = int32_t(g);
            o.original_routes[g] = int32_t(r);
            o.grouped_weights[g] = w[r];
        } else if (in) {
            o.inverse[r] = -1;
        }
    }
}

// ---------------------------------------------------------------- permutation
// Grouped row p <- token row original_routes[p] / 8: 4096 E4M3 bytes (one
// 16-byte vector per thread) and 128 scale bytes scattered into the token
// tile's scale blocks. Also the input gate of the path: a scale byte outside
// 105..247 or a NaN payload code raises kFaultInputScale, as the reference's
// activation view poisons them (kernels/b1/grouped.cu:28,36).
//
// With expert parallelism the request's token rows live on several GPUs (TokenSources): token t is row t - lo[k] of
// owner k, read through the peer mapping and around L1 (another GPU wrote it). `routes` is then read from the plan
// (only the routes to this GPU's experts are grouped).
struct TokenSources {
    uint32_t n;                 // 0: one local array
    uint32_t token_base;        // request-wide index of the pass's first token
    uint32_t lo[9];
    const uint8_t* xq[8];
    const uint8_t* xs[8];
};
__global__ void __launch_bounds__(256) permute_kernel(const uint8_t* __restrict__ xq, const uint8_t* __restrict__ xs,
                                                      const int32_t* __restrict__ ids,
                                                      const int32_t* __restrict__ original_routes,
                                                      const ExpertPlan* __restrict__ experts,
                                                      const PlanMeta* __restrict__ meta, uint32_t routes,
                                                      uint8_t* __restrict__ x_perm, uint8_t* __restrict__ sfb,
                                                      uint32_t* __restrict__ fault, TokenSources src) {
    if (meta->fault) return;   // a rejected plan leaves no valid route tables
    uint32_t bad = 0;
    if (src.n) {
        const ExpertPlan last = experts[kExperts - 1];
        routes = uint32_t(last.rbase + last.count);
    }
    for (uint32_t p = blockIdx.x; p < routes; p += gridDim.x) {
        const int32_t route = original_routes[p];
        uint32_t token = uint32_t(route) / kTopK;
        if (src.n) {
            token += src.token_base;
            uint32_t k = 0;
#pragma unroll
            for (uint32_t i = 1; i < 8; ++i)
                if (i < src.n && token >= src.lo[i]) k = i;
            token -= src.lo[k];
            xq = src.xq[k]; xs = src.xs[k];
        }
        const uint4 v = __ldcv(reinterpret_cast<const uint4*>(xq + size_t(token) * kHidden) + threadIdx.x);
        const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if ((((wv[i] & 0x7f7f7f7fu) + 0x01010101u) & 0x80808080u) != 0u) bad = kFaultInputScale;
        reinterpret_cast<uint4*>(x_perm + size_t(p) * kHidden)[threadIdx.x] = v;
        if (threadIdx.x < kHidden / kBlockK) {
            const ExpertPlan ep = experts[ids[route]];
            const uint32_t local = p - uint32_t(ep.rbase);
            const uint32_t tile = uint32_t(ep.tile_start) + local / uint32_t(ep.width), lr = local % uint32_t(ep.width);
            const uint8_t sb = __ldcv(xs + size_t(token) * (kHidden / kBlockK) + threadIdx.x);
            if (sb < 105 || sb > 247) bad = kFaultInputScale;
            const uint32_t chunk = threadIdx.x >> 2, kb = threadIdx.x & 3u;
            sfb[(size_t(tile) * (kHidden / kChunkK) + chunk) * kScaleBlockBytes + scale_block_offset(int(lr), int(kb))] = sb;
        }
    }
    if (bad) atomicOr(fault, bad);
}

// Quantiser and permutation in one pass, for requests that arrive as BF16 / FP32 rows and are too large for the fused
// small prologue: one CTA per token row quantises it once in registers (thread t holds elements 16 t .. 16 t + 15), writes
// the quantised row and its scales in request order (what the stage dumps and the parity tests read), and copies both into
// the row's eight places of the expert-sorted operand (x_perm rows, token-tile scale blocks). Against the two separate
// passes this saves one write and one read of the quantised rows and one launch. The input gate of the permutation
// applies to what the quantiser produced: a zero block under the wire codec (scale byte 0) raises kFaultInputScale.
template <int CODEC, typename IN>
__global__ void __launch_bounds__(256) quantize_permute_kernel(const IN* __restrict__ x, uint32_t rows, const int32_t* __restrict__ ids,
                                                               const int32_t* __restrict__ inverse,
                                                               const ExpertPlan* __restrict__ experts,
                                                               const PlanMeta* __restrict__ meta, uint8_t* __restrict__ xq,
                                                               uint8_t* __restrict__ xs, uint8_t* __restrict__ x_perm,
                                                               uint8_t* __restrict__ sfb, uint32_t* __restrict__ fault_quant,
                                                               uint32_t* __restrict__ fault_input) {
    __shared__ uint32_t dst_row[kTopK], dst_tile[kTopK], dst_lr[kTopK];
    const bool planned = meta->fault == 0;     // a rejected plan leaves no valid route tables: quantise only
    uint32_t bad_q = 0, bad_in = 0;
    for (uint32_t token = blockIdx.x; token < rows; token += gridDim.x) {
        if (planned && threadIdx.x < uint32_t(kTopK)) {
            const uint32_t route = token * kTopK + threadIdx.x;
            const uint32_t p = uint32_t(inverse[route]);
            const ExpertPlan ep = experts[ids[route]];
            const uint32_t local = p - uint32_t(ep.rbase);
            dst_row[threadIdx.x] = p;
            dst_tile[threadIdx.x] = uint32_t(ep.tile_start) + local / uint32_t(ep.width);
            dst_lr[threadIdx.x] = local % uint32_t(ep.width);
        }
        uint4 out;
        uint32_t sbyte;
        const uint64_t g = uint64_t(token) * (kHidden / 16) + threadIdx.x;
        const bool write = quant16<CODEC, IN>(x, g, true, out, sbyte, bad_q);
        __syncthreads();
        if (write) {
            const uint32_t wv[4] = {out.x, out.y, out.z, out.w};
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if ((((wv[i] & 0x7f7f7f7fu) + 0x01010101u) & 0x80808080u) != 0u) bad_in = kFaultInputScale;
            if (sbyte < 105 || sbyte > 247) bad_in = kFaultInputScale;
            reinterpret_cast<uint4*>(xq)[g] = out;
            const uint32_t blk = threadIdx.x >> 1;                  // K32 block of the row; the even thread stores its scale
            if ((threadIdx.x & 1u) == 0) xs[size_t(token) * (kHidden / kBlockK) + blk] = uint8_t(sbyte);
            if (planned) {
#pragma unroll
                for (int j = 0; j < kTopK; ++j) {
                    reinterpret_cast<uint4*>(x_perm + size_t(dst_row[j]) * kHidden)[threadIdx.x] = out;
                    if ((threadIdx.x & 1u) == 0)
                        sfb[(size_t(dst_tile[j]) * (kHidden / kChunkK) + (blk >> 2)) * kScaleBlockBytes +
                            scale_block_offset(int(dst_lr[j]), int(blk & 3u))] = uint8_t(sbyte);
                }
            }
        }
        __syncthreads();
    }
    if (bad_q) atomicOr(fault_quant, bad_q);
    if (bad_in) atomicOr(fault_input, bad_in);
}

// ---------------------------------------------------------------- combine
// Per (token, column): v = 0; v = add(v, mul(w_j, y_j)) for slot j = 0..7 with
// separate round-to-nearest multiply and add, then BF16 round-to-nearest-even
// (crates/mimo26-expert/kernels/b1/route_reduce.cu:61-74). Any nonfinite
// weight, value or partial sum, or a BF16 overflow, raises kFaultReduce.
__global__ void __launch_bounds__(256) route_reduce_kernel(const float* __restrict__ y, const float* __restrict__ w,
                                                           uint32_t rows, float* __restrict__ partial,
                                                           uint16_t* __restrict__ bf16, uint32_t* __restrict__ fault) {
    const float kMax = 3.402823466e+38f;
    const uint64_t n4 = uint64_t(rows) * (kHidden / 4);
    bool failed = false;
    grid_dep_wait();             // y comes from the FC2 kernel
    for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n4; i += uint64_t(gridDim.x) * blockDim.x) {
        const uint64_t row = i / (kHidden / 4), c4 = i % (kHidden / 4);
        float4 z[kTopK];
#pragma unroll
        for (int j = 0; j < kTopK; ++j) z[j] = reinterpret_cast<const float4*>(y)[(row * kTopK + j) * (kHidden / 4) + c4];
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        bool ok = true;
#pragma unroll
        for (int j = 0; j < kTopK; ++j) {
            const float wt = w[row * kTopK + j];
            ok = ok && wt >= 0.0f && wt <= kMax;
            const float zz[4] = {z[j].x, z[j].y, z[j].z, z[j].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                ok = ok && zz[k] >= -kMax && zz[k] <= kMax;
                v[k] = __fadd_rn(v[k], __fmul_rn(wt, zz[k]));
                ok = ok && v[k] >= -kMax && v[k] <= kMax;
            }
        }
        uint32_t code[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) { code[k] = bf16_rne_bits(v[k]); ok = ok && (code[k] & 0x7f80u) != 0x7f80u; }
        if (!ok) {
            failed = true;
            code[0] = code[1] = code[2] = code[3] = 0;
            v[0] = v[1] = v[2] = v[3] = __int_as_float(0x7fc00000);
        }
        if (partial) reinterpret_cast<float4*>(partial)[i] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<uint2*>(bf16)[i] = make_uint2(code[0] | (code[1] << 16), code[2] | (code[3] << 16));
    }
    if (__syncthreads_or(failed) && threadIdx.x == 0) atomicOr(fault, uint32_t(kFaultReduce));
}

// The same combine over BF16 route outputs (the route-output option; the reference's opt-in reduce_bf16y,
// crates/mimo26-spark/kernels/b1_serve.cu:98-143): each y is a BF16 value widened exactly to FP32, then the same
// ordered multiply / add, fault rules and BF16 rounding. Eight columns per thread (16-byte loads).
__global__ void __launch_bounds__(256) route_reduce_y16_kernel(const uint16_t* __restrict__ y, const float* __restrict__ w,
                                                               uint32_t rows, float* __restrict__ partial,
                                                               uint16_t* __restrict__ bf16, uint32_t* __restrict__ fault) {
    const float kMax = 3.402823466e+38f;
    const uint64_t n8 = uint64_t(rows) * (kHidden / 8);
    bool failed = false;
    grid_dep_wait();             // y comes from the FC2 kernel
    for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += uint64_t(gridDim.x) * blockDim.x) {
        const uint64_t row = i / (kHidden / 8), c8 = i % (kHidden / 8);
        uint4 z[kTopK];
#pragma unroll
        for (int j = 0; j < kTopK; ++j) z[j] = reinterpret_cast<const uint4*>(y)[(row * kTopK + j) * (kHidden / 8) + c8];
        float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        bool ok = true;
#pragma unroll
        for (int j = 0; j < kTopK; ++j) {
            const float wt = w[row * kTopK + j];
            ok = ok && wt >= 0.0f && wt <= kMax;
            const uint32_t words[4] = {z[j].x, z[j].y, z[j].z, z[j].w};
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float zv = __uint_as_float((k & 1) ? (words[k / 2] & 0xffff0000u) : (words[k / 2] << 16));
                ok = ok && zv >= -kMax && zv <= kMax;
                v[k] = __fadd_rn(v[k], __fmul_rn(wt, zv));
                ok = ok && v[k] >= -kMax && v[k] <= kMax;
            }
        }
        uint32_t code[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) { code[k] = bf16_rne_bits(v[k]); ok = ok && (code[k] & 0x7f80u) != 0x7f80u; }
        if (!ok) {
            failed = true;
#pragma unroll
            for (int k = 0; k < 8; ++k) { code[k] = 0; v[k] = __int_as_float(0x7fc00000); }
        }
        if (partial) {
            reinterpret_cast<float4*>(partial)[2 * i] = make_float4(v[0], v[1], v[2], v[3]);
            reinterpret_cast<float4*>(partial)[2 * i + 1] = make_float4(v[4], v[5], v[6], v[7]);
        }
        reinterpret_cast<uint4*>(bf16)[i] = make_uint4(code[0] | (code[1] << 16), code[2] | (code[3] << 16),
                                                       code[4] | (code[5] << 16), code[6] | (code[7] << 16));
    }
    if (__syncthreads_or(failed) && threadIdx.x == 0) atomicOr(fault, uint32_t(kFaultReduce));
}

// Cross-rank sum: s = 0; s = add(s, f32(bf16_r)) for r = 0..G-1 in rank order
// (crates/mimo26-coordinator/kernels/glue.cu:202-213, crates/mimo26-wire/src/l4.rs:169-244).
struct RankPlanes {
    const uint16_t* p[8];
};
// `residual` (may alias `out`): out = residual + s, the coordinator's next step (h += f,
// crates/mimo26-coordinator/kernels/glue.cu:55-59, src/dforward.rs:2294-2297) folded into the same pass.
__global__ void __launch_bounds__(256) rank_sum_kernel(RankPlanes planes, int n_ranks, uint64_t n, float* out,
                                                       const float* residual) {
    const uint64_t n8 = n / 8;
    for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += uint64_t(gridDim.x) * blockDim.x) {
        float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < n_ranks; ++r) {
            const uint4 v = reinterpret_cast<const uint4*>(planes.p[r])[i];
            const uint32_t wv[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                s[2 * k] = __fadd_rn(s[2 * k], __uint_as_float(wv[k] << 16));
                s[2 * k + 1] = __fadd_rn(s[2 * k + 1], __uint_as_float(wv[k] & 0xffff0000u));
            }
        }
        if (residual) {
            const float4 a = reinterpret_cast<const float4*>(residual)[2 * i], b = reinterpret_cast<const float4*>(residual)[2 * i + 1];
            s[0] = __fadd_rn(a.x, s[0]); s[1] = __fadd_rn(a.y, s[1]); s[2] = __fadd_rn(a.z, s[2]); s[3] = __fadd_rn(a.w, s[3]);
            s[4] = __fadd_rn(b.x, s[4]); s[5] = __fadd_rn(b.y, s[5]); s[6] = __fadd_rn(b.z, s[6]); s[7] = __fadd_rn(b.w, s[7]);
        }
        reinterpret_cast<float4*>(out)[2 * i] = make_float4(s[0], s[1], s[2], s[3]);
        reinterpret_cast<float4*>(out)[2 * i + 1] = make_float4(s[4], s[5], s[6], s[7]);
    }
    for (uint64_t i = n8 * 8 + uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += uint64_t(gridDim.x) * blockDim.x) {
        float s = 0.f;
        for (int r = 0; r < n_ranks; ++r) s = __fadd_rn(s, __uint_as_float(uint32_t(planes.p[r][i]) << 16));
        out[i] = residual ? __fadd_rn(residual[i], s) : s;
    }
}

// ---------------------------------------------------------------- plane exchange between GPUs
// The same rank-ordered sum, with the planes left where each rank's combine wrote them: every GPU reads its
// peers' planes through NVLink peer mappings while it adds, instead of gathering copies first.
//
// Each rank owns a window: flags[8] (flags[r] = the last step rank r has published), an error word, and two plane
// slots used alternately. One launch per rank and step:
//   1. CTA 0 publishes the step to every peer (a system-scope release store into the peer's flags[rank]; the
//      plane itself was finished by the previous kernel in the stream);
//   2. every CTA waits until every peer has published this step (system-scope acquire loads of its own flags);
//      the wait is bounded: past the limit the kernel records the peer in the error word and returns;
//   3. grid-stride sum over the planes in rank order; peer planes are read around L1, which is not coherent
//      with another GPU's writes.
// A slot is rewritten two steps later, after this rank has seen every peer publish the step in between, which a
// peer only does once its own reads of the earlier step have finished: two slots are enough.
struct ExchangeWindow {
    uint32_t flags[8];
    uint32_t error;            // bit r: gave up waiting for rank r
    uint32_t pad[55];          // planes start 256 bytes in
};
static_assert(sizeof(ExchangeWindow) == 256, "exchange window header is 256 bytes");
struct ExchangePeers {
    uint8_t* window[8];        // window[rank] is the local one
};
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__global__ void __launch_bounds__(256) exchange_sum_kernel(ExchangePeers peers, int rank, int world, uint32_t step,
                                                           uint64_t plane_offset, uint64_t n, long long wait_cycles,
                                                           float* out, const float* residual) {
    __shared__ uint32_t late;
    ExchangeWindow* mine = reinterpret_cast<ExchangeWindow*>(peers.window[rank]);
    grid_dep_wait();             // the local plane comes from the combine kernel before this one
    if (blockIdx.x == 0 && threadIdx.x < uint32_t(world) && int(threadIdx.x) != rank) {
        __threadfence_system();
        st_release_sys(&reinterpret_cast<ExchangeWindow*>(peers.window[threadIdx.x])->flags[rank], step);
    }
    if (threadIdx.x == 0) late = 0;
    __syncthreads();
    if (threadIdx.x < uint32_t(world) && int(threadIdx.x) != rank) {
        const long long t0 = clock64();
        while (int32_t(ld_acquire_sys(&mine->flags[threadIdx.x]) - step) < 0) {
            if (clock64() - t0 > wait_cycles) { atomicOr(&late, 1u << threadIdx.x); break; }
        }
    }
    __syncthreads();
    if (late) {
        if (threadIdx.x == 0) atomicOr(&mine->error, late);
        return;
    }
    const uint64_t n8 = n / 8;
    for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n8; i += uint64_t(gridDim.x) * blockDim.x) {
        float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        uint4 v[8];
#pragma unroll
        for (int r = 0; r < 8; ++r)
            if (r < world) v[r] = __ldcv(reinterpret_cast<const uint4*>(peers.window[r] + plane_offset) + i);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r >= world) break;
            const uint32_t wv[4] = {v[r].x, v[r].y, v[r].z, v[r].w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                s[2 * k] = __fadd_rn(s[2 * k], __uint_as_float(wv[k] << 16));
                s[2 * k + 1] = __fadd_rn(s[2 * k + 1], __uint_as_float(wv[k] & 0xffff0000u));
            }
        }
        if (residual) {      // h += f of the coordinator, in the same pass (may alias out)
            const float4 a = reinterpret_cast<const float4*>(residual)[2 * i], b = reinterpret_cast<const float4*>(residual)[2 * i + 1];
            s[0] = __fadd_rn(a.x, s[0]); s[1] = __fadd_rn(a.y, s[1]); s[2] = __fadd_rn(a.z, s[2]); s[3] = __fadd_rn(a.w, s[3]);
            s[4] = __fadd_rn(b.x, s[4]); s[5] = __fadd_rn(b.y, s[5]); s[6] = __fadd_rn(b.z, s[6]); s[7] = __fadd_rn(b.w, s[7]);
        }
        reinterpret_cast<float4*>(out)[2 * i] = make_float4(s[0], s[1], s[2], s[3]);
        reinterpret_cast<float4*>(out)[2 * i + 1] = make_float4(s[4], s[5], s[6], s[7]);
    }
}

// ---------------------------------------------------------------- combine + exchange in one kernel (push form)
// For decode-sized steps of a tensor-parallel rank the two kernels above (combine into the rank's own plane; exchange
// kernel that publishes, waits and reads the peers' planes over NVLink) become one. Every thread computes the ordered top-8
// combine of four columns, and stores the four BF16 codes TOGETHER WITH THE STEP NUMBER into every rank's window (its own
// and, with plain peer stores, the peers'): one 16-byte store {codes 0-1, step, codes 2-3, step}. NVLink delivers each
// 8-byte half whole, so a half whose flag word equals the step carries that step's data: no fence, no separate flag and no
// acknowledged round trip stand between a rank's store and a peer's use of it. Once its chunks are out, the CTA polls the
// same 16 bytes of every source's plane in its OWN window until both flags show the step (bounded; error word, status
// code 5) and adds the G planes in rank order from local memory. Pushes never wait for anything, so no rank can block
// another before it has delivered.
//
// Window area of the push form (behind the pull form's two plane slots): receive planes [2 slots][G sources][cap bytes],
// 4 bytes per plane element. A slot is rewritten two steps later, which a peer can only reach after this rank has pushed
// the step in between, which it does after it has finished reading. Flags are step numbers, so nothing is ever cleared.
constexpr uint32_t kPushRows = 512;        // largest step (tokens) the fused form serves: 8 MB per receive plane
struct PushLayout {
    uint64_t recv_off, cap;                // byte offset inside a window; bytes per receive plane
};
__device__ __forceinline__ uint4* push_plane(uint8_t* window, const PushLayout& lay, uint32_t slot, uint32_t world, uint32_t src) {
    return reinterpret_cast<uint4*>(window + lay.recv_off + (size_t(slot) * world + src) * lay.cap);
}
__device__ __forceinline__ void st_volatile_v4(uint4* p, uint4 v) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
// Host-side stand-in for a peer (single-process tests, an idle rank): marks every element of `plane` as delivered for
// `step`, leaving the data words as they are.
__global__ void push_mark_kernel(uint4* plane, uint32_t step, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        uint32_t* f = reinterpret_cast<uint32_t*>(plane + i);
        f[1] = step; f[3] = step;
    }
}
template <bool Y16>
__global__ void __launch_bounds__(256) reduce_exchange_kernel(const void* __restrict__ y_in, const float* __restrict__ w, uint32_t rows,
                                                              ExchangePeers peers, PushLayout lay, int rank, int world, uint32_t step,
                                                              long long wait_cycles, float* __restrict__ out,
                                                              const float* residual, uint32_t* __restrict__ fault) {
    const float kMax = 3.402823466e+38f;
    const uint32_t slot = step & 1u, tid = threadIdx.x;
    const uint64_t n4 = uint64_t(rows) * (kHidden / 4);                 // groups of four columns, one per thread and chunk
    const uint32_t chunks = uint32_t((n4 + 255) / 256);
    ExchangeWindow* mine = reinterpret_cast<ExchangeWindow*>(peers.window[rank]);
    bool failed = false;
    grid_dep_wait();             // y comes from the FC2 kernel
    // ---- phase 1: combine and push
    for (uint32_t c = blockIdx.x; c < chunks; c += gridDim.x) {
        const uint64_t i = uint64_t(c) * 256 + tid;
        if (i >= n4) break;
        const uint64_t row = i / (kHidden / 4), c4 = i % (kHidden / 4);
        float v[4] = {0.f, 0.f, 0.f, 0.f};
        bool ok = true;
        float z[kTopK][4];
#pragma unroll
        for (int j = 0; j < kTopK; ++j) {
            if constexpr (Y16) {
                const uint2 q = reinterpret_cast<const uint2*>(y_in)[(row * kTopK + j) * (kHidden / 4) + c4];
                z[j][0] = __uint_as_float(q.x << 16); z[j][1] = __uint_as_float(q.x & 0xffff0000u);
                z[j][2] = __uint_as_float(q.y << 16); z[j][3] = __uint_as_float(q.y & 0xffff0000u);
            } else {
                const float4 q = reinterpret_cast<const float4*>(y_in)[(row * kTopK + j) * (kHidden / 4) + c4];
                z[j][0] = q.x; z[j][1] = q.y; z[j][2] = q.z; z[j][3] = q.w;
            }
        }
#pragma unroll
        for (int j = 0; j < kTopK; ++j) {
            const float wt = w[row * kTopK + j];
            ok = ok && wt >= 0.0f && wt <= kMax;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                ok = ok && z[j][k] >= -kMax && z[j][k] <= kMax;
                v[k] = __fadd_rn(v[k], __fmul_rn(wt, z[j][k]));
                ok = ok && v[k] >= -kMax && v[k] <= kMax;
            }
        }
        uint32_t code[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) { code[k] = bf16_rne_bits(v[k]); ok = ok && (code[k] & 0x7f80u) != 0x7f80u; }
        if (!ok) { failed = true; code[0] = code[1] = code[2] = code[3] = 0; }
        const uint4 word = make_uint4(code[0] | (code[1] << 16), step, code[2] | (code[3] << 16), step);
#pragma unroll
        for (int r = 0; r < 8; ++r)
            if (r < world) st_volatile_v4(push_plane(peers.window[r], lay, slot, uint32_t(world), uint32_t(rank)) + i, word);
    }
    // ---- phase 2: every source's words of this rank's window, as they arrive; add in rank order
    uint32_t late = 0;
    for (uint32_t c = blockIdx.x; c < chunks && !late; c += gridDim.x) {
        const uint64_t i = uint64_t(c) * 256 + tid;
        if (i >= n4) break;
        uint4 q[8];
        uint32_t pending = (1u << world) - 1u;
        const long long t0 = clock64();
        while (pending) {
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                if (r < world && (pending >> r & 1u)) {
                    q[r] = ld_volatile_v4(push_plane(peers.window[rank], lay, slot, uint32_t(world), uint32_t(r)) + i);
                    if (q[r].y == step && q[r].w == step) pending &= ~(1u << r);
                }
            }
            if (pending && clock64() - t0 > wait_cycles) { late = pending; break; }
        }
        if (late) break;
        float s4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r >= world) break;
            s4[0] = __fadd_rn(s4[0], __uint_as_float(q[r].x << 16));
            s4[1] = __fadd_rn(s4[1], __uint_as_float(q[r].x & 0xffff0000u));
            s4[2] = __fadd_rn(s4[2], __uint_as_float(q[r].z << 16));
            s4[3] = __fadd_rn(s4[3], __uint_as_float(q[r].z & 0xffff0000u));
        }
        if (residual) {
            const float4 a = reinterpret_cast<const float4*>(residual)[i];
            s4[0] = __fadd_rn(a.x, s4[0]); s4[1] = __fadd_rn(a.y, s4[1]); s4[2] = __fadd_rn(a.z, s4[2]); s4[3] = __fadd_rn(a.w, s4[3]);
        }
        reinterpret_cast<float4*>(out)[i] = make_float4(s4[0], s4[1], s4[2], s4[3]);
    }
    if (late) atomicOr(&mine->error, late);
    if (__syncthreads_or(failed) && tid == 0) atomicOr(fault, uint32_t(kFaultReduce));
}

// ---------------------------------------------------------------- weight repack
// Source of one projection: payload u8 [E][rows][in/2] and scales u8
// [E][rows][in/32] with explicit strides, so the same kernels read the
// checkpoint tensors (crates/mimo26-expert/src/mxfp4.rs:13-19) and a per-rank
// canonical slice image (crates/mimo26-repack/src/geom.rs:36-50).
struct ProjSrc {
    const uint8_t* payload;
    const uint8_t* scales;
    uint64_t expert_stride_p, expert_stride_s;   // bytes between experts
    uint64_t row_stride_p, row_stride_s;         // bytes between rows
    uint64_t row0;                               // first row of this rank's slice
    uint64_t col0_p, col0_s;                     // first payload / scale byte of this rank's K slice
};

// w13[e][j][r][*]: r < 128 -> gate row 128 j + r, else up row 128 j + r - 128. 16 bytes per thread.
__global__ void __launch_bounds__(256) prep_w13_kernel(ProjSrc gate, ProjSrc up, int i_local, uint8_t* __restrict__ dst, int n_experts) {
    const uint64_t vec_per_row = kHidden / 2 / 16, tiles = uint64_t(i_local) / kTileM;
    const uint64_t total = uint64_t(n_experts) * tiles * kPairM * vec_per_row;
    for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += uint64_t(gridDim.x) * blockDim.x) {
        const uint64_t v = i % vec_per_row, row = i / vec_per_row;
        const uint64_t r = row % kPairM, j = (row / kPairM) % tiles, e = row / kPairM / tiles;
        const ProjSrc& s = r < kTileM ? gate : up;
        const uint64_t srow = s.row0 + j * kTileM + (r % kTileM);
        reinterpret_cast<uint4*>(dst)[i] =
            *reinterpret_cast<const uint4*>(s.payload + e * s.expert_stride_p + srow * s.row_stride_p + s.col0_p + v * 16);
    }
}
// s13[e][j][c][b][512], b = 0 gate / 1 up. One byte per thread; byte 255 (reserved) is stored as 254:
// the checkpoint contract clamps it to 2^127 (crates/mimo26-expert/src/mxfp4.rs:24-29).
__global__ void __launch_bounds__(256) prep_s13_kernel(ProjSrc gate, ProjSrc up, int i_local, uint8_t* __restrict__ dst,
                                                       uint32_t* __restrict__ abnormal, int n_experts) {
    const uint64_t chunks = kHidden / kChunkK, tiles = uint64_t(i_local) / kTileM;
    const uint64_t total = uint64_t(n_experts) * tiles * chunks * 2 * kScaleBlockBytes;
    uint32_t odd = 0;
    for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += uint64_t(gridDim.x) * blockDim.x) {
        const uint32_t o = uint32_t(i % kScaleBlockBytes);
        const uint64_t b = (i / kScaleBlockBytes) % 2, c = (i / kScaleBlockBytes / 2) % chunks;
        const uint64_t j = (i / kScaleBlockBytes / 2 / chunks) % tiles, e = i / kScaleBlockBytes / 2 / chunks / tiles;
        const uint32_t r = (o >> 4) + 32u * ((o >> 2) & 3u), kb = o & 3u;
        const ProjSrc& s = b == 0 ? gate : up;
        const uint64_t srow = s.row0 + j * kTileM + r;
        uint8_t v = s.scales[e * s.expert_stride_s + srow * s.row_stride_s + s.col0_s + c * 4 + kb];
        if (v < 2 || v > 252) odd = 1;
        dst[i] = v == 255 ? 254 : v;
    }
    if (odd) atomicOr(abnormal, 1u);
}
// s13h[e][j][h][c][512]: the scale block of half item h of tile pair j = rows 0..63 the gate rows 64 h .., rows 64..127 the
// up rows 64 h .. of the same features: per 16-byte lane row, 8 bytes of the gate block and 8 of the up block of s13.
__global__ void __launch_bounds__(256) prep_s13_half_kernel(const uint8_t* __restrict__ s13, int i_local, uint8_t* __restrict__ dst, int n_experts) {
    const uint64_t chunks = kHidden / kChunkK, tiles = uint64_t(i_local) / kTileM;
    const uint64_t total = uint64_t(n_experts) * tiles * 2 * chunks * kScaleBlockBytes;
    for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += uint64_t(gridDim.x) * blockDim.x) {
        const uint32_t o = uint32_t(i % kScaleBlockBytes);
        const uint64_t c = (i / kScaleBlockBytes) % chunks, h = (i / kScaleBlockBytes / chunks) % 2;
        const uint64_t ej = i / kScaleBlockBytes / chunks / 2;                  // e * tiles + j
        const uint32_t lane = o >> 4, grp = (o >> 2) & 3u, kb = o & 3u;
        const uint64_t b = grp >> 1;                                           // 0: gate block, 1: up block
        const uint32_t src_grp = uint32_t(h) * 2u + (grp & 1u);
        dst[i] = s13[((ej * chunks + c) * 2 + b) * kScaleBlockBytes + lane * 16 + src_grp * 4 + kb];
    }
}
// w2[e][h][i_local/2]: this rank's K slice of every down_proj row.
__global__ void __launch_bounds__(256) prep_w2_kernel(ProjSrc down, int i_local, uint8_t* __restrict__ dst, int n_experts) {
    const uint64_t vec_per_row = uint64_t(i_local) / 2 / 16;
    const uint64_t total = uint64_t(n_experts) * kHidden * vec_per_row;
    for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += uint64_t(gridDim.x) * blockDim.x) {
        const uint64_t v = i % vec_per_row, h = (i / vec_per_row) % kHidden, e = i / vec_per_row / kHidden;
        reinterpret_cast<uint4*>(dst)[i] = *reinterpret_cast<const uint4*>(
            down.payload + e * down.expert_stride_p + (down.row0 + h) * down.row_stride_p + down.col0_p + v * 16);
    }
}
// s2[e][h/256][c][b][512]: block b covers rows 256 t + 128 b + r.
__global__ void __launch_bounds__(256) prep_s2_kernel(ProjSrc down, int i_local, uint8_t* __restrict__ dst,
                                                      uint32_t* __restrict__ abnormal, int n_experts) {
    const uint64_t chunks = uint64_t(i_local) / kChunkK, mts = kHidden / kPairM;
    const uint64_t total = uint64_t(n_experts) * mts * chunks * 2 * kScaleBlockBytes;
    uint32_t odd = 0;
    for (uint64_t i = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += uint64_t(gridDim.x) * blockDim.x) {
        const uint32_t o = uint32_t(i % kScaleBlockBytes);
        const uint64_t b = (i / kScaleBlockBytes) % 2, c = (i / kScaleBlockBytes / 2) % chunks;
        const uint64_t mt = (i / kScaleBlockBytes / 2 / chunks) % mts, e = i / kScaleBlockBytes / 2 / chunks / mts;
        const uint32_t r = (o >> 4) + 32u * ((o >> 2) & 3u), kb = o & 3u;
        uint8_t v = down.scales[e * down.expert_stride_s + (down.row0 + mt * kPairM + b * kTileM + r) * down.row_stride_s +
                                down.col0_s + c * 4 + kb];
        if (v < 2 || v > 252) odd = 1;
        dst[i] = v == 255 ? 254 : v;
    }
    if (odd) atomicOr(abnormal, 1u);
}

}  // namespace m26b
