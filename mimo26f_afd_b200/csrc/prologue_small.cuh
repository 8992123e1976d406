// Everything in front of the first GEMM in one launch, for requests of at most 128 tokens (decode, verify rounds).
//
// The separate quantiser, route planner and permutation are each a few microseconds of launch latency around
// almost no work at this size, so here every CTA recomputes the whole route plan in shared memory (one thread per
// route: 256 threads for up to 32 tokens, 1024 for up to 128) and then produces its share of the grouped rows straight
// from the caller's activations, one row per 256 threads:
// quantise (or take the caller's E4M3 bytes), gate, and write the row and its scale bytes where the FC1 kernel's
// loads expect them. The plan tables themselves are written by CTAs 0..3, one table group each.
//
// The plan is the one plan_kernel makes (same validation, same stable expert-major order, same tiles and work
// items); the quantised bytes are the ones quantize_rows_kernel makes; the gate is permute_kernel's.
#pragma once
#include "ffn_kernels.cuh"

namespace m26b {

constexpr uint32_t kSmallRows = 32;      // one thread per route with 256 threads
constexpr uint32_t kMediumRows = 128;    // ... with 1024 threads

struct SmallIo {
    const void* x;           // IN 0: BF16 [rows][4096]; IN 1: FP32; IN 2: E4M3 payload
    const uint8_t* xs_in;    // IN 2: UE8M0 scales [rows][128]
    uint8_t* xq_out;         // IN 0/1: the quantised rows in token order (stage buffer for inspection), or null
    uint8_t* xs_out;
    uint8_t* x_perm;         // grouped rows
    uint8_t* sfb;            // their scale blocks
    uint32_t* fault_input;   // the input gate (scale byte outside 105..247, NaN code)
    uint32_t* fault_quant;   // IN 0/1 with quant_v1: nonfinite / overflow
};

template <int CODEC, int IN, int THREADS>
__global__ void __launch_bounds__(THREADS) small_prologue_kernel(SmallIo io, const int32_t* __restrict__ ids,
                                                             const float* __restrict__ w, uint32_t rows,
                                                             const int16_t* __restrict__ slots, int max_n, int mt_fc1,
                                                             int mt_fc2, int m_step2, PlanOut o) {
    mt_fc2 /= m_step2;      // an FC2 work item covers m_step2 consecutive weight tile pairs
    constexpr int kWarps = THREADS / 32;
    constexpr uint32_t kRowsAtOnce = THREADS / 256;      // grouped rows a CTA produces side by side
    __shared__ uint32_t wcnt[kWarps][kExperts];
    __shared__ uint32_t cnt[kExperts], rbase[kExperts], tstart[kExperts], width[kExperts], ntl[kExperts];
    __shared__ uint32_t i1base[kExperts], i2base[kExperts];
    __shared__ uint32_t wsum[4][8];
    __shared__ uint32_t max_count;
    __shared__ uint16_t row_tile[THREADS];
    __shared__ uint8_t row_token[THREADS], row_lr[THREADS], row_first[THREADS];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5, routes = rows * kTopK;
    grid_dep_launch();           // the FC1 kernel may set itself up meanwhile; it waits for this grid before it reads
    for (uint32_t i = tid; i < kWarps * kExperts; i += THREADS) (&wcnt[0][0])[i] = 0;
    if (tid == 0) max_count = 0;
    // ---- validate (the rules of plan_kernel) and count per (warp, expert)
    const bool live = tid < routes;
    int32_t e = -1;
    float wt = 0.f;
    bool ok = true;
    if (live) {
        e = ids[tid];
        wt = w[tid];
        ok = e >= 0 && e < kExperts && wt >= 0.0f && wt <= 3.402823466e+38f;
        ok = ok && slots[e] >= 0;
        if (ok)
            for (uint32_t k = (tid / kTopK) * kTopK; k < tid; ++k) ok = ok && ids[k] != e;
    }
    if (__syncthreads_or(!ok)) {
        if (blockIdx.x == 0 && tid == 0) { PlanMeta m{}; m.fault = kFaultPlan; *o.meta = m; }
        return;
    }
    const uint32_t peers = __match_any_sync(0xffffffffu, live ? e : -1 - int32_t(lane));
    const uint32_t rank = __popc(peers & ((1u << lane) - 1u));
    if (live && rank == 0) wcnt[warp][e] = __popc(peers);
    __syncthreads();
    // ---- thread = expert (the first 256 threads): totals, tile cuts, exclusive scans
    const bool is_expert = tid < uint32_t(kExperts);
    uint32_t c = 0, n = 0;
    uint32_t v[4] = {0, 0, 0, 0}, inc[4] = {0, 0, 0, 0};
    if (is_expert) {
        for (int wi = 0; wi < kWarps; ++wi) { const uint32_t t = wcnt[wi][tid]; wcnt[wi][tid] = c; c += t; }
        n = c ? (c + max_n - 1) / max_n : 0;
        const uint32_t per = n ? (c + n - 1) / n : 0;
        cnt[tid] = c; ntl[tid] = n; width[tid] = (per + 15u) & ~15u;
        atomicMax(&max_count, c);
        v[0] = c; v[1] = n; v[2] = n * uint32_t(mt_fc1); v[3] = n * uint32_t(mt_fc2);
#pragma unroll
        for (int k = 0; k < 4; ++k) { inc[k] = warp_inclusive_scan(v[k], lane); if (lane == 31) wsum[k][warp] = inc[k]; }
    }
    const uint32_t active = __syncthreads_count(is_expert && c > 0);
    if (is_expert) {
        uint32_t add[4] = {0, 0, 0, 0};
        for (uint32_t wi = 0; wi < warp; ++wi)
#pragma unroll
            for (int k = 0; k < 4; ++k) add[k] += wsum[k][wi];
        rbase[tid] = inc[0] - v[0] + add[0]; tstart[tid] = inc[1] - v[1] + add[1];
        i1base[tid] = inc[2] - v[2] + add[2]; i2base[tid] = inc[3] - v[3] + add[3];
        if (blockIdx.x == 0 && tid == kExperts - 1) {
            PlanMeta m{};
            m.fault = 0; m.n_tiles = tstart[tid] + n; m.n_items_fc1 = i1base[tid] + n * mt_fc1;
            m.n_items_fc2 = i2base[tid] + n * mt_fc2; m.active_experts = active; m.max_count = max_count;
            *o.meta = m;
        }
    }
    __syncthreads();
    // ---- thread = route again: its grouped row, that row's tile and position
    if (live) {
        const uint32_t local = wcnt[warp][e] + rank, g = rbase[e] + local;
        row_token[g] = uint8_t(tid / kTopK);
        row_tile[g] = uint16_t(tstart[e] + local / width[e]);
        row_lr[g] = uint8_t(local % width[e]);
        row_first[g] = uint8_t(tid % kTopK == 0);
        if (blockIdx.x == 0) {
            o.inverse[tid] = int32_t(g);
            o.original_routes[g] = int32_t(tid);
            o.grouped_weights[g] = wt;
        }
    }
    // ---- plan tables, one group per CTA (thread = expert)
    if (is_expert && blockIdx.x == 1u % gridDim.x) {
        o.experts[tid] = ExpertPlan{int32_t(c), int32_t(rbase[tid]), int32_t(tstart[tid]), int32_t(width[tid])};
        for (uint32_t j = 0; j < n; ++j) {
            const uint32_t wd = width[tid], nv = c - j * wd < wd ? c - j * wd : wd;
            o.tiles[tstart[tid] + j] = TokenTile{int32_t(slots[tid]) & kSlotMask, int32_t(rbase[tid] + j * wd), int32_t(nv), int32_t((nv + 15u) & ~15u)};
        }
    }
    if (is_expert && blockIdx.x == 2u % gridDim.x)
        for (uint32_t i = 0; i < n * uint32_t(mt_fc1); ++i)
            o.items_fc1[i1base[tid] + i] = WorkItem{int32_t(tstart[tid] + i % n), int32_t(i / n)};
    if (is_expert && blockIdx.x == 3u % gridDim.x)
        for (uint32_t i = 0; i < n * uint32_t(mt_fc2); ++i)
            o.items_fc2[i2base[tid] + i] = WorkItem{int32_t(tstart[tid] + i % n), int32_t(i / n) * m_step2};
    __syncthreads();
    // ---- grouped rows, kRowsAtOnce side by side: thread t of a row's 256 holds elements [16 t, 16 t + 16), a K32 block is
    // a pair of threads. The bound is the same for every thread of a warp (a warp never straddles two rows).
    uint32_t bad_in = 0, bad_q = 0;
    const uint32_t sub = tid >> 8, rt = tid & 255u;
    for (uint32_t g = blockIdx.x * kRowsAtOnce + sub; g < routes; g += gridDim.x * kRowsAtOnce) {
        const uint32_t token = row_token[g];
        uint32_t code[16];
        uint32_t sbyte = 0;
        bool write = true;
        if constexpr (IN == 2) {
            const uint4 q = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(io.x) + size_t(token) * kHidden)[rt];
            code[0] = q.x; code[1] = q.y; code[2] = q.z; code[3] = q.w;
            sbyte = io.xs_in[size_t(token) * (kHidden / kBlockK) + (rt >> 1)];
        } else {
            uint32_t bits[16];
            if constexpr (IN == 0) {
                const uint4* src = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(io.x) + size_t(token) * kHidden) + 2 * rt;
                const uint4 a = src[0], b = src[1];
                const uint32_t wv[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
                for (int i = 0; i < 8; ++i) { bits[2 * i] = wv[i] << 16; bits[2 * i + 1] = wv[i] & 0xffff0000u; }
            } else {
                const uint4* src = reinterpret_cast<const uint4*>(static_cast<const float*>(io.x) + size_t(token) * kHidden) + 4 * rt;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint4 a = src[i];
                    bits[4 * i] = a.x; bits[4 * i + 1] = a.y; bits[4 * i + 2] = a.z; bits[4 * i + 3] = a.w;
                }
            }
            uint32_t amax = 0;
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                uint32_t m = bits[i] & 0x7fffffffu;
                if (CODEC == 0 && m > 0x7f800000u) m = 0;
                amax = m > amax ? m : amax;
            }
            const uint32_t other = __shfl_xor_sync(0xffffffffu, amax, 1);
            amax = other > amax ? other : amax;
            uint32_t cb[16];
            if constexpr (CODEC == 0) {
                sbyte = wire_scale_byte(amax);
#pragma unroll
                for (int i = 0; i < 16; ++i) cb[i] = wire_payload(bits[i], sbyte);
            } else {
                bool over = false;
                if (amax >= 0x7f800000u) {
                    bad_q |= kFaultQuantNonfinite;
                    write = false;
#pragma unroll
                    for (int i = 0; i < 16; ++i) cb[i] = 0;
                } else {
                    const int k = quant_v1_scale_exp(amax);
                    sbyte = uint32_t(k + 127);
#pragma unroll
                    for (int i = 0; i < 16; ++i) { cb[i] = quant_v1_payload(bits[i], k); over |= !quant_v1_finite(cb[i], k); }
                }
                uint32_t ov = over ? 1u : 0u;
                ov |= __shfl_xor_sync(0xffffffffu, ov, 1);
                if (ov) { bad_q |= kFaultQuantOverflow; write = false; }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) code[i] = cb[4 * i] | (cb[4 * i + 1] << 8) | (cb[4 * i + 2] << 16) | (cb[4 * i + 3] << 24);
        }
        if (!write) continue;   // a faulting quant_v1 block writes nothing; the pair of threads agrees
        // the input gate of the path
#pragma unroll
        for (int i = 0; i < 4; ++i)
            if ((((code[i] & 0x7f7f7f7fu) + 0x01010101u) & 0x80808080u) != 0u) bad_in = kFaultInputScale;
        if (sbyte < 105u || sbyte > 247u) bad_in = kFaultInputScale;
        const uint4 q = make_uint4(code[0], code[1], code[2], code[3]);
        reinterpret_cast<uint4*>(io.x_perm + size_t(g) * kHidden)[rt] = q;
        const uint32_t blk = rt >> 1;
        if ((rt & 1u) == 0u)
            io.sfb[(size_t(row_tile[g]) * (kHidden / kChunkK) + (blk >> 2)) * kScaleBlockBytes +
                   scale_block_offset(int(row_lr[g]), int(blk & 3u))] = uint8_t(sbyte);
        if (IN != 2 && io.xq_out && row_first[g]) {
            reinterpret_cast<uint4*>(io.xq_out + size_t(token) * kHidden)[rt] = q;
            if ((rt & 1u) == 0u) io.xs_out[size_t(token) * (kHidden / kBlockK) + blk] = uint8_t(sbyte);
        }
    }
    if (bad_in) atomicOr(io.fault_input, bad_in);
    if (IN != 2 && bad_q) atomicOr(io.fault_quant, bad_q);
}

}  // namespace m26b
