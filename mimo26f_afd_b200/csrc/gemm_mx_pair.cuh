// The grouped block-scaled GEMM on CTA pairs (tcgen05 cta_group::2), used for prefill-sized requests.
//
// Same math and work decomposition as gemm_mx.cuh, but two CTAs of a cluster run one MMA together:
//     M = 256 = 128 weight rows from each CTA's shared memory, accumulated in that CTA's tensor memory,
//     N = the token tile, whose rows are split between the two CTAs' shared memories.
// A pair works on one token tile and two neighbouring 256-row weight tile pairs (CTA r takes pair 2j + r), so
// each SM fetches only half of the token rows. What bounds the single-CTA kernel at prefill is the L2 -> SM
// path (about 60 B/clk per SM through the copy engine against 64 B/clk needed at N = 128); the pair needs 48,
// and the smaller token buffer leaves shared memory for a fifth pipeline stage.
//
// Per CTA: one producer warp (its weight rows, its half of the token rows, its weight scales, the whole
// tile's token scales), sixteen epilogue warps (its 128 + 128 accumulator rows). The pair's first
// CTA also runs the MMA-issue warp. Barriers: the loads of both CTAs report to `full` of the first CTA, whose
// producer alone announces the byte count of both (a barrier operation on the partner's shared memory costs about a
// thousand cycles, one on its own a few; the partner's bytes may land before the announcement, which the barrier's
// transaction count allows); tcgen05.commit arrives on `empty` / `acc_full` of both; the epilogue warps of both CTAs
// arrive on `acc_empty` of the first. All loads are ordinary per-CTA copies.
//
// Accumulators. An item needs two 128-column accumulators per CTA (weight tiles 0 and 1 of its 256 rows); tensor
// memory (512 columns) holds a ring of three, plus the scale slots. Item i takes buffers 2i and 2i + 1 (mod 3): its
// tile 0 always finds a buffer nobody uses, its tile 1 takes the buffer the previous item's tile 0 is being drained
// from. So an item opens with the tile-0 MMAs of its first kLead chunks alone, and only then waits for the drain,
// issues the tile-1 MMAs of those chunks, and carries on with both tiles per chunk: the tensor pipe has kLead x 4
// MMAs queued while the accumulators change hands (commit -> epilogue warps wake -> tcgen05.ld -> remote arrive ->
// this thread wakes), instead of idling through it as it does with a single buffer set.
//
// Token rows are read from a copy permuted into expert order (boxed TMA loads). Two ways of fetching them straight
// from the request's rows inside this kernel were built, gave bit-identical results, and were slower at 8,192 tokens
// than the permutation pass they saved (0.10 ms): 16-byte cp.async from an extra warp (hardware arrive on a local
// barrier, relayed to the first CTA) made FC1 1.07 ms instead of 0.96 ms, and TMA tile::gather4 (128 x 1 box, four rows
// per instruction, sixteen instructions per stage and CTA) 1.80 ms.
#pragma once
#include "gemm_mx.cuh"

namespace m26b {

constexpr int kPairStages = 5;
constexpr int kPairThreads = kGemmThreads;
constexpr int kAccBufs = 3;                            // ring of 128-column accumulator buffers
constexpr uint32_t kPairSfSlot0 = kAccBufs * kMaxN;    // scale slots above the accumulators
constexpr uint32_t kPairSfSlots = 8;                   // 16 columns each: SFA tile 0, SFA tile 1, SFB
constexpr int kPairLead = 2;                           // chunks of tile 0 issued before tile 1 of the item starts (1, 2 and 3 time alike)
static_assert(kPairSfSlot0 + kPairSfSlots * kSfSlotStride <= kTmemCols, "tensor memory holds 512 columns");
static_assert(kPairLead >= 1 && kPairLead < kPairStages && kPairLead < int(kPairSfSlots), "the lead chunks hold their stages and scale slots");

struct PairMaps {
    CUtensorMap tok[5];     // token rows, boxes of 128 / 64 / 32 / 16 / 8 rows
    CUtensorMap sfa;        // weight scale blocks as rows of 128 u32; box 2 rows (the two tiles of a pair)
    CUtensorMap sfb;        // token scale blocks as rows of 128 u32; box 1 row
};

struct PairSmem {
    alignas(1024) uint8_t a[kPairStages][kPairM * 128];
    alignas(1024) uint8_t b[kPairStages][(kMaxN / 2) * 128];
    alignas(128) uint8_t sfa[kPairStages][2 * kScaleBlockBytes];
    alignas(128) uint8_t sfb[kPairStages][kScaleBlockBytes];
    uint64_t full[kPairStages], empty[kPairStages], acc_full[kAccBufs], acc_empty[kAccBufs];
    uint32_t tmem_base;
    uint32_t abort_flag;
};
static_assert(sizeof(PairSmem) + 1024 <= 232448, "a CTA has at most 227 KB of shared memory");

// Buffer and use count of accumulator job j (item 2 * local + tile) in the ring.
__device__ __forceinline__ uint32_t acc_buf(uint32_t job) { return job % kAccBufs; }
__device__ __forceinline__ uint32_t acc_use(uint32_t job) { return job / kAccBufs; }

template <int MODE, bool DUMP = false, bool Y16 = false>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
gemm_mx_pair_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ PairMaps maps, const GemmArgs p) {
    extern __shared__ uint8_t smem_raw[];
    PairSmem& s = *reinterpret_cast<PairSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const uint32_t pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
    // epilogue warps that drain one accumulator buffer, over both CTAs: FC1 needs gate and up in every warp, FC2's
    // warps split by weight tile
    constexpr uint32_t kDrainers = MODE == kModeFc1 ? 2 * kEpiWarps : kEpiWarps;

    if (threadIdx.x == 0) {
        for (int i = 0; i < kPairStages; ++i) { mbar_init(&s.full[i], 1); mbar_init(&s.empty[i], 1); }
        for (int i = 0; i < kAccBufs; ++i) { mbar_init(&s.acc_full[i], 1); mbar_init(&s.acc_empty[i], kDrainers); }
        s.abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) { tmem_alloc_pair(&s.tmem_base, kTmemCols); tmem_relinquish_pair(); }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // the partner's barriers exist before anything arrives on them
    tc_fence_after();
    grid_dep_wait();             // the plan and the token rows come from the kernels before this one
    grid_dep_launch();
    const uint32_t tb = s.tmem_base;
    const uint32_t n_items = *p.n_items;
    volatile uint32_t* abort_flag = &s.abort_flag;

    if (warp == 0) {
        // ------------------------------------------------------------ producer (both CTAs)
        if (elect_one()) {
            tma_prefetch_desc(&map_w);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            for (uint32_t it = pair_id; it < n_items && ok; it += n_pairs) {
                const ItemInfo cur = load_item(p, it, n_items);
                const WorkItem wi = cur.wi;
                const TokenTile tt = cur.tt;
                const int m_tile = wi.m_tile + int(rank);
                const int w_row = (tt.expert * p.m_tiles + m_tile) * kPairM;
                const int sfa_row = (tt.expert * p.m_tiles + m_tile) * p.k_chunks * 2;
                const int sfb_row = wi.tile * p.k_chunks;
                const int half = tt.n_mma >> 1;                   // token rows this CTA holds
                const int tok_row = tt.row_base + int(rank) * half;
                const uint32_t tx = kPairM * 64 + uint32_t(half) * 128 + 3 * kScaleBlockBytes;
                for (int c = 0; c < p.k_chunks; ++c) {
                    if (!mbar_wait(&s.empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
                    const uint32_t bar = cluster_map(smem_u32(&s.full[stage]), 0);
                    if (rank == 0) mbar_expect_tx(&s.full[stage], 2 * tx);   // the bytes of both CTAs' loads
                    tma_load_2d_pair(s.a[stage], &map_w, c * kChunkK, w_row, bar);
                    int r = 0;
#pragma unroll
                    for (int i = 1; i < 5; ++i) {
                        const int rows = 128 >> i;
                        if (half - r >= rows) {
                            tma_load_2d_pair(s.b[stage] + r * 128, &maps.tok[i], c * kChunkK, tok_row + r, bar);
                            r += rows;
                        }
                    }
                    tma_load_2d_pair(s.sfa[stage], &maps.sfa, 0, sfa_row + 2 * c, bar);
                    tma_load_2d_pair(s.sfb[stage], &maps.sfb, 0, sfb_row + c, bar);
                    if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) atomicOr(p.fault, uint32_t(kFaultPipeline));
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issue (first CTA of the pair only)
        if (rank == 0 && elect_one()) {
            uint32_t stage = 0, phase = 0, local = 0, sf_slot = 0;
            bool ok = true;
            const uint64_t a_desc0 = desc_sw128(smem_u32(s.a[0])), b_desc0 = desc_sw128(smem_u32(s.b[0]));
            const uint64_t sfa_desc0 = desc_scale_block(smem_u32(s.sfa[0])), sfb_desc0 = desc_scale_block(smem_u32(s.sfb[0]));
            constexpr uint64_t kAStage = sizeof(s.a[0]) >> 4, kBStage = sizeof(s.b[0]) >> 4;
            constexpr uint64_t kSfaStage = sizeof(s.sfa[0]) >> 4, kSfbStage = sizeof(s.sfb[0]) >> 4;
            constexpr uint64_t kTile1 = (kTileM * 128) >> 4;      // tile 1's rows inside a stage's weight buffer
            auto wait_full = [&](uint32_t st, uint32_t ph) { return mbar_wait(&s.full[st], ph, abort_flag); };
            for (uint32_t it = pair_id; it < n_items && ok; it += n_pairs, ++local) {
                const ItemInfo cur = load_item(p, it, n_items);
                const TokenTile tt = cur.tt;
                const uint32_t idesc0 = idesc_mx_pair(kFmtE2M1, kFmtE4M3, uint32_t(tt.n_mma), 0, 0);
                const uint32_t j0 = 2 * local, j1 = j0 + 1;
                const uint32_t d0 = tb + acc_buf(j0) * kMaxN, d1 = tb + acc_buf(j1) * kMaxN;
                const int lead = p.k_chunks < kPairLead ? p.k_chunks : kPairLead;
                // tile 0: its buffer was drained an item ago
                if (!mbar_wait(&s.acc_empty[acc_buf(j0)], (acc_use(j0) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t stage0 = stage, slot0 = sf_slot;
                for (int c = 0; c < lead && ok; ++c) {
                    if (!wait_full(stage, phase)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t t_sf = tb + kPairSfSlot0 + sf_slot * kSfSlotStride;
                    const uint64_t sfa_d = sfa_desc0 + stage * kSfaStage;
                    tc_cp_scales_pair(t_sf, sfa_d);
                    tc_cp_scales_pair(t_sf + 4, sfa_d + (kScaleBlockBytes >> 4));
                    tc_cp_scales_pair(t_sf + 8, sfb_desc0 + stage * kSfbStage);
                    const uint64_t ad = a_desc0 + stage * kAStage, bd = b_desc0 + stage * kBStage;
#pragma unroll
                    for (uint32_t kb = 0; kb < 4; ++kb)
                        tc_mma_mx_pair(d0, ad + 2 * kb, bd + 2 * kb, idesc0 | (kb << 4) | (kb << 29), t_sf, t_sf + 8, (c | int(kb)) ? 1u : 0u);
                    sf_slot = (sf_slot + 1) % kPairSfSlots;
                    if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                // tile 1: the buffer the previous item's tile 0 is being drained from
                if (!mbar_wait(&s.acc_empty[acc_buf(j1)], (acc_use(j1) & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                {
                    uint32_t st = stage0, slot = slot0;
                    for (int c = 0; c < lead; ++c) {
                        const uint32_t t_sf = tb + kPairSfSlot0 + slot * kSfSlotStride;
                        const uint64_t ad = a_desc0 + st * kAStage + kTile1, bd = b_desc0 + st * kBStage;
#pragma unroll
                        for (uint32_t kb = 0; kb < 4; ++kb)
                            tc_mma_mx_pair(d1, ad + 2 * kb, bd + 2 * kb, idesc0 | (kb << 4) | (kb << 29), t_sf + 4, t_sf + 8, (c | int(kb)) ? 1u : 0u);
                        tc_commit_pair(&s.empty[st]);
                        slot = (slot + 1) % kPairSfSlots;
                        if (++st == kPairStages) st = 0;
                    }
                }
                for (int c = lead; c < p.k_chunks; ++c) {
                    if (!wait_full(stage, phase)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t t_sf = tb + kPairSfSlot0 + sf_slot * kSfSlotStride;
                    const uint64_t sfa_d = sfa_desc0 + stage * kSfaStage;
                    tc_cp_scales_pair(t_sf, sfa_d);
                    tc_cp_scales_pair(t_sf + 4, sfa_d + (kScaleBlockBytes >> 4));
                    tc_cp_scales_pair(t_sf + 8, sfb_desc0 + stage * kSfbStage);
                    const uint64_t ad = a_desc0 + stage * kAStage, bd = b_desc0 + stage * kBStage;
#pragma unroll
                    for (uint32_t kb = 0; kb < 4; ++kb) {
                        // K32 slice kb: 32 bytes further into the swizzle atom; scale byte kb of each tensor-memory column
                        const uint32_t idesc = idesc0 | (kb << 4) | (kb << 29);
                        tc_mma_mx_pair(d0, ad + 2 * kb, bd + 2 * kb, idesc, t_sf, t_sf + 8, 1u);
                        tc_mma_mx_pair(d1, ad + kTile1 + 2 * kb, bd + 2 * kb, idesc, t_sf + 4, t_sf + 8, 1u);
                    }
                    tc_commit_pair(&s.empty[stage]);
                    sf_slot = (sf_slot + 1) % kPairSfSlots;
                    if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
                }
                if (ok) { tc_commit_pair(&s.acc_full[acc_buf(j0)]); tc_commit_pair(&s.acc_full[acc_buf(j1)]); }
            }
            if (!ok) atomicOr(p.fault, uint32_t(kFaultPipeline));
        }
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs)
        const uint32_t q = uint32_t(warp) & 3u;
        const uint32_t wq = uint32_t(warp - 2) >> 2;
        uint32_t local = 0;
        bool ok = true;
        for (uint32_t it = pair_id; it < n_items && ok; it += n_pairs, ++local) {
            const ItemInfo cur = load_item(p, it, n_items);
            const WorkItem wi = cur.wi;
            const TokenTile tt = cur.tt;
            const int m_tile = wi.m_tile + int(rank);
            const uint32_t j0 = 2 * local, j1 = j0 + 1;
            const uint32_t lane_base = (q * 32u) << 16;
            if constexpr (MODE == kModeFc2) {
                // warp (q, wq): weight tile (wq & 1) of the CTA's two, token groups (wq >> 1), +2, +4 ... of 8 tokens.
                // Lane l holds the route of token (wq >> 1) * 8 + 16 (l / 8) + l % 8 as the address of its output row
                // (0 for a padding column), fetched before the accumulators are waited for.
                unsigned long long row_lo = 0, row_hi = 0;
                {
                    const int t = (int(wq >> 1) + 2 * (lane >> 3)) * 8 + (lane & 7);
                    if (t < tt.n_valid) row_lo = reinterpret_cast<unsigned long long>(y_row<Y16>(p, p.original_routes[tt.row_base + t]));
                    if (t + 64 < tt.n_valid) row_hi = reinterpret_cast<unsigned long long>(y_row<Y16>(p, p.original_routes[tt.row_base + t + 64]));
                }
                const uint32_t tile = wq & 1u;
                const uint32_t job = tile ? j1 : j0;
                if (!mbar_wait(&s.acc_full[acc_buf(job)], acc_use(job) & 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t t_acc = tb + lane_base + acc_buf(job) * kMaxN;
                uint32_t r[8][8];
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    const int c0 = (int(wq >> 1) + 2 * g) * 8;
                    if (c0 < tt.n_mma) tmem_ld8(t_acc + uint32_t(c0), r[g]);
                }
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(cluster_map(smem_u32(&s.acc_empty[acc_buf(job)]), 0));
                const uint32_t ycol = uint32_t(m_tile) * kPairM + tile * kTileM + q * 32u + lane;
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    if ((int(wq >> 1) + 2 * g) * 8 >= tt.n_mma) break;      // warp-uniform: no columns beyond the tile
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const unsigned long long row = __shfl_sync(0xffffffffu, g < 4 ? row_lo : row_hi, (g & 3) * 8 + j);
                        if (row) y_store<Y16>(row, ycol, r[g][j]);
                    }
                }
            } else {
                // lanes are the 32 features of K32 block (4 m + q) of the intermediate; warp wq of the quadrant takes
                // token groups wq, wq + 4, wq + 8, wq + 12 of 8 tokens. Gate first: its buffer is the one the next
                // item's tile 1 waits for.
                uint32_t gt[4][8], up[4][8];
                if (!mbar_wait(&s.acc_full[acc_buf(j0)], acc_use(j0) & 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int c0 = (int(wq) + 4 * g) * 8;
                    if (c0 < tt.n_mma) tmem_ld8(tb + lane_base + acc_buf(j0) * kMaxN + uint32_t(c0), gt[g]);
                }
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(cluster_map(smem_u32(&s.acc_empty[acc_buf(j0)]), 0));
                if (!mbar_wait(&s.acc_full[acc_buf(j1)], acc_use(j1) & 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int c0 = (int(wq) + 4 * g) * 8;
                    if (c0 < tt.n_mma) tmem_ld8(tb + lane_base + acc_buf(j1) * kMaxN + uint32_t(c0), up[g]);
                }
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(cluster_map(smem_u32(&s.acc_empty[acc_buf(j1)]), 0));
                const int feat0 = m_tile * kTileM + int(q) * 32;
                uint8_t* sf_tile = p.mid_sf + (size_t(wi.tile) * (p.i_local / kChunkK) + m_tile) * kScaleBlockBytes;
                uint8_t* mq = p.mid_q + size_t(tt.row_base) * p.i_local + feat0 + lane;
                float* mf = DUMP ? p.mid_f32 + size_t(tt.row_base) * p.i_local + feat0 + lane : nullptr;
                uint32_t fault = 0;
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int c0 = (int(wq) + 4 * g) * 8;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int t = c0 + j;
                        if (t >= tt.n_valid) continue;   // warp-uniform
                        const float h = silu_mul(__uint_as_float(gt[g][j]), __uint_as_float(up[g][j]));
                        if constexpr (DUMP) mf[size_t(t) * p.i_local] = h;
                        const uint32_t bits = __float_as_uint(h);
                        const uint32_t amax = __reduce_max_sync(0xffffffffu, bits & 0x7fffffffu);
                        if (amax >= 0x7f800000u) { fault |= kFaultQuantNonfinite; continue; }
                        const int k = quant_v1_scale_exp(amax);
                        const uint32_t code = quant_v1_payload(bits, k);
                        if (k > 119 && __any_sync(0xffffffffu, !quant_v1_finite(code, k))) { fault |= kFaultQuantOverflow; continue; }
                        mq[size_t(t) * p.i_local] = uint8_t(code);
                        if (lane == 0) sf_tile[scale_block_offset(t, int(q))] = uint8_t(k + 127);
                    }
                }
                if (fault && lane == 0) atomicOr(p.fault, fault);
            }
        }
        if (!ok && lane == 0) atomicOr(p.fault, uint32_t(kFaultPipeline));
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();          // nothing of either CTA is torn down while the partner may still signal it
    if (warp == 1) tmem_dealloc_pair(tb, kTmemCols);
}

}  // namespace m26b
