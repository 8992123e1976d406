// Grouped block-scaled GEMM for the expert FFN on tcgen05 (sm_100a).
//
// Both projections run the same main loop with the weights as the MMA "A"
// operand and the routed tokens as "B":
//     D[weight row, token] = sum_k E2M1(w) 2^sw  *  E4M3(x) 2^sx
// A work item is (token tile of one expert) x (256 weight rows = two 128-row
// MMA tiles). Weight rows are the tcgen05 M = 128; the token count of the tile
// is the MMA N (a multiple of 16, at most 128), so one or two routed rows per
// expert at decode do not pad to a 128-row tile. The two MMA tiles of an item
// share the token operand in shared memory and accumulate side by side in
// tensor memory: for FC1 they are the gate and up rows of the same 128
// features, so a feature's gate and up land in the same tensor-memory lane.
//
//   producer warp : TMA loads per 128-wide K chunk - the 4-bit weight rows
//                   (unpacked to 8-bit containers by the 16U4_ALIGN16B tensor
//                   map), the E4M3 token rows, and the UE8M0 scale blocks.
//   MMA warp      : copies the scale blocks to tensor memory (tcgen05.cp) and
//                   issues 8 x tcgen05.mma kind::mxf8f6f4.block_scale per chunk
//                   into the accumulator pair in tensor memory.
//   16 epilogue   : four warps per lane quadrant. Each first pulls its slice of
//     warps         the accumulators into registers (64 values per thread) and
//                   hands tensor memory straight back to the MMA warp, so the
//                   next item's main loop runs while the epilogue math proceeds
//                   from registers; one accumulator buffer is enough, which is
//                   what lets the token tile be 128 wide.
//                   FC1: SiLU(gate)*up and the e4m3fn-k32-v1 quantiser run in
//                   registers - a warp's 32 lanes are the 32 features of one
//                   K32 block, so the block maximum is one warp reduction -
//                   and the quantised intermediate plus its scale bytes are
//                   stored in the layout FC2's loads want.
//                   FC2: FP32 rows are stored at their original route index.
//
// Reference behaviour: FC1 crates/mimo26-expert/kernels/b1/grouped.cu:71-113,
// quantiser kernels/b1/quant_v1.cuh:32-100, FC2 grouped.cu:136-154 and
// kernels/b1/connected.cu:48-79 (unweighted rows in original route order).
#pragma once
#include "sm100_ptx.cuh"
#include "layout.cuh"
#include "codec.cuh"

namespace m26b {

constexpr int kEpiWarps = 16;
constexpr int kGemmThreads = 64 + 32 * kEpiWarps;
// Tensor memory: weight tile 0 accumulates in columns [0, 128), tile 1 in [128, 256); the two
// scale slots sit above them.
constexpr int kAcc1 = kMaxN;
constexpr int kSfSlot0 = 256, kSfSlotStride = 16;      // slot: 4 cols SFA tile 0, 4 cols SFA tile 1, 4 cols SFB
constexpr uint32_t kTmemCols = 512;

enum { kModeFc1 = 1, kModeFc2 = 2 };

// Where FC2 puts its rows when the tokens belong to several GPUs (expert parallelism): token t of the request is row
// t - lo[k] of owner k, the k with lo[k] <= t < lo[k + 1]; route (t, slot) goes to y[k] + ((t - lo[k]) * 8 + slot) * 4096.
// The pointers are ordinary device addresses: the local buffer, or a peer's buffer mapped into this process.
// n = 0: everything goes to GemmArgs::y.
struct RouteSinks {
    uint32_t n;
    uint32_t token_base;        // request-wide index of the pass's first token
    uint32_t lo[9];
    float* y[8];
};

struct GemmArgs {
    const TokenTile* tiles;
    const WorkItem* items;
    const uint32_t* n_items;
    const uint8_t* sfa;         // weight scale blocks [E][m_tiles][k_chunks][2][512]
    const uint8_t* sfb;         // token scale blocks  [tile][k_chunks][512]
    int m_tiles;                // 256-row weight tile pairs per expert
    int m_span;                 // weight tile pairs one work item of the single-CTA kernel covers (consecutive, same token tile)
    int k_chunks;               // K / 128
    uint32_t* fault;            // one word, OR of fault codes
    // FC1 epilogue
    uint8_t* mid_q;             // [grouped rows][i_local] E4M3
    uint8_t* mid_sf;            // scale blocks for FC2 [tile][i_local/128][512]
    float* mid_f32;             // FP32 copy of silu(gate)*up, same indexing as mid_q (stage-dump instantiations only)
    int i_local;
    // FC2 epilogue
    float* y;                   // [routes][4096] FP32 (BF16 with the route-output option), original route order
    const int32_t* original_routes;
    RouteSinks sinks;
};

// A work item and its token tile (two dependent global loads at the top of an item in every role; loading the next
// item's pair one item ahead was tried and changed nothing for short items while costing FC1 3 %).
struct ItemInfo {
    WorkItem wi;
    TokenTile tt;
};
__device__ __forceinline__ ItemInfo load_item(const GemmArgs& p, uint32_t it, uint32_t n_items) {
    ItemInfo r{};
    if (it < n_items) { r.wi = p.items[it]; r.tt = p.tiles[r.wi.tile]; }
    return r;
}

// Row of the FC2 output for a route of the pass. Rows are FP32, or BF16 with the route-output option (Y16): the
// reference's MIMO26_B1_Y=bf16 mode, crates/mimo26-spark/kernels/b1_serve.cu:400-406.
template <bool Y16>
__device__ __forceinline__ uint8_t* y_row(const GemmArgs& p, int32_t route) {
    constexpr size_t kRowBytes = size_t(kHidden) * (Y16 ? 2 : 4);
    if (p.sinks.n == 0) return reinterpret_cast<uint8_t*>(p.y) + size_t(route) * kRowBytes;
    const uint32_t token = p.sinks.token_base + uint32_t(route) / kTopK, slot = uint32_t(route) % kTopK;
    uint32_t k = 0;
#pragma unroll
    for (uint32_t i = 1; i < 8; ++i)
        if (i < p.sinks.n && token >= p.sinks.lo[i]) k = i;
    return reinterpret_cast<uint8_t*>(p.sinks.y[k]) + (size_t(token - p.sinks.lo[k]) * kTopK + slot) * kRowBytes;
}
// One FC2 output element of column `col` into the row at `row`.
template <bool Y16>
__device__ __forceinline__ void y_store(unsigned long long row, uint32_t col, uint32_t f32_bits) {
    if constexpr (Y16) reinterpret_cast<uint16_t*>(row)[col] = uint16_t(bf16_rne_bits(__uint_as_float(f32_bits)));
    else reinterpret_cast<float*>(row)[col] = __uint_as_float(f32_bits);
}

// Token-operand tensor maps with boxes of 128, 64, 32 and 16 rows: a tile's rows are fetched with the fewest
// boxes (binary decomposition of its row count). One 128-row box costs the copy engine about 500 cycles, eight
// 16-row boxes about 680, and the main loop has 512 cycles per chunk to spare at N = 128.
struct TokenMaps {
    CUtensorMap box[4];
};

// A_TILES = 2: an item is a 256-row weight tile pair (two MMA tiles side by side in tensor memory). A_TILES = 1 (FC1 only):
// an item is HALF a tile pair - 64 gate rows and the 64 up rows of the same features in ONE 128-row MMA tile - so a
// decode step has twice as many, half as long items to spread over the SMs (a tensor-parallel rank of eight has 204 full
// items for 148 SMs: two rounds where 1.4 would do). Gate and up of a feature then sit in different tensor-memory lanes
// (quadrants 0-1 gate, 2-3 up): the up warps hand their values to the gate warps through `xup`.
// A stage of half items holds TWO K chunks, so that a stage (and with it every copy instruction and barrier hand-over)
// moves as many bytes as a stage of full items: [chunk][rows][128 bytes] for both operands, [chunk][512] for the scales.
template <int B_ROWS, int STAGES, int A_TILES = 2>
struct GemmSmem {
    static constexpr int kSub = A_TILES == 1 ? 2 : 1;      // K chunks per stage
    alignas(1024) uint8_t a[STAGES][kSub * A_TILES * kTileM * 128];
    alignas(1024) uint8_t b[STAGES][kSub * B_ROWS * 128];
    alignas(16) uint8_t sfa[STAGES][kSub * A_TILES * kScaleBlockBytes];
    alignas(16) uint8_t sfb[STAGES][kSub * kScaleBlockBytes];
    uint64_t full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
    uint32_t tmem_base;
    uint32_t abort_flag;
    alignas(16) uint32_t xup[A_TILES == 1 ? 8 : 1][A_TILES == 1 ? B_ROWS / 4 : 1][32];   // [warp pair][value][lane]
};

// Barrier `id` (1..15) over `threads` threads that also ORs a predicate over them: every participant gets the same answer.
__device__ __forceinline__ bool named_bar_or(uint32_t id, uint32_t threads, bool pred) {
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %3, 0;\n\tbar.red.or.pred q, %1, %2, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                 : "=r"(r) : "r"(id), "r"(threads), "r"(uint32_t(pred)) : "memory");
    return r != 0;
}
__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" :: "r"(id), "r"(threads) : "memory");
}

// E-ACT-CR32 activation: e = exp(-|g|) (never a positive exponential), s = g / (1 + e) or g e / (1 + e),
// h = s u. The exponential and the reciprocal of 1 + e (which lies in [1, 2]) use the hardware
// approximations (ex2.approx, rcp.approx: one instruction each, about one ulp): together under 1e-6 relative, inside
// the 1e-5 stage tolerance, at a fifth of the instructions of expf and an IEEE divide. Measured against the oracle the
// intermediate's relative L2 error is 1.3e-7 either way and the count of E4M3 bin crossings does not move; the
// correctly rounded reciprocal cost FC1 3 % at prefill. This runs once per intermediate element and the kernel is at
// the power limit, so every instruction here is clock.
__device__ __forceinline__ float silu_mul(float g, float u) {
    const float e = __expf(-fabsf(g));
    float r;
    asm("rcp.approx.f32 %0, %1;" : "=f"(r) : "f"(__fadd_rn(1.0f, e)));
    const float num = g >= 0.0f ? g : __fmul_rn(g, e);
    return __fmul_rn(__fmul_rn(num, r), u);
}

static_assert(sizeof(GemmSmem<32, 6>) + 1024 <= 232448 && sizeof(GemmSmem<kMaxN, 4>) + 1024 <= 232448 && sizeof(GemmSmem<64, 5>) + 1024 <= 232448 &&
              sizeof(GemmSmem<32, 5, 1>) + 1024 <= 232448,
              "a CTA has at most 227 KB of shared memory");

// DUMP: also store the FP32 intermediate (stage dumps of the parity tests). Y16: FC2 rows as BF16.
// A_TILES = 1 (FC1, token tiles of at most 64): half items; map_w is then the 3-D view of w13 [tile pair x gate/up][128 rows][K]
// with boxes of 2 x 64 rows, p.sfa names the half-item scale image [E][m_tiles][2 halves][k_chunks][512] and
// WorkItem::m_tile counts halves.
template <int MODE, int B_ROWS, int STAGES, bool DUMP = false, bool Y16 = false, int A_TILES = 2>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ TokenMaps maps_x, const GemmArgs p) {
    using Smem = GemmSmem<B_ROWS, STAGES, A_TILES>;
    constexpr bool kHalf = A_TILES == 1;
    constexpr int kSub = Smem::kSub;
    static_assert(!kHalf || (MODE == kModeFc1 && B_ROWS <= 64), "half items: FC1 with token tiles of at most 64");
    // Token tiles of at most 64 columns leave room for two accumulator sets in each tile's 128 tensor-memory columns
    // (set b at column offset b * B_ROWS): the MMAs of item i + 1 start while the epilogue still pulls item i. With items
    // as short as a rank's K slice under tensor parallelism (2-8 chunks) the hand-over would otherwise be half the time.
    constexpr uint32_t kAccSets = B_ROWS <= 64 ? 2u : 1u;
    extern __shared__ uint8_t smem_raw[];
    Smem& s = *reinterpret_cast<Smem*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) { mbar_init(&s.full[i], 1); mbar_init(&s.empty[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&s.acc_full[i], 1); mbar_init(&s.acc_empty[i], kEpiWarps); }
        s.abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) { tmem_alloc(&s.tmem_base, kTmemCols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    // The plan and the token rows come from the kernels before this one. FC2's producer warp waits later: the route plan
    // is older than the FC1 launch in front of it (FC1 let this grid start only after its own wait on the plan's
    // kernels), and the weights are static, so the weight half of its first stages is requested while FC1 still runs
    // on other SMs; only the intermediate rows and their scales need FC1 to be complete.
    constexpr bool kEarlyWeights = MODE == kModeFc2;
    if (!(kEarlyWeights && warp == 0)) { grid_dep_wait(); grid_dep_launch(); }
    const uint32_t tb = s.tmem_base;
    // FC2's producer warp has not waited for its predecessors yet: it reads the plan around L1 (the plan is older than
    // the FC1 launch in front of this grid, but only the wait makes earlier grids' writes visible to cached loads).
    const uint32_t n_items = (kEarlyWeights && warp == 0) ? __ldcv(p.n_items) : *p.n_items;
    volatile uint32_t* abort_flag = &s.abort_flag;

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (elect_one()) {
            tma_prefetch_desc(&map_w);
#pragma unroll
            for (int i = 0; i < 4; ++i) tma_prefetch_desc(&maps_x.box[i]);
            uint32_t stage = 0, phase = 0;
            bool ok = true;
            int early = 0;       // chunks of the first item whose weight boxes and weight scales are already in flight
            if constexpr (kEarlyWeights) {
                if (blockIdx.x < n_items) {
                    ItemInfo cur{};
                    {   // the same two records load_item() reads, around L1
                        const int2 wi = __ldcv(reinterpret_cast<const int2*>(p.items) + blockIdx.x);
                        const int4 tt = __ldcv(reinterpret_cast<const int4*>(p.tiles) + wi.x);
                        cur.wi = WorkItem{wi.x, wi.y};
                        cur.tt = TokenTile{tt.x, tt.y, tt.z, tt.w};
                    }
                    const int slot = cur.tt.expert * p.m_tiles + cur.wi.m_tile;
                    const uint8_t* sfa_g = p.sfa + size_t(slot) * p.k_chunks * 2 * kScaleBlockBytes;
                    const uint32_t tx = kPairM * 64 + cur.tt.n_mma * 128 + 3 * kScaleBlockBytes;
                    early = p.k_chunks < STAGES ? p.k_chunks : STAGES;       // every stage is free at the start
                    for (int c = 0; c < early; ++c) {
                        mbar_expect_tx(&s.full[c], tx);                       // the whole stage: the token half follows below
                        tma_load_2d(s.a[c], &map_w, c * kChunkK, slot * kPairM, &s.full[c]);
                        bulk_load(s.sfa[c], sfa_g + size_t(c) * 2 * kScaleBlockBytes, 2 * kScaleBlockBytes, &s.full[c]);
                    }
                }
                grid_dep_wait();
                grid_dep_launch();
            }
            for (uint32_t it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
                const ItemInfo cur = load_item(p, it, n_items);
                const WorkItem wi = cur.wi;
                const TokenTile tt = cur.tt;
                const uint8_t* sfb_g = p.sfb + size_t(wi.tile) * p.k_chunks * kScaleBlockBytes;
                const uint32_t tx = kSub * (A_TILES * kTileM * 64 + tt.n_mma * 128 + (A_TILES + 1) * kScaleBlockBytes);
                for (int mm = 0; mm < p.m_span && ok; ++mm) {
                    // half items: m_tile counts halves; half h of tile pair j = gate rows 64 h .. and up rows 128 + 64 h ..
                    const int m_pair = kHalf ? (wi.m_tile >> 1) : wi.m_tile + mm, half = kHalf ? (wi.m_tile & 1) : 0;
                    const int slot = tt.expert * p.m_tiles + m_pair;
                    const int w_row = slot * kPairM;
                    const uint8_t* sfa_g = p.sfa + (size_t(slot) * 2 + half) * p.k_chunks * kScaleBlockBytes;
                    for (int c = 0; c < p.k_chunks; c += kSub) {
                        const bool weights_in_flight = kEarlyWeights && it == blockIdx.x && mm == 0 && c < early;
                        if (!weights_in_flight) {
                            if (!mbar_wait(&s.empty[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
                            mbar_expect_tx(&s.full[stage], tx);
                            if constexpr (kHalf) {
#pragma unroll
                                for (int u = 0; u < kSub; ++u)      // one box: 64 gate rows, then the 64 up rows of the same features
                                    tma_load_3d(s.a[stage] + u * kTileM * 128, &map_w, (c + u) * kChunkK, half * (kTileM / 2), slot * 2, &s.full[stage]);
                            } else {
                                tma_load_2d(s.a[stage], &map_w, c * kChunkK, w_row, &s.full[stage]);
                            }
                            bulk_load(s.sfa[stage], sfa_g + size_t(c) * A_TILES * kScaleBlockBytes, kSub * A_TILES * kScaleBlockBytes, &s.full[stage]);
                        }
#pragma unroll
                        for (int u = 0; u < kSub; ++u) {
                            int r = 0;
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int rows = 128 >> i;
                                if (tt.n_mma - r >= rows) {   // n_mma <= 128: each size is needed at most once
                                    tma_load_2d(s.b[stage] + (u * B_ROWS + r) * 128, &maps_x.box[i], (c + u) * kChunkK, tt.row_base + r, &s.full[stage]);
                                    r += rows;
                                }
                            }
                        }
                        bulk_load(s.sfb[stage], sfb_g + size_t(c) * kScaleBlockBytes, kSub * kScaleBlockBytes, &s.full[stage]);
                        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                    }
                }
            }
            if (!ok) atomicOr(p.fault, uint32_t(kFaultPipeline));
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issue
        if (elect_one()) {
            uint32_t stage = 0, phase = 0, local = 0, sf_slot = 0;
            bool ok = true;
            // everything about a stage that does not change is computed once: this thread issues eleven tensor
            // operations per chunk and shares its scheduler with four epilogue warps
            const uint64_t a_desc0 = desc_sw128(smem_u32(s.a[0])), b_desc0 = desc_sw128(smem_u32(s.b[0]));
            const uint64_t sfa_desc0 = desc_scale_block(smem_u32(s.sfa[0])), sfb_desc0 = desc_scale_block(smem_u32(s.sfb[0]));
            constexpr uint64_t kAStage = sizeof(s.a[0]) >> 4, kBStage = sizeof(s.b[0]) >> 4;
            constexpr uint64_t kSfaStage = sizeof(s.sfa[0]) >> 4, kSfbStage = sizeof(s.sfb[0]) >> 4;
            for (uint32_t it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
                const ItemInfo cur = load_item(p, it, n_items);
                const TokenTile tt = cur.tt;
                const uint32_t idesc0 = idesc_mx(kFmtE2M1, kFmtE4M3, uint32_t(tt.n_mma), 0, 0);
              for (int mm = 0; mm < p.m_span && ok; ++mm, ++local) {
                // the accumulators are free once every epilogue warp has pulled its slice of the previous item
                const uint32_t aset = local % kAccSets, ause = local / kAccSets;
                if (!mbar_wait(&s.acc_empty[aset], (ause & 1u) ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d0 = tb + aset * B_ROWS, d1 = d0 + kAcc1;
                for (int c = 0; c < p.k_chunks; c += kSub) {
                    if (!mbar_wait(&s.full[stage], phase, abort_flag)) { ok = false; break; }
                    tc_fence_after();
#pragma unroll
                    for (int u = 0; u < kSub; ++u) {
                        // consecutive chunks alternate between two scale slots in tensor memory
                        const uint32_t t_sf = tb + kSfSlot0 + sf_slot * kSfSlotStride;
                        sf_slot ^= 1u;
                        const uint64_t sfa_d = sfa_desc0 + stage * kSfaStage + u * ((A_TILES * kScaleBlockBytes) >> 4);
                        tc_cp_scales(t_sf, sfa_d);
                        if constexpr (!kHalf) tc_cp_scales(t_sf + 4, sfa_d + (kScaleBlockBytes >> 4));
                        tc_cp_scales(t_sf + 8, sfb_desc0 + stage * kSfbStage + u * (kScaleBlockBytes >> 4));
                        const uint64_t ad = a_desc0 + stage * kAStage + u * ((A_TILES * kTileM * 128) >> 4);
                        const uint64_t bd = b_desc0 + stage * kBStage + u * ((B_ROWS * 128) >> 4);
#pragma unroll
                        for (uint32_t kb = 0; kb < 4; ++kb) {
                            // K32 slice kb: 32 bytes further into the swizzle atom (descriptor addresses count 16 bytes);
                            // scale-factor byte kb of each tensor-memory column (instruction-descriptor bits 4-5 and 29-30)
                            const uint32_t idesc = idesc0 | (kb << 4) | (kb << 29);
                            const uint32_t accum = (c | u | int(kb)) ? 1u : 0u;
                            tc_mma_mx(d0, ad + 2 * kb, bd + 2 * kb, idesc, t_sf, t_sf + 8, accum);
                            if constexpr (!kHalf) tc_mma_mx(d1, ad + ((kTileM * 128) >> 4) + 2 * kb, bd + 2 * kb, idesc, t_sf + 4, t_sf + 8, accum);
                        }
                    }
                    tc_commit(&s.empty[stage]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (ok) tc_commit(&s.acc_full[aset]);
              }
            }
            if (!ok) atomicOr(p.fault, uint32_t(kFaultPipeline));
        }
    } else {
        // ------------------------------------------------------------ epilogue
        const uint32_t q = uint32_t(warp) & 3u;            // tensor-memory lane quadrant this warp may read
        const uint32_t wq = uint32_t(warp - 2) >> 2;       // which of the quadrant's four warps this is
        static_assert(kEpiWarps == 16 && kMaxN == 128, "the register drain below is sized for 4 warps per quadrant");
        uint32_t local = 0;
        bool ok = true;
        for (uint32_t it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
            const ItemInfo cur = load_item(p, it, n_items);
            WorkItem wi = cur.wi;
            const TokenTile tt = cur.tt;
            // FC2: where this warp's token columns go. Lane l holds the route of token (wq >> 1) * 8 + 16 (l / 8) + l % 8 as
            // the address of its output row (0 for a padding column), fetched before the accumulators are waited for.
            unsigned long long row_lo = 0, row_hi = 0;
            if constexpr (MODE == kModeFc2) {
                const int t = (int(wq >> 1) + 2 * (lane >> 3)) * 8 + (lane & 7);
                if (t < tt.n_valid) row_lo = reinterpret_cast<unsigned long long>(y_row<Y16>(p, p.original_routes[tt.row_base + t]));
                if (t + 64 < tt.n_valid) row_hi = reinterpret_cast<unsigned long long>(y_row<Y16>(p, p.original_routes[tt.row_base + t + 64]));
            }
          // the item's weight tile pairs one after the other: same token tile, same output rows
          for (int mm = 0; mm < p.m_span && ok; ++mm, ++local, ++wi.m_tile) {
            const uint32_t aset = local % kAccSets, ause = local / kAccSets;
            const bool got = mbar_wait(&s.acc_full[aset], ause & 1u, abort_flag);
            const uint32_t t_acc = tb + ((q * 32u) << 16) + aset * B_ROWS;
            if constexpr (kHalf) {
                // lanes of quadrants 0, 1: gate of features 64 half + 32 q + lane; quadrants 2, 3: up of the same features.
                // Warp (q, wq) and warp (q + 2, wq) form a pair on named barrier 1 + pair: the up warp parks its values in
                // shared memory, the gate warp picks them up. The first barrier also carries "my wait ran out", so both
                // warps of a pair leave together and neither can be left waiting at a barrier.
                const uint32_t pair = (q & 1u) * 4u + wq;
                constexpr int kHalfGroups = B_ROWS / 32;       // groups of 8 token columns a warp takes (token tiles of at most B_ROWS)
                uint32_t gt[kHalfGroups][8];
                if (got) {
                    tc_fence_after();
#pragma unroll
                    for (int g = 0; g < kHalfGroups; ++g) {
                        const int c0 = (int(wq) + 4 * g) * 8;
                        if (c0 < tt.n_mma) tmem_ld8(t_acc + uint32_t(c0), gt[g]);
                    }
                    tmem_wait_ld();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&s.acc_empty[aset]);
                    if (q >= 2u) {
#pragma unroll
                        for (int g = 0; g < kHalfGroups; ++g) {
                            if ((int(wq) + 4 * g) * 8 >= tt.n_mma) break;
#pragma unroll
                            for (int j = 0; j < 8; ++j) s.xup[pair][g * 8 + j][lane] = gt[g][j];
                        }
                    }
                }
                if (named_bar_or(1u + pair, 64u, !got)) { ok = false; break; }
                if (q >= 2u) { named_bar_sync(1u + pair, 64u); continue; }
                uint32_t up[kHalfGroups][8];
#pragma unroll
                for (int g = 0; g < kHalfGroups; ++g) {
                    if ((int(wq) + 4 * g) * 8 >= tt.n_mma) break;
#pragma unroll
                    for (int j = 0; j < 8; ++j) up[g][j] = s.xup[pair][g * 8 + j][lane];
                }
                named_bar_sync(1u + pair, 64u);          // the up warp may overwrite its slots for the next item
                const int m_pair = wi.m_tile >> 1, half = wi.m_tile & 1;
                const int feat0 = m_pair * kTileM + half * (kTileM / 2) + int(q) * 32;
                uint8_t* sf_tile = p.mid_sf + (size_t(wi.tile) * (p.i_local / kChunkK) + m_pair) * kScaleBlockBytes;
                uint8_t* mq = p.mid_q + size_t(tt.row_base) * p.i_local + feat0 + lane;
                float* mf = DUMP ? p.mid_f32 + size_t(tt.row_base) * p.i_local + feat0 + lane : nullptr;
                uint32_t fault = 0;
#pragma unroll
                for (int g = 0; g < kHalfGroups; ++g) {
                    const int c0 = (int(wq) + 4 * g) * 8;
                    if (c0 >= tt.n_mma) break;
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
                        if (lane == 0) sf_tile[scale_block_offset(t, half * 2 + int(q))] = uint8_t(k + 127);
                    }
                }
                if (fault && lane == 0) atomicOr(p.fault, fault);
                continue;
            }
            if (!got) { ok = false; break; }
            tc_fence_after();
            if constexpr (MODE == kModeFc2) {
                // warp (q, wq): weight tile (wq & 1) of the pair, token groups (wq >> 1), +2, +4 ... of 8 tokens;
                // hidden row = 256 m + 128 tile + 32 q + lane
                const uint32_t tile = wq & 1u;
                uint32_t r[8][8];
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    const int c0 = (int(wq >> 1) + 2 * g) * 8;
                    if (c0 < tt.n_mma) tmem_ld8(t_acc + tile * kAcc1 + uint32_t(c0), r[g]);
                }
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s.acc_empty[aset]);
                const uint32_t ycol = uint32_t(wi.m_tile) * kPairM + tile * kTileM + q * 32u + lane;
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
                // token groups wq, wq + 4, wq + 8, wq + 12 of 8 tokens
                uint32_t gt[4][8], up[4][8];
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    const int c0 = (int(wq) + 4 * g) * 8;
                    if (c0 < tt.n_mma) {
                        tmem_ld8(t_acc + uint32_t(c0), gt[g]);
                        tmem_ld8(t_acc + kAcc1 + uint32_t(c0), up[g]);
                    }
                }
                tmem_wait_ld();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&s.acc_empty[aset]);
                const int feat0 = wi.m_tile * kTileM + int(q) * 32;
                uint8_t* sf_tile = p.mid_sf + (size_t(wi.tile) * (p.i_local / kChunkK) + wi.m_tile) * kScaleBlockBytes;
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
                        // a payload exponent is at most 8: payload * 2^k can only leave FP32 range when k > 119
                        if (k > 119 && __any_sync(0xffffffffu, !quant_v1_finite(code, k))) { fault |= kFaultQuantOverflow; continue; }
                        mq[size_t(t) * p.i_local] = uint8_t(code);
                        if (lane == 0) sf_tile[scale_block_offset(t, int(q))] = uint8_t(k + 127);
                    }
                }
                if (fault && lane == 0) atomicOr(p.fault, fault);
            }
          }
        }
        if (!ok && lane == 0) atomicOr(p.fault, uint32_t(kFaultPipeline));
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tb, kTmemCols);
}

}  // namespace m26b
