// Geometry of the routed-expert FFN and the device layouts shared by the
// planner, the repack kernels and the grouped GEMMs.
//
// Model constants follow the reference (crates/mimo26-repack/src/geom.rs:52-67):
// hidden 4096, expert intermediate 2048, 256 routed experts, top-8.
//
// Operand image of one layer on one tensor-parallel rank (I_local = 2048 / G):
//   w13  [E][I_local/128][256 rows][H/2 bytes]  rows 0..127 gate, 128..255 up of
//                                               the same 128 intermediate features
//   s13  [E][I_local/128][H/128][2][512 bytes]  scale blocks (see scale_block_offset):
//                                               block 0 the gate rows, block 1 the up rows
//   s13h [E][I_local/128][2][H/128][512 bytes]  the bytes of s13 regrouped for FC1's half items: block (tile, half h,
//                                               chunk) = gate rows 64 h .. 64 h + 63, then the up rows of the same features
//   w2   [E][H rows][I_local/2 bytes]           down_proj rows, this rank's K slice
//   s2   [E][H/256][I_local/128][2][512 bytes]  block b covers rows 256 t + 128 b + r
// A GEMM work item pairs two 128-row weight tiles (gate/up of the same
// features, or two consecutive down_proj row tiles) against one token tile:
// weights are 4-bit, so fetching more weight rows per token tile is the cheap
// way to raise arithmetic intensity on the L2 -> shared-memory path.
// Payload bytes keep the checkpoint's nibble order (low nibble = even k,
// crates/mimo26-expert/src/mxfp4.rs:20-22), which is also the order the TMA
// 4-bit unpack expects, so payload rows are copied, never re-nibbled.
#pragma once
#include <cstdint>

namespace m26b {

constexpr int kHidden = 4096;
constexpr int kInter = 2048;
constexpr int kExperts = 256;
constexpr int kTopK = 8;
constexpr int kBlockK = 32;            // one UE8M0 scale per 32 K elements
constexpr int kChunkK = 128;           // K elements per pipeline stage (4 MMA K-steps)
constexpr int kTileM = 128;            // weight rows per MMA (the tcgen05 M)
constexpr int kPairM = 256;            // weight rows per work item (two MMAs share the token tile)
constexpr int kMaxN = 128;             // largest token tile (the MMA N); two FP32 accumulators of N columns side by side
constexpr int kScaleBlockBytes = 512;  // 128 rows x 4 K32 blocks

// One 512-byte scale block covers 128 rows x 4 consecutive K32 blocks in the
// order tcgen05.cp.32x128b.warpx4 wants: row r, block kb -> this byte. After
// the copy, tensor-memory lane (r % 32), 32-bit column (r / 32), byte kb holds it.
__host__ __device__ constexpr int scale_block_offset(int row, int kb) {
    return (row % 32) * 16 + (row / 32) * 4 + kb;
}

// Per-layer expert table (256 x int16): which slot of the layer's weight image holds expert e, or kSlotNone. An
// expert-parallel rank may hold, besides its own block of the experts, copies of experts every rank holds
// ("replicated", flag kSlotReplicated): a route to such an expert is served by the rank that owns the route's token, so
// the rows of a popular expert spread over the ranks like the tokens do and never cross NVLink.
constexpr int kSlotNone = -1;
constexpr int kSlotReplicated = 0x4000;
constexpr int kSlotMask = 0x3fff;
// Does this rank serve a route of `token` (index inside the pass) to the expert with table entry `slot`?
// [own_lo, own_hi) = the tokens of the pass this rank owns.
__host__ __device__ inline bool slot_serves(int slot, uint32_t token, uint32_t own_lo, uint32_t own_hi) {
    return slot >= 0 && (!(slot & kSlotReplicated) || (token >= own_lo && token < own_hi));
}

// A run of routed rows of one expert that one MMA tile covers.
struct TokenTile {
    int32_t expert;     // the expert's slot in the layer's weight image
    int32_t row_base;   // first grouped (expert-sorted) route of the tile
    int32_t n_valid;    // routed rows in the tile
    int32_t n_mma;      // n_valid rounded up to a multiple of 16 (the MMA N)
};

// One unit of GEMM work: a token tile against one 256-row weight tile pair.
struct WorkItem {
    int32_t tile;
    int32_t m_tile;
};

// Launch classes: the host picks one from the token count alone (an expert
// can receive at most one route per token), so no device->host sync is needed.
struct LaunchClass {
    int max_n;     // largest token tile (MMA N) the planner will emit
    int b_rows;    // token rows of shared memory reserved per stage
    int stages;
};
// Measured on 64 uniform / 128 Zipf(1.2) tokens: {32, 6 stages} 0.501 / 0.189 ms per step, {64, 5} 0.511 / 0.183 ms,
// {128, 4} 0.540 / 0.189 ms: these steps stream weights, and what counts is how many stages of them are in flight.
__host__ __device__ constexpr LaunchClass launch_class(uint32_t tokens) {
    if (tokens <= 32) return LaunchClass{32, 32, 6};
    if (tokens <= 128) return LaunchClass{64, 64, 5};
    return LaunchClass{kMaxN, kMaxN, 4};
}

// Plan metadata written by the planner (one 32-byte record).
struct PlanMeta {
    uint32_t fault;       // 0 ok, 1 invalid route (id / residency / weight / duplicate)
    uint32_t n_tiles;
    uint32_t n_items_fc1;
    uint32_t n_items_fc2;
    uint32_t active_experts;
    uint32_t max_count;
    uint32_t pad[2];
};

// Numerical fault codes carried in the fault words (one word per stage).
enum : uint32_t {
    kFaultNone = 0,
    kFaultPlan = 1,
    kFaultInputScale = 2,     // activation scale byte outside 105..247 or NaN payload code
    kFaultPipeline = 3,       // a bounded wait in the GEMM pipeline ran out
    kFaultQuantNonfinite = 4, // intermediate quantizer: nonfinite input
    kFaultQuantOverflow = 5,  // intermediate quantizer: reconstruction overflow
    kFaultReduce = 8,         // route reduce: nonfinite weight / value / BF16 overflow
};

}  // namespace m26b
