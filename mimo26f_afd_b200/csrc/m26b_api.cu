// C ABI and host orchestration of the B200 routed-expert FFN.
// Declarations and the reference interfaces they replace: include/m26b_expert.h.
#include <cuda_runtime.h>
#include <cuda.h>
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../include/m26b_expert.h"
#include "layout.cuh"
#include "ffn_kernels.cuh"
#include "gemm_mx.cuh"
#include "gemm_mx_pair.cuh"
#include "prologue_small.cuh"
#include "ep_kernels.cuh"
#include "frame.inl"

using namespace m26b;

namespace {

constexpr uint32_t kMaxPassRows = 16384;   // token rows per pass of the pipeline (bounds scratch memory)

void set_err(char* err, size_t len, const char* what, cudaError_t e) {
    if (err && len) std::snprintf(err, len, "%s: %s", what, cudaGetErrorString(e));
}
void set_msg(char* err, size_t len, const char* msg) {
    if (err && len) std::snprintf(err, len, "%s", msg);
}

// Grow-only device buffer.
struct Dev {
    void* p = nullptr;
    size_t n = 0;
    cudaError_t ensure(size_t bytes, bool* grew = nullptr) {
        if (bytes <= n) return cudaSuccess;
        if (p) cudaFree(p);
        p = nullptr; n = 0;
        const size_t want = bytes < 256 ? 256 : bytes;
        const cudaError_t e = cudaMalloc(&p, want);
        if (e == cudaSuccess) { n = want; if (grew) *grew = true; }
        return e;
    }
    template <class T> T* as() const { return static_cast<T*>(p); }
    ~Dev() { if (p) cudaFree(p); }
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}
// 2-D K-major operand map: `cols` elements per row, 128-element x `box_rows` boxes, 128-byte swizzle.
bool make_map(CUtensorMap* m, bool fp4, void* base, uint64_t cols, uint64_t rows, uint64_t row_bytes, uint32_t box_rows) {
    EncodeTiledFn f = encode_fn();
    if (!f) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t es[2] = {1, 1};
    return f(m, fp4 ? CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, base, dims, strides, box,
             es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// The 4-bit FC1 weight image [rows][4096] seen as [blocks of 128 rows][128][4096] (blocks alternate gate / up) with boxes of
// 128 elements x 64 rows x 2 blocks: one copy brings the 64 gate rows and the 64 up rows of a half item's features.
bool make_map_half(CUtensorMap* m, void* base, uint64_t rows) {
    EncodeTiledFn f = encode_fn();
    if (!f) return false;
    cuuint64_t dims[3] = {uint64_t(kHidden), uint64_t(kTileM), rows / kTileM};
    cuuint64_t strides[2] = {uint64_t(kHidden) / 2, uint64_t(kTileM) * (kHidden / 2)};
    cuuint32_t box[3] = {128, kTileM / 2, 2};
    cuuint32_t es[3] = {1, 1, 1};
    return f(m, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, base, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Launch with the programmatic-serialization attribute: the kernel may be placed while the kernel before it in the
// stream drains, and orders itself with grid_dep_wait().
template <typename... P, typename... A>
cudaError_t launch_dependent(void (*kernel)(P...), unsigned grid, unsigned block, size_t smem, cudaStream_t st, A... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(block); cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute at{};
    at.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at.val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = &at; cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, P(args)...);
}

template <int MODE, int B_ROWS, int STAGES, bool DUMP, bool Y16, int A_TILES = 2>
cudaError_t launch_gemm(const CUtensorMap& mw, const TokenMaps& mx, const GemmArgs& a, int ctas, cudaStream_t st) {
    const int smem = int(sizeof(GemmSmem<B_ROWS, STAGES, A_TILES>)) + 1024;
    // the shared-memory opt-in is per kernel and per device: set once (one flag bit per device of this process)
    static std::atomic<uint64_t> opted{0};
    int dev = 0;
    cudaGetDevice(&dev);
    const uint64_t bit = 1ull << (dev & 63);
    if (!(opted.load(std::memory_order_relaxed) & bit)) {
        const cudaError_t e = cudaFuncSetAttribute(gemm_mx_kernel<MODE, B_ROWS, STAGES, DUMP, Y16, A_TILES>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return e;
        opted.fetch_or(bit, std::memory_order_relaxed);
    }
    return launch_dependent(gemm_mx_kernel<MODE, B_ROWS, STAGES, DUMP, Y16, A_TILES>, unsigned(ctas), kGemmThreads, size_t(smem), st, mw, mx, a);
}
// Scale blocks as a 2-D tensor of 128 x u32 rows (one 512-byte block per row), no swizzle.
bool make_sf_map(CUtensorMap* m, const void* base, uint64_t blocks, uint32_t box_rows) {
    EncodeTiledFn f = encode_fn();
    if (!f) return false;
    cuuint64_t dims[2] = {128, blocks};
    cuuint64_t strides[1] = {kScaleBlockBytes};
    cuuint32_t box[2] = {128, box_rows};
    cuuint32_t es[2] = {1, 1};
    return f(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void*>(base), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int MODE, bool DUMP, bool Y16>
cudaError_t launch_gemm_pair(const CUtensorMap& mw, const PairMaps& maps, const GemmArgs& a, int ctas, cudaStream_t st) {
    const int smem = int(sizeof(PairSmem)) + 1024;
    const cudaError_t e = cudaFuncSetAttribute(gemm_mx_pair_kernel<MODE, DUMP, Y16>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return e;
    return launch_dependent(gemm_mx_pair_kernel<MODE, DUMP, Y16>, unsigned(ctas & ~1), kPairThreads, size_t(smem), st, mw, maps, a);
}
cudaError_t launch_fc1_pair(bool dump, const CUtensorMap& mw, const PairMaps& maps, const GemmArgs& a, int ctas, cudaStream_t st) {
    return dump ? launch_gemm_pair<kModeFc1, true, false>(mw, maps, a, ctas, st) : launch_gemm_pair<kModeFc1, false, false>(mw, maps, a, ctas, st);
}
cudaError_t launch_fc2_pair(bool y16, const CUtensorMap& mw, const PairMaps& maps, const GemmArgs& a, int ctas, cudaStream_t st) {
    return y16 ? launch_gemm_pair<kModeFc2, false, true>(mw, maps, a, ctas, st) : launch_gemm_pair<kModeFc2, false, false>(mw, maps, a, ctas, st);
}

// How many CTAs of the pair kernels can be resident at once (2 x the co-resident clusters, at most one per SM).
// The kernels stride their work by the grid size, so a grid larger than this would run its tail as a second
// wave after the first has finished everything else. 0 if the device cannot place a single pair.
template <int MODE>
int pair_resident_ctas(int sms) {
    const int smem = int(sizeof(PairSmem)) + 1024;
    if (cudaFuncSetAttribute(gemm_mx_pair_kernel<MODE, false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(unsigned(sms & ~1));
    cfg.blockDim = dim3(kPairThreads);
    cfg.dynamicSmemBytes = size_t(smem);
    cudaLaunchAttribute at{};
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
    cfg.attrs = &at; cfg.numAttrs = 1;
    int clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&clusters, gemm_mx_pair_kernel<MODE, false, false>, &cfg) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    const int ctas = 2 * clusters;
    return ctas < (sms & ~1) ? ctas : (sms & ~1);
}

// Requests of at most this many tokens go up from the host in one copy (rows, scales, ids, weights packed into a
// pinned staging block) instead of three: a copy operation costs more than copying 70 KB on the host.
constexpr uint32_t kStageRows = 64;
constexpr size_t kStageBytes = size_t(kStageRows) * (kHidden + kHidden / kBlockK + kTopK * 8);

// Requests above this many tokens run the CTA-pair kernels (prefill); below, the single-CTA kernels (decode).
constexpr uint32_t kPairMinRows = 129;

// The single-CTA kernels by launch class; `variant` = the FP32 stage dump for FC1, BF16 route outputs for FC2.
template <int MODE, int B_ROWS, int STAGES>
cudaError_t launch_gemm_variant(bool variant, const CUtensorMap& mw, const TokenMaps& mx, const GemmArgs& a, int ctas, cudaStream_t st) {
    constexpr bool kFc1 = MODE == kModeFc1;
    return variant ? launch_gemm<MODE, B_ROWS, STAGES, kFc1, !kFc1>(mw, mx, a, ctas, st) : launch_gemm<MODE, B_ROWS, STAGES, false, false>(mw, mx, a, ctas, st);
}
template <int MODE>
cudaError_t launch_gemm_class(uint32_t rows, bool variant, const CUtensorMap& mw, const TokenMaps& mx, const GemmArgs& a, int ctas,
                              cudaStream_t st) {
    const LaunchClass lc = launch_class(rows);
    if (lc.b_rows == 32) return launch_gemm_variant<MODE, 32, 6>(variant, mw, mx, a, ctas, st);
    if (lc.b_rows == 64) return launch_gemm_variant<MODE, 64, 5>(variant, mw, mx, a, ctas, st);
    return launch_gemm_variant<MODE, kMaxN, 4>(variant, mw, mx, a, ctas, st);
}

// FC1 with half items (64 gate + 64 up rows per item): `mw` has 64-row boxes, a.sfa names the half-item scale image.
// Only the smallest launch class (at most 32 tokens) ever has few enough items for them to pay. Five stages of two K chunks.
cudaError_t launch_fc1_half(bool dump, const CUtensorMap& mw, const TokenMaps& mx, const GemmArgs& a, int ctas, cudaStream_t st) {
    return dump ? launch_gemm<kModeFc1, 32, 5, true, false, 1>(mw, mx, a, ctas, st) : launch_gemm<kModeFc1, 32, 5, false, false, 1>(mw, mx, a, ctas, st);
}

// Device status block of one pass: PlanMeta then four fault words.
struct Status {
    PlanMeta meta;
    uint32_t fault_input, fault_fc1, fault_fc2, fault_reduce;
    uint32_t pad[4];
};
static_assert(sizeof(Status) == 64, "status block is 64 bytes");

}  // namespace

struct m26b_layer {
    uint8_t *w13 = nullptr, *s13 = nullptr, *w2 = nullptr, *s2 = nullptr;
    uint8_t* s13h = nullptr;                    // the scale blocks of s13 regrouped for half items: [slot][tile][half][chunk][512]
    int16_t* slots = nullptr;                   // device, [256]: slot of each expert in the weight image (layout.cuh)
    int i_local = 0;
    uint32_t tp_rank = 0, tp_size = 1;
    int expert_lo = 0, n_local = kExperts;      // the rank's own experts: [expert_lo, expert_lo + n_local), slots 0 .. n_local - 1
    int n_rep = 0;                              // replicated experts held besides them, slots n_local .. n_local + n_rep - 1
    bool all_normal = false;
    int device = 0;
    CUtensorMap map_w13, map_w2, map_s13, map_s2;
    CUtensorMap map_w13h;                       // w13 with 64-row boxes (half items)
};

struct m26b_exchange {
    void* window = nullptr;
    ExchangePeers peers{};
    bool opened[8] = {false, false, false, false, false, false, false, false};
    int rank = 0, world = 1, device = 0, khz = 0;
    uint64_t plane_bytes = 0;
    uint32_t step = 0;                  // steps summed so far; the next step writes slot (step + 1) & 1
    long long wait_cycles = 0;
    PushLayout push{};                  // receive planes of the fused combine + exchange (small steps)
};

// Where a pass's combine goes when it is fused with the plane exchange of a tensor-parallel group.
struct PushSink {
    m26b_exchange* X;
    float* out;                         // FP32 rank-ordered sum (+ residual)
    const float* residual;
};

struct m26b_ep {
    void* window = nullptr;
    EpPeers peers{};
    EpLayout lay{};
    bool opened[8] = {false, false, false, false, false, false, false, false};
    int rank = 0, world = 1, device = 0, khz = 0;
    uint32_t tokens = 0;                 // tokens of a step, over all ranks
    uint32_t lo[9] = {0, 0, 0, 0, 0, 0, 0, 0, 0};   // token block of rank r: [lo[r], lo[r + 1])
    uint32_t step = 0;
    bool y16 = false;                    // result rows travel and are combined as BF16
    long long wait_cycles = 0;
    Dev ids, w;                          // every rank's routes, request order
    uint32_t* fault = nullptr;           // device word: quantiser / combine faults of the step
    uint32_t* hfault = nullptr;          // pinned copy
};

struct m26b_scratch {
    cudaStream_t st = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr, ea = nullptr, ec = nullptr;
    cudaEvent_t kev[7] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};   // per-kernel timing (debug bit 1)
    bool kev_quant = false, kev_valid = false;
    int device = 0, sms = 0;
    int pair_ctas = 0;          // resident CTAs of the pair kernels (0: the device cannot run them)
    uint32_t debug = 0;
    bool y16 = false;           // route outputs (FC2 rows) as BF16 instead of FP32
    Dev xq, xs, iw, dstage, inverse, original, gweights, experts, tiles, items1, items2, x_perm, sfb1, mid_q, mid_sf, mid_f32, y,
        partial, bf16, status, gather, plan_cnt, tp_sum;
    TokenMaps map_x, map_mid;
    PairMaps pair_x, pair_mid;
    void* pair_sfb1_base = nullptr; void* pair_midsf_base = nullptr; size_t pair_sfb1_n = 0, pair_midsf_n = 0;
    void* map_x_base = nullptr; void* map_mid_base = nullptr;
    uint64_t map_x_rows = 0, map_mid_rows = 0; int map_mid_cols = 0;
    uint8_t* hiw = nullptr; size_t hiw_n = 0;   // pinned, grow-only: ids and weights of a larger request
    uint8_t* hstage = nullptr;       // pinned: rows, scales, ids and weights of a small request, uploaded in one copy
    Status* hstatus = nullptr;       // pinned
    // last pass
    uint32_t last_rows = 0; int last_i_local = 0; bool pending = false; uint32_t n_status = 0; bool last_y16 = false;
    const int32_t* last_ids = nullptr; const uint8_t* last_xq = nullptr; const uint8_t* last_xs = nullptr;
};

namespace {

// Sources of a set of experts stacked in one group of six tensors.
struct ExpertSet {
    ProjSrc gate, up, down;
    int n;                    // experts in the set
};

// Repack `home` (the rank's own experts, ids expert_lo ..) and, for an expert-parallel rank, `rep` (copies of experts every
// rank holds, ids rep_ids[]) into one operand image: home in slots 0 .. n - 1, replicas behind them.
int prepare_layer(const ExpertSet& home, const ExpertSet* rep, const int32_t* rep_ids, uint32_t tp_rank, uint32_t tp_size,
                  m26b_layer** out, char* err, size_t errlen, int expert_lo = 0) {
    const int i_local = kInter / int(tp_size);
    // The repack kernels below run on the default stream and take no stream argument: whatever produced the source
    // tensors, on any stream of this device, is waited for here (this runs once per layer, off the serving path).
    {
        const cudaError_t se = cudaDeviceSynchronize();
        if (se != cudaSuccess) { set_err(err, errlen, "m26b layer: waiting for the source tensors", se); return 2; }
    }
    const int n_local = home.n, n_rep = rep ? rep->n : 0, n_slots = n_local + n_rep;
    int16_t table[kExperts];
    for (int e = 0; e < kExperts; ++e) table[e] = int16_t(kSlotNone);
    for (int i = 0; i < n_local; ++i) table[expert_lo + i] = int16_t(i);
    for (int i = 0; i < n_rep; ++i) {
        const int32_t e = rep_ids[i];
        if (e < 0 || e >= kExperts || (table[e] != kSlotNone && (table[e] & kSlotReplicated))) {
            set_msg(err, errlen, "m26b layer: bad or repeated replicated expert id");
            return 1;
        }
        // an expert of the rank's own block that is also replicated keeps one copy: the replica's slot
        table[e] = int16_t((n_local + i) | kSlotReplicated);
    }
    auto* L = new m26b_layer();
    L->i_local = i_local; L->tp_rank = tp_rank; L->tp_size = tp_size;
    L->expert_lo = expert_lo; L->n_local = n_local; L->n_rep = n_rep;
    cudaGetDevice(&L->device);
    const size_t w13_e = size_t(2) * i_local * (kHidden / 2), s13_e = size_t(2) * i_local * (kHidden / kBlockK);
    const size_t w2_e = size_t(kHidden) * (i_local / 2), s2_e = size_t(kHidden) * (i_local / kBlockK);
    const size_t w13_bytes = n_slots * w13_e, s13_bytes = n_slots * s13_e, w2_bytes = n_slots * w2_e, s2_bytes = n_slots * s2_e;
    cudaError_t e;
    uint32_t* flag = nullptr;
    auto fail = [&](const char* what, cudaError_t ce, int rc) {
        set_err(err, errlen, what, ce);
        if (flag) cudaFree(flag);
        m26b_layer_free(L);
        return rc;
    };
    if ((e = cudaMalloc(&L->w13, w13_bytes)) != cudaSuccess || (e = cudaMalloc(&L->s13, s13_bytes)) != cudaSuccess ||
        (e = cudaMalloc(&L->s13h, s13_bytes)) != cudaSuccess ||
        (e = cudaMalloc(&L->w2, w2_bytes)) != cudaSuccess || (e = cudaMalloc(&L->s2, s2_bytes)) != cudaSuccess ||
        (e = cudaMalloc(&L->slots, sizeof table)) != cudaSuccess || (e = cudaMalloc(&flag, 4)) != cudaSuccess)
        return fail("m26b layer alloc", e, 2);
    if ((e = cudaMemset(flag, 0, 4)) != cudaSuccess || (e = cudaMemcpy(L->slots, table, sizeof table, cudaMemcpyHostToDevice)) != cudaSuccess)
        return fail("m26b layer metadata", e, 2);
    const ExpertSet* sets[2] = {&home, rep};
    for (int k = 0; k < 2; ++k) {
        if (!sets[k] || sets[k]->n == 0) continue;
        const ExpertSet& src = *sets[k];
        const size_t first = k == 0 ? 0 : size_t(n_local);
        prep_w13_kernel<<<2048, 256>>>(src.gate, src.up, i_local, L->w13 + first * w13_e, src.n);
        prep_s13_kernel<<<2048, 256>>>(src.gate, src.up, i_local, L->s13 + first * s13_e, flag, src.n);
        prep_w2_kernel<<<2048, 256>>>(src.down, i_local, L->w2 + first * w2_e, src.n);
        prep_s2_kernel<<<2048, 256>>>(src.down, i_local, L->s2 + first * s2_e, flag, src.n);
    }
    prep_s13_half_kernel<<<2048, 256>>>(L->s13, i_local, L->s13h, n_slots);
    uint32_t h = 1;
    if ((e = cudaGetLastError()) != cudaSuccess || (e = cudaMemcpy(&h, flag, 4, cudaMemcpyDeviceToHost)) != cudaSuccess ||
        (e = cudaDeviceSynchronize()) != cudaSuccess)
        return fail("m26b layer prepare", e, 2);
    cudaFree(flag); flag = nullptr;
    L->all_normal = h == 0;
    if (!make_map(&L->map_w13, true, L->w13, kHidden, uint64_t(n_slots) * 2 * i_local, kHidden / 2, kPairM) ||
        !make_map_half(&L->map_w13h, L->w13, uint64_t(n_slots) * 2 * i_local) ||
        !make_map(&L->map_w2, true, L->w2, uint64_t(i_local), uint64_t(n_slots) * kHidden, uint64_t(i_local) / 2, kPairM)) {
        set_msg(err, errlen, "m26b layer: cuTensorMapEncodeTiled failed for the weight operands");
        m26b_layer_free(L);
        return 2;
    }
    if (!make_sf_map(&L->map_s13, L->s13, s13_bytes / kScaleBlockBytes, 2) ||
        !make_sf_map(&L->map_s2, L->s2, s2_bytes / kScaleBlockBytes, 2)) {
        set_msg(err, errlen, "m26b layer: cuTensorMapEncodeTiled failed for the weight scales");
        m26b_layer_free(L);
        return 2;
    }
    *out = L;
    return 0;
}

// The six checkpoint tensors stacked over `n` experts, as repack sources for a tensor-parallel slice.
ExpertSet checkpoint_set(const uint8_t* gate_w, const uint8_t* gate_s, const uint8_t* up_w, const uint8_t* up_s, const uint8_t* down_w,
                         const uint8_t* down_s, uint32_t tp_rank, uint32_t tp_size, int n) {
    const uint64_t il = kInter / tp_size;
    ExpertSet s{};
    s.n = n;
    s.gate.payload = gate_w; s.gate.scales = gate_s;
    s.gate.expert_stride_p = uint64_t(kInter) * (kHidden / 2); s.gate.expert_stride_s = uint64_t(kInter) * (kHidden / kBlockK);
    s.gate.row_stride_p = kHidden / 2; s.gate.row_stride_s = kHidden / kBlockK;
    s.gate.row0 = il * tp_rank;
    s.up = s.gate; s.up.payload = up_w; s.up.scales = up_s;
    s.down.payload = down_w; s.down.scales = down_s;
    s.down.expert_stride_p = uint64_t(kHidden) * (kInter / 2); s.down.expert_stride_s = uint64_t(kHidden) * (kInter / kBlockK);
    s.down.row_stride_p = kInter / 2; s.down.row_stride_s = kInter / kBlockK;
    s.down.col0_p = il * tp_rank / 2; s.down.col0_s = il * tp_rank / kBlockK;
    return s;
}

ProjSrc canonical_proj(const uint8_t* base, uint64_t image, uint64_t payload_off, uint64_t scale_off, uint64_t in_cols) {
    ProjSrc s{};
    s.payload = base + payload_off; s.scales = base + scale_off;
    s.expert_stride_p = s.expert_stride_s = image;
    s.row_stride_p = in_cols / 2; s.row_stride_s = in_cols / kBlockK;
    return s;
}

#define M26B_CK(expr, what) do { if ((e = (expr)) != cudaSuccess) { set_err(err, errlen, what, e); return 2; } } while (0)

// Buffers of one pass of `rows` tokens on a layer of width i_local.
int ensure_pass(m26b_scratch* S, uint32_t rows, int i_local, bool own_input, char* err, size_t errlen) {
    cudaError_t e;
    const size_t routes = size_t(rows) * kTopK;
    const LaunchClass lc = launch_class(rows);
    const size_t tiles_max = routes / lc.max_n + kExperts;
    const size_t rows_cap = routes + 256;
    if (own_input) {
        M26B_CK(S->xq.ensure(size_t(rows) * kHidden), "m26b x alloc");
        M26B_CK(S->xs.ensure(size_t(rows) * (kHidden / kBlockK)), "m26b xs alloc");
    }
    M26B_CK(S->inverse.ensure(routes * 4), "m26b inverse alloc");
    M26B_CK(S->original.ensure(routes * 4), "m26b original alloc");
    M26B_CK(S->gweights.ensure(routes * 4), "m26b gweights alloc");
    M26B_CK(S->experts.ensure(kExperts * sizeof(ExpertPlan)), "m26b experts alloc");
    M26B_CK(S->tiles.ensure(tiles_max * sizeof(TokenTile)), "m26b tiles alloc");
    M26B_CK(S->items1.ensure(tiles_max * (i_local / kTileM) * 2 * sizeof(WorkItem)), "m26b fc1 items alloc");   // x 2: half items
    M26B_CK(S->items2.ensure(tiles_max * (kHidden / kPairM) * sizeof(WorkItem)), "m26b fc2 items alloc");
    M26B_CK(S->sfb1.ensure(tiles_max * (kHidden / kChunkK) * kScaleBlockBytes), "m26b sfb alloc");
    M26B_CK(S->mid_sf.ensure(tiles_max * (i_local / kChunkK) * kScaleBlockBytes), "m26b mid scale alloc");
    if (S->debug & 1u) M26B_CK(S->mid_f32.ensure(rows_cap * i_local * 4), "m26b mid f32 alloc");
    M26B_CK(S->y.ensure(routes * kHidden * 4), "m26b y alloc");
    M26B_CK(S->partial.ensure(size_t(rows) * kHidden * 4), "m26b partial alloc");
    M26B_CK(S->bf16.ensure(size_t(rows) * kHidden * 2), "m26b bf16 alloc");
    M26B_CK(S->status.ensure(sizeof(Status) * 64), "m26b status alloc");
    M26B_CK(S->plan_cnt.ensure(128 * kExperts * 4), "m26b plan counts alloc");
    M26B_CK(S->x_perm.ensure(rows_cap * kHidden), "m26b x_perm alloc");
    M26B_CK(S->mid_q.ensure(rows_cap * i_local), "m26b mid alloc");
    const uint64_t xr = S->x_perm.n / kHidden, mr = S->mid_q.n / i_local;
    if (S->map_x_base != S->x_perm.p || S->map_x_rows != xr) {
        for (int i = 0; i < 4; ++i)
            if (!make_map(&S->map_x.box[i], false, S->x_perm.p, kHidden, xr, kHidden, 128u >> i)) {
                set_msg(err, errlen, "m26b: cuTensorMapEncodeTiled failed for the token operand");
                return 2;
            }
        for (int i = 0; i < 5; ++i)
            if (!make_map(&S->pair_x.tok[i], false, S->x_perm.p, kHidden, xr, kHidden, 128u >> i)) {
                set_msg(err, errlen, "m26b: cuTensorMapEncodeTiled failed for the token operand");
                return 2;
            }
        S->map_x_base = S->x_perm.p; S->map_x_rows = xr;
    }
    if (S->map_mid_base != S->mid_q.p || S->map_mid_rows != mr || S->map_mid_cols != i_local) {
        for (int i = 0; i < 4; ++i)
            if (!make_map(&S->map_mid.box[i], false, S->mid_q.p, uint64_t(i_local), mr, uint64_t(i_local), 128u >> i)) {
                set_msg(err, errlen, "m26b: cuTensorMapEncodeTiled failed for the intermediate operand");
                return 2;
            }
        for (int i = 0; i < 5; ++i)
            if (!make_map(&S->pair_mid.tok[i], false, S->mid_q.p, uint64_t(i_local), mr, uint64_t(i_local), 128u >> i)) {
                set_msg(err, errlen, "m26b: cuTensorMapEncodeTiled failed for the intermediate operand");
                return 2;
            }
        S->map_mid_base = S->mid_q.p; S->map_mid_rows = mr; S->map_mid_cols = i_local;
    }
    if (S->pair_sfb1_base != S->sfb1.p || S->pair_sfb1_n != S->sfb1.n) {
        if (!make_sf_map(&S->pair_x.sfb, S->sfb1.p, S->sfb1.n / kScaleBlockBytes, 1)) {
            set_msg(err, errlen, "m26b: cuTensorMapEncodeTiled failed for the token scales");
            return 2;
        }
        S->pair_sfb1_base = S->sfb1.p; S->pair_sfb1_n = S->sfb1.n;
    }
    if (S->pair_midsf_base != S->mid_sf.p || S->pair_midsf_n != S->mid_sf.n) {
        if (!make_sf_map(&S->pair_mid.sfb, S->mid_sf.p, S->mid_sf.n / kScaleBlockBytes, 1)) {
            set_msg(err, errlen, "m26b: cuTensorMapEncodeTiled failed for the intermediate scales");
            return 2;
        }
        S->pair_midsf_base = S->mid_sf.p; S->pair_midsf_n = S->mid_sf.n;
    }
    return 0;
}

// Activations that are not quantised yet: requests of at most kMediumRows tokens quantise inside the fused prologue,
// larger ones inside the permutation pass.
struct RawInput {
    const void* x;
    int dtype, codec;          // 0 BF16 / 1 FP32; 0 wire / 1 quant_v1
    uint32_t* fault_quant;
};

template <int CODEC, int IN>
void launch_small_prologue(uint32_t sms, cudaStream_t st, const SmallIo& io, const int32_t* ids, const float* w, uint32_t rows,
                           const int16_t* resident, int max_n, int mt1, int mt2, int span2, const PlanOut& po) {
    const uint32_t routes = rows * kTopK;
    if (rows <= kSmallRows) {
        small_prologue_kernel<CODEC, IN, 256><<<routes < sms ? routes : sms, 256, 0, st>>>(io, ids, w, rows, resident, max_n, mt1, mt2, span2, po);
    } else {
        const uint32_t need = (routes + 3u) / 4u;          // four rows side by side per CTA
        small_prologue_kernel<CODEC, IN, 1024><<<need < sms ? need : sms, 1024, 0, st>>>(io, ids, w, rows, resident, max_n, mt1, mt2, span2, po);
    }
}

// Half items for FC1 of a decode-sized pass? The host knows the token count, not the plan: it estimates the token tiles as
// one per routed expert (at most 256, at most one per route). Half items pay when full items would not fill four rounds
// of the SMs. Measured on one GPU, FC1 between events / whole step of a rank, full -> half items: 16 tokens on a rank of
// eight (204 full items for 148 SMs) 38.9 -> 35.9 / 66.6 -> 62.5 us, 4 tokens there 21.5 -> 17.4 / 42.0 -> 35.8 us, 32 tokens
// there 52.3 -> 50.2 / 89.1 -> 87.0 us, 4 tokens on one GPU 66.6 -> 64.5 / 105.5 -> 103.4 us; with more items the better
// spread no longer pays for the extra item hand-overs (16 tokens on one GPU, 1,632 full items: 158.8 -> 160.8 / 248.8 -> 250.9 us).
bool fc1_half_items(uint32_t rows, int mt1, int sms) {
    const uint32_t routes = rows * kTopK, tiles = routes < uint32_t(kExperts) ? routes : uint32_t(kExperts);
    return tiles * uint32_t(mt1) < 4u * uint32_t(sms);
}

// A pass of an expert-parallel step: where the pass's token rows live and where its FC2 rows go.
struct EpPass {
    TokenSources src;
    RouteSinks sinks;
    bool y16;
    uint32_t own_lo, own_hi;      // the tokens of the pass this rank owns (routes to replicated experts are served by the owner)
};

// Enqueue one pass: plan -> permute -> FC1 (+SwiGLU, quantiser) -> FC2 -> combine. `raw` names activations still to be
// quantised into xq / xs (not with expert parallelism); `status_cleared`: the caller has already zeroed the status
// block on the stream.
int enqueue_pass(const m26b_layer* L, m26b_scratch* S, const uint8_t* xq, const uint8_t* xs, const int32_t* ids,
                 const float* w, uint32_t rows, uint16_t* bf16_out, float* partial_out, Status* status,
                 cudaStream_t st, bool events, char* err, size_t errlen, const RawInput* raw = nullptr,
                 bool status_cleared = false, const EpPass* ep = nullptr, const PushSink* push = nullptr) {
    cudaError_t e;
    const uint32_t routes = rows * kTopK;
    const LaunchClass lc = launch_class(rows);
    const int mt1 = L->i_local / kTileM, mt2 = kHidden / kPairM;
    if (!status_cleared) M26B_CK(cudaMemsetAsync(status, 0, sizeof(Status), st), "m26b status clear");
    if (events) M26B_CK(cudaEventRecord(S->e0, st), "m26b event 0");
    PlanOut po{S->inverse.as<int32_t>(), S->original.as<int32_t>(), S->gweights.as<float>(), S->experts.as<ExpertPlan>(),
               S->tiles.as<TokenTile>(), S->items1.as<WorkItem>(), S->items2.as<WorkItem>(), &status->meta};
    const bool pair = rows >= kPairMinRows && (mt1 % 2 == 0) && S->pair_ctas >= S->sms / 2;
    const bool dump = (S->debug & 1u) != 0;
    const bool y16 = ep ? ep->y16 : S->y16;
    // FC2 items of the single-CTA kernel span several weight tile pairs when a rank's K slice is short (tensor parallelism:
    // 2 or 4 chunks): the item's records and output-row addresses are then fetched once per 8 chunks of work, not per 2
    const int k2 = L->i_local / kChunkK;
    const int span2 = pair ? 1 : (k2 >= 8 ? 1 : k2 >= 4 ? 2 : 4);
    const int m_step1 = pair ? 2 : 1, m_step2 = pair ? 2 : span2;
    // FC1 of a decode-sized pass: half items (twice as many, half as long) when full items would leave the SMs a ragged
    // last round
    const bool half1 = !pair && rows <= 32 && fc1_half_items(rows, mt1, S->sms);
    const int mt1_plan = half1 ? 2 * mt1 : mt1;
    const bool kt = (S->debug & 2u) != 0;
    if (kt) M26B_CK(cudaEventRecord(S->kev[1], st), "m26b event");
    const PlanScope scope{L->slots, ep ? ep->own_lo : 0u, ep ? ep->own_hi : rows, ep ? 1 : 0};
    const TokenSources src = ep ? ep->src : TokenSources{};
    if (rows <= kMediumRows && !ep) {
        // one launch: plan + (quantise) + gate + permutation; timed as the permutation, the plan slot reads zero
        if (kt) M26B_CK(cudaEventRecord(S->kev[2], st), "m26b event");
        SmallIo io{};
        io.x = raw ? raw->x : xq; io.xs_in = xs;
        io.xq_out = raw ? const_cast<uint8_t*>(xq) : nullptr; io.xs_out = raw ? const_cast<uint8_t*>(xs) : nullptr;
        io.x_perm = S->x_perm.as<uint8_t>(); io.sfb = S->sfb1.as<uint8_t>();
        io.fault_input = &status->fault_input; io.fault_quant = raw ? raw->fault_quant : nullptr;
        const uint32_t grid = uint32_t(S->sms);
        const int sel = raw ? raw->codec * 2 + raw->dtype : 4;
        switch (sel) {
            case 0: launch_small_prologue<0, 0>(grid, st, io, ids, w, rows, L->slots, lc.max_n, mt1_plan, mt2, span2, po); break;
            case 1: launch_small_prologue<0, 1>(grid, st, io, ids, w, rows, L->slots, lc.max_n, mt1_plan, mt2, span2, po); break;
            case 2: launch_small_prologue<1, 0>(grid, st, io, ids, w, rows, L->slots, lc.max_n, mt1_plan, mt2, span2, po); break;
            case 3: launch_small_prologue<1, 1>(grid, st, io, ids, w, rows, L->slots, lc.max_n, mt1_plan, mt2, span2, po); break;
            default: launch_small_prologue<0, 2>(grid, st, io, ids, w, rows, L->slots, lc.max_n, mt1_plan, mt2, span2, po); break;
        }
        M26B_CK(cudaGetLastError(), "m26b prologue launch");
    } else {
        if (routes <= 4096) {
            plan_kernel<<<1, 1024, 0, st>>>(ids, w, rows, scope, lc.max_n, mt1_plan, mt2, m_step1, m_step2, po);
        } else {
            // each CTA takes a whole number of 1024-route slabs, so every warp segment is a multiple of 32
            const uint32_t slabs = (routes + 1023u) / 1024u;
            const uint32_t n_cta = slabs < 128u ? slabs : 128u;
            const uint32_t cta_routes = ((slabs + n_cta - 1u) / n_cta) * 1024u;
            uint32_t* cta_cnt = S->plan_cnt.as<uint32_t>();
            plan_count_kernel<<<n_cta, 1024, 0, st>>>(ids, w, rows, scope, cta_routes, cta_cnt, &status->meta);
            plan_scan_kernel<<<1, 1024, 0, st>>>(n_cta, cta_cnt, lc.max_n, mt1_plan, mt2, m_step1, m_step2, L->slots, po);
            plan_place_kernel<<<n_cta, 1024, 0, st>>>(ids, w, rows, cta_routes, cta_cnt, po, scope);
        }
        M26B_CK(cudaGetLastError(), "m26b plan launch");
        if (kt) M26B_CK(cudaEventRecord(S->kev[2], st), "m26b event");
        if (raw) {
            // activations still to be quantised: quantiser and permutation in one pass over the rows
            uint8_t* xq_w = const_cast<uint8_t*>(xq);
            uint8_t* xs_w = const_cast<uint8_t*>(xs);
            const int32_t* inv = S->inverse.as<int32_t>();
            const ExpertPlan* ex = S->experts.as<ExpertPlan>();
            uint8_t* xp = S->x_perm.as<uint8_t>();
            uint8_t* sf = S->sfb1.as<uint8_t>();
            switch (raw->codec * 2 + raw->dtype) {
                case 0: quantize_permute_kernel<0, uint16_t><<<rows, 256, 0, st>>>(static_cast<const uint16_t*>(raw->x), rows, ids, inv, ex, &status->meta, xq_w, xs_w, xp, sf, raw->fault_quant, &status->fault_input); break;
                case 1: quantize_permute_kernel<0, float><<<rows, 256, 0, st>>>(static_cast<const float*>(raw->x), rows, ids, inv, ex, &status->meta, xq_w, xs_w, xp, sf, raw->fault_quant, &status->fault_input); break;
                case 2: quantize_permute_kernel<1, uint16_t><<<rows, 256, 0, st>>>(static_cast<const uint16_t*>(raw->x), rows, ids, inv, ex, &status->meta, xq_w, xs_w, xp, sf, raw->fault_quant, &status->fault_input); break;
                default: quantize_permute_kernel<1, float><<<rows, 256, 0, st>>>(static_cast<const float*>(raw->x), rows, ids, inv, ex, &status->meta, xq_w, xs_w, xp, sf, raw->fault_quant, &status->fault_input); break;
            }
            M26B_CK(cudaGetLastError(), "m26b quantise+permute launch");
        } else {
            permute_kernel<<<routes < 65535u * 8u ? routes : 65535u * 8u, 256, 0, st>>>(
                xq, xs, ids, S->original.as<int32_t>(), S->experts.as<ExpertPlan>(), &status->meta, routes,
                S->x_perm.as<uint8_t>(), S->sfb1.as<uint8_t>(), &status->fault_input, src);
            M26B_CK(cudaGetLastError(), "m26b permute launch");
        }
    }
    if (kt) M26B_CK(cudaEventRecord(S->kev[3], st), "m26b event");
    GemmArgs a{};
    a.tiles = S->tiles.as<TokenTile>();
    a.i_local = L->i_local;
    a.mid_q = S->mid_q.as<uint8_t>();
    a.mid_sf = S->mid_sf.as<uint8_t>();
    a.mid_f32 = dump ? S->mid_f32.as<float>() : nullptr;
    a.y = S->y.as<float>();
    a.original_routes = S->original.as<int32_t>();
    if (ep) a.sinks = ep->sinks;
    // FC1: weights w13 (K = hidden), tokens x_perm
    a.items = S->items1.as<WorkItem>(); a.n_items = &status->meta.n_items_fc1;
    a.sfa = L->s13; a.sfb = S->sfb1.as<uint8_t>(); a.m_tiles = mt1; a.k_chunks = kHidden / kChunkK; a.m_span = 1;
    a.fault = &status->fault_fc1;
    if (pair) {
        PairMaps pm = S->pair_x;
        pm.sfa = L->map_s13;
        M26B_CK(launch_fc1_pair(dump, L->map_w13, pm, a, S->pair_ctas, st), "m26b fc1 launch");
    } else if (half1) {
        a.sfa = L->s13h;
        M26B_CK(launch_fc1_half(dump, L->map_w13h, S->map_x, a, S->sms, st), "m26b fc1 launch");
    } else {
        M26B_CK(launch_gemm_class<kModeFc1>(rows, dump, L->map_w13, S->map_x, a, S->sms, st), "m26b fc1 launch");
    }
    const bool stage_events = events && (S->debug & 4u) != 0;    // events between the kernels cost their overlap
    if (stage_events) M26B_CK(cudaEventRecord(S->ea, st), "m26b event a");
    if (kt) M26B_CK(cudaEventRecord(S->kev[4], st), "m26b event");
    // FC2: weights w2 (K = i_local), tokens mid_q
    a.items = S->items2.as<WorkItem>(); a.n_items = &status->meta.n_items_fc2;
    a.sfa = L->s2; a.sfb = S->mid_sf.as<uint8_t>(); a.m_tiles = mt2; a.k_chunks = L->i_local / kChunkK; a.m_span = span2;
    a.fault = &status->fault_fc2;
    if (pair) {
        PairMaps pm = S->pair_mid;
        pm.sfa = L->map_s2;
        M26B_CK(launch_fc2_pair(y16, L->map_w2, pm, a, S->pair_ctas, st), "m26b fc2 launch");
    } else {
        M26B_CK(launch_gemm_class<kModeFc2>(rows, y16, L->map_w2, S->map_mid, a, S->sms, st), "m26b fc2 launch");
    }
    if (stage_events) M26B_CK(cudaEventRecord(S->ec, st), "m26b event c");
    if (kt) M26B_CK(cudaEventRecord(S->kev[5], st), "m26b event");
    if (push) {
        // combine, push into every rank's window, add the peers' chunks: one kernel, one step of the exchange
        m26b_exchange* X = push->X;
        X->step += 1;
        const uint32_t chunks = rows * (kHidden / 1024);
        const uint32_t blocks = chunks < uint32_t(S->sms) * 4u ? chunks : uint32_t(S->sms) * 4u;
        if (y16)
            M26B_CK(launch_dependent(reduce_exchange_kernel<true>, blocks, 256u, size_t(0), st, static_cast<const void*>(S->y.p), w, rows,
                                     X->peers, X->push, X->rank, X->world, X->step, X->wait_cycles, push->out, push->residual,
                                     &status->fault_reduce), "m26b reduce+exchange launch");
        else
            M26B_CK(launch_dependent(reduce_exchange_kernel<false>, blocks, 256u, size_t(0), st, static_cast<const void*>(S->y.p), w, rows,
                                     X->peers, X->push, X->rank, X->world, X->step, X->wait_cycles, push->out, push->residual,
                                     &status->fault_reduce), "m26b reduce+exchange launch");
    } else if (!ep) {   // an expert-parallel pass leaves its rows with the tokens' owners; they combine after the step's rendezvous
        if (y16) {
            const uint64_t n8 = uint64_t(rows) * (kHidden / 8);
            const uint32_t blocks = uint32_t(n8 / 256 + 1 < 16384 ? n8 / 256 + 1 : 16384);
            M26B_CK(launch_dependent(route_reduce_y16_kernel, blocks, 256u, size_t(0), st, static_cast<const uint16_t*>(S->y.as<uint16_t>()), w,
                                     rows, partial_out, bf16_out, &status->fault_reduce), "m26b reduce launch");
        } else {
            const uint64_t n4 = uint64_t(rows) * (kHidden / 4);
            const uint32_t blocks = uint32_t(n4 / 256 + 1 < 16384 ? n4 / 256 + 1 : 16384);
            M26B_CK(launch_dependent(route_reduce_kernel, blocks, 256u, size_t(0), st, static_cast<const float*>(S->y.as<float>()), w,
                                     rows, partial_out, bf16_out, &status->fault_reduce), "m26b reduce launch");
        }
    }
    if (events) M26B_CK(cudaEventRecord(S->e1, st), "m26b event 1");
    if (kt) { M26B_CK(cudaEventRecord(S->kev[6], st), "m26b event"); S->kev_valid = true; }
    S->last_y16 = y16;
    S->last_rows = rows; S->last_i_local = L->i_local; S->last_ids = ids; S->last_xq = xq; S->last_xs = xs;
    return 0;
}

// Host request -> device, on the scratch's stream: rows, scales, ids and weights. Requests of at most kStageRows tokens
// are packed into one pinned block and go up in one copy; larger ones in three copies (contiguous rows as linear
// copies), with ids and weights staged through pinned memory so that no copy falls back to the synchronous pageable path.
int upload_request(m26b_scratch* S, const uint8_t* payload, size_t payload_pitch, const uint8_t* scales, size_t scales_pitch,
                   const int32_t* ids, const float* weights, uint32_t rows, const uint8_t** xq_out, const uint8_t** xs_out,
                   const int32_t** ids_out, const float** w_out, char* err, size_t errlen) {
    cudaError_t e;
    const size_t routes = size_t(rows) * kTopK;
    const uint8_t* xq_d;
    const uint8_t* xs_d;
    const int32_t* ids_d;
    const float* w_d;
    if (rows <= kStageRows) {
        M26B_CK(S->dstage.ensure(kStageBytes), "m26b staging alloc");
        const size_t o_s = size_t(rows) * kHidden, o_i = o_s + size_t(rows) * (kHidden / kBlockK), o_w = o_i + routes * 4;
        for (uint32_t r = 0; r < rows; ++r) {
            std::memcpy(S->hstage + size_t(r) * kHidden, payload + size_t(r) * payload_pitch, kHidden);
            std::memcpy(S->hstage + o_s + size_t(r) * (kHidden / kBlockK), scales + size_t(r) * scales_pitch, kHidden / kBlockK);
        }
        std::memcpy(S->hstage + o_i, ids, routes * 4);
        std::memcpy(S->hstage + o_w, weights, routes * 4);
        M26B_CK(cudaMemcpyAsync(S->dstage.p, S->hstage, o_w + routes * 4, cudaMemcpyHostToDevice, S->st), "m26b request upload");
        xq_d = S->dstage.as<uint8_t>(); xs_d = xq_d + o_s;
        ids_d = reinterpret_cast<const int32_t*>(xq_d + o_i); w_d = reinterpret_cast<const float*>(xq_d + o_w);
    } else {
        M26B_CK(S->xq.ensure(size_t(rows) * kHidden), "m26b x alloc");
        M26B_CK(S->xs.ensure(size_t(rows) * (kHidden / kBlockK)), "m26b xs alloc");
        M26B_CK(S->iw.ensure(routes * 8), "m26b ids/w alloc");
        // contiguous rows go up as one linear copy (a pitched copy of the same bytes takes a slower path)
        if (payload_pitch == kHidden)
            M26B_CK(cudaMemcpyAsync(S->xq.p, payload, size_t(rows) * kHidden, cudaMemcpyHostToDevice, S->st), "m26b x upload");
        else
            M26B_CK(cudaMemcpy2DAsync(S->xq.p, kHidden, payload, payload_pitch, kHidden, rows, cudaMemcpyHostToDevice, S->st),
                    "m26b x upload");
        if (scales_pitch == kHidden / kBlockK)
            M26B_CK(cudaMemcpyAsync(S->xs.p, scales, size_t(rows) * (kHidden / kBlockK), cudaMemcpyHostToDevice, S->st), "m26b xs upload");
        else
            M26B_CK(cudaMemcpy2DAsync(S->xs.p, kHidden / kBlockK, scales, scales_pitch, kHidden / kBlockK, rows,
                                      cudaMemcpyHostToDevice, S->st), "m26b xs upload");
        if (S->hiw_n < routes * 8) {
            // the previous request's copy out of this block has finished: every host entry point ends with a stream sync
            if (S->hiw) cudaFreeHost(S->hiw);
            S->hiw = nullptr; S->hiw_n = 0;
            M26B_CK(cudaMallocHost(reinterpret_cast<void**>(&S->hiw), routes * 8), "m26b ids/w staging alloc");
            S->hiw_n = routes * 8;
        }
        std::memcpy(S->hiw, ids, routes * 4);
        std::memcpy(S->hiw + routes * 4, weights, routes * 4);
        M26B_CK(cudaMemcpyAsync(S->iw.p, S->hiw, routes * 8, cudaMemcpyHostToDevice, S->st), "m26b ids/w upload");
        xq_d = S->xq.as<uint8_t>(); xs_d = S->xs.as<uint8_t>();
        ids_d = S->iw.as<int32_t>(); w_d = reinterpret_cast<const float*>(S->iw.as<uint8_t>() + routes * 4);
    }
    *xq_out = xq_d; *xs_out = xs_d; *ids_out = ids_d; *w_out = w_d;
    return 0;
}

int decode_status(const Status* hs, uint32_t n, char* err, size_t errlen) {
    for (uint32_t i = 0; i < n; ++i) {
        const Status& s = hs[i];
        if (s.meta.fault) { set_msg(err, errlen, "m26b plan: invalid routes (id/residency/weight/duplicate)"); return 3; }
    }
    for (uint32_t i = 0; i < n; ++i) {
        const Status& s = hs[i];
        const uint32_t words[4] = {s.fault_input, s.fault_fc1, s.fault_fc2, s.fault_reduce};
        const char* names[4] = {"input", "fc1/quantizer", "fc2", "reduce"};
        for (int k = 0; k < 4; ++k)
            if (words[k]) {
                if (err && errlen) std::snprintf(err, errlen, "m26b %s fault %u (pass %u, tiles %u)", names[k], words[k], i, s.meta.n_tiles);
                return 4;
            }
    }
    return 0;
}

bool device_ok(int dev_of_handle, char* err, size_t errlen) {
    int d = -1;
    if (cudaGetDevice(&d) != cudaSuccess || d != dev_of_handle) {
        set_msg(err, errlen, "m26b: handle used on a different CUDA device than it was created on");
        return false;
    }
    return true;
}

}  // namespace

extern "C" {

const char* m26b_version(void) { return "m26b-expert 0.1 sm_100a"; }

int m26b_layer_new_tp(const uint8_t* canonical_dev, uint64_t canonical_bytes, uint32_t tp_rank, uint32_t tp_size,
                      m26b_layer** out, char* err, size_t errlen) {
    if (!out || !canonical_dev || !(tp_size == 1 || tp_size == 2 || tp_size == 4 || tp_size == 8) || tp_rank >= tp_size) {
        set_msg(err, errlen, "m26b layer: bad canonical extent/rank");
        return 1;
    }
    const uint64_t il = kInter / tp_size;
    const uint64_t gp = il * (kHidden / 2), gs = il * (kHidden / kBlockK);
    const uint64_t dp = uint64_t(kHidden) * (il / 2), ds = uint64_t(kHidden) * (il / kBlockK);
    const uint64_t image = 2 * (gp + gs) + dp + ds;
    if (canonical_bytes != image * kExperts) {
        set_msg(err, errlen, "m26b layer: bad canonical extent/rank");
        return 1;
    }
    ExpertSet home{};
    home.n = kExperts;
    home.gate = canonical_proj(canonical_dev, image, 0, gp, kHidden);
    home.up = canonical_proj(canonical_dev, image, gp + gs, gp + gs + gp, kHidden);
    home.down = canonical_proj(canonical_dev, image, 2 * (gp + gs), 2 * (gp + gs) + dp, il);
    return prepare_layer(home, nullptr, nullptr, tp_rank, tp_size, out, err, errlen);
}

int m26b_layer_new(const uint8_t* canonical_dev, uint64_t canonical_bytes, uint32_t rank, m26b_layer** out, char* err,
                   size_t errlen) {
    return m26b_layer_new_tp(canonical_dev, canonical_bytes, rank, 4, out, err, errlen);
}

int m26b_layer_new_from_checkpoint(const uint8_t* gate_w, const uint8_t* gate_s, const uint8_t* up_w,
                                   const uint8_t* up_s, const uint8_t* down_w, const uint8_t* down_s,
                                   uint32_t tp_rank, uint32_t tp_size, m26b_layer** out, char* err, size_t errlen) {
    if (!out || !gate_w || !gate_s || !up_w || !up_s || !down_w || !down_s ||
        !(tp_size == 1 || tp_size == 2 || tp_size == 4 || tp_size == 8) || tp_rank >= tp_size) {
        set_msg(err, errlen, "m26b layer: bad checkpoint tensors/rank");
        return 1;
    }
    return prepare_layer(checkpoint_set(gate_w, gate_s, up_w, up_s, down_w, down_s, tp_rank, tp_size, kExperts), nullptr, nullptr, tp_rank,
                         tp_size, out, err, errlen);
}

int m26b_layer_new_from_checkpoint_ep(const uint8_t* gate_w, const uint8_t* gate_s, const uint8_t* up_w,
                                      const uint8_t* up_s, const uint8_t* down_w, const uint8_t* down_s,
                                      uint32_t ep_rank, uint32_t ep_size, m26b_layer** out, char* err, size_t errlen) {
    if (!out || !gate_w || !gate_s || !up_w || !up_s || !down_w || !down_s ||
        !(ep_size == 1 || ep_size == 2 || ep_size == 4 || ep_size == 8) || ep_rank >= ep_size) {
        set_msg(err, errlen, "m26b layer: bad checkpoint tensors/rank");
        return 1;
    }
    const int n_local = kExperts / int(ep_size);
    return prepare_layer(checkpoint_set(gate_w, gate_s, up_w, up_s, down_w, down_s, 0, 1, n_local), nullptr, nullptr, 0, 1, out, err,
                         errlen, int(ep_rank) * n_local);
}

int m26b_layer_new_from_checkpoint_ep_replicated(const uint8_t* gate_w, const uint8_t* gate_s, const uint8_t* up_w,
                                                 const uint8_t* up_s, const uint8_t* down_w, const uint8_t* down_s,
                                                 const uint8_t* rep_gate_w, const uint8_t* rep_gate_s, const uint8_t* rep_up_w,
                                                 const uint8_t* rep_up_s, const uint8_t* rep_down_w, const uint8_t* rep_down_s,
                                                 const int32_t* rep_ids, uint32_t n_rep, uint32_t ep_rank, uint32_t ep_size,
                                                 m26b_layer** out, char* err, size_t errlen) {
    if (!out || !gate_w || !gate_s || !up_w || !up_s || !down_w || !down_s ||
        !(ep_size == 1 || ep_size == 2 || ep_size == 4 || ep_size == 8) || ep_rank >= ep_size || n_rep > uint32_t(kExperts) ||
        (n_rep && (!rep_gate_w || !rep_gate_s || !rep_up_w || !rep_up_s || !rep_down_w || !rep_down_s || !rep_ids))) {
        set_msg(err, errlen, "m26b layer: bad checkpoint tensors/rank");
        return 1;
    }
    const int n_local = kExperts / int(ep_size);
    const ExpertSet home = checkpoint_set(gate_w, gate_s, up_w, up_s, down_w, down_s, 0, 1, n_local);
    const ExpertSet rep = checkpoint_set(rep_gate_w, rep_gate_s, rep_up_w, rep_up_s, rep_down_w, rep_down_s, 0, 1, int(n_rep));
    return prepare_layer(home, n_rep ? &rep : nullptr, rep_ids, 0, 1, out, err, errlen, int(ep_rank) * n_local);
}

const void* m26b_layer_image(const m26b_layer* L, int which, uint64_t* bytes) {
    if (!L || which < 0 || which > 4) return nullptr;
    const uint64_t n = uint64_t(L->n_local + L->n_rep), il = uint64_t(L->i_local);
    const uint64_t size[5] = {n * 2 * il * (kHidden / 2), n * 2 * il * (kHidden / kBlockK), n * kHidden * (il / 2), n * kHidden * (il / kBlockK),
                              n * 2 * il * (kHidden / kBlockK)};
    const uint8_t* base[5] = {L->w13, L->s13, L->w2, L->s2, L->s13h};
    if (bytes) *bytes = size[which];
    return base[which];
}

int m26b_layer_all_normal(const m26b_layer* L) { return L && L->all_normal ? 1 : 0; }
int m26b_layer_i_local(const m26b_layer* L) { return L ? L->i_local : 0; }

void m26b_layer_free(m26b_layer* L) {
    if (!L) return;
    cudaFree(L->w13); cudaFree(L->s13); cudaFree(L->s13h); cudaFree(L->w2); cudaFree(L->s2); cudaFree(L->slots);
    delete L;
}

int m26b_scratch_new(m26b_scratch** out, char* err, size_t errlen) {
    if (!out) { set_msg(err, errlen, "m26b scratch: null out"); return 1; }
    auto* S = new m26b_scratch();
    cudaError_t e;
    cudaDeviceProp prop;
    if ((e = cudaGetDevice(&S->device)) != cudaSuccess || (e = cudaGetDeviceProperties(&prop, S->device)) != cudaSuccess) {
        set_err(err, errlen, "m26b scratch device", e);
        delete S;
        return 2;
    }
    if (prop.major != 10) {
        set_msg(err, errlen, "m26b scratch: this library is built for sm_100a (B200) only; no other device and no CPU path exists");
        delete S;
        return 2;
    }
    S->sms = prop.multiProcessorCount;
    {
        // the reference's opt-in for BF16 route outputs, read where it reads it (b1_serve.cu:402-405)
        const char* v = std::getenv("MIMO26_B1_Y");
        S->y16 = v && std::strcmp(v, "bf16") == 0;
    }
    {
        const int c1 = pair_resident_ctas<kModeFc1>(S->sms), c2 = pair_resident_ctas<kModeFc2>(S->sms);
        S->pair_ctas = c1 < c2 ? c1 : c2;
    }
    if ((e = cudaStreamCreateWithFlags(&S->st, cudaStreamNonBlocking)) != cudaSuccess ||
        (e = cudaEventCreate(&S->e0)) != cudaSuccess || (e = cudaEventCreate(&S->e1)) != cudaSuccess ||
        (e = cudaEventCreate(&S->ea)) != cudaSuccess || (e = cudaEventCreate(&S->ec)) != cudaSuccess ||
        (e = cudaMallocHost(reinterpret_cast<void**>(&S->hstatus), sizeof(Status) * 64)) != cudaSuccess ||
        (e = cudaMallocHost(reinterpret_cast<void**>(&S->hstage), kStageBytes)) != cudaSuccess ||
        (e = [&] { cudaError_t r = cudaSuccess; for (auto& ev : S->kev) if (r == cudaSuccess) r = cudaEventCreate(&ev); return r; }()) != cudaSuccess) {
        set_err(err, errlen, "m26b scratch stream/events", e);
        m26b_scratch_free(S);
        return 2;
    }
    *out = S;
    return 0;
}

void m26b_scratch_free(m26b_scratch* S) {
    if (!S) return;
    if (S->e0) cudaEventDestroy(S->e0);
    if (S->e1) cudaEventDestroy(S->e1);
    if (S->ea) cudaEventDestroy(S->ea);
    if (S->ec) cudaEventDestroy(S->ec);
    for (auto& ev : S->kev) if (ev) cudaEventDestroy(ev);
    if (S->st) cudaStreamDestroy(S->st);
    if (S->hstatus) cudaFreeHost(S->hstatus);
    if (S->hstage) cudaFreeHost(S->hstage);
    if (S->hiw) cudaFreeHost(S->hiw);
    delete S;
}

int m26b_scratch_set_debug(m26b_scratch* S, uint32_t flags) {
    if (!S) return 1;
    S->debug = flags;
    return 0;
}

int m26b_scratch_set_route_output(m26b_scratch* S, int dtype) {
    if (!S || dtype < 0 || dtype > 1) return 1;
    S->y16 = dtype == 1;
    return 0;
}

int m26b_ffn(const m26b_layer* L, m26b_scratch* S, const uint8_t* payload, size_t payload_pitch, const uint8_t* scales,
             size_t scales_pitch, const int32_t* ids, const float* weights, uint32_t rows, uint16_t* bf16_out, float* ms,
             char* err, size_t errlen) {
    if (!L || !S || !rows || rows > (1u << 20) || payload_pitch < kHidden || scales_pitch < kHidden / kBlockK || !payload ||
        !scales || !ids || !weights || !bf16_out) {
        set_msg(err, errlen, "m26b ffn: bad rows/handles/pitch");
        return 1;
    }
    if (!device_ok(L->device, err, errlen) || !device_ok(S->device, err, errlen)) return 1;
    cudaError_t e;
    const auto t0 = std::chrono::steady_clock::now();
    S->kev_quant = false;          // this entry point takes quantised rows: the quantiser slot of the timings reads zero
    const uint32_t pass_rows = rows < kMaxPassRows ? rows : kMaxPassRows;
    const uint32_t passes = (rows + kMaxPassRows - 1) / kMaxPassRows;
    if (passes > 64) { set_msg(err, errlen, "m26b ffn: bad rows/handles/pitch"); return 1; }
    M26B_CK(S->gather.ensure(size_t(rows) * kHidden * 2), "m26b out alloc");
    int rc = ensure_pass(S, pass_rows, L->i_local, false, err, errlen);
    if (rc) return rc;
    const uint8_t* xq_d;
    const uint8_t* xs_d;
    const int32_t* ids_d;
    const float* w_d;
    rc = upload_request(S, payload, payload_pitch, scales, scales_pitch, ids, weights, rows, &xq_d, &xs_d, &ids_d, &w_d, err, errlen);
    if (rc) return rc;
    uint16_t* const out_d = S->gather.as<uint16_t>();
    // GPU time of the pass from two events around it; the stage split (two more events between the kernels, which cost
    // the overlap of dependent launches: ~10 us of a decode step) only with debug flag 4
    const bool timed = ms != nullptr && passes == 1;
    const bool staged = timed && (S->debug & 4u) != 0;
    for (uint32_t ps = 0; ps < passes; ++ps) {
        const uint32_t r0 = ps * kMaxPassRows, n = rows - r0 < kMaxPassRows ? rows - r0 : kMaxPassRows;
        rc = enqueue_pass(L, S, xq_d + size_t(r0) * kHidden, xs_d + size_t(r0) * (kHidden / kBlockK),
                          ids_d + size_t(r0) * kTopK, w_d + size_t(r0) * kTopK, n, out_d + size_t(r0) * kHidden,
                          S->partial.as<float>(), S->status.as<Status>() + ps, S->st, timed, err, errlen);
        if (rc) return rc;
    }
    M26B_CK(cudaMemcpyAsync(bf16_out, out_d, size_t(rows) * kHidden * 2, cudaMemcpyDeviceToHost, S->st), "m26b bf16 download");
    M26B_CK(cudaMemcpyAsync(S->hstatus, S->status.p, sizeof(Status) * passes, cudaMemcpyDeviceToHost, S->st),
            "m26b status download");
    const auto t1 = std::chrono::steady_clock::now();
    M26B_CK(cudaStreamSynchronize(S->st), "m26b compute sync");
    S->pending = false;
    rc = decode_status(S->hstatus, passes, err, errlen);
    if (rc) return rc;
    const auto t2 = std::chrono::steady_clock::now();
    if (ms) {
        float gpu_ms = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
        if (timed) cudaEventElapsedTime(&gpu_ms, S->e0, S->e1);
        if (staged) {
            cudaEventElapsedTime(&p1, S->e0, S->ea);
            cudaEventElapsedTime(&p2, S->ea, S->ec);
            cudaEventElapsedTime(&p3, S->ec, S->e1);
        }
        ms[0] = std::chrono::duration<float, std::milli>(t1 - t0).count();
        ms[1] = gpu_ms;
        // what the host waited beyond the GPU's own time (the GPU starts before t1, so the difference can fall below zero)
        const float tail = std::chrono::duration<float, std::milli>(t2 - t1).count() - gpu_ms;
        ms[2] = tail > 0.f ? tail : 0.f;
        ms[3] = float(S->hstatus[0].meta.n_tiles);
        ms[4] = p1; ms[5] = 0.f; ms[6] = p2; ms[7] = p3;
    }
    return 0;
}

int m26b_quantize_dev(const void* x, int x_dtype, uint64_t n_elems, int codec, uint8_t* payload, uint8_t* scales,
                      uint32_t* fault_dev, void* stream, char* err, size_t errlen) {
    if (!x || !payload || !scales || !fault_dev || n_elems % 32 || x_dtype < 0 || x_dtype > 1 || codec < 0 || codec > 1) {
        set_msg(err, errlen, "m26b quantize: bad arguments");
        return 1;
    }
    if (!n_elems) return 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint64_t threads = n_elems / 16;
    const uint32_t blocks = uint32_t((threads + 255) / 256 < 148 * 64 ? (threads + 255) / 256 : 148 * 64);
    if (x_dtype == 0 && codec == 0) quantize_rows_kernel<0, uint16_t><<<blocks, 256, 0, st>>>(static_cast<const uint16_t*>(x), n_elems, payload, scales, fault_dev);
    else if (x_dtype == 0) quantize_rows_kernel<1, uint16_t><<<blocks, 256, 0, st>>>(static_cast<const uint16_t*>(x), n_elems, payload, scales, fault_dev);
    else if (codec == 0) quantize_rows_kernel<0, float><<<blocks, 256, 0, st>>>(static_cast<const float*>(x), n_elems, payload, scales, fault_dev);
    else quantize_rows_kernel<1, float><<<blocks, 256, 0, st>>>(static_cast<const float*>(x), n_elems, payload, scales, fault_dev);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_err(err, errlen, "m26b quantize launch", e); return 2; }
    return 0;
}

// Router top-8 and (optionally) the activation quantiser in one launch.
int m26b_produce_dev(const float* logits, const float* bias, uint32_t rows, int32_t* ids_out, float* weights_out, const void* x,
                     int x_dtype, int codec, uint8_t* payload, uint8_t* scales, uint32_t* fault_dev, void* stream, char* err,
                     size_t errlen) {
    const bool quant = x != nullptr;
    if (!logits || !ids_out || !weights_out || !rows ||
        (quant && (!payload || !scales || !fault_dev || x_dtype < 0 || x_dtype > 1 || codec < 0 || codec > 1))) {
        set_msg(err, errlen, "m26b produce: bad arguments");
        return 1;
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint32_t router_ctas = (rows + 7u) / 8u;
    const uint64_t n_elems = quant ? uint64_t(rows) * kHidden : 0;
    const uint64_t threads = n_elems / 16;
    const uint32_t qctas = quant ? uint32_t((threads + 255) / 256 < 148 * 64 ? (threads + 255) / 256 : 148 * 64) : 0u;
    const uint32_t grid = router_ctas + qctas;
    if (!quant || (x_dtype == 0 && codec == 0))
        produce_kernel<0, uint16_t><<<grid, 256, 0, st>>>(logits, bias, rows, router_ctas, ids_out, weights_out,
                                                           static_cast<const uint16_t*>(x), n_elems, payload, scales, fault_dev);
    else if (x_dtype == 0)
        produce_kernel<1, uint16_t><<<grid, 256, 0, st>>>(logits, bias, rows, router_ctas, ids_out, weights_out,
                                                           static_cast<const uint16_t*>(x), n_elems, payload, scales, fault_dev);
    else if (codec == 0)
        produce_kernel<0, float><<<grid, 256, 0, st>>>(logits, bias, rows, router_ctas, ids_out, weights_out,
                                                        static_cast<const float*>(x), n_elems, payload, scales, fault_dev);
    else
        produce_kernel<1, float><<<grid, 256, 0, st>>>(logits, bias, rows, router_ctas, ids_out, weights_out,
                                                        static_cast<const float*>(x), n_elems, payload, scales, fault_dev);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_err(err, errlen, "m26b produce launch", e); return 2; }
    return 0;
}

int m26b_ffn_dev(const m26b_layer* L, m26b_scratch* S, const void* x, int x_dtype, const uint8_t* x_scales, int codec,
                 const int32_t* ids, const float* weights, uint32_t rows, uint16_t* bf16_out, float* partial_out,
                 void* stream, char* err, size_t errlen) {
    if (!L || !S || !rows || rows > kMaxPassRows || !x || !ids || !weights || !bf16_out || x_dtype < 0 || x_dtype > 2 ||
        (x_dtype == 2 && !x_scales) || codec < 0 || codec > 1) {
        set_msg(err, errlen, "m26b ffn: bad rows/handles/pitch");
        return 1;
    }
    if (!device_ok(L->device, err, errlen) || !device_ok(S->device, err, errlen)) return 1;
    if (reinterpret_cast<uintptr_t>(x) & 15u) {
        set_msg(err, errlen, "m26b ffn: the activation pointer must be 16-byte aligned");
        return 1;
    }
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : S->st;
    int rc = ensure_pass(S, rows, L->i_local, x_dtype != 2, err, errlen);
    if (rc) return rc;
    Status* status = S->status.as<Status>();
    const uint8_t* xq = static_cast<const uint8_t*>(x);
    const uint8_t* xs = x_scales;
    RawInput raw{x, x_dtype, codec, &status[1].fault_input};
    if (x_dtype != 2) {
        // the quantiser's fault word (second status block) is cleared together with the pass's own block; the quantiser
        // itself runs inside the pass (fused prologue, or the quantise-and-permute kernel)
        cudaError_t e;
        M26B_CK(cudaMemsetAsync(status, 0, 2 * sizeof(Status), st), "m26b status clear");
        if (S->debug & 2u) M26B_CK(cudaEventRecord(S->kev[0], st), "m26b event");
        xq = S->xq.as<uint8_t>(); xs = S->xs.as<uint8_t>();
    }
    S->kev_quant = x_dtype != 2;
    rc = enqueue_pass(L, S, xq, xs, ids, weights, rows, bf16_out, partial_out ? partial_out : nullptr, status, st, false,
                      err, errlen, x_dtype != 2 ? &raw : nullptr, x_dtype != 2);
    if (rc) return rc;
    S->pending = true;
    S->n_status = x_dtype != 2 ? 2 : 1;
    return 0;
}

// m26b_ffn_dev for a rank of a tensor-parallel group: the pass's combine is fused with the plane exchange, so the call
// leaves the rank-ordered FP32 sum of every rank's BF16 plane (+ residual) in sum_out. Steps too large for the fused form
// run the combine into the rank's plane and the pull-form exchange kernel behind it; either way it is one exchange step.
int m26b_ffn_tp_dev(const m26b_layer* L, m26b_scratch* S, m26b_exchange* X, const void* x, int x_dtype, const uint8_t* x_scales,
                    int codec, const int32_t* ids, const float* weights, uint32_t rows, const float* residual, float* sum_out,
                    void* stream, char* err, size_t errlen) {
    if (!L || !S || !X || !rows || rows > kMaxPassRows || !x || !ids || !weights || !sum_out || x_dtype < 0 || x_dtype > 2 ||
        (x_dtype == 2 && !x_scales) || codec < 0 || codec > 1 || uint64_t(rows) * kHidden * 2 > X->plane_bytes) {
        set_msg(err, errlen, "m26b ffn_tp: bad rows/handles/pitch (the request must fit the exchange plane)");
        return 1;
    }
    if (!device_ok(L->device, err, errlen) || !device_ok(S->device, err, errlen) || !device_ok(X->device, err, errlen)) return 1;
    if (uint32_t(X->world) != L->tp_size || uint32_t(X->rank) != L->tp_rank) {
        set_msg(err, errlen, "m26b ffn_tp: the exchange window and the layer belong to different ranks");
        return 1;
    }
    for (int r = 0; r < X->world; ++r)
        if (!X->peers.window[r]) { set_msg(err, errlen, "m26b ffn_tp: the exchange is not connected to every peer"); return 1; }
    if (reinterpret_cast<uintptr_t>(x) & 15u) {
        set_msg(err, errlen, "m26b ffn: the activation pointer must be 16-byte aligned");
        return 1;
    }
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : S->st;
    int rc = ensure_pass(S, rows, L->i_local, x_dtype != 2, err, errlen);
    if (rc) return rc;
    Status* status = S->status.as<Status>();
    const uint8_t* xq = static_cast<const uint8_t*>(x);
    const uint8_t* xs = x_scales;
    RawInput raw{x, x_dtype, codec, &status[1].fault_input};
    if (x_dtype != 2) {
        cudaError_t e;
        M26B_CK(cudaMemsetAsync(status, 0, 2 * sizeof(Status), st), "m26b status clear");
        xq = S->xq.as<uint8_t>(); xs = S->xs.as<uint8_t>();
    }
    S->kev_quant = false;
    const bool fused = uint64_t(rows) * kHidden * 4 <= X->push.cap;
    const PushSink sink{X, sum_out, residual};
    rc = enqueue_pass(L, S, xq, xs, ids, weights, rows, fused ? nullptr : static_cast<uint16_t*>(m26b_exchange_plane(X)), nullptr,
                      status, st, false, err, errlen, x_dtype != 2 ? &raw : nullptr, x_dtype != 2, nullptr, fused ? &sink : nullptr);
    if (rc) return rc;
    S->pending = true;
    S->n_status = x_dtype != 2 ? 2 : 1;
    if (!fused) return m26b_exchange_sum_residual_dev(X, uint64_t(rows) * kHidden, residual, sum_out, st, err, errlen);
    return 0;
}

int m26b_scratch_status(m26b_scratch* S, void* stream, char* err, size_t errlen) {
    if (!S) { set_msg(err, errlen, "m26b status: null scratch"); return 1; }
    cudaError_t e;
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : S->st;
    const uint32_t n = S->n_status ? S->n_status : 1;
    M26B_CK(cudaMemcpyAsync(S->hstatus, S->status.p, sizeof(Status) * n, cudaMemcpyDeviceToHost, st), "m26b status download");
    M26B_CK(cudaStreamSynchronize(st), "m26b status sync");
    S->pending = false;
    return decode_status(S->hstatus, n, err, errlen);
}

int m26b_route_reduce_dev(const float* y, const float* weights, uint32_t rows, float* partial, uint16_t* bf16,
                          uint32_t* fault_dev, void* stream, char* err, size_t errlen) {
    if (!y || !weights || !bf16 || !fault_dev) { set_msg(err, errlen, "m26b reduce: bad arguments"); return 1; }
    if (!rows) return 0;
    const uint64_t n4 = uint64_t(rows) * (kHidden / 4);
    const uint32_t blocks = uint32_t(n4 / 256 + 1 < 16384 ? n4 / 256 + 1 : 16384);
    route_reduce_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(y, weights, rows, partial, bf16, fault_dev);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_err(err, errlen, "m26b reduce launch", e); return 2; }
    return 0;
}

int m26b_rank_sum_residual_dev(const uint16_t* const* planes, int n_ranks, uint64_t n, const float* residual, float* out,
                               void* stream, char* err, size_t errlen) {
    if (!planes || n_ranks < 1 || n_ranks > 8 || !out) { set_msg(err, errlen, "m26b rank sum: bad arguments"); return 1; }
    RankPlanes rp{};
    for (int r = 0; r < n_ranks; ++r) {
        if (!planes[r]) { set_msg(err, errlen, "m26b rank sum: bad arguments"); return 1; }
        rp.p[r] = planes[r];
    }
    if (!n) return 0;
    const uint64_t t = (n / 8 + 255) / 256 + 1;
    rank_sum_kernel<<<uint32_t(t < 148 * 16 ? t : 148 * 16), 256, 0, static_cast<cudaStream_t>(stream)>>>(rp, n_ranks, n, out, residual);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_err(err, errlen, "m26b rank sum launch", e); return 2; }
    return 0;
}

int m26b_rank_sum_dev(const uint16_t* const* planes, int n_ranks, uint64_t n, float* out, void* stream, char* err,
                      size_t errlen) {
    return m26b_rank_sum_residual_dev(planes, n_ranks, n, nullptr, out, stream, err, errlen);
}

// ---- plane exchange between the GPUs of one box ----------------------------------------------
int m26b_exchange_new(uint64_t plane_bytes, uint32_t rank, uint32_t world, m26b_exchange** out, uint8_t* handle_out,
                      char* err, size_t errlen) {
    if (!out || !plane_bytes || plane_bytes % 256 || world < 1 || world > 8 || rank >= world) {
        set_msg(err, errlen, "m26b exchange: bad plane size / rank / world (plane bytes must be a multiple of 256)");
        return 1;
    }
    cudaError_t e;
    m26b_exchange* X = new m26b_exchange();
    X->rank = int(rank); X->world = int(world); X->plane_bytes = plane_bytes;
    // behind the two plane slots of the pull form: the receive planes of the push form (steps of at most kPushRows tokens,
    // where a kernel boundary and a round trip matter; larger steps are bandwidth-bound and pull). 4 bytes per element:
    // every 8-byte half carries two BF16 codes and the step number. Zero-filled once: step numbers start at 1.
    const uint64_t push_cap = (plane_bytes < uint64_t(kPushRows) * kHidden * 2 ? plane_bytes : uint64_t(kPushRows) * kHidden * 2) * 2;
    X->push.cap = push_cap;
    X->push.recv_off = sizeof(ExchangeWindow) + 2 * plane_bytes;
    const uint64_t total = X->push.recv_off + uint64_t(2) * world * push_cap;
    if ((e = cudaGetDevice(&X->device)) != cudaSuccess ||
        (e = cudaMalloc(&X->window, total)) != cudaSuccess ||
        (e = cudaMemset(X->window, 0, sizeof(ExchangeWindow))) != cudaSuccess ||
        (e = cudaMemset(static_cast<uint8_t*>(X->window) + X->push.recv_off, 0, uint64_t(2) * world * push_cap)) != cudaSuccess) {
        set_err(err, errlen, "m26b exchange window", e);
        m26b_exchange_free(X);
        return 2;
    }
    int khz = 0;
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, X->device);
    X->khz = khz > 0 ? khz : 1965000;
    X->wait_cycles = 2000ll * X->khz;                      // two seconds at the nominal clock
    X->peers.window[rank] = static_cast<uint8_t*>(X->window);
    if (handle_out) {
        cudaIpcMemHandle_t h;
        if ((e = cudaIpcGetMemHandle(&h, X->window)) != cudaSuccess) {
            set_err(err, errlen, "m26b exchange export", e);
            m26b_exchange_free(X);
            return 2;
        }
        static_assert(sizeof(h) == 64, "IPC handle is 64 bytes");
        std::memcpy(handle_out, &h, 64);
    }
    *out = X;
    return 0;
}

int m26b_exchange_connect(m26b_exchange* X, const uint8_t* handles, char* err, size_t errlen) {
    if (!X || !handles) { set_msg(err, errlen, "m26b exchange connect: bad arguments"); return 1; }
    if (!device_ok(X->device, err, errlen)) return 1;
    for (int r = 0; r < X->world; ++r) {
        if (r == X->rank || X->peers.window[r]) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, handles + size_t(r) * 64, 64);
        void* p = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) { set_err(err, errlen, "m26b exchange: opening a peer window", e); return 2; }
        X->peers.window[r] = static_cast<uint8_t*>(p);
        X->opened[r] = true;
    }
    return 0;
}

int m26b_exchange_connect_local(m26b_exchange* X, m26b_exchange* const* all, char* err, size_t errlen) {
    if (!X || !all) { set_msg(err, errlen, "m26b exchange connect: bad arguments"); return 1; }
    for (int r = 0; r < X->world; ++r) {
        if (r == X->rank) continue;
        if (!all[r] || all[r]->world != X->world || all[r]->rank != r || all[r]->plane_bytes != X->plane_bytes) {
            set_msg(err, errlen, "m26b exchange connect: windows do not belong together");
            return 1;
        }
        X->peers.window[r] = static_cast<uint8_t*>(all[r]->window);
    }
    return 0;
}

void* m26b_exchange_plane(m26b_exchange* X) {
    if (!X) return nullptr;
    return static_cast<uint8_t*>(X->window) + sizeof(ExchangeWindow) + size_t((X->step + 1) & 1u) * X->plane_bytes;
}

int m26b_exchange_set_wait_ms(m26b_exchange* X, uint32_t ms) {
    if (!X || !ms) return 1;
    X->wait_cycles = (long long)ms * X->khz;
    return 0;
}

int m26b_exchange_publish_as(m26b_exchange* X, uint32_t peer_rank, void* stream, char* err, size_t errlen) {
    if (!X || int(peer_rank) >= X->world || int(peer_rank) == X->rank) { set_msg(err, errlen, "m26b exchange: bad peer"); return 1; }
    const uint32_t next = X->step + 1;
    cudaError_t e = cudaMemcpyAsync(&static_cast<ExchangeWindow*>(X->window)->flags[peer_rank], &next, 4,
                                    cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) { set_err(err, errlen, "m26b exchange publish", e); return 2; }
    // and the peer's receive plane of the fused form, for the slot the next step uses: flags only, data as they are
    uint4* pl = reinterpret_cast<uint4*>(static_cast<uint8_t*>(X->window) + X->push.recv_off +
                                         (size_t(next & 1u) * X->world + peer_rank) * X->push.cap);
    const uint32_t words = uint32_t(X->push.cap / 16);
    push_mark_kernel<<<(words + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(pl, next, words);
    if ((e = cudaGetLastError()) != cudaSuccess) { set_err(err, errlen, "m26b exchange publish", e); return 2; }
    // the marks must be in place before any kernel that waits for them is launched (on whatever stream)
    if ((e = cudaStreamSynchronize(static_cast<cudaStream_t>(stream))) != cudaSuccess) { set_err(err, errlen, "m26b exchange publish", e); return 2; }
    return 0;
}

int m26b_exchange_sum_dev(m26b_exchange* X, uint64_t n_elems, float* out_f32, void* stream, char* err, size_t errlen) {
    return m26b_exchange_sum_residual_dev(X, n_elems, nullptr, out_f32, stream, err, errlen);
}

int m26b_exchange_sum_residual_dev(m26b_exchange* X, uint64_t n_elems, const float* residual, float* out_f32, void* stream,
                                   char* err, size_t errlen) {
    if (!X || !out_f32 || !n_elems || n_elems % 8 || n_elems * 2 > X->plane_bytes) {
        set_msg(err, errlen, "m26b exchange sum: bad extent (a multiple of 8 elements that fits the plane)");
        return 1;
    }
    if (!device_ok(X->device, err, errlen)) return 1;
    for (int r = 0; r < X->world; ++r)
        if (!X->peers.window[r]) { set_msg(err, errlen, "m26b exchange sum: not connected to every peer"); return 1; }
    X->step += 1;
    const uint64_t off = sizeof(ExchangeWindow) + size_t(X->step & 1u) * X->plane_bytes;
    const uint64_t t = (n_elems / 8 + 255) / 256;
    const unsigned blocks = unsigned(t < 148 * 8 ? (t ? t : 1) : 148 * 8);
    const cudaError_t e = launch_dependent(exchange_sum_kernel, blocks, 256u, size_t(0), static_cast<cudaStream_t>(stream), X->peers,
                                           X->rank, X->world, X->step, off, n_elems, X->wait_cycles, out_f32, residual);
    if (e != cudaSuccess) { set_err(err, errlen, "m26b exchange sum launch", e); return 2; }
    return 0;
}

int m26b_exchange_status(m26b_exchange* X, void* stream, char* err, size_t errlen) {
    if (!X) { set_msg(err, errlen, "m26b exchange status: null handle"); return 1; }
    cudaError_t e;
    uint32_t word = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    M26B_CK(cudaMemcpyAsync(&word, &static_cast<ExchangeWindow*>(X->window)->error, 4, cudaMemcpyDeviceToHost, st), "m26b exchange status");
    M26B_CK(cudaStreamSynchronize(st), "m26b exchange status sync");
    if (word) {
        M26B_CK(cudaMemsetAsync(&static_cast<ExchangeWindow*>(X->window)->error, 0, 4, st), "m26b exchange status clear");
        M26B_CK(cudaStreamSynchronize(st), "m26b exchange status sync");
        if (err && errlen) std::snprintf(err, errlen, "m26b exchange: rank %d gave up waiting for peers (mask 0x%x) at step %u; that step's sum was not written", X->rank, word, X->step);
        return 5;
    }
    return 0;
}

void m26b_exchange_free(m26b_exchange* X) {
    if (!X) return;
    for (int r = 0; r < 8; ++r)
        if (X->opened[r] && X->peers.window[r]) cudaIpcCloseMemHandle(X->peers.window[r]);
    if (X->window) cudaFree(X->window);
    delete X;
}

// ---- expert parallelism inside one box ---------------------------------------------------------
namespace {
uint8_t* ep_ptr(const m26b_ep* E, int r, size_t off) { return E->peers.window[r] + off; }
bool ep_connected(const m26b_ep* E) {
    for (int r = 0; r < E->world; ++r)
        if (!E->peers.window[r]) return false;
    return true;
}
}  // namespace

int m26b_ep_new(uint32_t tokens, uint32_t rank, uint32_t world, m26b_ep** out, uint8_t* handle_out, char* err, size_t errlen) {
    if (!out || !tokens || tokens > (1u << 20) || !(world == 1 || world == 2 || world == 4 || world == 8) || rank >= world) {
        set_msg(err, errlen, "m26b ep: bad token count / rank / world");
        return 1;
    }
    cudaError_t e;
    m26b_ep* E = new m26b_ep();
    E->rank = int(rank); E->world = int(world); E->tokens = tokens;
    const uint32_t base = tokens / world, extra = tokens % world;    // contiguous blocks, the first `extra` one longer
    for (uint32_t r = 0; r <= world; ++r) E->lo[r] = r * base + (r < extra ? r : extra);
    for (uint32_t r = world + 1; r < 9; ++r) E->lo[r] = tokens;
    E->lay.cap = base + (extra ? 1u : 0u);
    if (E->lay.cap == 0) E->lay.cap = 1;
    if ((e = cudaGetDevice(&E->device)) != cudaSuccess || (e = cudaMalloc(&E->window, E->lay.bytes())) != cudaSuccess ||
        (e = cudaMemset(E->window, 0, sizeof(EpHeader))) != cudaSuccess || (e = cudaMalloc(&E->fault, 4)) != cudaSuccess ||
        (e = cudaMemset(E->fault, 0, 4)) != cudaSuccess ||
        (e = cudaMallocHost(reinterpret_cast<void**>(&E->hfault), 8)) != cudaSuccess ||
        (e = E->ids.ensure(size_t(tokens) * kTopK * 4)) != cudaSuccess || (e = E->w.ensure(size_t(tokens) * kTopK * 4)) != cudaSuccess) {
        set_err(err, errlen, "m26b ep window", e);
        m26b_ep_free(E);
        return 2;
    }
    int khz = 0;
    cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, E->device);
    E->khz = khz > 0 ? khz : 1965000;
    E->wait_cycles = 5000ll * E->khz;
    E->peers.window[rank] = static_cast<uint8_t*>(E->window);
    if (handle_out) {
        cudaIpcMemHandle_t h;
        if ((e = cudaIpcGetMemHandle(&h, E->window)) != cudaSuccess) {
            set_err(err, errlen, "m26b ep export", e);
            m26b_ep_free(E);
            return 2;
        }
        std::memcpy(handle_out, &h, 64);
    }
    *out = E;
    return 0;
}

int m26b_ep_connect(m26b_ep* E, const uint8_t* handles, char* err, size_t errlen) {
    if (!E || !handles) { set_msg(err, errlen, "m26b ep connect: bad arguments"); return 1; }
    if (!device_ok(E->device, err, errlen)) return 1;
    for (int r = 0; r < E->world; ++r) {
        if (r == E->rank || E->peers.window[r]) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, handles + size_t(r) * 64, 64);
        void* p = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) { set_err(err, errlen, "m26b ep: opening a peer window", e); return 2; }
        E->peers.window[r] = static_cast<uint8_t*>(p);
        E->opened[r] = true;
    }
    return 0;
}

int m26b_ep_connect_local(m26b_ep* E, m26b_ep* const* all, char* err, size_t errlen) {
    if (!E || !all) { set_msg(err, errlen, "m26b ep connect: bad arguments"); return 1; }
    for (int r = 0; r < E->world; ++r) {
        if (r == E->rank) continue;
        if (!all[r] || all[r]->world != E->world || all[r]->rank != r || all[r]->tokens != E->tokens) {
            set_msg(err, errlen, "m26b ep connect: windows do not belong together");
            return 1;
        }
        E->peers.window[r] = static_cast<uint8_t*>(all[r]->window);
    }
    return 0;
}

int m26b_ep_rows(const m26b_ep* E, uint32_t rank) { return E && int(rank) < E->world ? int(E->lo[rank + 1] - E->lo[rank]) : -1; }

int m26b_ep_set_route_output(m26b_ep* E, int dtype) {
    if (!E || dtype < 0 || dtype > 1) return 1;
    E->y16 = dtype == 1;
    return 0;
}

int m26b_ep_set_wait_ms(m26b_ep* E, uint32_t ms) {
    if (!E || !ms) return 1;
    E->wait_cycles = (long long)ms * E->khz;
    return 0;
}

int m26b_ep_publish_as(m26b_ep* E, uint32_t peer_rank, uint32_t which, void* stream, char* err, size_t errlen) {
    if (!E || int(peer_rank) >= E->world || int(peer_rank) == E->rank || which > 1) { set_msg(err, errlen, "m26b ep: bad peer"); return 1; }
    const uint32_t v = which == 0 ? E->step + 1 : E->step;     // rendezvous 0 opens a step, rendezvous 1 closes it
    const cudaError_t e = cudaMemcpyAsync(&static_cast<EpHeader*>(E->window)->flags[which][peer_rank], &v, 4, cudaMemcpyHostToDevice,
                                          static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) { set_err(err, errlen, "m26b ep publish", e); return 2; }
    return 0;
}

// Phase 1: this rank's tokens into its window (quantised rows, routes), then the "rows ready" rendezvous.
int m26b_ep_begin_dev(m26b_ep* E, const void* x, int x_dtype, const uint8_t* x_scales, int codec, const int32_t* ids,
                      const float* weights, uint32_t rows, void* stream, char* err, size_t errlen) {
    if (!E || !x || !ids || !weights || x_dtype < 0 || x_dtype > 2 || (x_dtype == 2 && !x_scales) || codec < 0 || codec > 1 ||
        rows != E->lo[E->rank + 1] - E->lo[E->rank]) {
        set_msg(err, errlen, "m26b ep begin: bad arguments (rows must be this rank's token block)");
        return 1;
    }
    if (!device_ok(E->device, err, errlen)) return 1;
    if (!ep_connected(E)) { set_msg(err, errlen, "m26b ep: not connected to every peer"); return 1; }
    cudaError_t e;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t* xq = ep_ptr(E, E->rank, E->lay.xq_off());
    uint8_t* xs = ep_ptr(E, E->rank, E->lay.xs_off());
    M26B_CK(cudaMemsetAsync(E->fault, 0, 4, st), "m26b ep fault clear");
    if (rows) {
        if (x_dtype == 2) {
            M26B_CK(cudaMemcpyAsync(xq, x, size_t(rows) * kHidden, cudaMemcpyDeviceToDevice, st), "m26b ep rows");
            M26B_CK(cudaMemcpyAsync(xs, x_scales, size_t(rows) * (kHidden / kBlockK), cudaMemcpyDeviceToDevice, st), "m26b ep scales");
        } else {
            const int rc = m26b_quantize_dev(x, x_dtype, uint64_t(rows) * kHidden, codec, xq, xs, E->fault, st, err, errlen);
            if (rc) return rc;
        }
        M26B_CK(cudaMemcpyAsync(ep_ptr(E, E->rank, E->lay.ids_off()), ids, size_t(rows) * kTopK * 4, cudaMemcpyDeviceToDevice, st), "m26b ep ids");
        M26B_CK(cudaMemcpyAsync(ep_ptr(E, E->rank, E->lay.w_off()), weights, size_t(rows) * kTopK * 4, cudaMemcpyDeviceToDevice, st), "m26b ep weights");
    }
    E->step += 1;
    ep_rendezvous_kernel<<<1, 32, 0, st>>>(E->peers, E->rank, E->world, 0, E->step, E->wait_cycles);
    M26B_CK(cudaGetLastError(), "m26b ep rendezvous launch");
    return 0;
}

// Phase 2: this rank's experts on every rank's tokens, in passes of at most kMaxPassRows tokens; then the
// "results complete" rendezvous.
int m26b_ep_compute_dev(m26b_ep* E, const m26b_layer* L, m26b_scratch* S, void* stream, char* err, size_t errlen) {
    if (!E || !L || !S) { set_msg(err, errlen, "m26b ep compute: null handle"); return 1; }
    if (!device_ok(E->device, err, errlen) || !device_ok(L->device, err, errlen) || !device_ok(S->device, err, errlen)) return 1;
    if (L->tp_size != 1 || L->n_local * E->world != kExperts || L->expert_lo != E->rank * L->n_local) {
        set_msg(err, errlen, "m26b ep compute: the layer does not hold this rank's block of experts");
        return 1;
    }
    cudaError_t e;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint32_t pass_rows = E->tokens < kMaxPassRows ? E->tokens : kMaxPassRows;
    const uint32_t passes = (E->tokens + kMaxPassRows - 1) / kMaxPassRows;
    if (passes > 64) { set_msg(err, errlen, "m26b ep compute: too many tokens"); return 1; }
    int rc = ensure_pass(S, pass_rows, L->i_local, false, err, errlen);
    if (rc) return rc;
    S->kev_quant = false;
    TokenSources shards{};
    shards.n = uint32_t(E->world);
    RouteSinks sinks{};
    sinks.n = uint32_t(E->world);
    for (int r = 0; r < 9; ++r) { shards.lo[r] = E->lo[r]; sinks.lo[r] = E->lo[r]; }
    for (int r = 0; r < E->world; ++r) {
        shards.xq[r] = ep_ptr(E, r, E->lay.xq_off());
        shards.xs[r] = ep_ptr(E, r, E->lay.xs_off());
        sinks.y[r] = reinterpret_cast<float*>(ep_ptr(E, r, E->lay.y_off()));
    }
    const uint32_t total = E->tokens * kTopK;
    const unsigned gb = (total + 255) / 256 < 1184 ? (total + 255) / 256 : 1184;
    ep_gather_routes_kernel<<<gb, 256, 0, st>>>(E->peers, E->lay, E->world, shards, E->ids.as<int32_t>(), E->w.as<float>());
    M26B_CK(cudaGetLastError(), "m26b ep gather launch");
    for (uint32_t ps = 0; ps < passes; ++ps) {
        const uint32_t r0 = ps * kMaxPassRows, n = E->tokens - r0 < kMaxPassRows ? E->tokens - r0 : kMaxPassRows;
        EpPass pass{shards, sinks, E->y16, 0u, 0u};
        pass.src.token_base = r0; pass.sinks.token_base = r0;
        {   // this rank's tokens inside the pass
            const uint32_t lo = E->lo[E->rank], hi = E->lo[E->rank + 1];
            const uint32_t a0 = lo > r0 ? lo - r0 : 0u, a1 = hi > r0 ? hi - r0 : 0u;
            pass.own_lo = a0 < n ? a0 : n;
            pass.own_hi = a1 < n ? a1 : n;
        }
        rc = enqueue_pass(L, S, nullptr, nullptr, E->ids.as<int32_t>() + size_t(r0) * kTopK, E->w.as<float>() + size_t(r0) * kTopK, n,
                          nullptr, nullptr, S->status.as<Status>() + ps, st, false, err, errlen, nullptr, false, &pass);
        if (rc) return rc;
    }
    S->pending = true;
    S->n_status = passes;
    ep_rendezvous_kernel<<<1, 32, 0, st>>>(E->peers, E->rank, E->world, 1, E->step, E->wait_cycles);
    M26B_CK(cudaGetLastError(), "m26b ep rendezvous launch");
    return 0;
}

// Phase 3: the ordered top-8 combine of this rank's tokens from the rows its peers (and itself) delivered.
int m26b_ep_finish_dev(m26b_ep* E, uint16_t* bf16_out, float* partial_out, void* stream, char* err, size_t errlen) {
    if (!E || !bf16_out) { set_msg(err, errlen, "m26b ep finish: bad arguments"); return 1; }
    if (!device_ok(E->device, err, errlen)) return 1;
    const uint32_t rows = E->lo[E->rank + 1] - E->lo[E->rank];
    if (!rows) return 0;
    const float* wts = reinterpret_cast<const float*>(ep_ptr(E, E->rank, E->lay.w_off()));
    if (E->y16) {
        const uint64_t n8 = uint64_t(rows) * (kHidden / 8);
        const uint32_t blocks = uint32_t(n8 / 256 + 1 < 16384 ? n8 / 256 + 1 : 16384);
        route_reduce_y16_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            reinterpret_cast<const uint16_t*>(ep_ptr(E, E->rank, E->lay.y_off())), wts, rows, partial_out, bf16_out, E->fault);
    } else {
        const uint64_t n4 = uint64_t(rows) * (kHidden / 4);
        const uint32_t blocks = uint32_t(n4 / 256 + 1 < 16384 ? n4 / 256 + 1 : 16384);
        route_reduce_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
            reinterpret_cast<const float*>(ep_ptr(E, E->rank, E->lay.y_off())), wts, rows, partial_out, bf16_out, E->fault);
    }
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { set_err(err, errlen, "m26b ep reduce launch", e); return 2; }
    return 0;
}

int m26b_ep_status(m26b_ep* E, void* stream, char* err, size_t errlen) {
    if (!E) { set_msg(err, errlen, "m26b ep status: null handle"); return 1; }
    cudaError_t e;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    M26B_CK(cudaMemcpyAsync(&E->hfault[0], &static_cast<EpHeader*>(E->window)->error, 4, cudaMemcpyDeviceToHost, st), "m26b ep status");
    M26B_CK(cudaMemcpyAsync(&E->hfault[1], E->fault, 4, cudaMemcpyDeviceToHost, st), "m26b ep status");
    M26B_CK(cudaStreamSynchronize(st), "m26b ep status sync");
    if (E->hfault[0]) {
        M26B_CK(cudaMemsetAsync(&static_cast<EpHeader*>(E->window)->error, 0, 4, st), "m26b ep status clear");
        M26B_CK(cudaStreamSynchronize(st), "m26b ep status sync");
        if (err && errlen)
            std::snprintf(err, errlen, "m26b ep: rank %d gave up waiting for peers (mask 0x%x: bits 0-7 rows ready, 8-15 results complete) at step %u",
                          E->rank, E->hfault[0], E->step);
        return 5;
    }
    if (E->hfault[1]) {
        if (err && errlen) std::snprintf(err, errlen, "m26b ep: quantizer/reduce fault %u on rank %d", E->hfault[1], E->rank);
        return 4;
    }
    return 0;
}

void m26b_ep_free(m26b_ep* E) {
    if (!E) return;
    for (int r = 0; r < 8; ++r)
        if (E->opened[r] && E->peers.window[r]) cudaIpcCloseMemHandle(E->peers.window[r]);
    if (E->window) cudaFree(E->window);
    if (E->fault) cudaFree(E->fault);
    if (E->hfault) cudaFreeHost(E->hfault);
    delete E;
}

// ---- host entry points of a tensor-parallel / expert-parallel rank -----------------------------------------------
// m26b_ffn for a rank of a tensor-parallel group inside one box: the request (host rows, as every rank of the
// reference receives the request frame) goes up, the rank's slice runs with its BF16 plane written straight into the
// exchange window, the planes are summed over NVLink by the exchange kernel, and the FP32 sum comes back to the host
// on the ranks that ask for it (sum_out != NULL; one rank is enough).
int m26b_ffn_tp(const m26b_layer* L, m26b_scratch* S, m26b_exchange* X, const uint8_t* payload, size_t payload_pitch,
                const uint8_t* scales, size_t scales_pitch, const int32_t* ids, const float* weights, uint32_t rows,
                float* sum_out, float* ms, char* err, size_t errlen) {
    if (!L || !S || !X || !rows || payload_pitch < kHidden || scales_pitch < kHidden / kBlockK || !payload || !scales || !ids ||
        !weights || uint64_t(rows) * kHidden * 2 > X->plane_bytes) {
        set_msg(err, errlen, "m26b ffn_tp: bad rows/handles/pitch (the request must fit the exchange plane)");
        return 1;
    }
    if (!device_ok(L->device, err, errlen) || !device_ok(S->device, err, errlen) || !device_ok(X->device, err, errlen)) return 1;
    if (uint32_t(X->world) != L->tp_size || uint32_t(X->rank) != L->tp_rank) {
        set_msg(err, errlen, "m26b ffn_tp: the exchange window and the layer belong to different ranks");
        return 1;
    }
    cudaError_t e;
    const auto t0 = std::chrono::steady_clock::now();
    S->kev_quant = false;
    const uint32_t pass_rows = rows < kMaxPassRows ? rows : kMaxPassRows;
    const uint32_t passes = (rows + kMaxPassRows - 1) / kMaxPassRows;
    if (passes > 64) { set_msg(err, errlen, "m26b ffn_tp: bad rows/handles/pitch"); return 1; }
    int rc = ensure_pass(S, pass_rows, L->i_local, false, err, errlen);
    if (rc) return rc;
    M26B_CK(S->tp_sum.ensure(size_t(rows) * kHidden * 4), "m26b sum alloc");
    const uint8_t* xq_d;
    const uint8_t* xs_d;
    const int32_t* ids_d;
    const float* w_d;
    rc = upload_request(S, payload, payload_pitch, scales, scales_pitch, ids, weights, rows, &xq_d, &xs_d, &ids_d, &w_d, err, errlen);
    if (rc) return rc;
    for (int r = 0; r < X->world; ++r)
        if (!X->peers.window[r]) { set_msg(err, errlen, "m26b ffn_tp: the exchange is not connected to every peer"); return 1; }
    uint16_t* const plane = static_cast<uint16_t*>(m26b_exchange_plane(X));
    M26B_CK(cudaEventRecord(S->e0, S->st), "m26b event 0");
    const bool fused = passes == 1 && uint64_t(rows) * kHidden * 4 <= X->push.cap;
    const PushSink sink{X, S->tp_sum.as<float>(), nullptr};
    if (fused) {
        rc = enqueue_pass(L, S, xq_d, xs_d, ids_d, w_d, rows, nullptr, nullptr, S->status.as<Status>(), S->st, false, err, errlen,
                          nullptr, false, nullptr, &sink);
        if (rc) return rc;
    }
    for (uint32_t ps = 0; ps < (fused ? 0u : passes); ++ps) {
        const uint32_t r0 = ps * kMaxPassRows, n = rows - r0 < kMaxPassRows ? rows - r0 : kMaxPassRows;
        rc = enqueue_pass(L, S, xq_d + size_t(r0) * kHidden, xs_d + size_t(r0) * (kHidden / kBlockK), ids_d + size_t(r0) * kTopK,
                          w_d + size_t(r0) * kTopK, n, plane + size_t(r0) * kHidden, nullptr, S->status.as<Status>() + ps, S->st,
                          false, err, errlen);
        if (rc) return rc;
    }
    if (!fused) {
        rc = m26b_exchange_sum_residual_dev(X, uint64_t(rows) * kHidden, nullptr, S->tp_sum.as<float>(), S->st, err, errlen);
        if (rc) return rc;
    }
    M26B_CK(cudaEventRecord(S->e1, S->st), "m26b event 1");
    if (sum_out)
        M26B_CK(cudaMemcpyAsync(sum_out, S->tp_sum.p, size_t(rows) * kHidden * 4, cudaMemcpyDeviceToHost, S->st), "m26b sum download");
    M26B_CK(cudaMemcpyAsync(S->hstatus, S->status.p, sizeof(Status) * passes, cudaMemcpyDeviceToHost, S->st), "m26b status download");
    // the exchange's error word rides in the unused tail of the pinned status block
    uint32_t* xerr = reinterpret_cast<uint32_t*>(S->hstatus + 63) + 15;
    M26B_CK(cudaMemcpyAsync(xerr, &static_cast<ExchangeWindow*>(X->window)->error, 4, cudaMemcpyDeviceToHost, S->st), "m26b exchange status");
    const auto t1 = std::chrono::steady_clock::now();
    M26B_CK(cudaStreamSynchronize(S->st), "m26b compute sync");
    S->pending = false;
    rc = decode_status(S->hstatus, passes, err, errlen);
    if (rc) return rc;
    if (*xerr) return m26b_exchange_status(X, S->st, err, errlen);      // clears the word and words the message
    if (ms) {
        float gpu_ms = 0.f;
        cudaEventElapsedTime(&gpu_ms, S->e0, S->e1);
        ms[0] = std::chrono::duration<float, std::milli>(t1 - t0).count();
        ms[1] = gpu_ms;
        const float tail = std::chrono::duration<float, std::milli>(std::chrono::steady_clock::now() - t1).count() - gpu_ms;
        ms[2] = tail > 0.f ? tail : 0.f;
        ms[3] = float(S->hstatus[0].meta.n_tiles);
        ms[4] = ms[5] = ms[6] = ms[7] = 0.f;
    }
    return 0;
}

// The same for a rank of an expert-parallel group: this rank's block of the step's tokens goes up (quantised rows, ids,
// weights), the three phases of the step run on the scratch's stream, and the rank's BF16 result rows come back.
int m26b_ep_ffn(m26b_ep* E, const m26b_layer* L, m26b_scratch* S, const uint8_t* payload, size_t payload_pitch,
                const uint8_t* scales, size_t scales_pitch, const int32_t* ids, const float* weights, uint32_t rows,
                uint16_t* bf16_out, char* err, size_t errlen) {
    if (!E || !L || !S || payload_pitch < kHidden || scales_pitch < kHidden / kBlockK || rows != E->lo[E->rank + 1] - E->lo[E->rank] ||
        (rows && (!payload || !scales || !ids || !weights || !bf16_out))) {
        set_msg(err, errlen, "m26b ep_ffn: bad rows/handles/pitch (rows must be this rank's token block)");
        return 1;
    }
    if (!device_ok(E->device, err, errlen) || !device_ok(S->device, err, errlen)) return 1;
    cudaError_t e;
    int rc;
    const uint8_t* xq_d = nullptr;
    const uint8_t* xs_d = nullptr;
    const int32_t* ids_d = nullptr;
    const float* w_d = nullptr;
    if (rows) {
        rc = upload_request(S, payload, payload_pitch, scales, scales_pitch, ids, weights, rows, &xq_d, &xs_d, &ids_d, &w_d, err, errlen);
        if (rc) return rc;
        M26B_CK(S->gather.ensure(size_t(rows) * kHidden * 2), "m26b out alloc");
    }
    // a rank without tokens still takes part in the step's rendezvous; begin_dev needs non-null pointers only for rows > 0
    static const uint8_t kNone[16] = {};
    rc = m26b_ep_begin_dev(E, rows ? static_cast<const void*>(xq_d) : kNone, 2, rows ? xs_d : kNone, 0,
                           rows ? ids_d : reinterpret_cast<const int32_t*>(kNone), rows ? w_d : reinterpret_cast<const float*>(kNone), rows,
                           S->st, err, errlen);
    if (rc) return rc;
    rc = m26b_ep_compute_dev(E, L, S, S->st, err, errlen);
    if (rc) return rc;
    if (rows) {
        rc = m26b_ep_finish_dev(E, S->gather.as<uint16_t>(), nullptr, S->st, err, errlen);
        if (rc) return rc;
        M26B_CK(cudaMemcpyAsync(bf16_out, S->gather.p, size_t(rows) * kHidden * 2, cudaMemcpyDeviceToHost, S->st), "m26b bf16 download");
    }
    rc = m26b_scratch_status(S, S->st, err, errlen);
    if (rc) return rc;
    return m26b_ep_status(E, S->st, err, errlen);
}

// ---- DS41RTE3 v3 frames ----------------------------------------------------------------------
uint64_t m26b_frame_request_bytes(uint32_t rows) {
    return m26b_frame::kHeaderLen + uint64_t(rows) * (m26b_frame::kDescLen + kTopK * m26b_frame::kRouteLen + m26b_frame::kHiddenRow);
}
uint64_t m26b_frame_return_bytes(uint32_t rows) { return m26b_frame::kHeaderLen + uint64_t(rows) * m26b_frame::kReturnRow; }
uint32_t m26b_frame_crc32c(const uint8_t* bytes, uint64_t n) { return m26b_frame::crc32c(bytes, size_t(n)); }
uint32_t m26b_frame_crc32c_table(const uint8_t* bytes, uint64_t n) { return m26b_frame::crc32c_table(bytes, size_t(n)); }

int m26b_frame_encode_request(uint8_t* out, uint64_t cap, uint64_t request_id, uint32_t layer_id, uint64_t executor_id, uint64_t seq,
                              const uint8_t* payload, size_t payload_pitch, const uint8_t* scales, size_t scales_pitch,
                              const int32_t* ids, const float* weights, uint32_t rows, int seal, uint64_t* len_out, char* err,
                              size_t errlen) {
    using namespace m26b_frame;
    if (!out || !payload || !scales || !ids || !weights || !rows || payload_pitch < kHidden || scales_pitch < kHidden / kBlockK) {
        set_msg(err, errlen, "m26b frame: bad arguments");
        return 1;
    }
    const uint64_t need = m26b_frame_request_bytes(rows);
    if (cap < need) {
        if (err && errlen) std::snprintf(err, errlen, "m26b frame: buffer too short: need %llu bytes, got %llu", (unsigned long long)need, (unsigned long long)cap);
        return 1;
    }
    const uint64_t routes = uint64_t(rows) * kTopK;
    Header h{};
    h.kind = kKindRequest; h.request_id = request_id; h.placement_version = 1; h.layer_id = layer_id; h.row_count = rows;
    h.dim = kHidden; h.dtype = kDtypeUe8m0K32; h.source_kind = 1; h.route_count = uint32_t(routes);
    h.desc_bytes = uint32_t(rows * kDescLen); h.route_bytes = uint32_t(routes * kRouteLen); h.payload_bytes = uint64_t(rows) * kHiddenRow;
    h.logical_bytes = uint64_t(rows) * (kDescLen + kTopK * kRouteLen + kHiddenRow); h.wire_bytes = need; h.flags = 0;
    h.row_stride = uint32_t(kHiddenRow); h.status = 0; h.executor_id = executor_id; h.token_position = 0; h.seq = seq;
    write_header(out, h);
    uint8_t* desc = out + kHeaderLen;
    uint8_t* route = desc + size_t(rows) * kDescLen;
    uint8_t* hidden = route + routes * kRouteLen;
    for (uint32_t t = 0; t < rows; ++t) {
        uint8_t* d = desc + size_t(t) * kDescLen;
        std::memset(d, 0, kDescLen);
        put64(d, 0, t); put16(d, 8, 1); put64(d, 12, request_id); put64(d, 20, t); put32(d, 28, t * kTopK); put32(d, 32, kTopK);
        for (uint32_t k = 0; k < uint32_t(kTopK); ++k) {
            uint8_t* r = route + (size_t(t) * kTopK + k) * kRouteLen;
            uint32_t wbits;
            std::memcpy(&wbits, &weights[size_t(t) * kTopK + k], 4);
            put32(r, 0, t); put32(r, 4, uint32_t(ids[size_t(t) * kTopK + k])); put32(r, 8, wbits);
        }
        std::memcpy(hidden + size_t(t) * kHiddenRow, payload + size_t(t) * payload_pitch, kHidden);
        std::memcpy(hidden + size_t(t) * kHiddenRow + kHidden, scales + size_t(t) * scales_pitch, kHidden / kBlockK);
    }
    if (seal) put32(out, oCrc, frame_crc(out, size_t(need)));
    if (len_out) *len_out = need;
    return 0;
}

// The checks serve_frame makes on a request, without running it (RequestView::parse + serve_b1_view's shape rules).
int m26b_frame_check_request(const uint8_t* request, uint64_t request_len, int check_crc, uint32_t* rows, uint64_t* request_id,
                             uint32_t* layer_id, char* err, size_t errlen) {
    using namespace m26b_frame;
    if (!request) { set_msg(err, errlen, "m26b frame: null frame"); return 1; }
    RequestView v{};
    char msg[160];
    if (const char* e = parse_request(request, size_t(request_len), check_crc != 0, v, msg, sizeof msg)) {
        if (err && errlen) std::snprintf(err, errlen, "m26b frame: %s", e);
        return 6;
    }
    if (v.h.row_stride != kHiddenRow) {
        if (err && errlen) std::snprintf(err, errlen, "serve b1: hidden row stride %u is not 4,096 E4M3 + 128 scales", v.h.row_stride);
        return 6;
    }
    for (uint32_t i = 0; i < v.h.row_count; ++i) {
        const uint8_t* d = v.desc + size_t(i) * kDescLen;
        if (get32(d, 32) != uint32_t(kTopK)) {
            if (err && errlen) std::snprintf(err, errlen, "serve b1: row %u has %u routes, want 8", i, get32(d, 32));
            return 6;
        }
        for (uint32_t j = 0; j < uint32_t(kTopK); ++j)
            if (get32(v.routes + size_t(get32(d, 28) + j) * kRouteLen, 0) != i) {
                if (err && errlen) std::snprintf(err, errlen, "serve b1: route row %u under row %u", get32(v.routes + size_t(get32(d, 28) + j) * kRouteLen, 0), i);
                return 6;
            }
    }
    if (rows) *rows = v.h.row_count;
    if (request_id) *request_id = v.h.request_id;
    if (layer_id) *layer_id = v.h.layer_id;
    return 0;
}

// One request frame in, one return frame out: the rank's whole job for a request
// (crates/mimo26-spark/src/serve.rs:206-246 serve_b1_view, then the return header of
// crates/mimo26-wire/src/frame.rs:987-1030 and the seal). The hidden rows are read in place at the frame's stride.
int m26b_serve_frame(const m26b_layer* L, m26b_scratch* S, const uint8_t* request, uint64_t request_len, uint8_t* reply,
                     uint64_t reply_cap, uint64_t* reply_len, int check_crc, uint64_t reply_seq, float* ms, char* err,
                     size_t errlen) {
    using namespace m26b_frame;
    if (!L || !S || !request || !reply) { set_msg(err, errlen, "m26b serve: null handle or buffer"); return 1; }
    RequestView v{};
    char msg[160];
    if (const char* e = parse_request(request, size_t(request_len), check_crc != 0, v, msg, sizeof msg)) {
        if (err && errlen) std::snprintf(err, errlen, "m26b serve: %s", e);
        return 6;
    }
    const uint32_t rows = v.h.row_count;
    if (v.h.row_stride != kHiddenRow) {
        if (err && errlen) std::snprintf(err, errlen, "serve b1: hidden row stride %u is not 4,096 E4M3 + 128 scales", v.h.row_stride);
        return 6;
    }
    const uint64_t need = m26b_frame_return_bytes(rows);
    if (reply_cap < need) {
        if (err && errlen) std::snprintf(err, errlen, "m26b serve: reply buffer too short: need %llu bytes, got %llu", (unsigned long long)need, (unsigned long long)reply_cap);
        return 1;
    }
    std::vector<int32_t> ids(size_t(rows) * kTopK);
    std::vector<float> weights(size_t(rows) * kTopK);
    for (uint32_t i = 0; i < rows; ++i) {
        const uint8_t* d = v.desc + size_t(i) * kDescLen;
        if (get32(d, 32) != uint32_t(kTopK)) {
            if (err && errlen) std::snprintf(err, errlen, "serve b1: row %u has %u routes, want 8", i, get32(d, 32));
            return 6;
        }
        const uint32_t off = get32(d, 28);
        for (uint32_t j = 0; j < uint32_t(kTopK); ++j) {
            const uint8_t* r = v.routes + size_t(off + j) * kRouteLen;
            if (get32(r, 0) != i) {
                if (err && errlen) std::snprintf(err, errlen, "serve b1: route row %u under row %u", get32(r, 0), i);
                return 6;
            }
            ids[size_t(i) * kTopK + j] = int32_t(get32(r, 4));
            const uint32_t wbits = get32(r, 8);
            std::memcpy(&weights[size_t(i) * kTopK + j], &wbits, 4);
        }
    }
    uint16_t* rows_out = reinterpret_cast<uint16_t*>(reply + kHeaderLen);   // 128 bytes in: 2-byte aligned if `reply` is
    const int rc = m26b_ffn(L, S, v.hidden, kHiddenRow, v.hidden + kHidden, kHiddenRow, ids.data(), weights.data(), rows, rows_out, ms,
                            err, errlen);
    if (rc) return rc;
    Header h{};
    h.kind = kKindReturn; h.request_id = v.h.request_id; h.placement_version = v.h.placement_version; h.layer_id = v.h.layer_id;
    h.row_count = rows; h.dim = kHidden; h.dtype = kDtypeBf16; h.source_kind = 1; h.route_count = kTopK; h.desc_bytes = 0; h.route_bytes = 0;
    h.payload_bytes = uint64_t(rows) * kReturnRow; h.logical_bytes = h.payload_bytes; h.wire_bytes = need; h.flags = kFlagReturnRequired;
    h.row_stride = uint32_t(kReturnRow); h.status = 0; h.executor_id = v.h.executor_id; h.token_position = v.h.token_position; h.seq = reply_seq;
    write_header(reply, h);
    if (check_crc) put32(reply, oCrc, frame_crc(reply, size_t(need)));
    if (reply_len) *reply_len = need;
    return 0;
}

// Coordinator side of a return frame: header checks (kind, status, the two flags an Ok return must carry, BF16 rows of
// 8,192 bytes) and the offset of the rows (crates/mimo26-wire/src/frame.rs:1127-1180 decode_return).
int m26b_frame_parse_return(const uint8_t* frame, uint64_t len, int check_crc, uint64_t* request_id, uint32_t* layer_id,
                            uint32_t* rows, uint32_t* status, uint64_t* seq, uint64_t* rows_offset, char* err, size_t errlen) {
    using namespace m26b_frame;
    if (!frame) { set_msg(err, errlen, "m26b frame: null frame"); return 1; }
    Header h{};
    char msg[160];
    if (const char* e = parse_header(frame, size_t(len), h, msg, sizeof msg)) {
        if (err && errlen) std::snprintf(err, errlen, "m26b frame: %s", e);
        return 6;
    }
    auto bad = [&](const char* what) { if (err && errlen) std::snprintf(err, errlen, "m26b frame: %s", what); return 6; };
    if (check_crc && frame_crc(frame, size_t(len)) != get32(frame, oCrc)) return bad("corrupt frame: CRC32C mismatch");
    if (h.kind != kKindReturn) return bad("not a return frame");
    if (h.status == 0 && (h.flags & kFlagReturnRequired) != kFlagReturnRequired) return bad("return frame is not a pre-summed compact BF16 return");
    if (h.row_count == 0 || h.dim != uint32_t(kHidden) || h.dtype != kDtypeBf16 || h.row_stride != kReturnRow ||
        h.payload_bytes != uint64_t(h.row_count) * kReturnRow || len != kHeaderLen + h.payload_bytes)
        return bad("return frame geometry is not rows x 8,192 bytes of BF16");
    if (request_id) *request_id = h.request_id;
    if (layer_id) *layer_id = h.layer_id;
    if (rows) *rows = h.row_count;
    if (status) *status = h.status;
    if (seq) *seq = h.seq;
    if (rows_offset) *rows_offset = kHeaderLen;
    return 0;
}

int m26b_scratch_timings(m26b_scratch* S, float* ms6, char* err, size_t errlen) {
    if (!S || !ms6 || !S->kev_valid) { set_msg(err, errlen, "m26b timings: enable debug flag 2 and run a pass first"); return 1; }
    cudaError_t e;
    M26B_CK(cudaEventSynchronize(S->kev[6]), "m26b timings sync");
    ms6[0] = 0.f;
    if (S->kev_quant) M26B_CK(cudaEventElapsedTime(&ms6[0], S->kev[0], S->kev[1]), "m26b timings");
    for (int i = 1; i < 6; ++i) M26B_CK(cudaEventElapsedTime(&ms6[i], S->kev[i], S->kev[i + 1]), "m26b timings");
    return 0;
}

// ---- allocation-free route planner ---------------------------------------------------------
// Scratch of m26b_plan_static: per-CTA expert counts, the expert table, token tiles and work
// items of the plan, and an identity slot table (every expert held). It lives in the library's data segment on every
// GPU that loads the library (about 0.47 MB) instead of coming from cudaMalloc.
namespace {
constexpr uint32_t kStaticPlanMaxRows = 4096;
constexpr size_t kStaticPlanTiles = size_t(kStaticPlanMaxRows) * kTopK / 32 + kExperts;
struct StaticPlanScratch {
    uint32_t cta_cnt[128 * kExperts];
    ExpertPlan experts[kExperts];
    TokenTile tiles[kStaticPlanTiles];
    WorkItem items_fc1[kStaticPlanTiles * (kInter / kTileM)];
    WorkItem items_fc2[kStaticPlanTiles * (kHidden / kPairM)];
    int16_t slots[kExperts];
};
}  // namespace
static __device__ __align__(256) unsigned char g_static_plan_scratch[sizeof(StaticPlanScratch)];
static __global__ void identity_slots_kernel(int16_t* slots) { slots[threadIdx.x] = int16_t(threadIdx.x); }

int m26b_plan_static(const int32_t* ids, const float* weights, uint32_t rows, int32_t* inverse, int32_t* original_routes,
                     float* grouped_weights, uint32_t* meta_out, void* stream, char* err, size_t errlen) {
    if (!ids || !weights || !inverse || !original_routes || !grouped_weights || !meta_out || !rows) {
        set_msg(err, errlen, "m26b plan_static: bad arguments");
        return 1;
    }
    if (rows > kStaticPlanMaxRows) {
        if (err && errlen)
            std::snprintf(err, errlen, "m26b plan_static: %u rows exceed the built-in scratch (at most %u rows per call)", rows,
                          kStaticPlanMaxRows);
        return 1;
    }
    cudaError_t e;
    int dev = -1;
    M26B_CK(cudaGetDevice(&dev), "m26b plan_static device");
    if (dev < 0 || dev >= 64) { set_msg(err, errlen, "m26b plan_static: device ordinal out of range"); return 1; }
    // In host code the array's name only stands for the symbol; the device address has to be asked for, once
    // per device, with that device current.
    static StaticPlanScratch* addr[64] = {};
    if (!addr[dev]) {
        void* p = nullptr;
        M26B_CK(cudaGetSymbolAddress(&p, g_static_plan_scratch), "m26b plan_static scratch address");
        addr[dev] = static_cast<StaticPlanScratch*>(p);
    }
    StaticPlanScratch* sc = addr[dev];
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    PlanMeta* meta = reinterpret_cast<PlanMeta*>(meta_out);
    // the array keeps the previous call's contents: the fault word and the residency table are rewritten
    // here, every other field is overwritten by the kernels before it is read
    M26B_CK(cudaMemsetAsync(meta, 0, sizeof(PlanMeta), st), "m26b plan_static clear");
    identity_slots_kernel<<<1, kExperts, 0, st>>>(sc->slots);      // every expert counts as held: slot e for expert e
    const uint32_t routes = rows * kTopK;
    const LaunchClass lc = launch_class(rows);
    const uint32_t slabs = (routes + 1023u) / 1024u;
    const uint32_t n_cta = slabs < 128u ? slabs : 128u;
    const uint32_t cta_routes = ((slabs + n_cta - 1u) / n_cta) * 1024u;
    PlanOut po{inverse, original_routes, grouped_weights, sc->experts, sc->tiles, sc->items_fc1, sc->items_fc2, meta};
    const PlanScope scope{sc->slots, 0u, rows, 0};
    plan_count_kernel<<<n_cta, 1024, 0, st>>>(ids, weights, rows, scope, cta_routes, sc->cta_cnt, meta);
    plan_scan_kernel<<<1, 1024, 0, st>>>(n_cta, sc->cta_cnt, lc.max_n, kInter / kTileM, kHidden / kPairM, 1, 1, sc->slots, po);
    plan_place_kernel<<<n_cta, 1024, 0, st>>>(ids, weights, rows, cta_routes, sc->cta_cnt, po, scope);
    M26B_CK(cudaGetLastError(), "m26b plan_static launch");
    return 0;
}

int m26b_scratch_peek(m26b_scratch* S, int what, void* host_dst, uint64_t bytes, char* err, size_t errlen) {
    if (!S || !host_dst || !S->last_rows) { set_msg(err, errlen, "m26b peek: nothing to read"); return 1; }
    cudaError_t e;
    M26B_CK(cudaDeviceSynchronize(), "m26b peek sync");
    const uint64_t rows = S->last_rows, routes = rows * kTopK, il = uint64_t(S->last_i_local);
    const void* src = nullptr;
    uint64_t have = 0;
    switch (what) {
        case M26B_PEEK_META: src = S->status.p; have = 32; break;
        case M26B_PEEK_INVERSE: src = S->inverse.p; have = routes * 4; break;
        case M26B_PEEK_ORIGINAL_ROUTES: src = S->original.p; have = routes * 4; break;
        case M26B_PEEK_GROUPED_WEIGHTS: src = S->gweights.p; have = routes * 4; break;
        case M26B_PEEK_X_PAYLOAD: src = S->last_xq; have = rows * kHidden; break;
        case M26B_PEEK_X_SCALES: src = S->last_xs; have = rows * (kHidden / kBlockK); break;
        case M26B_PEEK_MID_PAYLOAD: src = S->mid_q.p; have = routes * il; break;
        case M26B_PEEK_MID_F32: src = (S->debug & 1u) ? S->mid_f32.p : nullptr; have = routes * il * 4; break;
        case M26B_PEEK_Y: src = S->y.p; have = routes * kHidden * (S->last_y16 ? 2 : 4); break;
        case M26B_PEEK_PARTIAL: src = S->partial.p; have = rows * kHidden * 4; break;
        case M26B_PEEK_MID_SCALES: {
            // gather the scale blocks back to row-major [routes][il/32] on the host
            if (bytes != routes * (il / kBlockK)) { set_msg(err, errlen, "m26b peek: size mismatch"); return 1; }
            std::vector<ExpertPlan> ep(kExperts);
            std::vector<int32_t> orig(routes), hid(routes);
            std::vector<uint8_t> blocks(S->mid_sf.n);
            M26B_CK(cudaMemcpy(ep.data(), S->experts.p, kExperts * sizeof(ExpertPlan), cudaMemcpyDeviceToHost), "m26b peek copy");
            M26B_CK(cudaMemcpy(orig.data(), S->original.p, routes * 4, cudaMemcpyDeviceToHost), "m26b peek copy");
            M26B_CK(cudaMemcpy(hid.data(), S->last_ids, routes * 4, cudaMemcpyDeviceToHost), "m26b peek copy");
            M26B_CK(cudaMemcpy(blocks.data(), S->mid_sf.p, S->mid_sf.n, cudaMemcpyDeviceToHost), "m26b peek copy");
            uint8_t* dst = static_cast<uint8_t*>(host_dst);
            const uint64_t chunks = il / kChunkK;
            for (uint64_t g = 0; g < routes; ++g) {
                const ExpertPlan& p = ep[hid[orig[g]]];
                const uint64_t local = g - uint64_t(p.rbase), tile = uint64_t(p.tile_start) + local / uint64_t(p.width);
                const uint64_t lr = local % uint64_t(p.width);
                for (uint64_t b = 0; b < il / kBlockK; ++b)
                    dst[g * (il / kBlockK) + b] = blocks[(tile * chunks + b / 4) * kScaleBlockBytes + scale_block_offset(int(lr), int(b & 3))];
            }
            return 0;
        }
        default: break;
    }
    if (!src || bytes != have) { set_msg(err, errlen, "m26b peek: unknown buffer or size mismatch"); return 1; }
    M26B_CK(cudaMemcpy(host_dst, src, bytes, cudaMemcpyDeviceToHost), "m26b peek copy");
    return 0;
}

}  // extern "C"
