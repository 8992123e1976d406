// Stand-alone probe of the tensor-core primitive the expert GEMMs are built on:
// tcgen05.mma kind::mxf8f6f4.block_scale with A = E2M1 (4-bit weights unpacked by a
// 16U4_ALIGN16B tensor map) and B = E4M3, UE8M0 scales in tensor memory.
// Part 1: correctness of one 128 x 32 x 256 tile against a double-precision loop, plus dumps
//         of the unpacked shared-memory tile and of the scale columns in tensor memory.
// Part 2: the dense MMA rate the roofline is normalised by - cycles per MMA for N = 16..256 on
//         one SM (operands resident in shared memory), and the chip-wide TFLOP/s at N = 128 / 256.
// Build and run (one B200, a few seconds):
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -o mma_rate_probe mma_rate_probe.cu && ./mma_rate_probe
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <cmath>
#include <vector>
#include "sm100_ptx.cuh"
using namespace m26b;

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); exit(2); } } while (0)

typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                             const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                             CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeFn get_encode() {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
    if (!fn) { printf("no cuTensorMapEncodeTiled\n"); exit(2); }
    return (EncodeFn)fn;
}

constexpr int KTOT = 256;     // two K128 chunks
constexpr int NB = 32;        // tokens (B rows) in the correctness tile

struct SmemProbe {
    alignas(1024) uint8_t a[2][128 * 128];   // 16 KB per chunk (unpacked containers)
    alignas(1024) uint8_t b[2][NB * 128];
    alignas(16) uint8_t sfa[2][512];
    alignas(16) uint8_t sfb[2][512];
    uint64_t full[2];
    uint64_t done;
    uint32_t tmem_base;
    uint32_t abort_flag;
};

__global__ void __launch_bounds__(128) probe_correct(const __grid_constant__ CUtensorMap map_a,
                                                     const __grid_constant__ CUtensorMap map_b,
                                                     const uint8_t* sfa_g, const uint8_t* sfb_g, float* d_out,
                                                     uint8_t* smem_dump, uint32_t* sf_dump, uint32_t* err,
                                                     uint32_t a_fmt) {
    extern __shared__ uint8_t raw[];
    SmemProbe& s = *reinterpret_cast<SmemProbe*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    if (threadIdx.x == 0) {
        mbar_init(&s.full[0], 1); mbar_init(&s.full[1], 1); mbar_init(&s.done, 1);
        s.abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 0) { tmem_alloc(&s.tmem_base, 64); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tb = s.tmem_base;
    const uint32_t t_acc = tb, t_sfa = tb + 32, t_sfb = tb + 40;
    if (warp == 0 && elect_one()) {
        for (int c = 0; c < 2; ++c) {
            mbar_expect_tx(&s.full[c], 128 * 64 + NB * 128 + 512 + 512);  // the 4-bit tile counts its packed bytes
            tma_load_2d(s.a[c], &map_a, c * 128, 0, &s.full[c]);
            tma_load_2d(s.b[c], &map_b, c * 128, 0, &s.full[c]);
            bulk_load(s.sfa[c], sfa_g + c * 512, 512, &s.full[c]);
            bulk_load(s.sfb[c], sfb_g + c * 512, 512, &s.full[c]);
        }
    }
    if (warp == 1 && elect_one()) {
        bool ok = true;
        for (int c = 0; c < 2 && ok; ++c) {
            ok = mbar_wait(&s.full[c], 0, &s.abort_flag);
            if (!ok) { atomicOr(err, 1u << c); break; }
            tc_fence_after();
            tc_cp_scales(t_sfa + c * 4, desc_scale_block(smem_u32(s.sfa[c])));
            tc_cp_scales(t_sfb + c * 4, desc_scale_block(smem_u32(s.sfb[c])));
            for (int kb = 0; kb < 4; ++kb) {
                const uint64_t ad = desc_sw128(smem_u32(s.a[c]) + kb * 32);
                const uint64_t bd = desc_sw128(smem_u32(s.b[c]) + kb * 32);
                tc_mma_mx(t_acc, ad, bd, idesc_mx(a_fmt, kFmtE4M3, NB, kb, kb), t_sfa + c * 4, t_sfb + c * 4,
                          (c | kb) ? 1u : 0u);
            }
        }
        tc_commit(&s.done);
    }
    __syncwarp();
    // everyone waits for the MMAs
    const bool ok = mbar_wait(&s.done, 0, &s.abort_flag);
    if (!ok && threadIdx.x == 0) atomicOr(err, 0x100u);
    tc_fence_after();
    if (ok) {
        // D: lane = A row, column = B row (token)
        for (int c0 = 0; c0 < NB; c0 += 16) {
            uint32_t r[16];
            tmem_ld16(t_acc + (uint32_t(warp * 32) << 16) + c0, r);
            tmem_wait_ld();
            for (int j = 0; j < 16; ++j) d_out[(warp * 32 + lane) * NB + c0 + j] = __uint_as_float(r[j]);
        }
        uint32_t q[4];
        for (int c = 0; c < 4; ++c) {   // SFA chunk0, SFA chunk1, SFB chunk0, SFB chunk1
            tmem_ld4(t_sfa + c * 4 + (uint32_t(warp * 32) << 16), q);
            tmem_wait_ld();
            for (int j = 0; j < 4; ++j) sf_dump[((warp * 32 + lane) * 4 + c) * 4 + j] = q[j];
        }
    }
    for (int i = threadIdx.x; i < 128 * 128; i += blockDim.x) smem_dump[i] = s.a[0][i];
    for (int i = threadIdx.x; i < NB * 128; i += blockDim.x) smem_dump[128 * 128 + i] = s.b[0][i];
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tb, 64);
}

// ---- rate probe --------------------------------------------------------------
struct SmemRate {
    alignas(1024) uint8_t a[4][128 * 128];
    alignas(1024) uint8_t b[4][256 * 128];
    alignas(16) uint8_t sf[512];
    uint64_t done;
    uint32_t tmem_base;
    uint32_t abort_flag;
};

// `random_data`: operands are pseudo-random bytes (every E2M1 code, every finite E4M3 code) instead of a few small
// codes. The tensor pipe's rate per clock does not depend on the data, its power draw does, and with it the clock
// the GPU holds under its power limit.
__global__ void __launch_bounds__(128) probe_rate(uint32_t n, uint32_t iters, uint32_t a_fmt, uint32_t two_a,
                                                  long long* cycles, uint32_t* err, uint32_t random_data = 0) {
    extern __shared__ uint8_t raw[];
    SmemRate& s = *reinterpret_cast<SmemRate*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x / 32;
    // fill operands with small valid codes: E4M3 0x38 (=1.0) pattern mixed, E2M1 containers
    for (int i = threadIdx.x; i < int(sizeof(s.a)); i += blockDim.x) (&s.a[0][0])[i] = uint8_t((i * 37 + 11) & 0x33);
    for (int i = threadIdx.x; i < int(sizeof(s.b)); i += blockDim.x) (&s.b[0][0])[i] = uint8_t((i * 29 + 5) & 0x33);
    for (int i = threadIdx.x; i < 512; i += blockDim.x) s.sf[i] = 120;
    if (random_data) {
        auto mix = [](uint32_t v) { v ^= v >> 16; v *= 0x7feb352du; v ^= v >> 15; v *= 0x846ca68bu; v ^= v >> 16; return v; };
        for (int i = threadIdx.x; i < int(sizeof(s.a)); i += blockDim.x) (&s.a[0][0])[i] = uint8_t(mix(i * 2u + blockIdx.x * 7919u));
        for (int i = threadIdx.x; i < int(sizeof(s.b)); i += blockDim.x) {
            uint8_t v = uint8_t(mix(i * 2u + 1u + blockIdx.x * 104729u));
            if ((v & 0x7f) == 0x7f) v ^= 1;                  // no E4M3 NaN codes
            (&s.b[0][0])[i] = v;
        }
        for (int i = threadIdx.x; i < 512; i += blockDim.x) s.sf[i] = uint8_t(118 + (mix(i) & 7));
    }
    if (threadIdx.x == 0) { mbar_init(&s.done, 1); s.abort_flag = 0; mbar_init_fence(); }
    fence_async_smem();
    if (warp == 0) { tmem_alloc(&s.tmem_base, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tb = s.tmem_base;
    const uint32_t t_sf = tb + 496;   // SFA 4 columns, SFB up to 8
    long long t0 = 0, t1 = 0;
    if (warp == 1 && elect_one()) {
        tc_cp_scales(t_sf, desc_scale_block(smem_u32(s.sf)));
        tc_cp_scales(t_sf + 4, desc_scale_block(smem_u32(s.sf)));
        tc_cp_scales(t_sf + 8, desc_scale_block(smem_u32(s.sf)));
        t0 = clock64();
        for (uint32_t it = 0; it < iters; ++it) {
            const int st = (it >> 2) & 3, kb = it & 3;
            const uint64_t ad = desc_sw128(smem_u32(s.a[st]) + kb * 32);
            const uint64_t bd = desc_sw128(smem_u32(s.b[st]) + kb * 32);
            // two_a: alternate two accumulators with different A tiles and a shared B tile (FC1 gate/up pattern)
            const uint32_t acc = two_a ? ((it & 4) ? n : 0) : 0;
            tc_mma_mx(tb + acc, ad, bd, idesc_mx(a_fmt, kFmtE4M3, n, kb, kb), t_sf, t_sf + 4, it >= 8 ? 1u : 0u);
        }
        tc_commit(&s.done);
        const bool ok = mbar_wait(&s.done, 0, &s.abort_flag);
        t1 = clock64();
        if (!ok) atomicOr(err, 0x200u);
        cycles[blockIdx.x] = t1 - t0;
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tb, 512);
}

static float e2m1_val(int nib) {
    static const float t[8] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
    return (nib & 8) ? -t[nib & 7] : t[nib & 7];
}
static float e4m3_val(int c) {
    const int e = (c >> 3) & 15, m = c & 7;
    const float v = e ? ldexpf(1.f + m / 8.f, e - 7) : ldexpf(float(m), -9);
    return (c & 128) ? -v : v;
}

int main() {
    EncodeFn encode = get_encode();
    cudaDeviceProp prop; CK(cudaGetDeviceProperties(&prop, 0));
    printf("device %s sm_%d%d SMs %d\n", prop.name, prop.major, prop.minor, prop.multiProcessorCount);
    srand(1234);
    std::vector<uint8_t> a_packed(128 * KTOT / 2), a_sc(128 * (KTOT / 32)), b_codes(NB * KTOT), b_sc(NB * (KTOT / 32));
    for (auto& v : a_packed) v = uint8_t(rand() & 255);
    for (auto& v : a_sc) v = uint8_t(118 + rand() % 5);
    for (auto& v : b_codes) { do { v = uint8_t(rand() & 255); } while ((v & 0x7f) == 0x7f); }
    for (auto& v : b_sc) v = uint8_t(120 + rand() % 11);
    // scale blocks in atom order: chunk c -> 512 B, offset (r%32)*16 + (r/32)*4 + kb
    std::vector<uint8_t> sfa(2 * 512, 127), sfb(2 * 512, 127);
    for (int c = 0; c < 2; ++c)
        for (int r = 0; r < 128; ++r)
            for (int kb = 0; kb < 4; ++kb) {
                sfa[c * 512 + (r % 32) * 16 + (r / 32) * 4 + kb] = a_sc[r * 8 + c * 4 + kb];
                if (r < NB) sfb[c * 512 + (r % 32) * 16 + (r / 32) * 4 + kb] = b_sc[r * 8 + c * 4 + kb];
            }
    std::vector<double> ref(128 * NB);
    for (int m = 0; m < 128; ++m)
        for (int n = 0; n < NB; ++n) {
            double acc = 0;
            for (int k = 0; k < KTOT; ++k) {
                const int nib = (a_packed[m * (KTOT / 2) + k / 2] >> (4 * (k & 1))) & 15;
                acc += double(e2m1_val(nib)) * ldexp(1.0, a_sc[m * 8 + k / 32] - 127) *
                       double(e4m3_val(b_codes[n * KTOT + k])) * ldexp(1.0, b_sc[n * 8 + k / 32] - 127);
            }
            ref[m * NB + n] = acc;
        }
    uint8_t *d_a, *d_b, *d_sfa, *d_sfb, *d_dump; float* d_d; uint32_t *d_sf, *d_err;
    CK(cudaMalloc(&d_a, a_packed.size())); CK(cudaMalloc(&d_b, b_codes.size()));
    CK(cudaMalloc(&d_sfa, 1024)); CK(cudaMalloc(&d_sfb, 1024));
    CK(cudaMalloc(&d_dump, 128 * 128 + NB * 128)); CK(cudaMalloc(&d_d, 128 * NB * 4));
    CK(cudaMalloc(&d_sf, 128 * 16 * 4)); CK(cudaMalloc(&d_err, 4));
    CK(cudaMemcpy(d_a, a_packed.data(), a_packed.size(), cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_b, b_codes.data(), b_codes.size(), cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_sfa, sfa.data(), 1024, cudaMemcpyHostToDevice));
    CK(cudaMemcpy(d_sfb, sfb.data(), 1024, cudaMemcpyHostToDevice));
    CK(cudaMemset(d_err, 0, 4)); CK(cudaMemset(d_d, 0xff, 128 * NB * 4)); CK(cudaMemset(d_dump, 0xEE, 128 * 128 + NB * 128));
    CUtensorMap map_a, map_b;
    {
        cuuint64_t dims[2] = {KTOT, 128}; cuuint64_t strides[1] = {KTOT / 2}; cuuint32_t box[2] = {128, 128}; cuuint32_t es[2] = {1, 1};
        CUresult r = encode(&map_a, CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 2, d_a, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        printf("encode A (16U4_ALIGN16B) -> %d\n", int(r)); if (r) return 3;
        cuuint64_t dimsb[2] = {KTOT, NB}; cuuint64_t stridesb[1] = {KTOT}; cuuint32_t boxb[2] = {128, NB};
        r = encode(&map_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, d_b, dimsb, stridesb, boxb, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        printf("encode B (u8) -> %d\n", int(r)); if (r) return 3;
    }
    const int smem1 = sizeof(SmemProbe) + 1024;
    CK(cudaFuncSetAttribute(probe_correct, cudaFuncAttributeMaxDynamicSharedMemorySize, smem1));
    probe_correct<<<1, 128, smem1>>>(map_a, map_b, d_sfa, d_sfb, d_d, d_dump, d_sf, d_err, kFmtE2M1);
    CK(cudaGetLastError()); CK(cudaDeviceSynchronize());
    uint32_t herr = 0; CK(cudaMemcpy(&herr, d_err, 4, cudaMemcpyDeviceToHost));
    std::vector<float> dh(128 * NB); CK(cudaMemcpy(dh.data(), d_d, dh.size() * 4, cudaMemcpyDeviceToHost));
    std::vector<uint8_t> dump(128 * 128 + NB * 128); CK(cudaMemcpy(dump.data(), d_dump, dump.size(), cudaMemcpyDeviceToHost));
    std::vector<uint32_t> sfd(128 * 16); CK(cudaMemcpy(sfd.data(), d_sf, sfd.size() * 4, cudaMemcpyDeviceToHost));
    printf("probe_correct err=0x%x\n", herr);
    double maxerr = 0, maxref = 0; int bad = 0;
    for (int i = 0; i < 128 * NB; ++i) {
        const double e = fabs(double(dh[i]) - ref[i]); if (e > maxerr) maxerr = e; if (fabs(ref[i]) > maxref) maxref = fabs(ref[i]);
        if (!(e <= 1e-5 * fabs(ref[i]) + 1e-7)) ++bad;
    }
    printf("D vs ref: max abs err %.6g (max |ref| %.6g), elements beyond 1e-5 rel: %d of %d\n", maxerr, maxref, bad, 128 * NB);
    for (int m = 0; m < 3; ++m) { printf("row %d:", m); for (int n = 0; n < 6; ++n) printf(" %.6g/%.6g", dh[m * NB + n], ref[m * NB + n]); printf("\n"); }
    printf("row 33:"); for (int n = 0; n < 6; ++n) printf(" %.6g/%.6g", dh[33 * NB + n], ref[33 * NB + n]); printf("\n");
    printf("row 100:"); for (int n = 26; n < 32; ++n) printf(" %.6g/%.6g", dh[100 * NB + n], ref[100 * NB + n]); printf("\n");
    // smem A dump analysis: expected element (row r, k) at byte r*128 + ((k/16) ^ (r%8))*16 + (k%16)/2 (low nibble even k)
    int mism = 0, gapnz = 0;
    for (int r = 0; r < 128; ++r)
        for (int ch = 0; ch < 8; ++ch) {
            const uint8_t* p = &dump[r * 128 + ((ch ^ (r & 7)) * 16)];
            for (int j = 0; j < 8; ++j) if (p[j] != a_packed[r * (KTOT / 2) + ch * 8 + j]) ++mism;
            for (int j = 8; j < 16; ++j) if (p[j]) ++gapnz;
        }
    printf("smem A tile: packed-byte mismatches vs hypothesis %d, nonzero gap bytes %d\n", mism, gapnz);
    printf("smem A row0 first 64 B:"); for (int i = 0; i < 64; ++i) printf(" %02x", dump[i]); printf("\n");
    printf("gmem A row0 first 32 B:"); for (int i = 0; i < 32; ++i) printf(" %02x", a_packed[i]); printf("\n");
    printf("smem A row1 first 64 B:"); for (int i = 0; i < 64; ++i) printf(" %02x", dump[128 + i]); printf("\n");
    printf("gmem A row1 first 32 B:"); for (int i = 0; i < 32; ++i) printf(" %02x", a_packed[128 + i]); printf("\n");
    int sfbad = 0;
    for (int l = 0; l < 128; ++l)
        for (int c = 0; c < 2; ++c)
            for (int j = 0; j < 4; ++j) {
                uint32_t want = 0;
                for (int kb = 0; kb < 4; ++kb) want |= uint32_t(a_sc[((l % 32) + 32 * j) * 8 + c * 4 + kb]) << (8 * kb);
                if (sfd[(l * 4 + c) * 4 + j] != want) ++sfbad;
            }
    printf("TMEM SFA words differing from hypothesis (lane l word j = rows l%%32+32j, 4 k-blocks): %d of 1024\n", sfbad);
    printf("SFA lane0:"); for (int j = 0; j < 4; ++j) printf(" %08x", sfd[j]); printf("  lane33:"); for (int j = 0; j < 4; ++j) printf(" %08x", sfd[33 * 16 + j]); printf("\n");
    printf("a_sc rows 0,32,64,96 kb0-3: "); for (int j = 0; j < 4; ++j) { for (int kb = 0; kb < 4; ++kb) printf("%02x", a_sc[(32 * j) * 8 + kb]); printf(" "); } printf("\n");

    // rate
    const int smem2 = sizeof(SmemRate) + 1024;
    CK(cudaFuncSetAttribute(probe_rate, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2));
    long long* d_cyc; CK(cudaMalloc(&d_cyc, 8 * 256));
    const uint32_t ns[] = {16, 32, 64, 96, 112, 128, 192, 256};
    for (int two_a = 0; two_a < 2; ++two_a)
        for (uint32_t fmt : {uint32_t(kFmtE2M1), uint32_t(kFmtE4M3)})
            for (uint32_t n : ns) {
                if (two_a && n > 128) continue;
                const uint32_t iters = 4096;
                probe_rate<<<1, 128, smem2>>>(n, iters, fmt, two_a, d_cyc, d_err);
                CK(cudaGetLastError()); CK(cudaDeviceSynchronize());
                long long cyc; CK(cudaMemcpy(&cyc, d_cyc, 8, cudaMemcpyDeviceToHost));
                printf("rate 1CTA afmt=%u two_a=%d N=%3u: %.1f cycles/MMA  -> %.0f MAC/clk/SM\n", fmt, two_a, n, double(cyc) / iters,
                       128.0 * n * 32 * iters / double(cyc));
            }
    // whole chip, sustained: 148 CTAs, N=256 and N=128
    cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    for (uint32_t n : {128u, 256u}) {
        const uint32_t iters = 200000;
        probe_rate<<<prop.multiProcessorCount, 128, smem2>>>(n, 20000, kFmtE2M1, 0, d_cyc, d_err);  // warm
        CK(cudaEventRecord(e0));
        probe_rate<<<prop.multiProcessorCount, 128, smem2>>>(n, iters, kFmtE2M1, 0, d_cyc, d_err);
        CK(cudaEventRecord(e1)); CK(cudaDeviceSynchronize());
        float ms; CK(cudaEventElapsedTime(&ms, e0, e1));
        const double flops = 2.0 * 128 * n * 32 * double(iters) * prop.multiProcessorCount;
        printf("rate chip N=%u: %.3f ms, %.1f TFLOP/s (mxf8f6f4 dense, E2M1 x E4M3)\n", n, ms, flops / ms / 1e9);
    }
    // sustained: back-to-back launches for about three seconds, the rate of the last second and the SM clock in it
    // (cycles of one CTA / the launch's duration), for the small-code operands and for random operands
    for (uint32_t random_data : {0u, 1u}) {
        const uint32_t n = 128, iters = 200000;
        const double flops = 2.0 * 128 * n * 32 * double(iters) * prop.multiProcessorCount;
        double first_tf = 0, last_tf = 0, last_mhz = 0;
        float total = 0;
        for (int rep = 0; total < 3000.f && rep < 2000; ++rep) {
            CK(cudaEventRecord(e0));
            probe_rate<<<prop.multiProcessorCount, 128, smem2>>>(n, iters, kFmtE2M1, 0, d_cyc, d_err, random_data);
            CK(cudaEventRecord(e1)); CK(cudaDeviceSynchronize());
            float ms; CK(cudaEventElapsedTime(&ms, e0, e1));
            long long cyc; CK(cudaMemcpy(&cyc, d_cyc, 8, cudaMemcpyDeviceToHost));
            total += ms;
            if (rep == 0) first_tf = flops / ms / 1e9;
            last_tf = flops / ms / 1e9; last_mhz = double(cyc) / ms / 1e3;
        }
        printf("rate chip sustained N=128 %s operands: first launch %.1f TFLOP/s, after %.1f s %.1f TFLOP/s at %.0f MHz\n",
               random_data ? "random" : "small-code", first_tf, total / 1e3, last_tf, last_mhz);
    }
    CK(cudaMemcpy(&herr, d_err, 4, cudaMemcpyDeviceToHost));
    printf("final err=0x%x\n", herr);
    return 0;
}
