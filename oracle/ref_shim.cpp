// C entry points over the reference's own host-compilable B1 units, so the
// Python tests can call them through ctypes. TEST INFRASTRUCTURE ONLY: this
// file is compiled together with the reference sources where they lie
// (crates/mimo26-expert/kernels/b1/{quant_v1,group_plan,route_reduce,prepare}.cu,
// built as C++ exactly as the reference's own host tests do,
// crates/mimo26-expert/tests/b1/run.py:141-143). Nothing from the reference is
// copied into this repository; the output goes to oracle/_ref/.
#include <cstdint>
#include "quant_v1.cuh"
#include "group_plan.cuh"
#include "route_reduce.cuh"

extern "C" {

// quantize_host (kernels/b1/quant_v1.cu:23-32). Returns the Status value.
uint32_t ref_quantize_host(const float* values, uint64_t elements, uint8_t* payload, uint8_t* scales,
                           uint32_t* block_faults) {
    const m26b1::QuantInput in{values, elements};
    const m26b1::QuantOutput out{payload, scales, block_faults, elements, elements / 32, elements / 32};
    return static_cast<uint32_t>(m26b1::quantize_host(in, out));
}

// plan_host (kernels/b1/group_plan.cu:80-86). capacity in {256, 2048, 4096}; all
// arrays sized capacity*8 (groups: capacity*8*19 int32). Returns the Status value.
uint32_t ref_plan_host(uint32_t capacity, uint32_t rows, const int32_t* ids, const float* weights,
                       const uint8_t* resident, int32_t* inverse, int32_t* original_routes, float* grouped_weights,
                       int32_t* groups, uint32_t* group_count, uint32_t* fault) {
    const uint64_t cap = uint64_t(capacity) * 8;
    const m26b1::PlanInput in{capacity, rows, ids, weights, uint64_t(rows) * 8, resident, 256};
    const m26b1::PlanStorage st{inverse, original_routes, grouped_weights, reinterpret_cast<m26b1::Group*>(groups),
                                group_count, fault, cap, cap};
    return static_cast<uint32_t>(m26b1::plan_host(in, st));
}

// reduce_host (kernels/b1/route_reduce.cu:75-90). Returns the Status value.
uint32_t ref_reduce_host(uint32_t rows, const float* unweighted, const float* weights, float* partial, uint16_t* bf16,
                         uint32_t* fault) {
    const uint64_t n = uint64_t(rows) * 4096;
    const m26b1::RouteInput in{rows, unweighted, weights, n * 8, uint64_t(rows) * 8};
    const m26b1::RankOutput out{partial, bf16, n, n, fault};
    return static_cast<uint32_t>(m26b1::reduce_host(in, out));
}

}  // extern "C"
