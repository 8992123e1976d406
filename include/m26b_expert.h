/* C ABI of the B200 routed-expert FFN (one MoE layer, one tensor-parallel rank).
 *
 * Drop-in surface for the reference's expert-rank seam
 *   crates/mimo26-spark/kernels/b1_serve.cu:214-574   (extern "C" m26s_b1_*)
 *   crates/mimo26-spark/src/b1.rs:21-49               (the Rust declarations that bind it)
 * with the same conventions: opaque heap handles, plain pointers and sizes,
 * int return codes, a caller-owned NUL-terminated error buffer.
 *
 * Return codes (as b1_serve.cu): 0 ok; 1 bad argument / handle / pitch;
 * 2 CUDA error ("what: cudaGetErrorString"); 3 plan rejected (invalid id,
 * non-resident expert, weight outside [0, FLT_MAX], an expert twice in one row);
 * 4 numerical fault (stage name and fault code in the message). Outputs are
 * undefined on a nonzero return.
 *
 * Threading: handles may move between threads but are not shared; one call at
 * a time per scratch. Every entry point runs on the CUDA device that is
 * current when it is called; a handle must be used on the device it was made on.
 */
#ifndef M26B_EXPERT_H
#define M26B_EXPERT_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct m26b_layer m26b_layer;
typedef struct m26b_scratch m26b_scratch;
typedef struct m26b_exchange m26b_exchange;
typedef struct m26b_ep m26b_ep;

#define M26B_HIDDEN 4096
#define M26B_INTERMEDIATE 2048
#define M26B_EXPERTS 256
#define M26B_TOPK 8

/* Replaces m26s_b1_layer_new (b1_serve.cu:218-265): prepare one layer from the
 * reference's canonical-v2 rank image in device memory, 256 experts x 3,342,336
 * bytes, rank 0..3 of TP4 (crates/mimo26-repack/src/geom.rs:36-50). The image
 * may be freed after the call returns. Every m26b_layer_new* call first waits for all work queued on the current
 * device (cudaDeviceSynchronize), so source tensors produced on any stream are complete before they are repacked. */
int m26b_layer_new(const uint8_t* canonical_dev, uint64_t canonical_bytes, uint32_t rank, m26b_layer** out,
                   char* err, size_t errlen);

/* Same image layout generalised to tp_size in {1,2,4,8}: per expert
 * gate payload [I,2048] | gate scales [I,128] | up payload | up scales |
 * down payload [4096,I/2] | down scales [4096,I/32], I = 2048 / tp_size.
 * tp_size 4 is exactly m26b_layer_new. */
int m26b_layer_new_tp(const uint8_t* canonical_dev, uint64_t canonical_bytes, uint32_t tp_rank, uint32_t tp_size,
                      m26b_layer** out, char* err, size_t errlen);

/* From the checkpoint's own tensors (crates/mimo26-expert/src/mxfp4.rs:13-19),
 * all in device memory and stacked over the 256 experts: gate_proj / up_proj
 * weight u8 [256][2048][2048] + weight_scale u8 [256][2048][128], down_proj
 * weight u8 [256][4096][1024] + weight_scale u8 [256][4096][64]. The rank
 * keeps gate/up rows [tp_rank*I, (tp_rank+1)*I) and the matching down columns
 * (the reference's build_slice, crates/mimo26-repack/src/repack.rs:135-163). */
int m26b_layer_new_from_checkpoint(const uint8_t* gate_w, const uint8_t* gate_s, const uint8_t* up_w,
                                   const uint8_t* up_s, const uint8_t* down_w, const uint8_t* down_s,
                                   uint32_t tp_rank, uint32_t tp_size, m26b_layer** out, char* err, size_t errlen);

/* Replaces m26s_b1_layer_all_normal (b1_serve.cu:267-268): 1 if every weight
 * scale byte lies in [2, 252]. Informational here: the block-scaled MMA takes
 * every UE8M0 byte 0..254, and byte 255 is stored as 254 at prepare time. */
int m26b_layer_all_normal(const m26b_layer* layer);
/* Read-only view of the prepared operand image in device memory, for tests of the repack (the reference proves its
 * prepare step a byte permutation the same way: crates/mimo26-expert/kernels/b1/prepared.cuh:63-88, tests/b1/host.cpp).
 * which: 0 = gate/up payload [E][I/128][256 rows][2048 B] (rows 0..127 gate, 128..255 up of the same 128 features),
 * 1 = gate/up scale blocks [E][I/128][32 chunks][2][512 B], 2 = down payload [E][4096][I/2 B],
 * 3 = down scale blocks [E][16][I/128][2][512 B]; a 512-byte scale block holds rows r = 0..127 x K32 blocks kb = 0..3 of
 * one 128-wide K chunk at byte (r % 32) * 16 + (r / 32) * 4 + kb; 4 = the gate/up scale blocks regrouped for half items
 * [E][I/128][2 halves][32 chunks][512 B]: rows 0..63 of a block are the gate rows 64 h .. 64 h + 63 of the tile, rows
 * 64..127 the up rows of the same features. E = the experts the layer holds, I = its local
 * intermediate width. Returns NULL for a bad argument; *bytes (may be NULL) receives the image size. */
const void* m26b_layer_image(const m26b_layer* layer, int which, uint64_t* bytes);
/* Local intermediate width of the layer (2048 / tp_size). */
int m26b_layer_i_local(const m26b_layer* layer);
/* Replaces m26s_b1_layer_free (b1_serve.cu:270-276). */
void m26b_layer_free(m26b_layer* layer);

/* Replace m26s_b1_scratch_new / _free (b1_serve.cu:278-302): a non-blocking
 * stream, events and grow-only device buffers. */
int m26b_scratch_new(m26b_scratch** out, char* err, size_t errlen);
void m26b_scratch_free(m26b_scratch* scratch);

/* Replaces m26s_b1_ffn (b1_serve.cu:312-572), same arguments: HOST payload rows
 * of 4096 E4M3 bytes at payload_pitch, HOST scale rows of 128 UE8M0 bytes at
 * scales_pitch (4224 for both reads the request frame in place), HOST ids and
 * weights [rows*8] token-major, HOST bf16_out [rows*4096]. Synchronous.
 * rows may exceed the reference's 4096 (larger requests run in passes).
 * ms (or NULL) receives 8 floats: [0] host time to upload and enqueue, [1] GPU
 * time of the FFN, [2] host tail (download, checks), [3] token tiles (the
 * reference reports 16-row groups here), [4] plan+permute+FC1 (the
 * intermediate quantiser is fused into FC1), [5] 0, [6] FC2, [7] combine.
 * [4]..[7] are measured only with debug flag 4 (m26b_scratch_set_debug) and read 0 otherwise: the events between
 * the kernels they need cost the overlap of dependent launches, about 10 us of a 16-token step. */
int m26b_ffn(const m26b_layer* layer, m26b_scratch* scratch, const uint8_t* payload, size_t payload_pitch,
             const uint8_t* scales, size_t scales_pitch, const int32_t* ids, const float* weights, uint32_t rows,
             uint16_t* bf16_out, float* ms, char* err, size_t errlen);

/* Device-resident variant of the same call (the reference's older device-pointer
 * ABI shows the convention: crates/mimo26-expert/kernels/include/mimo26_expert_kernels.h:31-69).
 * x_dtype: 0 = BF16 [rows,4096], 1 = FP32 [rows,4096], 2 = E4M3 payload with x_scales [rows,128].
 * codec (x_dtype 0/1 only): 0 = the coordinator's wire quantiser
 * (crates/mimo26-coordinator/src/wire.rs:53-78), 1 = e4m3fn-k32-v1
 * (crates/mimo26-expert/kernels/b1/quant_v1.cuh).
 * All pointers are device pointers; work is enqueued on `stream` (a
 * cudaStream_t; NULL = the scratch's own stream) and the call returns without
 * synchronising. partial_out (FP32 [rows,4096], the pre-BF16 rank sum) may be
 * NULL. Faults are reported by m26b_scratch_status. rows <= 16384 per call. */
int m26b_ffn_dev(const m26b_layer* layer, m26b_scratch* scratch, const void* x, int x_dtype,
                 const uint8_t* x_scales, int codec, const int32_t* ids, const float* weights, uint32_t rows,
                 uint16_t* bf16_out, float* partial_out, void* stream, char* err, size_t errlen);

/* Waits for the scratch's last m26b_ffn_dev and returns its code (0, 2, 3 or 4). */
int m26b_scratch_status(m26b_scratch* scratch, void* stream, char* err, size_t errlen);

/* Stage dumps for parity tests (the reference's primitive cell dumps stages the
 * same way: crates/mimo26-expert/tests/b1_core/primitive.cu:173-196).
 * flags bit 0: keep an FP32 copy of silu(gate)*up before quantisation; bit 1: record per-kernel events;
 * bit 2 (value 4): m26b_ffn splits its GPU time into stages (ms[4..7]). */
int m26b_scratch_set_debug(m26b_scratch* scratch, uint32_t flags);
enum {
    M26B_PEEK_META = 0,            /* 8 x u32: fault, tiles, fc1 items, fc2 items, active experts, max count */
    M26B_PEEK_INVERSE = 1,         /* i32 [routes]  original route -> grouped route  (group_plan.cuh:19) */
    M26B_PEEK_ORIGINAL_ROUTES = 2, /* i32 [routes]  grouped route -> original route  (group_plan.cuh:20) */
    M26B_PEEK_GROUPED_WEIGHTS = 3, /* f32 [routes] */
    M26B_PEEK_X_PAYLOAD = 4,       /* u8 [rows,4096] quantised input */
    M26B_PEEK_X_SCALES = 5,        /* u8 [rows,128] */
    M26B_PEEK_MID_PAYLOAD = 6,     /* u8 [routes,I_local] grouped order */
    M26B_PEEK_MID_F32 = 7,         /* f32 [routes,I_local] grouped order (debug flag 1) */
    M26B_PEEK_Y = 8,               /* f32 [routes,4096] original route order, unweighted */
    M26B_PEEK_PARTIAL = 9,         /* f32 [rows,4096] */
    M26B_PEEK_MID_SCALES = 10      /* u8 [routes,I_local/32] grouped order, row-major (gathered from the scale blocks) */
};
/* Route outputs (the FC2 rows the ordered combine reads) as FP32 (dtype 0, the default: the reference's lattice,
 * bit-exact combine inputs) or BF16 (dtype 1): the reference's opt-in MIMO26_B1_Y=bf16
 * (crates/mimo26-spark/kernels/b1_serve.cu:98-143 reduce_bf16y, 400-406): FC2 rounds each row to BF16 (nearest even),
 * the combine widens them exactly and runs the same ordered multiply / add, fault rules and BF16 rounding. Halves
 * FC2's write and the combine's read; not bit-identical to the FP32 mode. A scratch created while the environment
 * holds MIMO26_B1_Y=bf16 starts in BF16 mode, as the reference's does. M26B_PEEK_Y then returns u16 [routes,4096]. */
int m26b_scratch_set_route_output(m26b_scratch* scratch, int dtype);
/* Per-kernel GPU time of the last pass in milliseconds, from CUDA events recorded on the launching stream
 * around each kernel when debug flag bit 1 (value 2) is set (the reference times its phases the same way,
 * b1_serve.cu:545-550): [0] input quantiser, [1] route plan, [2] permutation, [3] FC1 GEMM, [4] FC2 GEMM,
 * [5] combine. Waits for the pass to finish. */
int m26b_scratch_timings(m26b_scratch* scratch, float* ms6, char* err, size_t errlen);
/* Copies a buffer of the last pass to host memory; returns 0 or 1/2. */
int m26b_scratch_peek(m26b_scratch* scratch, int what, void* host_dst, uint64_t bytes, char* err, size_t errlen);

/* Stand-alone stages on device pointers, enqueued on `stream`.
 * Quantise n_elems (a multiple of 32) values: x_dtype 0 BF16 / 1 FP32, codec as
 * above; fault_dev is one u32 the kernel ORs fault codes into (4 nonfinite,
 * 5 reconstruction overflow; quant_v1 only). */
int m26b_quantize_dev(const void* x, int x_dtype, uint64_t n_elems, int codec, uint8_t* payload, uint8_t* scales,
                      uint32_t* fault_dev, void* stream, char* err, size_t errlen);
/* Ordered top-8 combine (crates/mimo26-expert/kernels/b1/route_reduce.cu:61-74):
 * y FP32 [rows,8,4096], weights [rows,8] -> partial FP32 [rows,4096] (or NULL) and bf16. */
int m26b_route_reduce_dev(const float* y, const float* weights, uint32_t rows, float* partial, uint16_t* bf16,
                          uint32_t* fault_dev, void* stream, char* err, size_t errlen);
/* Cross-rank sum in rank order (crates/mimo26-coordinator/kernels/glue.cu:202-213):
 * planes[r] BF16 [n], r < n_ranks <= 8 -> out FP32 [n]. `planes` is a HOST array of device pointers. */
int m26b_rank_sum_dev(const uint16_t* const* planes, int n_ranks, uint64_t n, float* out, void* stream, char* err,
                      size_t errlen);
/* The same with the coordinator's next step folded in (crates/mimo26-coordinator/src/dforward.rs:2294-2297: rank sum,
 * then h += f, kernels/glue.cu:55-59): out = residual + sum, one FP32 add after the rank-ordered sum, so the result
 * is bit-identical to the two launches. residual may be NULL (plain sum) and may alias out (in-place h += f). */
int m26b_rank_sum_residual_dev(const uint16_t* const* planes, int n_ranks, uint64_t n, const float* residual, float* out,
                               void* stream, char* err, size_t errlen);

/* The caller's producer step, on device pointers: the router's selection from FP32 logits
 * (crates/mimo26-coordinator/src/router.rs:42-80 router_from_logits, kernels/glue.cu:72-126 router_topk_kernel:
 * FP64 sigmoid, top 8 of 256 by score + bias with ties to the lower id, weights = unbiased scores normalised in
 * selection order) and, when x is not NULL, the activation quantiser of m26b_quantize_dev on x [rows,4096], both in
 * ONE launch. logits [rows,256] FP32; bias [256] FP32 or NULL; ids_out / weights_out [rows,8] are what m26b_ffn_dev
 * takes. Indices equal the reference's; a weight may differ from a host libm evaluation in its last FP32 bit (the
 * device's FP64 exp is not correctly rounded). */
int m26b_produce_dev(const float* logits, const float* bias, uint32_t rows, int32_t* ids_out, float* weights_out, const void* x,
                     int x_dtype, int codec, uint8_t* payload, uint8_t* scales, uint32_t* fault_dev, void* stream, char* err,
                     size_t errlen);

/* Plane exchange between the GPUs of one NVLink box, one process per GPU: replaces the return path + coordinator
 * sum of the reference (crates/mimo26-wire/src/l4.rs:169-244 collects the four ranks' BF16 planes over RDMA,
 * crates/mimo26-coordinator/kernels/glue.cu:202-213 adds them in rank order) when the ranks are GPUs that can map
 * each other's memory. Each rank owns a window with two plane slots; the combine writes the rank's BF16 plane into
 * the slot m26b_exchange_plane() names, and m26b_exchange_sum_dev() enqueues ONE kernel that publishes the plane,
 * waits (bounded) for every peer's, reads the peers' planes over NVLink and writes the rank-ordered FP32 sum.
 *   new:      allocate the window (plane_bytes a multiple of 256); handle_out receives 64 bytes for the peers
 *             (an IPC handle of the window), or pass NULL when every rank lives in this process. The window holds the
 *             two plane slots and, for m26b_ffn_tp_dev's fused form, two receive planes per rank of
 *             2 x min(plane_bytes, 4 MiB) bytes each (at most 128 MiB at eight ranks).
 *   connect:  `handles` = world x 64 bytes in rank order, gathered by the caller (e.g. an all-gather on the host).
 *   connect_local: the same for windows of one process (`all` = world handles in rank order).
 *   plane:    device address the NEXT step's BF16 plane must be written to (alternates between the two slots).
 *   sum_dev:  n_elems a multiple of 8; out_f32 [n_elems] on this rank. Every rank must call it once per step.
 *   status:   0, or 5 when a wait ran out (the message names the ranks). After code 5 the ranks are out of step: before
 *             the next step every rank must reach a host-side barrier with its stream synchronised (the two-slot
 *             scheme only protects a slot while every step's wait succeeds; a rank that keeps going after a lost
 *             step can overwrite a plane a slow peer is still reading). The same holds for the m26b_ep_* rendezvous.
 *   set_wait_ms: the bound of the wait (default 2000 ms).
 *   publish_as: marks the next step as published by `peer_rank` from the host (its plane flag and its chunk flags of
 *             m26b_ffn_tp_dev's fused form) and returns once the marks are in place (it synchronises `stream`); for
 *             single-process tests and for a coordinator that stands in for a rank it knows to be idle. */
int m26b_exchange_new(uint64_t plane_bytes, uint32_t rank, uint32_t world, m26b_exchange** out, uint8_t* handle_out,
                      char* err, size_t errlen);
int m26b_exchange_connect(m26b_exchange* x, const uint8_t* handles, char* err, size_t errlen);
int m26b_exchange_connect_local(m26b_exchange* x, m26b_exchange* const* all, char* err, size_t errlen);
void* m26b_exchange_plane(m26b_exchange* x);
int m26b_exchange_set_wait_ms(m26b_exchange* x, uint32_t ms);
int m26b_exchange_publish_as(m26b_exchange* x, uint32_t peer_rank, void* stream, char* err, size_t errlen);
int m26b_exchange_sum_dev(m26b_exchange* x, uint64_t n_elems, float* out_f32, void* stream, char* err, size_t errlen);
/* sum_dev with the residual add folded in, as m26b_rank_sum_residual_dev: out = residual + rank-ordered sum. */
int m26b_exchange_sum_residual_dev(m26b_exchange* x, uint64_t n_elems, const float* residual, float* out_f32, void* stream,
                                   char* err, size_t errlen);
int m26b_exchange_status(m26b_exchange* x, void* stream, char* err, size_t errlen);
void m26b_exchange_free(m26b_exchange* x);

/* m26b_ffn for one rank of a tensor-parallel group inside one box (one process per GPU): the host-pointer entry a
 * serving loop calls once per request on every rank, where the reference's ranks each receive the request frame and
 * return a BF16 partial for the coordinator to sum (crates/mimo26-spark/src/serve.rs:206-246, then
 * crates/mimo26-wire/src/l4.rs:169-244). The request goes up from HOST memory exactly as in m26b_ffn, the rank's slice
 * runs with its BF16 plane written into the exchange window `x`, the planes are summed in rank order over NVLink
 * (the fused kernel of m26b_ffn_tp_dev for requests of at most 512 tokens, else m26b_exchange_sum_dev), and the FP32 sum
 * [rows*4096] comes back to HOST memory on the ranks that pass sum_out (NULL
 * elsewhere: one rank downloading is enough). Every rank of the group must make the call for every request.
 * rows x 8192 bytes must fit the exchange plane. Synchronous. ms (or NULL): [0] upload + enqueue, [1] GPU time
 * including the exchange, [2] host tail, [3] token tiles, the rest 0. Returns m26b_ffn's codes, or 5 when a peer's
 * plane did not arrive within the exchange's bound. */
int m26b_ffn_tp(const m26b_layer* layer, m26b_scratch* scratch, m26b_exchange* x, const uint8_t* payload, size_t payload_pitch,
                const uint8_t* scales, size_t scales_pitch, const int32_t* ids, const float* weights, uint32_t rows,
                float* sum_out, float* ms, char* err, size_t errlen);
/* The device-pointer form, with the combine and the exchange in ONE kernel: m26b_ffn_dev's arguments (x, x_dtype,
 * x_scales, codec, ids, weights as there), and instead of the rank's BF16 plane the call leaves the rank-ordered FP32 sum
 * of all ranks' BF16 planes (+ residual, or NULL) in sum_out [rows*4096] on every rank: what the reference gets from the
 * ranks' return frames and the coordinator's sum (crates/mimo26-wire/src/l4.rs:169-244, kernels/glue.cu:202-213), bit for
 * bit. For steps of at most 512 tokens each CTA of the combine kernel stores its BF16 chunk into every peer's window
 * (plain peer stores over NVLink, one flag per 1,024-element chunk) and, once its chunks are out, adds the chunks the
 * peers pushed from local memory; the transfer overlaps the combine and no second kernel or read round trip follows.
 * Larger steps (bandwidth-bound) run m26b_ffn_dev into m26b_exchange_plane() and m26b_exchange_sum_residual_dev behind
 * it. One exchange step either way: every rank makes the call for every step, and the step counter is shared with
 * m26b_exchange_sum_dev. Asynchronous on `stream`; m26b_scratch_status and m26b_exchange_status report as for the two
 * calls it replaces (a peer's chunk that does not arrive within the bound: code 5 from m26b_exchange_status). */
int m26b_ffn_tp_dev(const m26b_layer* layer, m26b_scratch* scratch, m26b_exchange* x, const void* x_act, int x_dtype,
                    const uint8_t* x_scales, int codec, const int32_t* ids, const float* weights, uint32_t rows,
                    const float* residual, float* sum_out, void* stream, char* err, size_t errlen);

/* Expert parallelism inside one NVLink box, one process per GPU (the reference has no expert-
 * parallel mode: it shards every expert's intermediate dimension over its four ranks, crates/mimo26-repack/src/geom.rs:29-35).
 * Rank r holds experts [r 256/G, (r+1) 256/G) (m26b_layer_new_from_checkpoint_ep: the six checkpoint tensors stacked over
 * THOSE experts) and owns a contiguous block of the step's tokens (the first `tokens % G` ranks one token more;
 * m26b_ep_rows). A step on every rank, in this order, on one stream:
 *   begin_dev:   quantise this rank's rows (or copy rows already quantised, x_dtype 2) and its routes into the rank's
 *                window, then rendezvous "rows ready";
 *   compute_dev: pull every rank's routes, plan the routes that go to this rank's experts, gather their token rows from
 *                the owners' windows (peer loads), FC1, FC2 with every output row written into the owner's window
 *                (peer stores) at its route index, then rendezvous "results complete";
 *   finish_dev:  the ordered top-8 combine of this rank's own tokens -> BF16 [rows,4096] (+ optional FP32 plane).
 * The result equals the single-GPU result bit for bit (rows of the GEMMs do not depend on how routes are tiled).
 * Plan and numerical faults of compute_dev are read with m26b_scratch_status; m26b_ep_status returns 5 when a
 * rendezvous ran out of time (default bound 5 s), 4 on a quantiser / combine fault. Windows are connected like the plane
 * exchange's (64-byte handles gathered by the caller, or connect_local inside one process); publish_as marks a
 * rendezvous (0 rows ready of the NEXT step, 1 results complete of the CURRENT step) as reached by `peer_rank`. */
int m26b_layer_new_from_checkpoint_ep(const uint8_t* gate_w, const uint8_t* gate_s, const uint8_t* up_w, const uint8_t* up_s,
                                      const uint8_t* down_w, const uint8_t* down_s, uint32_t ep_rank, uint32_t ep_size,
                                      m26b_layer** out, char* err, size_t errlen);
/* The same with replicated experts, for skewed routing: besides its own block the rank holds copies of n_rep experts
 * (ids rep_ids[], a HOST array; their six tensors stacked in that order in the rep_* arguments). EVERY rank of the group
 * must be built with the same rep_ids. A route to a replicated expert is served by the rank that owns the route's token,
 * so a popular expert's rows spread over the ranks as evenly as the tokens do and neither its token rows nor its result
 * rows cross NVLink; routes to all other experts go to the rank whose block holds them, as before. Results stay equal to
 * the single-GPU layer bit for bit. Cost: 13,369,344 bytes of HBM per replicated expert and rank. n_rep = 0 is exactly
 * m26b_layer_new_from_checkpoint_ep. */
int m26b_layer_new_from_checkpoint_ep_replicated(const uint8_t* gate_w, const uint8_t* gate_s, const uint8_t* up_w, const uint8_t* up_s,
                                                 const uint8_t* down_w, const uint8_t* down_s, const uint8_t* rep_gate_w,
                                                 const uint8_t* rep_gate_s, const uint8_t* rep_up_w, const uint8_t* rep_up_s,
                                                 const uint8_t* rep_down_w, const uint8_t* rep_down_s, const int32_t* rep_ids,
                                                 uint32_t n_rep, uint32_t ep_rank, uint32_t ep_size, m26b_layer** out, char* err,
                                                 size_t errlen);
int m26b_ep_new(uint32_t tokens, uint32_t rank, uint32_t world, m26b_ep** out, uint8_t* handle_out, char* err, size_t errlen);
int m26b_ep_connect(m26b_ep* e, const uint8_t* handles, char* err, size_t errlen);
int m26b_ep_connect_local(m26b_ep* e, m26b_ep* const* all, char* err, size_t errlen);
int m26b_ep_rows(const m26b_ep* e, uint32_t rank);
int m26b_ep_set_wait_ms(m26b_ep* e, uint32_t ms);
/* Result rows cross NVLink and are combined as FP32 (0, default) or BF16 (1), as m26b_scratch_set_route_output; every
 * rank of a step must use the same setting. */
int m26b_ep_set_route_output(m26b_ep* e, int dtype);
int m26b_ep_publish_as(m26b_ep* e, uint32_t peer_rank, uint32_t which, void* stream, char* err, size_t errlen);
int m26b_ep_begin_dev(m26b_ep* e, const void* x, int x_dtype, const uint8_t* x_scales, int codec, const int32_t* ids,
                      const float* weights, uint32_t rows, void* stream, char* err, size_t errlen);
int m26b_ep_compute_dev(m26b_ep* e, const m26b_layer* l, m26b_scratch* s, void* stream, char* err, size_t errlen);
int m26b_ep_finish_dev(m26b_ep* e, uint16_t* bf16_out, float* partial_out, void* stream, char* err, size_t errlen);
int m26b_ep_status(m26b_ep* e, void* stream, char* err, size_t errlen);
/* One expert-parallel step from HOST memory on the scratch's stream: this rank's block of the step's tokens goes up
 * (quantised rows at payload_pitch / scales_pitch as in m26b_ffn, ids, weights; rows = m26b_ep_rows of this rank, which
 * may be 0), begin / compute / finish run, and the rank's BF16 rows [rows*4096] come back. Synchronous; every rank
 * must make the call. Returns 0, or the first failing stage's code. */
int m26b_ep_ffn(m26b_ep* e, const m26b_layer* l, m26b_scratch* s, const uint8_t* payload, size_t payload_pitch,
                const uint8_t* scales, size_t scales_pitch, const int32_t* ids, const float* weights, uint32_t rows,
                uint16_t* bf16_out, char* err, size_t errlen);
void m26b_ep_free(m26b_ep* e);

/* DS41RTE3 v3 frames (host memory): the request a rank receives and the compact return it sends
 * (crates/mimo26-wire/src/layout.rs:64-115 field offsets, src/frame.rs:311-455, 868-955, 987-1041; checksum CRC32C over the
 * frame with its own field zero, src/crc32c.rs). Return code 6 = frame rejected, with the reference's reason in `err`.
 *   request_bytes / return_bytes: frame sizes for `rows` tokens with 8 routes each (128 + rows x 4360, 128 + rows x 8192).
 *   encode_request: the frame of encode_request_meta_into (frame.rs:569-652: decode-kind rows, row t = id and position t,
 *     routes t*8.., placement version 1) with the hidden rows copied in and, if `seal`, the checksum written.
 *   serve_frame: what the expert daemon does per request (crates/mimo26-spark/src/serve.rs:206-246 + main.rs:386-413):
 *     validate the request in place, run m26b_ffn on its rows at the frame's stride, write the return frame (BF16 rows
 *     straight behind the header, flags = pre-summed + compact BF16, ids copied from the request) and seal it.
 *     `check_crc` = verify the request's checksum and seal the reply (0 = the reference's MIMO26_WIRE_NOCRC=1 mode).
 *   parse_return: the coordinator's checks on a return frame; rows_offset = where the BF16 rows start. */
uint64_t m26b_frame_request_bytes(uint32_t rows);
uint64_t m26b_frame_return_bytes(uint32_t rows);
uint32_t m26b_frame_crc32c(const uint8_t* bytes, uint64_t n);        /* the CPU's CRC32C instruction where it exists */
uint32_t m26b_frame_crc32c_table(const uint8_t* bytes, uint64_t n);  /* table path only: the cross-check of the former */
int m26b_frame_encode_request(uint8_t* out, uint64_t cap, uint64_t request_id, uint32_t layer_id, uint64_t executor_id, uint64_t seq,
                              const uint8_t* payload, size_t payload_pitch, const uint8_t* scales, size_t scales_pitch,
                              const int32_t* ids, const float* weights, uint32_t rows, int seal, uint64_t* len_out, char* err,
                              size_t errlen);
/* serve_frame's checks on a request frame without running it (no GPU needed). */
int m26b_frame_check_request(const uint8_t* request, uint64_t request_len, int check_crc, uint32_t* rows, uint64_t* request_id,
                             uint32_t* layer_id, char* err, size_t errlen);
int m26b_serve_frame(const m26b_layer* l, m26b_scratch* s, const uint8_t* request, uint64_t request_len, uint8_t* reply,
                     uint64_t reply_cap, uint64_t* reply_len, int check_crc, uint64_t reply_seq, float* ms, char* err,
                     size_t errlen);
int m26b_frame_parse_return(const uint8_t* frame, uint64_t len, int check_crc, uint64_t* request_id, uint32_t* layer_id,
                            uint32_t* rows, uint32_t* status, uint64_t* seq, uint64_t* rows_offset, char* err, size_t errlen);

/* Route plan without any allocation. No counterpart in the reference.
 * For callers that must not allocate device memory while they run: a serving loop that gave every free byte of the
 * GPU to resident expert weights at start-up, a request handler that has to stay clear of cudaMalloc's device-wide
 * synchronisation while other streams compute, or code running where an allocation failure cannot be handled.
 * It is the multi-CTA stable planner of m26b_ffn / m26b_ffn_dev (expert-major, stable inside an expert); its
 * working memory (per-CTA expert counts, expert table, token tiles and work items, about 0.47 MB) is a fixed array
 * inside the library, present on every GPU that loads it until the process exits.
 * ids / weights: device, [rows*8], token-major top-8. Outputs, device: inverse[rows*8] (original route -> grouped
 * route), original_routes[rows*8] (grouped route -> original route), grouped_weights[rows*8], meta_out[8]
 * (word 0: 0 ok / 1 plan rejected, word 1 token tiles, 4 experts with routes, 5 largest per-expert count). Work is
 * enqueued on `stream`; nothing is synchronised. rows <= 4096, larger requests return 1 with a message.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress); make that call before any
 * stream capture. All calls on one GPU share the array: calls whose kernels overlap on the GPU race, so keep them on
 * one stream or order them with events. Calls cudaMalloc / cudaFree never. */
int m26b_plan_static(const int32_t* ids, const float* weights, uint32_t rows, int32_t* inverse, int32_t* original_routes,
                     float* grouped_weights, uint32_t* meta_out, void* stream, char* err, size_t errlen);

/* Library identity: "m26b-expert <version> sm_100a". */
const char* m26b_version(void);

#ifdef __cplusplus
}
#endif
#endif
