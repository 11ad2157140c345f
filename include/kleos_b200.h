/*
 * kleos_b200 — C ABI of the B200-native distributed MoE layer forward pass.
 *
 * Every entry point below replaces one inline C++ host function of the reference project
 * (namespace kleos); the reference file:line each one stands in for is cited beside it.
 * All functions return 0 on success or a negative KLEOS_E_* code; none of them exits the
 * process (the reference prints and calls exit()/quick_exit(), debug.cuh:19-43).
 *
 * Threading model is the reference's: one host thread per process, one process per GPU,
 * global state, not re-entrant (types.cuh:440,1011-1013).
 */
#ifndef KLEOS_B200_H
#define KLEOS_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    KLEOS_OK = 0,
    KLEOS_E_CONFIG = -1,      /* unreadable or invalid kleos_config.json            */
    KLEOS_E_STATE = -2,       /* call order: not initialised / already initialised  */
    KLEOS_E_CUDA = -3,        /* a CUDA runtime or driver call failed               */
    KLEOS_E_BOOTSTRAP = -4,   /* NCCL bootstrap or peer mapping failed              */
    KLEOS_E_MISMATCH = -5,    /* ranks disagree on the configuration                */
    KLEOS_E_DEVICE = -6,      /* the device reported a timeout or a bounds error    */
    KLEOS_E_UNSUPPORTED = -7, /* dtype / shape outside what the kernels implement   */
    KLEOS_E_ARG = -8          /* null pointer or out-of-range argument              */
};

/* Where a device-side problem was detected (kleos_status.where). */
enum {
    KLEOS_AT_NONE = 0,
    KLEOS_AT_PLAN_WAIT = 1,     /* waiting for dispatch flags from the source ranks */
    KLEOS_AT_COMBINE_WAIT = 2,  /* waiting for result flags from the expert ranks   */
    KLEOS_AT_GEMM_PRODUCER = 3, /* TMA producer waiting for a free pipeline stage   */
    KLEOS_AT_GEMM_MMA = 4,      /* MMA issuer waiting for operands or accumulator   */
    KLEOS_AT_GEMM_EPILOGUE = 5, /* epilogue waiting for an accumulator              */
    KLEOS_AT_BOUNDS = 6,        /* an index outside its table                       */
    KLEOS_AT_GRID_BARRIER = 7   /* blocks of the persistent kernel waiting for one another */
};

typedef struct kleos_status {
    int32_t code;   /* 0, or KLEOS_E_DEVICE */
    int32_t where;  /* KLEOS_AT_*           */
    int32_t detail; /* rank / cell / tile the detector was looking at */
    int32_t epoch;  /* forward-call counter when it happened */
} kleos_status;

typedef struct kleos_layer_info {
    int32_t rank, world, local_experts;
    int32_t S, H, I, E, K, EC, pEC, PX;
    int32_t torch_dtype, hidden_act, elem_bytes;
    int64_t input_elems;  /* elements in the packed input buffer  iP */
    int64_t output_elems; /* elements in the packed output buffer oP */
} kleos_layer_info;

/* Bootstrap helper: rank 0 creates the 128-byte NCCL unique id that every rank passes to
 * kleos_initialize.  The reference bootstraps through nvshmem_init() under an MPI/PMI
 * launcher instead (bootstrap.cuh:295). */
int kleos_get_unique_id(void* out_id128);

/* Select the CUDA device before kleos_initialize (reference: setDevice(),
 * bootstrap.cuh:549-553).  Default is rank % device count. */
int kleos_set_device(int device);

/* Read kleos_config.json (same keys as kleos_config.schema.json:5-89, parsed at run time
 * instead of being baked in by CMake), allocate the symmetric cells, flags and bookkeeping,
 * and map every peer's cells.  Replaces kleos::initialize() (bootstrap.cuh:532-547).
 * nccl_id may be NULL when world == 1. */
int kleos_initialize(const char* config_json_path, int rank, int world, const void* nccl_id);

/* Parse a kleos_config.json and report the derived sizes for a given world size without
 * touching the GPU (rank is reported as 0).  Same derivations as the reference's compile-time
 * ACC struct (types.cuh:442-513). */
int kleos_config_probe(const char* config_json_path, int world, kleos_layer_info* out);

/* Optional per-expert logit bias (E floats, host memory).  The reference gate has no bias
 * (moe/gate.cuh:87-88); the load-imbalanced benchmark layer needs one.  NULL clears it. */
int kleos_set_gate_bias(const float* host_bias, int n);

/* One layer forward, asynchronous on `stream` (a cudaStream_t, or NULL for the per-thread
 * default stream the reference uses, types.cuh:1013).  iP and oP are DEVICE pointers to the
 * packed buffers of moe.cuh:92-98:
 *   iP = [A S*H][Wg PX*H][W1 nLx*I*H][W2 nLx*H*I][b1 nLx*I][b2 nLx*H]
 *   oP = [gate probabilities S*PX][layer output S*H]
 * With num_experts == 1 the layer is the plain FFN over the rank's own tokens, as in the
 * reference (moe/moe.cuh:197-204 launches moe/fffn.cuh:31-167): no gate and no exchange, every
 * rank holds the one expert (nLx = 1, any world size, no NCCL id needed), and the packed
 * buffers lose their gate sections:
 *   iP = [A S*H][W1 I*H][W2 H*I][b1 I][b2 H]      oP = [layer output S*H]
 * Replaces kleos::moe::forwardHost(iP, oP) (moe/moe.cuh:186-205). */
int kleos_forward(const void* iP, void* oP, void* stream);

/* skip warm-up forwards, then trials forwards between two CUDA events; *ms = mean per
 * forward.  Synchronises.  Replaces forwardHostBench<skip,trials> (moe/moe.cuh:146-184). */
int kleos_forward_bench(const void* iP, void* oP, int skip, int trials, float* ms);

/* End-to-end call with HOST buffers: copies S*H activations host->device into the A section
 * of iP, runs one forward, copies the S*H layer output device->host, and synchronises.
 * Weights stay resident in iP.  The reference driver does the same copies by hand
 * (main.cu:64-66). */
int kleos_forward_host(const void* host_activations, void* iP, void* oP, void* host_output);

/* Pipelined form of kleos_forward_host for a stream of batches: returns as soon as the step is
 * queued.  Activations and layer output are double-buffered inside the library, so the
 * host->device copy of step i+1 and the device->host copy of step i-1 overlap the forward of
 * step i (three streams).  host_output of a step is valid after kleos_host_sync(), which also
 * reports device-side errors.  The gate probabilities still land in oP.  The reference has no
 * counterpart (its driver copies once and loops on the device, main.cu:64-68). */
int kleos_forward_host_async(const void* host_activations, void* iP, void* oP, void* host_output);
int kleos_host_sync(void);

/* Reference: getRank() (bootstrap.cuh:555-559) and hostBookkeeping.nLx (main.cu:22). */
int kleos_get_rank(void);
int kleos_local_experts(void);
int kleos_get_info(kleos_layer_info* out);

/* Device-side status of the last forward calls; synchronises the library's stream.
 * The reference has no equivalent: its device waits spin forever (atomics.cuh:96-138). */
int kleos_last_status(kleos_status* out);
/* Forget a recorded device-side error (the first one sticks until cleared). */
int kleos_clear_status(void);

/* Routing results of the last forward, copied to host memory (any pointer may be NULL):
 * topk [S*K] expert ids, slots [S*K] slot inside the expert cell or -1 when dropped,
 * counts [E] unclamped tokens per expert, mcw [S] sum of the k winning probabilities.
 * The reference keeps these in its bookkeeping arena (types.cuh:697-1008) without an
 * accessor; parity tests need them. */
int kleos_debug_routing(int32_t* topk, int32_t* slots, uint32_t* counts, float* mcw);

/* Per-phase device time of the most recent kleos_forward_bench, in milliseconds averaged over
 * its trials: [0] route, [1] slots, [2] dispatch, [3] plan(wait), [4] GEMM1, [5] GEMM2,
 * [6] combine, [7] whole forward.  n = number of floats the caller provides (>= 8). */
int kleos_phase_times(float* ms, int n);

/* With KLEOS_FLOW=1 16-bit routed layers run the router, dispatch, plan, both expert GEMMs and the
 * combine as ONE persistent kernel (the reference's arrangement, moe/moe.cuh:77-144); the phases above are
 * then read from the blocks' global-timer stamps: [0] gate GEMM + top-k up to the first grid
 * barrier, [1] slots up to the second; [2] last row dispatched and [3] tile plan known, both
 * counted from the second barrier; [4] span of the GEMM1 tiles; [5] from the last GEMM1 tile to
 * the last tile; [6] from the last tile to the kernel's end.  This call returns the raw
 * milestones of the most recent kleos_forward_bench, milliseconds after the earliest block's
 * start, latest block each: [0] 0, [1] plan known, [2] first tile begins (earliest block),
 * [3] last GEMM1 tile done, [4] last tile done, [5] last row dispatched, [6] last token combined,
 * [7] last block ends, [8] routing done (first grid barrier), [9] slots done (second),
 * [10] gate logits of the last token tile complete, [11] ... and turned into choices; with
 * n >= 19 also the router's inner steps: [12] top-k and softmax sum known, [13] near-ties
 * re-evaluated and probabilities stored, [14] base slots of the block's tile known, [15] slots
 * written, [16] set-up over and gate GEMM begins, [17] first K slice of the gate GEMM in shared
 * memory, [18] first pass over the logits done.  n >= 12.
 * KLEOS_E_STATE when the layer runs as separate launches (float and TF32 layers, the dense
 * layer, and every layer unless KLEOS_FLOW=1 is set). */
int kleos_flow_timeline(float* ms, int n);

/* The same stamps block by block, as written by the last timed forward of kleos_forward_bench:
 * ns[b * per_block + k] = global-timer nanoseconds of milestone k in block b (0: that block never
 * passed it).  *blocks and *per_block are always set; ns may be null to ask for the sizes only,
 * otherwise capacity >= *blocks * *per_block.  A tuning aid with no counterpart in the reference. */
int kleos_debug_flow_stamps(long long* ns, int capacity, int* blocks, int* per_block);

/* Wait times of the persistent kernel's tile-stream roles in the LAST timed forward of
 * kleos_forward_bench, milliseconds averaged over the blocks that recorded a value:
 * [0] producer waiting for a free stage, [1] for cell data / GEMM1 counters, [2] producer total,
 * [3] MMA issuer waiting for an accumulator, [4] for operands, [5] for the next claimed tile,
 * [6] issuer total, [7] read-back warp waiting for an accumulator, [8] publishing, [9] reading back
 * and storing, [10] read-back total, [11] producer's proxy fences.  n >= 12.  A tuning aid with no counterpart in
 * the reference. */
int kleos_debug_flow_stalls(float* ms, int n);

/* The segment order of the persistent kernel's tile queue for `local_experts` experts and a lag
 * of `lag` segments: phase[s] is 0 for the first expert GEMM and 1 for the second, expert[s] the
 * local expert of segment s; returns the number of segments (2 * local_experts).  Host only,
 * needs no GPU and no kleos_initialize; lets a test check that every second-GEMM segment follows
 * the first-GEMM segment it consumes (the reference chains the two per row panel at run time,
 * os/processor/processor.cuh:717-729). */
int kleos_debug_tile_order(int local_experts, int lag, int32_t* phase, int32_t* expert);

/* Kernels this library has launched for forward calls since kleos_initialize (every launch site
 * counts itself; memory copies and memsets are not kernels).  A benchmark reads it before and
 * after its timed region.  Negative (KLEOS_E_STATE) when not initialised.  No counterpart in the
 * reference, whose forward is always one launch (moe/moe.cuh:198). */
long long kleos_launch_count(void);

/* Stall counters of the last GEMM1 and GEMM2 launches, only when the environment variable
 * KLEOS_GEMM_STATS=1 was set at initialise time: [2][blocks][12] clock cycles per block
 * {producer wait-empty, producer total, MMA wait-accumulator, MMA wait-operands, MMA total,
 *  epilogue wait-accumulator, epilogue total, epilogue TMEM wait, plan prologue, producer wait
 *  for cell data, dispatch finished at, unused}.  Returns the number of values written.
 * A tuning aid with no counterpart in the reference. */
int kleos_debug_gemm_stats(long long* out, int max_values);

/* Router only, for callers that cannot allocate device memory when they call (inside another
 * runtime's allocator callback, in a serving loop with a frozen memory budget, ...).  It has no
 * counterpart in the reference, which always routes inside its fused kernel.  It needs no
 * kleos_initialize: the scratch it uses (near-tie list, fp64 logits, counters; 2,130,432 bytes)
 * is a fixed array inside the library that every GPU loading it keeps until the process ends,
 * and the call performs no cudaMalloc / cudaFree.
 *   A [S,H], Wg [64,H] (row e = expert e, rows >= E zero), gate_bias [E] floats or NULL,
 *   probs [S,64] (element type), topk [S,K], mcw [S]: all DEVICE pointers owned by the caller;
 *   A and Wg must be 16-byte aligned (KLEOS_E_ARG otherwise).
 *   Limits: S <= 4096, E <= 64, K <= min(E, 8), H a multiple of 64, torch_dtype 0 or 2; anything
 *   larger is refused with KLEOS_E_ARG and a message on stderr.
 * The first call on each device looks up the array's device address; make that call before any
 * stream capture.  All calls share the one array and each call first clears the part that must
 * start at zero, so two calls that overlap on the GPU (different streams, different threads)
 * race: serialise them.  Asynchronous on `stream` (NULL = per-thread default stream). */
int kleos_route_static(const void* A, const void* Wg, const float* gate_bias, int S, int H, int E,
                       int K, int torch_dtype, void* probs, int32_t* topk, float* mcw,
                       void* stream);

/* Training-mode gate statistics of the last forward on this rank (is_training = 1 in the
 * configuration, num_experts > 1), the three quantities the reference keeps in its device
 * bookkeeping (types.cuh:944-960) and never copies out:
 *   mean_prob[e]  = (1/S) sum_t p(t,e), fp32 softmax probabilities      (moe/gate.cuh:607-635)
 *   mean_count[e] = (tokens of this rank that chose e, before capacity) / S   (:698-705)
 *   loss          = sum_e mean_prob[e] * mean_count[e] / E              (:763-773)
 * Host pointers, E floats / E floats / 1 float; any may be NULL.  The reference accumulates
 * with atomicAdd and never clears between launches; here every forward overwrites the values
 * and the sums run in a fixed order.  KLEOS_E_STATE when the layer was not set up for training. */
int kleos_gate_stats(float* mean_prob, float* mean_count, float* loss);

/* Init-time placement planner (host only, needs no GPU and no kleos_initialize): restates the
 * reference's Decider and expert assignment (os/decider/decider.cuh:37-329, used at start-up in
 * bootstrap.cuh:170-265).  From a latency / inverse-bandwidth matrix (alpha in ms, beta in ms per
 * MB, entry [i*world + j] = link i -> j), per-device throughput and the number of experts each
 * device can hold, it merges devices into expert-parallel groups and assigns the experts of the
 * asking rank's group to its members in proportion to throughput.
 *   device_to_group  [world]  representative device of every device's group
 *   group_ranks      [world]  first group_size entries: devices of rank's group, ascending
 *   expert_to_member [E]      index into group_ranks of the device that holds each expert
 * Output pointers may be NULL.  matches_data_path is 1 when the plan is the even contiguous
 * sharding over all ranks that kleos_initialize implements (the case of one NVSwitch node with
 * identical GPUs); other plans are reported but not executed by this library. */
typedef struct kleos_placement_request {
    int32_t world, rank, num_experts, expert_cost, is_training;
    uint32_t moe_stages, p2p_buffer_mb, grad_buffer_mb; /* see kleos_placement_model */
    const float* alpha;  /* [world*world] */
    const float* beta;   /* [world*world] */
    const float* rate;   /* [world] expert cost units per ms */
    const uint32_t* mem; /* [world] experts that fit */
} kleos_placement_request;

typedef struct kleos_placement_result {
    int32_t feasible, group_size, group_rank, local_experts, expert_slots, widest_group;
    int32_t matches_data_path;
} kleos_placement_result;

int kleos_plan_placement(const kleos_placement_request* request, kleos_placement_result* result,
                         uint32_t* device_to_group, uint32_t* group_ranks, uint32_t* expert_to_member);

/* The three cost-model constants the reference derives from the compiled layer
 * (types.cuh:487-494): global MoE stages, and the dispatch and gradient buffers in MB. */
int kleos_placement_model(const char* config_json_path, uint32_t* moe_stages, uint32_t* p2p_buffer_mb,
                          uint32_t* grad_buffer_mb);

/* Test hook for the failure path: while on, the expert FFN does not raise its "results
 * returned" flags, so the combine's bounded wait runs out, the forward records
 * {KLEOS_E_DEVICE, KLEOS_AT_COMBINE_WAIT} and returns with the context intact.  Nothing is
 * faulted or hung; the wait budget is KLEOS_WAIT_MS.  No counterpart in the reference, whose
 * waits spin forever (atomics.cuh:96-138). */
int kleos_debug_suppress_return_flag(int on);

/* Free everything.  Replaces kleos::finalize() (bootstrap.cuh:561-588). */
int kleos_finalize(void);

const char* kleos_error_string(int code);

#ifdef __cplusplus
}
#endif
#endif /* KLEOS_B200_H */
