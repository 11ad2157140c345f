// Host layer and C ABI of the B200-native MoE forward pass.
//
// Stands in for the reference's inline host API: kleos::initialize / finalize / getRank
// (csrc/include/kleos/bootstrap.cuh:532-588) and moe::forwardHost / forwardHostBench
// (csrc/include/kleos/moe/moe.cuh:146-205).  The reference allocates an NVSHMEM symmetric
// heap plus flags (bootstrap.cuh:348-362) and eleven bookkeeping buffers (:365-397); here the
// symmetric arena is an ordinary device allocation whose CUDA IPC handle is all-gathered once
// over NCCL and mapped by every peer, after which all traffic is in-kernel stores and flags.
#include <cuda.h>
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>
#include <type_traits>
#include <vector>

#include <nvtx3/nvToolsExt.h>

#include "config.hpp"
#include "gemm_simt.cuh"
#include "gemm_tc2.cuh"
#include "gemm_tf32.cuh"
#include "moe_flow.cuh"
#include "placement.hpp"
#include "route.cuh"
#include "route_tc.cuh"
#include "transport.cuh"

namespace kleos {
namespace {

constexpr int kPhases = 8;  // route, slots, dispatch, plan, gemm1, gemm2, combine, total

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

struct State {
    bool initialised = false;
    int device = -1;
    int sm_count = 0;
    LayerConfig cfg;
    int rank = 0, world = 1, nLx = 0;
    uint32_t epoch = 0;
    long long wait_cycles = 20000000000LL;  // about ten seconds of SM clock (ranks may start far apart)
    bool use_tc = false;       // 16-bit layers: tcgen05 router and FFN GEMMs
    bool use_tf32_tc = false;  // TF32 layers: tcgen05 kind::tf32 FFN GEMMs (the router stays on FP32 FMA)
    // num_experts == 1: the layer is a plain FFN over this rank's tokens (the reference switches
    // to its fffn kernel, moe/moe.cuh:174-177,197-204): no gate, no exchange, and the packed
    // buffers carry no gate weight and no probabilities (moe/fffn.cuh:47-53)
    bool dense = false;
    bool suppress_return_flag = false;  // test hook: see kleos_debug_suppress_return_flag
    // KLEOS_FLOW=1, 16-bit routed layers: router, dispatch, plan, both expert GEMMs and the combine run
    // as ONE persistent kernel (moe_flow.cuh) instead of separate launches.
    bool use_flow = false;
    bool fuse_route = false;                 // ... and the router runs inside it too (KLEOS_FUSE_ROUTE=0: separate launches)
    bool route_by_flow = false;              // separate launches: the router is the persistent kernel's routing phase alone
    int flow_grid = 0;                       // blocks of the persistent kernel (co-resident pairs x 2)
    flow::Counters* flow_ctr = nullptr;      // [2] scheduler state, see moe_flow.cuh
    long long* flow_stamps = nullptr;        // [flow_grid][kStampSlots] timeline of a timed forward
    long long* flow_stalls = nullptr;        // [flow_grid][kStallSlots] wait cycles of a timed forward
    int flow_debug = 0;                      // KLEOS_FLOW_DEBUG
    int flow_unit_rows = flow::kUnitRows;    // KLEOS_UNIT_ROWS
    int flow_sub = 0;                        // KLEOS_FLOW_SUB: 1 or 2 forces the stage depth
    double clock_khz = 0;
    float flow_ms[flow::kStampSlots] = {};   // last kleos_forward_bench: milestones after kernel start
    std::vector<long long> flow_raw;         // ... and the blocks' own stamps of its last timed forward

    // symmetric arena
    ArenaLayout lay{};
    char* arena = nullptr;
    PeerTable peers{};
    bool peer_opened[kMaxWorld] = {};

    // local bookkeeping
    void* y1 = nullptr;
    int *topk = nullptr, *slots = nullptr, *cell_tokens = nullptr, *refine_list = nullptr,
        *refine_count = nullptr, *le_start = nullptr, *refine_done = nullptr, *tile_hist = nullptr;
    double* refine_logits = nullptr;
    float *mcw = nullptr, *bias = nullptr;
    // training mode (is_training = 1): per-router-block probability column sums and the
    // statistics [mean_prob E][mean_count E][loss] of the last forward
    float *col_partial = nullptr, *gate_stats = nullptr;
    unsigned *counts = nullptr, *done_dispatch = nullptr, *done_gemm2 = nullptr,
             *cell_counts = nullptr;
    PanelEntry* panels = nullptr;
    DeviceStatus* status = nullptr;
    long long* gemm_stats = nullptr;  // [2][grid][8] when KLEOS_GEMM_STATS=1

    // tensor maps (rebuilt when the caller's weight pointer changes)
    const void* maps_for_iP = nullptr;
    // map_w1 / map_w2: whole 256-row weight tiles (TF32 GEMM); map_w1h / map_w2h: the half tile
    // each block of a pair loads (16-bit GEMMs)
    CUtensorMap map_x{}, map_w1{}, map_y1{}, map_w2{}, map_act{}, map_wg{}, map_w1h{}, map_w2h{}, map_wgh{};

    // pipelined host-buffer path (kleos_forward_host_async): double-buffered staging of the
    // activations and of the layer output, one stream per direction
    struct HostPipe {
        bool ready = false;
        cudaStream_t in = nullptr, out = nullptr;
        char* act[2] = {};
        char* res[2] = {};
        CUtensorMap map_act[2] = {};
        cudaEvent_t in_done[2] = {}, comp_done[2] = {}, out_done[2] = {};
        unsigned long long step = 0;
    } hp;

    ncclComm_t comm = nullptr;
    cudaEvent_t ev[kPhases + 1] = {};
    cudaEvent_t ev_last = nullptr;  // recorded behind every forward on the caller's stream
    unsigned long long launches = 0;  // kernels launched by the forward paths since initialise
    float phase_ms[kPhases] = {};
    std::string last_error;
};

// Scoped NVTX range in the domain "Kleos", the domain the reference uses for its ranges around
// initialisation, forward and finalisation (telemetry.cuh:17-20, bootstrap.cuh:534-536,563-565,
// moe/moe.cuh:149-151,188-190).  The reference compiles them in with KLEOS_NVTX; here the
// environment variable KLEOS_NVTX=1 turns them on when the first entry point runs, and nothing
// of NVTX is touched otherwise.
class TraceRange {
public:
    explicit TraceRange(const char* name) : on_(enabled()) {
        if (!on_) return;
        nvtxEventAttributes_t a{};
        a.version = NVTX_VERSION;
        a.size = NVTX_EVENT_ATTRIB_STRUCT_SIZE;
        a.messageType = NVTX_MESSAGE_TYPE_ASCII;
        a.message.ascii = name;
        nvtxDomainRangePushEx(domain(), &a);
    }
    ~TraceRange() {
        if (on_) nvtxDomainRangePop(domain());
    }
    TraceRange(const TraceRange&) = delete;
    TraceRange& operator=(const TraceRange&) = delete;

private:
    static bool enabled() {
        static const bool on = [] {
            const char* v = std::getenv("KLEOS_NVTX");
            return v && v[0] == '1';
        }();
        return on;
    }
    static nvtxDomainHandle_t domain() {
        static nvtxDomainHandle_t d = nvtxDomainCreateA("Kleos");
        return d;
    }
    bool on_;
};

State g;
NcclApi nccl;
int g_device_request = -1;

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g.last_error = buf;
    std::fprintf(stderr, "[kleos_b200] %s\n", buf);
    return code;
}

#define KLEOS_CUDA(expr)                                                                  \
    do {                                                                                  \
        cudaError_t err__ = (expr);                                                       \
        if (err__ != cudaSuccess)                                                         \
            return fail(KLEOS_E_CUDA, "%s failed: %s (%s:%d)", #expr,                     \
                        cudaGetErrorString(err__), __FILE__, __LINE__);                   \
    } while (0)

#define KLEOS_NCCL(expr)                                                                  \
    do {                                                                                  \
        ncclResult_t r__ = (expr);                                                        \
        if (r__ != ncclSuccess)                                                           \
            return fail(KLEOS_E_BOOTSTRAP, "%s failed: %s", #expr,                        \
                        nccl.GetErrorString ? nccl.GetErrorString(r__) : "nccl error");   \
    } while (0)

int load_nccl() {
    if (nccl.handle) return KLEOS_OK;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        nccl.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (nccl.handle) break;
    }
    if (!nccl.handle) return fail(KLEOS_E_BOOTSTRAP, "cannot load libnccl: %s", dlerror());
    auto sym = [&](const char* s) { return dlsym(nccl.handle, s); };
    nccl.GetUniqueId = reinterpret_cast<decltype(nccl.GetUniqueId)>(sym("ncclGetUniqueId"));
    nccl.CommInitRank = reinterpret_cast<decltype(nccl.CommInitRank)>(sym("ncclCommInitRank"));
    nccl.AllGather = reinterpret_cast<decltype(nccl.AllGather)>(sym("ncclAllGather"));
    nccl.CommDestroy = reinterpret_cast<decltype(nccl.CommDestroy)>(sym("ncclCommDestroy"));
    nccl.GetErrorString = reinterpret_cast<decltype(nccl.GetErrorString)>(sym("ncclGetErrorString"));
    if (!nccl.GetUniqueId || !nccl.CommInitRank || !nccl.AllGather || !nccl.CommDestroy)
        return fail(KLEOS_E_BOOTSTRAP, "libnccl lacks a required symbol");
    return KLEOS_OK;
}

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

template <typename T>
int dev_alloc(T** p, size_t count) {
    KLEOS_CUDA(cudaMalloc(reinterpret_cast<void**>(p), count * sizeof(T)));
    KLEOS_CUDA(cudaMemset(*p, 0, count * sizeof(T)));
    return KLEOS_OK;
}

// All-gather `bytes` bytes per rank through a temporary device buffer.
int all_gather_bytes(const void* mine, void* all, size_t bytes) {
    if (!g.comm || !nccl.AllGather) return fail(KLEOS_E_STATE, "ranks are not connected");
    struct Temp {  // freed on every way out
        char* p = nullptr;
        ~Temp() { cudaFree(p); }
    } d;
    KLEOS_CUDA(cudaMalloc(&d.p, bytes * (g.world + 1)));
    KLEOS_CUDA(cudaMemcpy(d.p, mine, bytes, cudaMemcpyHostToDevice));
    KLEOS_NCCL(nccl.AllGather(d.p, d.p + bytes, bytes, ncclChar, g.comm, cudaStreamPerThread));
    KLEOS_CUDA(cudaStreamSynchronize(cudaStreamPerThread));
    KLEOS_CUDA(cudaMemcpy(all, d.p + bytes, bytes * g.world, cudaMemcpyDeviceToHost));
    return KLEOS_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;

// Matrix [rows][cols] of the layer's element type with cols contiguous; box = box_cols columns x
// box_rows rows, 128-byte swizzle (64 16-bit or 32 4-byte elements = 128 bytes, the swizzle span).
int make_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint32_t box_rows,
             uint32_t box_cols = 64, bool swizzle = true, int promo = 3) {
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        KLEOS_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q));
        if (!fn || q != cudaDriverEntryPointSuccess)
            return fail(KLEOS_E_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
        g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    const cuuint64_t dims[2] = {cols, rows};
    const cuuint64_t strides[1] = {cols * (cuuint64_t)g.cfg.elem_bytes};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapDataType dt = g.cfg.torch_dtype == 3   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                   : g.cfg.torch_dtype == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                            : CU_TENSOR_MAP_DATA_TYPE_FLOAT32;
    const CUresult r = g_encode(map, dt, 2, const_cast<void*>(base),
                                dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                swizzle ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                                promo == 0 ? CU_TENSOR_MAP_L2_PROMOTION_NONE
                                : promo == 1 ? CU_TENSOR_MAP_L2_PROMOTION_L2_64B
                                : promo == 2 ? CU_TENSOR_MAP_L2_PROMOTION_L2_128B
                                             : CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(KLEOS_E_CUDA, "cuTensorMapEncodeTiled failed: %d", (int)r);
    return KLEOS_OK;
}

struct Sections {
    const char *A, *Wg, *W1, *W2, *b1, *b2;
    char *probs, *out;
};

Sections slice(const void* iP, void* oP) {
    const LayerConfig& c = g.cfg;
    const size_t eb = c.elem_bytes;
    Sections s;
    s.A = static_cast<const char*>(iP);
    s.Wg = s.A + (size_t)c.S * c.H * eb;
    s.W1 = s.Wg + (g.dense ? 0 : (size_t)c.PX * c.H * eb);
    s.W2 = s.W1 + (size_t)g.nLx * c.I * c.H * eb;
    s.b1 = s.W2 + (size_t)g.nLx * c.H * c.I * eb;
    s.b2 = s.b1 + (size_t)g.nLx * c.I * eb;
    s.probs = static_cast<char*>(oP);
    s.out = s.probs + (g.dense ? 0 : (size_t)c.S * c.PX * eb);
    return s;
}

int ensure_maps(const Sections& s) {
    if ((!g.use_tc && !g.use_tf32_tc) || g.maps_for_iP == s.A) return KLEOS_OK;
    const LayerConfig& c = g.cfg;
    // the dense layer multiplies the activations where they lie: S rows instead of the cells
    const uint64_t cell_rows = g.dense ? (uint64_t)c.S : (uint64_t)g.world * g.nLx * c.pEC;
    int rc;
    if (g.use_tf32_tc) {
        const uint32_t bk = gemm_tf32::BK;
        if ((rc = make_map(&g.map_x, g.dense ? s.A : g.arena + g.lay.xcell, cell_rows, c.H, gemm_tf32::BM, bk))) return rc;
        if ((rc = make_map(&g.map_w1, s.W1, (uint64_t)g.nLx * c.I, c.H, gemm_tf32::BN, bk))) return rc;
        if ((rc = make_map(&g.map_y1, g.y1, cell_rows, c.I, gemm_tf32::BM, bk))) return rc;
        if ((rc = make_map(&g.map_w2, s.W2, (uint64_t)g.nLx * c.H, c.I, gemm_tf32::BN, bk))) return rc;
        if (c.PX <= 128 && !g.dense) {
            if ((rc = make_map(&g.map_act, s.A, c.S, c.H, route_tc::BM, bk))) return rc;
            if ((rc = make_map(&g.map_wg, s.Wg, c.PX, c.H, c.PX, bk))) return rc;
        }
        g.maps_for_iP = s.A;
        return KLEOS_OK;
    }
    if ((rc = make_map(&g.map_x, g.dense ? s.A : g.arena + g.lay.xcell, cell_rows, c.H, gemm_tc2::BM))) return rc;
    if ((rc = make_map(&g.map_y1, g.y1, cell_rows, c.I, gemm_tc2::BM))) return rc;
    const int promo = 3;  // 256-byte L2 promotion; 0/64/128 bytes measured the same on the C3 layer
    if ((rc = make_map(&g.map_w1h, s.W1, (uint64_t)g.nLx * c.I, c.H, gemm_tc2::BN / 2, 64, true, promo))) return rc;
    if ((rc = make_map(&g.map_w2h, s.W2, (uint64_t)g.nLx * c.H, c.I, gemm_tc2::BN / 2, 64, true, promo))) return rc;
    if (c.PX <= 128 && !g.dense) {
        if ((rc = make_map(&g.map_act, s.A, c.S, c.H, route_tc::BM))) return rc;
        if ((rc = make_map(&g.map_wg, s.Wg, c.PX, c.H, c.PX))) return rc;
        // the half of the gate weight each block of a pair loads when the router runs inside the
        // persistent kernel
        if ((rc = make_map(&g.map_wgh, s.Wg, c.PX, c.H, c.PX / 2))) return rc;
    }
    g.maps_for_iP = s.A;
    return KLEOS_OK;
}

template <typename T>
int launch_route(const RouteArgs& ra, cudaStream_t st) {
    const int grid = (ra.S + 63) / 64;
    if (ra.PX == 64) {
        { ++g.launches; route_kernel<T, 64><<<grid, 256, route_smem_bytes<64>(), st>>>(ra); }
    } else if (ra.PX == 128) {
        { ++g.launches; route_kernel<T, 128><<<grid, 256, route_smem_bytes<128>(), st>>>(ra); }
    } else if (ra.PX == 256) {
        static bool attr_set = false;
        if (!attr_set) {
            KLEOS_CUDA(cudaFuncSetAttribute(route_kernel<T, 256>,
                                            cudaFuncAttributeMaxDynamicSharedMemorySize,
                                            (int)route_smem_bytes<256>()));
            attr_set = true;
        }
        { ++g.launches; route_kernel<T, 256><<<grid, 256, route_smem_bytes<256>(), st>>>(ra); }
    } else {
        return fail(KLEOS_E_UNSUPPORTED, "more than 256 experts are not supported by the router");
    }
    { ++g.launches; refine_kernel<T><<<148, 256, 0, st>>>(ra); }
    return KLEOS_OK;
}

// The paired GEMM comes in two pipeline shapes (see gemm_tc2.cuh): deep = three 128-wide stages,
// otherwise six 64-wide stages.
template <typename TE, int kEpi>
void launch_tc2(bool deep, int grid, cudaStream_t st, const CUtensorMap& map_a, const CUtensorMap& map_b,
                const GemmArgs& ga) {
    if (deep)
        { ++g.launches; ffn_gemm_tc2<TE, kEpi, 2><<<grid, 256, gemm_tc2::SMEM_BYTES, st>>>(map_a, map_b, ga); }
    else
        { ++g.launches; ffn_gemm_tc2<TE, kEpi, 1><<<grid, 256, gemm_tc2::SMEM_BYTES, st>>>(map_a, map_b, ga); }
}

// The persistent kernel, instantiated per activation and per compile-time top-k of the combine.
template <typename TE>
void launch_flow(int act, int K, cudaStream_t st, const flow::Args& fa, const CUtensorMap* fa_act) {
    const int grid = g.flow_grid, smem = flow::SMEM_BYTES, thr = flow::kThreads;
    if (act == 0 && K == 2) { ++g.launches; moe_flow_kernel<TE, 0, 2><<<grid, thr, smem, st>>>(g.map_x, g.map_w1h, g.map_y1, g.map_w2h, *fa_act, g.map_wgh, fa); }
    else if (act == 0) { ++g.launches; moe_flow_kernel<TE, 0, 0><<<grid, thr, smem, st>>>(g.map_x, g.map_w1h, g.map_y1, g.map_w2h, *fa_act, g.map_wgh, fa); }
    else if (K == 2) { ++g.launches; moe_flow_kernel<TE, 1, 2><<<grid, thr, smem, st>>>(g.map_x, g.map_w1h, g.map_y1, g.map_w2h, *fa_act, g.map_wgh, fa); }
    else { ++g.launches; moe_flow_kernel<TE, 1, 0><<<grid, thr, smem, st>>>(g.map_x, g.map_w1h, g.map_y1, g.map_w2h, *fa_act, g.map_wgh, fa); }
}

// TF32 layers: one launch of the kind::tf32 GEMM with the epilogue chosen at compile time.
void launch_tf32(int epi, cudaStream_t st, const CUtensorMap& map_a, const CUtensorMap& map_b,
                 const GemmArgs& ga) {
    const int grid = g.sm_count, smem = gemm_tf32::SMEM_BYTES;
    if (epi == 0) { ++g.launches; ffn_gemm_tf32<0><<<grid, 256, smem, st>>>(map_a, map_b, ga); }
    else if (epi == 1) { ++g.launches; ffn_gemm_tf32<1><<<grid, 256, smem, st>>>(map_a, map_b, ga); }
    else { ++g.launches; ffn_gemm_tf32<2><<<grid, 256, smem, st>>>(map_a, map_b, ga); }
}

// Optional replacement of the activation input and the layer-output destination of one
// forward (used by the pipelined host path, whose staging buffers live outside iP / oP).
struct Staging {
    const char* A;
    char* out;
    const CUtensorMap* map_act;
};

// num_experts == 1: out = (act(A W1^T + b1)) W2^T + b2 over this rank's S tokens, both GEMMs by
// the expert-FFN kernels in their local-output mode over a fixed panel list (one panel per 128
// tokens, written once at initialisation).  Follows the reference's dense kernel
// (moe/fffn.cuh:31-167): intermediate rounded to the element type, identity epilogue on the
// second GEMM, no gate, no scaling.
template <typename T>
int forward_dense(const Sections& s, const CUtensorMap* map_a, cudaStream_t st, bool timed) {
    const LayerConfig& c = g.cfg;
    int evi = 0;
    auto mark = [&]() -> cudaError_t { return timed ? cudaEventRecord(g.ev[evi++], st) : cudaSuccess; };
    for (int i = 0; i < 5; ++i) KLEOS_CUDA(mark());  // start, route, slots, dispatch, plan: nothing to do
    GemmArgs ga{};
    ga.panels = g.panels; ga.le_start = g.le_start; ga.peers = g.peers; ga.lay = g.lay;
    ga.status = g.status; ga.wait_cycles = g.wait_cycles; ga.stats = nullptr;
    ga.nLx = 1; ga.pEC = c.S; ga.rank = g.rank; ga.elem_bytes = c.elem_bytes; ga.epoch = g.epoch;
    ga.le_begin = 0; ga.le_end = 1; ga.mode = 0;
    GemmArgs g1 = ga;
    g1.A = s.A; g1.B = s.W1; g1.bias = s.b1; g1.y1 = g.y1; g1.N = c.I; g1.Kd = c.H;
    g1.hidden_act = c.hidden_act;
    GemmArgs g2 = ga;
    g2.A = g.y1; g2.B = s.W2; g2.bias = s.b2; g2.y1 = s.out; g2.N = c.H; g2.Kd = c.I;
    g2.hidden_act = 2;  // identity
    if (g.use_tc) {
        if constexpr (sizeof(T) == 2) {
            const int grid = g.sm_count & ~1;
            const bool deep = c.S >= 512;
            if (c.hidden_act == 0)
                launch_tc2<T, 0>(deep, grid, st, *map_a, g.map_w1h, g1);
            else
                launch_tc2<T, 1>(deep, grid, st, *map_a, g.map_w1h, g1);
            KLEOS_CUDA(mark());
            launch_tc2<T, 2>(deep, grid, st, g.map_y1, g.map_w2h, g2);
        }
    } else if (g.use_tf32_tc) {
        launch_tf32(c.hidden_act, st, *map_a, g.map_w1, g1);
        KLEOS_CUDA(mark());
        launch_tf32(2, st, g.map_y1, g.map_w2, g2);
    } else {
        { ++g.launches; ffn_gemm_simt<T><<<g.sm_count * 2, 256, 0, st>>>(g1); }
        KLEOS_CUDA(mark());
        { ++g.launches; ffn_gemm_simt<T><<<g.sm_count * 2, 256, 0, st>>>(g2); }
    }
    KLEOS_CUDA(mark());
    KLEOS_CUDA(mark());  // combine: nothing to do
    KLEOS_CUDA(cudaGetLastError());
    return KLEOS_OK;
}

template <typename T>
int forward_typed(const void* iP, void* oP, cudaStream_t st, bool timed, const Staging* stg) {
    const LayerConfig& c = g.cfg;
    Sections s = slice(iP, oP);
    int rc = ensure_maps(s);
    if (rc) return rc;
    const CUtensorMap* act_map = &g.map_act;
    if (stg) {
        s.A = stg->A;
        s.out = stg->out;
        act_map = stg->map_act;
    }
    g.epoch += 1;
    if (g.dense) return forward_dense<T>(s, stg ? stg->map_act : &g.map_x, st, timed);
    int evi = 0;
    auto mark = [&]() -> cudaError_t { return timed ? cudaEventRecord(g.ev[evi++], st) : cudaSuccess; };
    KLEOS_CUDA(mark());

    bool routed_in_kernel = g.use_flow && g.fuse_route;
    if (routed_in_kernel) {
        KLEOS_CUDA(mark());
        KLEOS_CUDA(mark());
    } else if (g.route_by_flow) {
        if constexpr (sizeof(T) == 2) {
            // router of the separate launches: the routing phase of moe_flow_kernel on its own (gate
            // GEMM, top-k, in-place near-tie re-evaluation, grid barrier, slots, counts)
            flow::Args fr{};
            fr.tokens = s.A; fr.probs = s.probs; fr.topk = g.topk; fr.slots = g.slots; fr.mcw = g.mcw;
            fr.cell_tokens = g.cell_tokens; fr.counts = g.counts; fr.peers = g.peers; fr.lay = g.lay;
            fr.ctr = g.flow_ctr; fr.status = g.status; fr.wait_cycles = g.wait_cycles;
            fr.S = c.S; fr.H = c.H; fr.I = c.I; fr.E = c.E; fr.K = c.K; fr.PX = c.PX; fr.EC = c.EC;
            fr.pEC = c.pEC; fr.nLx = g.nLx; fr.rank = g.rank; fr.world = g.world; fr.epoch = g.epoch;
            fr.sub = 1; fr.unit_rows = flow::kUnitRows; fr.fuse_route = 1; fr.route_only = 1;
            fr.Wg = s.Wg; fr.gate_bias = g.bias; fr.tile_hist = g.tile_hist; fr.tie_eps = 1e-4f;
            launch_flow<T>(c.hidden_act, c.K, st, fr, act_map);
        }
        KLEOS_CUDA(mark());
        KLEOS_CUDA(mark());
        routed_in_kernel = true;  // nothing left to launch for routing and slots
    }
    // 1. router
    if (!routed_in_kernel) KLEOS_CUDA(cudaMemsetAsync(g.refine_count, 0, sizeof(int), st));
    RouteArgs ra{};
    ra.A = s.A; ra.Wg = s.Wg; ra.bias = g.bias; ra.probs = s.probs; ra.topk = g.topk;
    ra.mcw = g.mcw; ra.refine_list = g.refine_list; ra.refine_count = g.refine_count;
    ra.refine_logits = g.refine_logits; ra.refine_done = g.refine_done;
    ra.S = c.S; ra.H = c.H; ra.E = c.E; ra.K = c.K; ra.PX = c.PX; ra.tie_eps = 1e-4f;
    ra.col_partial = g.col_partial;  // null unless is_training
    int route_blocks = (c.S + 63) / 64;
    if (routed_in_kernel) {
        // nothing to launch here
    } else if ((g.use_tc || g.use_tf32_tc) && c.PX <= 128) {
        route_blocks = (c.S + route_tc::BM - 1) / route_tc::BM;
        if constexpr (!std::is_same<T, float>::value) {
            const int grid = (c.S + route_tc::BM - 1) / route_tc::BM;
            if (c.PX == 64)
                { ++g.launches; route_tc_kernel<T, 64><<<grid, 256, route_tc::Shape<64>::SMEM_BYTES, st>>>(
                    *act_map, g.map_wg, ra, g.status, g.wait_cycles, (int)g.epoch); }
            else
                { ++g.launches; route_tc_kernel<T, 128><<<grid, 256, route_tc::Shape<128>::SMEM_BYTES, st>>>(
                    *act_map, g.map_wg, ra, g.status, g.wait_cycles, (int)g.epoch); }
            { ++g.launches; refine_kernel<T><<<148, 256, 0, st>>>(ra); }
        }
    } else if ((rc = launch_route<T>(ra, st))) {
        return rc;
    }
    if (!routed_in_kernel) KLEOS_CUDA(mark());

    // 2. slots
    SlotArgs sa{};
    sa.topk = g.topk; sa.slots = g.slots; sa.cell_tokens = g.cell_tokens; sa.counts = g.counts;
    sa.S = c.S; sa.K = c.K; sa.E = c.E; sa.EC = c.EC; sa.pEC = c.pEC;
    for (int r = 0; r < kMaxWorld; ++r) sa.peer_arena[r] = g.peers.arena[r];
    sa.cflag_offset = g.lay.cflag; sa.rank = g.rank; sa.nLx = g.nLx; sa.epoch = g.epoch;
    sa.tile_hist = g.tile_hist;
    if (!routed_in_kernel) {
        { ++g.launches; tile_hist_kernel<<<(c.S + kSlotTile - 1) / kSlotTile, 256, 0, st>>>(sa); }
        { ++g.launches; slot_kernel<<<(c.S + kSlotTile - 1) / kSlotTile, 256, 0, st>>>(sa); }
        if (g.col_partial)
            { ++g.launches; gate_stats_kernel<<<1, 256, 0, st>>>(g.col_partial, route_blocks, c.PX, g.counts, c.S, c.E, g.gate_stats); }
        KLEOS_CUDA(mark());
    }

    if (g.use_flow) {
        if constexpr (sizeof(T) == 2) {
            // 3.-7. one persistent kernel: dispatch, plan, GEMM1, GEMM2, combine
            flow::Args fa{};
            fa.tokens = s.A; fa.b1 = s.b1; fa.b2 = s.b2; fa.y1 = g.y1; fa.out = s.out; fa.probs = s.probs;
            fa.topk = g.topk; fa.slots = g.slots; fa.mcw = g.mcw; fa.cell_tokens = g.cell_tokens;
            fa.counts = g.counts; fa.peers = g.peers; fa.lay = g.lay; fa.ctr = g.flow_ctr;
            fa.status = g.status; fa.stamps = timed ? g.flow_stamps : nullptr;
            fa.stalls = timed ? g.flow_stalls : nullptr; fa.debug = g.flow_debug;
            fa.wait_cycles = g.wait_cycles; fa.S = c.S; fa.H = c.H; fa.I = c.I; fa.E = c.E; fa.K = c.K;
            fa.PX = c.PX; fa.EC = c.EC; fa.pEC = c.pEC; fa.nLx = g.nLx; fa.rank = g.rank;
            fa.world = g.world; fa.epoch = g.epoch; fa.suppress = g.suppress_return_flag ? 1 : 0;
            // deep stages when an expert sees enough rows for the tensor pipe, not the weight
            // stream from HBM, to be the limit (about 260 FLOP per weight byte on this part)
            fa.sub = (long long)g.world * c.EC >= 512 ? 2 : 1;
            if (g.flow_sub) fa.sub = g.flow_sub;  // KLEOS_FLOW_SUB
            fa.unit_rows = g.flow_unit_rows;
            fa.fuse_route = routed_in_kernel ? 1 : 0;
            fa.Wg = s.Wg; fa.gate_bias = g.bias; fa.tile_hist = g.tile_hist; fa.tie_eps = 1e-4f;
            if (timed) {
                KLEOS_CUDA(cudaMemsetAsync(g.flow_stamps, 0,
                                           sizeof(long long) * g.flow_grid * flow::kStampSlots, st));
                KLEOS_CUDA(cudaMemsetAsync(g.flow_stalls, 0,
                                           sizeof(long long) * g.flow_grid * flow::kStallSlots, st));
            }
            for (int i = 0; i < 4; ++i) KLEOS_CUDA(mark());  // dispatch .. GEMM2: inside the kernel
            launch_flow<T>(c.hidden_act, c.K, st, fa, act_map);
        }
        KLEOS_CUDA(mark());
        KLEOS_CUDA(cudaGetLastError());
        return KLEOS_OK;
    }

    // 3. dispatch
    DispatchArgs da{};
    da.A = s.A; da.cell_tokens = g.cell_tokens; da.counts = g.counts; da.peers = g.peers;
    da.lay = g.lay; da.done_counter = g.done_dispatch; da.H = c.H; da.E = c.E; da.EC = c.EC;
    da.pEC = c.pEC; da.nLx = g.nLx; da.rank = g.rank; da.world = g.world; da.epoch = g.epoch;
    da.elem_bytes = c.elem_bytes; da.le_begin = 0; da.le_end = g.nLx;
    { ++g.launches; dispatch_kernel<<<g.sm_count * 4, 256, 0, st>>>(da); }
    KLEOS_CUDA(mark());
    // 4. plan: wait for every source's rows, list the panels
    PlanArgs pa{};
    pa.arena = g.arena; pa.lay = g.lay; pa.panels = g.panels; pa.le_start = g.le_start;
    pa.cell_counts = g.cell_counts; pa.status = g.status; pa.world = g.world; pa.nLx = g.nLx;
    pa.pEC = c.pEC; pa.epoch = g.epoch; pa.wait_cycles = g.wait_cycles; pa.rank = g.rank;
    pa.le_begin = 0; pa.le_end = g.nLx;
    { ++g.launches; plan_kernel<<<1, 1024, 0, st>>>(pa); }
    KLEOS_CUDA(mark());

    // 5./6. expert FFN
    GemmArgs ga{};
    ga.panels = g.panels; ga.le_start = g.le_start; ga.y1 = g.y1; ga.peers = g.peers;
    ga.lay = g.lay; ga.status = g.status; ga.wait_cycles = g.wait_cycles; ga.stats = nullptr;
    ga.hidden_act = c.hidden_act; ga.nLx = g.nLx; ga.pEC = c.pEC; ga.rank = g.rank;
    ga.elem_bytes = c.elem_bytes; ga.epoch = g.epoch; ga.le_begin = 0; ga.le_end = g.nLx;
    ga.ret.peers = g.peers; ga.ret.lay = g.lay; ga.ret.done_counter = g.done_gemm2;
    ga.ret.rank = g.rank; ga.ret.world = g.world; ga.ret.epoch = g.epoch;
    ga.ret.suppress = g.suppress_return_flag ? 1 : 0;
    GemmArgs g1 = ga;
    g1.A = g.arena + g.lay.xcell; g1.B = s.W1; g1.bias = s.b1; g1.N = c.I; g1.Kd = c.H; g1.mode = 0;
    GemmArgs g2 = ga;
    g2.A = g.y1; g2.B = s.W2; g2.bias = s.b2; g2.N = c.H; g2.Kd = c.I; g2.mode = 1;
    if (g.gemm_stats) {
        g1.stats = g.gemm_stats;
        g2.stats = g.gemm_stats + (size_t)g.sm_count * kStatSlots;
    }
    if (g.use_tc) {
        if constexpr (sizeof(T) == 2) {
            const int grid = g.sm_count & ~1;
            const bool deep = (long long)g.world * c.EC >= 512;
            if (c.hidden_act == 0)
                launch_tc2<T, 0>(deep, grid, st, g.map_x, g.map_w1h, g1);
            else
                launch_tc2<T, 1>(deep, grid, st, g.map_x, g.map_w1h, g1);
            KLEOS_CUDA(mark());
            launch_tc2<T, 2>(deep, grid, st, g.map_y1, g.map_w2h, g2);
            KLEOS_CUDA(mark());
        }
    } else if (g.use_tf32_tc) {
        launch_tf32(c.hidden_act, st, g.map_x, g.map_w1, g1);
        KLEOS_CUDA(mark());
        launch_tf32(2, st, g.map_y1, g.map_w2, g2);
        KLEOS_CUDA(mark());
    } else {
        { ++g.launches; ffn_gemm_simt<T><<<g.sm_count * 2, 256, 0, st>>>(g1); }
        KLEOS_CUDA(mark());
        { ++g.launches; ffn_gemm_simt<T><<<g.sm_count * 2, 256, 0, st>>>(g2); }
        KLEOS_CUDA(mark());
    }

    // 7. combine
    CombineArgs ca{};
    ca.arena = g.arena; ca.lay = g.lay; ca.probs = s.probs; ca.topk = g.topk; ca.slots = g.slots;
    ca.mcw = g.mcw; ca.out = s.out; ca.status = g.status; ca.S = c.S; ca.H = c.H; ca.K = c.K;
    ca.PX = c.PX; ca.pEC = c.pEC; ca.world = g.world; ca.epoch = g.epoch;
    ca.wait_cycles = g.wait_cycles;
    if (c.K == 2)
        { ++g.launches; combine_kernel<T, 2><<<g.sm_count * 4, 256, 0, st>>>(ca); }
    else if (c.K == 1)
        { ++g.launches; combine_kernel<T, 1><<<g.sm_count * 4, 256, 0, st>>>(ca); }
    else
        { ++g.launches; combine_kernel<T, 0><<<g.sm_count * 4, 256, 0, st>>>(ca); }
    KLEOS_CUDA(mark());
    KLEOS_CUDA(cudaGetLastError());
    return KLEOS_OK;
}

int forward_any(const void* iP, void* oP, cudaStream_t st, bool timed, const Staging* stg = nullptr) {
    if (!g.initialised) return fail(KLEOS_E_STATE, "kleos_forward before kleos_initialize");
    if (!iP || !oP) return fail(KLEOS_E_ARG, "null buffer");
    int rc;
    if (g.cfg.torch_dtype == 0) rc = forward_typed<float>(iP, oP, st, timed, stg);
    else if (g.cfg.torch_dtype == 1) rc = forward_typed<tf32_t>(iP, oP, st, timed, stg);
    else if (g.cfg.torch_dtype == 3) rc = forward_typed<__half>(iP, oP, st, timed, stg);
    else rc = forward_typed<__nv_bfloat16>(iP, oP, st, timed, stg);
    if (rc) return rc;
    // the status and debug accessors wait for this event: the caller's stream need not be the
    // per-thread default stream and may be non-blocking
    KLEOS_CUDA(cudaEventRecord(g.ev_last, st));
    return KLEOS_OK;
}

// Waits until the most recent forward has finished, whatever stream it was queued on.
int sync_last_forward() {
    KLEOS_CUDA(cudaEventSynchronize(g.ev_last));
    KLEOS_CUDA(cudaStreamSynchronize(cudaStreamPerThread));
    return KLEOS_OK;
}

template <typename TE>
int set_tc_attributes() {
    const auto dyn = cudaFuncAttributeMaxDynamicSharedMemorySize;
    KLEOS_CUDA(cudaFuncSetAttribute(route_tc_kernel<TE, 64>, dyn, route_tc::Shape<64>::SMEM_BYTES));
    KLEOS_CUDA(cudaFuncSetAttribute(route_tc_kernel<TE, 128>, dyn, route_tc::Shape<128>::SMEM_BYTES));
    KLEOS_CUDA(cudaFuncSetAttribute(ffn_gemm_tc2<TE, 0, 1>, dyn, gemm_tc2::SMEM_BYTES));
    KLEOS_CUDA(cudaFuncSetAttribute(ffn_gemm_tc2<TE, 0, 2>, dyn, gemm_tc2::SMEM_BYTES));
    KLEOS_CUDA(cudaFuncSetAttribute(ffn_gemm_tc2<TE, 1, 1>, dyn, gemm_tc2::SMEM_BYTES));
    KLEOS_CUDA(cudaFuncSetAttribute(ffn_gemm_tc2<TE, 1, 2>, dyn, gemm_tc2::SMEM_BYTES));
    KLEOS_CUDA(cudaFuncSetAttribute(ffn_gemm_tc2<TE, 2, 1>, dyn, gemm_tc2::SMEM_BYTES));
    KLEOS_CUDA(cudaFuncSetAttribute(ffn_gemm_tc2<TE, 2, 2>, dyn, gemm_tc2::SMEM_BYTES));
    KLEOS_CUDA(cudaFuncSetAttribute(moe_flow_kernel<TE, 0, 2>, dyn, flow::SMEM_BYTES));
    KLEOS_CUDA(cudaFuncSetAttribute(moe_flow_kernel<TE, 0, 0>, dyn, flow::SMEM_BYTES));
    KLEOS_CUDA(cudaFuncSetAttribute(moe_flow_kernel<TE, 1, 2>, dyn, flow::SMEM_BYTES));
    KLEOS_CUDA(cudaFuncSetAttribute(moe_flow_kernel<TE, 1, 0>, dyn, flow::SMEM_BYTES));
    // how many block pairs of the persistent kernel the device holds at once: its blocks wait on
    // one another, so the grid must not exceed that
    cudaLaunchConfig_t lc{};
    lc.gridDim = dim3((unsigned)(g.sm_count & ~1));
    lc.blockDim = dim3(flow::kThreads);
    lc.dynamicSmemBytes = flow::SMEM_BYTES;
    cudaLaunchAttribute at{};
    at.id = cudaLaunchAttributeClusterDimension;
    at.val.clusterDim.x = 2;
    at.val.clusterDim.y = 1;
    at.val.clusterDim.z = 1;
    lc.attrs = &at;
    lc.numAttrs = 1;
    int pairs = 0;
    KLEOS_CUDA(cudaOccupancyMaxActiveClusters(&pairs, moe_flow_kernel<TE, 0, 2>, &lc));
    g.flow_grid = 2 * std::min(pairs, g.sm_count / 2);
    return KLEOS_OK;
}

int ensure_host_pipe() {
    State::HostPipe& hp = g.hp;
    if (hp.ready) return KLEOS_OK;
    const LayerConfig& c = g.cfg;
    const size_t bytes = (size_t)c.S * c.H * c.elem_bytes;
    KLEOS_CUDA(cudaStreamCreateWithFlags(&hp.in, cudaStreamNonBlocking));
    KLEOS_CUDA(cudaStreamCreateWithFlags(&hp.out, cudaStreamNonBlocking));
    for (int b = 0; b < 2; ++b) {
        KLEOS_CUDA(cudaMalloc(reinterpret_cast<void**>(&hp.act[b]), bytes));
        KLEOS_CUDA(cudaMalloc(reinterpret_cast<void**>(&hp.res[b]), bytes));
        KLEOS_CUDA(cudaEventCreateWithFlags(&hp.in_done[b], cudaEventDisableTiming));
        KLEOS_CUDA(cudaEventCreateWithFlags(&hp.comp_done[b], cudaEventDisableTiming));
        KLEOS_CUDA(cudaEventCreateWithFlags(&hp.out_done[b], cudaEventDisableTiming));
        if (g.use_tc && c.PX <= 128) {
            int rc = make_map(&hp.map_act[b], hp.act[b], c.S, c.H, route_tc::BM);
            if (rc) return rc;
        } else if (g.use_tf32_tc && (g.dense || c.PX <= 128)) {
            // same box (128 rows x 32 words) serves the tf32 router and the dense layer's GEMM1
            int rc = make_map(&hp.map_act[b], hp.act[b], c.S, c.H, gemm_tf32::BM, gemm_tf32::BK);
            if (rc) return rc;
        }
    }
    hp.ready = true;
    return KLEOS_OK;
}

void release_all() {
    for (int r = 0; r < g.world; ++r)
        if (g.peer_opened[r]) cudaIpcCloseMemHandle(g.peers.arena[r]);
    cudaFree(g.arena);
    cudaFree(g.y1); cudaFree(g.topk); cudaFree(g.slots); cudaFree(g.cell_tokens);
    cudaFree(g.refine_list); cudaFree(g.refine_count); cudaFree(g.tile_hist); cudaFree(g.refine_done); cudaFree(g.refine_logits); cudaFree(g.le_start); cudaFree(g.mcw);
    cudaFree(g.bias); cudaFree(g.counts); cudaFree(g.done_dispatch); cudaFree(g.done_gemm2);
    cudaFree(g.cell_counts); cudaFree(g.flow_ctr); cudaFree(g.flow_stamps); cudaFree(g.flow_stalls); cudaFree(g.panels); cudaFree(g.status); cudaFree(g.gemm_stats);
    cudaFree(g.col_partial); cudaFree(g.gate_stats);
    for (auto& e : g.ev)
        if (e) cudaEventDestroy(e);
    if (g.hp.ready) {
        for (int b = 0; b < 2; ++b) {
            cudaFree(g.hp.act[b]); cudaFree(g.hp.res[b]);
            cudaEventDestroy(g.hp.in_done[b]); cudaEventDestroy(g.hp.comp_done[b]); cudaEventDestroy(g.hp.out_done[b]);
        }
        cudaStreamDestroy(g.hp.in); cudaStreamDestroy(g.hp.out);
    }
    if (g.ev_last) cudaEventDestroy(g.ev_last);
    if (g.comm && nccl.CommDestroy) nccl.CommDestroy(g.comm);
    g = State();
}

// Sizes reported to the caller.  A single-expert layer is the dense FFN: its packed input has no
// gate weight and its packed output no probabilities (reference moe/fffn.cuh:47-53), and every
// rank holds the one expert.
void fill_info(const LayerConfig& c, int rank, int world, kleos_layer_info* out) {
    const bool dense = c.E == 1;
    const int nlx = dense ? 1 : c.E / world;
    out->rank = rank; out->world = world; out->local_experts = nlx;
    out->S = c.S; out->H = c.H; out->I = c.I; out->E = c.E; out->K = c.K; out->EC = c.EC;
    out->pEC = c.pEC; out->PX = c.PX; out->torch_dtype = c.torch_dtype;
    out->hidden_act = c.hidden_act; out->elem_bytes = c.elem_bytes;
    out->input_elems = (int64_t)c.S * c.H + (dense ? 0 : (int64_t)c.PX * c.H) + 2LL * nlx * c.I * c.H +
                       (int64_t)nlx * (c.I + c.H);
    out->output_elems = (dense ? 0 : (int64_t)c.S * c.PX) + (int64_t)c.S * c.H;
}

}  // namespace
}  // namespace kleos

using namespace kleos;

extern "C" {

const char* kleos_error_string(int code) {
    switch (code) {
        case KLEOS_OK: return "ok";
        case KLEOS_E_CONFIG: return "invalid configuration";
        case KLEOS_E_STATE: return "wrong call order";
        case KLEOS_E_CUDA: return "CUDA call failed";
        case KLEOS_E_BOOTSTRAP: return "bootstrap failed";
        case KLEOS_E_MISMATCH: return "ranks disagree on the configuration";
        case KLEOS_E_DEVICE: return "device reported a timeout or bounds error";
        case KLEOS_E_UNSUPPORTED: return "unsupported dtype or shape";
        case KLEOS_E_ARG: return "bad argument";
        default: return "unknown";
    }
}

int kleos_get_unique_id(void* out_id128) {
    if (!out_id128) return fail(KLEOS_E_ARG, "null id buffer");
    int rc = load_nccl();
    if (rc) return rc;
    static_assert(sizeof(ncclUniqueId) == 128, "NCCL unique id is 128 bytes");
    ncclUniqueId id;
    KLEOS_NCCL(nccl.GetUniqueId(&id));
    std::memcpy(out_id128, &id, sizeof(id));
    return KLEOS_OK;
}

int kleos_config_probe(const char* config_json_path, int world, kleos_layer_info* out) {
    if (!config_json_path || !out) return fail(KLEOS_E_ARG, "null argument");
    LayerConfig c;
    const std::string err = load_config(config_json_path, &c);
    if (!err.empty()) return fail(KLEOS_E_CONFIG, "%s: %s", config_json_path, err.c_str());
    if (world < 1 || world > kMaxWorld || (c.E != 1 && c.E % world))
        return fail(KLEOS_E_CONFIG, "num_experts %d does not divide over %d ranks", c.E, world);
    fill_info(c, 0, world, out);
    return KLEOS_OK;
}

int kleos_set_device(int device) {
    if (g.initialised) return fail(KLEOS_E_STATE, "kleos_set_device after kleos_initialize");
    g_device_request = device;
    return KLEOS_OK;
}

static int initialize_impl(const char* config_json_path, int rank, int world, const void* nccl_id);

int kleos_initialize(const char* config_json_path, int rank, int world, const void* nccl_id) {
    TraceRange trace("kleos_initialize");
    if (g.initialised) return fail(KLEOS_E_STATE, "already initialised");
    const int rc = initialize_impl(config_json_path, rank, world, nccl_id);
    if (rc != KLEOS_OK) {
        // a failed set-up leaves nothing behind: device buffers, events, streams, peer mappings
        // and the communicator created so far are released, so the caller may try again
        const std::string why = g.last_error;
        release_all();
        g.last_error = why;
    }
    return rc;
}

static int initialize_impl(const char* config_json_path, int rank, int world, const void* nccl_id) {
    if (!config_json_path) return fail(KLEOS_E_ARG, "null config path");
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world)
        return fail(KLEOS_E_ARG, "rank %d / world %d out of range (max world %d)", rank, world, kMaxWorld);
    LayerConfig cfg;
    const std::string err = load_config(config_json_path, &cfg);
    if (!err.empty()) return fail(KLEOS_E_CONFIG, "%s: %s", config_json_path, err.c_str());
    const bool dense = cfg.E == 1;
    if (!dense && cfg.E % world)
        return fail(KLEOS_E_CONFIG, "num_experts %d does not divide over %d ranks", cfg.E, world);
    if (cfg.K > kMaxTopK) return fail(KLEOS_E_UNSUPPORTED, "expert_top_k > %d", kMaxTopK);
    if (cfg.E > 256) return fail(KLEOS_E_UNSUPPORTED, "num_experts > 256");
    if (world > 1 && !nccl_id && !dense) return fail(KLEOS_E_ARG, "world > 1 needs an NCCL unique id");

    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || ndev == 0)
        return fail(KLEOS_E_CUDA, "no CUDA device: this library has no CPU path");
    g.device = g_device_request >= 0 ? g_device_request : rank % ndev;
    KLEOS_CUDA(cudaSetDevice(g.device));
    cudaDeviceProp prop;
    KLEOS_CUDA(cudaGetDeviceProperties(&prop, g.device));
    if (prop.major != 10)
        return fail(KLEOS_E_UNSUPPORTED, "device is sm_%d%d; this library is built for sm_100a only",
                    prop.major, prop.minor);
    g.sm_count = prop.multiProcessorCount;
    g.clock_khz = prop.clockRate;
    g.cfg = cfg;
    g.rank = rank;
    g.world = world;
    g.dense = dense;
    g.nLx = dense ? 1 : cfg.E / world;
    g.epoch = 0;
    if (const char* w = std::getenv("KLEOS_WAIT_MS")) {
        // device wait budget in milliseconds (converted with the SM clock rate)
        g.wait_cycles = (long long)(std::atof(w) * 1e-3 * prop.clockRate * 1e3);
    }
    const char* simt = std::getenv("KLEOS_DEBUG_SIMT_GEMM");
    g.use_tc = (cfg.torch_dtype == 2 || cfg.torch_dtype == 3) && !(simt && simt[0] == '1');
    g.use_tf32_tc = cfg.torch_dtype == 1 && !(simt && simt[0] == '1');

    const size_t eb = cfg.elem_bytes;
    const size_t cell_bytes = (size_t)cfg.E * cfg.pEC * cfg.H * eb;  // world*nLx == E
    g.lay.xcell = 0;
    g.lay.ycell = align_up(g.lay.xcell + cell_bytes, 1024);
    g.lay.xflag = align_up(g.lay.ycell + cell_bytes, 1024);
    g.lay.cflag = align_up(g.lay.xflag + (size_t)cfg.E * 8, 1024);
    g.lay.yflag = align_up(g.lay.cflag + (size_t)cfg.E * 8, 1024);
    g.lay.ypflag = align_up(g.lay.yflag + (size_t)kMaxWorld * 8, 1024);
    g.lay.bytes = align_up(g.lay.ypflag + (size_t)cfg.E * (cfg.pEC / kTileM) * 8, 1024);

    int rc;
    if ((rc = dev_alloc(&g.arena, g.lay.bytes))) return rc;
    char* y1 = nullptr;
    if ((rc = dev_alloc(&y1, (size_t)cfg.E * cfg.pEC * cfg.I * eb))) return rc;
    g.y1 = y1;
    if ((rc = dev_alloc(&g.topk, (size_t)cfg.S * cfg.K))) return rc;
    if ((rc = dev_alloc(&g.slots, (size_t)cfg.S * cfg.K))) return rc;
    if ((rc = dev_alloc(&g.cell_tokens, (size_t)cfg.E * cfg.pEC))) return rc;
    if ((rc = dev_alloc(&g.refine_list, (size_t)cfg.S))) return rc;
    if ((rc = dev_alloc(&g.refine_count, 1))) return rc;
    if ((rc = dev_alloc(&g.tile_hist, (size_t)((cfg.S + kSlotTile - 1) / kSlotTile) * cfg.E))) return rc;
    if ((rc = dev_alloc(&g.refine_done, (size_t)cfg.S))) return rc;
    if ((rc = dev_alloc(&g.refine_logits, (size_t)cfg.S * cfg.E))) return rc;
    if ((rc = dev_alloc(&g.le_start, (size_t)g.nLx + 1))) return rc;
    if ((rc = dev_alloc(&g.mcw, (size_t)cfg.S))) return rc;
    if ((rc = dev_alloc(&g.bias, (size_t)cfg.E))) return rc;
    if ((rc = dev_alloc(&g.counts, (size_t)cfg.E))) return rc;
    if ((rc = dev_alloc(&g.done_dispatch, 1))) return rc;
    if ((rc = dev_alloc(&g.done_gemm2, 1))) return rc;
    if ((rc = dev_alloc(&g.cell_counts, (size_t)cfg.E))) return rc;
    if ((rc = dev_alloc(&g.panels, (size_t)cfg.E * cfg.pEC / kTileM))) return rc;
    if ((rc = dev_alloc(&g.status, 1))) return rc;
    if (cfg.is_training && !dense) {
        if ((rc = dev_alloc(&g.col_partial, (size_t)((cfg.S + 63) / 64) * cfg.PX))) return rc;
        if ((rc = dev_alloc(&g.gate_stats, (size_t)2 * cfg.E + 1))) return rc;
    }
    for (auto& e : g.ev) KLEOS_CUDA(cudaEventCreate(&e));
    KLEOS_CUDA(cudaEventCreateWithFlags(&g.ev_last, cudaEventDisableTiming));
    if (const char* gs = std::getenv("KLEOS_GEMM_STATS"))
        if (gs[0] == '1' && (rc = dev_alloc(&g.gemm_stats, (size_t)2 * g.sm_count * kStatSlots))) return rc;

    if (g.use_tc) {
        if (cfg.torch_dtype == 2) rc = set_tc_attributes<__nv_bfloat16>();
        else rc = set_tc_attributes<__half>();
        if (rc) return rc;
    }
    if (g.use_tf32_tc) {
        const auto dyn = cudaFuncAttributeMaxDynamicSharedMemorySize;
        KLEOS_CUDA(cudaFuncSetAttribute(ffn_gemm_tf32<0>, dyn, gemm_tf32::SMEM_BYTES));
        KLEOS_CUDA(cudaFuncSetAttribute(ffn_gemm_tf32<1>, dyn, gemm_tf32::SMEM_BYTES));
        KLEOS_CUDA(cudaFuncSetAttribute(ffn_gemm_tf32<2>, dyn, gemm_tf32::SMEM_BYTES));
        KLEOS_CUDA(cudaFuncSetAttribute(route_tc_kernel<tf32_t, 64>, dyn, route_tc::Shape<64>::SMEM_BYTES));
        KLEOS_CUDA(cudaFuncSetAttribute(route_tc_kernel<tf32_t, 128>, dyn, route_tc::Shape<128>::SMEM_BYTES));
    }
    // KLEOS_FLOW=1 runs 16-bit routed layers as ONE persistent kernel (moe_flow.cuh).  It is the
    // reference's arrangement and passes the same parity tests, but on this machine it has so far
    // measured slower than the separate launches at every world size (its dispatch and combine
    // traffic share the SMs' memory pipeline with the tile stream), so the separate launches stay
    // the default.  The kernel keeps its panel list and per-cell tables in shared memory; layers
    // beyond those tables always run as separate launches.
    const char* flow_env = std::getenv("KLEOS_FLOW");
    g.use_flow = g.use_tc && !dense && flow_env && flow_env[0] == '1' && g.flow_grid >= 2 &&
                 (size_t)cfg.E * cfg.pEC / kTileM <= (size_t)flow::kMaxPanels && cfg.E <= flow::kMaxCells &&
                 g.nLx <= flow::kMaxLocal;
    const char* fr = std::getenv("KLEOS_FUSE_ROUTE");
    g.fuse_route = g.use_flow && cfg.PX <= 128 && !cfg.is_training && !(fr && fr[0] == '0');
    // Separate launches of a 16-bit layer use the same kernel's routing phase as their router
    // (KLEOS_ROUTE_KERNELS=1: the gate, near-tie, histogram and slot kernels instead)
    const char* rk = std::getenv("KLEOS_ROUTE_KERNELS");
    g.route_by_flow = g.use_tc && !dense && !g.use_flow && cfg.PX <= 128 && !cfg.is_training &&
                      g.flow_grid >= 2 && cfg.E <= flow::kMaxCells && !(rk && rk[0] == '1');
    if (g.use_flow || g.route_by_flow) {
        flow::Counters* ctr = nullptr;
        if ((rc = dev_alloc(&ctr, 2))) return rc;
        g.flow_ctr = ctr;
        if ((rc = dev_alloc(&g.flow_stamps, (size_t)g.flow_grid * flow::kStampSlots))) return rc;
        if ((rc = dev_alloc(&g.flow_stalls, (size_t)g.flow_grid * flow::kStallSlots))) return rc;
        if (const char* dbg = std::getenv("KLEOS_FLOW_DEBUG")) g.flow_debug = std::atoi(dbg);
        if (const char* fs = std::getenv("KLEOS_FLOW_SUB")) g.flow_sub = std::atoi(fs) == 1 ? 1 : (std::atoi(fs) == 2 ? 2 : 0);
        if (const char* ur = std::getenv("KLEOS_UNIT_ROWS"))
            g.flow_unit_rows = std::min(flow::kUnitRows, std::max(1, std::atoi(ur)));
    }

    for (int r = 0; r < kMaxWorld; ++r) g.peers.arena[r] = nullptr;
    g.peers.arena[rank] = g.arena;
    if (dense) {
        // fixed work list of the dense layer: one panel per 128 tokens, one "expert"
        const int np = (cfg.S + kTileM - 1) / kTileM;
        std::vector<PanelEntry> panels(np);
        for (int i = 0; i < np; ++i) panels[i] = PanelEntry{i * kTileM, std::min(kTileM, cfg.S - i * kTileM), 0, rank};
        const int le_start[2] = {0, np};
        KLEOS_CUDA(cudaMemcpy(g.panels, panels.data(), sizeof(PanelEntry) * np, cudaMemcpyHostToDevice));
        KLEOS_CUDA(cudaMemcpy(g.le_start, le_start, sizeof(le_start), cudaMemcpyHostToDevice));
    }
    // ranks of a dense layer never exchange anything, so they are not connected
    if (world > 1 && !dense) {
        if ((rc = load_nccl())) return rc;
        ncclUniqueId id;
        std::memcpy(&id, nccl_id, sizeof(id));
        KLEOS_NCCL(nccl.CommInitRank(&g.comm, world, id, rank));
        // every rank must have read the same layer
        struct Hello {
            int v[12];
            cudaIpcMemHandle_t h;
        } mine{}, all[kMaxWorld];
        const int fields[12] = {cfg.S, cfg.H, cfg.I, cfg.E, cfg.K, cfg.EC, cfg.pEC, cfg.PX,
                                cfg.torch_dtype, cfg.hidden_act, world, (int)(g.lay.bytes >> 10)};
        std::memcpy(mine.v, fields, sizeof(fields));
        KLEOS_CUDA(cudaIpcGetMemHandle(&mine.h, g.arena));
        if ((rc = all_gather_bytes(&mine, all, sizeof(Hello)))) return rc;
        for (int r = 0; r < world; ++r)
            if (std::memcmp(all[r].v, mine.v, sizeof(mine.v)) != 0)
                return fail(KLEOS_E_MISMATCH, "rank %d read a different layer configuration than rank %d", r, rank);
        for (int r = 0; r < world; ++r) {
            if (r == rank) continue;
            void* p = nullptr;
            const cudaError_t e = cudaIpcOpenMemHandle(&p, all[r].h, cudaIpcMemLazyEnablePeerAccess);
            if (e != cudaSuccess)
                return fail(KLEOS_E_BOOTSTRAP, "cannot map the cells of rank %d: %s", r, cudaGetErrorString(e));
            g.peers.arena[r] = static_cast<char*>(p);
            g.peer_opened[r] = true;
        }
        // second exchange doubles as a barrier: nobody stores into a peer before it is mapped
        int token = rank, tokens[kMaxWorld];
        if ((rc = all_gather_bytes(&token, tokens, sizeof(int)))) return rc;
    }
    KLEOS_CUDA(cudaDeviceSynchronize());
    g.initialised = true;
    return KLEOS_OK;
}

int kleos_set_gate_bias(const float* host_bias, int n) {
    if (!g.initialised) return fail(KLEOS_E_STATE, "not initialised");
    if (!host_bias) {
        KLEOS_CUDA(cudaMemset(g.bias, 0, sizeof(float) * g.cfg.E));
        return KLEOS_OK;
    }
    if (n != g.cfg.E) return fail(KLEOS_E_ARG, "gate bias needs %d values, got %d", g.cfg.E, n);
    KLEOS_CUDA(cudaMemcpy(g.bias, host_bias, sizeof(float) * n, cudaMemcpyHostToDevice));
    return KLEOS_OK;
}

int kleos_forward(const void* iP, void* oP, void* stream) {
    TraceRange trace("kleos_forward");
    cudaStream_t st = stream ? static_cast<cudaStream_t>(stream) : cudaStreamPerThread;
    return forward_any(iP, oP, st, false);
}

int kleos_forward_bench(const void* iP, void* oP, int skip, int trials, float* ms) {
    TraceRange trace("kleos_forward_bench");
    if (!ms || trials < 1 || skip < 0) return fail(KLEOS_E_ARG, "bad bench arguments");
    cudaStream_t st = cudaStreamPerThread;
    int rc;
    for (int i = 0; i < skip; ++i)
        if ((rc = forward_any(iP, oP, st, false))) return rc;
    KLEOS_CUDA(cudaStreamSynchronize(st));
    float acc[kPhases] = {};
    double macc[flow::kStampSlots] = {};
    std::vector<long long> stamps;
    // timed trials record per-phase events; the total is first event to last event
    for (int i = 0; i < trials; ++i) {
        // three untimed forwards run straight into the timed one, so that the ranks enter it the way
        // they do in a stream of forwards (coupled by the exit handshake of the forward before)
        // and not skewed by the host's synchronise of the previous trial
        for (int w = 0; w < 3; ++w)
            if ((rc = forward_any(iP, oP, st, false))) return rc;
        if ((rc = forward_any(iP, oP, st, true))) return rc;
        KLEOS_CUDA(cudaStreamSynchronize(st));
        for (int p = 0; p < kPhases - 1; ++p) {
            float v = 0;
            KLEOS_CUDA(cudaEventElapsedTime(&v, g.ev[p], g.ev[p + 1]));
            acc[p] += v;
        }
        float v = 0;
        KLEOS_CUDA(cudaEventElapsedTime(&v, g.ev[0], g.ev[kPhases - 1]));
        acc[kPhases - 1] += v;
        if (g.use_flow && !g.dense) {
            // milestones of the persistent kernel from the blocks' global-timer stamps: the latest
            // block for each, counted from the earliest block's start (first tile: the earliest)
            stamps.resize((size_t)g.flow_grid * flow::kStampSlots);
            KLEOS_CUDA(cudaMemcpy(stamps.data(), g.flow_stamps, stamps.size() * sizeof(long long),
                                  cudaMemcpyDeviceToHost));
            long long t0 = 0, hi[flow::kStampSlots] = {}, first_tile = 0;
            for (int b = 0; b < g.flow_grid; ++b) {
                const long long* sb = &stamps[(size_t)b * flow::kStampSlots];
                if (sb[flow::kStart] && (!t0 || sb[flow::kStart] < t0)) t0 = sb[flow::kStart];
                if (sb[flow::kFirstTile] && (!first_tile || sb[flow::kFirstTile] < first_tile)) first_tile = sb[flow::kFirstTile];
                for (int k = 0; k < flow::kStampSlots; ++k) hi[k] = std::max(hi[k], sb[k]);
            }
            hi[flow::kFirstTile] = first_tile;
            g.flow_raw = stamps;
            for (int k = 0; k < flow::kStampSlots; ++k) macc[k] += hi[k] > t0 ? (double)(hi[k] - t0) * 1e-6 : 0.0;
        }
    }
    for (int p = 0; p < kPhases; ++p) g.phase_ms[p] = acc[p] / trials;
    if (g.use_flow && !g.dense) {
        float* m = g.flow_ms;
        for (int k = 0; k < flow::kStampSlots; ++k) m[k] = (float)(macc[k] / trials);
        // the per-phase slots, as far as phases still exist inside one kernel: when the last row was
        // dispatched and the plan was known (both from kernel start), the GEMM1 and GEMM2 spans of the
        // tile stream, and the tail between the last tile and the end (combine of the last tokens)
        g.phase_ms[2] = m[flow::kDispatched] - m[flow::kSlotted];
        g.phase_ms[3] = m[flow::kPlanned] - m[flow::kSlotted];
        if (g.fuse_route) {  // the router's two stages, each ended by a grid barrier
            g.phase_ms[0] = m[flow::kRouted];
            g.phase_ms[1] = m[flow::kSlotted] - m[flow::kRouted];
        }
        g.phase_ms[4] = m[flow::kLastGemm1] - m[flow::kFirstTile];
        g.phase_ms[5] = m[flow::kLastTile] - m[flow::kLastGemm1];
        g.phase_ms[6] = m[flow::kEnd] - m[flow::kLastTile];
    }
    // back-to-back launches between one pair of events, as the reference times it
    cudaEvent_t a = g.ev[0], b = g.ev[kPhases];
    KLEOS_CUDA(cudaEventRecord(a, st));
    for (int i = 0; i < trials; ++i)
        if ((rc = forward_any(iP, oP, st, false))) return rc;
    KLEOS_CUDA(cudaEventRecord(b, st));
    KLEOS_CUDA(cudaStreamSynchronize(st));
    float total = 0;
    KLEOS_CUDA(cudaEventElapsedTime(&total, a, b));
    *ms = total / trials;
    kleos_status s;
    if ((rc = kleos_last_status(&s))) return rc;
    if (s.code) return fail(KLEOS_E_DEVICE, "device status: where=%d detail=%d epoch=%d", s.where, s.detail, s.epoch);
    return KLEOS_OK;
}

int kleos_forward_host(const void* host_activations, void* iP, void* oP, void* host_output) {
    TraceRange trace("kleos_forward_host");
    if (!g.initialised) return fail(KLEOS_E_STATE, "not initialised");
    if (!host_activations || !iP || !oP || !host_output) return fail(KLEOS_E_ARG, "null buffer");
    const LayerConfig& c = g.cfg;
    cudaStream_t st = cudaStreamPerThread;
    const size_t act_bytes = (size_t)c.S * c.H * c.elem_bytes;
    KLEOS_CUDA(cudaMemcpyAsync(iP, host_activations, act_bytes, cudaMemcpyHostToDevice, st));
    int rc = forward_any(iP, oP, st, false);
    if (rc) return rc;
    const char* out = static_cast<const char*>(oP) + (g.dense ? 0 : (size_t)c.S * c.PX * c.elem_bytes);
    KLEOS_CUDA(cudaMemcpyAsync(host_output, out, act_bytes, cudaMemcpyDeviceToHost, st));
    KLEOS_CUDA(cudaStreamSynchronize(st));
    return KLEOS_OK;
}

int kleos_forward_host_async(const void* host_activations, void* iP, void* oP, void* host_output) {
    TraceRange trace("kleos_forward_host_async");
    if (!g.initialised) return fail(KLEOS_E_STATE, "not initialised");
    if (!host_activations || !iP || !oP || !host_output) return fail(KLEOS_E_ARG, "null buffer");
    int rc = ensure_host_pipe();
    if (rc) return rc;
    State::HostPipe& hp = g.hp;
    const LayerConfig& c = g.cfg;
    const size_t bytes = (size_t)c.S * c.H * c.elem_bytes;
    cudaStream_t st = cudaStreamPerThread;
    const int b = (int)(hp.step & 1);
    const bool reuse = hp.step >= 2;  // the step that last used these staging buffers
    if (reuse) KLEOS_CUDA(cudaStreamWaitEvent(hp.in, hp.comp_done[b], 0));
    KLEOS_CUDA(cudaMemcpyAsync(hp.act[b], host_activations, bytes, cudaMemcpyHostToDevice, hp.in));
    KLEOS_CUDA(cudaEventRecord(hp.in_done[b], hp.in));
    KLEOS_CUDA(cudaStreamWaitEvent(st, hp.in_done[b], 0));
    if (reuse) KLEOS_CUDA(cudaStreamWaitEvent(st, hp.out_done[b], 0));
    const Staging stg{hp.act[b], hp.res[b], &hp.map_act[b]};
    if ((rc = forward_any(iP, oP, st, false, &stg))) return rc;
    KLEOS_CUDA(cudaEventRecord(hp.comp_done[b], st));
    KLEOS_CUDA(cudaStreamWaitEvent(hp.out, hp.comp_done[b], 0));
    KLEOS_CUDA(cudaMemcpyAsync(host_output, hp.res[b], bytes, cudaMemcpyDeviceToHost, hp.out));
    KLEOS_CUDA(cudaEventRecord(hp.out_done[b], hp.out));
    hp.step += 1;
    return KLEOS_OK;
}

int kleos_host_sync(void) {
    TraceRange trace("kleos_host_sync");
    if (!g.initialised) return fail(KLEOS_E_STATE, "not initialised");
    if (g.hp.ready) {
        KLEOS_CUDA(cudaStreamSynchronize(g.hp.in));
        KLEOS_CUDA(cudaStreamSynchronize(cudaStreamPerThread));
        KLEOS_CUDA(cudaStreamSynchronize(g.hp.out));
    }
    kleos_status s;
    int rc = kleos_last_status(&s);
    if (rc) return rc;
    if (s.code) return fail(KLEOS_E_DEVICE, "device status: where=%d detail=%d epoch=%d", s.where, s.detail, s.epoch);
    return KLEOS_OK;
}

int kleos_get_rank(void) { return g.initialised ? g.rank : KLEOS_E_STATE; }
int kleos_local_experts(void) { return g.initialised ? g.nLx : KLEOS_E_STATE; }

int kleos_get_info(kleos_layer_info* out) {
    if (!g.initialised) return fail(KLEOS_E_STATE, "not initialised");
    if (!out) return fail(KLEOS_E_ARG, "null info");
    fill_info(g.cfg, g.rank, g.world, out);
    return KLEOS_OK;
}

int kleos_last_status(kleos_status* out) {
    if (!g.initialised) return fail(KLEOS_E_STATE, "not initialised");
    if (!out) return fail(KLEOS_E_ARG, "null status");
    { const int src = sync_last_forward(); if (src) return src; }
    DeviceStatus d;
    KLEOS_CUDA(cudaMemcpy(&d, g.status, sizeof(d), cudaMemcpyDeviceToHost));
    out->code = d.code; out->where = d.where; out->detail = d.detail; out->epoch = d.epoch;
    return KLEOS_OK;
}

int kleos_clear_status(void) {
    if (!g.initialised) return fail(KLEOS_E_STATE, "not initialised");
    { const int src = sync_last_forward(); if (src) return src; }
    KLEOS_CUDA(cudaMemset(g.status, 0, sizeof(DeviceStatus)));
    return KLEOS_OK;
}

int kleos_debug_routing(int32_t* topk, int32_t* slots, uint32_t* counts, float* mcw) {
    if (!g.initialised) return fail(KLEOS_E_STATE, "not initialised");
    if (g.dense) return fail(KLEOS_E_UNSUPPORTED, "a single-expert layer does no routing");
    const LayerConfig& c = g.cfg;
    { const int src = sync_last_forward(); if (src) return src; }
    const size_t sk = (size_t)c.S * c.K;
    if (topk) KLEOS_CUDA(cudaMemcpy(topk, g.topk, sk * 4, cudaMemcpyDeviceToHost));
    if (slots) KLEOS_CUDA(cudaMemcpy(slots, g.slots, sk * 4, cudaMemcpyDeviceToHost));
    if (counts) KLEOS_CUDA(cudaMemcpy(counts, g.counts, (size_t)c.E * 4, cudaMemcpyDeviceToHost));
    if (mcw) KLEOS_CUDA(cudaMemcpy(mcw, g.mcw, (size_t)c.S * 4, cudaMemcpyDeviceToHost));
    return KLEOS_OK;
}

int kleos_placement_model(const char* config_json_path, uint32_t* moe_stages, uint32_t* p2p_buffer_mb,
                          uint32_t* grad_buffer_mb) {
    if (!config_json_path || !moe_stages || !p2p_buffer_mb || !grad_buffer_mb)
        return fail(KLEOS_E_ARG, "null argument");
    LayerConfig c;
    const std::string err = load_config(config_json_path, &c);
    if (!err.empty()) return fail(KLEOS_E_CONFIG, "%s: %s", config_json_path, err.c_str());
    if (c.mini_batch < 1 || c.moe_frequency < 1) return fail(KLEOS_E_CONFIG, "mini_batch and moe_frequency must be >= 1");
    // types.cuh:487-494: global MoE stages, parameter count, gradient and dispatch buffers in MB
    const long long mib = 1024LL * 1024LL;
    *moe_stages = (uint32_t)((c.is_training ? 3 : 1) * (c.global_batch / c.mini_batch) * (c.num_layers / c.moe_frequency));
    const long long H = c.H;
    const long long pc = H * ((long long)c.num_layers * (12 * H + 13) + ((long long)c.vocab_size + H));
    *grad_buffer_mb = (uint32_t)((pc + mib - 1) / mib);
    *p2p_buffer_mb = (uint32_t)(((long long)c.S * H + mib - 1) / mib);
    return KLEOS_OK;
}

int kleos_plan_placement(const kleos_placement_request* rq, kleos_placement_result* res,
                         uint32_t* device_to_group, uint32_t* group_ranks, uint32_t* expert_to_member) {
    TraceRange trace("kleos_plan_placement");
    if (!rq || !res) return fail(KLEOS_E_ARG, "null argument");
    if (rq->world < 1 || rq->world > 4096 || rq->num_experts < 1 || rq->num_experts > 65535 ||
        rq->expert_cost < 1 || rq->expert_cost > 65535 || !rq->alpha || !rq->beta || !rq->rate || !rq->mem)
        return fail(KLEOS_E_ARG, "planner request out of range");
    placement::Inputs in;
    in.world = rq->world;
    const size_t ww = (size_t)rq->world * rq->world;
    in.alpha.assign(rq->alpha, rq->alpha + ww);
    in.beta.assign(rq->beta, rq->beta + ww);
    in.rate.assign(rq->rate, rq->rate + rq->world);
    in.mem.assign(rq->mem, rq->mem + rq->world);
    in.num_experts = rq->num_experts;
    in.expert_cost = rq->expert_cost;
    in.training = rq->is_training != 0;
    in.model = placement::Model{rq->moe_stages, rq->p2p_buffer_mb, rq->grad_buffer_mb};
    placement::Plan p;
    std::string why;
    if (!placement::make_plan(in, rq->rank, &p, &why)) return fail(KLEOS_E_ARG, "%s", why.c_str());
    *res = kleos_placement_result{};
    res->feasible = p.feasible ? 1 : 0;
    if (device_to_group) std::copy(p.device_to_group.begin(), p.device_to_group.end(), device_to_group);
    if (!p.feasible) return KLEOS_OK;
    res->group_size = (int32_t)p.group_ranks.size();
    res->group_rank = (int32_t)p.group_rank;
    res->local_experts = (int32_t)p.local_experts;
    res->expert_slots = (int32_t)p.expert_slots;
    res->widest_group = (int32_t)p.widest_group;
    // the data path of this library shards the experts evenly and contiguously over all ranks
    res->matches_data_path = 1;
    if ((int)p.group_ranks.size() != rq->world || rq->num_experts % rq->world) res->matches_data_path = 0;
    for (int e = 0; e < rq->num_experts && res->matches_data_path; ++e)
        if ((int)p.group_ranks[p.expert_to_member[e]] != e / (rq->num_experts / rq->world)) res->matches_data_path = 0;
    if (group_ranks) std::copy(p.group_ranks.begin(), p.group_ranks.end(), group_ranks);
    if (expert_to_member) std::copy(p.expert_to_member.begin(), p.expert_to_member.end(), expert_to_member);
    return KLEOS_OK;
}

int kleos_gate_stats(float* mean_prob, float* mean_count, float* loss) {
    if (!g.initialised) return fail(KLEOS_E_STATE, "not initialised");
    if (!g.gate_stats)
        return fail(KLEOS_E_STATE, "gate statistics are kept only when is_training = 1 (and num_experts > 1)");
    { const int src = sync_last_forward(); if (src) return src; }
    const int E = g.cfg.E;
    if (mean_prob) KLEOS_CUDA(cudaMemcpy(mean_prob, g.gate_stats, sizeof(float) * E, cudaMemcpyDeviceToHost));
    if (mean_count) KLEOS_CUDA(cudaMemcpy(mean_count, g.gate_stats + E, sizeof(float) * E, cudaMemcpyDeviceToHost));
    if (loss) KLEOS_CUDA(cudaMemcpy(loss, g.gate_stats + 2 * E, sizeof(float), cudaMemcpyDeviceToHost));
    return KLEOS_OK;
}

int kleos_debug_gemm_stats(long long* out, int max_values) {
    if (!g.initialised) return fail(KLEOS_E_STATE, "not initialised");
    if (!g.gemm_stats) return fail(KLEOS_E_STATE, "set KLEOS_GEMM_STATS=1 before kleos_initialize");
    const int n = 2 * g.sm_count * kStatSlots;
    if (!out || max_values < n) return fail(KLEOS_E_ARG, "need room for %d values", n);
    { const int src = sync_last_forward(); if (src) return src; }
    KLEOS_CUDA(cudaMemcpy(out, g.gemm_stats, sizeof(long long) * n, cudaMemcpyDeviceToHost));
    return n;
}

int kleos_debug_suppress_return_flag(int on) {
    if (!g.initialised) return fail(KLEOS_E_STATE, "not initialised");
    g.suppress_return_flag = on != 0;
    return KLEOS_OK;
}

int kleos_phase_times(float* ms, int n) {
    if (!ms || n < kPhases) return fail(KLEOS_E_ARG, "need room for %d floats", kPhases);
    for (int p = 0; p < kPhases; ++p) ms[p] = g.phase_ms[p];
    return KLEOS_OK;
}

int kleos_debug_tile_order(int local_experts, int lag, int32_t* phase, int32_t* expert) {
    if (local_experts < 1 || local_experts > flow::kMaxLocal || lag < 1 || lag > local_experts || !phase || !expert)
        return fail(KLEOS_E_ARG, "tile order: 1 <= lag <= local experts <= %d", flow::kMaxLocal);
    for (int s = 0; s < 2 * local_experts; ++s) {
        int ph, le;
        flow::segment_of(s, local_experts, lag, &ph, &le);
        phase[s] = ph;
        expert[s] = le;
    }
    return 2 * local_experts;
}

long long kleos_launch_count(void) { return g.initialised ? (long long)g.launches : (long long)KLEOS_E_STATE; }

int kleos_debug_flow_stalls(float* ms, int n) {
    if (!ms || n < flow::kStallSlots) return fail(KLEOS_E_ARG, "need room for %d floats", flow::kStallSlots);
    if (!g.initialised || !g.use_flow) return fail(KLEOS_E_STATE, "this layer does not run the persistent kernel");
    { const int src = sync_last_forward(); if (src) return src; }
    std::vector<long long> v((size_t)g.flow_grid * flow::kStallSlots);
    KLEOS_CUDA(cudaMemcpy(v.data(), g.flow_stalls, v.size() * sizeof(long long), cudaMemcpyDeviceToHost));
    for (int k = 0; k < flow::kStallSlots; ++k) {
        double sum = 0;
        int cnt = 0;
        for (int b = 0; b < g.flow_grid; ++b) {
            const long long c = v[(size_t)b * flow::kStallSlots + k];
            if (c > 0) {
                sum += (double)c;
                ++cnt;
            }
        }
        ms[k] = cnt ? (float)(sum / cnt / g.clock_khz) : 0.f;  // cycles / kHz = milliseconds
    }
    return KLEOS_OK;
}

int kleos_flow_timeline(float* ms, int n) {
    if (!ms || n < 12) return fail(KLEOS_E_ARG, "need room for at least 12 floats");
    if (!g.initialised || !g.use_flow) return fail(KLEOS_E_STATE, "this layer does not run the persistent kernel");
    for (int k = 0; k < n; ++k) ms[k] = k < flow::kStampSlots ? g.flow_ms[k] : 0.f;
    return KLEOS_OK;
}

int kleos_debug_flow_stamps(long long* ns, int capacity, int* blocks, int* per_block) {
    if (!blocks || !per_block) return fail(KLEOS_E_ARG, "null argument");
    if (!g.initialised || !g.use_flow) return fail(KLEOS_E_STATE, "this layer does not run the persistent kernel");
    *blocks = g.flow_grid;
    *per_block = flow::kStampSlots;
    if (!ns) return KLEOS_OK;  // sizes only
    if ((size_t)capacity < g.flow_raw.size()) return fail(KLEOS_E_ARG, "need room for %zu values", g.flow_raw.size());
    std::copy(g.flow_raw.begin(), g.flow_raw.end(), ns);
    return KLEOS_OK;
}

int kleos_finalize(void) {
    TraceRange trace("kleos_finalize");
    if (!g.initialised) return fail(KLEOS_E_STATE, "not initialised");
    cudaDeviceSynchronize();
    if (g.world > 1 && g.comm) {
        // nobody unmaps while a peer may still be storing into its cells (ranks of a dense
        // layer were never connected: they exchange nothing and have nothing to wait for)
        int token = g.rank, tokens[kMaxWorld];
        all_gather_bytes(&token, tokens, sizeof(int));
    }
    release_all();
    return KLEOS_OK;
}

}  // extern "C"

// Allocation-free router entry point (kleos_route_static) with its fixed device scratch array.
#include "route_static.cuh"
