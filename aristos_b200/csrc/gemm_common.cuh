// Arguments and tile decoding shared by the expert-FFN GEMM kernels.
//
// The two GEMMs of the expert FFN (reference os/processor/processor.cuh:706-741):
//   mode 0 (GEMM1): y1 = act(x * W1[e]^T + b1[e]), rounded to the element type, kept in this
//                   rank's memory, row space identical to the dispatched cells;
//   mode 1 (GEMM2): y2 = y1 * W2[e]^T + b2[e], rounded, stored straight into the SOURCE
//                   rank's result cell for (global expert, slot) over NVLink, as the
//                   reference's peer path does (os/packet.cuh:338-340).
#pragma once

#include "common.cuh"
#include "transport.cuh"

namespace kleos {

constexpr int kStatSlots = 12;  // per-block stall counters (see kleos_debug_gemm_stats)

struct GemmArgs {
    const PanelEntry* panels;
    const int* le_start;  // [nLx+1]
    const void* A;        // [cells*pEC][Kd] rows, K contiguous
    const void* B;        // [nLx*N][Kd] weight rows, K contiguous
    const void* bias;     // [nLx*N]
    void* y1;             // mode 0 output [cells*pEC][N]
    PeerTable peers;      // mode 1 output
    ArenaLayout lay;
    ReturnFlagArgs ret;   // mode 1: flags raised by the last block
    DeviceStatus* status;
    long long* stats;     // optional [grid][kStatSlots] per-role stall counters (cycles), or null
    long long wait_cycles;
    int N, Kd, mode, hidden_act;
    int nLx, pEC, rank, elem_bytes;
    int le_begin, le_end;  // local experts this launch works on
    uint32_t epoch;
};

struct TileCoord {
    int panel, nt, le;
};

// Tiles are ordered: local expert, then N tile, then panel, so that consecutive tiles (which
// persistent blocks pick up at about the same time) read the same weight tile from L2.
__device__ __forceinline__ bool decode_tile(int t, const int* le_start, int le_begin, int le_end,
                                            int NT, TileCoord* c) {
    for (int le = le_begin; le < le_end; ++le) {
        const int p0 = le_start[le], np = le_start[le + 1] - p0;
        const int tiles = np * NT;
        if (t < tiles) {
            c->le = le;
            c->nt = t / np;
            c->panel = p0 + (t - c->nt * np);
            return true;
        }
        t -= tiles;
    }
    return false;
}

// Address of output element (row r of the panel, column n) for either mode.
template <typename T>
__device__ __forceinline__ T* out_ptr(const GemmArgs& g, const PanelEntry& p, int r, int n) {
    if (g.mode == 0)
        return static_cast<T*>(g.y1) + (size_t)(p.row_base + r) * g.N + n;
    const int cell = p.src * g.nLx + p.le;
    const int r0 = p.row_base - cell * g.pEC;
    const size_t e_global = (size_t)g.rank * g.nLx + p.le;
    return reinterpret_cast<T*>(g.peers.arena[p.src] + g.lay.ycell) +
           (e_global * g.pEC + r0 + r) * g.N + n;
}

}  // namespace kleos
