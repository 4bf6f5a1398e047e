// Internal definitions shared by the CUDA translation units of libaprnet_b200.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cstdarg>
#include <string>
#include <vector>
#include <map>
#include <cuda_runtime.h>
#include "../../include/aprnet_b200.h"

#define APRNET_MAX_LEVELS 20

// Encoding of neighbour / child table entries:
//   v >= 0 : index into the feature vector (APR particle, or upgraded tree node stored behind them)
//   v == -1: nothing there (outside the domain) -> value 0
//   v <= -2: tree node t = -2 - v (value comes from the tree scratch)
#define APRNET_NONE (-1)
__host__ __device__ inline int32_t aprnet_enc_tree(long long t) { return (int32_t) (-2 - t); }
__host__ __device__ inline long long aprnet_dec_tree(int32_t v) { return -2 - (long long) v; }

// Per-level geometry and index ranges; passed to kernels by value.
struct LevelMeta {
    int level_min, level_max;                    // particle levels; the tree spans level_min-1 .. level_max-1
    int z_num[APRNET_MAX_LEVELS], x_num[APRNET_MAX_LEVELS], y_num[APRNET_MAX_LEVELS];
    long long row_off[APRNET_MAX_LEVELS + 1];    // first particle row of each level
    long long trow_off[APRNET_MAX_LEVELS + 1];   // first tree row of each level
    long long lvl_begin[APRNET_MAX_LEVELS + 1];  // first particle index of each level ([l+1] = end of l)
    long long tlvl_begin[APRNET_MAX_LEVELS + 1]; // first tree node index of each level
};

struct AprPlan {                 // cached per level_delta
    int level_delta = 0;
    long long n = 0;             // number of output locations (= number_parts)
    long long tree_size = 0;
    int32_t* nbr = nullptr;      // [27][n]
};

// Cross-level edges of one level_delta: every (output location p, tap) whose source ("target" of the
// gradient) is a coarser particle or a tree node.  Targets are numbered as particle index, or
// N + tree index.  The edges of one (target, tap) form a "virtual row": their dO rows are summed before
// the contraction, because they all meet the same weight matrix.  Virtual rows are numbered by
// ascending target, then tap; vsrc[vstart[v] .. vstart[v + 1]) lists the locations p of row v in
// ascending order.  active[] lists the targets that have at least one edge (ascending), vnbr[tap][a] is
// the virtual row of (active[a], tap) or -1.
struct ActiveSeg { long long begin, end; int location_level; };     // range of active[] whose edges come from one level
struct EdgePlan {
    long long n_edges = 0, n_targets = 0, n_active = 0, n_vrows = 0;
    int32_t* vsrc = nullptr;       // [n_edges]
    int32_t* vstart = nullptr;     // [n_vrows + 1]
    int32_t* active = nullptr;     // [n_active]
    int32_t* vnbr = nullptr;       // [27][n_active]
    std::vector<ActiveSeg> segs;   // by level, in active[] order
    // coarse map for splitting the work when the virtual rows do not fit the workspace: chunk k starts at
    // active index chunk_a[k] and virtual row chunk_v[k]; chunks hold about VROW_GRANULE rows
    std::vector<long long> chunk_a, chunk_v;
};

struct aprnet_apr {
    int device = 0;
    LevelMeta meta;
    long long n_particles = 0, n_tree = 0, n_rows = 0, n_tree_rows = 0;
    long long* row_ptr = nullptr;        // device
    uint16_t* y = nullptr;
    long long* tree_row_ptr = nullptr;
    uint16_t* tree_y = nullptr;
    int32_t* child = nullptr;            // [8][n_tree]
    float* tree_scale = nullptr;         // [n_tree] weight of each child in its parent's mean
    std::map<int, AprPlan> plans;
    std::map<int, EdgePlan> edge_plans;
    // parent tree node of every tree node (-1: none) and, per level delta, of every feature location (particle or
    // upgraded node); built on first use by the tree-mean adjoint (aprnet_node_parent_table / aprnet_loc_parent_table)
    mutable int32_t* node_parent = nullptr;
    mutable std::map<int, int32_t*> loc_parent;
    mutable long long device_bytes = 0;

    int cml(int dl) const { return meta.level_max - dl; }
    long long number_parts(int dl) const {
        const int c = cml(dl);
        long long n = meta.lvl_begin[c + 1];
        if (c <= meta.level_max - 1) n += meta.tlvl_begin[c + 1] - meta.tlvl_begin[c];
        return n;
    }
    long long tree_size(int dl) const { return meta.tlvl_begin[cml(dl)]; }   // nodes of levels <= cml-1
    long long tree_offset(int level) const { return meta.lvl_begin[level + 1] - meta.tlvl_begin[level]; }
    bool valid_dl(int dl) const { return dl >= 0 && cml(dl) >= meta.level_min; }
};

void aprnet_set_error(const char* fmt, ...);
int aprnet_check_device(const aprnet_apr* a);      // APRNET_OK when the current device is the handle's device

#define APRNET_CUDA_CHECK(expr)                                                                     \
    do {                                                                                            \
        cudaError_t _e = (expr);                                                                    \
        if (_e != cudaSuccess) {                                                                    \
            aprnet_set_error("%s failed at %s:%d: %s", #expr, __FILE__, __LINE__, cudaGetErrorString(_e)); \
            return APRNET_ERR_CUDA;                                                                 \
        }                                                                                           \
    } while (0)

#define APRNET_LAUNCH_CHECK() APRNET_CUDA_CHECK(cudaGetLastError())

#define APRNET_ARG_CHECK(cond, msg)                                                                 \
    do { if (!(cond)) { aprnet_set_error("%s: %s", __func__, msg); return APRNET_ERR_ARG; } } while (0)

#define APRNET_DEVICE_CHECK(a)                                                                      \
    do { const int _rc = aprnet_check_device(a); if (_rc != APRNET_OK) return _rc; } while (0)

inline int aprnet_ceil_div(long long a, long long b) { return (int) ((a + b - 1) / b); }

// A contiguous range of output locations that shares one stencil slot.
struct Segment { long long begin, end; int slot; int level; };
// Segments of level_delta dl for a filter bank with `num_slots` slots: level l -> slot
// min(cml - l, num_slots - 1); the upgraded tree nodes ride with the level-cml particles.
// With merge=true, consecutive levels that share a slot are fused into one range (1x1x1 conv).
std::vector<Segment> aprnet_segments(const aprnet_apr* apr, int dl, int num_slots, bool merge);

const AprPlan* aprnet_get_plan(aprnet_apr* apr, int dl, cudaStream_t stream);
const int32_t* aprnet_node_parent_table(const aprnet_apr* apr, cudaStream_t stream);            // nullptr on failure
const int32_t* aprnet_loc_parent_table(const aprnet_apr* apr, int dl, cudaStream_t stream);     // nullptr on failure

// Optional per-kernel timing (aprnet_profile_enable): brackets a launch site with two CUDA events on
// the launching stream.  Costs nothing when profiling is off.
struct AprnetProfScope {
    int slot;
    cudaStream_t stream;
    AprnetProfScope(const char* name, cudaStream_t st);
    ~AprnetProfScope();
};

// tensor-core helpers shared between translation units (conv333_tc.cu / conv333_tc_dw.cu)
int* aprnet_tc_error_flag_device();
extern "C" int aprnet_conv333_backward_weights_tc(aprnet_apr* a, int dl, int cin, int cout, int slots, const void* xrows, int xpad,
                                                  const void* grows, int gpad, float* gw, float* partial, void* stream);
extern "C" int64_t aprnet_conv333_tc_dw_partial_elems(int cin, int cout);
extern "C" int aprnet_conv333_backward_input_cross_level(aprnet_apr* a, int dl, int dtype, int cin, int cout, int slots,
                                                         const void* gout, int64_t ld_out, const void* w, void* gin,
                                                         int64_t ld_in, void* gtree, int64_t ld_tree, void* stream);

EdgePlan* aprnet_get_edge_plan(aprnet_apr* apr, int dl, cudaStream_t stream);
void aprnet_free_edge_plan(EdgePlan& ep);
// gather GEMM over the active targets [a0, a1) of an edge plan: grad[target] += sum over taps of
// W[slot][:, :, tap]^T times virtual row vnbr[tap][a] (rows: bf16 [.. ][gpad], row index relative to `vrows`)
int aprnet_tc_gather_targets(aprnet_apr* a, int dl, int cin, int cout, int slots, const void* vrows, int gpad, long long zero_row,
                             const void* wp_packed, const EdgePlan* ep, long long a0, long long a1,
                             float* gin, long long ld_in, float* gtree, long long ld_tree, cudaStream_t st);
// CUDA-core fp32 kernels for Cin <= 4 (conv333_small.cu), used by the tensor-core drivers for such layers:
// vals = channel-major staging buffer [cin][N + T + 1] (particles, tree means, zero)
bool aprnet_small_cin(int cin);
int aprnet_small_stage(const float* x, long long ld_x, long long n, const float* tree, long long ld_tree, long long t, int cin, float* vals, cudaStream_t st);
int aprnet_small_forward(aprnet_apr* a, int dl, int cin, int cout, int slots, const float* vals, const float* w, float* out, long long ld_out, cudaStream_t st);
int aprnet_small_backward_weights(aprnet_apr* a, int dl, int cin, int cout, int slots, const float* vals, const float* gout, long long ld_out,
                                  float* gw, float* partial, cudaStream_t st);
int aprnet_tc_pack_weights(const float* w, int slots, int cin, int cout, int mode, void* wp, cudaStream_t st);
size_t aprnet_tc_weight_bytes(int k_dim, int n_dim, int slots);
size_t aprnet_tc_rows_bytes(long long rows, int channels);
int aprnet_tc_pad(int channels);
extern "C" int64_t aprnet_edge_workspace_bytes(const aprnet_apr* a, int dl, int cout);
extern "C" int aprnet_conv333_backward_input_cross_level_tc(aprnet_apr* a, int dl, int cin, int cout, int slots,
                                                            const void* grows, int gpad, const float* w, float* gin,
                                                            int64_t ld_in, float* gtree, int64_t ld_tree, void* wp_ws,
                                                            void* edge_ws, int64_t edge_ws_bytes, void* stream);
// same, with the final tree adjoint (grad_tree folded into grad_input) optional
int aprnet_cross_level_tc(aprnet_apr* a, int dl, int cin, int cout, int slots, const void* grows, int gpad, const float* w, float* gin,
                          long long ld_in, float* gtree, long long ld_tree, void* wp_ws, void* edge_ws, long long edge_ws_bytes, void* stream,
                          bool tree_adjoint);
