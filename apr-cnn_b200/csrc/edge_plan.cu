// Cross-level part of the 3x3x3 input gradient without atomics.
//
// A tap of an output location p whose source is a coarser particle or a tree node ("cross-level edge")
// contributes W[tap]^T dO[p] to that source.  The reference scatters these with atomicAdd
// (pyapr/aprnet/cuda/src/conv333_gpu_backward.cu:184-192,417,643).  Here the edges of a level_delta are
// enumerated once (cached in the APR handle): edge ids run tap-major, then by location, so all edges of
// one (tap, level) form a contiguous range that shares one weight matrix.  The gradient is then
//   pass 1: an edge-list GEMM on the tensor cores (rows of dO gathered by edge, times W[tap]^T) that
//           writes one result row per edge, and
//   pass 2: a pull: every target sums the rows of its incoming edges in ascending edge order.
// Both passes are deterministic.  The edge rows go through a bounded workspace, a chunk of whole
// (tap, level) groups at a time.
#include "apr_device.cuh"
#include <cub/cub.cuh>
#include <algorithm>

namespace {

typedef long long ll;

struct LevelRanges { int n; ll begin[APRNET_MAX_LEVELS], end[APRNET_MAX_LEVELS]; };

// flag[f] = 1 when entry f = tap * N + p of the neighbour table is a cross-level source
__global__ void edge_flag_kernel(const int32_t* __restrict__ nbr, ll N, LevelRanges lr, int32_t* __restrict__ flag) {
    const ll f = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (f > 27 * N) return;
    int32_t v = 0;
    if (f < 27 * N) {
        const ll p = f % N;
        const int32_t q = nbr[f];
        if (q < APRNET_NONE) v = 1;
        else if (q >= 0) {
            ll lo = 0;
            for (int i = 0; i < lr.n; ++i) if (p >= lr.begin[i] && p < lr.end[i]) lo = lr.begin[i];
            v = q < lo;
        }
    }
    flag[f] = v;
}

__global__ void edge_emit_kernel(const int32_t* __restrict__ nbr, ll N, const int32_t* __restrict__ scan,
                                 int32_t* __restrict__ src, int32_t* __restrict__ tgt, int32_t* __restrict__ count) {
    const ll f = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (f >= 27 * N) return;
    const int32_t e = scan[f];
    if (scan[f + 1] == e) return;
    const int32_t q = nbr[f];
    const int32_t t = q >= 0 ? q : (int32_t) (N + aprnet_dec_tree(q));
    src[e] = (int32_t) (f % N);
    tgt[e] = t;
    atomicAdd(count + t, 1);
}

__global__ void edge_fill_kernel(const int32_t* __restrict__ tgt, ll E, int32_t* __restrict__ cursor, int32_t* __restrict__ tgt_edge) {
    const ll e = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= E) return;
    tgt_edge[atomicAdd(cursor + tgt[e], 1)] = (int32_t) e;
}

// ascending edge order inside every target's list (the fill order above depends on scheduling)
__global__ void edge_sort_kernel(const int32_t* __restrict__ ptr, ll n_targets, int32_t* __restrict__ tgt_edge, int32_t* __restrict__ is_active) {
    const ll t = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (t > n_targets) return;
    if (t == n_targets) { is_active[t] = 0; return; }
    const int32_t b = ptr[t], e = ptr[t + 1];
    is_active[t] = e > b;
    for (int32_t i = b + 1; i < e; ++i) {
        const int32_t v = tgt_edge[i];
        int32_t j = i - 1;
        while (j >= b && tgt_edge[j] > v) { tgt_edge[j + 1] = tgt_edge[j]; --j; }
        tgt_edge[j + 1] = v;
    }
}

__global__ void edge_compact_active_kernel(const int32_t* __restrict__ pos, ll n_targets, int32_t* __restrict__ active) {
    const ll t = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_targets) return;
    if (pos[t + 1] != pos[t]) active[pos[t]] = (int32_t) t;
}

// pass 2: thread = (active target, block of 16 channels); sums the rows of the incoming edges that lie in
// the current chunk [e0, e1) and adds them to the gradient of the particle / tree node.
__global__ void edge_pull_kernel(const int32_t* __restrict__ active, ll n_active, const int32_t* __restrict__ ptr,
                                 const int32_t* __restrict__ tgt_edge, ll e0, ll e1, const float* __restrict__ rows, int row_pad,
                                 float* __restrict__ gin, ll ld_in, float* __restrict__ gtree, ll ld_tree, ll N, int cin) {
    const ll a = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (a >= n_active) return;
    const int t = active[a];
    int b = ptr[t];
    const int e = ptr[t + 1];
    {   // first incoming edge >= e0
        int hi = e;
        while (b < hi) { const int m = (b + hi) >> 1; if (tgt_edge[m] < e0) b = m + 1; else hi = m; }
    }
    if (b >= e || tgt_edge[b] >= e1) return;
    const int c0 = blockIdx.y * 16;
    float acc[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) acc[i] = 0.f;
    for (; b < e; ++b) {
        const ll ed = tgt_edge[b];
        if (ed >= e1) break;
        const float4* r = reinterpret_cast<const float4*>(rows + (ed - e0) * row_pad + c0);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 v = r[i];
            acc[4 * i] += v.x; acc[4 * i + 1] += v.y; acc[4 * i + 2] += v.z; acc[4 * i + 3] += v.w;
        }
    }
    float* dst = t < N ? gin + t : gtree + (t - N);
    const ll ld = t < N ? ld_in : ld_tree;
#pragma unroll
    for (int i = 0; i < 16; ++i)
        if (c0 + i < cin) dst[(ll) (c0 + i) * ld] += acc[i];
}

template<typename T>
int dev_alloc(T** p, size_t n, long long* bytes) {
    APRNET_CUDA_CHECK(cudaMalloc((void**) p, std::max<size_t>(n, 1) * sizeof(T)));
    if (bytes) *bytes += (long long) (std::max<size_t>(n, 1) * sizeof(T));
    return APRNET_OK;
}

} // namespace

void aprnet_free_edge_plan(EdgePlan& ep) {
    cudaFree(ep.src); cudaFree(ep.tgt_ptr); cudaFree(ep.tgt_edge); cudaFree(ep.active); cudaFree(ep.groups_dev);
    ep = EdgePlan();
}

static int build_edge_plan(aprnet_apr* a, int dl, const AprPlan* plan, EdgePlan& ep, cudaStream_t st) {
    const ll N = plan->n, T = plan->tree_size, NT = N + T;
    const ll F = 27 * N;
    if (F + 1 >= (1ll << 31)) { aprnet_set_error("edge plan: neighbour table too large for 32-bit edge ids"); return APRNET_ERR_UNSUPPORTED; }
    const std::vector<Segment> segs = aprnet_segments(a, dl, 1, false);
    LevelRanges lr;
    lr.n = (int) segs.size();
    for (int i = 0; i < lr.n; ++i) { lr.begin[i] = segs[i].begin; lr.end[i] = segs[i].end; }

    int32_t *scan = nullptr, *tgt = nullptr, *count = nullptr;
    void* temp = nullptr;
    int rc = APRNET_OK;
    auto cleanup = [&]() { cudaFree(scan); cudaFree(tgt); cudaFree(count); cudaFree(temp); };
#define EP_CHECK(expr) do { cudaError_t _e = (expr); if (_e != cudaSuccess) { aprnet_set_error("%s failed: %s", #expr, cudaGetErrorString(_e)); cleanup(); return APRNET_ERR_CUDA; } } while (0)

    EP_CHECK(cudaMalloc((void**) &scan, (size_t) (F + 1) * sizeof(int32_t)));
    edge_flag_kernel<<<aprnet_ceil_div(F + 1, 256), 256, 0, st>>>(plan->nbr, N, lr, scan);
    size_t temp_bytes = 0, temp2 = 0;
    EP_CHECK(cub::DeviceScan::ExclusiveSum(nullptr, temp_bytes, scan, scan, (int) (F + 1), st));
    EP_CHECK(cub::DeviceScan::ExclusiveSum(nullptr, temp2, scan, scan, (int) (NT + 1), st));
    temp_bytes = std::max(temp_bytes, temp2);
    EP_CHECK(cudaMalloc(&temp, std::max<size_t>(temp_bytes, 1)));
    EP_CHECK(cub::DeviceScan::ExclusiveSum(temp, temp_bytes, scan, scan, (int) (F + 1), st));

    // group boundaries: edge id at the start of every (tap, level) range
    std::vector<int32_t> bounds((size_t) 27 * lr.n * 2);
    int32_t total = 0;
    for (int tap = 0; tap < 27; ++tap)
        for (int i = 0; i < lr.n; ++i) {
            EP_CHECK(cudaMemcpyAsync(&bounds[(size_t) (tap * lr.n + i) * 2], scan + tap * N + lr.begin[i], sizeof(int32_t), cudaMemcpyDeviceToHost, st));
            EP_CHECK(cudaMemcpyAsync(&bounds[(size_t) (tap * lr.n + i) * 2 + 1], scan + tap * N + lr.end[i], sizeof(int32_t), cudaMemcpyDeviceToHost, st));
        }
    EP_CHECK(cudaMemcpyAsync(&total, scan + F, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    EP_CHECK(cudaStreamSynchronize(st));
    ep.n_edges = total; ep.n_targets = NT;
    ep.groups.clear();
    for (int tap = 0; tap < 27; ++tap)
        for (int i = 0; i < lr.n; ++i) {
            EdgeGroup g;
            g.begin = bounds[(size_t) (tap * lr.n + i) * 2]; g.end = bounds[(size_t) (tap * lr.n + i) * 2 + 1];
            g.tap = tap; g.level = segs[i].level;
            if (g.end > g.begin) ep.groups.push_back(g);
        }

    const size_t E = (size_t) total;
    if ((rc = dev_alloc(&ep.src, E, &a->device_bytes)) || (rc = dev_alloc(&ep.tgt_edge, E, &a->device_bytes)) ||
        (rc = dev_alloc(&ep.tgt_ptr, (size_t) NT + 1, &a->device_bytes))) { cleanup(); return rc; }
    EP_CHECK(cudaMalloc((void**) &tgt, std::max<size_t>(E, 1) * sizeof(int32_t)));
    EP_CHECK(cudaMalloc((void**) &count, (size_t) (NT + 1) * sizeof(int32_t)));
    EP_CHECK(cudaMemsetAsync(count, 0, (size_t) (NT + 1) * sizeof(int32_t), st));
    edge_emit_kernel<<<aprnet_ceil_div(F, 256), 256, 0, st>>>(plan->nbr, N, scan, ep.src, tgt, count);
    EP_CHECK(cub::DeviceScan::ExclusiveSum(temp, temp_bytes, count, ep.tgt_ptr, (int) (NT + 1), st));
    EP_CHECK(cudaMemcpyAsync(count, ep.tgt_ptr, (size_t) (NT + 1) * sizeof(int32_t), cudaMemcpyDeviceToDevice, st));   // cursors
    if (E) edge_fill_kernel<<<aprnet_ceil_div((ll) E, 256), 256, 0, st>>>(tgt, (ll) E, count, ep.tgt_edge);
    // sort the lists, flag active targets (flags reuse `count`), compact them
    edge_sort_kernel<<<aprnet_ceil_div(NT + 1, 128), 128, 0, st>>>(ep.tgt_ptr, NT, ep.tgt_edge, count);
    EP_CHECK(cub::DeviceScan::ExclusiveSum(temp, temp_bytes, count, count, (int) (NT + 1), st));
    int32_t n_active = 0;
    EP_CHECK(cudaMemcpyAsync(&n_active, count + NT, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    EP_CHECK(cudaStreamSynchronize(st));
    ep.n_active = n_active;
    if ((rc = dev_alloc(&ep.active, (size_t) n_active, &a->device_bytes))) { cleanup(); return rc; }
    if (NT) edge_compact_active_kernel<<<aprnet_ceil_div(NT, 256), 256, 0, st>>>(count, NT, ep.active);
    EP_CHECK(cudaGetLastError());
    EP_CHECK(cudaStreamSynchronize(st));
#undef EP_CHECK
    cleanup();
    return APRNET_OK;
}

EdgePlan* aprnet_get_edge_plan(aprnet_apr* a, int dl, cudaStream_t st) {
    auto it = a->edge_plans.find(dl);
    if (it != a->edge_plans.end()) return &it->second;
    const AprPlan* plan = aprnet_get_plan(a, dl, st);
    if (!plan) return nullptr;
    EdgePlan ep;
    if (build_edge_plan(a, dl, plan, ep, st) != APRNET_OK) { aprnet_free_edge_plan(ep); return nullptr; }
    auto res = a->edge_plans.emplace(dl, ep);
    return &res.first->second;
}

// Builds (once; cached) the cross-level edge lists of a level delta.  Allocates; call it up front.
extern "C" int aprnet_edge_plan_build(aprnet_apr* a, int dl, void* stream) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl), "bad handle or level_delta");
    return aprnet_get_edge_plan(a, dl, (cudaStream_t) stream) ? APRNET_OK : APRNET_ERR_CUDA;
}

extern "C" int64_t aprnet_edge_workspace_bytes(const aprnet_apr* a, int dl, int cin) {
    if (!a || !a->valid_dl(dl)) return -1;
    const ll cap = 8ll << 30;     // bounds the edge-row workspace; larger = fewer pull passes over the target list
    const ll all = 27 * a->number_parts(dl) * (ll) aprnet_tc_pad(cin) * 4;
    return (int64_t) std::max<ll>(256, std::min(cap, all));
}

// Cross-level part of the input gradient (added to grad_input / grad_tree, which the call zero-fills)
// followed by the tree adjoint.  packed_grad_output_rows: channels-last bf16 dO rows with a zero row at
// index N; weights fp32 (slots, Cout, Cin, 27); wp_ws: space for the packed transposed weights;
// edge_ws: aprnet_edge_workspace_bytes() bytes.
extern "C" int aprnet_conv333_backward_input_cross_level_tc(aprnet_apr* a, int dl, int cin, int cout, int slots,
                                                            const void* grows, int gpad, const float* w, float* gin,
                                                            int64_t ld_in, float* gtree, int64_t ld_tree, void* wp_ws,
                                                            void* edge_ws, int64_t edge_ws_bytes, void* stream) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && cin > 0 && cout > 0 && slots > 0 && grows && w && gin && gtree && wp_ws && edge_ws, "bad argument");
    cudaStream_t st = (cudaStream_t) stream;
    EdgePlan* ep = aprnet_get_edge_plan(a, dl, st);
    if (!ep) return APRNET_ERR_CUDA;
    const ll N = a->number_parts(dl), ts = a->tree_size(dl);
    if (ts > 0) APRNET_CUDA_CHECK(cudaMemset2DAsync(gtree, (size_t) ld_tree * sizeof(float), 0, (size_t) ts * sizeof(float), (size_t) cin, st));
    const int row_pad = aprnet_tc_pad(cin);
    const ll cap_edges = edge_ws_bytes / ((ll) row_pad * 4);
    int rc = aprnet_tc_pack_weights(w, slots, cin, cout, 2, wp_ws, st);
    if (rc) return rc;
    const int ng = (int) ep->groups.size();
    int g0 = 0;
    while (g0 < ng) {
        int g1 = g0;
        ll cnt = 0;
        while (g1 < ng && cnt + (ep->groups[g1].end - ep->groups[g1].begin) <= cap_edges) { cnt += ep->groups[g1].end - ep->groups[g1].begin; ++g1; }
        if (g1 == g0) { aprnet_set_error("edge workspace too small for one (tap, level) group of %lld edges", (ll) (ep->groups[g0].end - ep->groups[g0].begin)); return APRNET_ERR_ARG; }
        rc = aprnet_tc_edge_gemm(a, dl, cin, cout, slots, grows, gpad, N, wp_ws, ep, g0, g1, (float*) edge_ws, row_pad, st);
        if (rc) return rc;
        const ll e0 = ep->groups[g0].begin, e1 = ep->groups[g1 - 1].end;
        if (ep->n_active > 0) {
            dim3 grid((unsigned) aprnet_ceil_div(ep->n_active, 128), (unsigned) (row_pad / 16));
            { AprnetProfScope _prof("edge_pull", st);
            edge_pull_kernel<<<grid, 128, 0, st>>>(ep->active, ep->n_active, ep->tgt_ptr, ep->tgt_edge, e0, e1, (const float*) edge_ws, row_pad,
                                                   gin, ld_in, gtree, ld_tree, N, cin);
            }
            APRNET_LAUNCH_CHECK();
        }
        g0 = g1;
    }
    return aprnet_fill_tree_mean_backward(a, dl, APRNET_F32, cin, gin, ld_in, gtree, ld_tree, st);
}
