// Cross-level part of the 3x3x3 input gradient without atomics.
//
// A tap of an output location p whose source is a coarser particle or a tree node ("cross-level edge")
// contributes W[tap]^T dO[p] to that source.  The reference scatters these with atomicAdd
// (pyapr/aprnet/cuda/src/conv333_gpu_backward.cu:184-192,417,643).  Here the edges of a level_delta are
// enumerated once (cached in the APR handle) and grouped by (target, tap): all edges of one group meet
// the same weight matrix (their locations lie on one level), so their dO rows are summed first
// ("virtual row", pass 1: a segmented sum in ascending location order) and the contraction becomes an
// ordinary 27-tap gather GEMM over the targets that have edges (pass 2, on the tensor cores), whose
// result is added to the gradient of the particle / tree node by exactly one thread.  Both passes are
// deterministic, and the work is proportional to the number of (target, tap) groups, not edges.
#include "apr_device.cuh"
#include <cub/cub.cuh>
#include <cuda_bf16.h>
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

struct TapBegin { int32_t b[28]; };      // first edge id of every tap (edge ids are tap-major)

// virtual rows of one active target = runs of equal tap in its ascending edge list
__global__ void vrow_count_kernel(const int32_t* __restrict__ active, ll n_active, const int32_t* __restrict__ ptr,
                                  const int32_t* __restrict__ tgt_edge, TapBegin tb, int32_t* __restrict__ nruns) {
    const ll a = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (a > n_active) return;
    int runs = 0;
    if (a < n_active) {
        const int t = active[a];
        int cur = -1, tap = 0;
        for (int i = ptr[t]; i < ptr[t + 1]; ++i) {
            const int32_t e = tgt_edge[i];
            while (e >= tb.b[tap + 1]) ++tap;
            if (tap != cur) { ++runs; cur = tap; }
        }
    }
    nruns[a] = runs;
}

__global__ void vrow_fill_kernel(const int32_t* __restrict__ active, ll n_active, const int32_t* __restrict__ ptr,
                                 const int32_t* __restrict__ tgt_edge, const int32_t* __restrict__ src, TapBegin tb,
                                 const int32_t* __restrict__ vfirst, ll n_edges, int32_t* __restrict__ vstart,
                                 int32_t* __restrict__ vnbr, int32_t* __restrict__ vsrc) {
    const ll a = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (a >= n_active) return;
    if (a == 0) vstart[vfirst[n_active]] = (int32_t) n_edges;
    const int t = active[a];
    int cur = -1, tap = 0;
    int32_t v = vfirst[a] - 1;
    for (int i = ptr[t]; i < ptr[t + 1]; ++i) {
        const int32_t e = tgt_edge[i];
        while (e >= tb.b[tap + 1]) ++tap;
        if (tap != cur) { cur = tap; ++v; vstart[v] = i; vnbr[(ll) tap * n_active + a] = v; }
        vsrc[i] = src[e];
    }
}

// out[k] = first index i of sorted[0, n) with sorted[i] >= key[k]
__global__ void lower_bound_kernel(const int32_t* __restrict__ sorted, ll n, const ll* __restrict__ key, int nkeys, ll* __restrict__ out) {
    const int k = blockIdx.x * blockDim.x + threadIdx.x;
    if (k >= nkeys) return;
    ll lo = 0, hi = n;
    while (lo < hi) { const ll m = (lo + hi) >> 1; if ((ll) sorted[m] < key[k]) lo = m + 1; else hi = m; }
    out[k] = lo;
}

// pass 1: thread = (VPT consecutive virtual rows, 8-channel chunk); sums the dO rows of each row's locations in
// ascending order (fp32) and writes the bf16 row 1 + v - v0 of the workspace (row 0 is the zero row).  The three
// dependent accesses (row starts -> source locations -> dO rows) are each requested for all VPT rows and up to four
// locations per row before any is used (runs are 1-4 locations long; longer ones continue in a loop).
constexpr int VROW_VPT = 2;          // measured: 2 rows per thread 20 % faster than 1, 4 slower (registers)

template<int VPT>
__global__ void __launch_bounds__(256) vrow_reduce_kernel(const int32_t* __restrict__ vstart, const int32_t* __restrict__ vsrc, ll v0, ll v1,
                                                          const __nv_bfloat16* __restrict__ grows, int gpad, __nv_bfloat16* __restrict__ out) {
    const int nch = gpad >> 3;
    const ll e = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    const ll vb = v0 + (e / nch) * VPT;
    if (vb >= v1) return;
    const int c = (int) (e % nch);
    int s[VPT + 1];
#pragma unroll
    for (int u = 0; u <= VPT; ++u) s[u] = __ldg(vstart + min(vb + u, v1));
    int32_t src[VPT][4];
#pragma unroll
    for (int u = 0; u < VPT; ++u)
#pragma unroll
        for (int k = 0; k < 4; ++k) src[u][k] = s[u] + k < s[u + 1] ? __ldg(vsrc + s[u] + k) : -1;
    uint4 q[VPT][4];
#pragma unroll
    for (int u = 0; u < VPT; ++u)
#pragma unroll
        for (int k = 0; k < 4; ++k)
            q[u][k] = src[u][k] >= 0 ? __ldg(reinterpret_cast<const uint4*>(grows + (ll) src[u][k] * gpad + c * 8)) : make_uint4(0, 0, 0, 0);
#pragma unroll
    for (int u = 0; u < VPT; ++u) {
        if (vb + u >= v1) break;
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        auto add = [&](const uint4& r) {
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
            for (int k = 0; k < 4; ++k) { const float2 f = __bfloat1622float2(h[k]); acc[2 * k] += f.x; acc[2 * k + 1] += f.y; }
        };
#pragma unroll
        for (int k = 0; k < 4; ++k) add(q[u][k]);              // ascending location order (absent entries add zeros)
        for (int i = s[u] + 4; i < s[u + 1]; ++i)
            add(__ldg(reinterpret_cast<const uint4*>(grows + (ll) __ldg(vsrc + i) * gpad + c * 8)));
        __nv_bfloat162 o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) o[k] = __floats2bfloat162_rn(acc[2 * k], acc[2 * k + 1]);
        *reinterpret_cast<uint4*>(out + (1 + vb + u - v0) * gpad + c * 8) = *reinterpret_cast<const uint4*>(o);
    }
}

constexpr ll VROW_GRANULE = 4ll << 20;      // virtual rows per entry of the chunk map

template<typename T>
int dev_alloc(T** p, size_t n, long long* bytes) {
    APRNET_CUDA_CHECK(cudaMalloc((void**) p, std::max<size_t>(n, 1) * sizeof(T)));
    if (bytes) *bytes += (long long) (std::max<size_t>(n, 1) * sizeof(T));
    return APRNET_OK;
}

} // namespace

void aprnet_free_edge_plan(EdgePlan& ep) {
    cudaFree(ep.vsrc); cudaFree(ep.vstart); cudaFree(ep.active); cudaFree(ep.vnbr);
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

    // temporaries: flags / scan, per-edge source and target, per-target lists
    int32_t *scan = nullptr, *src = nullptr, *tgt = nullptr, *count = nullptr, *tgt_ptr = nullptr, *tgt_edge = nullptr, *vfirst = nullptr;
    ll *keys = nullptr, *found = nullptr;
    void* temp = nullptr;
    int rc = APRNET_OK;
    auto cleanup = [&]() { cudaFree(scan); cudaFree(src); cudaFree(tgt); cudaFree(count); cudaFree(tgt_ptr); cudaFree(tgt_edge);
                           cudaFree(vfirst); cudaFree(keys); cudaFree(found); cudaFree(temp); };
#define EP_CHECK(expr) do { cudaError_t _e = (expr); if (_e != cudaSuccess) { aprnet_set_error("%s failed: %s", #expr, cudaGetErrorString(_e)); cleanup(); return APRNET_ERR_CUDA; } } while (0)

    EP_CHECK(cudaMalloc((void**) &scan, (size_t) (F + 1) * sizeof(int32_t)));
    edge_flag_kernel<<<aprnet_ceil_div(F + 1, 256), 256, 0, st>>>(plan->nbr, N, lr, scan);
    size_t temp_bytes = 0, temp2 = 0;
    EP_CHECK(cub::DeviceScan::ExclusiveSum(nullptr, temp_bytes, scan, scan, (int) (F + 1), st));
    EP_CHECK(cub::DeviceScan::ExclusiveSum(nullptr, temp2, scan, scan, (int) (NT + 2), st));
    temp_bytes = std::max(temp_bytes, temp2);
    EP_CHECK(cudaMalloc(&temp, std::max<size_t>(temp_bytes, 1)));
    EP_CHECK(cub::DeviceScan::ExclusiveSum(temp, temp_bytes, scan, scan, (int) (F + 1), st));

    // first edge id of every tap
    TapBegin tb;
    for (int tap = 0; tap <= 27; ++tap)
        EP_CHECK(cudaMemcpyAsync(&tb.b[tap], scan + (ll) tap * N, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    EP_CHECK(cudaStreamSynchronize(st));
    const ll E = tb.b[27];
    ep.n_edges = E; ep.n_targets = NT;

    // per-edge source and target, per-target ascending edge lists, active targets
    EP_CHECK(cudaMalloc((void**) &src, std::max<size_t>(E, 1) * sizeof(int32_t)));
    EP_CHECK(cudaMalloc((void**) &tgt, std::max<size_t>(E, 1) * sizeof(int32_t)));
    EP_CHECK(cudaMalloc((void**) &tgt_edge, std::max<size_t>(E, 1) * sizeof(int32_t)));
    EP_CHECK(cudaMalloc((void**) &tgt_ptr, (size_t) (NT + 1) * sizeof(int32_t)));
    EP_CHECK(cudaMalloc((void**) &count, (size_t) (NT + 1) * sizeof(int32_t)));
    EP_CHECK(cudaMemsetAsync(count, 0, (size_t) (NT + 1) * sizeof(int32_t), st));
    edge_emit_kernel<<<aprnet_ceil_div(F, 256), 256, 0, st>>>(plan->nbr, N, scan, src, tgt, count);
    EP_CHECK(cub::DeviceScan::ExclusiveSum(temp, temp_bytes, count, tgt_ptr, (int) (NT + 1), st));
    EP_CHECK(cudaMemcpyAsync(count, tgt_ptr, (size_t) (NT + 1) * sizeof(int32_t), cudaMemcpyDeviceToDevice, st));   // cursors
    if (E) edge_fill_kernel<<<aprnet_ceil_div(E, 256), 256, 0, st>>>(tgt, E, count, tgt_edge);
    edge_sort_kernel<<<aprnet_ceil_div(NT + 1, 128), 128, 0, st>>>(tgt_ptr, NT, tgt_edge, count);     // also flags active targets in `count`
    EP_CHECK(cub::DeviceScan::ExclusiveSum(temp, temp_bytes, count, count, (int) (NT + 1), st));
    int32_t n_active = 0;
    EP_CHECK(cudaMemcpyAsync(&n_active, count + NT, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    EP_CHECK(cudaStreamSynchronize(st));
    ep.n_active = n_active;
    if ((rc = dev_alloc(&ep.active, (size_t) n_active, &a->device_bytes))) { cleanup(); return rc; }
    if (NT) edge_compact_active_kernel<<<aprnet_ceil_div(NT, 256), 256, 0, st>>>(count, NT, ep.active);
    cudaFree(scan); scan = nullptr;
    cudaFree(tgt); tgt = nullptr;

    // virtual rows: runs of equal tap in every active target's list
    EP_CHECK(cudaMalloc((void**) &vfirst, (size_t) (n_active + 1) * sizeof(int32_t)));
    vrow_count_kernel<<<aprnet_ceil_div((ll) n_active + 1, 128), 128, 0, st>>>(ep.active, n_active, tgt_ptr, tgt_edge, tb, vfirst);
    EP_CHECK(cub::DeviceScan::ExclusiveSum(temp, temp_bytes, vfirst, vfirst, n_active + 1, st));
    int32_t n_vrows = 0;
    EP_CHECK(cudaMemcpyAsync(&n_vrows, vfirst + n_active, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    EP_CHECK(cudaStreamSynchronize(st));
    ep.n_vrows = n_vrows;
    if ((rc = dev_alloc(&ep.vsrc, (size_t) E, &a->device_bytes)) || (rc = dev_alloc(&ep.vstart, (size_t) n_vrows + 1, &a->device_bytes)) ||
        (rc = dev_alloc(&ep.vnbr, (size_t) 27 * std::max(n_active, 1), &a->device_bytes))) { cleanup(); return rc; }
    EP_CHECK(cudaMemsetAsync(ep.vnbr, 0xFF, (size_t) 27 * std::max(n_active, 1) * sizeof(int32_t), st));       // APRNET_NONE
    EP_CHECK(cudaMemsetAsync(ep.vstart, 0, ((size_t) n_vrows + 1) * sizeof(int32_t), st));
    if (n_active) vrow_fill_kernel<<<aprnet_ceil_div(n_active, 128), 128, 0, st>>>(ep.active, n_active, tgt_ptr, tgt_edge, src, tb, vfirst, E,
                                                                                  ep.vstart, ep.vnbr, ep.vsrc);

    // ranges of active[] by level of the locations their edges come from, and the chunk map
    const int cml = a->cml(dl);
    std::vector<ll> key_h;
    std::vector<int> key_level;
    for (int l = a->meta.level_min; l <= cml; ++l) {        // particle targets of level l <- locations of level l + 1
        key_h.push_back(a->meta.lvl_begin[l]); key_level.push_back(l + 1);
    }
    for (int l = a->meta.level_min - 1; l <= cml - 1; ++l) {    // tree targets of level l <- locations of level l
        key_h.push_back(N + a->meta.tlvl_begin[l]); key_level.push_back(l);
    }
    key_h.push_back(NT); key_level.push_back(-1);
    const int nkeys = (int) key_h.size();
    const int nchunk = (int) (n_vrows / VROW_GRANULE) + 1;
    EP_CHECK(cudaMalloc((void**) &keys, (size_t) std::max(nkeys, nchunk + 1) * sizeof(ll)));
    EP_CHECK(cudaMalloc((void**) &found, (size_t) std::max(nkeys, nchunk + 1) * sizeof(ll)));
    std::vector<ll> found_h(std::max(nkeys, nchunk + 1));
    EP_CHECK(cudaMemcpyAsync(keys, key_h.data(), nkeys * sizeof(ll), cudaMemcpyHostToDevice, st));
    lower_bound_kernel<<<1, 64, 0, st>>>(ep.active, n_active, keys, nkeys, found);
    EP_CHECK(cudaMemcpyAsync(found_h.data(), found, nkeys * sizeof(ll), cudaMemcpyDeviceToHost, st));
    EP_CHECK(cudaStreamSynchronize(st));
    ep.segs.clear();
    for (int k = 0; k + 1 < nkeys; ++k) {
        ActiveSeg sg; sg.begin = found_h[k]; sg.end = found_h[k + 1]; sg.location_level = key_level[k];
        if (sg.end > sg.begin && sg.location_level >= a->meta.level_min && sg.location_level <= cml) ep.segs.push_back(sg);
        else if (sg.end > sg.begin) { aprnet_set_error("edge plan: edges from level %d outside [%d, %d]", sg.location_level, a->meta.level_min, cml); cleanup(); return APRNET_ERR_CUDA; }
    }
    std::vector<ll> ckey(nchunk + 1);
    for (int k = 0; k < nchunk; ++k) ckey[k] = (ll) k * VROW_GRANULE;
    ckey[nchunk] = (ll) n_vrows + 1;        // beyond the last value: maps to n_active
    EP_CHECK(cudaMemcpyAsync(keys, ckey.data(), (nchunk + 1) * sizeof(ll), cudaMemcpyHostToDevice, st));
    lower_bound_kernel<<<aprnet_ceil_div(nchunk + 1, 64), 64, 0, st>>>(vfirst, n_active, keys, nchunk + 1, found);
    EP_CHECK(cudaMemcpyAsync(found_h.data(), found, (nchunk + 1) * sizeof(ll), cudaMemcpyDeviceToHost, st));
    EP_CHECK(cudaStreamSynchronize(st));
    std::vector<int32_t> vf(nchunk + 1);
    ep.chunk_a.clear(); ep.chunk_v.clear();
    for (int k = 0; k <= nchunk; ++k) {
        const ll ca = std::min<ll>(found_h[k], n_active);
        if (!ep.chunk_a.empty() && ep.chunk_a.back() == ca) continue;
        int32_t v = 0;
        EP_CHECK(cudaMemcpyAsync(&v, vfirst + ca, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
        EP_CHECK(cudaStreamSynchronize(st));
        ep.chunk_a.push_back(ca); ep.chunk_v.push_back(v);
    }
    if (ep.chunk_a.back() != n_active) { ep.chunk_a.push_back(n_active); ep.chunk_v.push_back(n_vrows); }
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

extern "C" int64_t aprnet_edge_workspace_bytes(const aprnet_apr* a, int dl, int cout) {
    if (!a || !a->valid_dl(dl)) return -1;
    const ll cap = 8ll << 30;     // bounds the virtual-row workspace; smaller = more passes
    const ll row = (ll) aprnet_tc_pad(cout) * 2;
    auto it = a->edge_plans.find(dl);
    const ll rows = it != a->edge_plans.end() ? it->second.n_vrows + 2 : 27 * a->number_parts(dl) + 2;
    return (int64_t) std::max<ll>(256, std::min(cap, rows * row));
}

// Cross-level part of the input gradient (added to grad_input, which holds the same-level part, and to
// grad_tree, which the call zero-fills) followed by the tree adjoint.  packed_grad_output_rows:
// channels-last bf16 dO rows; weights fp32 (slots, Cout, Cin, 27); wp_ws: space for the packed
// transposed weights; edge_ws: aprnet_edge_workspace_bytes() bytes.
int aprnet_cross_level_tc(aprnet_apr* a, int dl, int cin, int cout, int slots, const void* grows, int gpad, const float* w, float* gin,
                          long long ld_in, float* gtree, long long ld_tree, void* wp_ws, void* edge_ws, long long edge_ws_bytes, void* stream,
                          bool tree_adjoint) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && cin > 0 && cout > 0 && slots > 0 && grows && w && gin && gtree && wp_ws && edge_ws, "bad argument");
    APRNET_ARG_CHECK(gpad == aprnet_tc_pad(cout), "packed row width does not match the padded channel count");
    cudaStream_t st = (cudaStream_t) stream;
    EdgePlan* ep = aprnet_get_edge_plan(a, dl, st);
    if (!ep) return APRNET_ERR_CUDA;
    const ll ts = a->tree_size(dl);
    if (ts > 0) APRNET_CUDA_CHECK(cudaMemset2DAsync(gtree, (size_t) ld_tree * sizeof(float), 0, (size_t) ts * sizeof(float), (size_t) cin, st));
    if (ep->n_active > 0) {
        int rc = aprnet_tc_pack_weights(w, slots, cin, cout, 2, wp_ws, st);
        if (rc) return rc;
        __nv_bfloat16* vrows = reinterpret_cast<__nv_bfloat16*>(edge_ws);
        APRNET_CUDA_CHECK(cudaMemsetAsync(vrows, 0, (size_t) gpad * 2, st));          // row 0: zeros
        const ll cap_rows = edge_ws_bytes / ((ll) gpad * 2) - 1;
        const int nk = (int) ep->chunk_a.size() - 1;
        int k0 = 0;
        while (k0 < nk) {
            int k1 = k0 + 1;
            while (k1 < nk && ep->chunk_v[k1 + 1] - ep->chunk_v[k0] <= cap_rows) ++k1;
            const ll v0 = ep->chunk_v[k0], v1 = ep->chunk_v[k1], a0 = ep->chunk_a[k0], a1 = ep->chunk_a[k1];
            if (v1 - v0 > cap_rows) { aprnet_set_error("edge workspace too small for %lld virtual rows", v1 - v0); return APRNET_ERR_ARG; }
            if (v1 > v0) {
                { AprnetProfScope _prof("edge_reduce", st);
                vrow_reduce_kernel<VROW_VPT><<<aprnet_ceil_div(aprnet_ceil_div(v1 - v0, VROW_VPT) * (gpad / 8), 256), 256, 0, st>>>(
                    ep->vstart, ep->vsrc, v0, v1, (const __nv_bfloat16*) grows, gpad, vrows);
                }
                APRNET_LAUNCH_CHECK();
                // row index r of the gather = virtual row id; the zero row is addressed as v0 - 1
                rc = aprnet_tc_gather_targets(a, dl, cin, cout, slots, vrows + (1 - v0) * gpad, gpad, v0 - 1, wp_ws, ep, a0, a1,
                                              gin, ld_in, gtree, ld_tree, st);
                if (rc) return rc;
            }
            k0 = k1;
        }
    }
    if (!tree_adjoint) return APRNET_OK;
    return aprnet_fill_tree_mean_backward(a, dl, APRNET_F32, cin, gin, ld_in, gtree, ld_tree, st);
}

extern "C" int aprnet_conv333_backward_input_cross_level_tc(aprnet_apr* a, int dl, int cin, int cout, int slots,
                                                            const void* grows, int gpad, const float* w, float* gin,
                                                            int64_t ld_in, float* gtree, int64_t ld_tree, void* wp_ws,
                                                            void* edge_ws, int64_t edge_ws_bytes, void* stream) {
    return aprnet_cross_level_tc(a, dl, cin, cout, slots, grows, gpad, w, gin, ld_in, gtree, ld_tree, wp_ws, edge_ws, edge_ws_bytes, stream, true);
}
