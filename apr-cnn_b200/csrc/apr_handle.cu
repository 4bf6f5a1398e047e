// Device-side APR access structure, tree child table and per-level_delta neighbour tables.
//
// The reference re-derives "which rows hold anything" and re-stages dense (z, x, y) patches on every
// forward and backward call (pyapr/aprnet/cuda/src/nonempty_rows.cu:26-230,
// conv333_gpu.cu:63-118, fill_tree_gpu.cu:1098).  Here the sparse-row searches run once per APR
// (child table) and once per (APR, level_delta) (neighbour table); the hot kernels are pure
// index-driven gathers.
#include "apr_device.cuh"
#include <cstring>
#include <algorithm>

static thread_local std::string g_last_error;

void aprnet_set_error(const char* fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_last_error = buf;
}

extern "C" const char* aprnet_last_error(void) { return g_last_error.c_str(); }

// ---- per-kernel event timing -----------------------------------------------------------------
namespace {
struct ProfRecord { std::string name; cudaEvent_t start, stop; };
bool g_prof_on = false;
std::vector<ProfRecord> g_prof_records;
}

AprnetProfScope::AprnetProfScope(const char* name, cudaStream_t st) : slot(-1), stream(st) {
    if (!g_prof_on) return;
    ProfRecord r;
    r.name = name;
    if (cudaEventCreate(&r.start) != cudaSuccess || cudaEventCreate(&r.stop) != cudaSuccess) return;
    cudaEventRecord(r.start, st);
    g_prof_records.push_back(r);
    slot = (int) g_prof_records.size() - 1;
}

AprnetProfScope::~AprnetProfScope() {
    if (slot >= 0) cudaEventRecord(g_prof_records[slot].stop, stream);
}

extern "C" void aprnet_profile_enable(int on) { g_prof_on = on != 0; }

extern "C" int64_t aprnet_profile_read(char* buf, int64_t buflen) {
    std::map<std::string, std::pair<long long, double>> agg;
    for (ProfRecord& r : g_prof_records) {
        float ms = 0;
        if (cudaEventSynchronize(r.stop) == cudaSuccess && cudaEventElapsedTime(&ms, r.start, r.stop) == cudaSuccess) {
            agg[r.name].first += 1;
            agg[r.name].second += ms;
        }
        cudaEventDestroy(r.start);
        cudaEventDestroy(r.stop);
    }
    g_prof_records.clear();
    std::string out;
    for (auto& kv : agg) {
        char line[256];
        snprintf(line, sizeof(line), "%s %lld %.6f\n", kv.first.c_str(), kv.second.first, kv.second.second);
        out += line;
    }
    if (buf && buflen > 0) {
        const size_t n = std::min<size_t>(out.size(), (size_t) buflen - 1);
        memcpy(buf, out.data(), n);
        buf[n] = 0;
    }
    return (int64_t) out.size();
}

namespace {

typedef long long ll;

// first position in [b, e) whose y is >= target
__device__ __forceinline__ ll lower_bound_y(const uint16_t* __restrict__ y, ll b, ll e, int target) {
    while (b < e) {
        const ll mid = (b + e) >> 1;
        if ((int) y[mid] < target) b = mid + 1; else e = mid;
    }
    return b;
}

__device__ __forceinline__ ll find_y(const uint16_t* __restrict__ y, ll b, ll e, int target) {
    const ll p = lower_bound_y(y, b, e, target);
    return (p < e && (int) y[p] == target) ? p : -1;
}

// One warp per tree row of level `l`; lanes stride over the row's nodes.
__global__ void build_child_table_kernel(LevelMeta m, const ll* __restrict__ row_ptr, const uint16_t* __restrict__ y,
                                         const ll* __restrict__ trow_ptr, const uint16_t* __restrict__ ty,
                                         int32_t* __restrict__ child, float* __restrict__ scale, ll n_tree, int l) {
    const ll row = ((ll) blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const ll rows = (ll) m.z_num[l] * m.x_num[l];
    if (row >= rows) return;
    const int z = (int) (row / m.x_num[l]), x = (int) (row % m.x_num[l]);
    const ll tr = m.trow_off[l] + row;
    const ll tb = trow_ptr[tr], te = trow_ptr[tr + 1];
    const int cl = l + 1;
    const int bx = ((2 * m.x_num[l]) != m.x_num[cl]) && (x == m.x_num[l] - 1);
    const int bz = ((2 * m.z_num[l]) != m.z_num[cl]) && (z == m.z_num[l] - 1);
    const float f_xz = fmaxf(2.0f * (float) (bx + bz), 1.0f) / 8.0f;
    const bool y_odd = (2 * m.y_num[l]) != m.y_num[cl];
    const bool child_tree = cl <= m.level_max - 1;

    for (ll t = tb + lane; t < te; t += 32) {
        const int yp = ty[t];
        scale[t] = (y_odd && yp == m.y_num[l] - 1) ? 2.0f * f_xz : f_xz;
        for (int s4 = 0; s4 < 4; ++s4) {
            const int cz = 2 * z + (s4 >> 1), cx = 2 * x + (s4 & 1);
            int32_t v0 = APRNET_NONE, v1 = APRNET_NONE;
            if (cz < m.z_num[cl] && cx < m.x_num[cl]) {
                const ll crow = (ll) cz * m.x_num[cl] + cx;
                const ll pr = m.row_off[cl] + crow;
                const ll pb = row_ptr[pr], pe = row_ptr[pr + 1];
                ll p = lower_bound_y(y, pb, pe, 2 * yp);
                if (p < pe && (int) y[p] == 2 * yp) { v0 = (int32_t) p; ++p; }
                if (p < pe && (int) y[p] == 2 * yp + 1) v1 = (int32_t) p;
                if (child_tree && (v0 == APRNET_NONE || v1 == APRNET_NONE)) {
                    const ll ctr = m.trow_off[cl] + crow;
                    const ll cb = trow_ptr[ctr], ce = trow_ptr[ctr + 1];
                    ll q = lower_bound_y(ty, cb, ce, 2 * yp);
                    if (q < ce && (int) ty[q] == 2 * yp) { if (v0 == APRNET_NONE) v0 = aprnet_enc_tree(q); ++q; }
                    if (q < ce && (int) ty[q] == 2 * yp + 1 && v1 == APRNET_NONE) v1 = aprnet_enc_tree(q);
                }
            }
            child[(ll) (2 * s4) * n_tree + t] = v0;
            child[(ll) (2 * s4 + 1) * n_tree + t] = v1;
        }
    }
}

// One warp per output row of level `l`.  Output locations are the APR particles of the row
// (outputs_are_tree == 0) or, at the current max level of a pooled tensor, its tree nodes
// (outputs_are_tree == 1, stored at tree index + tree_off).  Cell resolution order follows
// pyapr/aprnet/src/helpers.hpp:373-408: same-level particle, else the covering particle one level
// coarser, else the tree node of that cell (stored value at l == cml, tree mean below), else nothing.
__global__ void build_nbr_table_kernel(LevelMeta m, const ll* __restrict__ row_ptr, const uint16_t* __restrict__ y,
                                       const ll* __restrict__ trow_ptr, const uint16_t* __restrict__ ty,
                                       int32_t* __restrict__ nbr, ll N, int l, int cml, ll tree_off, int outputs_are_tree) {
    const ll row = ((ll) blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int xn = m.x_num[l], zn = m.z_num[l], yn = m.y_num[l];
    if (row >= (ll) zn * xn) return;
    const int z = (int) (row / xn), x = (int) (row % xn);

    ll ob, oe;
    const uint16_t* oy;
    ll shift;
    if (outputs_are_tree) {
        const ll tr = m.trow_off[l] + row;
        ob = trow_ptr[tr]; oe = trow_ptr[tr + 1]; oy = ty; shift = tree_off;
    } else {
        const ll r = m.row_off[l] + row;
        ob = row_ptr[r]; oe = row_ptr[r + 1]; oy = y; shift = 0;
    }
    if (ob == oe) return;
    const bool has_parent = l > m.level_min;
    const bool has_tree = l <= m.level_max - 1;

    for (int dz = -1; dz <= 1; ++dz) {
        for (int dx = -1; dx <= 1; ++dx) {
            const int nz = z + dz, nx = x + dx;
            const int tap0 = ((dz + 1) * 3 + (dx + 1)) * 3;
            const bool inside = nz >= 0 && nx >= 0 && nz < zn && nx < xn;
            ll sb = 0, se = 0, pb = 0, pe = 0, tb = 0, te = 0;
            if (inside) {
                const ll r = m.row_off[l] + (ll) nz * xn + nx;
                sb = row_ptr[r]; se = row_ptr[r + 1];
                if (has_parent) {
                    const ll pr = m.row_off[l - 1] + (ll) (nz >> 1) * m.x_num[l - 1] + (nx >> 1);
                    pb = row_ptr[pr]; pe = row_ptr[pr + 1];
                }
                if (has_tree) {
                    const ll tr = m.trow_off[l] + (ll) nz * xn + nx;
                    tb = trow_ptr[tr]; te = trow_ptr[tr + 1];
                }
            }
            for (ll i = ob + lane; i < oe; i += 32) {
                const int yo = oy[i];
                const ll p = i + shift;
                for (int dy = -1; dy <= 1; ++dy) {
                    const int yq = yo + dy;
                    int32_t v = APRNET_NONE;
                    if (inside && yq >= 0 && yq < yn) {
                        ll f = find_y(y, sb, se, yq);
                        if (f >= 0) v = (int32_t) f;
                        else {
                            f = has_parent ? find_y(y, pb, pe, yq >> 1) : -1;
                            if (f >= 0) v = (int32_t) f;
                            else {
                                f = has_tree ? find_y(ty, tb, te, yq) : -1;
                                if (f >= 0) v = (l == cml) ? (int32_t) (f + tree_off) : aprnet_enc_tree(f);
                            }
                        }
                    }
                    nbr[(ll) (tap0 + dy + 1) * N + p] = v;
                }
            }
        }
    }
}

template<typename T>
int upload(T** dst, const T* src, size_t n, long long* bytes) {
    APRNET_CUDA_CHECK(cudaMalloc((void**) dst, std::max<size_t>(n, 1) * sizeof(T)));
    if (n) APRNET_CUDA_CHECK(cudaMemcpy(*dst, src, n * sizeof(T), cudaMemcpyHostToDevice));
    *bytes += (long long) (std::max<size_t>(n, 1) * sizeof(T));
    return APRNET_OK;
}

} // namespace

std::vector<Segment> aprnet_segments(const aprnet_apr* apr, int dl, int num_slots, bool merge) {
    std::vector<Segment> segs;
    const int cml = apr->cml(dl);
    const long long N = apr->number_parts(dl);
    for (int l = apr->meta.level_min; l <= cml; ++l) {
        Segment s;
        s.begin = apr->meta.lvl_begin[l];
        s.end = (l == cml) ? N : apr->meta.lvl_begin[l + 1];
        s.slot = std::min(cml - l, num_slots - 1);
        s.level = l;
        if (s.end <= s.begin) continue;
        if (merge && !segs.empty() && segs.back().slot == s.slot && segs.back().end == s.begin) segs.back().end = s.end;
        else segs.push_back(s);
    }
    return segs;
}

extern "C" int aprnet_apr_create(aprnet_apr** out, int level_min, int level_max, const int* dims,
                                 const int64_t* row_ptr, const uint16_t* y,
                                 const int64_t* tree_row_ptr, const uint16_t* tree_y, int device) {
    APRNET_ARG_CHECK(out && dims && row_ptr && tree_row_ptr, "null argument");
    APRNET_ARG_CHECK(level_min >= 1 && level_max >= level_min && level_max < APRNET_MAX_LEVELS - 1, "bad level range");
    // the structure is built on `device`; the caller's current device is restored on every way out
    struct DeviceRestore { int prev = -1; ~DeviceRestore() { if (prev >= 0) cudaSetDevice(prev); } } restore;
    if (cudaGetDevice(&restore.prev) != cudaSuccess) { restore.prev = -1; cudaGetLastError(); }
    APRNET_CUDA_CHECK(cudaSetDevice(device));
    aprnet_apr* a = new aprnet_apr();
    a->device = device;
    LevelMeta& m = a->meta;
    memset(&m, 0, sizeof(m));
    m.level_min = level_min; m.level_max = level_max;
    for (int l = 0; l <= level_max; ++l) { m.z_num[l] = dims[3 * l]; m.x_num[l] = dims[3 * l + 1]; m.y_num[l] = dims[3 * l + 2]; }
    for (int l = 0; l <= level_max; ++l) {
        m.row_off[l + 1] = m.row_off[l] + (l >= level_min ? (long long) m.z_num[l] * m.x_num[l] : 0);
        m.trow_off[l + 1] = m.trow_off[l] + ((l >= level_min - 1 && l <= level_max - 1) ? (long long) m.z_num[l] * m.x_num[l] : 0);
    }
    for (int l = level_max + 1; l < APRNET_MAX_LEVELS; ++l) { m.row_off[l + 1] = m.row_off[l]; m.trow_off[l + 1] = m.trow_off[l]; }
    a->n_rows = m.row_off[level_max + 1];
    a->n_tree_rows = m.trow_off[level_max];
    for (int l = 0; l <= APRNET_MAX_LEVELS; ++l) {
        m.lvl_begin[l] = row_ptr[std::min(m.row_off[std::min(l, APRNET_MAX_LEVELS)], a->n_rows)];
        m.tlvl_begin[l] = tree_row_ptr[std::min(m.trow_off[std::min(l, APRNET_MAX_LEVELS)], a->n_tree_rows)];
    }
    a->n_particles = row_ptr[a->n_rows];
    a->n_tree = tree_row_ptr[a->n_tree_rows];
    if (a->n_particles >= (1ll << 31) - 2 || a->n_tree >= (1ll << 31) - 2) {
        delete a;
        aprnet_set_error("aprnet_apr_create: more than 2^31 particles are not supported by the 32-bit tables");
        return APRNET_ERR_UNSUPPORTED;
    }
    static_assert(sizeof(long long) == sizeof(int64_t), "int64 layout");
    int rc;
    if ((rc = upload(&a->row_ptr, (const long long*) row_ptr, (size_t) a->n_rows + 1, &a->device_bytes))) { delete a; return rc; }
    if ((rc = upload(&a->y, y, (size_t) a->n_particles, &a->device_bytes))) { delete a; return rc; }
    if ((rc = upload(&a->tree_row_ptr, (const long long*) tree_row_ptr, (size_t) a->n_tree_rows + 1, &a->device_bytes))) { delete a; return rc; }
    if ((rc = upload(&a->tree_y, tree_y, (size_t) a->n_tree, &a->device_bytes))) { delete a; return rc; }

    const size_t nt = (size_t) std::max<long long>(a->n_tree, 1);
    APRNET_CUDA_CHECK(cudaMalloc((void**) &a->child, 8 * nt * sizeof(int32_t)));
    APRNET_CUDA_CHECK(cudaMalloc((void**) &a->tree_scale, nt * sizeof(float)));
    a->device_bytes += (long long) (8 * nt * sizeof(int32_t) + nt * sizeof(float));
    for (int l = level_min - 1; l <= level_max - 1; ++l) {
        const long long rows = (long long) m.z_num[l] * m.x_num[l];
        const int blocks = aprnet_ceil_div(rows * 32, 128);
        build_child_table_kernel<<<blocks, 128>>>(m, a->row_ptr, a->y, a->tree_row_ptr, a->tree_y, a->child,
                                                  a->tree_scale, a->n_tree, l);
        APRNET_LAUNCH_CHECK();
    }
    APRNET_CUDA_CHECK(cudaDeviceSynchronize());
    *out = a;
    return APRNET_OK;
}

extern "C" void aprnet_apr_destroy(aprnet_apr* a) {
    if (!a) return;
    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess) { prev = -1; cudaGetLastError(); }
    cudaSetDevice(a->device);
    cudaFree(a->row_ptr); cudaFree(a->y); cudaFree(a->tree_row_ptr); cudaFree(a->tree_y);
    cudaFree(a->child); cudaFree(a->tree_scale);
    for (auto& kv : a->plans) cudaFree(kv.second.nbr);
    cudaFree(a->node_parent);
    for (auto& kv : a->loc_parent) cudaFree(kv.second);
    for (auto& kv : a->edge_plans) aprnet_free_edge_plan(kv.second);
    delete a;
    if (prev >= 0) cudaSetDevice(prev);
}

// Every entry point launches on the current device with pointers that live on the handle's device: a mismatch is
// an argument error here instead of an illegal address inside a kernel.
int aprnet_check_device(const aprnet_apr* a) {
    int cur = -1;
    if (cudaGetDevice(&cur) != cudaSuccess) { cudaGetLastError(); aprnet_set_error("no current CUDA device"); return APRNET_ERR_CUDA; }
    if (a && cur != a->device) {
        aprnet_set_error("the access structure lives on device %d but the current device is %d", a->device, cur);
        return APRNET_ERR_ARG;
    }
    return APRNET_OK;
}

extern "C" int64_t aprnet_number_parts(const aprnet_apr* a, int dl) { return (a && a->valid_dl(dl)) ? a->number_parts(dl) : -1; }
extern "C" int64_t aprnet_tree_size(const aprnet_apr* a, int dl) { return (a && a->valid_dl(dl)) ? a->tree_size(dl) : -1; }
extern "C" int64_t aprnet_total_tree_nodes(const aprnet_apr* a) { return a ? a->n_tree : -1; }
extern "C" int64_t aprnet_device_bytes(const aprnet_apr* a) { return a ? a->device_bytes : -1; }

const AprPlan* aprnet_get_plan(aprnet_apr* a, int dl, cudaStream_t stream) {
    if (aprnet_check_device(a) != APRNET_OK) return nullptr;
    auto it = a->plans.find(dl);
    if (it != a->plans.end()) return &it->second;
    AprPlan p;
    p.level_delta = dl;
    p.n = a->number_parts(dl);
    p.tree_size = a->tree_size(dl);
    const size_t elems = 27 * (size_t) std::max<long long>(p.n, 1);
    if (cudaMalloc((void**) &p.nbr, elems * sizeof(int32_t)) != cudaSuccess) {
        aprnet_set_error("aprnet_plan_build: cudaMalloc of %zu bytes failed", elems * sizeof(int32_t));
        cudaGetLastError();
        return nullptr;
    }
    a->device_bytes += (long long) (elems * sizeof(int32_t));
    const LevelMeta& m = a->meta;
    const int cml = a->cml(dl);
    const long long toff = (cml <= m.level_max - 1) ? a->tree_offset(cml) : 0;
    for (int l = m.level_min; l <= cml; ++l) {
        const long long rows = (long long) m.z_num[l] * m.x_num[l];
        const int blocks = aprnet_ceil_div(rows * 32, 128);
        build_nbr_table_kernel<<<blocks, 128, 0, stream>>>(m, a->row_ptr, a->y, a->tree_row_ptr, a->tree_y, p.nbr,
                                                           p.n, l, cml, toff, 0);
        if (l == cml && dl > 0)
            build_nbr_table_kernel<<<blocks, 128, 0, stream>>>(m, a->row_ptr, a->y, a->tree_row_ptr, a->tree_y, p.nbr,
                                                               p.n, l, cml, toff, 1);
    }
    if (cudaGetLastError() != cudaSuccess) {
        aprnet_set_error("aprnet_plan_build: kernel launch failed");
        cudaFree(p.nbr);
        return nullptr;
    }
    auto res = a->plans.emplace(dl, p);
    return &res.first->second;
}

// Parent tables from the child table: every child slot of tree node t names a particle (v >= 0), a tree node (coded) or,
// at the finest tree level of a level delta > 0 (use_up), an upgraded node that lives in the feature vector at
// up_off + index.  Either output may be null.
__global__ void build_parent_tables_kernel(const int32_t* __restrict__ child, long long n_tree, long long tb, long long te,
                                           long long up_off, int use_up, int32_t* __restrict__ loc_parent, int32_t* __restrict__ node_parent) {
    const long long t = tb + (long long) blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= te) return;
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        const int32_t v = child[(long long) s * n_tree + t];
        if (v >= 0) { if (loc_parent) loc_parent[v] = (int32_t) t; }
        else if (v != APRNET_NONE) {
            if (use_up) { if (loc_parent) loc_parent[aprnet_dec_tree(v) + up_off] = (int32_t) t; }
            else if (node_parent) node_parent[aprnet_dec_tree(v)] = (int32_t) t;
        }
    }
}

static int32_t* alloc_minus_one(const aprnet_apr* a, long long n, cudaStream_t stream, const char* what) {
    int32_t* p = nullptr;
    n = std::max<long long>(n, 1);
    if (cudaMalloc((void**) &p, (size_t) n * sizeof(int32_t)) != cudaSuccess) {
        aprnet_set_error("%s: cudaMalloc of %zu bytes failed", what, (size_t) n * sizeof(int32_t));
        cudaGetLastError();
        return nullptr;
    }
    a->device_bytes += n * (long long) sizeof(int32_t);
    cudaMemsetAsync(p, 0xFF, (size_t) n * sizeof(int32_t), stream);
    return p;
}

const int32_t* aprnet_node_parent_table(const aprnet_apr* a, cudaStream_t stream) {
    if (a->node_parent) return a->node_parent;
    int32_t* tab = alloc_minus_one(a, a->n_tree, stream, "aprnet_node_parent_table");
    if (!tab) return nullptr;
    const LevelMeta& m = a->meta;
    for (int lp = m.level_min - 1; lp <= m.level_max - 1; ++lp) {
        const long long tb = m.tlvl_begin[lp], te = m.tlvl_begin[lp + 1];
        if (te > tb) build_parent_tables_kernel<<<aprnet_ceil_div(te - tb, 256), 256, 0, stream>>>(a->child, a->n_tree, tb, te, 0, 0, nullptr, tab);
    }
    if (cudaGetLastError() != cudaSuccess) { aprnet_set_error("aprnet_node_parent_table: kernel launch failed"); cudaFree(tab); return nullptr; }
    a->node_parent = tab;
    return tab;
}

const int32_t* aprnet_loc_parent_table(const aprnet_apr* a, int dl, cudaStream_t stream) {
    auto it = a->loc_parent.find(dl);
    if (it != a->loc_parent.end()) return it->second;
    int32_t* tab = alloc_minus_one(a, a->number_parts(dl), stream, "aprnet_loc_parent_table");
    if (!tab) return nullptr;
    const LevelMeta& m = a->meta;
    const int cml = a->cml(dl);
    const long long up = (dl > 0) ? a->tree_offset(cml) : 0;
    for (int lp = m.level_min - 1; lp <= cml - 1; ++lp) {
        const long long tb = m.tlvl_begin[lp], te = m.tlvl_begin[lp + 1];
        if (te > tb) build_parent_tables_kernel<<<aprnet_ceil_div(te - tb, 256), 256, 0, stream>>>(a->child, a->n_tree, tb, te, up,
                                                                                                 (dl > 0 && lp + 1 == cml) ? 1 : 0, tab, nullptr);
    }
    if (cudaGetLastError() != cudaSuccess) { aprnet_set_error("aprnet_loc_parent_table: kernel launch failed"); cudaFree(tab); return nullptr; }
    a->loc_parent.emplace(dl, tab);
    return tab;
}

extern "C" int aprnet_plan_build(aprnet_apr* a, int dl, void* stream) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl), "bad handle or level_delta");
    if (!aprnet_get_plan(a, dl, (cudaStream_t) stream)) return APRNET_ERR_CUDA;
    if (!aprnet_node_parent_table(a, (cudaStream_t) stream) || !aprnet_loc_parent_table(a, dl, (cudaStream_t) stream)) return APRNET_ERR_CUDA;
    return APRNET_OK;
}

extern "C" int aprnet_plan_copy_nbr_table(aprnet_apr* a, int dl, int32_t* host_out) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && host_out, "bad argument");
    const AprPlan* p = aprnet_get_plan(a, dl, 0);
    if (!p) return APRNET_ERR_CUDA;
    APRNET_CUDA_CHECK(cudaDeviceSynchronize());
    APRNET_CUDA_CHECK(cudaMemcpy(host_out, p->nbr, 27 * (size_t) p->n * sizeof(int32_t), cudaMemcpyDeviceToHost));
    return APRNET_OK;
}

extern "C" int aprnet_copy_child_table(aprnet_apr* a, int32_t* host_out) {
    APRNET_ARG_CHECK(a && host_out, "bad argument");
    APRNET_CUDA_CHECK(cudaMemcpy(host_out, a->child, 8 * (size_t) a->n_tree * sizeof(int32_t), cudaMemcpyDeviceToHost));
    return APRNET_OK;
}
