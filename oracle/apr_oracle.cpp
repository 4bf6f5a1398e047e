// TEST INFRASTRUCTURE ONLY — CPU restatement of the reference's particle-domain CNN operators.
//
// Only tests, the smoke check and the benchmark's CPU-baseline leg may load this library; the
// product (the CUDA library and its Python/pybind host layer) never links, imports or calls it.
//
// Each function restates one reference routine in a *direct* form (every neighbour cell is resolved
// by searching the sparse rows) instead of the reference's rolling dense-row buffers, so that the two
// formulations cross-check each other.  Citations are paths inside the reference project
// (AdaptiveParticles/APR-CNN).  Parity status: pinned against the reference's own CPU code compiled
// unmodified (oracle/build_ref.py) through the committed vectors in tests/golden/ and, when that
// module is present, live on random structures (tests/test_oracle.py).
//
// Plain C ABI, plain pointers; build: g++ -O2 -fopenmp -shared -fPIC apr_oracle.cpp -o libapr_oracle.so
#include <cstdint>
#include <cstring>
#include <cmath>
#include <vector>
#include <algorithm>

namespace {

struct Access {
    int level_min = 0, level_max = 0;
    std::vector<int> z_num, x_num, y_num;
    std::vector<int64_t> row_off;
    const int64_t* row_ptr = nullptr;
    const uint16_t* y = nullptr;

    void init(int lmin, int lmax, const int* dims_zxy, const int64_t* rp, const uint16_t* yy) {
        level_min = lmin; level_max = lmax;
        z_num.resize(lmax + 1); x_num.resize(lmax + 1); y_num.resize(lmax + 1);
        for (int l = 0; l <= lmax; ++l) { z_num[l] = dims_zxy[3 * l]; x_num[l] = dims_zxy[3 * l + 1]; y_num[l] = dims_zxy[3 * l + 2]; }
        row_off.assign(lmax + 2, 0);
        for (int l = 0; l <= lmax; ++l) row_off[l + 1] = row_off[l] + (l >= lmin ? int64_t(z_num[l]) * x_num[l] : 0);
        row_ptr = rp; y = yy;
    }
    inline int64_t row(int l, int z, int x) const { return row_off[l] + int64_t(z) * x_num[l] + x; }
    inline int64_t level_begin(int l) const { return row_ptr[row_off[l]]; }
    inline int64_t level_end(int l) const { return row_ptr[row_off[l + 1]]; }
    inline bool has_level(int l) const { return l >= level_min && l <= level_max; }
    // index of the particle with coordinate yq in row (l, z, x), or -1
    inline int64_t find(int l, int z, int x, int yq) const {
        if (!has_level(l) || z < 0 || x < 0 || z >= z_num[l] || x >= x_num[l]) return -1;
        const int64_t r = row(l, z, x);
        const uint16_t* b = y + row_ptr[r];
        const uint16_t* e = y + row_ptr[r + 1];
        const uint16_t* it = std::lower_bound(b, e, (uint16_t) yq);
        return (it != e && *it == yq) ? (it - y) : -1;
    }
};

struct Apr {
    Access parts, tree;
    std::vector<int64_t> rp, trp;
    std::vector<uint16_t> yv, tyv;
    int level_min() const { return parts.level_min; }
    int level_max() const { return parts.level_max; }
    // pyapr/aprnet/src/helpers.hpp:113-117 (compute_tree_offset)
    int64_t tree_offset(int level) const { return parts.level_end(level) - tree.level_begin(level); }
    // pyapr/aprnet/src/helpers.hpp:86-101 (number_parts)
    int64_t number_parts(int dl) const {
        const int cml = level_max() - dl;
        int64_t n = parts.level_end(cml);
        if (cml <= tree.level_max) n += tree.level_end(cml) - tree.level_begin(cml);
        return n;
    }
    // number of tree nodes with level <= cml - 1 (size of the tree scratch; helpers.hpp:166)
    int64_t tree_size(int dl) const { return tree.level_end(level_max() - dl - 1); }
};

// Neighbour / child table encoding shared with the CUDA plan builder:
//   v >= 0 : index into the feature vector (particle, or "upgraded" tree node at tree_offset + t)
//   v == -1: no source (outside the domain) -> contributes zero
//   v <= -2: index t = -2 - v into the tree scratch (mean of the finer particles)
constexpr int32_t NONE = -1;
inline int32_t enc_tree(int64_t t) { return (int32_t) (-2 - t); }

// Which value fills cell (l; z, x, y) of the dense neighbourhood of a level-l row.
// pyapr/aprnet/src/helpers.hpp:373-408 (update_dense_array): same-level particle, else the covering
// particle one level coarser (3x3x3 stencils consult ONE parent level, helpers.hpp:353-355,380-393),
// else the tree node of that cell: the stored "upgraded" value when l == current max level
// (:398-402) or the tree mean (:404-406).  Outside the level's extent the buffer is zero
// (:410-419, zero_boundary_x/z :481-502).
inline int32_t resolve(const Apr& a, int cml, int l, int z, int x, int y) {
    const Access& P = a.parts; const Access& T = a.tree;
    if (z < 0 || x < 0 || y < 0 || z >= P.z_num[l] || x >= P.x_num[l] || y >= P.y_num[l]) return NONE;
    int64_t i = P.find(l, z, x, y);
    if (i >= 0) return (int32_t) i;
    if (l > P.level_min) {
        i = P.find(l - 1, z / 2, x / 2, y / 2);
        if (i >= 0) return (int32_t) i;
    }
    if (l < P.level_max) {
        i = T.find(l, z, x, y);
        if (i >= 0) return (l == cml) ? (int32_t) (i + a.tree_offset(l)) : enc_tree(i);
    }
    return NONE;
}

// helpers.hpp:133-153 (_compute_scale_factor_xz / _yxz): 1/8 per child, doubled for every axis in
// which the parent sits on an odd-sized border (so the mean runs over the existing children only).
inline float scale_xz(const Access& child, const Access& parent, int level, int z, int x) {
    float s = float(((2 * parent.x_num[level - 1]) != child.x_num[level]) && ((x / 2) == (parent.x_num[level - 1] - 1))) +
              float(((2 * parent.z_num[level - 1]) != child.z_num[level]) && ((z / 2) == (parent.z_num[level - 1] - 1)));
    return std::max(s * 2.0f, 1.0f) / 8.0f;
}
inline float scale_yxz(float sxz, const Access& child, const Access& parent, int level) {
    return ((2 * parent.y_num[level - 1]) != child.y_num[level]) ? sxz * 2.0f : sxz;
}

// Visit every child -> parent link of one child level.  `child` is the particle access (APR
// particles at `level`) or the tree access (tree nodes at `level`); parents are tree nodes at
// level-1 found by merging the sorted child y/2 with the sorted parent y (helpers.hpp:185-195).
template<typename F>
void for_each_link(const Access& child, const Access& tree, int level, F&& f) {
    if (!child.has_level(level)) return;
    for (int z = 0; z < child.z_num[level]; ++z) {
        for (int x = 0; x < child.x_num[level]; ++x) {
            const float sxz = scale_xz(child, tree, level, z, x);
            const float syxz = scale_yxz(sxz, child, tree, level);
            const int64_t r = child.row(level, z, x);
            const int64_t pr = tree.row(level - 1, z / 2, x / 2);
            int64_t p = tree.row_ptr[pr];
            for (int64_t c = child.row_ptr[r]; c < child.row_ptr[r + 1]; ++c) {
                while (tree.y[p] < child.y[c] / 2) ++p;
                const float s = (tree.y[p] == tree.y_num[level - 1] - 1) ? syxz : sxz;
                f(c, p, s);
            }
        }
    }
}

// helpers.hpp:156-252 (fill_tree_mean)
template<typename T>
void fill_tree_mean(const Apr& a, int dl, const T* in, T* tree) {
    const int cml = a.level_max() - dl;
    std::fill(tree, tree + a.tree_size(dl), T(0));
    if (cml < a.level_max()) {                                   // upgraded nodes (:174-198)
        const int64_t off = a.tree_offset(cml);
        for_each_link(a.tree, a.tree, cml, [&](int64_t c, int64_t p, float s) { tree[p] += s * in[c + off]; });
    }
    for (int l = cml; l >= a.level_min(); --l)                   // APR particles (:201-224)
        for_each_link(a.parts, a.tree, l, [&](int64_t c, int64_t p, float s) { tree[p] += s * in[c]; });
    for (int l = std::min(cml - 1, a.tree.level_max); l > a.tree.level_min; --l)   // tree -> tree (:227-250)
        for_each_link(a.tree, a.tree, l, [&](int64_t c, int64_t p, float s) { tree[p] += s * tree[c]; });
}

// helpers.hpp:255-350 (fill_tree_mean_backward): root -> leaf, then onto particles / upgraded nodes
template<typename T>
void fill_tree_mean_backward(const Apr& a, int dl, T* grad_in, T* grad_tree) {
    const int cml = a.level_max() - dl;
    for (int l = a.tree.level_min + 1; l <= std::min(cml - 1, a.tree.level_max); ++l)
        for_each_link(a.tree, a.tree, l, [&](int64_t c, int64_t p, float s) { grad_tree[c] += s * grad_tree[p]; });
    for (int l = cml; l >= a.level_min(); --l)
        for_each_link(a.parts, a.tree, l, [&](int64_t c, int64_t p, float s) { grad_in[c] += s * grad_tree[p]; });
    if (cml < a.level_max()) {
        const int64_t off = a.tree_offset(cml);
        for_each_link(a.tree, a.tree, cml, [&](int64_t c, int64_t p, float s) { grad_in[c + off] += s * grad_tree[p]; });
    }
}

// Visit every output location of level_delta dl: APR particles of levels <= cml and, when dl > 0,
// the upgraded tree nodes of level cml (conv.hpp:123-191; helpers.hpp:521,547-549).
template<typename F>
void for_each_output(const Apr& a, int dl, F&& f) {
    const int cml = a.level_max() - dl;
    for (int l = cml; l >= a.level_min(); --l) {
        const Access& P = a.parts;
        for (int z = 0; z < P.z_num[l]; ++z)
            for (int x = 0; x < P.x_num[l]; ++x) {
                const int64_t r = P.row(l, z, x);
                for (int64_t i = P.row_ptr[r]; i < P.row_ptr[r + 1]; ++i) f(i, l, z, x, (int) P.y[i]);
                if (l == cml && l < a.level_max()) {
                    const Access& T = a.tree;
                    const int64_t off = a.tree_offset(l);
                    const int64_t tr = T.row(l, z, x);
                    for (int64_t i = T.row_ptr[tr]; i < T.row_ptr[tr + 1]; ++i) f(i + off, l, z, x, (int) T.y[i]);
                }
            }
    }
}

void nbr_table(const Apr& a, int dl, int32_t* out) {
    const int cml = a.level_max() - dl;
    const int64_t N = a.number_parts(dl);
    for_each_output(a, dl, [&](int64_t p, int l, int z, int x, int y) {
        int tap = 0;
        for (int dz = -1; dz <= 1; ++dz)
            for (int dx = -1; dx <= 1; ++dx)
                for (int dy = -1; dy <= 1; ++dy, ++tap)
                    out[int64_t(tap) * N + p] = resolve(a, cml, l, z + dz, x + dx, y + dy);
    });
}

// conv.hpp:83-195 (Convolution<3,3,3>::forward_impl) + helpers.hpp:505-575 (accumulate_convolution).
// Weights use the CUDA layout (L, Cout, Cin, 3, 3, 3) (pyapr/aprnet/cuda/conv.py:77); the stencil for
// level l is slot min(cml - l, L - 1) (conv.hpp:124).  Correlation, taps ordered (z, x, y).
template<typename T>
void conv333_forward(const Apr& a, int dl, int Cin, int Cout, int L, const T* in, const T* w, T* out) {
    const int cml = a.level_max() - dl;
    const int64_t N = a.number_parts(dl), TS = a.tree_size(dl);
    std::vector<int32_t> nb(27 * N);
    nbr_table(a, dl, nb.data());
    std::vector<uint8_t> sten(N);
    for_each_output(a, dl, [&](int64_t p, int l, int, int, int) { sten[p] = (uint8_t) std::min(cml - l, L - 1); });
    std::fill(out, out + int64_t(Cout) * N, T(0));
    std::vector<T> tree(std::max<int64_t>(TS, 1));
    for (int ci = 0; ci < Cin; ++ci) {                           // ch_in outermost, as conv.hpp:107
        const T* xin = in + int64_t(ci) * N;
        fill_tree_mean(a, dl, xin, tree.data());
#pragma omp parallel for schedule(static)
        for (int64_t p = 0; p < N; ++p) {
            T v[27];
            for (int t = 0; t < 27; ++t) {
                const int32_t q = nb[int64_t(t) * N + p];
                v[t] = q >= 0 ? xin[q] : (q == NONE ? T(0) : tree[-2 - q]);
            }
            for (int co = 0; co < Cout; ++co) {
                const T* wp = w + ((int64_t(sten[p]) * Cout + co) * Cin + ci) * 27;
                T res = 0;
                for (int t = 0; t < 27; ++t) res += v[t] * wp[t];
                out[int64_t(co) * N + p] += res;
            }
        }
    }
}

// conv.hpp:289-481 (backward_impl) + helpers.hpp:423-478,578-648: adjoint of the gather, then
// fill_tree_mean_backward folds the tree gradient into the particle gradient (conv.hpp:478).
template<typename T>
void conv333_backward(const Apr& a, int dl, int Cin, int Cout, int L, const T* in, const T* w,
                      const T* gout, T* gin, T* gw) {
    const int cml = a.level_max() - dl;
    const int64_t N = a.number_parts(dl), TS = a.tree_size(dl);
    std::vector<int32_t> nb(27 * N);
    nbr_table(a, dl, nb.data());
    std::vector<uint8_t> sten(N);
    for_each_output(a, dl, [&](int64_t p, int l, int, int, int) { sten[p] = (uint8_t) std::min(cml - l, L - 1); });
    std::fill(gin, gin + int64_t(Cin) * N, T(0));
    std::fill(gw, gw + int64_t(L) * Cout * Cin * 27, T(0));
    std::vector<T> tree(std::max<int64_t>(TS, 1)), gtree(std::max<int64_t>(TS, 1));
    for (int ci = 0; ci < Cin; ++ci) {
        const T* xin = in + int64_t(ci) * N;
        T* g = gin + int64_t(ci) * N;
        fill_tree_mean(a, dl, xin, tree.data());
        std::fill(gtree.begin(), gtree.end(), T(0));
        for (int64_t p = 0; p < N; ++p) {
            T v[27];
            for (int t = 0; t < 27; ++t) {
                const int32_t q = nb[int64_t(t) * N + p];
                v[t] = q >= 0 ? xin[q] : (q == NONE ? T(0) : tree[-2 - q]);
            }
            T gv[27];
            for (int t = 0; t < 27; ++t) gv[t] = 0;
            for (int co = 0; co < Cout; ++co) {
                const T dO = gout[int64_t(co) * N + p];
                const int64_t wo = ((int64_t(sten[p]) * Cout + co) * Cin + ci) * 27;
                for (int t = 0; t < 27; ++t) { gv[t] += dO * w[wo + t]; gw[wo + t] += dO * v[t]; }
            }
            for (int t = 0; t < 27; ++t) {
                const int32_t q = nb[int64_t(t) * N + p];
                if (q >= 0) g[q] += gv[t]; else if (q != NONE) gtree[-2 - q] += gv[t];
            }
        }
        fill_tree_mean_backward(a, dl, g, gtree.data());
    }
}

// conv.hpp:199-256 (Convolution<1,1,1>::forward_impl): per-level channel mix; upgraded nodes use
// stencil 0 (:241-251).  Weights (S, Cout, Cin) in the CUDA layout.
inline int stencil_of_index(const Apr& a, int cml, int S, int64_t p) {
    for (int l = cml; l >= a.level_min(); --l)
        if (p >= a.parts.level_begin(l) && p < a.parts.level_end(l)) return std::min(S - 1, cml - l);
    return 0;   // upgraded tree nodes
}

template<typename T>
void conv111_forward(const Apr& a, int dl, int Cin, int Cout, int S, const T* in, const T* w, T* out) {
    const int cml = a.level_max() - dl;
    const int64_t N = a.number_parts(dl);
    std::fill(out, out + int64_t(Cout) * N, T(0));
    for (int co = 0; co < Cout; ++co)
        for (int ci = 0; ci < Cin; ++ci)
            for (int64_t p = 0; p < N; ++p) {
                const int s = stencil_of_index(a, cml, S, p);
                out[int64_t(co) * N + p] += w[(int64_t(s) * Cout + co) * Cin + ci] * in[int64_t(ci) * N + p];
            }
}

// conv.hpp:484-554
template<typename T>
void conv111_backward(const Apr& a, int dl, int Cin, int Cout, int S, const T* in, const T* w,
                      const T* gout, T* gin, T* gw) {
    const int cml = a.level_max() - dl;
    const int64_t N = a.number_parts(dl);
    std::fill(gin, gin + int64_t(Cin) * N, T(0));
    std::fill(gw, gw + int64_t(S) * Cout * Cin, T(0));
    std::vector<int> st(N);
    for (int64_t p = 0; p < N; ++p) st[p] = stencil_of_index(a, cml, S, p);
    for (int ci = 0; ci < Cin; ++ci)
        for (int co = 0; co < Cout; ++co)
            for (int64_t p = 0; p < N; ++p) {
                const int64_t wi = (int64_t(st[p]) * Cout + co) * Cin + ci;
                gw[wi] += in[int64_t(ci) * N + p] * gout[int64_t(co) * N + p];
                gin[int64_t(ci) * N + p] += w[wi] * gout[int64_t(co) * N + p];
            }
}

// kernel.hpp:54-128 (RestrictKernel<3,3,3>::forward_impl): slots < S copied; slot k >= S is the last
// given stencil box-averaged onto a grid 2^(k-S+1) times coarser.  `CC` = Cout*Cin filters, each 27.
template<typename T>
void restrict333(int S, int L, int64_t CC, const T* w, T* out, bool backward) {
    // forward: out (L, CC, 27) from w (S, CC, 27); backward: out (S, CC, 27) from w (L, CC, 27)
    const int n_in = backward ? L : S, n_out = backward ? S : L;
    (void) n_in;
    std::fill(out, out + int64_t(n_out) * CC * 27, T(0));
    for (int k = 0; k < S; ++k)
        for (int64_t i = 0; i < CC * 27; ++i) out[int64_t(k) * CC * 27 + i] = w[int64_t(k) * CC * 27 + i];
    const int src = S - 1;
    for (int k = S; k < L; ++k) {
        const int step = 1 << (k - src);
        const float factor = float(step) * float(step) * float(step);
        const int off = step - 1;                                   // (3/2)*step - 3/2
        for (int zi = 0; zi < 3; ++zi) for (int xi = 0; xi < 3; ++xi) for (int yi = 0; yi < 3; ++yi)
            for (int zo = 0; zo < 3; ++zo) {
                const float oz = float(std::min((zo + 1) * step, off + zi + step) - std::max(zo * step, off + zi));
                if (oz <= 0) continue;
                for (int xo = 0; xo < 3; ++xo) {
                    const float ox = float(std::min((xo + 1) * step, off + xi + step) - std::max(xo * step, off + xi));
                    if (ox <= 0) continue;
                    for (int yo = 0; yo < 3; ++yo) {
                        const float oy = float(std::min((yo + 1) * step, off + yi + step) - std::max(yo * step, off + yi));
                        if (oy <= 0) continue;
                        const float ov = ox * oy * oz / factor;
                        const int ti = (zi * 3 + xi) * 3 + yi, to = (zo * 3 + xo) * 3 + yo;
                        for (int64_t c = 0; c < CC; ++c) {
                            if (!backward) out[(int64_t(k) * CC + c) * 27 + to] += ov * w[(int64_t(src) * CC + c) * 27 + ti];
                            else           out[(int64_t(src) * CC + c) * 27 + ti] += ov * w[(int64_t(k) * CC + c) * 27 + to];
                        }
                    }
                }
            }
    }
}

// maxpool.hpp:70-147 (MaxPool::forward_impl).  Output initialised to -1e17 and indices to 0 (:51-52);
// strict '>' so the first maximum in visiting order wins: all APR-particle children in (z, x, y) row
// order (:105-117), then all upgraded-node children in the same order (:122-142).
template<typename T>
void maxpool_forward(const Apr& a, int dl, int C, const T* in, T* out, int64_t* idx) {
    const int cml = a.level_max() - dl;
    const int64_t N = a.number_parts(dl), M = a.number_parts(dl + 1);
    const int64_t ncopy = a.parts.level_end(cml - 1);
    const int64_t out_off = a.tree_offset(cml - 1);
    for (int c = 0; c < C; ++c) {
        const T* x = in + int64_t(c) * N; T* o = out + int64_t(c) * M; int64_t* ix = idx + int64_t(c) * M;
        for (int64_t i = 0; i < M; ++i) { o[i] = T(-1e17f); ix[i] = 0; }
        for (int64_t i = 0; i < ncopy; ++i) o[i] = x[i];
        for_each_link(a.parts, a.tree, cml, [&](int64_t ch, int64_t p, float) {
            if (x[ch] > o[p + out_off]) { o[p + out_off] = x[ch]; ix[p + out_off] = ch; }
        });
        if (cml < a.level_max()) {
            const int64_t in_off = a.tree_offset(cml);
            for_each_link(a.tree, a.tree, cml, [&](int64_t ch, int64_t p, float) {
                if (x[ch + in_off] > o[p + out_off]) { o[p + out_off] = x[ch + in_off]; ix[p + out_off] = ch + in_off; }
            });
        }
    }
}

// maxpool.hpp:176-230 (backward_impl): copy for kept particles, scatter through max_indices otherwise
template<typename T>
void maxpool_backward(const Apr& a, int dl, int C, const T* gout, const int64_t* idx, T* gin) {
    const int cml = a.level_max() - dl;
    const int64_t N = a.number_parts(dl), M = a.number_parts(dl + 1);
    const int64_t nfixed = a.parts.level_end(cml - 1);
    for (int c = 0; c < C; ++c) {
        T* g = gin + int64_t(c) * N; const T* go = gout + int64_t(c) * M; const int64_t* ix = idx + int64_t(c) * M;
        std::fill(g, g + N, T(0));
        for (int64_t i = 0; i < nfixed; ++i) g[i] = go[i];
        for (int64_t i = nfixed; i < M; ++i) g[ix[i]] = go[i];
    }
}

// upsample.hpp:70-142 (UpSampleConst::forward_impl): dl -> dl-1, children take the parent's value
template<typename T>
void upsample_forward(const Apr& a, int dl, int C, const T* in, T* out) {
    const int in_max = a.level_max() - dl, out_max = in_max + 1;
    const int64_t N = a.number_parts(dl), M = a.number_parts(dl - 1);
    const int64_t ncopy = a.parts.level_end(in_max);
    const int64_t in_off = a.tree_offset(in_max);
    for (int c = 0; c < C; ++c) {
        const T* x = in + int64_t(c) * N; T* o = out + int64_t(c) * M;
        std::fill(o, o + M, T(0));
        for (int64_t i = 0; i < ncopy; ++i) o[i] = x[i];
        for_each_link(a.parts, a.tree, out_max, [&](int64_t ch, int64_t p, float) { o[ch] = x[p + in_off]; });
        if (out_max <= a.tree.level_max) {
            const int64_t out_off = a.tree_offset(out_max);
            for_each_link(a.tree, a.tree, out_max, [&](int64_t ch, int64_t p, float) { o[ch + out_off] = x[p + in_off]; });
        }
    }
}

// upsample.hpp:166-236 (backward_impl): parents sum their children's gradients
template<typename T>
void upsample_backward(const Apr& a, int dl, int C, const T* gout, T* gin) {
    const int in_max = a.level_max() - dl, out_max = in_max + 1;
    const int64_t N = a.number_parts(dl), M = a.number_parts(dl - 1);
    const int64_t ncopy = a.parts.level_end(in_max);
    const int64_t in_off = a.tree_offset(in_max);
    for (int c = 0; c < C; ++c) {
        T* g = gin + int64_t(c) * N; const T* go = gout + int64_t(c) * M;
        std::fill(g, g + N, T(0));
        for (int64_t i = 0; i < ncopy; ++i) g[i] = go[i];
        for_each_link(a.parts, a.tree, out_max, [&](int64_t ch, int64_t p, float) { g[p + in_off] += go[ch]; });
        if (out_max <= a.tree.level_max) {
            const int64_t out_off = a.tree_offset(out_max);
            for_each_link(a.tree, a.tree, out_max, [&](int64_t ch, int64_t p, float) { g[p + in_off] += go[ch + out_off]; });
        }
    }
}

// pyapr/tree/fill_tree.py:46-71 -> LibAPR APRTreeNumerics::fill_tree_max (source absent from the
// reference checkout: PARITY UNPINNED for interior nodes).  Restated as: every tree node holds the
// maximum over its descendants; pinned only by pyapr/tests/test_tree.py:39-40 (root == global max).
template<typename T>
void fill_tree_max(const Apr& a, const T* in, T* tree) {
    const int64_t TS = a.tree.level_end(a.tree.level_max);
    std::vector<uint8_t> seen(TS, 0);
    auto upd = [&](int64_t p, T v) { if (!seen[p] || v > tree[p]) { tree[p] = v; seen[p] = 1; } };
    for (int l = a.level_max(); l >= a.level_min(); --l)
        for_each_link(a.parts, a.tree, l, [&](int64_t c, int64_t p, float) { upd(p, in[c]); });
    for (int l = a.tree.level_max; l > a.tree.level_min; --l)
        for_each_link(a.tree, a.tree, l, [&](int64_t c, int64_t p, float) { upd(p, tree[c]); });
}

} // namespace

extern "C" {

void* orc_apr_create(int level_min, int level_max, const int* dims_zxy, const int64_t* row_ptr, int64_t n_rows,
                     const uint16_t* y, int64_t n, const int64_t* tree_row_ptr, int64_t n_tree_rows,
                     const uint16_t* tree_y, int64_t nt) {
    Apr* a = new Apr();
    a->rp.assign(row_ptr, row_ptr + n_rows + 1);
    a->yv.assign(y, y + n);
    a->trp.assign(tree_row_ptr, tree_row_ptr + n_tree_rows + 1);
    a->tyv.assign(tree_y, tree_y + nt);
    a->parts.init(level_min, level_max, dims_zxy, a->rp.data(), a->yv.data());
    a->tree.init(level_min - 1, level_max - 1, dims_zxy, a->trp.data(), a->tyv.data());
    return a;
}
void orc_apr_destroy(void* h) { delete (Apr*) h; }
int64_t orc_number_parts(void* h, int dl) { return ((Apr*) h)->number_parts(dl); }
int64_t orc_tree_size(void* h, int dl) { return ((Apr*) h)->tree_size(dl); }
int64_t orc_tree_offset(void* h, int level) { return ((Apr*) h)->tree_offset(level); }
void orc_nbr_table(void* h, int dl, int32_t* out) { nbr_table(*(Apr*) h, dl, out); }

// child table of every tree node: slot (dz*2+dx)*2+dy; >=0 particle index, <=-2 tree node, -1 none
void orc_child_table(void* h, int32_t* out) {
    const Apr& a = *(Apr*) h;
    const Access& T = a.tree;
    const int64_t TS = T.level_end(T.level_max);
    for (int l = T.level_min; l <= T.level_max; ++l)
        for (int z = 0; z < T.z_num[l]; ++z)
            for (int x = 0; x < T.x_num[l]; ++x) {
                const int64_t r = T.row(l, z, x);
                for (int64_t t = T.row_ptr[r]; t < T.row_ptr[r + 1]; ++t)
                    for (int s = 0; s < 8; ++s) {
                        const int cz = 2 * z + (s >> 2), cx = 2 * x + ((s >> 1) & 1), cy = 2 * T.y[t] + (s & 1);
                        int64_t i = a.parts.find(l + 1, cz, cx, cy);
                        int32_t v = NONE;
                        if (i >= 0) v = (int32_t) i;
                        else if (l + 1 <= T.level_max) { i = T.find(l + 1, cz, cx, cy); if (i >= 0) v = enc_tree(i); }
                        out[int64_t(s) * TS + t] = v;
                    }
            }
}

#define ORC_EXPORT(T, SFX)                                                                                   \
void orc_fill_tree_mean_##SFX(void* h, int dl, int C, const T* in, T* tree) {                                \
    const Apr& a = *(Apr*) h; const int64_t N = a.number_parts(dl), TS = a.tree_size(dl);                   \
    for (int c = 0; c < C; ++c) fill_tree_mean(a, dl, in + c * N, tree + c * TS); }                         \
void orc_fill_tree_mean_backward_##SFX(void* h, int dl, int C, T* gin, T* gtree) {                          \
    const Apr& a = *(Apr*) h; const int64_t N = a.number_parts(dl), TS = a.tree_size(dl);                   \
    for (int c = 0; c < C; ++c) fill_tree_mean_backward(a, dl, gin + c * N, gtree + c * TS); }              \
void orc_fill_tree_max_##SFX(void* h, const T* in, T* tree) { fill_tree_max(*(Apr*) h, in, tree); }          \
void orc_conv333_forward_##SFX(void* h, int dl, int Cin, int Cout, int L, const T* in, const T* w, T* out) { \
    conv333_forward(*(Apr*) h, dl, Cin, Cout, L, in, w, out); }                                              \
void orc_conv333_backward_##SFX(void* h, int dl, int Cin, int Cout, int L, const T* in, const T* w,          \
                                const T* gout, T* gin, T* gw) {                                              \
    conv333_backward(*(Apr*) h, dl, Cin, Cout, L, in, w, gout, gin, gw); }                                   \
void orc_conv111_forward_##SFX(void* h, int dl, int Cin, int Cout, int S, const T* in, const T* w, T* out) { \
    conv111_forward(*(Apr*) h, dl, Cin, Cout, S, in, w, out); }                                              \
void orc_conv111_backward_##SFX(void* h, int dl, int Cin, int Cout, int S, const T* in, const T* w,          \
                                const T* gout, T* gin, T* gw) {                                              \
    conv111_backward(*(Apr*) h, dl, Cin, Cout, S, in, w, gout, gin, gw); }                                   \
void orc_restrict333_forward_##SFX(int S, int L, int64_t CC, const T* w, T* out) { restrict333(S, L, CC, w, out, false); } \
void orc_restrict333_backward_##SFX(int S, int L, int64_t CC, const T* gw, T* out) { restrict333(S, L, CC, gw, out, true); } \
void orc_maxpool_forward_##SFX(void* h, int dl, int C, const T* in, T* out, int64_t* idx) {                  \
    maxpool_forward(*(Apr*) h, dl, C, in, out, idx); }                                                       \
void orc_maxpool_backward_##SFX(void* h, int dl, int C, const T* gout, const int64_t* idx, T* gin) {         \
    maxpool_backward(*(Apr*) h, dl, C, gout, idx, gin); }                                                    \
void orc_upsample_forward_##SFX(void* h, int dl, int C, const T* in, T* out) {                               \
    upsample_forward(*(Apr*) h, dl, C, in, out); }                                                           \
void orc_upsample_backward_##SFX(void* h, int dl, int C, const T* gout, T* gin) {                            \
    upsample_backward(*(Apr*) h, dl, C, gout, gin); }

ORC_EXPORT(float, f32)
ORC_EXPORT(double, f64)

} // extern "C"
