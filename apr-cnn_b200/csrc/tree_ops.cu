// Tree fill (mean / max), max pooling and constant up-sampling.
//
// All four are child <-> parent transfers along the APR tree.  They run as index-driven gathers over
// the cached child table: one thread per parent tree node, eight child slots, channels looped inside
// the thread so the indices are read once.  Consecutive threads hold consecutive nodes of a sparse
// row, whose children are consecutive in the child rows, so the value accesses coalesce.  The adjoint of the
// tree mean is the exception: it runs child-centric over cached parent tables (see its kernel).
// Arithmetic follows pyapr/aprnet/src/helpers.hpp:156-350 (tree mean and its adjoint),
// pyapr/aprnet/src/maxpool.hpp:70-230 and pyapr/aprnet/src/upsample.hpp:70-236.
#include "apr_device.cuh"

namespace {

typedef long long ll;
constexpr int TPB = 256;                 // threads (= parent nodes) per block
constexpr int CH_PER_BLOCK = 8;          // channels a block loops over with the child slots resolved once

template<typename T> struct DT;
template<> struct DT<float> { static constexpr int id = APRNET_F32; };
template<> struct DT<double> { static constexpr int id = APRNET_F64; };

// parent level lp: tree[t] = scale[t] * sum(children).  All child values of the block's channels are
// requested before any is used (CH_PER_BLOCK x 8 independent loads in flight per thread).
template<typename T>
__global__ void __launch_bounds__(TPB) tree_mean_level_kernel(const int32_t* __restrict__ child, const float* __restrict__ scale, ll n_tree,
                                       ll tb, ll te, const T* __restrict__ in, ll ld_in, T* __restrict__ tree,
                                       ll ld_tree, int C, ll up_off, int use_up) {
    const ll t = tb + (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= te) return;
    // resolve the eight child slots once: pointer to the child's value in channel c0 and the channel stride
    const int c0 = blockIdx.y * CH_PER_BLOCK;
    const T* src[8];
    unsigned coded = 0;                 // slots whose child is a tree node (summed after the particles)
    const unsigned in_tree = use_up ? 0u : 0xffu;      // coded children live in the tree scratch unless they are upgraded nodes
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        const int32_t v = child[(ll) s * n_tree + t];
        src[s] = nullptr;
        if (v >= 0) src[s] = in + (ll) c0 * ld_in + v;
        else if (v != APRNET_NONE) {
            coded |= 1u << s;
            src[s] = use_up ? in + (ll) c0 * ld_in + aprnet_dec_tree(v) + up_off : tree + (ll) c0 * ld_tree + aprnet_dec_tree(v);
        }
    }
    const T f = (T) scale[t];
    const int nch = min(CH_PER_BLOCK, C - c0);
    T vals[CH_PER_BLOCK][8];
#pragma unroll
    for (int k = 0; k < CH_PER_BLOCK; ++k) {
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            vals[k][s] = (src[s] && k < nch) ? *src[s] : T(0);
            src[s] += (coded & in_tree) >> s & 1 ? ld_tree : ld_in;
        }
    }
    T* dst = tree + (ll) c0 * ld_tree + t;
#pragma unroll
    for (int k = 0; k < CH_PER_BLOCK; ++k) {
        if (k >= nch) break;
        T s_part = 0, s_tree = 0;       // particles first, then tree children (fixed order)
#pragma unroll
        for (int s = 0; s < 8; ++s) { if (coded >> s & 1) s_tree += vals[k][s]; else s_part += vals[k][s]; }
        dst[(ll) k * ld_tree] = f * (s_part + s_tree);
    }
}

// Adjoint, child-centric: entry u of `dst` (a tree node of one level, or a feature location) receives
// scale[t] * grad_tree[t] of its parent node t = parent[u].  One thread per child and CH_PER_BLOCK channels: the child
// axis is streamed (coalesced read-modify-write, one writer per entry), the parents' values come from a few cache lines
// per warp.  The parent-centric form (one thread per parent, eight scattered children) touched every sector of the
// gradient half at a time and ran at half this speed.  dst and gtree may be the same array (node levels): a level only
// reads the level above it.
template<typename T>
__global__ void __launch_bounds__(TPB) tree_mean_backward_children_kernel(const int32_t* __restrict__ parent, const float* __restrict__ scale,
                                                                          ll ub, ll ue, T* dst, ll ld_dst, const T* gtree, ll ld_tree, int C) {
    const ll u = ub + (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (u >= ue) return;
    const int c0 = blockIdx.y * CH_PER_BLOCK;
    T old[CH_PER_BLOCK];
#pragma unroll
    for (int k = 0; k < CH_PER_BLOCK; ++k) old[k] = dst[(ll) min(c0 + k, C - 1) * ld_dst + u];        // independent of the parent
    const int32_t t = parent[u];
    if (t < 0) return;
    const T f = (T) scale[t];
    T g[CH_PER_BLOCK];
#pragma unroll
    for (int k = 0; k < CH_PER_BLOCK; ++k) g[k] = gtree[(ll) min(c0 + k, C - 1) * ld_tree + t];
#pragma unroll
    for (int k = 0; k < CH_PER_BLOCK; ++k)
        if (c0 + k < C) dst[(ll) (c0 + k) * ld_dst + u] = old[k] + f * g[k];
}

template<typename T>
__global__ void tree_max_level_kernel(const int32_t* __restrict__ child, ll n_tree, ll tb, ll te,
                                      const T* __restrict__ in, ll ld_in, T* __restrict__ tree, ll ld_tree, int C) {
    const ll t = tb + (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= te) return;
    int32_t ch[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) ch[s] = child[(ll) s * n_tree + t];
    const int c0 = blockIdx.y * CH_PER_BLOCK, c1 = min(C, c0 + CH_PER_BLOCK);
    for (int c = c0; c < c1; ++c) {
        const T* x = in + (ll) c * ld_in;
        const T* tr = tree + (ll) c * ld_tree;
        bool seen = false;
        T best = 0;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const int32_t v = ch[s];
            if (v == APRNET_NONE) continue;
            const T val = v >= 0 ? x[v] : tr[aprnet_dec_tree(v)];
            if (!seen || val > best) { best = val; seen = true; }
        }
        tree[(ll) c * ld_tree + t] = best;
    }
}

// Max pooling: one thread per tree node of level cml-1.  Visiting order = APR-particle children in
// slot order (dz, dx, dy), then upgraded-node children in slot order; strict '>' against an initial
// -1e17 with index 0 (pyapr/aprnet/src/maxpool.hpp:51-52,105-142).
template<typename T>
__global__ void maxpool_kernel(const int32_t* __restrict__ child, ll n_tree, ll tb, ll te, ll out_off,
                               const T* __restrict__ in, ll ld_in, T* __restrict__ out, long long* __restrict__ idx,
                               ll ld_out, int C, ll up_off) {
    const ll t = tb + (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= te) return;
    int32_t ch[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) ch[s] = child[(ll) s * n_tree + t];
    const int c0 = blockIdx.y * CH_PER_BLOCK, c1 = min(C, c0 + CH_PER_BLOCK);
    for (int c = c0; c < c1; ++c) {
        const T* x = in + (ll) c * ld_in;
        T best = (T) -1e17f;
        ll arg = 0;
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const int32_t v = ch[s];
            if (v >= 0) { const T val = x[v]; if (val > best) { best = val; arg = v; } }
        }
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const int32_t v = ch[s];
            if (v < APRNET_NONE) { const ll q = aprnet_dec_tree(v) + up_off; const T val = x[q]; if (val > best) { best = val; arg = q; } }
        }
        out[(ll) c * ld_out + t + out_off] = best;
        idx[(ll) c * ld_out + t + out_off] = arg;
    }
}

template<typename T>
__global__ void maxpool_backward_kernel(const T* __restrict__ gout, const long long* __restrict__ idx, ll ld_out,
                                        T* __restrict__ gin, ll ld_in, ll nfixed, ll m, int C) {
    const ll i = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= m) return;
    const int c0 = blockIdx.y * CH_PER_BLOCK, c1 = min(C, c0 + CH_PER_BLOCK);
    for (int c = c0; c < c1; ++c) {
        const T g = gout[(ll) c * ld_out + i];
        const ll dst = i < nfixed ? i : idx[(ll) c * ld_out + i];
        gin[(ll) c * ld_in + dst] = g;
    }
}

// Up-sampling: one thread per tree node t of the input's max level; its stored value sits at
// t + in_off; children are APR particles of the next level or its tree nodes (stored at + out_off).
template<typename T, bool BACKWARD>
__global__ void upsample_kernel(const int32_t* __restrict__ child, ll n_tree, ll tb, ll te, ll in_off, ll out_off,
                                const T* __restrict__ src, ll ld_src, T* __restrict__ dst, ll ld_dst, int C) {
    const ll t = tb + (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= te) return;
    int32_t ch[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) ch[s] = child[(ll) s * n_tree + t];
    const int c0 = blockIdx.y * CH_PER_BLOCK, c1 = min(C, c0 + CH_PER_BLOCK);
    for (int c = c0; c < c1; ++c) {
        if (!BACKWARD) {        // src = input (coarse), dst = output (fine)
            const T v = src[(ll) c * ld_src + t + in_off];
            T* o = dst + (ll) c * ld_dst;
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                const int32_t q = ch[s];
                if (q >= 0) o[q] = v; else if (q != APRNET_NONE) o[aprnet_dec_tree(q) + out_off] = v;
            }
        } else {                // src = grad_output (fine), dst = grad_input (coarse)
            const T* go = src + (ll) c * ld_src;
            T s_part = 0, s_tree = 0;
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                const int32_t q = ch[s];
                if (q >= 0) s_part += go[q]; else if (q != APRNET_NONE) s_tree += go[aprnet_dec_tree(q) + out_off];
            }
            dst[(ll) c * ld_dst + t + in_off] = s_part + s_tree;
        }
    }
}

inline dim3 node_grid(ll count, int C) { return dim3((unsigned) aprnet_ceil_div(count, TPB), (unsigned) aprnet_ceil_div(C, CH_PER_BLOCK)); }

template<typename T>
int copy_rows(T* dst, ll ld_dst, const T* src, ll ld_src, ll count, int C, cudaStream_t st) {
    if (count <= 0 || C <= 0) return APRNET_OK;
    APRNET_CUDA_CHECK(cudaMemcpy2DAsync(dst, (size_t) ld_dst * sizeof(T), src, (size_t) ld_src * sizeof(T),
                                        (size_t) count * sizeof(T), (size_t) C, cudaMemcpyDeviceToDevice, st));
    return APRNET_OK;
}

template<typename T>
int fill_tree_mean_fwd(const aprnet_apr* a, int dl, int C, const T* in, ll ld_in, T* tree, ll ld_tree, cudaStream_t st) {
    const LevelMeta& m = a->meta;
    const int cml = a->cml(dl);
    const ll up = (dl > 0) ? a->tree_offset(cml) : 0;
    for (int lp = cml - 1; lp >= m.level_min - 1; --lp) {
        const ll tb = m.tlvl_begin[lp], te = m.tlvl_begin[lp + 1];
        if (te <= tb) continue;
        { AprnetProfScope _prof("tree_mean_fwd", st);
        tree_mean_level_kernel<T><<<node_grid(te - tb, C), TPB, 0, st>>>(a->child, a->tree_scale, a->n_tree, tb, te, in,
                                                                          ld_in, tree, ld_tree, C, up, (dl > 0 && lp + 1 == cml) ? 1 : 0);
        }
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

template<typename T>
int fill_tree_mean_bwd(const aprnet_apr* a, int dl, int C, T* gin, ll ld_in, T* gtree, ll ld_tree, cudaStream_t st) {
    const LevelMeta& m = a->meta;
    const int cml = a->cml(dl);
    const int32_t* node_parent = aprnet_node_parent_table(a, st);
    const int32_t* loc_parent = aprnet_loc_parent_table(a, dl, st);
    if (!node_parent || !loc_parent) return APRNET_ERR_CUDA;
    // tree nodes, coarse to fine: level l receives from level l - 1, whose gradient is complete by then
    for (int l = m.level_min; l <= cml - 1; ++l) {
        const ll ub = m.tlvl_begin[l], ue = m.tlvl_begin[l + 1];
        if (ue <= ub) continue;
        AprnetProfScope _prof("tree_mean_bwd", st);
        tree_mean_backward_children_kernel<T><<<node_grid(ue - ub, C), TPB, 0, st>>>(node_parent, a->tree_scale, ub, ue, gtree, ld_tree, gtree, ld_tree, C);
    }
    // then every feature location (particles of all levels, upgraded nodes) from its parent node
    const ll n = a->number_parts(dl);
    if (n > 0) {
        AprnetProfScope _prof("tree_mean_bwd", st);
        tree_mean_backward_children_kernel<T><<<node_grid(n, C), TPB, 0, st>>>(loc_parent, a->tree_scale, 0, n, gin, ld_in, gtree, ld_tree, C);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

template<typename T>
int fill_tree_max_impl(const aprnet_apr* a, int C, const T* in, ll ld_in, T* tree, ll ld_tree, cudaStream_t st) {
    const LevelMeta& m = a->meta;
    for (int lp = m.level_max - 1; lp >= m.level_min - 1; --lp) {
        const ll tb = m.tlvl_begin[lp], te = m.tlvl_begin[lp + 1];
        if (te <= tb) continue;
        { AprnetProfScope _prof("tree_max", st);
        tree_max_level_kernel<T><<<node_grid(te - tb, C), TPB, 0, st>>>(a->child, a->n_tree, tb, te, in, ld_in, tree, ld_tree, C);
        }
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

template<typename T>
int maxpool_fwd(const aprnet_apr* a, int dl, int C, const T* in, ll ld_in, T* out, long long* idx, ll ld_out, cudaStream_t st) {
    const LevelMeta& m = a->meta;
    const int cml = a->cml(dl);
    const ll ncopy = m.lvl_begin[cml];                       // particles of levels <= cml-1
    int rc = copy_rows(out, ld_out, in, ld_in, ncopy, C, st);
    if (rc) return rc;
    const ll tb = m.tlvl_begin[cml - 1], te = m.tlvl_begin[cml];
    if (te > tb) {
        const ll up = (dl > 0) ? a->tree_offset(cml) : 0;
        { AprnetProfScope _prof("maxpool_fwd", st);
        maxpool_kernel<T><<<node_grid(te - tb, C), TPB, 0, st>>>(a->child, a->n_tree, tb, te, a->tree_offset(cml - 1), in,
                                                                  ld_in, out, idx, ld_out, C, up);
        }
        APRNET_LAUNCH_CHECK();
    }
    return APRNET_OK;
}

template<typename T>
int maxpool_bwd(const aprnet_apr* a, int dl, int C, const T* gout, const long long* idx, ll ld_out, T* gin, ll ld_in, cudaStream_t st) {
    const ll mcount = a->number_parts(dl + 1);
    const ll nfixed = a->meta.lvl_begin[a->cml(dl)];
    if (mcount > 0) {
        { AprnetProfScope _prof("maxpool_bwd", st);
        maxpool_backward_kernel<T><<<node_grid(mcount, C), TPB, 0, st>>>(gout, idx, ld_out, gin, ld_in, nfixed, mcount, C);
        }
        APRNET_LAUNCH_CHECK();
    }
    return APRNET_OK;
}

template<typename T, bool BACKWARD>
int upsample_impl(const aprnet_apr* a, int dl, int C, const T* src, ll ld_src, T* dst, ll ld_dst, cudaStream_t st) {
    const LevelMeta& m = a->meta;
    const int in_max = a->cml(dl), out_max = in_max + 1;
    const ll ncopy = m.lvl_begin[in_max + 1];                // particles of levels <= in_max
    int rc = copy_rows(dst, ld_dst, src, ld_src, ncopy, C, st);
    if (rc) return rc;
    const ll tb = m.tlvl_begin[in_max], te = m.tlvl_begin[in_max + 1];
    if (te > tb) {
        const ll out_off = (out_max <= m.level_max - 1) ? a->tree_offset(out_max) : 0;
        { AprnetProfScope _prof("upsample", st);
        upsample_kernel<T, BACKWARD><<<node_grid(te - tb, C), TPB, 0, st>>>(a->child, a->n_tree, tb, te, a->tree_offset(in_max),
                                                                             out_off, src, ld_src, dst, ld_dst, C);
        }
        APRNET_LAUNCH_CHECK();
    }
    return APRNET_OK;
}

} // namespace

#define DISPATCH(dtype, CALL_F, CALL_D)                                                   \
    switch (dtype) {                                                                      \
        case APRNET_F32: return CALL_F;                                                   \
        case APRNET_F64: return CALL_D;                                                   \
        default: aprnet_set_error("%s: unknown dtype %d", __func__, dtype); return APRNET_ERR_ARG; \
    }

extern "C" int aprnet_fill_tree_mean_forward(const aprnet_apr* a, int dl, int dtype, int C, const void* in, int64_t ld_in,
                                             void* tree, int64_t ld_tree, void* stream) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && in && tree && C > 0, "bad argument");
    APRNET_DEVICE_CHECK(a);
    APRNET_ARG_CHECK(ld_in >= a->number_parts(dl) && ld_tree >= a->tree_size(dl), "leading dimension too small");
    cudaStream_t st = (cudaStream_t) stream;
    DISPATCH(dtype, fill_tree_mean_fwd<float>(a, dl, C, (const float*) in, ld_in, (float*) tree, ld_tree, st),
             fill_tree_mean_fwd<double>(a, dl, C, (const double*) in, ld_in, (double*) tree, ld_tree, st));
}

extern "C" int aprnet_fill_tree_mean_full(const aprnet_apr* a, int dtype, int C, const void* in, int64_t ld_in, void* tree,
                                          int64_t ld_tree, void* stream) {
    return aprnet_fill_tree_mean_forward(a, 0, dtype, C, in, ld_in, tree, ld_tree, stream);
}

extern "C" int aprnet_fill_tree_mean_backward(const aprnet_apr* a, int dl, int dtype, int C, void* gin, int64_t ld_in,
                                              void* gtree, int64_t ld_tree, void* stream) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && gin && gtree && C > 0, "bad argument");
    APRNET_DEVICE_CHECK(a);
    APRNET_ARG_CHECK(ld_in >= a->number_parts(dl) && ld_tree >= a->tree_size(dl), "leading dimension too small");
    cudaStream_t st = (cudaStream_t) stream;
    DISPATCH(dtype, fill_tree_mean_bwd<float>(a, dl, C, (float*) gin, ld_in, (float*) gtree, ld_tree, st),
             fill_tree_mean_bwd<double>(a, dl, C, (double*) gin, ld_in, (double*) gtree, ld_tree, st));
}

extern "C" int aprnet_fill_tree_max(const aprnet_apr* a, int dtype, int C, const void* in, int64_t ld_in, void* tree,
                                    int64_t ld_tree, void* stream) {
    APRNET_ARG_CHECK(a && in && tree && C > 0, "bad argument");
    APRNET_DEVICE_CHECK(a);
    APRNET_ARG_CHECK(ld_in >= a->n_particles && ld_tree >= a->n_tree, "leading dimension too small");
    cudaStream_t st = (cudaStream_t) stream;
    DISPATCH(dtype, fill_tree_max_impl<float>(a, C, (const float*) in, ld_in, (float*) tree, ld_tree, st),
             fill_tree_max_impl<double>(a, C, (const double*) in, ld_in, (double*) tree, ld_tree, st));
}

extern "C" int aprnet_maxpool_forward(const aprnet_apr* a, int dl, int dtype, int C, const void* in, int64_t ld_in,
                                      void* out, int64_t* idx, int64_t ld_out, void* stream) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && a->valid_dl(dl + 1) && in && out && idx && C > 0, "bad argument");
    APRNET_DEVICE_CHECK(a);
    APRNET_ARG_CHECK(ld_in >= a->number_parts(dl) && ld_out >= a->number_parts(dl + 1), "leading dimension too small");
    cudaStream_t st = (cudaStream_t) stream;
    DISPATCH(dtype, maxpool_fwd<float>(a, dl, C, (const float*) in, ld_in, (float*) out, (long long*) idx, ld_out, st),
             maxpool_fwd<double>(a, dl, C, (const double*) in, ld_in, (double*) out, (long long*) idx, ld_out, st));
}

extern "C" int aprnet_maxpool_backward(const aprnet_apr* a, int dl, int dtype, int C, const void* gout, const int64_t* idx,
                                       int64_t ld_out, void* gin, int64_t ld_in, void* stream) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && a->valid_dl(dl + 1) && gout && gin && idx && C > 0, "bad argument");
    APRNET_DEVICE_CHECK(a);
    APRNET_ARG_CHECK(ld_in >= a->number_parts(dl) && ld_out >= a->number_parts(dl + 1), "leading dimension too small");
    cudaStream_t st = (cudaStream_t) stream;
    DISPATCH(dtype, maxpool_bwd<float>(a, dl, C, (const float*) gout, (const long long*) idx, ld_out, (float*) gin, ld_in, st),
             maxpool_bwd<double>(a, dl, C, (const double*) gout, (const long long*) idx, ld_out, (double*) gin, ld_in, st));
}

extern "C" int aprnet_upsample_forward(const aprnet_apr* a, int dl, int dtype, int C, const void* in, int64_t ld_in, void* out,
                                       int64_t ld_out, void* stream) {
    APRNET_ARG_CHECK(a && dl > 0 && a->valid_dl(dl) && in && out && C > 0, "bad argument (level_delta must be > 0)");
    APRNET_DEVICE_CHECK(a);
    APRNET_ARG_CHECK(ld_in >= a->number_parts(dl) && ld_out >= a->number_parts(dl - 1), "leading dimension too small");
    cudaStream_t st = (cudaStream_t) stream;
    DISPATCH(dtype, (upsample_impl<float, false>(a, dl, C, (const float*) in, ld_in, (float*) out, ld_out, st)),
             (upsample_impl<double, false>(a, dl, C, (const double*) in, ld_in, (double*) out, ld_out, st)));
}

extern "C" int aprnet_upsample_backward(const aprnet_apr* a, int dl, int dtype, int C, const void* gout, int64_t ld_out,
                                        void* gin, int64_t ld_in, void* stream) {
    APRNET_ARG_CHECK(a && dl > 0 && a->valid_dl(dl) && gout && gin && C > 0, "bad argument (level_delta must be > 0)");
    APRNET_DEVICE_CHECK(a);
    APRNET_ARG_CHECK(ld_in >= a->number_parts(dl) && ld_out >= a->number_parts(dl - 1), "leading dimension too small");
    cudaStream_t st = (cudaStream_t) stream;
    DISPATCH(dtype, (upsample_impl<float, true>(a, dl, C, (const float*) gout, ld_out, (float*) gin, ld_in, st)),
             (upsample_impl<double, true>(a, dl, C, (const double*) gout, ld_out, (double*) gin, ld_in, st)));
}
