// 3x3x3 particle convolution: forward, input gradient and weight gradient (CUDA-core path,
// float and double).
//
// Replaces pyapr/aprnet/cuda/src/conv333_gpu.cu and conv333_gpu_backward.cu.  The reference puts the
// input channel in grid.z and combines channels with atomicAdd into a zero-filled output, re-stages a
// dense (z, x, y) patch per block and re-enumerates non-empty tiles on every call.  Here the cell
// resolution is a cached neighbour table (27 int32 per output location, apr_handle.cu), and
//   * forward: one thread owns one output location and a block of output channels, loops over all
//     input channels and taps, and writes each output exactly once;
//   * input gradient: same-level taps are gathered through the mirrored table entry; cross-level taps (parent-level
//     particle, tree node) are pulled per target over the cached edge plan in a fixed order (conv333_cross_pull_kernel;
//     an atomicAdd scatter remains for structures too large for the plan's 32-bit edge ids);
//   * weight gradient: block-local partial sums in registers over a contiguous particle range,
//     written to a workspace and reduced in a fixed order (deterministic).
// Arithmetic: pyapr/aprnet/src/conv.hpp:83-195,289-481 and helpers.hpp:358-478,505-704.
#include "apr_device.cuh"
#include <algorithm>

namespace {

typedef long long ll;
constexpr int MAX_SEGS = APRNET_MAX_LEVELS;

struct SegTable {
    int n;
    ll begin[MAX_SEGS], end[MAX_SEGS];
    int slot[MAX_SEGS];
    int tile_begin[MAX_SEGS + 1];
};

inline SegTable make_seg_table(const std::vector<Segment>& segs, int tile) {
    SegTable t;
    t.n = (int) segs.size();
    t.tile_begin[0] = 0;
    for (int i = 0; i < t.n; ++i) {
        t.begin[i] = segs[i].begin; t.end[i] = segs[i].end; t.slot[i] = segs[i].slot;
        t.tile_begin[i + 1] = t.tile_begin[i] + aprnet_ceil_div(segs[i].end - segs[i].begin, tile);
    }
    return t;
}

template<typename T>
__device__ __forceinline__ T gather_value(const T* __restrict__ x, const T* __restrict__ tree, int32_t q) {
    if (q >= 0) return x[q];
    if (q == APRNET_NONE) return T(0);
    return tree[aprnet_dec_tree(q)];
}

// ---------------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------------
// grid.x: tiles of TPB output locations (never straddling a level), grid.y: blocks of OB output
// channels.  Shared memory holds the weights of the tile's stencil slot for IB input channels at a
// time, laid out [tap][i][o] so that the OB weights of one (tap, i) are read as broadcast vectors.
template<typename T, int OB, int IB, int TPB>
__global__ void __launch_bounds__(TPB) conv333_forward_kernel(SegTable segs, const int32_t* __restrict__ nbr, ll N,
                                                              const T* __restrict__ in, ll ld_in,
                                                              const T* __restrict__ tree, ll ld_tree,
                                                              const T* __restrict__ w, T* __restrict__ out, ll ld_out,
                                                              int cin, int cout) {
    extern __shared__ unsigned char smem_raw[];
    T* wsm = reinterpret_cast<T*>(smem_raw);                      // [27][IB][OB]
    int seg = 0;
    while (seg + 1 < segs.n && (int) blockIdx.x >= segs.tile_begin[seg + 1]) ++seg;
    const ll p = segs.begin[seg] + (ll) (blockIdx.x - segs.tile_begin[seg]) * TPB + threadIdx.x;
    const bool active = p < segs.end[seg];
    const int o0 = blockIdx.y * OB;
    const T* wslot = w + (ll) segs.slot[seg] * cout * cin * 27;

    T acc[OB];
#pragma unroll
    for (int o = 0; o < OB; ++o) acc[o] = 0;

    for (int i0 = 0; i0 < cin; i0 += IB) {
        __syncthreads();
        for (int e = threadIdx.x; e < 27 * IB * OB; e += TPB) {
            const int tap = e % 27, i = (e / 27) % IB, o = e / (27 * IB);       // global reads contiguous in tap
            const bool ok = (o0 + o < cout) && (i0 + i < cin);
            wsm[(tap * IB + i) * OB + o] = ok ? wslot[((ll) (o0 + o) * cin + (i0 + i)) * 27 + tap] : T(0);
        }
        __syncthreads();
        if (!active) continue;
        const int ib = min(IB, cin - i0);
        for (int tap = 0; tap < 27; ++tap) {
            const int32_t q = nbr[(ll) tap * N + p];
            if (q == APRNET_NONE) continue;
            const T* src = (q >= 0) ? (in + (ll) i0 * ld_in + q) : (tree + (ll) i0 * ld_tree + aprnet_dec_tree(q));
            const ll lds = (q >= 0) ? ld_in : ld_tree;
            const T* wt = wsm + tap * IB * OB;
            if (ib == IB) {
                T v[IB];
#pragma unroll
                for (int i = 0; i < IB; ++i) v[i] = src[(ll) i * lds];
#pragma unroll
                for (int i = 0; i < IB; ++i)
#pragma unroll
                    for (int o = 0; o < OB; ++o) acc[o] = fma(v[i], wt[i * OB + o], acc[o]);
            } else {
                for (int i = 0; i < ib; ++i) {
                    const T v = src[(ll) i * lds];
#pragma unroll
                    for (int o = 0; o < OB; ++o) acc[o] = fma(v, wt[i * OB + o], acc[o]);
                }
            }
        }
    }
    if (active) {
#pragma unroll
        for (int o = 0; o < OB; ++o)
            if (o0 + o < cout) out[(ll) (o0 + o) * ld_out + p] = acc[o];
    }
}

// ---------------------------------------------------------------------------------------------
// input gradient
// ---------------------------------------------------------------------------------------------
// Thread = output location q, block of IB input channels (grid.y); output channels staged OB at a
// time.  For tap t (offset d): if the cell at -d holds a same-level output location j (mirrored table
// entry 26 - t) then q receives W[t]^T dO[j]: a gather.  If the cell at +d resolved to a coarser
// particle or a tree node, W[t]^T dO[q] is scattered there with atomicAdd (cross_only = 0 or 1; with cross_only = 2 the
// scatter is left to conv333_cross_pull_kernel).
template<typename T, int OB, int IB, int TPB>
__global__ void __launch_bounds__(TPB) conv333_backward_input_kernel(SegTable segs, const int32_t* __restrict__ nbr, ll N,
                                                                     const T* __restrict__ gout, ll ld_out,
                                                                     const T* __restrict__ w, T* __restrict__ gin, ll ld_in,
                                                                     T* __restrict__ gtree, ll ld_tree, int cin, int cout, int cross_only) {
    extern __shared__ unsigned char smem_raw[];
    T* wsm = reinterpret_cast<T*>(smem_raw);                      // [27][OB][IB]
    int seg = 0;
    while (seg + 1 < segs.n && (int) blockIdx.x >= segs.tile_begin[seg + 1]) ++seg;
    const ll q = segs.begin[seg] + (ll) (blockIdx.x - segs.tile_begin[seg]) * TPB + threadIdx.x;
    const ll lo = segs.begin[seg], hi = segs.end[seg];
    const bool active = q < hi;
    const int i0 = blockIdx.y * IB;
    const T* wslot = w + (ll) segs.slot[seg] * cout * cin * 27;

    T acc[IB];
#pragma unroll
    for (int i = 0; i < IB; ++i) acc[i] = 0;

    for (int o0 = 0; o0 < cout; o0 += OB) {
        __syncthreads();
        for (int e = threadIdx.x; e < 27 * IB * OB; e += TPB) {
            const int tap = e % 27, i = (e / 27) % IB, o = e / (27 * IB);
            const bool ok = (o0 + o < cout) && (i0 + i < cin);
            wsm[(tap * OB + o) * IB + i] = ok ? wslot[((ll) (o0 + o) * cin + (i0 + i)) * 27 + tap] : T(0);
        }
        __syncthreads();
        if (!active) continue;
        const int ob = min(OB, cout - o0);
        for (int tap = 0; tap < 27; ++tap) {
            // gather from the same-level location at the mirrored offset
            const int32_t j = nbr[(ll) (26 - tap) * N + q];
            if (cross_only != 1 && j >= lo && j < hi) {
                const T* g = gout + (ll) o0 * ld_out + j;
                const T* wt = wsm + tap * OB * IB;
                for (int o = 0; o < ob; ++o) {
                    const T d = g[(ll) o * ld_out];
#pragma unroll
                    for (int i = 0; i < IB; ++i) acc[i] = fma(d, wt[o * IB + i], acc[i]);
                }
            }
            // scatter to a cross-level source
            const int32_t t = nbr[(ll) tap * N + q];
            const bool coarser = t >= 0 && t < lo;
            if (cross_only != 2 && (coarser || t < APRNET_NONE)) {
                T s[IB];
#pragma unroll
                for (int i = 0; i < IB; ++i) s[i] = 0;
                const T* g = gout + (ll) o0 * ld_out + q;
                const T* wt = wsm + tap * OB * IB;
                for (int o = 0; o < ob; ++o) {
                    const T d = g[(ll) o * ld_out];
#pragma unroll
                    for (int i = 0; i < IB; ++i) s[i] = fma(d, wt[o * IB + i], s[i]);
                }
                T* dst = coarser ? (gin + (ll) i0 * ld_in + t) : (gtree + (ll) i0 * ld_tree + aprnet_dec_tree(t));
                const ll ldd = coarser ? ld_in : ld_tree;
#pragma unroll
                for (int i = 0; i < IB; ++i)
                    if (i0 + i < cin) atomicAdd(dst + (ll) i * ldd, s[i]);
            }
        }
    }
    if (active && cross_only != 1) {
#pragma unroll
        for (int i = 0; i < IB; ++i)
            if (i0 + i < cin) atomicAdd(gin + (ll) (i0 + i) * ld_in + q, acc[i]);
    }
}

// Cross-level part of the input gradient as a PULL over the cached edge plan (deterministic: one thread owns a target and
// IB input channels and visits taps, then the locations of each (target, tap) group, in ascending order):
//   grad[target][i] += sum over taps, locations q of the group, output channels o of dO[o][q] * w[slot][o][i][tap].
// Replaces the atomicAdd scatter of conv333_backward_input_kernel (cross_only = 2 there leaves the scatter out).
template<typename T, int OB, int IB, int TPB>
__global__ void __launch_bounds__(TPB) conv333_cross_pull_kernel(const int32_t* __restrict__ active, const int32_t* __restrict__ vnbr, ll n_active,
                                                                 ll a_begin, ll a_end, const int32_t* __restrict__ vstart,
                                                                 const int32_t* __restrict__ vsrc, const T* __restrict__ gout, ll ld_out,
                                                                 const T* __restrict__ wslot, T* __restrict__ gin, ll ld_in,
                                                                 T* __restrict__ gtree, ll ld_tree, ll n_split, int cin, int cout) {
    extern __shared__ unsigned char smem_raw[];
    T* wsm = reinterpret_cast<T*>(smem_raw);                      // [27][OB][IB]
    const ll a = a_begin + (ll) blockIdx.x * TPB + threadIdx.x;
    const bool live = a < a_end;
    const int i0 = blockIdx.y * IB;
    T acc[IB];
#pragma unroll
    for (int i = 0; i < IB; ++i) acc[i] = 0;
    for (int o0 = 0; o0 < cout; o0 += OB) {
        __syncthreads();
        for (int e = threadIdx.x; e < 27 * IB * OB; e += TPB) {
            const int tap = e % 27, i = (e / 27) % IB, o = e / (27 * IB);
            const bool ok = (o0 + o < cout) && (i0 + i < cin);
            wsm[(tap * OB + o) * IB + i] = ok ? wslot[((ll) (o0 + o) * cin + (i0 + i)) * 27 + tap] : T(0);
        }
        __syncthreads();
        if (!live) continue;
        const int ob = min(OB, cout - o0);
        for (int tap = 0; tap < 27; ++tap) {
            const int32_t v = vnbr[(ll) tap * n_active + a];
            if (v < 0) continue;
            const T* wt = wsm + tap * OB * IB;
            const int e1 = vstart[v + 1];
            for (int e = vstart[v]; e < e1; ++e) {
                const T* g = gout + (ll) o0 * ld_out + vsrc[e];
                for (int o = 0; o < ob; ++o) {
                    const T d = g[(ll) o * ld_out];
#pragma unroll
                    for (int i = 0; i < IB; ++i) acc[i] = fma(d, wt[o * IB + i], acc[i]);
                }
            }
        }
    }
    if (!live) return;
    const ll t = active[a];
    T* dst = t < n_split ? gin + (ll) i0 * ld_in + t : gtree + (ll) i0 * ld_tree + (t - n_split);
    const ll ldd = t < n_split ? ld_in : ld_tree;
#pragma unroll
    for (int i = 0; i < IB; ++i)
        if (i0 + i < cin) dst[(ll) i * ldd] += acc[i];           // the only writer of this entry in this launch
}

// ---------------------------------------------------------------------------------------------
// weight gradient
// ---------------------------------------------------------------------------------------------
// One block reduces a contiguous range of output locations of one level for a tile of IB input x OB
// output channels and all 27 taps.  Q = IB*OB/OPT threads cover the (i, o-group) pairs; the
// TPB/Q "slices" split the particles of each staged chunk and are summed through shared memory at
// the end.  Each thread keeps 27 x OPT accumulators in registers.
template<typename T, int IB, int OB, int OPT, int KCH, int TPB>
__global__ void __launch_bounds__(TPB) conv333_dw_partial_kernel(ll seg_begin, ll seg_end, ll range_len,
                                                                 const int32_t* __restrict__ nbr, ll N,
                                                                 const T* __restrict__ in, ll ld_in,
                                                                 const T* __restrict__ tree, ll ld_tree,
                                                                 const T* __restrict__ gout, ll ld_out,
                                                                 T* __restrict__ partial, int cin, int cout) {
    constexpr int Q = IB * OB / OPT;
    constexpr int NS = TPB / Q;
    constexpr int XP = IB + 1;                                    // padded row of the staged inputs
    static_assert(TPB % Q == 0 && NS >= 1, "thread mapping");
    extern __shared__ unsigned char smem_raw[];
    T* xs = reinterpret_cast<T*>(smem_raw);                       // [27][KCH][XP]
    T* gs = xs + 27 * KCH * XP;                                   // [KCH][OB]

    const int nib = (cin + IB - 1) / IB;
    const int i0 = (blockIdx.y % nib) * IB, o0 = (blockIdx.y / nib) * OB;
    const ll pb = seg_begin + (ll) blockIdx.x * range_len;
    const ll pe = min(seg_end, pb + range_len);

    const int pair = threadIdx.x % Q, slice = threadIdx.x / Q;
    const int ti = pair % IB, tog = pair / IB;                    // input channel, group of OPT output channels

    T acc[27][OPT];
#pragma unroll
    for (int t = 0; t < 27; ++t)
#pragma unroll
        for (int o = 0; o < OPT; ++o) acc[t][o] = 0;

    for (ll p0 = pb; p0 < pe; p0 += KCH) {
        __syncthreads();
        for (int e = threadIdx.x; e < KCH * OB; e += TPB) {
            const int k = e % KCH, o = e / KCH;
            const bool ok = (p0 + k < pe) && (o0 + o < cout);
            gs[k * OB + o] = ok ? gout[(ll) (o0 + o) * ld_out + p0 + k] : T(0);
        }
        for (int e = threadIdx.x; e < 27 * KCH * IB; e += TPB) {
            const int k = e % KCH, i = (e / KCH) % IB, tap = e / (KCH * IB);
            T v = 0;
            if (p0 + k < pe && i0 + i < cin) {
                const int32_t q = nbr[(ll) tap * N + p0 + k];
                v = gather_value(in + (ll) (i0 + i) * ld_in, tree + (ll) (i0 + i) * ld_tree, q);
            }
            xs[(tap * KCH + k) * XP + i] = v;
        }
        __syncthreads();
        for (int k = slice; k < KCH; k += NS) {
            T d[OPT];
#pragma unroll
            for (int o = 0; o < OPT; ++o) d[o] = gs[k * OB + tog * OPT + o];
#pragma unroll
            for (int t = 0; t < 27; ++t) {
                const T x = xs[(t * KCH + k) * XP + ti];
#pragma unroll
                for (int o = 0; o < OPT; ++o) acc[t][o] = fma(d[o], x, acc[t][o]);
            }
        }
    }

    T* dst = partial + (ll) blockIdx.x * cout * cin * 27;
    if (NS > 1) {
        // sum the slices in slice order through shared memory (reuses the staging buffer)
        __syncthreads();
        T* red = xs;                                              // [Q][27*OPT] per slice pass
        for (int s = 1; s < NS; ++s) {
            if (slice == s) {
#pragma unroll
                for (int t = 0; t < 27; ++t)
#pragma unroll
                    for (int o = 0; o < OPT; ++o) red[(t * OPT + o) * Q + pair] = acc[t][o];
            }
            __syncthreads();
            if (slice == 0) {
#pragma unroll
                for (int t = 0; t < 27; ++t)
#pragma unroll
                    for (int o = 0; o < OPT; ++o) acc[t][o] += red[(t * OPT + o) * Q + pair];
            }
            __syncthreads();
        }
    }
    if (slice == 0 && i0 + ti < cin) {
#pragma unroll
        for (int o = 0; o < OPT; ++o) {
            const int oc = o0 + tog * OPT + o;
            if (oc < cout) {
#pragma unroll
                for (int t = 0; t < 27; ++t) dst[((ll) oc * cin + i0 + ti) * 27 + t] = acc[t][o];
            }
        }
    }
}

template<typename T>
__global__ void reduce_partial_kernel(const T* __restrict__ partial, int nchunks, ll elems, T* __restrict__ dst) {
    const ll e = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= elems) return;
    T s = 0;
    for (int c = 0; c < nchunks; ++c) s += partial[(ll) c * elems + e];
    dst[e] += s;
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
template<typename T> struct FwdCfg;
template<> struct FwdCfg<float> { static constexpr int OB = 32, IB = 8, TPB = 256; };
template<> struct FwdCfg<double> { static constexpr int OB = 16, IB = 8, TPB = 128; };

template<typename T, int OB, int IB, int TPB>
int launch_forward(const SegTable& segs, const AprPlan* plan, const T* in, ll ld_in, const T* tree, ll ld_tree, const T* w,
                   T* out, ll ld_out, int cin, int cout, cudaStream_t st, const char* pname) {
    const size_t smem = (size_t) 27 * IB * OB * sizeof(T);
    auto kern = conv333_forward_kernel<T, OB, IB, TPB>;
    if (smem > 48 * 1024) APRNET_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    dim3 grid((unsigned) segs.tile_begin[segs.n], (unsigned) aprnet_ceil_div(cout, OB));
    { AprnetProfScope _prof(pname, st);
    kern<<<grid, TPB, smem, st>>>(segs, plan->nbr, plan->n, in, ld_in, tree, ld_tree, w, out, ld_out, cin, cout);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

template<typename T>
int conv333_fwd(aprnet_apr* a, int dl, int cin, int cout, int slots, const T* in, ll ld_in, const T* w, T* out, ll ld_out,
                T* tree, ll ld_tree, cudaStream_t st, bool tree_valid = false) {
    const AprPlan* plan = aprnet_get_plan(a, dl, st);
    if (!plan) return APRNET_ERR_CUDA;
    int rc = tree_valid ? APRNET_OK : aprnet_fill_tree_mean_forward(a, dl, sizeof(T) == 4 ? APRNET_F32 : APRNET_F64, cin, in, ld_in, tree, ld_tree, st);
    if (rc) return rc;
    typedef FwdCfg<T> C;
    char pname[64];
    snprintf(pname, sizeof(pname), "conv333_fwd:ci%d:co%d:dl%d", cin, cout, dl);
    const SegTable segs = make_seg_table(aprnet_segments(a, dl, slots, false), C::TPB);
    if (segs.tile_begin[segs.n] == 0) return APRNET_OK;
    if (cout <= 4 && sizeof(T) == 4)
        return launch_forward<T, 4, C::IB, C::TPB>(segs, plan, in, ld_in, tree, ld_tree, w, out, ld_out, cin, cout, st, pname);
    if (cout <= 16)
        return launch_forward<T, 16, C::IB, C::TPB>(segs, plan, in, ld_in, tree, ld_tree, w, out, ld_out, cin, cout, st, pname);
    return launch_forward<T, C::OB, C::IB, C::TPB>(segs, plan, in, ld_in, tree, ld_tree, w, out, ld_out, cin, cout, st, pname);
}

template<typename T, int OB, int IB, int TPB>
int launch_backward_input(const SegTable& segs, const AprPlan* plan, const T* gout, ll ld_out, const T* w, T* gin, ll ld_in,
                          T* gtree, ll ld_tree, int cin, int cout, cudaStream_t st, const char* pname, int cross_only) {
    const size_t smem = (size_t) 27 * IB * OB * sizeof(T);
    auto kern = conv333_backward_input_kernel<T, OB, IB, TPB>;
    if (smem > 48 * 1024) APRNET_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    dim3 grid((unsigned) segs.tile_begin[segs.n], (unsigned) aprnet_ceil_div(cin, IB));
    { AprnetProfScope _prof(pname, st);
    kern<<<grid, TPB, smem, st>>>(segs, plan->nbr, plan->n, gout, ld_out, w, gin, ld_in, gtree, ld_tree, cin, cout, cross_only);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

template<typename T>
int conv333_bwd_input(aprnet_apr* a, int dl, int cin, int cout, int slots, const T* gout, ll ld_out, const T* w, T* gin,
                      ll ld_in, T* gtree, ll ld_tree, cudaStream_t st, int cross_only = 0, bool tree_adjoint = true) {
    const AprPlan* plan = aprnet_get_plan(a, dl, st);
    if (!plan) return APRNET_ERR_CUDA;
    const ll ts = a->tree_size(dl);
    if (ts > 0)
        APRNET_CUDA_CHECK(cudaMemset2DAsync(gtree, (size_t) ld_tree * sizeof(T), 0, (size_t) ts * sizeof(T), (size_t) cin, st));
    constexpr int TPB = sizeof(T) == 4 ? 256 : 128;
    const SegTable segs = make_seg_table(aprnet_segments(a, dl, slots, false), TPB);
    char pname[64];
    snprintf(pname, sizeof(pname), "%s:ci%d:co%d:dl%d", cross_only ? "conv333_bwd_cross" : "conv333_bwd_input", cin, cout, dl);
    // complete pass: the cross-level part is pulled over the edge plan (fixed summation order) where the plan's 32-bit edge
    // ids suffice; the atomic scatter remains for larger structures and for the cross-only entry point
    EdgePlan* ep = (!cross_only && 27 * plan->n + 1 < (1ll << 31)) ? aprnet_get_edge_plan(a, dl, st) : nullptr;
    if (!cross_only && 27 * plan->n + 1 < (1ll << 31) && !ep) return APRNET_ERR_CUDA;
    const int mode = ep ? 2 : cross_only;
    if (segs.tile_begin[segs.n] > 0) {
        int rc;
        if (cin <= 4) rc = launch_backward_input<T, 8, 4, TPB>(segs, plan, gout, ld_out, w, gin, ld_in, gtree, ld_tree, cin, cout, st, pname, mode);
        else rc = launch_backward_input<T, 8, 16, TPB>(segs, plan, gout, ld_out, w, gin, ld_in, gtree, ld_tree, cin, cout, st, pname, mode);
        if (rc) return rc;
    }
    if (ep && ep->n_active > 0) {
        constexpr int OB = 8, IB = 16;
        const size_t smem = (size_t) 27 * IB * OB * sizeof(T);
        auto kern = conv333_cross_pull_kernel<T, OB, IB, TPB>;
        if (smem > 48 * 1024) APRNET_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
        const int cml = a->cml(dl);
        char pname2[64];
        snprintf(pname2, sizeof(pname2), "conv333_bwd_cross_pull:ci%d:co%d:dl%d", cin, cout, dl);
        for (const ActiveSeg& sg : ep->segs) {
            if (sg.end <= sg.begin) continue;
            const int slot = std::min(cml - sg.location_level, slots - 1);
            dim3 grid((unsigned) aprnet_ceil_div(sg.end - sg.begin, TPB), (unsigned) aprnet_ceil_div(cin, IB));
            AprnetProfScope _prof(pname2, st);
            kern<<<grid, TPB, smem, st>>>(ep->active, ep->vnbr, ep->n_active, sg.begin, sg.end, ep->vstart, ep->vsrc, gout, ld_out,
                                          w + (ll) slot * cout * cin * 27, gin, ld_in, gtree, ld_tree, plan->n, cin, cout);
        }
        APRNET_LAUNCH_CHECK();
    }
    if (!tree_adjoint) return APRNET_OK;
    return aprnet_fill_tree_mean_backward(a, dl, sizeof(T) == 4 ? APRNET_F32 : APRNET_F64, cin, gin, ld_in, gtree, ld_tree, st);
}

constexpr int DW_MAX_RANGES = 128;
constexpr ll DW_PARTIAL_BUDGET = 64ll << 20;      // elements

inline int dw_max_ranges(int cin, int cout) {
    const ll per = (ll) 27 * cin * cout;
    return (int) std::max<ll>(4, std::min<ll>(DW_MAX_RANGES, DW_PARTIAL_BUDGET / per));
}

template<typename T, int IB, int OB, int OPT, int KCH, int TPB>
int launch_dw(ll sb, ll se, int nranges, ll range_len, const AprPlan* plan, const T* in, ll ld_in, const T* tree, ll ld_tree,
              const T* gout, ll ld_out, T* partial, int cin, int cout, cudaStream_t st, const char* pname) {
    const size_t smem = (size_t) (27 * KCH * (IB + 1) + KCH * OB) * sizeof(T);
    auto kern = conv333_dw_partial_kernel<T, IB, OB, OPT, KCH, TPB>;
    if (smem > 48 * 1024) APRNET_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    dim3 grid((unsigned) nranges, (unsigned) (aprnet_ceil_div(cin, IB) * aprnet_ceil_div(cout, OB)));
    { AprnetProfScope _prof(pname, st);
    kern<<<grid, TPB, smem, st>>>(sb, se, range_len, plan->nbr, plan->n, in, ld_in, tree, ld_tree, gout, ld_out, partial, cin, cout);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

template<typename T>
int conv333_bwd_weights(aprnet_apr* a, int dl, int cin, int cout, int slots, const T* in, ll ld_in, const T* tree, ll ld_tree,
                        const T* gout, ll ld_out, T* gw, T* partial, cudaStream_t st) {
    const AprPlan* plan = aprnet_get_plan(a, dl, st);
    if (!plan) return APRNET_ERR_CUDA;
    const ll elems = (ll) 27 * cin * cout;
    const int max_ranges = dw_max_ranges(cin, cout);
    char pname[64];
    snprintf(pname, sizeof(pname), "conv333_dw:ci%d:co%d:dl%d", cin, cout, dl);
    for (const Segment& s : aprnet_segments(a, dl, slots, false)) {
        const ll len = s.end - s.begin;
        const int nranges = (int) std::min<ll>(max_ranges, (len + 511) / 512);
        const ll range_len = (len + nranges - 1) / nranges;
        int rc;
        if (sizeof(T) == 8) {
            rc = launch_dw<T, 16, 16, 1, 16, 256>(s.begin, s.end, nranges, range_len, plan, in, ld_in, tree, ld_tree, gout, ld_out, partial, cin, cout, st, pname);
        } else if (cin >= 24) {
            rc = launch_dw<T, 32, 32, 4, 32, 256>(s.begin, s.end, nranges, range_len, plan, in, ld_in, tree, ld_tree, gout, ld_out, partial, cin, cout, st, pname);
        } else if (cin > 2) {
            rc = launch_dw<T, 8, 32, 4, 32, 256>(s.begin, s.end, nranges, range_len, plan, in, ld_in, tree, ld_tree, gout, ld_out, partial, cin, cout, st, pname);
        } else {
            rc = launch_dw<T, 2, 32, 4, 64, 256>(s.begin, s.end, nranges, range_len, plan, in, ld_in, tree, ld_tree, gout, ld_out, partial, cin, cout, st, pname);
        }
        if (rc) return rc;
        { AprnetProfScope _prof("conv333_dw_reduce", st);
        reduce_partial_kernel<T><<<aprnet_ceil_div(elems, 256), 256, 0, st>>>(partial, nranges, elems, gw + (ll) s.slot * elems);
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

#define CONV_CHECKS()                                                                                           \
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && cin > 0 && cout > 0 && slots > 0, "bad argument");                \
    APRNET_ARG_CHECK(a->cml(dl) <= a->meta.level_max, "level_delta out of range");                              \
    APRNET_ARG_CHECK(ld_in >= a->number_parts(dl) && ld_out >= a->number_parts(dl) && ld_tree >= a->tree_size(dl), \
                     "leading dimension too small")

extern "C" int aprnet_conv333_forward(aprnet_apr* a, int dl, int dtype, int cin, int cout, int slots, const void* in,
                                      int64_t ld_in, const void* w, void* out, int64_t ld_out, void* tree, int64_t ld_tree,
                                      void* stream) {
    CONV_CHECKS();
    APRNET_ARG_CHECK(in && w && out && tree, "null pointer");
    cudaStream_t st = (cudaStream_t) stream;
    DISPATCH(dtype, conv333_fwd<float>(a, dl, cin, cout, slots, (const float*) in, ld_in, (const float*) w, (float*) out, ld_out, (float*) tree, ld_tree, st),
             conv333_fwd<double>(a, dl, cin, cout, slots, (const double*) in, ld_in, (const double*) w, (double*) out, ld_out, (double*) tree, ld_tree, st));
}

extern "C" int aprnet_conv333_backward_input(aprnet_apr* a, int dl, int dtype, int cin, int cout, int slots, const void* gout,
                                             int64_t ld_out, const void* w, void* gin, int64_t ld_in, void* gtree,
                                             int64_t ld_tree, void* stream) {
    CONV_CHECKS();
    APRNET_ARG_CHECK(gout && w && gin && gtree, "null pointer");
    cudaStream_t st = (cudaStream_t) stream;
    DISPATCH(dtype, conv333_bwd_input<float>(a, dl, cin, cout, slots, (const float*) gout, ld_out, (const float*) w, (float*) gin, ld_in, (float*) gtree, ld_tree, st),
             conv333_bwd_input<double>(a, dl, cin, cout, slots, (const double*) gout, ld_out, (const double*) w, (double*) gin, ld_in, (double*) gtree, ld_tree, st));
}

// Split forms for a caller that exchanges tree values between the tree fill and the gather (one z-slab of an
// APR per GPU): the forward pass takes the tree means as given, the input gradient leaves grad_tree unfolded.
extern "C" int aprnet_conv333_forward_pretree(aprnet_apr* a, int dl, int dtype, int cin, int cout, int slots, const void* in,
                                              int64_t ld_in, const void* w, void* out, int64_t ld_out, const void* tree, int64_t ld_tree,
                                              void* stream) {
    CONV_CHECKS();
    APRNET_ARG_CHECK(in && w && out && tree, "null pointer");
    cudaStream_t st = (cudaStream_t) stream;
    DISPATCH(dtype, conv333_fwd<float>(a, dl, cin, cout, slots, (const float*) in, ld_in, (const float*) w, (float*) out, ld_out, (float*) tree, ld_tree, st, true),
             conv333_fwd<double>(a, dl, cin, cout, slots, (const double*) in, ld_in, (const double*) w, (double*) out, ld_out, (double*) tree, ld_tree, st, true));
}

extern "C" int aprnet_conv333_backward_input_pretree(aprnet_apr* a, int dl, int dtype, int cin, int cout, int slots, const void* gout,
                                                     int64_t ld_out, const void* w, void* gin, int64_t ld_in, void* gtree,
                                                     int64_t ld_tree, void* stream) {
    CONV_CHECKS();
    APRNET_ARG_CHECK(gout && w && gin && gtree, "null pointer");
    cudaStream_t st = (cudaStream_t) stream;
    DISPATCH(dtype, conv333_bwd_input<float>(a, dl, cin, cout, slots, (const float*) gout, ld_out, (const float*) w, (float*) gin, ld_in, (float*) gtree, ld_tree, st, 0, false),
             conv333_bwd_input<double>(a, dl, cin, cout, slots, (const double*) gout, ld_out, (const double*) w, (double*) gin, ld_in, (double*) gtree, ld_tree, st, 0, false));
}

extern "C" int64_t aprnet_conv333_partial_elems(int cin, int cout) { return (int64_t) dw_max_ranges(cin, cout) * 27 * cin * cout; }

extern "C" int aprnet_conv333_backward_weights(aprnet_apr* a, int dl, int dtype, int cin, int cout, int slots, const void* in,
                                               int64_t ld_in, const void* tree, int64_t ld_tree, const void* gout,
                                               int64_t ld_out, void* gw, void* partial, void* stream) {
    CONV_CHECKS();
    APRNET_ARG_CHECK(in && tree && gout && gw && partial, "null pointer");
    cudaStream_t st = (cudaStream_t) stream;
    DISPATCH(dtype, conv333_bwd_weights<float>(a, dl, cin, cout, slots, (const float*) in, ld_in, (const float*) tree, ld_tree, (const float*) gout, ld_out, (float*) gw, (float*) partial, st),
             conv333_bwd_weights<double>(a, dl, cin, cout, slots, (const double*) in, ld_in, (const double*) tree, ld_tree, (const double*) gout, ld_out, (double*) gw, (double*) partial, st));
}

// Cross-level part of the input gradient only (coarser particles and tree nodes, then the tree
// adjoint); the same-level part must already be in grad_input (tensor-core path).
extern "C" int aprnet_conv333_backward_input_cross_level(aprnet_apr* a, int dl, int dtype, int cin, int cout, int slots,
                                                         const void* gout, int64_t ld_out, const void* w, void* gin,
                                                         int64_t ld_in, void* gtree, int64_t ld_tree, void* stream) {
    CONV_CHECKS();
    APRNET_ARG_CHECK(gout && w && gin && gtree, "null pointer");
    cudaStream_t st = (cudaStream_t) stream;
    DISPATCH(dtype, conv333_bwd_input<float>(a, dl, cin, cout, slots, (const float*) gout, ld_out, (const float*) w, (float*) gin, ld_in, (float*) gtree, ld_tree, st, 1),
             conv333_bwd_input<double>(a, dl, cin, cout, slots, (const double*) gout, ld_out, (const double*) w, (double*) gin, ld_in, (double*) gtree, ld_tree, st, 1));
}
