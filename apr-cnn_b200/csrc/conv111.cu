// 1x1x1 particle convolution (per-level channel mixing) and stencil restriction.
//
// Replaces pyapr/aprnet/cuda/src/conv111_gpu.cu:9-232 and restrict_gpu.cu:5-235.  The reference
// splits input channels over grid.z and combines them with atomicAdd into a zero-filled output; here
// one thread owns a particle and a block of output channels, loops over all input channels and
// writes each output once (no atomics, deterministic).  Weight gradients are block-local partial
// sums followed by a fixed-order second pass.
#include "apr_device.cuh"
#include <algorithm>

namespace {

typedef long long ll;
constexpr int MAX_SEGS = APRNET_MAX_LEVELS;

struct SegTable {
    int n;
    ll begin[MAX_SEGS], end[MAX_SEGS];
    int slot[MAX_SEGS];
    int tile_begin[MAX_SEGS + 1];     // cumulative tile counts
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

// 16-byte vector of T (4 floats / 2 doubles): the staged weights are read from shared memory in such pieces, so that
// one shared-memory instruction feeds several multiply-adds (with scalar reads the kernel is bound by the
// shared-memory pipe, one broadcast read per multiply-add).
template<typename T> struct Vec16;
template<> struct Vec16<float> { typedef float4 type; static constexpr int N = 4; };
template<> struct Vec16<double> { typedef double2 type; static constexpr int N = 2; };

// out[o][p] = sum_i w[slot][o][i] * in[i][p]; weight element (s, o, i) at w[s*ws + o*wo + i*wi]
// (forward: wo = Cin, wi = 1; input gradient: roles of the channel axes swapped, wo = 1, wi = Cin_fwd).
// A thread owns PPT locations (p, p + TPB, ...) and OB output channels: every 16-byte weight read from shared memory
// feeds 4 * PPT multiply-adds.  (With one location per thread the kernel ran at 84 % of the load/store pipe and 32 % of
// DRAM: bound by the broadcast weight reads.)
template<typename T, int OB, int TPB, int PPT>
__global__ void __launch_bounds__(TPB, sizeof(T) == 4 ? 2 : 1) conv111_kernel(SegTable segs, const T* __restrict__ in, ll ld_in,
                                                      const T* __restrict__ w, ll ws, ll wo, ll wi,
                                                      T* __restrict__ out, ll ld_out, int n_in, int n_out) {
    typedef typename Vec16<T>::type V;
    constexpr int VN = Vec16<T>::N;
    static_assert(OB % VN == 0, "output block is a whole number of 16-byte vectors");
    extern __shared__ __align__(16) unsigned char smem_raw[];
    T* wsm = reinterpret_cast<T*>(smem_raw);              // [n_in][OB]
    int seg = 0;
    while (seg + 1 < segs.n && (int) blockIdx.x >= segs.tile_begin[seg + 1]) ++seg;
    const ll p0 = segs.begin[seg] + (ll) (blockIdx.x - segs.tile_begin[seg]) * (TPB * PPT) + threadIdx.x;
    const ll pend = segs.end[seg];
    const int o0 = blockIdx.y * OB;
    const T* wslot = w + (ll) segs.slot[seg] * ws;
    for (int e = threadIdx.x; e < n_in * OB; e += TPB) {
        const int i = e / OB, o = e % OB;
        wsm[e] = (o0 + o < n_out) ? wslot[(ll) (o0 + o) * wo + (ll) i * wi] : T(0);
    }
    __syncthreads();
    if (p0 >= pend) return;
    T acc[PPT][OB];
#pragma unroll
    for (int q = 0; q < PPT; ++q)
#pragma unroll
        for (int o = 0; o < OB; ++o) acc[q][o] = 0;
    constexpr int IU = PPT == 1 ? 8 : 4;     // input channels whose loads are in flight together
    auto mix = [&](const T (&v)[PPT], const int i) {
        const V* wr = reinterpret_cast<const V*>(wsm + i * OB);
#pragma unroll
        for (int o = 0; o < OB / VN; ++o) {
            const V wv = wr[o];
            const T* we = reinterpret_cast<const T*>(&wv);
#pragma unroll
            for (int e = 0; e < VN; ++e)
#pragma unroll
                for (int q = 0; q < PPT; ++q) acc[q][o * VN + e] = fma(v[q], we[e], acc[q][o * VN + e]);
        }
    };
    int i = 0;
    for (; i + IU <= n_in; i += IU) {
        T v[IU][PPT];
#pragma unroll
        for (int k = 0; k < IU; ++k)
#pragma unroll
            for (int q = 0; q < PPT; ++q) v[k][q] = (p0 + (ll) q * TPB < pend) ? in[(ll) (i + k) * ld_in + p0 + (ll) q * TPB] : T(0);
#pragma unroll
        for (int k = 0; k < IU; ++k) mix(v[k], i + k);
    }
    for (; i < n_in; ++i) {
        T v[PPT];
#pragma unroll
        for (int q = 0; q < PPT; ++q) v[q] = (p0 + (ll) q * TPB < pend) ? in[(ll) i * ld_in + p0 + (ll) q * TPB] : T(0);
        mix(v, i);
    }
#pragma unroll
    for (int q = 0; q < PPT; ++q) {
        const ll p = p0 + (ll) q * TPB;
        if (p >= pend) break;
#pragma unroll
        for (int o = 0; o < OB; ++o)
            if (o0 + o < n_out) out[(ll) (o0 + o) * ld_out + p] = acc[q][o];
    }
}

// Weight gradient of one segment: partial[chunk][o][i] = sum over the chunk's particles of
// gout[o][p] * in[i][p].  Block tile 64 (o) x 64 (i), 256 threads, 4x4 outputs per thread: per particle a thread
// reads 4 + 4 values from shared memory (two 16-byte reads for floats) for 16 multiply-adds.
template<typename T>
__global__ void __launch_bounds__(256) conv111_dw_partial_kernel(ll seg_begin, ll seg_end, ll chunk_len,
                                                                 const T* __restrict__ in, ll ld_in,
                                                                 const T* __restrict__ gout, ll ld_out,
                                                                 T* __restrict__ partial, int cin, int cout) {
    constexpr int TILE = 64, KC = 32;
    // [particle][channel]: a thread's four channels are contiguous; rows padded by 4 so that the transposing stores of a
    // warp (32 particles of one channel) spread over 8 banks instead of one
    __shared__ __align__(16) T gs[KC][TILE + 4];
    __shared__ __align__(16) T xs[KC][TILE + 4];
    const int nib = (cin + TILE - 1) / TILE;
    const int ob = blockIdx.y / nib, ib = blockIdx.y % nib;
    const ll pb = seg_begin + (ll) blockIdx.x * chunk_len;
    const ll pe = min(seg_end, pb + chunk_len);
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;          // 4 input channels, 4 output channels
    T acc[4][4];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) acc[a][b] = 0;
    for (ll p0 = pb; p0 < pe; p0 += KC) {
        // consecutive threads read consecutive particles of one channel row (coalesced), stored transposed
        for (int e = threadIdx.x; e < TILE * KC; e += 256) {
            const int r = e / KC, k = e % KC;
            const bool inr = p0 + k < pe;
            const int o = ob * TILE + r, i = ib * TILE + r;
            gs[k][r] = (inr && o < cout) ? gout[(ll) o * ld_out + p0 + k] : T(0);
            xs[k][r] = (inr && i < cin) ? in[(ll) i * ld_in + p0 + k] : T(0);
        }
        __syncthreads();
#pragma unroll 8
        for (int k = 0; k < KC; ++k) {
            T g[4], x[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) { g[a] = gs[k][4 * ty + a]; x[a] = xs[k][4 * tx + a]; }
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int b = 0; b < 4; ++b) acc[a][b] = fma(g[a], x[b], acc[a][b]);
        }
        __syncthreads();
    }
    T* dst = partial + (ll) blockIdx.x * cout * cin;
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) {
            const int o = ob * TILE + 4 * ty + a, i = ib * TILE + 4 * tx + b;
            if (o < cout && i < cin) dst[(ll) o * cin + i] = acc[a][b];
        }
}

// Weight gradient for few output channels (CO <= 4, e.g. a classification head): a lane owns one particle
// of a 32-particle strip and keeps the CO x 32 products of one block of 32 input channels; strips are
// visited in a fixed order, lanes and warps are combined in a fixed order.
template<typename T, int CO>
__global__ void __launch_bounds__(256) conv111_dw_small_kernel(ll seg_begin, ll seg_end, ll chunk_len,
                                                               const T* __restrict__ in, ll ld_in,
                                                               const T* __restrict__ gout, ll ld_out,
                                                               T* __restrict__ partial, int cin, int cout) {
    __shared__ T red[8][CO * 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int i0 = blockIdx.y * 32;
    const ll pb = seg_begin + (ll) blockIdx.x * chunk_len;
    const ll pe = min(seg_end, pb + chunk_len);
    T acc[CO][32];
#pragma unroll
    for (int o = 0; o < CO; ++o)
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[o][i] = 0;
    for (ll p = pb + warp * 32 + lane; p < pe; p += 256) {
        T g[CO];
#pragma unroll
        for (int o = 0; o < CO; ++o) g[o] = o < cout ? gout[(ll) o * ld_out + p] : T(0);
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            const T x = i0 + i < cin ? in[(ll) (i0 + i) * ld_in + p] : T(0);
#pragma unroll
            for (int o = 0; o < CO; ++o) acc[o][i] = fma(g[o], x, acc[o][i]);
        }
    }
#pragma unroll
    for (int o = 0; o < CO; ++o)
#pragma unroll
        for (int i = 0; i < 32; ++i) {
            T v = acc[o][i];
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
            if (lane == 0) red[warp][o * 32 + i] = v;
        }
    __syncthreads();
    T* dst = partial + (ll) blockIdx.x * cout * cin;
    for (int e = threadIdx.x; e < CO * 32; e += 256) {
        const int o = e / 32, i = i0 + e % 32;
        T v = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) v += red[w][e];
        if (o < cout && i < cin) dst[(ll) o * cin + i] = v;
    }
}

// dst[e] += sum_{c < nchunks} partial[c][e], chunks visited in ascending order
template<typename T>
__global__ void reduce_partial_kernel(const T* __restrict__ partial, int nchunks, ll elems, T* __restrict__ dst) {
    const ll e = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= elems) return;
    T s = 0;
    for (int c = 0; c < nchunks; ++c) s += partial[(ll) c * elems + e];
    dst[e] += s;
}

// block partials of the weight gradient: many chunks for small filters (parallelism), fewer for large ones (workspace)
inline int dw_max_chunks(int cin, int cout) { return (int) std::max<ll>(128, std::min<ll>(2048, (16ll << 20) / ((ll) cin * cout))); }

template<typename T, int OB, int TPB, int PPT>
int conv111_launch(const aprnet_apr* a, int dl, int S, const T* in, ll ld_in, const T* w, ll ws, ll wo, ll wi, T* out, ll ld_out,
                   int n_in, int n_out, cudaStream_t st) {
    const SegTable segs = make_seg_table(aprnet_segments(a, dl, S, true), TPB * PPT);
    const int tiles = segs.tile_begin[segs.n];
    if (tiles == 0) return APRNET_OK;
    const size_t smem = (size_t) n_in * OB * sizeof(T);
    if (smem > 48 * 1024)
        APRNET_CUDA_CHECK(cudaFuncSetAttribute(conv111_kernel<T, OB, TPB, PPT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    dim3 grid((unsigned) tiles, (unsigned) aprnet_ceil_div(n_out, OB));
    { AprnetProfScope _prof("conv111", st);
    conv111_kernel<T, OB, TPB, PPT><<<grid, TPB, smem, st>>>(segs, in, ld_in, w, ws, wo, wi, out, ld_out, n_in, n_out);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

template<typename T>
int conv111_apply(const aprnet_apr* a, int dl, int n_in, int n_out, int S, const T* in, ll ld_in, const T* w,
                  ll ws, ll wo, ll wi, T* out, ll ld_out, cudaStream_t st) {
    constexpr int TPB = 256;
    if (n_out <= 4) return conv111_launch<T, 4, TPB, 4>(a, dl, S, in, ld_in, w, ws, wo, wi, out, ld_out, n_in, n_out, st);      // e.g. a classification head
    if (n_out <= 16) return conv111_launch<T, 16, TPB, 2>(a, dl, S, in, ld_in, w, ws, wo, wi, out, ld_out, n_in, n_out, st);
    // the input is read once per 32 outputs; two locations per thread (fp32) halve the shared-memory reads per multiply-add
    if (sizeof(T) == 4) return conv111_launch<T, 32, TPB, 2>(a, dl, S, in, ld_in, w, ws, wo, wi, out, ld_out, n_in, n_out, st);
    return conv111_launch<T, 32, TPB, 1>(a, dl, S, in, ld_in, w, ws, wo, wi, out, ld_out, n_in, n_out, st);
}

template<typename T>
int conv111_dw(const aprnet_apr* a, int dl, int cin, int cout, int S, const T* in, ll ld_in, const T* gout, ll ld_out,
               T* gw, T* partial, cudaStream_t st) {
    const std::vector<Segment> segs = aprnet_segments(a, dl, S, true);
    const ll elems = (ll) cin * cout;
    for (const Segment& s : segs) {
        const ll len = s.end - s.begin;
        const int nchunks = (int) std::min<ll>(dw_max_chunks(cin, cout), (len + 1023) / 1024);
        const ll chunk_len = ((len + nchunks - 1) / nchunks + 31) / 32 * 32;
        // few outputs: blocks of 32 input channels (conv111_dw_small_kernel); else 64 x 64 tiles
        const unsigned gy = cout <= 4 ? (unsigned) aprnet_ceil_div(cin, 32) : (unsigned) (aprnet_ceil_div(cout, 64) * aprnet_ceil_div(cin, 64));
        dim3 grid((unsigned) nchunks, gy);
        { AprnetProfScope _prof("conv111_dw", st);
        if (cout <= 4) conv111_dw_small_kernel<T, 4><<<grid, 256, 0, st>>>(s.begin, s.end, chunk_len, in, ld_in, gout, ld_out, partial, cin, cout);
        else conv111_dw_partial_kernel<T><<<grid, 256, 0, st>>>(s.begin, s.end, chunk_len, in, ld_in, gout, ld_out, partial, cin, cout);
        }
        { AprnetProfScope _prof("conv111_dw_reduce", st);
        reduce_partial_kernel<T><<<aprnet_ceil_div(elems, 256), 256, 0, st>>>(partial, nchunks, elems, gw + (ll) s.slot * elems);
        }
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

// Stencil restriction.  pyapr/aprnet/src/kernel.hpp:54-128: slots < S are copied; slot k >= S is the
// last given stencil box-averaged onto a grid 2^(k-S+1) times coarser (overlap lengths per axis,
// divided by step^3).  One thread per (extra level, filter); 27x27 overlap products each.
// overlap weight between fine tap ti and coarse tap to along one axis, for a grid `step` times coarser
__device__ __forceinline__ float restrict_overlap(int step, int fine_tap, int coarse_tap) {
    const int off = step - 1;
    return (float) (min((coarse_tap + 1) * step, off + fine_tap + step) - max(coarse_tap * step, off + fine_tap));
}

// forward: one thread per (extra slot k, filter f): dst[k][f][to] = sum_ti ov(ti, to) * src[S-1][f][ti]
template<typename T>
__global__ void restrict333_forward_kernel(int S, ll filters, const T* __restrict__ src, T* __restrict__ dst) {
    const ll f = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (f >= filters) return;
    const int k = S + blockIdx.y;
    const int step = 1 << (k - (S - 1));
    const float factor = (float) step * (float) step * (float) step;
    const T* fine = src + ((ll) (S - 1) * filters + f) * 27;
    T* coarse = dst + ((ll) k * filters + f) * 27;
    for (int zo = 0; zo < 3; ++zo) for (int xo = 0; xo < 3; ++xo) for (int yo = 0; yo < 3; ++yo) {
        T acc = 0;
        for (int zi = 0; zi < 3; ++zi) {
            const float oz = restrict_overlap(step, zi, zo);
            if (oz <= 0) continue;
            for (int xi = 0; xi < 3; ++xi) {
                const float ox = restrict_overlap(step, xi, xo);
                if (ox <= 0) continue;
                for (int yi = 0; yi < 3; ++yi) {
                    const float oy = restrict_overlap(step, yi, yo);
                    if (oy <= 0) continue;
                    acc += (T) (ox * oy * oz / factor) * fine[(zi * 3 + xi) * 3 + yi];
                }
            }
        }
        coarse[(zo * 3 + xo) * 3 + yo] = acc;
    }
}

// backward (transpose): one thread per filter folds every extra slot into slot S-1, slots in
// ascending order, so the sum order is fixed.
template<typename T>
__global__ void restrict333_backward_kernel(int S, int L, ll filters, const T* __restrict__ src, T* __restrict__ dst) {
    // one thread per (filter, fine tap): 27 times the parallelism of one thread per filter, same summation order
    const ll e = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= filters * 27) return;
    const ll f = e / 27;
    const int tap = (int) (e - f * 27);
    const int zi = tap / 9, xi = (tap / 3) % 3, yi = tap % 3;
    T acc = src[((ll) (S - 1) * filters + f) * 27 + tap];
    for (int k = S; k < L; ++k) {
        const int step = 1 << (k - (S - 1));
        const float factor = (float) step * (float) step * (float) step;
        const T* coarse = src + ((ll) k * filters + f) * 27;
        for (int zo = 0; zo < 3; ++zo) {
            const float oz = restrict_overlap(step, zi, zo);
            if (oz <= 0) continue;
            for (int xo = 0; xo < 3; ++xo) {
                const float ox = restrict_overlap(step, xi, xo);
                if (ox <= 0) continue;
                for (int yo = 0; yo < 3; ++yo) {
                    const float oy = restrict_overlap(step, yi, yo);
                    if (oy <= 0) continue;
                    acc += (T) (ox * oy * oz / factor) * coarse[(zo * 3 + xo) * 3 + yo];
                }
            }
        }
    }
    dst[((ll) (S - 1) * filters + f) * 27 + tap] = acc;
}

template<typename T>
int restrict333(int S, int L, ll filters, const T* src, T* dst, bool backward, cudaStream_t st) {
    APRNET_CUDA_CHECK(cudaMemcpyAsync(dst, src, (size_t) S * filters * 27 * sizeof(T), cudaMemcpyDeviceToDevice, st));
    if (L > S) {
        if (backward) {
            restrict333_backward_kernel<T><<<aprnet_ceil_div(filters * 27, 128), 128, 0, st>>>(S, L, filters, src, dst);
        } else {
            dim3 grid((unsigned) aprnet_ceil_div(filters, 128), (unsigned) (L - S));
            restrict333_forward_kernel<T><<<grid, 128, 0, st>>>(S, filters, src, dst);
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

extern "C" int aprnet_conv111_forward(const aprnet_apr* a, int dl, int dtype, int cin, int cout, int S, const void* in,
                                      int64_t ld_in, const void* w, void* out, int64_t ld_out, void* stream) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && in && w && out && cin > 0 && cout > 0 && S > 0, "bad argument");
    APRNET_DEVICE_CHECK(a);
    APRNET_ARG_CHECK(ld_in >= a->number_parts(dl) && ld_out >= a->number_parts(dl), "leading dimension too small");
    cudaStream_t st = (cudaStream_t) stream;
    const ll ws = (ll) cin * cout;
    DISPATCH(dtype, conv111_apply<float>(a, dl, cin, cout, S, (const float*) in, ld_in, (const float*) w, ws, cin, 1, (float*) out, ld_out, st),
             conv111_apply<double>(a, dl, cin, cout, S, (const double*) in, ld_in, (const double*) w, ws, cin, 1, (double*) out, ld_out, st));
}

extern "C" int aprnet_conv111_backward_input(const aprnet_apr* a, int dl, int dtype, int cin, int cout, int S,
                                             const void* gout, int64_t ld_out, const void* w, void* gin, int64_t ld_in,
                                             void* stream) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && gout && w && gin && cin > 0 && cout > 0 && S > 0, "bad argument");
    APRNET_DEVICE_CHECK(a);
    APRNET_ARG_CHECK(ld_in >= a->number_parts(dl) && ld_out >= a->number_parts(dl), "leading dimension too small");
    cudaStream_t st = (cudaStream_t) stream;
    const ll ws = (ll) cin * cout;
    DISPATCH(dtype, conv111_apply<float>(a, dl, cout, cin, S, (const float*) gout, ld_out, (const float*) w, ws, 1, cin, (float*) gin, ld_in, st),
             conv111_apply<double>(a, dl, cout, cin, S, (const double*) gout, ld_out, (const double*) w, ws, 1, cin, (double*) gin, ld_in, st));
}

extern "C" int64_t aprnet_conv111_partial_elems(int cin, int cout) { return (int64_t) dw_max_chunks(cin, cout) * cin * cout; }

extern "C" int aprnet_conv111_backward_weights(const aprnet_apr* a, int dl, int dtype, int cin, int cout, int S,
                                               const void* in, int64_t ld_in, const void* gout, int64_t ld_out,
                                               void* gw, void* partial, void* stream) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && in && gout && gw && partial && cin > 0 && cout > 0 && S > 0, "bad argument");
    APRNET_DEVICE_CHECK(a);
    APRNET_ARG_CHECK(ld_in >= a->number_parts(dl) && ld_out >= a->number_parts(dl), "leading dimension too small");
    cudaStream_t st = (cudaStream_t) stream;
    DISPATCH(dtype, conv111_dw<float>(a, dl, cin, cout, S, (const float*) in, ld_in, (const float*) gout, ld_out, (float*) gw, (float*) partial, st),
             conv111_dw<double>(a, dl, cin, cout, S, (const double*) in, ld_in, (const double*) gout, ld_out, (double*) gw, (double*) partial, st));
}

extern "C" int aprnet_restrict333_forward(int dtype, int S, int L, int64_t filters, const void* w, void* expanded, void* stream) {
    APRNET_ARG_CHECK(w && expanded && S > 0 && L >= S && filters > 0, "requires num_levels >= num_stencils");
    cudaStream_t st = (cudaStream_t) stream;
    DISPATCH(dtype, restrict333<float>(S, L, filters, (const float*) w, (float*) expanded, false, st),
             restrict333<double>(S, L, filters, (const double*) w, (double*) expanded, false, st));
}

extern "C" int aprnet_restrict333_backward(int dtype, int S, int L, int64_t filters, const void* gexp, void* gw, void* stream) {
    APRNET_ARG_CHECK(gexp && gw && S > 0 && L >= S && filters > 0, "requires num_stencils <= expanded levels");
    cudaStream_t st = (cudaStream_t) stream;
    DISPATCH(dtype, restrict333<float>(S, L, filters, (const float*) gexp, (float*) gw, true, st),
             restrict333<double>(S, L, filters, (const double*) gexp, (double*) gw, true, st));
}
