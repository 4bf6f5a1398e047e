// 3x3x3 convolution for very few input channels (Cin <= 4: the first layer of a network) on CUDA cores,
// fp32, used by the tensor-core drivers instead of the implicit GEMM: with Cin = 1 a packed bf16 row would
// carry one useful value in 32 bytes and the 27 x Cin x Cout products per location are far too few to
// amortise a gathered operand tile.  Values are read from a channel-major buffer
//     vals[ci][r],  r in [0, N) particles, [N, N + T) tree means, r = N + T: zero
// through the cached neighbour table, so a tap is one 4-byte load per input channel.
// Arithmetic: pyapr/aprnet/src/helpers.hpp:505-575 (forward) and :624-702 (weight gradient).
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

inline SegTable make_seg_table(const std::vector<Segment>& segs, ll tile) {
    SegTable t;
    t.n = (int) segs.size();
    t.tile_begin[0] = 0;
    for (int i = 0; i < t.n; ++i) {
        t.begin[i] = segs[i].begin; t.end[i] = segs[i].end; t.slot[i] = segs[i].slot;
        t.tile_begin[i + 1] = t.tile_begin[i] + aprnet_ceil_div(segs[i].end - segs[i].begin, tile);
    }
    return t;
}

struct alignas(16) F4 { float a[4]; };

__device__ __forceinline__ ll resolve_row(int32_t v, ll n, ll zero_row) {
    return v >= 0 ? (ll) v : (v == APRNET_NONE ? zero_row : n + aprnet_dec_tree(v));
}

// vals[ci][0, n) = x[ci], vals[ci][n, n + t) = tree[ci], vals[ci][n + t] = 0
__global__ void small_stage_kernel(const float* __restrict__ x, ll ld_x, ll n, const float* __restrict__ tree, ll ld_tree, ll t,
                                   int cin, float* __restrict__ vals) {
    const ll R = n + t + 1;
    const ll r = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= R) return;
    for (int ci = 0; ci < cin; ++ci)
        vals[(ll) ci * R + r] = r < n ? x[(ll) ci * ld_x + r] : (r < n + t ? tree[(ll) ci * ld_tree + (r - n)] : 0.f);
}

// forward: thread = output location x block of 32 output channels; weights of the level's stencil in
// shared memory as [tap][ci][32] (read four at a time)
template<int CIN>
__global__ void __launch_bounds__(128) conv333_small_forward_kernel(SegTable segs, const int32_t* __restrict__ nbr, ll N, ll T,
                                                                    const float* __restrict__ vals, const float* __restrict__ w,
                                                                    int cout, float* __restrict__ out, ll ld_out) {
    __shared__ F4 ws[27 * CIN * 8];
    int seg = 0;
    while (seg + 1 < segs.n && (int) blockIdx.x >= segs.tile_begin[seg + 1]) ++seg;
    const ll p = segs.begin[seg] + (ll) (blockIdx.x - segs.tile_begin[seg]) * 128 + threadIdx.x;
    const int co0 = blockIdx.y * 32;
    const float* wslot = w + (ll) segs.slot[seg] * cout * CIN * 27;
    for (int e = threadIdx.x; e < 27 * CIN * 32; e += 128) {
        const int co = e & 31, ci = (e >> 5) % CIN, tap = e / (32 * CIN);
        reinterpret_cast<float*>(ws)[e] = co0 + co < cout ? wslot[((ll) (co0 + co) * CIN + ci) * 27 + tap] : 0.f;
    }
    __syncthreads();
    if (p >= segs.end[seg]) return;
    const ll R = N + T + 1;
    float acc[32];
#pragma unroll
    for (int o = 0; o < 32; ++o) acc[o] = 0.f;
    // all 27 table entries, then all 27 values of a channel, are requested before any is used (the kernel is bound by
    // the latency of these gathers, not by a unit); row numbers fit 32 bits (N + T + 1 < 2^31, checked by the driver)
    int32_t rows[27];
#pragma unroll
    for (int tap = 0; tap < 27; ++tap) rows[tap] = (int32_t) resolve_row(__ldg(nbr + (ll) tap * N + p), N, N + T);
#pragma unroll 1
    for (int ci = 0; ci < CIN; ++ci) {
        float v[27];
        const float* vc = vals + (ll) ci * R;
#pragma unroll
        for (int tap = 0; tap < 27; ++tap) v[tap] = __ldg(vc + rows[tap]);
#pragma unroll
        for (int tap = 0; tap < 27; ++tap) {
            const F4* wr = ws + (tap * CIN + ci) * 8;
#pragma unroll
            for (int o4 = 0; o4 < 8; ++o4) {
                const F4 q = wr[o4];
#pragma unroll
                for (int k = 0; k < 4; ++k) acc[4 * o4 + k] = fmaf(v[tap], q.a[k], acc[4 * o4 + k]);
            }
        }
    }
#pragma unroll
    for (int o = 0; o < 32; ++o)
        if (co0 + o < cout) out[(ll) (co0 + o) * ld_out + p] = acc[o];
}

// weight gradient of one level: block = range of locations x block of 32 output channels.  The 27 x CIN
// gathered values and the 32 dO values of KP locations are staged in shared memory; a thread owns a 4 x 4
// tile of (tap, ci) x co products; the 4 thread groups of a block take different quarters of every staged
// step and are combined in a fixed order.  partial[range][co][ci][tap].
template<int CIN>
__global__ void __launch_bounds__(256) conv333_small_dw_kernel(ll seg_begin, ll seg_end, ll range_len, const int32_t* __restrict__ nbr, ll N, ll T,
                                                               const float* __restrict__ vals, const float* __restrict__ gout, ll ld_out,
                                                               int cout, float* __restrict__ partial) {
    constexpr int ROWS = 27 * CIN, RQ = (ROWS + 3) / 4;                 // (tap, ci) rows, row quads
    constexpr int KP = CIN <= 2 ? 64 : 32;                              // staged locations per step
    constexpr int XSTRIDE = RQ | 1;                                     // odd: consecutive locations fall on different banks
    __shared__ F4 xs[KP][XSTRIDE];
    __shared__ F4 gs[KP][8 + 1];
    __shared__ float red[RQ * 4 * 32];
    const int co0 = blockIdx.y * 32;
    const ll pb = seg_begin + (ll) blockIdx.x * range_len, pe = min(seg_end, pb + range_len);
    const ll R = N + T + 1;
    const int grp = threadIdx.x >> 6, t64 = threadIdx.x & 63;
    const int rq = t64 >> 3, cq = t64 & 7;                             // 8 row quads per pass of 64 threads
    constexpr int PASSES = (RQ + 7) / 8;
    float acc[PASSES][4][4];
#pragma unroll
    for (int ps = 0; ps < PASSES; ++ps)
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int b = 0; b < 4; ++b) acc[ps][a][b] = 0.f;
    for (ll p0 = pb; p0 < pe; p0 += KP) {
        for (int e = threadIdx.x; e < KP * RQ * 4; e += 256) {          // consecutive threads take consecutive locations of one row
            const int k = e % KP, row = e / KP;
            float v = 0.f;
            if (row < ROWS && p0 + k < pe) {
                const int tap = row / CIN, ci = row % CIN;
                v = __ldg(vals + (ll) ci * R + resolve_row(__ldg(nbr + (ll) tap * N + p0 + k), N, N + T));
            }
            xs[k][row >> 2].a[row & 3] = v;
        }
        for (int e = threadIdx.x; e < KP * 32; e += 256) {
            const int k = e % KP, co = e / KP;
            gs[k][co >> 2].a[co & 3] = (p0 + k < pe && co0 + co < cout) ? gout[(ll) (co0 + co) * ld_out + p0 + k] : 0.f;
        }
        __syncthreads();
#pragma unroll 4
        for (int k = grp * (KP / 4); k < (grp + 1) * (KP / 4); ++k) {
            const F4 g = gs[k][cq];
#pragma unroll
            for (int ps = 0; ps < PASSES; ++ps) {
                if (ps * 8 + rq < RQ) {
                    const F4 x = xs[k][ps * 8 + rq];
#pragma unroll
                    for (int a = 0; a < 4; ++a)
#pragma unroll
                        for (int b = 0; b < 4; ++b) acc[ps][a][b] = fmaf(x.a[a], g.a[b], acc[ps][a][b]);
                }
            }
        }
        __syncthreads();
    }
    // the four groups add their tiles one after the other: fixed order
    for (int gsel = 0; gsel < 4; ++gsel) {
        if (grp == gsel) {
#pragma unroll
            for (int ps = 0; ps < PASSES; ++ps)
                if (ps * 8 + rq < RQ)
#pragma unroll
                    for (int a = 0; a < 4; ++a)
#pragma unroll
                        for (int b = 0; b < 4; ++b) {
                            float* r = red + ((ps * 8 + rq) * 4 + a) * 32 + cq * 4 + b;
                            *r = gsel == 0 ? acc[ps][a][b] : *r + acc[ps][a][b];
                        }
        }
        __syncthreads();
    }
    float* dst = partial + (ll) blockIdx.x * cout * CIN * 27;
    for (int e = threadIdx.x; e < ROWS * 32; e += 256) {
        const int row = e >> 5, co = co0 + (e & 31);
        if (co < cout) dst[((ll) co * CIN + row % CIN) * 27 + row / CIN] = red[e];
    }
}

__global__ void small_reduce_partial_kernel(const float* __restrict__ partial, int nchunks, ll elems, float* __restrict__ dst) {
    const ll e = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= elems) return;
    float s = 0;
    for (int c = 0; c < nchunks; ++c) s += partial[(ll) c * elems + e];
    dst[e] += s;
}

} // namespace

bool aprnet_small_cin(int cin) { return cin <= 4; }

int aprnet_small_stage(const float* x, ll ld_x, ll n, const float* tree, ll ld_tree, ll t, int cin, float* vals, cudaStream_t st) {
    AprnetProfScope _prof("small_stage", st);
    small_stage_kernel<<<aprnet_ceil_div(n + t + 1, 256), 256, 0, st>>>(x, ld_x, n, tree, ld_tree, t, cin, vals);
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

int aprnet_small_forward(aprnet_apr* a, int dl, int cin, int cout, int slots, const float* vals, const float* w, float* out, ll ld_out, cudaStream_t st) {
    const AprPlan* plan = aprnet_get_plan(a, dl, st);
    if (!plan) return APRNET_ERR_CUDA;
    const SegTable segs = make_seg_table(aprnet_segments(a, dl, slots, false), 128);
    const int tiles = segs.tile_begin[segs.n];
    if (tiles == 0) return APRNET_OK;
    dim3 grid((unsigned) tiles, (unsigned) aprnet_ceil_div(cout, 32));
    char pname[64];
    snprintf(pname, sizeof(pname), "conv333_small_fwd:ci%d:co%d:dl%d", cin, cout, dl);
    AprnetProfScope _prof(pname, st);
    switch (cin) {
        case 1: conv333_small_forward_kernel<1><<<grid, 128, 0, st>>>(segs, plan->nbr, plan->n, plan->tree_size, vals, w, cout, out, ld_out); break;
        case 2: conv333_small_forward_kernel<2><<<grid, 128, 0, st>>>(segs, plan->nbr, plan->n, plan->tree_size, vals, w, cout, out, ld_out); break;
        case 3: conv333_small_forward_kernel<3><<<grid, 128, 0, st>>>(segs, plan->nbr, plan->n, plan->tree_size, vals, w, cout, out, ld_out); break;
        case 4: conv333_small_forward_kernel<4><<<grid, 128, 0, st>>>(segs, plan->nbr, plan->n, plan->tree_size, vals, w, cout, out, ld_out); break;
        default: aprnet_set_error("small-Cin path called with cin = %d", cin); return APRNET_ERR_ARG;
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

// grad_weights (slots, Cout, Cin, 27) is accumulated into; partial: aprnet_conv333_tc_dw_partial_elems() floats
int aprnet_small_backward_weights(aprnet_apr* a, int dl, int cin, int cout, int slots, const float* vals, const float* gout, ll ld_out,
                                  float* gw, float* partial, cudaStream_t st) {
    const AprPlan* plan = aprnet_get_plan(a, dl, st);
    if (!plan) return APRNET_ERR_CUDA;
    const ll elems = (ll) 27 * cin * cout;
    const ll max_ranges = aprnet_conv333_tc_dw_partial_elems(cin, cout) / elems;
    char pname[64];
    snprintf(pname, sizeof(pname), "conv333_small_dw:ci%d:co%d:dl%d", cin, cout, dl);
    for (const Segment& s : aprnet_segments(a, dl, slots, false)) {
        const ll len = s.end - s.begin;
        const int nranges = (int) std::max<ll>(1, std::min<ll>(std::min<ll>(max_ranges, 1184), (len + 511) / 512));
        const ll range_len = ((len + nranges - 1) / nranges + 63) / 64 * 64;
        dim3 grid((unsigned) nranges, (unsigned) aprnet_ceil_div(cout, 32));
        { AprnetProfScope _prof(pname, st);
        switch (cin) {
            case 1: conv333_small_dw_kernel<1><<<grid, 256, 0, st>>>(s.begin, s.end, range_len, plan->nbr, plan->n, plan->tree_size, vals, gout, ld_out, cout, partial); break;
            case 2: conv333_small_dw_kernel<2><<<grid, 256, 0, st>>>(s.begin, s.end, range_len, plan->nbr, plan->n, plan->tree_size, vals, gout, ld_out, cout, partial); break;
            case 3: conv333_small_dw_kernel<3><<<grid, 256, 0, st>>>(s.begin, s.end, range_len, plan->nbr, plan->n, plan->tree_size, vals, gout, ld_out, cout, partial); break;
            case 4: conv333_small_dw_kernel<4><<<grid, 256, 0, st>>>(s.begin, s.end, range_len, plan->nbr, plan->n, plan->tree_size, vals, gout, ld_out, cout, partial); break;
            default: aprnet_set_error("small-Cin path called with cin = %d", cin); return APRNET_ERR_ARG;
        }
        }
        { AprnetProfScope _prof("conv333_dw_reduce", st);
        small_reduce_partial_kernel<<<aprnet_ceil_div(elems, 256), 256, 0, st>>>(partial, nranges, elems, gw + (ll) s.slot * elems);
        }
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}
