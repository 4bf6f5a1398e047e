// GroupNorm + ReLU over (batch, channels, particles) feature tensors, forward and backward.
//
// The reference's network blocks apply torch.nn.GroupNorm followed by ReLU to every convolution
// output (apr_models/apr_models/unet/unet_parts.py:18-26), with one group per channel by default.  On a
// (B, C, N) tensor with N in the tens of millions that is B*G rows of C/G*N elements; the stock
// kernels reduce one row per thread block, so a handful of blocks walk gigabytes serially.  Here the
// statistics are a two-stage reduction (many blocks per row, double-precision partial sums, fixed
// order: deterministic), normalisation and ReLU are one fused pass, and the backward pass is one
// reduction pass plus one elementwise pass; the ReLU mask is recomputed from the input instead of
// being stored.  Same arithmetic as torch: biased variance, eps inside the square root, statistics
// over the whole (padded) particle axis.
#include "apr_device.cuh"
#include <algorithm>

namespace {

typedef long long ll;
constexpr int GN_TPB = 256;
constexpr int GN_MAX_CHUNKS = 512;

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    return v;
}

// block-wide sum of two doubles; result valid in thread 0
__device__ __forceinline__ void block_sum2(double& a, double& b) {
    __shared__ double sa[GN_TPB / 32], sb[GN_TPB / 32];
    a = warp_sum(a); b = warp_sum(b);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    if (l == 0) { sa[w] = a; sb[w] = b; }
    __syncthreads();
    if (w == 0) {
        a = l < GN_TPB / 32 ? sa[l] : 0.0;
        b = l < GN_TPB / 32 ? sb[l] : 0.0;
        a = warp_sum(a); b = warp_sum(b);
    }
    __syncthreads();
}

// stage 1 of the statistics: partial[row][chunk] = (sum x, sum x^2) over the chunk
template<typename T>
__global__ void __launch_bounds__(GN_TPB) gn_partial_stats_kernel(const T* __restrict__ x, ll n, ll chunk_len, double* __restrict__ partial, int nchunks) {
    const ll row = blockIdx.y;
    const ll b0 = (ll) blockIdx.x * chunk_len, b1 = min(n, b0 + chunk_len);
    const T* xr = x + row * n;
    double s = 0.0, ss = 0.0;
    ll i = b0 + threadIdx.x;
    for (; i + 3 * GN_TPB < b1; i += 4 * GN_TPB) {        // four independent loads in flight; same summation order
        T v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = xr[i + u * GN_TPB];
#pragma unroll
        for (int u = 0; u < 4; ++u) { const double d = (double) v[u]; s += d; ss += d * d; }
    }
    for (; i < b1; i += GN_TPB) { const double v = (double) xr[i]; s += v; ss += v * v; }
    block_sum2(s, ss);
    if (threadIdx.x == 0) { partial[(row * nchunks + blockIdx.x) * 2] = s; partial[(row * nchunks + blockIdx.x) * 2 + 1] = ss; }
}

// stage 2: one thread per (batch item, group): mean and 1/sqrt(var + eps)
template<typename T>
__global__ void gn_finalize_stats_kernel(const double* __restrict__ partial, int nchunks, int rows_per_group, ll n, int ngroups_total,
                                         double eps, T* __restrict__ mean, T* __restrict__ rstd) {
    const int g = blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= ngroups_total) return;
    double s = 0.0, ss = 0.0;
    for (int r = 0; r < rows_per_group; ++r)
        for (int c = 0; c < nchunks; ++c) {
            const ll o = (((ll) g * rows_per_group + r) * nchunks + c) * 2;
            s += partial[o]; ss += partial[o + 1];
        }
    const double m = (double) rows_per_group * (double) n;
    const double mu = s / m;
    const double var = fmax(ss / m - mu * mu, 0.0);
    mean[g] = (T) mu;
    rstd[g] = (T) (1.0 / sqrt(var + eps));
}

// y = max((x - mean) * rstd * gamma + beta, 0)
template<typename T>
__global__ void __launch_bounds__(GN_TPB) gn_relu_apply_kernel(const T* __restrict__ x, ll n, int C, int ch_per_group, const T* __restrict__ gamma,
                                                               const T* __restrict__ beta, const T* __restrict__ mean, const T* __restrict__ rstd,
                                                               T* __restrict__ y, int relu) {
    const ll row = blockIdx.y;                       // b * C + c
    const int c = (int) (row % C);
    const ll g = row / ch_per_group;                 // (b * C + c) / ch_per_group = b * G + c / ch_per_group
    const T mu = mean[g], rs = rstd[g];
    const T ga = gamma ? gamma[c] : T(1), be = beta ? beta[c] : T(0);
    const T* xr = x + row * n;
    T* yr = y + row * n;
    for (ll i = (ll) blockIdx.x * GN_TPB + threadIdx.x; i < n; i += (ll) gridDim.x * GN_TPB) {
        const T v = (xr[i] - mu) * rs * ga + be;        // same expression as the backward pass uses for the ReLU mask
        yr[i] = (relu && v < T(0)) ? T(0) : v;
    }
}

// backward stage 1: partial[row][chunk] = (sum dy_eff, sum dy_eff * xhat), dy_eff = dy * [y > 0]
template<typename T>
__global__ void __launch_bounds__(GN_TPB) gn_backward_partial_kernel(const T* __restrict__ x, const T* __restrict__ dy, ll n, ll chunk_len, int C,
                                                                     int ch_per_group, const T* __restrict__ gamma, const T* __restrict__ beta,
                                                                     const T* __restrict__ mean, const T* __restrict__ rstd,
                                                                     double* __restrict__ partial, int nchunks, int relu) {
    const ll row = blockIdx.y;
    const int c = (int) (row % C);
    const ll g = row / ch_per_group;
    const T mu = mean[g], rs = rstd[g];
    const T ga = gamma ? gamma[c] : T(1), be = beta ? beta[c] : T(0);
    const ll b0 = (ll) blockIdx.x * chunk_len, b1 = min(n, b0 + chunk_len);
    const T* xr = x + row * n;
    const T* dr = dy + row * n;
    double s = 0.0, sx = 0.0;
    auto add = [&](T xv, T d) {
        const T xh = (xv - mu) * rs;
        if (relu && xh * ga + be <= T(0)) d = T(0);
        s += (double) d; sx += (double) d * (double) xh;
    };
    ll i = b0 + threadIdx.x;
    for (; i + 3 * GN_TPB < b1; i += 4 * GN_TPB) {        // eight independent loads in flight; same summation order
        T xv[4], dv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) { xv[u] = xr[i + u * GN_TPB]; dv[u] = dr[i + u * GN_TPB]; }
#pragma unroll
        for (int u = 0; u < 4; ++u) add(xv[u], dv[u]);
    }
    for (; i < b1; i += GN_TPB) add(xr[i], dr[i]);
    block_sum2(s, sx);
    if (threadIdx.x == 0) { partial[(row * nchunks + blockIdx.x) * 2] = s; partial[(row * nchunks + blockIdx.x) * 2 + 1] = sx; }
}

// backward stage 2a: per row sums A = sum dy_eff, Bx = sum dy_eff * xhat  (row_sums[row] = (A, Bx))
__global__ void gn_backward_rows_kernel(const double* __restrict__ partial, int nchunks, ll rows, double* __restrict__ row_sums) {
    const ll r = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    double a = 0.0, b = 0.0;
    for (int c = 0; c < nchunks; ++c) { a += partial[(r * nchunks + c) * 2]; b += partial[(r * nchunks + c) * 2 + 1]; }
    row_sums[r * 2] = a; row_sums[r * 2 + 1] = b;
}

// backward stage 2b: dgamma[c] = sum_b Bx, dbeta[c] = sum_b A; group terms mA, mB per (b, g)
template<typename T>
__global__ void gn_backward_finalize_kernel(const double* __restrict__ row_sums, int B, int C, int ch_per_group, ll n, const T* __restrict__ gamma,
                                            T* __restrict__ dgamma, T* __restrict__ dbeta, T* __restrict__ group_terms) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int G = C / ch_per_group;
    if (i < C) {
        double a = 0.0, b = 0.0;
        for (int bb = 0; bb < B; ++bb) { a += row_sums[((ll) bb * C + i) * 2]; b += row_sums[((ll) bb * C + i) * 2 + 1]; }
        if (dbeta) dbeta[i] = (T) a;
        if (dgamma) dgamma[i] = (T) b;
    }
    if (i < B * G) {
        const int bb = i / G, g = i % G;
        double a = 0.0, b = 0.0;
        for (int k = 0; k < ch_per_group; ++k) {
            const int c = g * ch_per_group + k;
            const double ga = gamma ? (double) gamma[c] : 1.0;
            a += ga * row_sums[((ll) bb * C + c) * 2]; b += ga * row_sums[((ll) bb * C + c) * 2 + 1];
        }
        const double m = (double) ch_per_group * (double) n;
        group_terms[2 * i] = (T) (a / m); group_terms[2 * i + 1] = (T) (b / m);
    }
}

// backward stage 3: dx = rstd * (dy_eff * gamma - mA - xhat * mB)
template<typename T>
__global__ void __launch_bounds__(GN_TPB) gn_backward_apply_kernel(const T* __restrict__ x, const T* __restrict__ dy, ll n, int C, int ch_per_group,
                                                                   const T* __restrict__ gamma, const T* __restrict__ beta, const T* __restrict__ mean,
                                                                   const T* __restrict__ rstd, const T* __restrict__ group_terms, T* __restrict__ dx, int relu) {
    const ll row = blockIdx.y;
    const int c = (int) (row % C);
    const ll g = row / ch_per_group;
    const T mu = mean[g], rs = rstd[g], mA = group_terms[2 * g], mB = group_terms[2 * g + 1];
    const T ga = gamma ? gamma[c] : T(1), be = beta ? beta[c] : T(0);
    const T* xr = x + row * n;
    const T* dr = dy + row * n;
    T* o = dx + row * n;
    for (ll i = (ll) blockIdx.x * GN_TPB + threadIdx.x; i < n; i += (ll) gridDim.x * GN_TPB) {
        const T xh = (xr[i] - mu) * rs;
        T d = dr[i];
        if (relu && xh * ga + be <= T(0)) d = T(0);
        o[i] = rs * (d * ga - mA - xh * mB);
    }
}

inline int gn_chunks(ll n, ll rows) {
    ll want = std::max<ll>(1, (148ll * 8 + rows - 1) / rows);
    want = std::min<ll>(want, (n + 4095) / 4096);
    return (int) std::max<ll>(1, std::min<ll>(GN_MAX_CHUNKS, want));
}

template<typename T>
int gn_forward(int B, int C, ll n, int groups, const T* x, const T* gamma, const T* beta, double eps, T* y, T* mean, T* rstd, double* ws, int relu, cudaStream_t st) {
    const ll rows = (ll) B * C;
    const int cpg = C / groups;
    const int nchunks = gn_chunks(n, rows);
    const ll chunk_len = (n + nchunks - 1) / nchunks;
    { AprnetProfScope _p("groupnorm_stats", st);
    gn_partial_stats_kernel<T><<<dim3(nchunks, (unsigned) rows), GN_TPB, 0, st>>>(x, n, chunk_len, ws, nchunks);
    gn_finalize_stats_kernel<T><<<aprnet_ceil_div((ll) B * groups, 128), 128, 0, st>>>(ws, nchunks, cpg, n, B * groups, eps, mean, rstd);
    }
    const int gx = (int) std::max<ll>(1, std::min<ll>((n + GN_TPB * 8 - 1) / (GN_TPB * 8), 4096));
    { AprnetProfScope _p("groupnorm_relu_apply", st);
    gn_relu_apply_kernel<T><<<dim3(gx, (unsigned) rows), GN_TPB, 0, st>>>(x, n, C, cpg, gamma, beta, mean, rstd, y, relu);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

template<typename T>
int gn_backward(int B, int C, ll n, int groups, const T* x, const T* dy, const T* gamma, const T* beta, const T* mean, const T* rstd,
                T* dx, T* dgamma, T* dbeta, double* ws, int relu, cudaStream_t st) {
    const ll rows = (ll) B * C;
    const int cpg = C / groups;
    const int nchunks = gn_chunks(n, rows);
    const ll chunk_len = (n + nchunks - 1) / nchunks;
    double* row_sums = ws + rows * nchunks * 2;
    T* group_terms = reinterpret_cast<T*>(row_sums + rows * 2);
    { AprnetProfScope _p("groupnorm_bwd_reduce", st);
    gn_backward_partial_kernel<T><<<dim3(nchunks, (unsigned) rows), GN_TPB, 0, st>>>(x, dy, n, chunk_len, C, cpg, gamma, beta, mean, rstd, ws, nchunks, relu);
    gn_backward_rows_kernel<<<aprnet_ceil_div(rows, 128), 128, 0, st>>>(ws, nchunks, rows, row_sums);
    gn_backward_finalize_kernel<T><<<aprnet_ceil_div(std::max<ll>(C, (ll) B * groups), 128), 128, 0, st>>>(row_sums, B, C, cpg, n, gamma, dgamma, dbeta, group_terms);
    }
    const int gx = (int) std::max<ll>(1, std::min<ll>((n + GN_TPB * 8 - 1) / (GN_TPB * 8), 4096));
    { AprnetProfScope _p("groupnorm_bwd_apply", st);
    gn_backward_apply_kernel<T><<<dim3(gx, (unsigned) rows), GN_TPB, 0, st>>>(x, dy, n, C, cpg, gamma, beta, mean, rstd, group_terms, dx, relu);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

} // namespace

// bytes of workspace for either direction
extern "C" int64_t aprnet_groupnorm_workspace_bytes(int batch, int channels, int groups) {
    const ll rows = (ll) batch * channels;
    return (int64_t) ((rows * GN_MAX_CHUNKS * 2 + rows * 2) * sizeof(double) + (ll) batch * groups * 2 * sizeof(double) + 256);
}

extern "C" int aprnet_groupnorm_relu_forward(int dtype, int batch, int channels, int64_t n, int groups, const void* x, const void* gamma,
                                             const void* beta, double eps, void* y, void* mean, void* rstd, void* workspace, int relu, void* stream) {
    APRNET_ARG_CHECK(batch > 0 && channels > 0 && n > 0 && groups > 0 && channels % groups == 0 && x && y && mean && rstd && workspace, "bad argument");
    cudaStream_t st = (cudaStream_t) stream;
    if (dtype == APRNET_F32) return gn_forward<float>(batch, channels, n, groups, (const float*) x, (const float*) gamma, (const float*) beta, eps, (float*) y, (float*) mean, (float*) rstd, (double*) workspace, relu, st);
    if (dtype == APRNET_F64) return gn_forward<double>(batch, channels, n, groups, (const double*) x, (const double*) gamma, (const double*) beta, eps, (double*) y, (double*) mean, (double*) rstd, (double*) workspace, relu, st);
    aprnet_set_error("aprnet_groupnorm_relu_forward: unknown dtype %d", dtype);
    return APRNET_ERR_ARG;
}

extern "C" int aprnet_groupnorm_relu_backward(int dtype, int batch, int channels, int64_t n, int groups, const void* x, const void* grad_y,
                                              const void* gamma, const void* beta, const void* mean, const void* rstd, void* grad_x,
                                              void* grad_gamma, void* grad_beta, void* workspace, int relu, void* stream) {
    APRNET_ARG_CHECK(batch > 0 && channels > 0 && n > 0 && groups > 0 && channels % groups == 0 && x && grad_y && mean && rstd && grad_x && workspace, "bad argument");
    cudaStream_t st = (cudaStream_t) stream;
    if (dtype == APRNET_F32) return gn_backward<float>(batch, channels, n, groups, (const float*) x, (const float*) grad_y, (const float*) gamma, (const float*) beta, (const float*) mean, (const float*) rstd, (float*) grad_x, (float*) grad_gamma, (float*) grad_beta, (double*) workspace, relu, st);
    if (dtype == APRNET_F64) return gn_backward<double>(batch, channels, n, groups, (const double*) x, (const double*) grad_y, (const double*) gamma, (const double*) beta, (const double*) mean, (const double*) rstd, (double*) grad_x, (double*) grad_gamma, (double*) grad_beta, (double*) workspace, relu, st);
    aprnet_set_error("aprnet_groupnorm_relu_backward: unknown dtype %d", dtype);
    return APRNET_ERR_ARG;
}

// ---- split forms: the caller combines the sums of several devices before the statistics are applied --------
// (one z-slab of an APR per GPU: every rank sums over the particles it owns, the sums are all-reduced, every rank
// applies the same mean / rstd).  row_sums: double [batch * channels][2].
template<typename T>
static int gn_row_sums(int B, int C, ll n, const T* x, double* ws, double* row_sums, cudaStream_t st) {
    const ll rows = (ll) B * C;
    const int nchunks = gn_chunks(n, rows);
    const ll chunk_len = (n + nchunks - 1) / nchunks;
    { AprnetProfScope _p("groupnorm_stats", st);
    gn_partial_stats_kernel<T><<<dim3(nchunks, (unsigned) rows), GN_TPB, 0, st>>>(x, n, chunk_len, ws, nchunks);
    gn_backward_rows_kernel<<<aprnet_ceil_div(rows, 128), 128, 0, st>>>(ws, nchunks, rows, row_sums);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

template<typename T>
static int gn_apply(int B, int C, ll n, int groups, const T* x, const T* gamma, const T* beta, const T* mean, const T* rstd, T* y, int relu, cudaStream_t st) {
    const ll rows = (ll) B * C;
    const int gx = (int) std::max<ll>(1, std::min<ll>((n + GN_TPB * 8 - 1) / (GN_TPB * 8), 4096));
    { AprnetProfScope _p("groupnorm_relu_apply", st);
    gn_relu_apply_kernel<T><<<dim3(gx, (unsigned) rows), GN_TPB, 0, st>>>(x, n, C, C / groups, gamma, beta, mean, rstd, y, relu);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

template<typename T>
static int gn_bwd_row_sums(int B, int C, ll n, int groups, const T* x, const T* dy, const T* gamma, const T* beta, const T* mean, const T* rstd,
                           double* ws, double* row_sums, int relu, cudaStream_t st) {
    const ll rows = (ll) B * C;
    const int nchunks = gn_chunks(n, rows);
    const ll chunk_len = (n + nchunks - 1) / nchunks;
    { AprnetProfScope _p("groupnorm_bwd_reduce", st);
    gn_backward_partial_kernel<T><<<dim3(nchunks, (unsigned) rows), GN_TPB, 0, st>>>(x, dy, n, chunk_len, C, C / groups, gamma, beta, mean, rstd, ws, nchunks, relu);
    gn_backward_rows_kernel<<<aprnet_ceil_div(rows, 128), 128, 0, st>>>(ws, nchunks, rows, row_sums);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

template<typename T>
static int gn_bwd_apply(int B, int C, ll n, int groups, const T* x, const T* dy, const T* gamma, const T* beta, const T* mean, const T* rstd,
                        const T* group_terms, T* dx, int relu, cudaStream_t st) {
    const ll rows = (ll) B * C;
    const int gx = (int) std::max<ll>(1, std::min<ll>((n + GN_TPB * 8 - 1) / (GN_TPB * 8), 4096));
    { AprnetProfScope _p("groupnorm_bwd_apply", st);
    gn_backward_apply_kernel<T><<<dim3(gx, (unsigned) rows), GN_TPB, 0, st>>>(x, dy, n, C, C / groups, gamma, beta, mean, rstd, group_terms, dx, relu);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

#define GN_DISPATCH(F32_CALL, F64_CALL)                                               \
    if (dtype == APRNET_F32) return F32_CALL;                                         \
    if (dtype == APRNET_F64) return F64_CALL;                                         \
    aprnet_set_error("%s: unknown dtype %d", __func__, dtype);                       \
    return APRNET_ERR_ARG;

extern "C" int aprnet_groupnorm_row_sums(int dtype, int batch, int channels, int64_t n, const void* x, void* workspace, double* row_sums, void* stream) {
    APRNET_ARG_CHECK(batch > 0 && channels > 0 && n > 0 && x && workspace && row_sums, "bad argument");
    cudaStream_t st = (cudaStream_t) stream;
    GN_DISPATCH(gn_row_sums<float>(batch, channels, n, (const float*) x, (double*) workspace, row_sums, st),
                gn_row_sums<double>(batch, channels, n, (const double*) x, (double*) workspace, row_sums, st))
}

extern "C" int aprnet_groupnorm_relu_apply(int dtype, int batch, int channels, int64_t n, int groups, const void* x, const void* gamma, const void* beta,
                                           const void* mean, const void* rstd, void* y, int relu, void* stream) {
    APRNET_ARG_CHECK(batch > 0 && channels > 0 && n > 0 && groups > 0 && channels % groups == 0 && x && y && mean && rstd, "bad argument");
    cudaStream_t st = (cudaStream_t) stream;
    GN_DISPATCH(gn_apply<float>(batch, channels, n, groups, (const float*) x, (const float*) gamma, (const float*) beta, (const float*) mean, (const float*) rstd, (float*) y, relu, st),
                gn_apply<double>(batch, channels, n, groups, (const double*) x, (const double*) gamma, (const double*) beta, (const double*) mean, (const double*) rstd, (double*) y, relu, st))
}

extern "C" int aprnet_groupnorm_backward_row_sums(int dtype, int batch, int channels, int64_t n, int groups, const void* x, const void* grad_y,
                                                  const void* gamma, const void* beta, const void* mean, const void* rstd, void* workspace,
                                                  double* row_sums, int relu, void* stream) {
    APRNET_ARG_CHECK(batch > 0 && channels > 0 && n > 0 && groups > 0 && channels % groups == 0 && x && grad_y && mean && rstd && workspace && row_sums, "bad argument");
    cudaStream_t st = (cudaStream_t) stream;
    GN_DISPATCH(gn_bwd_row_sums<float>(batch, channels, n, groups, (const float*) x, (const float*) grad_y, (const float*) gamma, (const float*) beta, (const float*) mean, (const float*) rstd, (double*) workspace, row_sums, relu, st),
                gn_bwd_row_sums<double>(batch, channels, n, groups, (const double*) x, (const double*) grad_y, (const double*) gamma, (const double*) beta, (const double*) mean, (const double*) rstd, (double*) workspace, row_sums, relu, st))
}

extern "C" int aprnet_groupnorm_backward_apply(int dtype, int batch, int channels, int64_t n, int groups, const void* x, const void* grad_y,
                                               const void* gamma, const void* beta, const void* mean, const void* rstd, const void* group_terms,
                                               void* grad_x, int relu, void* stream) {
    APRNET_ARG_CHECK(batch > 0 && channels > 0 && n > 0 && groups > 0 && channels % groups == 0 && x && grad_y && mean && rstd && group_terms && grad_x, "bad argument");
    cudaStream_t st = (cudaStream_t) stream;
    GN_DISPATCH(gn_bwd_apply<float>(batch, channels, n, groups, (const float*) x, (const float*) grad_y, (const float*) gamma, (const float*) beta, (const float*) mean, (const float*) rstd, (const float*) group_terms, (float*) grad_x, relu, st),
                gn_bwd_apply<double>(batch, channels, n, groups, (const double*) x, (const double*) grad_y, (const double*) gamma, (const double*) beta, (const double*) mean, (const double*) rstd, (const double*) group_terms, (double*) grad_x, relu, st))
}
