// Weight gradient of the 1x1x1 particle convolution for callers that cannot allocate device memory.
//
// Some hosts of this library never get to call cudaMalloc on the path where they invoke it: a serving
// process whose own arena owns the whole device, a plug-in that runs under a fixed memory budget
// negotiated at start-up, or a latency-critical loop in which an allocation's implicit device-wide
// synchronisation is not acceptable.  The regular entry point (aprnet_conv111_backward_weights) asks
// such a caller for a workspace it has no means to provide.  This variant carries its workspace inside
// the library image instead: a fixed array in device global memory that every GPU loading the library
// holds until the process exits (APRNET_STATIC_SCRATCH_BYTES, 4 MiB).
//
// Consequences of sharing one array:
//   * the array keeps whatever the previous call left in it.  Nothing here relies on it starting at
//     zero: the first kernel overwrites every element that the second one reads;
//   * two calls that overlap on the same GPU (different streams, or different host threads) race on
//     the array and produce garbage.  Serialise them.
//   * problem sizes whose block-partial sums do not fit are rejected with APRNET_ERR_UNSUPPORTED.
//
// The device address of the array is looked up with cudaGetSymbolAddress the first time the entry
// point runs on a given device (with that device current) and cached per device.  That first call
// should be made before any stream capture is started.
#include "apr_device.cuh"
#include <mutex>

namespace {

typedef long long ll;

constexpr ll STATIC_SCRATCH_ELEMS = 1ll << 20;                      // floats
static __device__ __align__(256) float g_static_scratch[STATIC_SCRATCH_ELEMS];

constexpr int MAX_DEVICES = 64;
float* g_scratch_addr[MAX_DEVICES] = {nullptr};
std::mutex g_scratch_mutex;

// Device address of the scratch array on the CURRENT device.  In host code the symbol name is only a
// handle; the address a kernel can use has to come from the runtime.
int static_scratch(float** out) {
    int dev = -1;
    APRNET_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) { aprnet_set_error("static scratch: device index %d out of range", dev); return APRNET_ERR_UNSUPPORTED; }
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_addr[dev]) {
        float* p = nullptr;
        APRNET_CUDA_CHECK(cudaGetSymbolAddress((void**) &p, g_static_scratch));
        g_scratch_addr[dev] = p;
    }
    *out = g_scratch_addr[dev];
    return APRNET_OK;
}

constexpr int STATIC_MAX_CHUNKS = 64;
constexpr int STATIC_MAX_SEGS = APRNET_MAX_LEVELS;

// partial[chunk][o][i] = sum over the chunk's particles of gout[o][p] * in[i][p]; 16x16 tile per block
__global__ void __launch_bounds__(256) conv111_dw_static_partial(ll seg_begin, ll seg_end, ll chunk_len,
                                                                 const float* __restrict__ in, ll ld_in,
                                                                 const float* __restrict__ gout, ll ld_out,
                                                                 float* __restrict__ partial, int cin, int cout) {
    __shared__ float gs[16][65];
    __shared__ float xs[16][65];
    const int nib = (cin + 15) / 16;
    const int ob = blockIdx.y / nib, ib = blockIdx.y % nib;
    const ll pb = seg_begin + (ll) blockIdx.x * chunk_len;
    const ll pe = min(seg_end, pb + chunk_len);
    const int ti = threadIdx.x & 15, to = threadIdx.x >> 4;
    float acc = 0.f;
    for (ll p0 = pb; p0 < pe; p0 += 64) {
        for (int e = threadIdx.x; e < 16 * 64; e += 256) {
            const int r = e >> 6, k = e & 63;
            const bool inr = p0 + k < pe;
            const int o = ob * 16 + r, i = ib * 16 + r;
            gs[r][k] = (inr && o < cout) ? gout[(ll) o * ld_out + p0 + k] : 0.f;
            xs[r][k] = (inr && i < cin) ? in[(ll) i * ld_in + p0 + k] : 0.f;
        }
        __syncthreads();
#pragma unroll 16
        for (int k = 0; k < 64; ++k) acc = fmaf(gs[to][k], xs[ti][k], acc);
        __syncthreads();
    }
    const int o = ob * 16 + to, i = ib * 16 + ti;
    if (o < cout && i < cin) partial[(ll) blockIdx.x * cout * cin + (ll) o * cin + i] = acc;
}

__global__ void conv111_dw_static_reduce(const float* __restrict__ partial, int nchunks, ll elems, float* __restrict__ dst) {
    const ll e = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= elems) return;
    float s = 0.f;
    for (int c = 0; c < nchunks; ++c) s += partial[(ll) c * elems + e];
    dst[e] += s;
}

} // namespace

extern "C" int64_t aprnet_static_scratch_bytes(void) { return (int64_t) (STATIC_SCRATCH_ELEMS * sizeof(float)); }

extern "C" int aprnet_conv111_backward_weights_static(const aprnet_apr* a, int dl, int cin, int cout, int S,
                                                      const float* in, int64_t ld_in, const float* gout, int64_t ld_out,
                                                      float* gw, void* stream) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && in && gout && gw && cin > 0 && cout > 0 && S > 0, "bad argument");
    APRNET_DEVICE_CHECK(a);
    APRNET_ARG_CHECK(ld_in >= a->number_parts(dl) && ld_out >= a->number_parts(dl), "leading dimension too small");
    const ll elems = (ll) cin * cout;
    if (elems * 4 > STATIC_SCRATCH_ELEMS) {
        aprnet_set_error("aprnet_conv111_backward_weights_static: cin*cout = %lld exceeds the built-in workspace "
                         "(limit %lld); use aprnet_conv111_backward_weights with a caller-provided workspace",
                         elems, (ll) (STATIC_SCRATCH_ELEMS / 4));
        return APRNET_ERR_UNSUPPORTED;
    }
    float* scratch = nullptr;
    const int rc = static_scratch(&scratch);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t) stream;
    const int max_chunks = (int) std::min<ll>(STATIC_MAX_CHUNKS, STATIC_SCRATCH_ELEMS / elems);

    // level ranges that share a stencil (same rule as the regular entry point), without heap use:
    // level l -> stencil min(cml - l, S - 1); the upgraded tree nodes ride with level cml.
    const int cml = a->cml(dl);
    const ll n = a->number_parts(dl);
    ll seg_begin[STATIC_MAX_SEGS], seg_end[STATIC_MAX_SEGS];
    int seg_slot[STATIC_MAX_SEGS], nseg = 0;
    for (int l = a->meta.level_min; l <= cml; ++l) {
        const ll b = a->meta.lvl_begin[l], e = (l == cml) ? n : a->meta.lvl_begin[l + 1];
        const int slot = std::min(cml - l, S - 1);
        if (e <= b) continue;
        if (nseg > 0 && seg_slot[nseg - 1] == slot && seg_end[nseg - 1] == b) seg_end[nseg - 1] = e;
        else { seg_begin[nseg] = b; seg_end[nseg] = e; seg_slot[nseg] = slot; ++nseg; }
    }
    for (int s = 0; s < nseg; ++s) {
        const ll len = seg_end[s] - seg_begin[s];
        const int nchunks = (int) std::min<ll>(max_chunks, (len + 2047) / 2048);
        const ll chunk_len = ((len + nchunks - 1) / nchunks + 63) / 64 * 64;
        dim3 grid((unsigned) nchunks, (unsigned) (aprnet_ceil_div(cout, 16) * aprnet_ceil_div(cin, 16)));
        conv111_dw_static_partial<<<grid, 256, 0, st>>>(seg_begin[s], seg_end[s], chunk_len, in, ld_in, gout, ld_out, scratch, cin, cout);
        conv111_dw_static_reduce<<<aprnet_ceil_div(elems, 256), 256, 0, st>>>(scratch, nchunks, elems, gw + (ll) seg_slot[s] * elems);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}
