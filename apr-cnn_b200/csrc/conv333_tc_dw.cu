// Weight gradient of the 3x3x3 particle convolution on the tensor cores (tcgen05 + TMEM), bf16
// operands with fp32 accumulation, deterministic.
//
//     dW[tap][ci][co] = sum over output locations p of  X[nbr(tap, p)][ci] * dO[p][co]
//
// is a GEMM whose contraction index is the particle.  Per block: a contiguous range of locations of
// one level, one block of KCI input channels and one block of NCO output channels.  The accumulator
// D[(tap, ci)][co] lives in TMEM for the whole range: 128-row tiles of 128/KCI taps x KCI channels,
// ceil(27 / (128/KCI)) tiles side by side, NCO fp32 columns each (<= 448 of the 512 columns).  Both
// operands are MN-major: the gathered neighbour rows of a tap ([8-channel chunk][particle][8]) are the
// A operand with M = channels and K = particles as they lie in shared memory after the 16-byte
// cp.async row copies, and the dO rows are the B operand in the same arrangement.  Each block writes
// its partial sums once; a second pass adds the ranges in ascending order (no atomics).
// Reference arithmetic: pyapr/aprnet/src/helpers.hpp:624-702 (accumulate_convolution_backward, dW part).
#include "apr_device.cuh"
#include <cuda_bf16.h>
#include <algorithm>

namespace {

typedef long long ll;
constexpr int PT = 128;            // particles per staged chunk (= threads per block)
constexpr int XS = 4;              // ring of gathered-row stages
constexpr int XAHEAD = 2;          // stages of copies in flight (ring slots are refilled two MMA steps after they were read)
constexpr unsigned SPIN_LIMIT = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t) __cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
#ifdef APRNET_TC_CG
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
#else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src) : "memory");
#endif
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template<int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                 "selp.b32 %0, 1, 0, p;\n\t}\n" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (unsigned it = 0; it < SPIN_LIMIT; ++it)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory"); }
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() { asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
                 ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory"); }

// MN-major, no swizzle: core matrix = 8 K-rows x 16 bytes (8 M/N elements); consecutive K rows are
// 16 bytes apart; LBO = byte distance between groups of 8 K rows, SBO = between 8-element M/N chunks.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t) ((saddr >> 4) & 0x3FFF) | ((uint64_t) ((lbo >> 4) & 0x3FFF) << 16) |
           ((uint64_t) ((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46);
}
// D fp32, A/B bf16, both MN-major, M = 128, N = n
__host__ __device__ constexpr uint32_t make_idesc_mn(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) | ((uint32_t) (n >> 3) << 17) | ((uint32_t) (128 >> 4) << 24);
}

struct DwParams {
    ll seg_begin, seg_end, range_len;      // output locations [seg_begin, seg_end) split into ranges of range_len
    const int32_t* nbr; ll N;
    const __nv_bfloat16* xrows; int xpad;  // packed inputs [N + T + 1][xpad]; tree rows start at tree_base, zeros at zero_row
    ll tree_base, zero_row;
    const __nv_bfloat16* grows; int gpad;  // packed dO [N + 1][gpad], zeros at row g_zero_row
    ll g_zero_row;
    float* partial;                        // [range][cout][cin][27]
    int cin, cout, ci_blocks;
    int* error_flag;
};

template<int KCI, int NCO>
__global__ void __launch_bounds__(PT) conv333_tc_dw_kernel(const DwParams P) {
    constexpr int TPM = 128 / KCI;                      // taps per 128-row accumulator tile
    constexpr int MT = (27 + TPM - 1) / TPM;            // accumulator tiles
    constexpr int XCH = KCI / 8;                        // 16-byte chunks per gathered row
    constexpr int X_BYTES = 128 * PT * 2;               // one stage: TPM taps x KCI channels x PT particles
    constexpr int G_BYTES = NCO * PT * 2;
    constexpr int NEED_COLS = MT * NCO + (NCO < 32 ? 32 - NCO : 0);     // accumulators are read back 32 columns at a time
    constexpr int TMEM_COLS = (NEED_COLS <= 32) ? 32 : (NEED_COLS <= 64) ? 64 : (NEED_COLS <= 128) ? 128 : (NEED_COLS <= 256) ? 256 : 512;
    static_assert(NEED_COLS <= 512, "accumulators must fit the 512 TMEM columns");
    constexpr uint32_t IDESC = make_idesc_mn(NCO);

    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* xs = smem;                                                   // XS * X_BYTES
    unsigned char* gs = xs + XS * X_BYTES;                                      // 2 * G_BYTES
    int32_t* idx_s = reinterpret_cast<int32_t*>(gs + 2 * G_BYTES);             // 2 x [27][PT] source rows (by chunk parity)
    uint64_t* bars = reinterpret_cast<uint64_t*>(idx_s + 2 * 27 * PT);         // XS + 1
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + XS + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cib = blockIdx.y % P.ci_blocks, cob = blockIdx.y / P.ci_blocks;
    const ll pb = P.seg_begin + (ll) blockIdx.x * P.range_len;
    const ll pe = min(P.seg_end, pb + P.range_len);
    const int nchunks = pe > pb ? (int) ((pe - pb + PT - 1) / PT) : 0;
    const int nstages = nchunks * MT;

    if (tid == 0) {
        for (int i = 0; i <= XS; ++i) mbar_init(smem_u32(bars + i), 1);
        fence_mbar_init();
    }
    if (warp == 0) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_slot;

    auto load_idx = [&](int chunk) {          // source rows of this thread's particle for all taps
        const ll p = pb + (ll) chunk * PT + tid;
        int32_t* dst = idx_s + (chunk & 1) * 27 * PT;
        int32_t q[27];          // one batch of independent loads, then the dependent stores
#pragma unroll
        for (int tap = 0; tap < 27; ++tap) q[tap] = (p < pe) ? __ldg(P.nbr + (ll) tap * P.N + p) : APRNET_NONE;
#pragma unroll
        for (int tap = 0; tap < 27; ++tap) {
            ll r = P.zero_row;
            if (q[tap] >= 0) r = q[tap]; else if (q[tap] != APRNET_NONE) r = P.tree_base + aprnet_dec_tree(q[tap]);
            dst[tap * PT + tid] = (int32_t) r;
        }
    };
    auto issue_loads = [&](int stage) {
        const int chunk = stage / MT, mt = stage % MT;
        unsigned char* x_s = xs + (stage % XS) * X_BYTES;
        const int32_t* idx = idx_s + (chunk & 1) * 27 * PT;
        // lanes sweep the 16-byte chunks of a row first: a warp instruction reads whole rows
        {
            const int j = tid % XCH, r0 = tid / XCH;
#pragma unroll
            for (int t = 0; t < TPM; ++t) {
                const int tap = mt * TPM + t;
#pragma unroll
                for (int i = 0; i < XCH; ++i) {
                    const int p = i * (PT / XCH) + r0;
                    const ll r = tap < 27 ? (ll) idx[tap * PT + p] : P.zero_row;
                    cp_async16(smem_u32(x_s + ((t * XCH + j) * PT + p) * 16), P.xrows + r * P.xpad + cib * KCI + j * 8);
                }
            }
        }
        if (mt == 0) {
            constexpr int GCH = NCO / 8;
            unsigned char* g_s = gs + (chunk & 1) * G_BYTES;
            const int j = tid % GCH, r0 = tid / GCH;
#pragma unroll
            for (int i = 0; i < GCH; ++i) {
                const int pl = i * (PT / GCH) + r0;
                const ll p = pb + (ll) chunk * PT + pl;
                cp_async16(smem_u32(g_s + (j * PT + pl) * 16), P.grows + (p < pe ? p : P.g_zero_row) * P.gpad + cob * NCO + j * 8);
            }
        }
    };

    bool failed = false;
    if (nchunks > 0) load_idx(0);
    __syncthreads();
    for (int s = 0; s < XAHEAD; ++s) {
        if (s < nstages) {
            issue_loads(s);
        }
        cp_async_commit();
    }
    for (int stage = 0; stage < nstages; ++stage) {
        const int chunk = stage / MT, mt = stage % MT;
        cp_async_wait<XAHEAD - 1>();
        fence_proxy_async();
        if (__syncthreads_or(failed ? 1 : 0)) { failed = true; break; }
        if (mt == 0 && chunk + 1 < nchunks) load_idx(chunk + 1);      // read by other threads from stage (chunk, MT - XAHEAD) on, after further barriers
        if (tid == 0) {
            tc_fence_after();
            const uint32_t a_addr = smem_u32(xs + (stage % XS) * X_BYTES);
            const uint32_t b_addr = smem_u32(gs + (chunk & 1) * G_BYTES);
#pragma unroll
            for (int k = 0; k < PT / 16; ++k) {
                const uint64_t da = make_desc(a_addr + k * 256, 128, PT * 16);
                const uint64_t db = make_desc(b_addr + k * 256, 128, PT * 16);
                umma_bf16(tmem_d + mt * NCO, da, db, IDESC, (chunk > 0 || k > 0) ? 1u : 0u);
            }
            umma_commit(smem_u32(bars + stage % XS));
            if (stage == nstages - 1) umma_commit(smem_u32(bars + XS));
        }
        const int nxt = stage + XAHEAD;
        if (nxt < nstages) {
            if (nxt >= XS) {
                const uint32_t use = nxt / XS;
                if (!mbar_wait(smem_u32(bars + nxt % XS), (use - 1) & 1)) failed = true;
            }
            if (!failed) issue_loads(nxt);
        }
        cp_async_commit();
    }

    if (nstages > 0 && !failed) {
        const bool ok = mbar_wait(smem_u32(bars + XS), 0);
        if (__syncthreads_or(ok ? 0 : 1)) failed = true;
    }
    if (!failed && nstages > 0) {
        tc_fence_after();
        float* dst = P.partial + (ll) blockIdx.x * P.cout * P.cin * 27;
        const int row = warp * 32 + lane;                 // accumulator row = (tap within tile) * KCI + ci
        const int t_in = row / KCI, ci = cib * KCI + row % KCI;
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const int tap = mt * TPM + t_in;
#pragma unroll
            for (int c0 = 0; c0 < NCO; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_d + ((uint32_t) (warp * 32) << 16) + mt * NCO + c0, r);
                tmem_ld_wait();
                if (tap < 27 && ci < P.cin) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int co = cob * NCO + c0 + j;
                        if (c0 + j < NCO && co < P.cout) dst[((ll) co * P.cin + ci) * 27 + tap] = __uint_as_float(r[j]);
                    }
                }
            }
        }
    } else if (!failed) {
        // empty range: this block still owns its slice of the partial buffer
        float* dst = P.partial + (ll) blockIdx.x * P.cout * P.cin * 27;
        for (int e = tid; e < KCI * NCO * 27; e += PT) {
            const int tap = e % 27, ci = cib * KCI + (e / 27) % KCI, co = cob * NCO + e / (27 * KCI);
            if (ci < P.cin && co < P.cout) dst[((ll) co * P.cin + ci) * 27 + tap] = 0.f;
        }
    }
    cp_async_wait<0>();
    if (failed && P.error_flag) *P.error_flag = 1;
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_d, TMEM_COLS);
}

template<typename T>
__global__ void reduce_partial_kernel(const T* __restrict__ partial, int nchunks, ll elems, T* __restrict__ dst) {
    const ll e = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= elems) return;
    T s = 0;
    for (int c = 0; c < nchunks; ++c) s += partial[(ll) c * elems + e];
    dst[e] += s;
}

template<int KCI, int NCO>
int launch_dw(const DwParams& P, int nranges, int blocks_y, cudaStream_t st, const char* pname) {
    constexpr int MT = (27 + 128 / KCI - 1) / (128 / KCI);
    (void) MT;
    const size_t smem = (size_t) XS * 128 * PT * 2 + 2 * (size_t) NCO * PT * 2 + 2 * 27 * PT * 4 + (XS + 1) * 8 + 16;
    auto kern = conv333_tc_dw_kernel<KCI, NCO>;
    APRNET_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    dim3 grid((unsigned) nranges, (unsigned) blocks_y);
    { AprnetProfScope _prof(pname, st);
    kern<<<grid, PT, smem, st>>>(P);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

} // namespace

extern "C" int64_t aprnet_conv333_tc_dw_partial_elems(int cin, int cout) {
    const ll per = (ll) 27 * cin * cout;
    const ll ranges = std::max<ll>(8, std::min<ll>(1024, (64ll << 20) / per));
    return (int64_t) (ranges * per);
}

// xrows / grows: channels-last bf16 copies of the input (+ tree means + zero row) and of grad_output
// (+ zero row) as produced by aprnet_pack_rows_bf16.  grad_weights (slots, Cout, Cin, 27) fp32 is
// accumulated into.
extern "C" int aprnet_conv333_backward_weights_tc(aprnet_apr* a, int dl, int cin, int cout, int slots, const void* xrows, int xpad,
                                                  const void* grows, int gpad, float* gw, float* partial, void* stream) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && cin > 0 && cout > 0 && slots > 0 && xrows && grows && gw && partial, "bad argument");
    APRNET_ARG_CHECK(xpad % 16 == 0 && gpad % 16 == 0 && xpad >= cin && gpad >= cout, "packed row widths must be multiples of 16");
    cudaStream_t st = (cudaStream_t) stream;
    const AprPlan* plan = aprnet_get_plan(a, dl, st);
    if (!plan) return APRNET_ERR_CUDA;
    const ll n = plan->n, t = plan->tree_size;
    const int kci = (xpad % 32 == 0) ? 32 : 16;
    const int nco = (gpad % 64 == 0) ? 64 : ((gpad % 32 == 0) ? 32 : 16);
    const int ci_blocks = xpad / kci, co_blocks = gpad / nco;
    const ll elems = (ll) 27 * cin * cout;
    const ll max_ranges = aprnet_conv333_tc_dw_partial_elems(cin, cout) / elems;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    char pname[64];
    snprintf(pname, sizeof(pname), "conv333_tc_dw:ci%d:co%d:dl%d", cin, cout, dl);
    for (const Segment& s : aprnet_segments(a, dl, slots, false)) {
        const ll len = s.end - s.begin;
        // enough ranges to fill the GPU a few times over, each at least 4 chunks long
        ll want = std::max<ll>(1, (ll) 3 * sms / std::max(1, ci_blocks * co_blocks));
        want = std::min<ll>(want, (len + 4 * PT - 1) / (4 * PT));
        const int nranges = (int) std::max<ll>(1, std::min<ll>(max_ranges, want));
        DwParams P;
        P.seg_begin = s.begin; P.seg_end = s.end;
        P.range_len = ((len + nranges - 1) / nranges + PT - 1) / PT * PT;
        P.nbr = plan->nbr; P.N = n;
        P.xrows = (const __nv_bfloat16*) xrows; P.xpad = xpad; P.tree_base = n; P.zero_row = n + t;
        P.grows = (const __nv_bfloat16*) grows; P.gpad = gpad; P.g_zero_row = n;
        P.partial = partial; P.cin = cin; P.cout = cout; P.ci_blocks = ci_blocks;
        P.error_flag = aprnet_tc_error_flag_device();
        int rc;
#define DW_CASE(KCI_, NCO_) if (kci == KCI_ && nco == NCO_) rc = launch_dw<KCI_, NCO_>(P, nranges, ci_blocks * co_blocks, st, pname); else
        DW_CASE(32, 64) DW_CASE(32, 32) DW_CASE(32, 16) DW_CASE(16, 64) DW_CASE(16, 32) DW_CASE(16, 16)
        { aprnet_set_error("conv333 tensor-core weight gradient: unsupported blocking"); return APRNET_ERR_UNSUPPORTED; }
#undef DW_CASE
        if (rc) return rc;
        { AprnetProfScope _prof("conv333_dw_reduce", st);
        reduce_partial_kernel<float><<<aprnet_ceil_div(elems, 256), 256, 0, st>>>(partial, nranges, elems, gw + (ll) s.slot * elems);
        }
        APRNET_LAUNCH_CHECK();
    }
    return APRNET_OK;
}
