// Weight gradient of the 3x3x3 particle convolution on the tensor cores (tcgen05 + TMEM), bf16
// operands with fp32 accumulation, deterministic.
//
//     dW[tap][ci][co] = sum over output locations p of  X[nbr(tap, p)][ci] * dO[p][co]
//
// is a GEMM whose contraction index is the particle.  One block owns a contiguous range of locations of
// one level, a group of taps, a block of CIB input channels and up to 256 output channels.  Its
// accumulators D[(tap, ci)][co] stay in TMEM for the whole range: 128-row tiles of 128 / CIB taps x CIB
// channels, NCOL fp32 columns each, side by side in the 512 columns; the tap group is as large as the
// columns allow, so the gathered rows are read once (CIB = all channels) and only the small dO rows are
// re-read per tap group.  Both operands are MN-major with the 128-byte hardware swizzle: a gathered
// neighbour row piece (CIB channels) and a dO row are contiguous in shared memory as they are in global
// memory, with K = particles.  Warp roles: 8 producer warps (two stages in issue at once, four warps of
// 32 particles each per stage; table entries are loaded by the lane that owns the particle, one stage
// ahead, and passed between lanes by shuffles; arrival on the stage barrier is asynchronous), one MMA
// thread, epilogue by warps 0-3 after the last MMA.  Each block writes its partial sums once; a second
// pass adds the ranges in ascending order (no atomics).
// Reference arithmetic: pyapr/aprnet/src/helpers.hpp:624-702 (accumulate_convolution_backward, dW part).
#include "apr_device.cuh"
#include "tc_ptx.cuh"
#include <cuda_bf16.h>
#include <algorithm>

extern int g_dw_waves_override;

namespace {

using namespace tcptx;
typedef long long ll;
constexpr int PT = 128;                       // particles per stage (K extent of one stage)
constexpr int DW_THREADS = 9 * 32;            // 8 producer warps + 1 MMA warp
constexpr int DW_MAX_STAGES = 6;
constexpr int A_STAGE = 2 * PT * 128;         // 128 accumulator rows = two 64-element swizzle atoms per particle

constexpr int DW_MAX_SEGS = APRNET_MAX_LEVELS;
struct DwParams {
    // the levels of the level delta, each cut into chunks of PT locations that its blocks take in turn: block r
    // with range_first[i] <= r < range_first[i + 1] belongs to level i and takes that level's chunks
    // r - range_first[i], + cnt, + 2 cnt, ... (cnt = blocks of the level).  Blocks that run at the same time
    // thus walk through the level side by side, and the rows one of them gathers for the neighbouring z planes
    // are still in L2 when the others (and the blocks of the other tap groups) ask for them.
    int n_segs;
    ll seg_begin[DW_MAX_SEGS], seg_end[DW_MAX_SEGS];
    int range_first[DW_MAX_SEGS + 1];
    const int32_t* nbr; ll N;
    const __nv_bfloat16* xrows; int xpad;  // packed inputs [N + T + 1][xpad]; tree rows start at tree_base, zeros at zero_row
    ll tree_base, zero_row;
    const __nv_bfloat16* grows; int gpad;  // packed dO [N + 1][gpad], zeros at row g_zero_row
    ll g_zero_row;
    float* partial;                        // [range][cout][cin][27]
    int cin, cout, ci_blocks, groups, taps_per_group;
    int* error_flag;
};

template<int CIB, int NCOL>
__global__ void __launch_bounds__(DW_THREADS, 1) conv333_tc_dw_kernel(const DwParams P, const int nstage) {
    constexpr int TPT = 128 / CIB;                      // taps per 128-row accumulator tile
    constexpr int PC = CIB / 8;                         // 16-byte chunks per gathered row piece
    constexpr int G_BYTES = (NCOL / 64) * PT * 128;     // one dO chunk: NCOL / 64 swizzle atoms per particle
    constexpr uint32_t IDESC = make_idesc(NCOL, true, true);
    constexpr uint32_t ATOM_STRIDE = PT * 128;          // between 64-element atoms along M (or N)

    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* a_ring = smem;                                               // nstage * A_STAGE
    unsigned char* g_ring = a_ring + (size_t) nstage * A_STAGE;                 // 2 * G_BYTES
    uint64_t* bars = reinterpret_cast<uint64_t*>(g_ring + 2 * G_BYTES);
    uint64_t* full = bars;                       // [nstage] gathered rows landed (4 warps x 32 lanes)
    uint64_t* empty = bars + DW_MAX_STAGES;      // [nstage] MMAs that read the stage completed
    uint64_t* dfull = empty + DW_MAX_STAGES;     // [2] dO chunk landed
    uint64_t* dempty = dfull + 2;                // [2] MMAs that read the dO chunk completed
    uint64_t* done = dempty + 2;                 // all MMAs of the range completed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int grp = blockIdx.y % P.groups, cib = (blockIdx.y / P.groups) % P.ci_blocks, cob = blockIdx.y / (P.groups * P.ci_blocks);
    const int tap0 = grp * P.taps_per_group;
    const int ntaps = min(P.taps_per_group, 27 - tap0);
    const int MT = (ntaps + TPT - 1) / TPT;             // accumulator tiles of this block
    int seg = 0;
    while (seg + 1 < P.n_segs && (int) blockIdx.x >= P.range_first[seg + 1]) ++seg;
    const int rl = (int) blockIdx.x - P.range_first[seg], cnt = P.range_first[seg + 1] - P.range_first[seg];
    const ll pb = P.seg_begin[seg] + (ll) rl * PT, pe = P.seg_end[seg];
    const ll pstride = (ll) cnt * PT;                   // between two chunks of this block
    const ll seg_chunks = (pe - P.seg_begin[seg] + PT - 1) / PT;
    const int nchunks = rl < seg_chunks ? (int) ((seg_chunks - rl + cnt - 1) / cnt) : 0;
    const int total_stages = nchunks * MT;
    const int gpiece = min(256, P.gpad - cob * 256);    // dO channels of this block

    // dO columns beyond gpiece are never copied: they must read as zeros
    for (int e = tid; e < 2 * G_BYTES / 16; e += DW_THREADS) reinterpret_cast<uint4*>(g_ring)[e] = make_uint4(0, 0, 0, 0);
    fence_proxy_async();
    if (tid == 0) {
        for (int i = 0; i < nstage; ++i) { mbar_init(smem_u32(full + i), 128); mbar_init(smem_u32(empty + i), 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(smem_u32(dfull + i), 128); mbar_init(smem_u32(dempty + i), 1); }
        mbar_init(smem_u32(done), 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 8) { tmem_alloc(smem_u32(tmem_slot), 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_slot;
    bool failed = false;

    if (warp < 8 && total_stages > 0) {
        // ---------------- producers ----------------
        const int gq = warp >> 2, wq = warp & 3;        // stage parity handled / 32-particle quarter of the stage
        const int c = lane % PC, r0 = lane / PC;
        constexpr int RPI = 32 / PC;                    // particles covered by one copy instruction
        int32_t rows_cur[TPT], raw_nxt[TPT];
        // table entries of this lane's particle for the taps of stage s: requested here, decoded only when the
        // stage is issued, so that the load latency overlaps the copies of the stage in between
        auto request_rows = [&](int s, int32_t (&raw)[TPT]) {
            const int chunk = s / MT, mt = s - chunk * MT;
            const ll p = pb + (ll) chunk * pstride + wq * 32 + lane;
#pragma unroll
            for (int tl = 0; tl < TPT; ++tl) {
                const int t = mt * TPT + tl;
                raw[tl] = (p < pe && t < ntaps) ? __ldg(P.nbr + (ll) (tap0 + t) * P.N + p) : APRNET_NONE;
            }
        };
        auto decode_rows = [&](const int32_t (&raw)[TPT], int32_t (&rows)[TPT]) {
#pragma unroll
            for (int tl = 0; tl < TPT; ++tl) {
                const int32_t v = raw[tl];
                rows[tl] = (int32_t) (v >= 0 ? (ll) v : (v == APRNET_NONE ? P.zero_row : P.tree_base + aprnet_dec_tree(v)));
            }
        };
        int s = gq;
        if (s < total_stages) { request_rows(s, raw_nxt); decode_rows(raw_nxt, rows_cur); }
        while (s < total_stages) {
            const int s_nxt = s + 2;
            if (s_nxt < total_stages) request_rows(s_nxt, raw_nxt);      // in flight while this stage is issued
            const int chunk = s / MT, mt = s - chunk * MT;
            const uint32_t slot = (uint32_t) s % (uint32_t) nstage, use = (uint32_t) s / (uint32_t) nstage;
            if (use > 0 && !mbar_wait_warp(smem_u32(empty + slot), (use - 1) & 1, abort_flag)) { failed = true; break; }
            if (mt == 0) {
                // this warp's 32 rows of the dO chunk
                const uint32_t db = chunk & 1, duse = chunk >> 1;
                if (duse > 0 && !mbar_wait_warp(smem_u32(dempty + db), (duse - 1) & 1, abort_flag)) { failed = true; break; }
                unsigned char* g_s = g_ring + db * G_BYTES;
                const int gc = gpiece / 8;
                for (int e = lane; e < 32 * gc; e += 32) {
                    const int pl = e / gc, cc = e - pl * gc, k = wq * 32 + pl;
                    const ll p = pb + (ll) chunk * pstride + k;
                    cp_async16(smem_u32(g_s + (cc >> 3) * ATOM_STRIDE + k * 128 + (((cc & 7) ^ (k & 7)) << 4)),
                               P.grows + (p < pe ? p : P.g_zero_row) * P.gpad + cob * 256 + cc * 8);
                }
                cp_async_arrive_noinc(smem_u32(dfull + db));
            }
            unsigned char* a_s = a_ring + (size_t) slot * A_STAGE;
            const __nv_bfloat16* src0 = P.xrows + cib * CIB + c * 8;
#pragma unroll
            for (int tl = 0; tl < TPT; ++tl) {
                const int m = tl * CIB + c * 8;                        // accumulator row of this chunk's first channel
                const uint32_t dst0 = smem_u32(a_s + (m >> 6) * ATOM_STRIDE);
                const int cc = (m & 63) >> 3;
#pragma unroll
                for (int pi = 0; pi < PC; ++pi) {
                    const int pl = pi * RPI + r0;
                    const int32_t r = __shfl_sync(0xffffffffu, rows_cur[tl], pl);
                    const int k = wq * 32 + pl;
                    cp_async16(dst0 + k * 128 + ((cc ^ (k & 7)) << 4), src0 + (ll) r * P.xpad);
                }
            }
            // the stage's barrier receives this thread's arrival when the copies above have landed
            cp_async_arrive_noinc(smem_u32(full + slot));
            if (s_nxt < total_stages) decode_rows(raw_nxt, rows_cur);
            s = s_nxt;
        }
        cp_async_commit();
        cp_async_wait<0>();
    } else if (warp == 8 && total_stages > 0) {
        // ---------------- MMA issue ----------------
        if (lane == 0) {
            uint32_t slot = 0, use = 0;
            for (int chunk = 0; chunk < nchunks && !failed; ++chunk) {
                const uint32_t db = chunk & 1, duse = chunk >> 1;
                const uint32_t b_addr = smem_u32(g_ring + db * G_BYTES);
                for (int mt = 0; mt < MT; ++mt) {
                    if (!mbar_wait(smem_u32(full + slot), use & 1, abort_flag)) { failed = true; break; }
                    if (mt == 0 && !mbar_wait(smem_u32(dfull + db), duse & 1, abort_flag)) { failed = true; break; }
                    fence_proxy_async();          // generic-proxy writes of the cp.async copies -> tensor-core (async proxy) reads
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(a_ring + (size_t) slot * A_STAGE);
#pragma unroll
                    for (int k = 0; k < PT / 16; ++k) {
                        // 16 particles = two 8-row groups of 1024 bytes; atoms along M / N are ATOM_STRIDE apart
                        const uint64_t da = make_desc(a_addr + k * 2048, ATOM_STRIDE, 1024, 2);
                        const uint64_t dbd = make_desc(b_addr + k * 2048, ATOM_STRIDE, 1024, 2);
                        umma_bf16(tmem_d + mt * NCOL, da, dbd, IDESC, (chunk > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(smem_u32(empty + slot));
                    if (mt == MT - 1) umma_commit(smem_u32(dempty + db));
                    if (++slot == (uint32_t) nstage) { slot = 0; ++use; }
                }
            }
            if (!failed) umma_commit(smem_u32(done));
        }
    }

    // ---------------- epilogue: warps 0-3 ----------------
    float* dst = P.partial + (ll) blockIdx.x * P.cout * P.cin * 27;
    if (warp < 4 && total_stages > 0 && !failed) {
        if (!mbar_wait_warp(smem_u32(done), 0, abort_flag)) failed = true;
        if (!failed) {
            tc_fence_after();
            const int row = warp * 32 + lane;                 // accumulator row = (tap within tile) * CIB + ci
            const int tl = row / CIB, ci = cib * CIB + row % CIB;
            for (int mt = 0; mt < MT; ++mt) {
                const int t = mt * TPT + tl;
#pragma unroll
                for (int c0 = 0; c0 < NCOL; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32(tmem_d + ((uint32_t) (warp * 32) << 16) + mt * NCOL + c0, r);
                    tmem_ld_wait();
                    if (t < ntaps && ci < P.cin) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const int co = cob * 256 + c0 + j;
                            if (co < P.cout) dst[((ll) co * P.cin + ci) * 27 + tap0 + t] = __uint_as_float(r[j]);
                        }
                    }
                }
            }
        }
    } else if (total_stages == 0) {
        // empty range: this block still owns its slice of the partial buffer
        for (int e = tid; e < CIB * 256 * ntaps; e += DW_THREADS) {
            const int t = e % ntaps, ci = cib * CIB + (e / ntaps) % CIB, co = cob * 256 + e / (ntaps * CIB);
            if (ci < P.cin && co < P.cout) dst[((ll) co * P.cin + ci) * 27 + tap0 + t] = 0.f;
        }
    }

    if (failed) {
        *abort_flag = 1;
        if (P.error_flag) *P.error_flag = 1;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) tmem_dealloc(tmem_d, 512);
}

template<typename T>
__global__ void reduce_partial_kernel(const T* __restrict__ partial, int nchunks, ll elems, T* __restrict__ dst) {
    const ll e = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= elems) return;
    T s = 0;
    for (int c = 0; c < nchunks; ++c) s += partial[(ll) c * elems + e];
    dst[e] += s;
}

template<int CIB, int NCOL>
int launch_dw(const DwParams& P, int nranges, int blocks_y, cudaStream_t st, const char* pname) {
    constexpr size_t G_BYTES = (size_t) (NCOL / 64) * PT * 128;
    const size_t fixed = 2 * G_BYTES + (2 * DW_MAX_STAGES + 5) * 8 + 16 + 1024;
    const int nstage = (int) std::min<size_t>(DW_MAX_STAGES, (227 * 1024 - 1024 - fixed) / A_STAGE);
    if (nstage < 2) { aprnet_set_error("conv333 tensor-core weight gradient: tile does not fit shared memory"); return APRNET_ERR_UNSUPPORTED; }
    const size_t smem = (size_t) nstage * A_STAGE + fixed;
    auto kern = conv333_tc_dw_kernel<CIB, NCOL>;
    APRNET_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    dim3 grid((unsigned) nranges, (unsigned) blocks_y);
    { AprnetProfScope _prof(pname, st);
    kern<<<grid, DW_THREADS, smem, st>>>(P, nstage);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

} // namespace

int g_dw_waves_override = 0;     // aprnet_tc_set_option("dw_waves", n): waves of blocks of the weight gradient, measurement switch

extern "C" int64_t aprnet_conv333_tc_dw_partial_elems(int cin, int cout) {
    const ll per = (ll) 27 * cin * cout;
    const ll ranges = std::max<ll>(32, std::min<ll>(1024, (64ll << 20) / per));     // at least one per level plus room for a wave
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
    // input-channel block: the widest of 128 / 64 / 32 / 16 that divides the padded width (gathered once when it covers all channels)
    const int cibk = (xpad % 128 == 0) ? 128 : ((xpad % 64 == 0) ? 64 : ((xpad % 32 == 0) ? 32 : 16));
    const int ci_blocks = xpad / cibk;
    const int co_blocks = (gpad + 255) / 256;
    const int ncol = (std::min(gpad, 256) + 63) / 64 * 64;                 // accumulator columns per tile
    const int tpt = 128 / cibk;
    const int max_taps = (512 / ncol) * tpt;                               // taps whose accumulators fit the 512 TMEM columns
    const int groups = (27 + max_taps - 1) / max_taps;
    const int taps_per_group = ((27 + groups - 1) / groups + tpt - 1) / tpt * tpt;
    const int blocks_y = groups * ci_blocks * co_blocks;
    const ll elems = (ll) 27 * cin * cout;
    const ll max_ranges = aprnet_conv333_tc_dw_partial_elems(cin, cout) / elems;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    char pname[64];
    snprintf(pname, sizeof(pname), "conv333_tc_dw:ci%d:co%d:dl%d", cin, cout, dl);
    // one launch over all levels, blocks for `waves` waves of one block per SM where the partial buffer and the number
    // of levels allow it: every level gets blocks in proportion to its chunks (at most `per_block` chunks each, at least 4
    // where the level has that many); a level's partial sums are added into the slot of that level afterwards
    const std::vector<Segment> segs = aprnet_segments(a, dl, slots, false);
    ll total_chunks = 0;
    for (const Segment& sg : segs) total_chunks += (sg.end - sg.begin + PT - 1) / PT;
    if (total_chunks == 0) return APRNET_OK;
    // two waves: a short level then costs a short block rather than an idle SM (1 to 4 waves measured within 5 % of each other)
    const int waves = g_dw_waves_override > 0 ? g_dw_waves_override : 2;
    ll budget = std::max<ll>((ll) segs.size(), ((ll) waves * sms + blocks_y - 1) / blocks_y);
    budget = std::max<ll>(1, std::min<ll>(budget, max_ranges));
    auto blocks_for = [&](ll per_block) { ll b = 0; for (const Segment& sg : segs) b += ((sg.end - sg.begin + PT - 1) / PT + per_block - 1) / per_block; return b; };
    ll per_block = std::max<ll>(4, (total_chunks + budget - 1) / budget);
    while (blocks_for(per_block) > budget) ++per_block;
    DwParams P;
    P.n_segs = (int) segs.size();
    P.range_first[0] = 0;
    for (int i = 0; i < P.n_segs; ++i) {
        P.seg_begin[i] = segs[i].begin; P.seg_end[i] = segs[i].end;
        P.range_first[i + 1] = P.range_first[i] + (int) (((segs[i].end - segs[i].begin + PT - 1) / PT + per_block - 1) / per_block);
    }
    const int nranges = P.range_first[P.n_segs];
    if (nranges > max_ranges) { aprnet_set_error("conv333 tensor-core weight gradient: %d ranges exceed the partial buffer", nranges); return APRNET_ERR_ARG; }
    P.nbr = plan->nbr; P.N = n;
    P.xrows = (const __nv_bfloat16*) xrows; P.xpad = xpad; P.tree_base = n; P.zero_row = n + t;
    P.grows = (const __nv_bfloat16*) grows; P.gpad = gpad; P.g_zero_row = n;
    P.partial = partial; P.cin = cin; P.cout = cout; P.ci_blocks = ci_blocks; P.groups = groups; P.taps_per_group = taps_per_group;
    P.error_flag = aprnet_tc_error_flag_device();
    int rc;
#define DW_CASE(CIB_, NCOL_) if (cibk == CIB_ && ncol == NCOL_) rc = launch_dw<CIB_, NCOL_>(P, nranges, blocks_y, st, pname); else
    DW_CASE(16, 64) DW_CASE(16, 128) DW_CASE(16, 192) DW_CASE(16, 256)
    DW_CASE(32, 64) DW_CASE(32, 128) DW_CASE(32, 192) DW_CASE(32, 256)
    DW_CASE(64, 64) DW_CASE(64, 128) DW_CASE(64, 192) DW_CASE(64, 256)
    DW_CASE(128, 64) DW_CASE(128, 128) DW_CASE(128, 192) DW_CASE(128, 256)
    { aprnet_set_error("conv333 tensor-core weight gradient: unsupported blocking"); return APRNET_ERR_UNSUPPORTED; }
#undef DW_CASE
    if (rc) return rc;
    for (int i = 0; i < P.n_segs; ++i) {
        const int cnt = P.range_first[i + 1] - P.range_first[i];
        if (cnt == 0) continue;
        AprnetProfScope _prof("conv333_dw_reduce", st);
        reduce_partial_kernel<float><<<aprnet_ceil_div(elems, 256), 256, 0, st>>>(partial + (ll) P.range_first[i] * elems, cnt, elems, gw + (ll) segs[i].slot * elems);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}
