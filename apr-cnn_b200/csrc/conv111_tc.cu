// 1x1x1 particle convolution on the tensor cores (bf16 operands, fp32 accumulate).
//
// Replaces pyapr/aprnet/cuda/src/conv111_gpu.cu:9-232 for float32 tensors when the layer's precision is "bf16".
// out[o][p] = sum_i w[slot(level of p)][o][i] * in[i][p] is a plain [locations x Cin] . [Cin x Cout] product per
// level; with 2 * Cin * Cout flops against 4 * (Cin + Cout) bytes per location the CUDA-core kernel sits at the
// fp32 multiply-add bound, the tensor-core kernel at the HBM bound.
//
// One persistent block per SM, 17 warps:
//   warps 0-7   producers, two groups of 128 threads on alternate tiles of 128 locations.  A thread owns one location:
//               it requests up to 32 input channels at a time (4-byte loads, coalesced across the warp along the location
//               axis of the channel-major tensor), rounds them to bf16 and writes them as 16-byte pieces of the K-major,
//               hardware-swizzled A operand (the transposition happens in registers), then one arrival per thread on the
//               stage's barrier;
//   warp 8      one thread waits for the stage, fences the generic-proxy writes against the tensor core's reads and
//               issues the Cin / 16 tcgen05.mma (M = 128, N = padded Cout) of each tile and commits the
//               stage's "slot free" barrier and the accumulator's "complete" barrier;
//   warps 9-16  epilogue, two sets of four warps on alternate tiles: TMEM -> registers -> coalesced fp32 stores of out[o][p].
// The weights of one level (B operand, bf16, all of Cin x Cout) stay in shared memory; the block walks the levels one
// after the other and converts the next level's weights from the fp32 tensor between two block-wide barriers.
// Every wait is bounded and polls a block-wide abort flag; after an expiry the block raises the library's error flag,
// skips the remaining work (all block-wide barriers are still reached) and returns.
#include "apr_device.cuh"
#include "tc_ptx.cuh"
#include <cuda_bf16.h>
#include <algorithm>

int* aprnet_tc_error_flag_device();

namespace {

using namespace tcptx;
typedef long long ll;
constexpr int TILE_M = 128;
constexpr int C1_THREADS = 17 * 32;
constexpr int C1_THREADS_DW = 13 * 32;
constexpr int C1_MAX_STAGES = 8;
constexpr int C1_MAX_ACC = 4;
constexpr int C1_MAX_SEGS = APRNET_MAX_LEVELS;

struct C1Params {
    int n_segs;
    ll seg_begin[C1_MAX_SEGS], seg_end[C1_MAX_SEGS];
    int seg_slot[C1_MAX_SEGS];
    const float* in; ll ld_in; int n_in;           // K = n_in channels
    const float* w; ll ws, wo, wi;                 // element (slot, o, i) at w[slot * ws + o * wo + i * wi]
    float* out; ll ld_out; int n_out;
    int kpad;                                      // n_in padded to 16, 32 or a multiple of 64
    int* error_flag;
};

template<int KS> __device__ __forceinline__ int swz_chunk(int row, int c) {      // position of 16-byte chunk c of row `row`
    return KS == 64 ? (c ^ (row & 7)) : (KS == 32 ? (c ^ ((row >> 1) & 3)) : (c ^ ((row >> 2) & 1)));
}

__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}

template<int NT, int KS>
__global__ void __launch_bounds__(C1_THREADS, 1) conv111_tc_kernel(const C1Params P, const int stages) {
    constexpr int ACC_COLS = NT < 32 ? 32 : NT;                 // TMEM columns per accumulator
    constexpr int NACC = NT <= 128 ? 4 : 2;
    constexpr int ROW_BYTES = KS * 2;
    constexpr int A_SUB = TILE_M * ROW_BYTES;                   // one K chunk of KS channels
    constexpr uint32_t A_LAYOUT = KS == 64 ? 2u : (KS == 32 ? 4u : 6u);
    constexpr uint32_t IDESC = make_idesc(NT, false, false);
    constexpr int KB = KS < 32 ? KS : 32;                       // channels a producer thread requests together

    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int kchunks = P.kpad / KS;
    const int a_stage = kchunks * A_SUB;
    unsigned char* a_ring = smem;                                                   // stages x [kchunks][128][KS] bf16, swizzled
    unsigned char* b_s = a_ring + (size_t) stages * a_stage;                        // [kpad / 8][NT][8] bf16
    uint64_t* bars = reinterpret_cast<uint64_t*>(b_s + (size_t) NT * P.kpad * 2);
    uint64_t* full = bars;                              // [stages] operand written (128 producer threads)
    uint64_t* empty = bars + C1_MAX_STAGES;             // [stages] MMAs that read the stage completed
    uint64_t* tmem_full = empty + C1_MAX_STAGES;        // [NACC]   accumulator complete
    uint64_t* tmem_empty = tmem_full + C1_MAX_ACC;      // [NACC]   accumulator read back (4 epilogue warps)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + C1_MAX_ACC);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < stages; ++i) { mbar_init(smem_u32(full + i), 128); mbar_init(smem_u32(empty + i), 1); }
        for (int i = 0; i < NACC; ++i) { mbar_init(smem_u32(tmem_full + i), 1); mbar_init(smem_u32(tmem_empty + i), 4); }
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 8) { tmem_alloc(smem_u32(tmem_slot), NACC * ACC_COLS); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_slot;
    bool failed = false;
    uint32_t j_base = 0;                    // tiles this block has been given in the levels before the current one

    for (int seg = 0; seg < P.n_segs; ++seg) {
        const ll sb = P.seg_begin[seg], se = P.seg_end[seg];
        const int seg_tiles = (int) ((se - sb + TILE_M - 1) / TILE_M);
        const int mine = (int) blockIdx.x < seg_tiles ? (seg_tiles - (int) blockIdx.x + (int) gridDim.x - 1) / (int) gridDim.x : 0;
        // ---- the level's weights -> B operand (every accumulator of the previous level has been read back) ----
        __syncthreads();
        {
            const float* wslot = P.w + (ll) P.seg_slot[seg] * P.ws;
            const int nk8 = P.kpad / 8;
            for (int e = tid; e < NT * nk8; e += C1_THREADS) {
                const int n = e % NT, k8 = e / NT;
                float v[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int k = k8 * 8 + q;
                    v[q] = (n < P.n_out && k < P.n_in) ? __ldg(wslot + (ll) n * P.wo + (ll) k * P.wi) : 0.f;
                }
                uint4 pk;
                pk.x = pack_bf16x2(v[0], v[1]); pk.y = pack_bf16x2(v[2], v[3]); pk.z = pack_bf16x2(v[4], v[5]); pk.w = pack_bf16x2(v[6], v[7]);
                *reinterpret_cast<uint4*>(b_s + ((size_t) k8 * NT + n) * 16) = pk;
            }
            fence_proxy_async();
        }
        __syncthreads();
        tc_fence_after();

        if (warp < 8) {
            // ---------------- producers ----------------
            const int grp = tid >> 7, row = tid & 127;
            for (int it = grp; it < mine && !failed; it += 2) {
                const uint32_t j = j_base + (uint32_t) it, slot = j % (uint32_t) stages, use = j / (uint32_t) stages;
                const ll p = sb + ((ll) blockIdx.x + (ll) it * gridDim.x) * TILE_M + row;
                const bool valid = p < se;
                const float* src = P.in + (valid ? p : sb);
                float v[KB];
                auto request = [&](int kb) {
#pragma unroll
                    for (int q = 0; q < KB; ++q) v[q] = (valid && kb + q < P.n_in) ? src[(ll) (kb + q) * P.ld_in] : 0.f;
                };
                request(0);             // in flight while this warp waits for the ring slot
                if (use > 0 && !mbar_wait_warp(smem_u32(empty + slot), (use - 1) & 1, abort_flag)) { failed = true; break; }
                unsigned char* a_s = a_ring + (size_t) slot * a_stage;
                for (int kb = 0; kb < P.kpad; kb += KB) {
                    if (kb > 0) request(kb);
                    unsigned char* sub = a_s + (size_t) (kb / KS) * A_SUB + row * ROW_BYTES;
                    const int c0 = (kb % KS) / 8;
#pragma unroll
                    for (int q8 = 0; q8 < KB / 8; ++q8) {
                        uint4 pk;
                        pk.x = pack_bf16x2(v[q8 * 8 + 0], v[q8 * 8 + 1]); pk.y = pack_bf16x2(v[q8 * 8 + 2], v[q8 * 8 + 3]);
                        pk.z = pack_bf16x2(v[q8 * 8 + 4], v[q8 * 8 + 5]); pk.w = pack_bf16x2(v[q8 * 8 + 6], v[q8 * 8 + 7]);
                        *reinterpret_cast<uint4*>(sub + (swz_chunk<KS>(row, c0 + q8) << 4)) = pk;
                    }
                }
                // (no proxy fence here: the MMA thread fences after its wait)
                mbar_arrive(smem_u32(full + slot));
            }
        } else if (warp == 8) {
            // ---------------- MMA issue ----------------
            if (lane == 0) {
                for (int it = 0; it < mine && !failed; ++it) {
                    const uint32_t j = j_base + (uint32_t) it, slot = j % (uint32_t) stages, use = j / (uint32_t) stages;
                    const uint32_t acc = j % NACC, acc_use = j / NACC;
                    if (acc_use > 0 && !mbar_wait(smem_u32(tmem_empty + acc), (acc_use - 1) & 1, abort_flag)) { failed = true; break; }
                    if (!mbar_wait(smem_u32(full + slot), use & 1, abort_flag)) { failed = true; break; }
                    fence_proxy_async();          // generic-proxy writes of the producers -> tensor-core (async proxy) reads
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(a_ring + (size_t) slot * a_stage);
                    const uint64_t db0 = make_desc(smem_u32(b_s), NT * 16, 128, 0);
                    for (int kc = 0; kc < kchunks; ++kc) {
                        const uint64_t da0 = make_desc(a_addr + kc * A_SUB, 16, 8 * ROW_BYTES, A_LAYOUT);
#pragma unroll
                        for (int k = 0; k < KS / 16; ++k)
                            umma_bf16(tmem_d + acc * ACC_COLS, da0 + (uint64_t) ((k * 32) >> 4),
                                      db0 + (uint64_t) (((kc * (KS / 16) + k) * 2 * (NT * 16)) >> 4), IDESC, (kc > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(smem_u32(empty + slot));
                    umma_commit(smem_u32(tmem_full + acc));
                }
            }
        } else {
            // ---------------- epilogue ----------------
            // two sets of four warps on alternate tiles (twice the stores in flight)
            const int q = warp & 3;                           // TMEM lane group this warp may read
            const int row = q * 32 + lane;
            for (int it = (warp - 9) >> 2; it < mine && !failed; it += 2) {
                const uint32_t j = j_base + (uint32_t) it, acc = j % NACC, acc_use = j / NACC;
                const ll p = sb + ((ll) blockIdx.x + (ll) it * gridDim.x) * TILE_M + row;
                if (!mbar_wait_warp(smem_u32(tmem_full + acc), acc_use & 1, abort_flag)) { failed = true; break; }
                tc_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < NT; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32(tmem_d + ((uint32_t) (q * 32) << 16) + acc * ACC_COLS + c0, r);
                    tmem_ld_wait();
                    if (p < se) {
#pragma unroll
                        for (int jj = 0; jj < 32; ++jj)
                            if (c0 + jj < P.n_out) P.out[(ll) (c0 + jj) * P.ld_out + p] = __uint_as_float(r[jj]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(tmem_empty + acc));
            }
        }
        if (failed) *abort_flag = 1;
        j_base += (uint32_t) mine;
    }

    if (failed) {
        *abort_flag = 1;
        if (P.error_flag) *P.error_flag = 1;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) tmem_dealloc(tmem_d, NACC * ACC_COLS);
}

inline int pad_k(int c) { return c <= 16 ? 16 : (c <= 32 ? 32 : (c + 63) / 64 * 64); }
inline int pick_nt(int n) { return n <= 16 ? 16 : (n <= 32 ? 32 : (n <= 64 ? 64 : (n <= 128 ? 128 : 256))); }

template<int NT, int KS>
int launch_c1(const C1Params& P, ll total_tiles, cudaStream_t st, const char* pname) {
    const size_t a_stage = (size_t) TILE_M * P.kpad * 2, b_bytes = (size_t) NT * P.kpad * 2;
    const size_t fixed = b_bytes + (2 * C1_MAX_STAGES + 2 * C1_MAX_ACC) * 8 + 16 + 1024;
    if (fixed + 2 * a_stage > 227 * 1024 - 1024) return APRNET_ERR_UNSUPPORTED;
    const int stages = (int) std::min<size_t>(C1_MAX_STAGES, (227 * 1024 - 1024 - fixed) / a_stage);
    const size_t smem = (size_t) stages * a_stage + fixed;
    auto kern = conv111_tc_kernel<NT, KS>;
    APRNET_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int grid = (int) std::min<ll>(total_tiles, sms);
    { AprnetProfScope _prof(pname, st);
    kern<<<grid, C1_THREADS, smem, st>>>(P, stages);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

// out[o][p] = sum_i w[slot][o][i] in[i][p] over the locations of level delta dl
int run_conv111_tc(const aprnet_apr* a, int dl, int n_in, int n_out, int slots, const float* in, ll ld_in, const float* w, ll ws, ll wo, ll wi,
                   float* out, ll ld_out, cudaStream_t st, const char* pname) {
    // narrow layers (a classifier head) are bound by their one wide tensor either way and run faster on the CUDA cores
    if (n_out > 256 || n_in > 256 || n_in < 8 || n_out < 8) return APRNET_ERR_UNSUPPORTED;
    const std::vector<Segment> segs = aprnet_segments(a, dl, slots, true);
    C1Params P;
    P.n_segs = 0;
    ll total_tiles = 0;
    for (const Segment& s : segs) {
        if (s.end <= s.begin) continue;
        if (P.n_segs >= C1_MAX_SEGS) return APRNET_ERR_UNSUPPORTED;
        P.seg_begin[P.n_segs] = s.begin; P.seg_end[P.n_segs] = s.end; P.seg_slot[P.n_segs] = s.slot;
        total_tiles = std::max<ll>(total_tiles, (s.end - s.begin + TILE_M - 1) / TILE_M);
        ++P.n_segs;
    }
    if (P.n_segs == 0) return APRNET_OK;
    P.in = in; P.ld_in = ld_in; P.n_in = n_in; P.w = w; P.ws = ws; P.wo = wo; P.wi = wi; P.out = out; P.ld_out = ld_out; P.n_out = n_out;
    P.kpad = pad_k(n_in);
    P.error_flag = aprnet_tc_error_flag_device();
    const int nt = pick_nt(n_out), ks = std::min(64, P.kpad);
#define C1_CASE(NT_, KS_) if (nt == NT_ && ks == KS_) return launch_c1<NT_, KS_>(P, total_tiles, st, pname);
    C1_CASE(16, 16) C1_CASE(16, 32) C1_CASE(16, 64) C1_CASE(32, 16) C1_CASE(32, 32) C1_CASE(32, 64)
    C1_CASE(64, 16) C1_CASE(64, 32) C1_CASE(64, 64) C1_CASE(128, 16) C1_CASE(128, 32) C1_CASE(128, 64)
    C1_CASE(256, 16) C1_CASE(256, 32) C1_CASE(256, 64)
#undef C1_CASE
    return APRNET_ERR_UNSUPPORTED;
}


// ---- weight gradient -----------------------------------------------------------------------------------
// gw[slot][o][i] += sum over the locations p of the slot's levels of gout[o][p] * in[i][p]: M = output channels (padded
// to 128 per accumulator), N = input channels, K = locations.  Both tensors are channel-major, i.e. K-major operands
// as they lie in memory; they only have to be rounded to bf16.  One persistent block per SM walks its share of the
// 128-location tiles of ONE level range and keeps the accumulators in TMEM until the end:
//   warps 0-7   producers: a warp takes channel rows of both tensors in turn, 32 consecutive locations per load
//               instruction (coalesced), and writes each value as a 2-byte piece of the swizzled K-major operand row
//               (conflict-free: the 32 lanes fill 64 bytes of one 128-byte row); locations past the end are zeros;
//   warp 8      one thread issues 8 tcgen05.mma per accumulator and stage;
//   warps 9-12  after the last tile: TMEM -> partial sums of this block; a second kernel adds the blocks in fixed order.
struct C1DwParams {
    ll seg_begin, seg_end;
    const float* in; ll ld_in; int cin;
    const float* gout; ll ld_out; int cout;
    float* partial;                         // [block][cout][cin]
    int* error_flag;
};

template<int NT>
__global__ void __launch_bounds__(C1_THREADS_DW, 1) conv111_tc_dw_kernel(const C1DwParams P, const int stages, const int mtiles) {
    constexpr int SUB = 64;                                  // locations per swizzle atom row (128 bytes)
    constexpr uint32_t IDESC = make_idesc(NT, false, false);
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    const int a_rows = mtiles * 128;
    const int stage_bytes = (a_rows + NT) * 256;             // two 64-location halves of 128 bytes per channel row
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (size_t) stages * stage_bytes);
    uint64_t* full = bars;                                   // [stages] operands written (256 producer threads)
    uint64_t* empty = bars + C1_MAX_STAGES;                  // [stages] MMAs that read the stage completed
    uint64_t* done = empty + C1_MAX_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(done + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t tmem_cols = mtiles * NT <= 32 ? 32u : (mtiles * NT <= 64 ? 64u : (mtiles * NT <= 128 ? 128u : (mtiles * NT <= 256 ? 256u : 512u)));
    if (tid == 0) {
        for (int i = 0; i < stages; ++i) { mbar_init(smem_u32(full + i), 256); mbar_init(smem_u32(empty + i), 1); }
        mbar_init(smem_u32(done), 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 8) { tmem_alloc(smem_u32(tmem_slot), tmem_cols); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_slot;
    bool failed = false;
    const ll sb = P.seg_begin, se = P.seg_end;
    const int seg_tiles = (int) ((se - sb + TILE_M - 1) / TILE_M);
    const int mine = (int) blockIdx.x < seg_tiles ? (seg_tiles - (int) blockIdx.x + (int) gridDim.x - 1) / (int) gridDim.x : 0;

    if (warp < 8) {
        // ---------------- producers ----------------
        const int nrows = P.cout + P.cin;                    // channel rows of a stage: gout rows, then in rows
        for (int it = 0; it < mine && !failed; ++it) {
            const uint32_t slot = (uint32_t) it % (uint32_t) stages, use = (uint32_t) it / (uint32_t) stages;
            const ll p0 = sb + ((ll) blockIdx.x + (ll) it * gridDim.x) * TILE_M;
            if (use > 0 && !mbar_wait_warp(smem_u32(empty + slot), (use - 1) & 1, abort_flag)) { failed = true; break; }
            unsigned char* st = smem + (size_t) slot * stage_bytes;
            for (int r0 = warp; r0 < nrows; r0 += 8 * 8) {   // 8 rows of this warp x 4 quarters of 32 locations in flight
                float v[8][4];
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int r = r0 + u * 8;
                    const float* src = r < P.cout ? P.gout + (ll) r * P.ld_out : P.in + (ll) (r - P.cout) * P.ld_in;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const ll p = p0 + q * 32 + lane;
                        v[u][q] = (r < nrows && p < se) ? src[p] : 0.f;
                    }
                }
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                    const int r = r0 + u * 8;
                    if (r >= nrows) break;
                    // operand row: gout rows first (accumulator rows), in rows after a_rows
                    const int orow = r < P.cout ? r : a_rows + (r - P.cout);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const int pl = q * 32 + lane;                     // location within the tile
                        const int half = pl / SUB, k = pl % SUB;
                        unsigned char* dst = st + (size_t) half * ((size_t) (a_rows + NT) * 128) + (size_t) orow * 128
                                           + ((((k >> 3) ^ (orow & 7)) << 4) | ((k & 7) << 1));
                        *reinterpret_cast<__nv_bfloat16*>(dst) = __float2bfloat16(v[u][q]);
                    }
                }
            }
            mbar_arrive(smem_u32(full + slot));               // the MMA thread fences the generic-proxy writes after its wait
        }
    } else if (warp == 8) {
        // ---------------- MMA issue ----------------
        if (lane == 0) {
            for (int it = 0; it < mine && !failed; ++it) {
                const uint32_t slot = (uint32_t) it % (uint32_t) stages, use = (uint32_t) it / (uint32_t) stages;
                if (!mbar_wait(smem_u32(full + slot), use & 1, abort_flag)) { failed = true; break; }
                fence_proxy_async();
                tc_fence_after();
                const uint32_t base = smem_u32(smem + (size_t) slot * stage_bytes);
                for (int half = 0; half < 2; ++half) {
                    const uint32_t hb = base + half * ((a_rows + NT) * 128);
                    const uint64_t db0 = make_desc(hb + a_rows * 128, 16, 1024, 2);
                    for (int mt = 0; mt < mtiles; ++mt) {
                        const uint64_t da0 = make_desc(hb + mt * 128 * 128, 16, 1024, 2);
#pragma unroll
                        for (int k = 0; k < SUB / 16; ++k)
                            umma_bf16(tmem_d + mt * NT, da0 + (uint64_t) ((k * 32) >> 4), db0 + (uint64_t) ((k * 32) >> 4), IDESC,
                                      (it > 0 || half > 0 || k > 0) ? 1u : 0u);
                    }
                }
                umma_commit(smem_u32(empty + slot));
            }
            if (!failed) umma_commit(smem_u32(done));
        }
    }
    // ---------------- epilogue: warps 9-12 ----------------
    float* dst = P.partial + (ll) blockIdx.x * P.cout * P.cin;
    if (warp >= 9 && mine > 0 && !failed) {
        if (!mbar_wait_warp(smem_u32(done), 0, abort_flag)) failed = true;
        if (!failed) {
            tc_fence_after();
            const int q = warp & 3, row = q * 32 + lane;
            for (int mt = 0; mt < mtiles; ++mt) {
                const int o = mt * 128 + row;
#pragma unroll
                for (int c0 = 0; c0 < NT; c0 += 32) {
                    uint32_t r[32];
                    tmem_ld32(tmem_d + ((uint32_t) (q * 32) << 16) + mt * NT + c0, r);
                    tmem_ld_wait();
                    if (o < P.cout) {
#pragma unroll
                        for (int jj = 0; jj < 32; ++jj)
                            if (c0 + jj < P.cin) dst[(ll) o * P.cin + c0 + jj] = __uint_as_float(r[jj]);
                    }
                }
            }
        }
    } else if (mine == 0) {
        for (int e = tid; e < P.cout * P.cin; e += C1_THREADS_DW) dst[e] = 0.f;       // this block still owns its slice
    }
    if (failed) {
        *abort_flag = 1;
        if (P.error_flag) *P.error_flag = 1;
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 8) tmem_dealloc(tmem_d, tmem_cols);
}

__global__ void c1_reduce_partial_kernel(const float* __restrict__ partial, int nblocks, ll elems, float* __restrict__ dst) {
    const ll e = (ll) blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= elems) return;
    float s = 0.f;
    for (int c = 0; c < nblocks; ++c) s += partial[(ll) c * elems + e];
    dst[e] += s;
}

template<int NT>
int launch_c1_dw(const C1DwParams& P, int grid, int mtiles, cudaStream_t st) {
    const size_t stage = (size_t) (mtiles * 128 + NT) * 256;
    const size_t fixed = (2 * C1_MAX_STAGES + 1) * 8 + 16 + 1024;
    if (fixed + 2 * stage > 227 * 1024 - 1024) return APRNET_ERR_UNSUPPORTED;
    const int stages = (int) std::min<size_t>(C1_MAX_STAGES, (227 * 1024 - 1024 - fixed) / stage);
    const size_t smem = (size_t) stages * stage + fixed;
    auto kern = conv111_tc_dw_kernel<NT>;
    APRNET_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    kern<<<grid, C1_THREADS_DW, smem, st>>>(P, stages, mtiles);
    return APRNET_OK;
}

} // namespace

extern "C" int aprnet_conv111_forward_tc(const aprnet_apr* a, int dl, int cin, int cout, int S, const float* in, int64_t ld_in,
                                         const float* w, float* out, int64_t ld_out, void* stream) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && in && w && out && cin > 0 && cout > 0 && S > 0, "bad argument");
    APRNET_DEVICE_CHECK(a);
    APRNET_ARG_CHECK(ld_in >= a->number_parts(dl) && ld_out >= a->number_parts(dl), "leading dimension too small");
    char pname[64];
    snprintf(pname, sizeof(pname), "conv111_tc:ci%d:co%d:dl%d", cin, cout, dl);
    return run_conv111_tc(a, dl, cin, cout, S, in, ld_in, w, (ll) cin * cout, cin, 1, out, ld_out, (cudaStream_t) stream, pname);
}

extern "C" int aprnet_conv111_backward_input_tc(const aprnet_apr* a, int dl, int cin, int cout, int S, const float* gout, int64_t ld_out,
                                                const float* w, float* gin, int64_t ld_in, void* stream) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && gout && w && gin && cin > 0 && cout > 0 && S > 0, "bad argument");
    APRNET_DEVICE_CHECK(a);
    APRNET_ARG_CHECK(ld_in >= a->number_parts(dl) && ld_out >= a->number_parts(dl), "leading dimension too small");
    char pname[64];
    snprintf(pname, sizeof(pname), "conv111_tc:ci%d:co%d:dl%d", cout, cin, dl);
    return run_conv111_tc(a, dl, cout, cin, S, gout, ld_out, w, (ll) cin * cout, 1, cin, gin, ld_in, (cudaStream_t) stream, pname);
}

extern "C" int aprnet_conv111_backward_weights_tc(const aprnet_apr* a, int dl, int cin, int cout, int S, const float* in, int64_t ld_in,
                                                  const float* gout, int64_t ld_out, float* gw, float* partial, int64_t partial_elems,
                                                  void* stream) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && in && gout && gw && partial && cin > 0 && cout > 0 && S > 0, "bad argument");
    APRNET_DEVICE_CHECK(a);
    APRNET_ARG_CHECK(ld_in >= a->number_parts(dl) && ld_out >= a->number_parts(dl), "leading dimension too small");
    if (cin > 256 || cout > 256) return APRNET_ERR_UNSUPPORTED;      // (narrow layers included: the padding costs no memory traffic)
    cudaStream_t st = (cudaStream_t) stream;
    const ll elems = (ll) cin * cout;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int max_blocks = (int) std::min<ll>(sms, partial_elems / elems);
    if (max_blocks < 1) return APRNET_ERR_UNSUPPORTED;
    const int nt = pick_nt(cin), mtiles = (cout + 127) / 128;
    if (mtiles * nt > 512) return APRNET_ERR_UNSUPPORTED;
    for (const Segment& sg : aprnet_segments(a, dl, S, true)) {
        if (sg.end <= sg.begin) continue;
        C1DwParams P;
        P.seg_begin = sg.begin; P.seg_end = sg.end; P.in = in; P.ld_in = ld_in; P.cin = cin; P.gout = gout; P.ld_out = ld_out; P.cout = cout;
        P.partial = partial; P.error_flag = aprnet_tc_error_flag_device();
        const int grid = (int) std::min<ll>(max_blocks, (sg.end - sg.begin + TILE_M - 1) / TILE_M);
        int rc = APRNET_ERR_UNSUPPORTED;
        { AprnetProfScope _prof("conv111_tc_dw", st);
        switch (nt) {
            case 16: rc = launch_c1_dw<16>(P, grid, mtiles, st); break;
            case 32: rc = launch_c1_dw<32>(P, grid, mtiles, st); break;
            case 64: rc = launch_c1_dw<64>(P, grid, mtiles, st); break;
            case 128: rc = launch_c1_dw<128>(P, grid, mtiles, st); break;
            case 256: rc = launch_c1_dw<256>(P, grid, mtiles, st); break;
        }
        }
        if (rc) return rc;
        { AprnetProfScope _prof("conv111_dw_reduce", st);
        c1_reduce_partial_kernel<<<aprnet_ceil_div(elems, 256), 256, 0, st>>>(partial, grid, elems, gw + (ll) sg.slot * elems);
        }
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}
