// 3x3x3 particle convolution as an implicit GEMM on the 5th-generation tensor cores (tcgen05 + TMEM):
// bf16 operands, fp32 accumulation.  sm_100a only.
//
// The reference has no tensor-core path at all (its kernels are CUDA-core code with atomics,
// pyapr/aprnet/cuda/src/conv333_gpu.cu:11-579).  Formulation used here, per tile of 128 output
// locations of one level:
//
//     D[128 x Cout] (TMEM, fp32)  +=  A_tap[128 x Cin] (smem, bf16)  *  W_tap[Cin x Cout] (smem, bf16)     for the 27 taps
//
// A_tap is the gather of the tap's neighbour rows through the cached neighbour table.  To make that a
// plain row copy, the input (C, N) fp32 tensor (and the tree means) is first repacked into a
// channels-last bf16 matrix [row][Cpad]; a neighbour is then Cpad*2 contiguous bytes that go from
// global to shared memory with 16-byte cp.async copies, straight into a hardware-swizzled K-major
// operand layout.  Weights are packed once per call into the canonical unswizzled K-major layout and
// fetched with bulk copies.  One elected thread issues tcgen05.mma; completion is tracked with mbarriers
// (tcgen05.commit); accumulators are read back with tcgen05.ld and written once, coalesced, to the fp32
// (C, N) output.  Every wait is bounded: on expiry the block raises an error flag in host-mapped memory,
// drains its copies, frees its TMEM and returns.
//
// The same kernel computes the same-level part of the input gradient (input = dO, weights transposed
// and mirrored, neighbour entries masked to the location's own level) and the cross-level part (a
// gather over the targets of the edge plan, rows = per-(target, tap) sums of dO, result added to the
// gradient of the target).
#include "apr_device.cuh"
#include "tc_ptx.cuh"
#include <cuda_bf16.h>
#include <cuda.h>
#include <algorithm>
#include <cstring>

extern int g_dw_waves_override;     // defined with the weight-gradient kernel

namespace {

using namespace tcptx;
typedef long long ll;
constexpr int MAX_SEGS = APRNET_MAX_LEVELS;
constexpr int TILE_M = 128;

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

template<int KS> __device__ __forceinline__ int swizzled_chunk(int row, int c) {      // position of 16-byte chunk c of row `row`
    return KS == 64 ? (c ^ (row & 7)) : (KS == 32 ? (c ^ ((row >> 1) & 3)) : (c ^ ((row >> 2) & 1)));
}

// ---- operand packing --------------------------------------------------------------------------------
// rows [0, n): x[:, p]; rows [n, n + t): tree[:, p - n]; row n + t: zeros.  Channels padded to cpad.
__global__ void __launch_bounds__(256) pack_rows_bf16_kernel(const float* __restrict__ x, ll ld_x, ll n, const float* __restrict__ tree, ll ld_tree, ll t,
                                                             int c, int cpad, __nv_bfloat16* __restrict__ out) {
    // tile: 32 channels x 128 rows.  Reads are coalesced along the row (particle) axis of the channel-major
    // source, writes are 16-byte pieces (8 channels) of the packed rows.
    __shared__ float tile[32][129];
    const ll r0 = (ll) blockIdx.x * 128;
    const int c0 = blockIdx.y * 32;
    const ll rows = n + t + 1;
    const int lane = threadIdx.x & 31, wrp = threadIdx.x >> 5;      // 8 warps
#pragma unroll
    for (int cc = wrp; cc < 32; cc += 8) {
        const int ch = c0 + cc;
        float v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const ll r = r0 + lane + 32 * k;
            v[k] = 0.f;
            if (ch < c && r < n + t) v[k] = (r < n) ? x[(ll) ch * ld_x + r] : tree[(ll) ch * ld_tree + (r - n)];
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) tile[cc][lane + 32 * k] = v[k];
    }
    __syncthreads();
    // 128 rows x 4 pieces of 8 channels; consecutive threads take consecutive pieces of a row
#pragma unroll
    for (int e = threadIdx.x; e < 128 * 4; e += 256) {
        const int rr = e >> 2, piece = e & 3;
        const ll r = r0 + rr;
        if (r < rows && c0 + piece * 8 < cpad) {
            __nv_bfloat162 h[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(tile[piece * 8 + 2 * i][rr], tile[piece * 8 + 2 * i + 1][rr]);
            *reinterpret_cast<uint4*>(out + r * cpad + c0 + piece * 8) = *reinterpret_cast<uint4*>(h);
        }
    }
}

// Packed weights: [slot][tap][n_tile][k chunk j][n][8] bf16 (canonical K-major operand per (slot,tap,n_tile)).
// forward:  B[n = co][k = ci] = w[slot][co][ci][tap]
// backward == 1: B[n = ci][k = co] = w[slot][co][ci][26 - tap];  backward == 2: B[n = ci][k = co] = w[slot][co][ci][tap]
__global__ void pack_weights_bf16_kernel(const float* __restrict__ w, int slots, int cin, int cout, int backward,
                                         int n_dim, int k_dim, int nt, int n_tiles, int kpad, __nv_bfloat16* __restrict__ out) {
    const ll total = (ll) slots * 27 * n_tiles * (kpad / 8) * nt * 8;
    for (ll e = (ll) blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (ll) gridDim.x * blockDim.x) {
        ll r = e;
        const int k8 = (int) (r % 8); r /= 8;
        const int nn = (int) (r % nt); r /= nt;
        const int j = (int) (r % (kpad / 8)); r /= (kpad / 8);
        const int ntile = (int) (r % n_tiles); r /= n_tiles;
        const int tap = (int) (r % 27); r /= 27;
        const int slot = (int) r;
        const int nidx = ntile * nt + nn, kidx = j * 8 + k8;
        float v = 0.f;
        if (nidx < n_dim && kidx < k_dim) {
            const int co = backward ? kidx : nidx, ci = backward ? nidx : kidx;
            const int tp = (backward == 1) ? 26 - tap : tap;
            v = w[(((ll) slot * cout + co) * cin + ci) * 27 + tp];
        }
        out[e] = __float2bfloat16(v);
    }
}

// ---- kernel parameters -------------------------------------------------------------------------------
struct TcParams {
    SegTable segs;
    const int32_t* nbr; ll N;              // neighbour table [27][N]
    const __nv_bfloat16* rows; int kpad;   // packed source rows [R][kpad]
    ll tree_base, zero_row;                // row index of tree node 0 and of the zero row
    const __nv_bfloat16* wp;               // packed weights
    float* out; ll ld_out; int n_dim;      // output (n_dim, ld_out)
    int n_tiles;
    int same_level_only;                   // input-gradient mode: mask entries outside the tile's level
    int* error_flag;
    // target mode (cross-level input gradient): location a stands for target out_map[a]; the result is
    // added to out[:, t] for t < out_split and to out2[:, t - out_split] otherwise
    const int32_t* out_map; ll out_split;
    float* out2; ll ld_out2;
};

// ---- warp-specialised gather kernel ---------------------------------------------------------------
// One persistent block per SM, 13 warps (forward pass and both parts of the input gradient).  The unit of
// hand-over between the roles is a STAGE: TAPS consecutive taps x KS channels x 128 rows of the A operand plus the
// TAPS weight tiles that meet them.  Consecutive taps differ in dy only (tap = (dz * 3 + dx) * 3 + dy), so with
// TAPS = 3 a stage holds the three y-neighbours of one neighbour row.  A dependent mbarrier wait costs the waiting
// thread about 200 cycles and a tcgen05.commit about 50 whatever the stage holds (measured), so the MMA thread, which
// consumes the stages in order, wants few and large stages; a producer warp, on the other hand, sustains only one
// 512-byte copy instruction per ~100 cycles, so all eight must copy all the time.
//   warps 0-7   producers in groups of WPS warps.  A stage belongs to ONE group (group q fills the stages q,
//               q + NG, q + 2 NG ... of the block's stage sequence, NG = 8 / WPS groups work on NG stages at once);
//               inside the group warp s copies rows [s * 128 / WPS, (s + 1) * 128 / WPS) of every tap of the stage
//               with 16-byte cp.async copies straight into the hardware-swizzled K-major operand layout.  Every
//               lane attaches an asynchronous arrival to the stage's barrier (cp.async.mbarrier.arrive.noinc), so the
//               stage is handed to the MMA thread the moment its copies land and no producer ever waits for its own
//               copies; the first lane of the group streams the stage's weight tiles with bulk copies
//               (byte-counting arrival).  Producers only block on a ring slot the tensor core still reads;
//   warp 8      one thread issues the TAPS * KS / 16 tcgen05.mma of each stage back to back, in stage order, as soon
//               as the stage's barrier completes, and commits the stage's "slot free" barrier; accumulators rotate
//               through NACC TMEM buffers so that later tiles start while earlier ones are read back;
//   warps 9-12  epilogue: TMEM -> registers -> global for tile i; the neighbour-table entries of tile
//               i + NIDX are requested into registers before the wait for tile i and decoded into the
//               source-row buffer tile i has released afterwards, so their DRAM latency is never exposed.
// All waits are bounded and poll a block-wide abort flag.
constexpr int WS_NPROD = 8;
constexpr int WS_THREADS = (WS_NPROD + 5) * 32;
constexpr int WS_MAX_STAGES = 20;
constexpr int WS_MAX_ACC = 4;
constexpr int WS_NIDX = 3;

struct TileInfo { ll lo, hi, p0; int slot, ntile; };

__device__ __forceinline__ TileInfo tile_info(const TcParams& P, int work) {
    TileInfo t;
    const int tile = P.n_tiles == 1 ? work : work / P.n_tiles;
    t.ntile = P.n_tiles == 1 ? 0 : work % P.n_tiles;
    int seg = 0;
    while (seg + 1 < P.segs.n && tile >= P.segs.tile_begin[seg + 1]) ++seg;
    t.lo = P.segs.begin[seg]; t.hi = P.segs.end[seg];
    t.p0 = t.lo + (ll) (tile - P.segs.tile_begin[seg]) * TILE_M;
    t.slot = P.segs.slot[seg];
    return t;
}

template<int NT, int KS, int TAPS, int WPS, int TT, int NACC>
__global__ void __launch_bounds__(WS_THREADS, 1) conv333_tc_ws_kernel(const TcParams P, const int stages, const __grid_constant__ CUtensorMap row_map) {
    // A operand: K-major with the hardware swizzle whose width equals the row piece of one stage (KS
    // channels = 32, 64 or 128 bytes).  A gathered row piece is then contiguous in shared memory as it is
    // in global memory (its 16-byte chunks permuted inside the piece), so the lanes that copy one piece
    // write one contiguous block; with the unswizzled layout every 16-byte chunk of a row goes to a
    // different plane and each 32-byte sector costs its own pass of the shared-memory write pipe.
    constexpr int NIDX = WS_NIDX;
    constexpr int NG = WS_NPROD / WPS;                       // producer groups = stages in issue at once
    constexpr int CH = KS / 8;                               // 16-byte chunks per gathered row piece
    constexpr int RW = 32 / CH;                              // rows covered by one copy instruction of a warp
    constexpr int WROWS = TILE_M / WPS;                      // rows of a tap that one warp of the group copies
    constexpr int NI = WROWS / RW;                           // its copy instructions per tap
    constexpr int ROW_BYTES = KS * 2;
    constexpr uint32_t A_LAYOUT = KS == 64 ? 2u : (KS == 32 ? 4u : 6u);     // SWIZZLE_128B / 64B / 32B
    constexpr int A_TAP = TILE_M * ROW_BYTES;
    constexpr int B_TAP = NT * KS * 2;
    constexpr int STAGE_BYTES = TAPS * (A_TAP + B_TAP);
    constexpr int NTG = (27 + TAPS - 1) / TAPS;              // tap groups per tile
    constexpr uint32_t IDESC = make_idesc(NT, false, false);
    static_assert(WS_NPROD % WPS == 0 && NI >= 1 && WROWS % RW == 0, "a producer warp copies whole instructions");
    static_assert(TT >= 0 && TT < TAPS || (TT == 0), "the last TT taps of a stage come through the TMA unit, the others through cp.async");
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // swizzle atoms (8 rows) must start on a multiple of their size: align the ring to 1024 bytes
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* stage_base = smem;
    int32_t* idx_s = reinterpret_cast<int32_t*>(smem + (size_t) stages * STAGE_BYTES);      // NIDX x [27][128] source rows
    uint64_t* bars = reinterpret_cast<uint64_t*>(idx_s + NIDX * 27 * TILE_M);
    uint64_t* full = bars;                          // [stages]  copies of the stage landed (WPS x 32 lanes + weight bytes)
    uint64_t* empty = bars + WS_MAX_STAGES;         // [stages]  MMAs that read the stage completed
    uint64_t* tmem_full = empty + WS_MAX_STAGES;    // [NACC]    accumulator complete
    uint64_t* tmem_empty = tmem_full + WS_MAX_ACC;  // [NACC]    accumulator read back (one arrival per epilogue warp)
    uint64_t* idx_full = tmem_empty + WS_MAX_ACC;   // [NIDX]    source rows of a tile written (one arrival per epilogue warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(idx_full + WS_MAX_ACC);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kchunks = P.kpad / KS;
    const int steps_per_tile = NTG * kchunks;
    const int total_tiles = P.segs.tile_begin[P.segs.n] * P.n_tiles;
    const int my_tiles = (int) blockIdx.x < total_tiles ? (total_tiles - (int) blockIdx.x + (int) gridDim.x - 1) / (int) gridDim.x : 0;
    const int ngroups = min(NG, stages);            // groups that take part (every group's first stage has its own slot)

    if (tid == 0) {
        for (int i = 0; i < stages; ++i) { mbar_init(smem_u32(full + i), WPS * 32 + 1); mbar_init(smem_u32(empty + i), 1); }
        for (int i = 0; i < NACC; ++i) { mbar_init(smem_u32(tmem_full + i), 1); mbar_init(smem_u32(tmem_empty + i), 4); }
        for (int i = 0; i < NIDX; ++i) mbar_init(smem_u32(idx_full + i), 4);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == WS_NPROD) { tmem_alloc(smem_u32(tmem_slot), NACC * NT); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_slot;
    bool failed = false;
    bool bulk_issued = false;

    if (warp < WS_NPROD) {
        // ---------------- producers ----------------
        const int grp = warp / WPS, sub = warp % WPS;
        if (grp < ngroups) {
            const int j = lane % CH, r0 = sub * WROWS + lane / CH;
            const uint32_t total_stages = (uint32_t) my_tiles * (uint32_t) steps_per_tile;
            uint32_t g = grp, slot = grp, use = 0;
            int it = 0, step = grp, cur_it = -1;
            const int32_t* idx = idx_s;
            const unsigned char* wsrc = nullptr;
            const ll w_tap_stride = (ll) P.n_tiles * P.kpad * NT * 2;
            while (g < total_stages) {
                while (step >= steps_per_tile) { step -= steps_per_tile; ++it; }
                if (it != cur_it) {
                    cur_it = it;
                    if (!mbar_wait_warp(smem_u32(idx_full + it % NIDX), (it / NIDX) & 1, abort_flag)) { failed = true; break; }
                    idx = idx_s + (it % NIDX) * 27 * TILE_M + r0;
                    if (sub == 0 && lane == 0) {      // packed weights of one (slot, tap, n tile) are [k chunk][n][8]; a stage takes KS / 8 chunks of TAPS taps
                        const TileInfo ti = tile_info(P, blockIdx.x + it * gridDim.x);
                        wsrc = reinterpret_cast<const unsigned char*>(P.wp + ((ll) ti.slot * 27 * P.n_tiles + ti.ntile) * ((ll) P.kpad * NT));
                    }
                }
                const int tg = step / kchunks, kc = step - tg * kchunks;
                const int t0 = tg * TAPS;
                if (use > 0 && !mbar_wait_warp(smem_u32(empty + slot), (use - 1) & 1, abort_flag)) { failed = true; break; }
                unsigned char* a_s = stage_base + (size_t) slot * STAGE_BYTES;
                if (sub == 0 && lane == 0) {
                    const int nt = min(TAPS, 27 - t0);
                    mbar_expect_tx(smem_u32(full + slot), nt * B_TAP + max(0, nt - (TAPS - TT)) * A_TAP);
                    for (int t = 0; t < nt; ++t)
                        bulk_copy_g2s(smem_u32(a_s + TAPS * A_TAP + t * B_TAP), wsrc + (ll) (t0 + t) * w_tap_stride + (ll) kc * KS * NT * 2,
                                      B_TAP, smem_u32(full + slot));
                    bulk_issued = true;
                }
                if (TT > 0 && sub == WPS - 1) {
                    // the stage's last TT taps: lane l asks the TMA unit for rows 4l..4l+3 of the tap (tile::gather4 writes
                    // the same swizzled layout); the bytes count against the arrival that the group's first lane
                    // announces (a copy that completes earlier only drives the byte count negative until then)
#pragma unroll
                    for (int t = TAPS - TT; t < TAPS; ++t) {
                        if (t0 + t < 27) {
                            const int4 r = *reinterpret_cast<const int4*>(idx - r0 + (t0 + t) * TILE_M + 4 * lane);
                            tma_gather4(smem_u32(a_s + t * A_TAP + 4 * lane * ROW_BYTES), &row_map, kc * KS, r.x, r.y, r.z, r.w, smem_u32(full + slot));
                            bulk_issued = true;
                        }
                    }
                }
                const __nv_bfloat16* src0 = P.rows + kc * KS + j * 8;
#pragma unroll
                for (int t = 0; t < TAPS - TT; ++t) {
                    if (t0 + t < 27) {
                        const int32_t* idx_t = idx + (t0 + t) * TILE_M;
                        int32_t src_row[NI];          // read together first: the copy instructions order memory accesses, a read between two of them would wait
#pragma unroll
                        for (int i = 0; i < NI; ++i) src_row[i] = idx_t[i * RW];
#pragma unroll
                        for (int i = 0; i < NI; ++i) {
                            const int row = r0 + i * RW;
                            cp_async16(smem_u32(a_s + t * A_TAP + row * ROW_BYTES + (swizzled_chunk<KS>(row, j) << 4)), src0 + (ll) src_row[i] * P.kpad);
                        }
                    }
                }
                // the stage's barrier receives this thread's arrival when the copies above have landed
                cp_async_arrive_noinc(smem_u32(full + slot));
                g += ngroups; step += ngroups; slot += ngroups;
                if (slot >= (uint32_t) stages) { slot -= stages; ++use; }
            }
            cp_async_commit();
            cp_async_wait<0>();
        }
    } else if (warp == WS_NPROD) {
        // ---------------- MMA issue ----------------
        if (lane == 0) {
            uint32_t slot = 0, use = 0;
            for (int it = 0; it < my_tiles && !failed; ++it) {
                const uint32_t acc = (uint32_t) it % NACC, acc_use = (uint32_t) it / NACC;
                if (acc_use > 0 && !mbar_wait(smem_u32(tmem_empty + acc), (acc_use - 1) & 1, abort_flag)) { failed = true; break; }
                tc_fence_after();
                const uint32_t d_addr = tmem_d + acc * NT;
                int t0 = 0, kc = 0;
                for (int step = 0; step < steps_per_tile; ++step) {
                    if (!mbar_wait(smem_u32(full + slot), use & 1, abort_flag)) { failed = true; break; }
                    fence_proxy_async();          // generic-proxy writes of the cp.async copies -> tensor-core (async proxy) reads
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(stage_base + (size_t) slot * STAGE_BYTES);
                    // descriptors of the stage's first MMA; the others add the encoded byte offset of their operand
                    const uint64_t da0 = make_desc(a_addr, 16, 8 * ROW_BYTES, A_LAYOUT);
                    const uint64_t db0 = make_desc(a_addr + TAPS * A_TAP, NT * 16, 128, 0);
#pragma unroll
                    for (int t = 0; t < TAPS; ++t) {
                        if (t0 + t < 27) {
#pragma unroll
                            for (int k = 0; k < KS / 16; ++k)
                                umma_bf16(d_addr, da0 + (uint64_t) ((t * A_TAP + k * 32) >> 4), db0 + (uint64_t) ((t * B_TAP + k * 2 * (NT * 16)) >> 4),
                                          IDESC, (step > 0 || t > 0 || k > 0) ? 1u : 0u);
                        }
                    }
                    umma_commit(smem_u32(empty + slot));
                    if (++slot == (uint32_t) stages) { slot = 0; ++use; }
                    if (++kc == kchunks) { kc = 0; t0 += TAPS; }
                }
                if (!failed) umma_commit(smem_u32(tmem_full + acc));
            }
        }
    } else if (warp >= WS_NPROD + 1) {
        // ---------------- epilogue + source-row staging ----------------
        const int q = warp & 3;                           // TMEM lane group this warp may read
        const int row = q * 32 + lane;
        int32_t v[27];
        auto request_idx = [&](int it) {                  // table entries of this thread's row of tile `it` -> registers
            if (it >= my_tiles) return;
            const TileInfo ti = tile_info(P, blockIdx.x + it * gridDim.x);
            const ll p = ti.p0 + row;
#pragma unroll
            for (int tap = 0; tap < 27; ++tap) v[tap] = (p < ti.hi) ? __ldg(P.nbr + (ll) tap * P.N + p) : APRNET_NONE;
        };
        auto publish_idx = [&](int it) {                  // decode and hand the rows to the producers
            if (it >= my_tiles) return;
            const TileInfo ti = tile_info(P, blockIdx.x + it * gridDim.x);
            int32_t* dst = idx_s + (it % NIDX) * 27 * TILE_M;
#pragma unroll
            for (int tap = 0; tap < 27; ++tap) {
                ll r = P.zero_row;
                if (P.same_level_only) { if (v[tap] >= ti.lo && v[tap] < ti.hi) r = v[tap]; }
                else if (v[tap] >= 0) r = v[tap];
                else if (v[tap] != APRNET_NONE) r = P.tree_base + aprnet_dec_tree(v[tap]);
                dst[tap * TILE_M + row] = (int32_t) r;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(idx_full + it % NIDX));
        };
        for (int it = 0; it < NIDX; ++it) { request_idx(it); publish_idx(it); }
        for (int it = 0; it < my_tiles; ++it) {
            const TileInfo ti = tile_info(P, blockIdx.x + it * gridDim.x);
            const ll p = ti.p0 + row;
            const bool valid = p < ti.hi;
            float* acc_dst = nullptr; ll acc_ld = 0;
            if (P.out_map && valid) {
                const ll t = P.out_map[p];
                acc_dst = t < P.out_split ? P.out + t : P.out2 + (t - P.out_split);
                acc_ld = t < P.out_split ? P.ld_out : P.ld_out2;
            }
            const uint32_t acc = (uint32_t) it % NACC, acc_use = (uint32_t) it / NACC;
            request_idx(it + NIDX);       // lands while this warp waits for the accumulator
            if (!mbar_wait_warp(smem_u32(tmem_full + acc), acc_use & 1, abort_flag)) { failed = true; break; }
            tc_fence_after();
#pragma unroll
            for (int c0 = 0; c0 < NT; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_d + ((uint32_t) (q * 32) << 16) + acc * NT + c0, r);
                tmem_ld_wait();
                if (valid && !P.out_map) {
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj) {
                        const int n = ti.ntile * NT + c0 + jj;
                        if (n < P.n_dim) P.out[(ll) n * P.ld_out + p] = __uint_as_float(r[jj]);
                    }
                } else if (valid) {          // this thread is the only writer of its target: read all, then add and write
#pragma unroll
                    for (int h = 0; h < 32; h += 16) {        // 16 independent loads at a time
                        float old[16];
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj) {
                            const int n = ti.ntile * NT + c0 + h + jj;
                            old[jj] = n < P.n_dim ? acc_dst[(ll) n * acc_ld] : 0.f;
                        }
#pragma unroll
                        for (int jj = 0; jj < 16; ++jj) {
                            const int n = ti.ntile * NT + c0 + h + jj;
                            if (n < P.n_dim) acc_dst[(ll) n * acc_ld] = old[jj] + __uint_as_float(r[h + jj]);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(tmem_empty + acc));
            // every copy that read the source rows of tile `it` has landed (its accumulator is complete)
            publish_idx(it + NIDX);
        }
    }

    // teardown (also the error path): the gather copies were drained above; after a failure the bulk
    // copies still in flight get time to land before the block's shared memory is released
    if (failed) {
        *abort_flag = 1;
        if (P.error_flag) *P.error_flag = 1;
    }
    tc_fence_before();
    __syncthreads();
    if (bulk_issued && *abort_flag) for (int i = 0; i < 2000; ++i) __nanosleep(100);
    if (warp == WS_NPROD) tmem_dealloc(tmem_d, NACC * NT);
}

// ---- host side ----------------------------------------------------------------------------------------
int* g_error_flag_host = nullptr;     // host-mapped; written by kernels whose bounded waits expired
int* g_error_flag_dev = nullptr;

int ensure_error_flag() {
    if (g_error_flag_host) return APRNET_OK;
    APRNET_CUDA_CHECK(cudaHostAlloc((void**) &g_error_flag_host, sizeof(int), cudaHostAllocMapped));
    *g_error_flag_host = 0;
    APRNET_CUDA_CHECK(cudaHostGetDevicePointer((void**) &g_error_flag_dev, g_error_flag_host, 0));
    return APRNET_OK;
}

inline int pad_to(int v, int m) { return (v + m - 1) / m * m; }
inline int pick_nt(int n) { return n <= 32 ? 32 : (n <= 64 ? 64 : (n <= 128 ? 128 : 256)); }

struct TcGeom { int kpad, ks, nt, n_tiles; size_t rows_bytes, w_bytes; };

int g_ks_override = 0;       // aprnet_tc_set_option("ks", n): channels per stage, measurement switch

TcGeom tc_geometry(ll rows, int k_dim, int n_dim, int slots) {
    TcGeom g;
    g.kpad = pad_to(k_dim, 16);
    g.nt = pick_nt(n_dim);
    g.ks = (g.kpad % 64 == 0 && g.nt <= 128) ? 64 : ((g.kpad % 32 == 0) ? 32 : 16);
    // 64 output channels: stages of 3 taps x 32 channels (5 ring slots, 4 producer groups) measured 3-10 % faster than
    // 2 taps x 64 channels (3 slots, 2 groups); for 32 and 128 outputs the 64-channel stages win
    if (g.nt == 64 && g.ks == 64) g.ks = 32;
    if (g_ks_override > 0 && g.kpad % g_ks_override == 0 && (g_ks_override < 64 || g.nt <= 128)) g.ks = g_ks_override;
    g.n_tiles = (n_dim + g.nt - 1) / g.nt;
    g.rows_bytes = ((size_t) rows * g.kpad * 2 + 255) / 256 * 256;
    g.w_bytes = ((size_t) slots * 27 * g.n_tiles * g.kpad * g.nt * 2 + 255) / 256 * 256;
    return g;
}

// Stage geometry per tile shape: (taps per stage, producer warps per stage).  The ring needs one slot per producer
// group plus one for the tensor core; stages are as large as that allows, because the MMA thread pays a fixed
// ~250 cycles (dependent barrier wait + commit) per stage.
int g_taps_override = 0, g_wps_override = 0, g_tma_taps_override = 0;      // aprnet_tc_set_option("taps" / "wps" / "tma_taps", n): measurement switches

constexpr size_t WS_FIXED = (size_t) WS_NIDX * 27 * TILE_M * 4 + (2 * WS_MAX_STAGES + 3 * WS_MAX_ACC) * 8 + 16 + 1024;      // + alignment slack
constexpr size_t WS_SMEM = 227 * 1024 - 1024;

inline int ws_stages(int nt, int ks, int taps) {
    const size_t stage = (size_t) taps * ((size_t) TILE_M * ks * 2 + (size_t) nt * ks * 2);
    return (int) std::min<size_t>(WS_MAX_STAGES, (WS_SMEM - WS_FIXED) / stage);
}

// (output tile width, channels per stage, taps per stage, warps per stage) combinations that are compiled
#define TC_VARIANTS(X) \
    X(32, 16, 1, 1) X(32, 16, 3, 1) X(32, 16, 9, 2) X(32, 32, 1, 1) X(32, 32, 3, 1) X(32, 32, 3, 2) X(32, 32, 9, 4) \
    X(32, 64, 1, 1) X(32, 64, 3, 2) X(32, 64, 3, 4) \
    X(64, 16, 1, 1) X(64, 16, 3, 1) X(64, 16, 9, 2) X(64, 32, 1, 1) X(64, 32, 3, 2) X(64, 64, 1, 1) X(64, 64, 2, 2) X(64, 64, 2, 4) X(64, 64, 3, 4) \
    X(128, 16, 1, 1) X(128, 16, 3, 2) X(128, 32, 1, 1) X(128, 32, 2, 2) X(128, 32, 3, 4) X(128, 64, 1, 1) X(128, 64, 1, 2) X(128, 64, 2, 4) \
    X(256, 16, 1, 1) X(256, 16, 3, 2) X(256, 32, 1, 1) X(256, 32, 2, 2) X(256, 32, 2, 4)

// the same with the last TT taps of every stage fetched by the TMA unit
#define TC_TMA_VARIANTS(X) \
    X(32, 32, 3, 2, 1) X(64, 64, 2, 2, 1) X(32, 64, 3, 2, 1)

inline bool tc_variant_ok(int nt, int ks, int taps, int wps, int tt = 0) {
    bool compiled = false;
#define X(NT_, KS_, TAPS_, WPS_) if (tt == 0 && nt == NT_ && ks == KS_ && taps == TAPS_ && wps == WPS_) compiled = true;
    TC_VARIANTS(X)
#undef X
#define X(NT_, KS_, TAPS_, WPS_, TT_) if (tt == TT_ && nt == NT_ && ks == KS_ && taps == TAPS_ && wps == WPS_) compiled = true;
    TC_TMA_VARIANTS(X)
#undef X
    return compiled && ws_stages(nt, ks, taps) >= WS_NPROD / wps + 1;
}

// default choice: the compiled variant with the most taps per stage whose ring holds all producer groups plus one
// slot; among equals the one with the fewest warps per stage (more stages in issue at once)
inline void pick_stage_shape(int nt, int ks, bool allow_tma, int* taps, int* wps, int* tt) {
    *tt = 0;
    const int tt_want = allow_tma ? g_tma_taps_override : 0;
    if (g_taps_override > 0 && g_wps_override > 0 && tc_variant_ok(nt, ks, g_taps_override, g_wps_override, tt_want)) {
        *taps = g_taps_override; *wps = g_wps_override; *tt = tt_want; return;
    }
    // 32-channel rows into 32-wide tiles: one of three taps through the TMA unit measured 3-6 % faster than all by cp.async
    if (allow_tma && nt == 32 && ks == 32 && g_taps_override == 0 && tc_variant_ok(nt, ks, 3, 2, 1)) { *taps = 3; *wps = 2; *tt = 1; return; }
    *taps = 1; *wps = 1;
    static const int tcand[4] = {9, 3, 2, 1}, wcand[3] = {1, 2, 4};
    for (int t : tcand)
        for (int w : wcand)
            if (tc_variant_ok(nt, ks, t, w)) { *taps = t; *wps = w; return; }
}

// Tensor map of the packed rows [n_rows][kpad] (bf16) with a box of one row piece (ks channels) and the
// swizzle mode whose span equals the piece: tile::gather4 copies four such pieces per instruction.
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int make_row_map(CUtensorMap* map, const void* rows, ll n_rows, int kpad, int ks) {
    static EncodeTiledFn encode = nullptr;
    if (!encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn) {
            cudaGetLastError();
            return APRNET_ERR_UNSUPPORTED;
        }
        encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
    if ((reinterpret_cast<uintptr_t>(rows) & 15) || n_rows <= 0 || n_rows >= (1ll << 31)) return APRNET_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t) kpad, (cuuint64_t) n_rows};
    const cuuint64_t strides[1] = {(cuuint64_t) kpad * 2};
    const cuuint32_t box[2] = {(cuuint32_t) ks, 1};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapSwizzle sw = ks == 64 ? CU_TENSOR_MAP_SWIZZLE_128B : (ks == 32 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
    const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(rows), dims, strides, box, estr,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? APRNET_OK : APRNET_ERR_UNSUPPORTED;
}

template<int NT, int KS, int TAPS, int WPS, int TT>
int launch_tc_ws(const TcParams& P, int total_tiles, cudaStream_t st, const char* pname) {
    constexpr size_t STAGE = (size_t) TAPS * ((size_t) TILE_M * KS * 2 + (size_t) NT * KS * 2);
    constexpr int NACC = NT <= 128 ? 4 : 2;          // accumulators in flight: the SM's 512 TMEM columns, at most 4
    auto kern = conv333_tc_ws_kernel<NT, KS, TAPS, WPS, TT, NACC>;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // one block per SM with all of its shared memory (227 KB, 1 KB reserved) as the stage ring
    const int stages = ws_stages(NT, KS, TAPS);
    if (stages < 2) { aprnet_set_error("conv333 tensor-core path: tile nt=%d ks=%d taps=%d does not fit shared memory", NT, KS, TAPS); return APRNET_ERR_UNSUPPORTED; }
    const size_t smem = (size_t) stages * STAGE + WS_FIXED;
    APRNET_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    const int grid = std::min(total_tiles, sms);
    CUtensorMap row_map;
    memset(&row_map, 0, sizeof(row_map));
    // the map ends before the zero row: that coordinate is then out of bounds and the TMA unit fills the piece with
    // zeros without touching memory
    if (TT > 0 && make_row_map(&row_map, P.rows, P.zero_row, P.kpad, KS) != APRNET_OK) {
        aprnet_set_error("conv333 tensor-core path: no tensor map for the packed rows");
        return APRNET_ERR_UNSUPPORTED;
    }
    { AprnetProfScope _prof(pname, st);
    kern<<<grid, WS_THREADS, smem, st>>>(P, stages, row_map);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

int dispatch_tc(const TcParams& P, const TcGeom& g, int total_tiles, cudaStream_t st, const char* pname) {
    int taps = 1, wps = 1, tt = 0;
    // the rows of the cross-level pass are addressed from a shifted base with the zero row in front: no tensor map for them
    pick_stage_shape(g.nt, g.ks, P.out_map == nullptr, &taps, &wps, &tt);
#define X(NT_, KS_, TAPS_, WPS_) if (tt == 0 && g.nt == NT_ && g.ks == KS_ && taps == TAPS_ && wps == WPS_) return launch_tc_ws<NT_, KS_, TAPS_, WPS_, 0>(P, total_tiles, st, pname);
    TC_VARIANTS(X)
#undef X
#define X(NT_, KS_, TAPS_, WPS_, TT_) if (tt == TT_ && g.nt == NT_ && g.ks == KS_ && taps == TAPS_ && wps == WPS_) return launch_tc_ws<NT_, KS_, TAPS_, WPS_, TT_>(P, total_tiles, st, pname);
    TC_TMA_VARIANTS(X)
#undef X
    aprnet_set_error("conv333 tensor-core path: unsupported tile geometry nt=%d ks=%d taps=%d wps=%d", g.nt, g.ks, taps, wps);
    return APRNET_ERR_UNSUPPORTED;
}

int run_pack_rows(const float* x, ll ld_x, ll n, const float* tree, ll ld_tree, ll t, int c, int cpad, __nv_bfloat16* out, cudaStream_t st) {
    dim3 grid((unsigned) aprnet_ceil_div(n + t + 1, 128), (unsigned) aprnet_ceil_div(cpad, 32));
    { AprnetProfScope _prof("pack_rows_bf16", st);
    pack_rows_bf16_kernel<<<grid, 256, 0, st>>>(x, ld_x, n, tree, ld_tree, t, c, cpad, out);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

} // namespace

int* aprnet_tc_error_flag_device() { return ensure_error_flag() == APRNET_OK ? g_error_flag_dev : nullptr; }

int aprnet_tc_pack_rows(const float* x, ll ld_x, ll n, const float* tree, ll ld_tree, ll t, int c, int cpad, void* out, cudaStream_t st) {
    return run_pack_rows(x, ld_x, n, tree, ld_tree, t, c, cpad, reinterpret_cast<__nv_bfloat16*>(out), st);
}

// Gather-GEMM over packed rows.  backward == 0: out[n = co] from rows of the input (k = ci);
// backward == 1: out[n = ci] from rows of grad_output (k = co), same-level neighbours only, mirrored taps.
int aprnet_tc_gather_conv(aprnet_apr* a, int dl, int backward, int cin, int cout, int slots, const void* rows, int kpad,
                          ll tree_base, ll zero_row, const float* w, void* wp_ws, float* out, ll ld_out, cudaStream_t st) {
    int rc = ensure_error_flag();
    if (rc) return rc;
    if (*g_error_flag_host) { aprnet_set_error("a previous tensor-core kernel gave up waiting on a barrier"); return APRNET_ERR_CUDA; }
    const AprPlan* plan = aprnet_get_plan(a, dl, st);
    if (!plan) return APRNET_ERR_CUDA;
    const int k_dim = backward ? cout : cin, n_dim = backward ? cin : cout;
    const TcGeom g = tc_geometry(1, k_dim, n_dim, slots);
    if (g.kpad != kpad) { aprnet_set_error("packed row width %d does not match the padded channel count %d", kpad, g.kpad); return APRNET_ERR_ARG; }
    __nv_bfloat16* wp = reinterpret_cast<__nv_bfloat16*>(wp_ws);
    { AprnetProfScope _prof("pack_weights_bf16", st);
    pack_weights_bf16_kernel<<<std::min(1024, aprnet_ceil_div((ll) slots * 27 * g.n_tiles * g.kpad * g.nt, 256)), 256, 0, st>>>(
        w, slots, cin, cout, backward, n_dim, k_dim, g.nt, g.n_tiles, g.kpad, wp);
    }
    APRNET_LAUNCH_CHECK();
    TcParams P;
    P.segs = make_seg_table(aprnet_segments(a, dl, slots, false), TILE_M);
    P.nbr = plan->nbr; P.N = plan->n; P.rows = reinterpret_cast<const __nv_bfloat16*>(rows); P.kpad = g.kpad;
    P.tree_base = tree_base; P.zero_row = zero_row;
    P.wp = wp; P.out = out; P.ld_out = ld_out; P.n_dim = n_dim; P.n_tiles = g.n_tiles; P.same_level_only = backward;
    P.error_flag = g_error_flag_dev;
    P.out_map = nullptr; P.out_split = 0; P.out2 = nullptr; P.ld_out2 = 0;

    const int total = P.segs.tile_begin[P.segs.n] * g.n_tiles;
    if (total == 0) return APRNET_OK;
    char pname[64];
    snprintf(pname, sizeof(pname), "%s:ci%d:co%d:dl%d", backward ? "conv333_tc_bwd_gather" : "conv333_tc_fwd", cin, cout, dl);
    return dispatch_tc(P, g, total, st, pname);
}

int aprnet_tc_pack_weights(const float* w, int slots, int cin, int cout, int mode, void* wp, cudaStream_t st) {
    const int k_dim = mode ? cout : cin, n_dim = mode ? cin : cout;
    const TcGeom g = tc_geometry(1, k_dim, n_dim, slots);
    { AprnetProfScope _prof("pack_weights_bf16", st);
    pack_weights_bf16_kernel<<<std::min(1024, aprnet_ceil_div((ll) slots * 27 * g.n_tiles * g.kpad * g.nt, 256)), 256, 0, st>>>(
        w, slots, cin, cout, mode, n_dim, k_dim, g.nt, g.n_tiles, g.kpad, reinterpret_cast<__nv_bfloat16*>(wp));
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

// Gather GEMM over the active targets [a0, a1) of an edge plan (weights already packed with mode 2).
int aprnet_tc_gather_targets(aprnet_apr* a, int dl, int cin, int cout, int slots, const void* vrows, int gpad, ll zero_row,
                             const void* wp_packed, const EdgePlan* ep, ll a0, ll a1,
                             float* gin, ll ld_in, float* gtree, ll ld_tree, cudaStream_t st) {
    int rc = ensure_error_flag();
    if (rc) return rc;
    if (*g_error_flag_host) { aprnet_set_error("a previous tensor-core kernel gave up waiting on a barrier"); return APRNET_ERR_CUDA; }
    const TcGeom g = tc_geometry(1, cout, cin, slots);
    if (g.kpad != gpad) { aprnet_set_error("packed row width %d does not match the padded channel count %d", gpad, g.kpad); return APRNET_ERR_ARG; }
    const int cml = a->cml(dl);
    std::vector<Segment> segs;
    for (const ActiveSeg& sg : ep->segs) {
        Segment s;
        s.begin = std::max(sg.begin, a0); s.end = std::min(sg.end, a1);
        s.level = sg.location_level; s.slot = std::min(cml - sg.location_level, slots - 1);
        if (s.end > s.begin) segs.push_back(s);
    }
    if (segs.empty()) return APRNET_OK;
    TcParams P;
    memset(&P, 0, sizeof(P));
    P.segs = make_seg_table(segs, TILE_M);
    P.nbr = ep->vnbr; P.N = ep->n_active;
    P.rows = reinterpret_cast<const __nv_bfloat16*>(vrows); P.kpad = g.kpad; P.zero_row = zero_row; P.tree_base = zero_row;
    P.wp = reinterpret_cast<const __nv_bfloat16*>(wp_packed); P.n_dim = cin; P.n_tiles = g.n_tiles;
    P.same_level_only = 0; P.error_flag = g_error_flag_dev;
    P.out = gin; P.ld_out = ld_in; P.out_map = ep->active; P.out_split = a->number_parts(dl); P.out2 = gtree; P.ld_out2 = ld_tree;
    const int total = P.segs.tile_begin[P.segs.n] * g.n_tiles;
    char pname[64];
    snprintf(pname, sizeof(pname), "conv333_tc_cross:ci%d:co%d:dl%d", cin, cout, dl);
    return dispatch_tc(P, g, total, st, pname);
}

size_t aprnet_tc_rows_bytes(ll rows, int channels) { return tc_geometry(rows, channels, 16, 1).rows_bytes; }
size_t aprnet_tc_weight_bytes(int k_dim, int n_dim, int slots) { return tc_geometry(1, k_dim, n_dim, slots).w_bytes; }
int aprnet_tc_pad(int channels) { return pad_to(channels, 16); }

extern "C" int aprnet_tc_error_flag(void) { return g_error_flag_host ? *g_error_flag_host : 0; }

namespace {
// One thread waits, with the given poll limit, on an mbarrier that nothing arrives at: the wait runs out, the block
// raises the error flag like the convolution kernels do, and returns.  Exercises the error path without a hang.
__global__ void wait_timeout_selftest_kernel(unsigned max_polls, int* error_flag) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); fence_mbar_init(); }
    __syncthreads();
    if (threadIdx.x == 0) {
        bool done = false;
        for (unsigned it = 0; it < max_polls && !done; ++it) done = mbar_try_wait(smem_u32(&bar), 0);
        if (!done && error_flag) *error_flag = 1;
    }
}
} // namespace

extern "C" int aprnet_tc_selftest_wait_timeout(int max_polls, void* stream) {
    APRNET_ARG_CHECK(max_polls > 0 && max_polls <= (1 << 20), "poll limit must be in [1, 2^20]");
    int rc = ensure_error_flag();
    if (rc) return rc;
    wait_timeout_selftest_kernel<<<1, 32, 0, (cudaStream_t) stream>>>((unsigned) max_polls, g_error_flag_dev);
    APRNET_LAUNCH_CHECK();
    APRNET_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t) stream));
    return APRNET_OK;
}

extern "C" void aprnet_tc_error_reset(void) { if (g_error_flag_host) *g_error_flag_host = 0; }

extern "C" int aprnet_tc_set_option(const char* name, int value) {
    APRNET_ARG_CHECK(name, "null option name");
    if (!strcmp(name, "taps")) { g_taps_override = value; return APRNET_OK; }
    if (!strcmp(name, "wps")) { g_wps_override = value; return APRNET_OK; }
    if (!strcmp(name, "tma_taps")) { g_tma_taps_override = value; return APRNET_OK; }
    if (!strcmp(name, "dw_waves")) { g_dw_waves_override = value; return APRNET_OK; }
    if (!strcmp(name, "ks")) {
        APRNET_ARG_CHECK(value == 0 || value == 16 || value == 32 || value == 64, "channels per stage must be 0 (automatic), 16, 32 or 64");
        g_ks_override = value;
        return APRNET_OK;
    }
    aprnet_set_error("aprnet_tc_set_option: unknown option '%s'", name);
    return APRNET_ERR_ARG;
}

extern "C" int64_t aprnet_conv333_tc_workspace_bytes(const aprnet_apr* a, int dl, int cin, int cout, int slots) {
    if (!a || !a->valid_dl(dl)) return -1;
    const ll n = a->number_parts(dl), t = a->tree_size(dl);
    // forward: packed input rows + packed weights.  backward: packed input rows, packed dO rows,
    // packed (transposed) weights.  One size serves both calls.
    const size_t fwd = aprnet_tc_rows_bytes(n + t + 1, cin) + aprnet_tc_weight_bytes(cin, cout, slots);
    const size_t bwd = aprnet_tc_rows_bytes(n + t + 1, cin) + aprnet_tc_rows_bytes(n + 1, cout) + aprnet_tc_weight_bytes(cout, cin, slots) +
                       (size_t) aprnet_edge_workspace_bytes(a, dl, cout);
    return (int64_t) std::max(fwd, bwd);
}

extern "C" int64_t aprnet_conv333_tc_forward_workspace_bytes(const aprnet_apr* a, int dl, int cin, int cout, int slots) {
    if (!a || !a->valid_dl(dl)) return -1;
    return (int64_t) (aprnet_tc_rows_bytes(a->number_parts(dl) + a->tree_size(dl) + 1, cin) + aprnet_tc_weight_bytes(cin, cout, slots));
}

// forward: out = conv(in) with bf16 operands / fp32 accumulation; tree_scratch receives the fp32 tree means
static int conv333_forward_tc_impl(aprnet_apr* a, int dl, int cin, int cout, int slots, const float* in, int64_t ld_in,
                                   const float* w, float* out, int64_t ld_out, float* tree, int64_t ld_tree,
                                   void* workspace, void* stream, bool tree_valid) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && cin > 0 && cout > 0 && slots > 0 && in && w && out && tree && workspace, "bad argument");
    APRNET_ARG_CHECK(ld_in >= a->number_parts(dl) && ld_out >= a->number_parts(dl) && ld_tree >= a->tree_size(dl), "leading dimension too small");
    cudaStream_t st = (cudaStream_t) stream;
    int rc = tree_valid ? APRNET_OK : aprnet_fill_tree_mean_forward(a, dl, APRNET_F32, cin, in, ld_in, tree, ld_tree, st);
    if (rc) return rc;
    const ll n = a->number_parts(dl), t = a->tree_size(dl);
    const int kpad = aprnet_tc_pad(cin);
    char* ws = (char*) workspace;
    void* rows = ws;
    void* wp = ws + aprnet_tc_rows_bytes(n + t + 1, cin);
    if (aprnet_small_cin(cin)) {         // first-layer widths: fp32 CUDA-core kernels; the rows area holds the fp32 staging buffer instead
        if ((rc = aprnet_small_stage(in, ld_in, n, tree, ld_tree, t, cin, (float*) rows, st))) return rc;
        return aprnet_small_forward(a, dl, cin, cout, slots, (const float*) rows, w, out, ld_out, st);
    }
    rc = aprnet_tc_pack_rows(in, ld_in, n, tree, ld_tree, t, cin, kpad, rows, st);
    if (rc) return rc;
    return aprnet_tc_gather_conv(a, dl, 0, cin, cout, slots, rows, kpad, n, n + t, w, wp, out, ld_out, st);
}

extern "C" int aprnet_conv333_forward_tc(aprnet_apr* a, int dl, int cin, int cout, int slots, const float* in, int64_t ld_in,
                                         const float* w, float* out, int64_t ld_out, float* tree, int64_t ld_tree,
                                         void* workspace, void* stream) {
    return conv333_forward_tc_impl(a, dl, cin, cout, slots, in, ld_in, w, out, ld_out, tree, ld_tree, workspace, stream, false);
}

// Split form (see aprnet_conv333_forward_pretree): the tree means are taken as given.
extern "C" int aprnet_conv333_forward_tc_pretree(aprnet_apr* a, int dl, int cin, int cout, int slots, const float* in, int64_t ld_in,
                                                 const float* w, float* out, int64_t ld_out, const float* tree, int64_t ld_tree,
                                                 void* workspace, void* stream) {
    return conv333_forward_tc_impl(a, dl, cin, cout, slots, in, ld_in, w, out, ld_out, const_cast<float*>(tree), ld_tree, workspace, stream, true);
}

// Backward pass of the 3x3x3 convolution with the contractions on the tensor cores, from the packed
// bf16 rows of the input that the forward call left at the start of its workspace
// (aprnet_conv333_tc_packed_rows_bytes() bytes: particles, tree means, zero row; for Cin <= 4 the same
// area holds an fp32 channel-major copy instead, see conv333_small.cu): nothing of the fp32 input is needed.  grad_weights is accumulated into, grad_input (float32 (Cin, ld_in)) written; null: skipped.
//   packed dO rows -> weight gradient (tcgen05, deterministic) -> same-level input gradient (tcgen05 gather)
//   -> cross-level part (per-(target, tap) sums + gather over the targets) and tree adjoint.
// workspace: aprnet_conv333_tc_workspace_bytes() bytes (its leading part is not touched, so the forward
// workspace itself may be passed as packed_input_rows).
static int conv333_backward_tc_rows_impl(aprnet_apr* a, int dl, int cin, int cout, int slots, const void* packed_input_rows,
                                         const float* gout, int64_t ld_out, const float* w, float* gin, int64_t ld_in, float* gw,
                                         float* gtree, int64_t ld_tree, float* partial, void* workspace, void* stream, bool tree_adjoint) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && cin > 0 && cout > 0 && slots > 0 && packed_input_rows && gout && w && gw && gtree && partial && workspace, "bad argument");
    APRNET_ARG_CHECK(ld_out >= a->number_parts(dl) && (!gin || ld_in >= a->number_parts(dl)) && ld_tree >= a->tree_size(dl), "leading dimension too small");
    cudaStream_t st = (cudaStream_t) stream;
    const ll n = a->number_parts(dl), t = a->tree_size(dl);
    const int xpad = aprnet_tc_pad(cin), gpad = aprnet_tc_pad(cout);
    char* ws = (char*) workspace;
    void* grows = ws + aprnet_tc_rows_bytes(n + t + 1, cin);
    void* wp = (char*) grows + aprnet_tc_rows_bytes(n + 1, cout);
    int rc;
    if (!(aprnet_small_cin(cin) && !gin) && (rc = aprnet_tc_pack_rows(gout, ld_out, n, nullptr, 0, 0, cout, gpad, grows, st))) return rc;
    if (aprnet_small_cin(cin)) {
        if ((rc = aprnet_small_backward_weights(a, dl, cin, cout, slots, (const float*) packed_input_rows, gout, ld_out, gw, partial, st))) return rc;
    } else if ((rc = aprnet_conv333_backward_weights_tc(a, dl, cin, cout, slots, packed_input_rows, xpad, grows, gpad, gw, partial, st))) return rc;
    if (!gin) return APRNET_OK;          // the caller does not need the input gradient (first layer of a network)
    if ((rc = aprnet_tc_gather_conv(a, dl, 1, cin, cout, slots, grows, gpad, n, n, w, wp, gin, ld_in, st))) return rc;
    void* edge_ws = (char*) wp + aprnet_tc_weight_bytes(cout, cin, slots);
    if (27 * n + 1 >= (1ll << 31)) {
        // more than 79.5 M locations: the 32-bit edge ids of the edge plan run out.  The cross-level part then runs on the
        // fp32 scatter kernel (atomic adds: correct, but the summation order is no longer fixed).
        if (!tree_adjoint) { aprnet_set_error("the split backward form needs the edge plan, which supports up to 79.5 M locations"); return APRNET_ERR_UNSUPPORTED; }
        return aprnet_conv333_backward_input_cross_level(a, dl, APRNET_F32, cin, cout, slots, gout, ld_out, w, gin, ld_in, gtree, ld_tree, stream);
    }
    return aprnet_cross_level_tc(a, dl, cin, cout, slots, grows, gpad, w, gin, ld_in, gtree, ld_tree, wp, edge_ws,
                                 aprnet_edge_workspace_bytes(a, dl, cout), st, tree_adjoint);
}

extern "C" int aprnet_conv333_backward_tc_rows(aprnet_apr* a, int dl, int cin, int cout, int slots, const void* packed_input_rows,
                                               const float* gout, int64_t ld_out, const float* w, float* gin, int64_t ld_in, float* gw,
                                               float* gtree, int64_t ld_tree, float* partial, void* workspace, void* stream) {
    return conv333_backward_tc_rows_impl(a, dl, cin, cout, slots, packed_input_rows, gout, ld_out, w, gin, ld_in, gw, gtree, ld_tree, partial, workspace, stream, true);
}

// Split form: grad_input holds the direct contributions only and grad_tree the gradient of the tree means; the
// caller folds them with aprnet_fill_tree_mean_backward after it has exchanged the halo parts.
extern "C" int aprnet_conv333_backward_tc_rows_pretree(aprnet_apr* a, int dl, int cin, int cout, int slots, const void* packed_input_rows,
                                                       const float* gout, int64_t ld_out, const float* w, float* gin, int64_t ld_in, float* gw,
                                                       float* gtree, int64_t ld_tree, float* partial, void* workspace, void* stream) {
    return conv333_backward_tc_rows_impl(a, dl, cin, cout, slots, packed_input_rows, gout, ld_out, w, gin, ld_in, gw, gtree, ld_tree, partial, workspace, stream, false);
}

extern "C" int64_t aprnet_conv333_tc_packed_rows_bytes(const aprnet_apr* a, int dl, int cin) {
    if (!a || !a->valid_dl(dl)) return -1;
    return (int64_t) aprnet_tc_rows_bytes(a->number_parts(dl) + a->tree_size(dl) + 1, cin);
}

// Complete backward pass from the fp32 input: fills the tree means (unless tree_valid), packs the input
// rows into the workspace and continues as aprnet_conv333_backward_tc_rows.
extern "C" int aprnet_conv333_backward_tc(aprnet_apr* a, int dl, int cin, int cout, int slots, const float* in, int64_t ld_in,
                                          const float* gout, int64_t ld_out, const float* w, float* gin, float* gw,
                                          float* tree, int tree_valid, float* gtree, int64_t ld_tree, float* partial,
                                          void* workspace, void* stream) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && cin > 0 && cout > 0 && slots > 0 && in && gout && w && gw && tree && gtree && partial && workspace, "bad argument");
    APRNET_ARG_CHECK(ld_in >= a->number_parts(dl) && ld_out >= a->number_parts(dl) && ld_tree >= a->tree_size(dl), "leading dimension too small");
    cudaStream_t st = (cudaStream_t) stream;
    int rc = tree_valid ? APRNET_OK : aprnet_fill_tree_mean_forward(a, dl, APRNET_F32, cin, in, ld_in, tree, ld_tree, st);
    if (rc) return rc;
    const ll n = a->number_parts(dl), t = a->tree_size(dl);
    if (aprnet_small_cin(cin)) { if ((rc = aprnet_small_stage(in, ld_in, n, tree, ld_tree, t, cin, (float*) workspace, st))) return rc; }
    else if ((rc = aprnet_tc_pack_rows(in, ld_in, n, tree, ld_tree, t, cin, aprnet_tc_pad(cin), workspace, st))) return rc;
    return aprnet_conv333_backward_tc_rows(a, dl, cin, cout, slots, workspace, gout, ld_out, w, gin, ld_in, gw, gtree, ld_tree, partial, workspace, stream);
}
