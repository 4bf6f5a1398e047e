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
// global to shared memory with 16-byte cp.async copies, straight into the canonical K-major
// no-swizzle operand layout ([8-channel chunk][row][8 channels], 8 rows x 16 B core matrices).  Weights
// are packed once per call into the same canonical layout.  One elected thread issues tcgen05.mma;
// completion is tracked with mbarriers (tcgen05.commit); accumulators are read back with tcgen05.ld
// and written once, coalesced, to the fp32 (C, N) output.  Every wait is bounded: on expiry the block
// raises an error flag in host-mapped memory, drains its copies, frees its TMEM and returns.
//
// The same kernel computes the same-level part of the input gradient (input = dO, weights transposed
// and mirrored, neighbour entries masked to the location's own level).
#include "apr_device.cuh"
#include <cuda_bf16.h>
#include <algorithm>
#include <cstring>
#include <cstdlib>

namespace {

typedef long long ll;
constexpr int MAX_SEGS = APRNET_MAX_LEVELS;
constexpr int TILE_M = 128;
#ifndef APRNET_TC_STAGES
#define APRNET_TC_STAGES 6
#endif
#ifndef APRNET_TC_AHEAD
#define APRNET_TC_AHEAD 4
#endif
constexpr int STAGES = APRNET_TC_STAGES;            // shared-memory ring
constexpr int AHEAD = APRNET_TC_AHEAD;             // stages of copies in flight; the ring slot being refilled was read by the MMAs of two steps ago
constexpr unsigned SPIN_LIMIT = 1u << 22;

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

// ---- PTX wrappers ---------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
#ifdef APRNET_TC_DBG_NOLOAD
    return;
#endif
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
#ifdef APRNET_TC_TESTWAIT
                 "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
#else
                 "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
#endif
                 "selp.b32 %0, 1, 0, p;\n\t}\n" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// bounded wait; returns false when the limit expired
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
#ifdef APRNET_TC_DBG_NOMMA
    return true;
#endif
    for (unsigned it = 0; it < SPIN_LIMIT; ++it)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
// bulk (TMA, non-tensor) copy global -> shared of a contiguous 16-byte-aligned block; completion is
// signalled on an mbarrier as transferred bytes
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
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
// D[tmem] (+)= A[smem desc] * B[smem desc], bf16 x bf16 -> fp32
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

// Shared-memory matrix descriptor, K-major, no swizzle: 8-row x 16-byte core matrices; LBO = byte
// distance between the two 8-element K chunks of one MMA, SBO = byte distance between 8-row groups.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t) ((saddr >> 4) & 0x3FFF) | ((uint64_t) ((lbo >> 4) & 0x3FFF) << 16) |
           ((uint64_t) ((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46);
}
// K-major operand stored with a hardware swizzle: rows of 32/64/128 bytes, 8-row atoms `sbo` bytes apart;
// layout 2 = 128-byte, 4 = 64-byte, 6 = 32-byte swizzle.  The 16-byte chunk c of row r sits at chunk
// position c ^ f(r) (address bits [4,7) xor-ed with bits [7,10), restricted to the swizzle width).  A K
// step of 16 elements advances the start address by 32 bytes inside the atom.
__device__ __forceinline__ uint64_t make_desc_swizzled(uint32_t saddr, uint32_t sbo, uint32_t layout) {
    return (uint64_t) ((saddr >> 4) & 0x3FFF) | (1ull << 16) | ((uint64_t) ((sbo >> 4) & 0x3FFF) << 32) | (1ull << 46) |
           ((uint64_t) layout << 61);
}
template<int KS> __device__ __forceinline__ int swizzled_chunk(int row, int c) {
    return KS == 64 ? (c ^ (row & 7)) : (KS == 32 ? (c ^ ((row >> 1) & 3)) : (c ^ ((row >> 2) & 1)));
}
// Instruction descriptor: D fp32, A/B bf16, both K-major, M = 128, N = n
__host__ __device__ constexpr uint32_t make_idesc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t) (n >> 3) << 17) | ((uint32_t) (TILE_M >> 4) << 24);
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

// ---- main kernel -----------------------------------------------------------------------------------
struct EdgeGroupDev { ll begin, end; int tile_begin, tap, slot, pad; };   // edges [begin, end) share one tap and one stencil slot

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
    // edge mode (cross-level part of the input gradient): one tap per tile, source rows from an edge list,
    // result rows written channels-last as float [edge - edge_origin][row_pad]
    int edge_mode;
    const int32_t* edge_src;
    const EdgeGroupDev* groups; int n_groups;
    ll edge_origin;
    float* out_rows; int row_pad;
};

template<int NT, int KS>
__global__ void __launch_bounds__(TILE_M) conv333_tc_kernel(const TcParams P) {
    constexpr int A_BYTES = TILE_M * KS * 2;
    constexpr int B_BYTES = NT * KS * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t IDESC = make_idesc(NT);
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char* stage_base = smem;                                            // STAGES * STAGE_BYTES
    int32_t* idx_s = reinterpret_cast<int32_t*>(smem + STAGES * STAGE_BYTES);    // [27][128] source rows
    uint64_t* bars = reinterpret_cast<uint64_t*>(idx_s + 27 * TILE_M);           // STAGES (slot free) + 1 (tile done) + STAGES (weights landed)
    uint64_t* bfull = bars + STAGES + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bfull + STAGES);

    const int tid = threadIdx.x, warp = tid >> 5;
    const int kchunks = P.kpad / KS;

    if (tid == 0) {
        for (int i = 0; i <= 2 * STAGES; ++i) mbar_init(smem_u32(bars + i), 1);
        fence_mbar_init();
    }
    if (warp == 0) { tmem_alloc(smem_u32(tmem_slot), NT); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_slot;

    const int ntaps = P.edge_mode ? 1 : 27;
    const int steps_per_tile = ntaps * kchunks;
    const int total_tiles = (P.edge_mode ? P.groups[P.n_groups - 1].tile_begin +
                                               (int) ((P.groups[P.n_groups - 1].end - P.groups[P.n_groups - 1].begin + TILE_M - 1) / TILE_M)
                                         : P.segs.tile_begin[P.segs.n]) * P.n_tiles;
    uint32_t gstep = 0;           // stages issued so far by this block (selects buffer and mbarrier phase)
    uint32_t tiles_done = 0;
    uint32_t bulk_issued = 0;     // stages whose weight copy thread 0 has issued
    bool failed = false;

#ifdef APRNET_TC_DBG_TIMING
    long long tm[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long t0; int ntl = 0;
#define TM_START() t0 = clock64()
#define TM_ADD(i) tm[i] += clock64() - t0
#else
#define TM_START()
#define TM_ADD(i)
#endif
    for (int work = blockIdx.x; work < total_tiles; work += gridDim.x) {
        const int tile = work / P.n_tiles, ntile = work % P.n_tiles;
        TM_START();
        ll lo, hi, p;
        int slot, tap_base;
        if (P.edge_mode) {
            int g0 = 0, g1 = P.n_groups - 1;              // last group whose tile_begin <= tile
            while (g0 < g1) { const int m = (g0 + g1 + 1) >> 1; if (P.groups[m].tile_begin <= tile) g0 = m; else g1 = m - 1; }
            lo = P.groups[g0].begin; hi = P.groups[g0].end;
            p = lo + (ll) (tile - P.groups[g0].tile_begin) * TILE_M + tid;       // p is an edge id here
            slot = P.groups[g0].slot; tap_base = P.groups[g0].tap;
        } else {
            int seg = 0;
            while (seg + 1 < P.segs.n && tile >= P.segs.tile_begin[seg + 1]) ++seg;
            lo = P.segs.begin[seg]; hi = P.segs.end[seg];
            p = lo + (ll) (tile - P.segs.tile_begin[seg]) * TILE_M + tid;
            slot = P.segs.slot[seg]; tap_base = 0;
        }
        const bool valid = p < hi;
        const __nv_bfloat16* wtile = P.wp + ((ll) (slot * 27 + tap_base) * P.n_tiles + ntile) * ((ll) P.kpad * NT);
        const ll w_tap_stride = (ll) P.n_tiles * P.kpad * NT;

        // source row of every tap for this thread's output location.  The 27 table entries are fetched
        // as one batch of independent loads (a rolled loop with a dependent use per iteration would
        // pay 27 DRAM round trips per tile).
        if (P.edge_mode) {
            idx_s[tid] = valid ? P.edge_src[p] : (int32_t) P.zero_row;
        } else {
            int32_t q[27];
#pragma unroll
            for (int tap = 0; tap < 27; ++tap) q[tap] = valid ? __ldg(P.nbr + (ll) tap * P.N + p) : APRNET_NONE;
#pragma unroll
            for (int tap = 0; tap < 27; ++tap) {
                ll r = P.zero_row;
                if (P.same_level_only) { if (q[tap] >= lo && q[tap] < hi) r = q[tap]; }
                else if (q[tap] >= 0) r = q[tap];
                else if (q[tap] != APRNET_NONE) r = P.tree_base + aprnet_dec_tree(q[tap]);
                idx_s[tap * TILE_M + tid] = (int32_t) r;
            }
        }
        __syncthreads();          // source rows are read by other threads of the block
        TM_ADD(0);

        auto issue_loads = [&](int step) {
            const int tap = step / kchunks, kc = step % kchunks;
            const uint32_t buf = (gstep + (uint32_t) step) % STAGES;
            unsigned char* a_s = stage_base + buf * STAGE_BYTES;
            unsigned char* b_s = a_s + A_BYTES;
            // lanes sweep the 16-byte chunks of a row first, so one warp instruction reads whole rows
            // (contiguous 32/64-byte pieces) instead of 32 scattered sectors
            constexpr int CH = KS / 8, RPP = TILE_M / CH;
            const int j = tid % CH, r0 = tid / CH;
#pragma unroll
            for (int i = 0; i < CH; ++i) {
                const int row = i * RPP + r0;
                const __nv_bfloat16* src = P.rows + (ll) idx_s[tap * TILE_M + row] * P.kpad + kc * KS + j * 8;
                cp_async16(smem_u32(a_s + (j * TILE_M + row) * 16), src);
            }
            // weights of (tap, kc): chunks j in [kc*KS/8, (kc+1)*KS/8), each NT x 16 B, contiguous in global memory
            // one bulk copy by one thread (the packed block is contiguous in global memory)
            if (tid == 0) {
                const unsigned char* wsrc = reinterpret_cast<const unsigned char*>(wtile + (ll) tap * w_tap_stride + (ll) kc * KS * NT);
                mbar_expect_tx(smem_u32(bfull + buf), B_BYTES);
                bulk_copy_g2s(smem_u32(b_s), wsrc, B_BYTES, smem_u32(bfull + buf));
                bulk_issued = gstep + (uint32_t) step + 1;
            }
        };

        // prologue: fill AHEAD buffers (their previous readers, if any, must have finished)
        for (int s = 0; s < AHEAD; ++s) {
            if (s < steps_per_tile) {
                const uint32_t g = gstep + s;
                if (g >= STAGES) {
                    const uint32_t use = g / STAGES;
                    if (!mbar_wait(smem_u32(bars + g % STAGES), (use - 1) & 1)) failed = true;
                }
                issue_loads(s);
            }
            cp_async_commit();
        }

        for (int step = 0; step < steps_per_tile; ++step) {
            TM_START();
            cp_async_wait<AHEAD - 1>();
            TM_ADD(1); TM_START();           // this thread's copies of `step` have landed
            fence_proxy_async();                  // make them visible to the tensor-core (async) proxy
            if (__syncthreads_or(failed ? 1 : 0)) { failed = true; break; }     // uniform decision for the whole block
            const uint32_t g = gstep + step;
            TM_ADD(2); TM_START();
#ifndef APRNET_TC_DBG_NOMMA
            if (tid == 0) {
                if (!mbar_wait(smem_u32(bfull + g % STAGES), (g / STAGES) & 1)) failed = true;      // weights of this stage
                tc_fence_after();
                const uint32_t a_addr = smem_u32(stage_base + (g % STAGES) * STAGE_BYTES);
                const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                for (int k = 0; k < KS / 16; ++k) {
                    const uint64_t da = make_desc(a_addr + k * 2 * (TILE_M * 16), TILE_M * 16, 128);
                    const uint64_t db = make_desc(b_addr + k * 2 * (NT * 16), NT * 16, 128);
                    umma_bf16(tmem_d, da, db, IDESC, (step > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(smem_u32(bars + g % STAGES));
                if (step == steps_per_tile - 1) umma_commit(smem_u32(bars + STAGES));
            }
#endif
            TM_ADD(3); TM_START();
            // refill the ring slot last read by the MMAs issued STAGES - AHEAD steps ago
            const int nxt = step + AHEAD;
            if (nxt < steps_per_tile) {
                const uint32_t gn = gstep + nxt;
                if (gn >= STAGES) {
                    const uint32_t use = gn / STAGES;
                    if (!mbar_wait(smem_u32(bars + gn % STAGES), (use - 1) & 1)) failed = true;
                }
                TM_ADD(4); TM_START();
                if (!failed) issue_loads(nxt);
                TM_ADD(5); TM_START();
            }
            cp_async_commit();
        }
        gstep += steps_per_tile;
        if (__syncthreads_or(failed ? 1 : 0)) { failed = true; break; }

        // epilogue: accumulators -> registers -> global (coalesced along the particle axis)
        TM_START();
        {
            const bool ok = mbar_wait(smem_u32(bars + STAGES), tiles_done & 1);
            if (__syncthreads_or(ok ? 0 : 1)) { failed = true; break; }
        }
        ++tiles_done;
        TM_ADD(6); TM_START();
        tc_fence_after();
#pragma unroll
        for (int c0 = 0; c0 < NT; c0 += 32) {
            uint32_t r[32];
            tmem_ld32(tmem_d + ((uint32_t) (warp * 32) << 16) + c0, r);
            tmem_ld_wait();
            if (valid && P.edge_mode) {
                float4* dst = reinterpret_cast<float4*>(P.out_rows + (p - P.edge_origin) * P.row_pad + ntile * NT + c0);
#pragma unroll
                for (int j = 0; j < 32; j += 4)
                    if (ntile * NT + c0 + j < P.row_pad)
                        dst[j >> 2] = make_float4(__uint_as_float(r[j]), __uint_as_float(r[j + 1]), __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            } else if (valid) {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int n = ntile * NT + c0 + j;
                    if (n < P.n_dim) P.out[(ll) n * P.ld_out + p] = __uint_as_float(r[j]);
                }
            }
        }
        tc_fence_before();
        __syncthreads();          // all TMEM reads done before the next tile's first MMA overwrites D
        TM_ADD(7);
#ifdef APRNET_TC_DBG_TIMING
        ++ntl;
#endif
    }
#ifdef APRNET_TC_DBG_TIMING
    if (blockIdx.x == 7 && (tid == 0 || tid == 77)) printf("tid %d tiles %d steps/tile %d | idx %lld | cpwait %lld | fence+bar %lld | mma %lld | mbarwait %lld | issue %lld | epi-wait %lld | epi %lld (cycles per tile)\n", tid, ntl, steps_per_tile, tm[0]/ntl, tm[1]/ntl, tm[2]/ntl, tm[3]/ntl, tm[4]/ntl, tm[5]/ntl, tm[6]/ntl, tm[7]/ntl);
#endif

    // teardown (also the error path): drain copies, release TMEM
    cp_async_wait<0>();
    if (failed && tid == 0) {      // bulk copies still in flight must land before the block's shared memory is released
        for (uint32_t g = bulk_issued > STAGES ? bulk_issued - STAGES : 0; g < bulk_issued; ++g)
            mbar_wait(smem_u32(bfull + g % STAGES), (g / STAGES) & 1);
    }
    if (failed && P.error_flag) *P.error_flag = 1;
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_d, NT);
}

// ---- warp-specialised gather kernel ---------------------------------------------------------------
// One persistent block per SM, 14 warps (forward pass and same-level input gradient):
//   warps 0-7   producers.  A stage (one tap, KS channels, 128 rows) belongs to ONE warp: warp w fills the
//               stages w, w + 8, w + 16 ... of the block's stage sequence, so eight stages are being issued
//               at once and the per-stage bookkeeping (slot wait, weight copy, barrier arrival) is paid
//               once per 4 * KS / 8 copy instructions.  Lane 0 streams the stage's weight tile with one bulk
//               copy (byte-counting arrival); every lane attaches an asynchronous arrival to the stage's
//               barrier (cp.async.mbarrier.arrive.noinc), so the stage is handed to the MMA warp the moment
//               its copies land.  Producers only block on a ring slot the tensor core still reads;
//   warp 8      one thread issues the tcgen05.mma of each stage, in stage order, as soon as its barrier
//               completes, and commits the stage's "slot free" barrier; accumulators rotate through
//               NACC TMEM buffers so that later tiles start while earlier ones are read back;
//   warps 10-13 epilogue: TMEM -> registers -> global for tile i; the neighbour-table entries of tile
//               i + NIDX are requested into registers before the wait for tile i and decoded into the
//               source-row buffer tile i has released afterwards, so their DRAM latency is never exposed.
// All waits are bounded and poll a block-wide abort flag.
constexpr int WS_NPROD = 8;
constexpr int WS_THREADS = (WS_NPROD + 6) * 32;
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

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool ws_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (unsigned it = 0; it < SPIN_LIMIT; ++it) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 63) == 63 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}
// one lane polls, the warp follows
__device__ __forceinline__ bool warp_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    int ok = 1;
    if ((threadIdx.x & 31) == 0) ok = ws_wait(bar, parity, abort_flag) ? 1 : 0;
    ok = __shfl_sync(0xffffffffu, ok, 0);
    return ok != 0;
}
// arrival on an mbarrier that is triggered when all earlier cp.async copies of this thread have completed
// (counts as one of the barrier's expected arrivals)
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];\n" ::"r"(bar) : "memory");
}

template<int NT, int KS, int NACC>
__global__ void __launch_bounds__(WS_THREADS, 1) conv333_tc_ws_kernel(const TcParams P, const int stages) {
    // A operand: K-major with the hardware swizzle whose width equals the row piece of one stage (KS
    // channels = 32, 64 or 128 bytes).  A gathered row piece is then contiguous in shared memory as it is
    // in global memory (its 16-byte chunks permuted inside the piece), so the lanes that copy one piece
    // write one contiguous block; with the unswizzled layout every 16-byte chunk of a row goes to a
    // different plane and each 32-byte sector costs its own pass of the shared-memory write pipe.
    constexpr int NIDX = WS_NIDX;
    constexpr int CH = KS / 8;                               // 16-byte chunks per gathered row piece
    constexpr int RW = 32 / CH;                              // rows covered by one copy instruction of a warp
    constexpr int NI = TILE_M / RW;                          // copy instructions per stage
    constexpr int ROW_BYTES = KS * 2;
    constexpr uint32_t A_LAYOUT = KS == 64 ? 2u : (KS == 32 ? 4u : 6u);     // SWIZZLE_128B / 64B / 32B
    constexpr int A_BYTES = TILE_M * ROW_BYTES;
    constexpr int B_BYTES = NT * KS * 2;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr uint32_t IDESC = make_idesc(NT);
    extern __shared__ __align__(128) unsigned char smem_raw[];
    // swizzle atoms (8 rows) must start on a multiple of their size: align the ring to 1024 bytes
    unsigned char* smem = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
    unsigned char* stage_base = smem;
    int32_t* idx_s = reinterpret_cast<int32_t*>(smem + (size_t) stages * STAGE_BYTES);      // NIDX x [27][128] source rows
    uint64_t* bars = reinterpret_cast<uint64_t*>(idx_s + NIDX * 27 * TILE_M);
    uint64_t* full = bars;                          // [stages]  copies of the stage landed (32 lanes + weight bytes)
    uint64_t* empty = bars + WS_MAX_STAGES;         // [stages]  MMAs that read the stage completed
    uint64_t* tmem_full = empty + WS_MAX_STAGES;    // [NACC]    accumulator complete
    uint64_t* tmem_empty = tmem_full + WS_MAX_ACC;  // [NACC]    accumulator read back (one arrival per epilogue warp)
    uint64_t* idx_full = tmem_empty + WS_MAX_ACC;   // [NIDX]    source rows of a tile written (one arrival per epilogue warp)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(idx_full + WS_MAX_ACC);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kchunks = P.kpad / KS;
    const int steps_per_tile = 27 * kchunks;
    const int total_tiles = P.segs.tile_begin[P.segs.n] * P.n_tiles;
    const int my_tiles = (int) blockIdx.x < total_tiles ? (total_tiles - (int) blockIdx.x + (int) gridDim.x - 1) / (int) gridDim.x : 0;
    const int nprod = min(WS_NPROD, stages);

    if (tid == 0) {
        for (int i = 0; i < stages; ++i) { mbar_init(smem_u32(full + i), 32 + 1); mbar_init(smem_u32(empty + i), 1); }
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
#ifdef APRNET_TC_DBG_TIMING
    long long wt[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long w0 = clock64(); const long long wstart = w0;
#define WT(i) { const long long w1 = clock64(); wt[i] += w1 - w0; w0 = w1; }
#else
#define WT(i)
#endif

    if (warp < WS_NPROD) {
        // ---------------- producers ----------------
        if (warp < nprod) {
            const int j = lane % CH, r0 = lane / CH;
            const uint32_t total_stages = (uint32_t) my_tiles * (uint32_t) steps_per_tile;
            uint32_t g = warp, slot = warp, use = 0;       // nprod <= stages: the first stage of every warp has its own slot
            int it = 0, step = warp, cur_it = -1;
            const int32_t* idx = idx_s;
            const unsigned char* wsrc = nullptr;
            const ll w_tap_stride = (ll) P.n_tiles * P.kpad * NT * 2;
            while (g < total_stages) {
                while (step >= steps_per_tile) { step -= steps_per_tile; ++it; }
                if (it != cur_it) {
                    cur_it = it;
                    WT(7);
                    if (!warp_wait(smem_u32(idx_full + it % NIDX), (it / NIDX) & 1, abort_flag)) { failed = true; break; }
                    WT(0);
                    idx = idx_s + (it % NIDX) * 27 * TILE_M;
                    if (lane == 0) {      // packed weights of one (slot, tap, n tile) are [k chunk][n][8]; a stage takes KS / 8 chunks
                        const TileInfo ti = tile_info(P, blockIdx.x + it * gridDim.x);
                        wsrc = reinterpret_cast<const unsigned char*>(P.wp + ((ll) ti.slot * 27 * P.n_tiles + ti.ntile) * ((ll) P.kpad * NT));
                    }
                }
                const int tap = step / kchunks, kc = step - tap * kchunks;
                if (use > 0 && !warp_wait(smem_u32(empty + slot), (use - 1) & 1, abort_flag)) { failed = true; break; }
                WT(1);
                unsigned char* a_s = stage_base + (size_t) slot * STAGE_BYTES;
                if (lane == 0) {
                    mbar_expect_tx(smem_u32(full + slot), B_BYTES);
                    bulk_copy_g2s(smem_u32(a_s + A_BYTES), wsrc + (ll) tap * w_tap_stride + (ll) kc * KS * NT * 2, B_BYTES, smem_u32(full + slot));
                    bulk_issued = true;
                }
                const int32_t* idx_t = idx + tap * TILE_M + r0;
                const __nv_bfloat16* src0 = P.rows + kc * KS + j * 8;
#pragma unroll
                for (int i = 0; i < NI; ++i) {
                    const int row = i * RW + r0;
                    cp_async16(smem_u32(a_s + row * ROW_BYTES + (swizzled_chunk<KS>(row, j) << 4)), src0 + (ll) idx_t[i * RW] * P.kpad);
                }
                WT(2);
                // the stage's barrier receives this thread's arrival when the copies above have landed
                cp_async_arrive_noinc(smem_u32(full + slot));
                WT(3);
                g += nprod; step += nprod; slot += nprod;
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
                if (acc_use > 0 && !ws_wait(smem_u32(tmem_empty + acc), (acc_use - 1) & 1, abort_flag)) { failed = true; break; }
                tc_fence_after();
                WT(0);
                for (int step = 0; step < steps_per_tile; ++step) {
                    if (!ws_wait(smem_u32(full + slot), use & 1, abort_flag)) { failed = true; break; }
                    WT(1);
                    fence_proxy_async();          // generic-proxy writes of the cp.async copies -> tensor-core (async proxy) reads
                    tc_fence_after();
                    const uint32_t a_addr = smem_u32(stage_base + (size_t) slot * STAGE_BYTES);
                    const uint32_t b_addr = a_addr + A_BYTES;
#pragma unroll
                    for (int k = 0; k < KS / 16; ++k) {
                        const uint64_t da = make_desc_swizzled(a_addr + k * 32, 8 * ROW_BYTES, A_LAYOUT);
                        const uint64_t db = make_desc(b_addr + k * 2 * (NT * 16), NT * 16, 128);
                        umma_bf16(tmem_d + acc * NT, da, db, IDESC, (step > 0 || k > 0) ? 1u : 0u);
                    }
                    WT(2);
                    umma_commit(smem_u32(empty + slot));
                    WT(3);
                    if (++slot == (uint32_t) stages) { slot = 0; ++use; }
                }
                if (!failed) umma_commit(smem_u32(tmem_full + acc));
            }
        }
    } else if (warp >= WS_NPROD + 2) {
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
            WT(7);
            const TileInfo ti = tile_info(P, blockIdx.x + it * gridDim.x);
            const ll p = ti.p0 + row;
            const bool valid = p < ti.hi;
            const uint32_t acc = (uint32_t) it % NACC, acc_use = (uint32_t) it / NACC;
            request_idx(it + NIDX);       // lands while this warp waits for the accumulator
            WT(2);
            if (!warp_wait(smem_u32(tmem_full + acc), acc_use & 1, abort_flag)) { failed = true; break; }
            WT(0);
            tc_fence_after();
#pragma unroll
            for (int c0 = 0; c0 < NT; c0 += 32) {
                uint32_t r[32];
                tmem_ld32(tmem_d + ((uint32_t) (q * 32) << 16) + acc * NT + c0, r);
                tmem_ld_wait();
                if (valid) {
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj) {
                        const int n = ti.ntile * NT + c0 + jj;
                        if (n < P.n_dim) P.out[(ll) n * P.ld_out + p] = __uint_as_float(r[jj]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(tmem_empty + acc));
            WT(1);
            // every copy that read the source rows of tile `it` has landed (its accumulator is complete)
            publish_idx(it + NIDX);
            WT(3);
        }
    }

#ifdef APRNET_TC_DBG_TIMING
    if (blockIdx.x == 7 && (tid == 0 || tid == 32 * WS_NPROD || tid == 32 * (WS_NPROD + 2))) {
        const long long tot = clock64() - wstart;
        printf("ws tid %d total %lld | %lld %lld %lld %lld %lld %lld %lld %lld | stages %d nacc %d tiles %d steps/tile %d\n", tid, tot, wt[0], wt[1], wt[2], wt[3], wt[4], wt[5], wt[6], wt[7], stages, NACC, my_tiles, steps_per_tile);
    }
#endif
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

__global__ void set_group_tile_begin_kernel(EdgeGroupDev* g, int n, int tile) {
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        int acc = 0;
        for (int i = 0; i < n; ++i) { g[i].tile_begin = acc; acc += (int) ((g[i].end - g[i].begin + tile - 1) / tile); }
    }
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

TcGeom tc_geometry(ll rows, int k_dim, int n_dim, int slots) {
    TcGeom g;
    g.kpad = pad_to(k_dim, 16);
    g.nt = pick_nt(n_dim);
    g.ks = (g.kpad % 64 == 0 && g.nt <= 128) ? 64 : ((g.kpad % 32 == 0) ? 32 : 16);
    g.n_tiles = (n_dim + g.nt - 1) / g.nt;
    g.rows_bytes = ((size_t) rows * g.kpad * 2 + 255) / 256 * 256;
    g.w_bytes = ((size_t) slots * 27 * g.n_tiles * g.kpad * g.nt * 2 + 255) / 256 * 256;
    return g;
}

template<int NT, int KS>
int launch_tc(const TcParams& P, int total_tiles, cudaStream_t st, const char* pname) {
    const size_t smem = (size_t) STAGES * (TILE_M * KS * 2 + NT * KS * 2) + 27 * TILE_M * 4 + (2 * STAGES + 1) * 8 + 16;
    auto kern = conv333_tc_kernel<NT, KS>;
    APRNET_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int per_sm = std::max(1, std::min(std::min(4, 512 / NT), (int) (225 * 1024 / (smem + 1024))));
    // tuning knobs (environment): blocks per SM and the shared-memory carve-out in percent; the part of the
    // 256 KB array that is not carved out for shared memory serves as L1 for the cp.async.ca gathers
    if (const char* e = getenv("APRNET_TC_BLOCKS_PER_SM")) per_sm = std::max(1, std::min(per_sm, atoi(e)));
    int carve = -1;
    if (const char* e = getenv("APRNET_TC_CARVEOUT")) carve = atoi(e);
    if (carve >= 0) APRNET_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, carve));
    const int grid = std::min(total_tiles, sms * per_sm);
    { AprnetProfScope _prof(pname, st);
    kern<<<grid, TILE_M, smem, st>>>(P);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

template<int NT, int KS>
int launch_tc_ws(const TcParams& P, int total_tiles, cudaStream_t st, const char* pname) {
    constexpr size_t STAGE = (size_t) TILE_M * KS * 2 + (size_t) NT * KS * 2;
    constexpr size_t FIXED = (size_t) WS_NIDX * 27 * TILE_M * 4 + (2 * WS_MAX_STAGES + 3 * WS_MAX_ACC) * 8 + 16 + 1024;      // + alignment slack
    constexpr int NACC = NT <= 128 ? 4 : 2;          // accumulators in flight: the SM's 512 TMEM columns, at most 4
    auto kern = conv333_tc_ws_kernel<NT, KS, NACC>;
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    // one block per SM with all of its shared memory (227 KB, 1 KB reserved) as the stage ring
    int stages = (int) std::min<size_t>(WS_MAX_STAGES, (227 * 1024 - 1024 - FIXED) / STAGE);
    if (const char* e = getenv("APRNET_TC_WS_STAGES")) stages = std::max(2, std::min(stages, atoi(e)));
    if (stages < 2) { aprnet_set_error("conv333 tensor-core path: tile nt=%d ks=%d does not fit shared memory", NT, KS); return APRNET_ERR_UNSUPPORTED; }
    const size_t smem = (size_t) stages * STAGE + FIXED;
    APRNET_CUDA_CHECK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
    const int grid = std::min(total_tiles, sms);
    { AprnetProfScope _prof(pname, st);
    kern<<<grid, WS_THREADS, smem, st>>>(P, stages);
    }
    APRNET_LAUNCH_CHECK();
    return APRNET_OK;
}

int dispatch_tc(const TcParams& P, const TcGeom& g, int total_tiles, cudaStream_t st, const char* pname) {
    static const bool legacy = getenv("APRNET_TC_LEGACY") != nullptr;
    if (legacy || P.edge_mode) {          // the edge-list GEMM (one or a few stages per tile) stays on the block-synchronous kernel
        const int ks = std::min(g.ks, 32);
#define TC_CASE(NT_, KS_) if (g.nt == NT_ && ks == KS_) return launch_tc<NT_, KS_>(P, total_tiles, st, pname);
        TC_CASE(32, 16) TC_CASE(32, 32) TC_CASE(64, 16) TC_CASE(64, 32) TC_CASE(128, 16) TC_CASE(128, 32) TC_CASE(256, 16) TC_CASE(256, 32)
#undef TC_CASE
    } else {
#define TC_CASE(NT_, KS_) if (g.nt == NT_ && g.ks == KS_) return launch_tc_ws<NT_, KS_>(P, total_tiles, st, pname);
        TC_CASE(32, 16) TC_CASE(32, 32) TC_CASE(32, 64) TC_CASE(64, 16) TC_CASE(64, 32) TC_CASE(64, 64)
        TC_CASE(128, 16) TC_CASE(128, 32) TC_CASE(128, 64) TC_CASE(256, 16) TC_CASE(256, 32)
#undef TC_CASE
    }
    aprnet_set_error("conv333 tensor-core path: unsupported tile geometry nt=%d ks=%d", g.nt, g.ks);
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
    P.edge_mode = 0; P.edge_src = nullptr; P.groups = nullptr; P.n_groups = 0; P.edge_origin = 0; P.out_rows = nullptr; P.row_pad = 0;

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

// Edge-list GEMM for the groups [g0, g1) of an edge plan (weights already packed with mode 2).
int aprnet_tc_edge_gemm(aprnet_apr* a, int dl, int cin, int cout, int slots, const void* grows, int gpad, ll zero_row,
                        const void* wp_packed, EdgePlan* ep, int g0, int g1, float* rows_out, int row_pad, cudaStream_t st) {
    int rc = ensure_error_flag();
    if (rc) return rc;
    if (*g_error_flag_host) { aprnet_set_error("a previous tensor-core kernel gave up waiting on a barrier"); return APRNET_ERR_CUDA; }
    const TcGeom g = tc_geometry(1, cout, cin, slots);
    if (g.kpad != gpad) { aprnet_set_error("packed row width %d does not match the padded channel count %d", gpad, g.kpad); return APRNET_ERR_ARG; }
    // device tile table: one entry per group with the stencil slot of its level (depends on `slots`)
    const int cml = a->cml(dl);
    if (ep->groups_slots != slots) {
        std::vector<EdgeGroupDev> tab(ep->groups.size());
        for (size_t i = 0; i < tab.size(); ++i) {
            tab[i].begin = ep->groups[i].begin; tab[i].end = ep->groups[i].end; tab[i].tap = ep->groups[i].tap;
            tab[i].slot = std::min(cml - ep->groups[i].level, slots - 1); tab[i].tile_begin = 0; tab[i].pad = 0;
        }
        if (!ep->groups_dev) APRNET_CUDA_CHECK(cudaMalloc(&ep->groups_dev, std::max<size_t>(1, tab.size()) * sizeof(EdgeGroupDev)));
        APRNET_CUDA_CHECK(cudaMemcpyAsync(ep->groups_dev, tab.data(), tab.size() * sizeof(EdgeGroupDev), cudaMemcpyHostToDevice, st));
        APRNET_CUDA_CHECK(cudaStreamSynchronize(st));       // `tab` is a stack object; one-time per (plan, slot count)
        ep->groups_slots = slots;
    }
    if (g1 <= g0) return APRNET_OK;
    TcParams P;
    memset(&P, 0, sizeof(P));
    P.rows = reinterpret_cast<const __nv_bfloat16*>(grows); P.kpad = g.kpad; P.zero_row = zero_row; P.tree_base = zero_row;
    P.wp = reinterpret_cast<const __nv_bfloat16*>(wp_packed); P.n_dim = cin; P.n_tiles = g.n_tiles;
    P.error_flag = g_error_flag_dev;
    P.edge_mode = 1; P.edge_src = ep->src; P.edge_origin = ep->groups[g0].begin; P.out_rows = rows_out; P.row_pad = row_pad;
    // tile_begin is relative to the launch: computed in a tiny kernel-free way by launching per chunk with a
    // host-built prefix: the table on the device holds absolute groups, so pass the sub-range and rebase.
    P.groups = reinterpret_cast<const EdgeGroupDev*>(ep->groups_dev) + g0; P.n_groups = g1 - g0;
    int total = 0;
    std::vector<int> tile_begin(g1 - g0);
    for (int i = g0; i < g1; ++i) { tile_begin[i - g0] = total; total += aprnet_ceil_div(ep->groups[i].end - ep->groups[i].begin, TILE_M); }
    set_group_tile_begin_kernel<<<aprnet_ceil_div(g1 - g0, 128), 128, 0, st>>>(
        reinterpret_cast<EdgeGroupDev*>(ep->groups_dev) + g0, g1 - g0, TILE_M);
    APRNET_LAUNCH_CHECK();
    total *= g.n_tiles;
    if (total == 0) return APRNET_OK;
    char pname[64];
    snprintf(pname, sizeof(pname), "conv333_tc_edge:ci%d:co%d:dl%d", cin, cout, dl);
    return dispatch_tc(P, g, total, st, pname);
}

size_t aprnet_tc_rows_bytes(ll rows, int channels) { return tc_geometry(rows, channels, 16, 1).rows_bytes; }
size_t aprnet_tc_weight_bytes(int k_dim, int n_dim, int slots) { return tc_geometry(1, k_dim, n_dim, slots).w_bytes; }
int aprnet_tc_pad(int channels) { return pad_to(channels, 16); }

extern "C" int aprnet_tc_error_flag(void) { return g_error_flag_host ? *g_error_flag_host : 0; }

extern "C" int64_t aprnet_conv333_tc_workspace_bytes(const aprnet_apr* a, int dl, int cin, int cout, int slots) {
    if (!a || !a->valid_dl(dl)) return -1;
    const ll n = a->number_parts(dl), t = a->tree_size(dl);
    // forward: packed input rows + packed weights.  backward: packed input rows, packed dO rows,
    // packed (transposed) weights.  One size serves both calls.
    const size_t fwd = aprnet_tc_rows_bytes(n + t + 1, cin) + aprnet_tc_weight_bytes(cin, cout, slots);
    const size_t bwd = aprnet_tc_rows_bytes(n + t + 1, cin) + aprnet_tc_rows_bytes(n + 1, cout) + aprnet_tc_weight_bytes(cout, cin, slots) +
                       (size_t) aprnet_edge_workspace_bytes(a, dl, cin);
    return (int64_t) std::max(fwd, bwd);
}

extern "C" int64_t aprnet_conv333_tc_forward_workspace_bytes(const aprnet_apr* a, int dl, int cin, int cout, int slots) {
    if (!a || !a->valid_dl(dl)) return -1;
    return (int64_t) (aprnet_tc_rows_bytes(a->number_parts(dl) + a->tree_size(dl) + 1, cin) + aprnet_tc_weight_bytes(cin, cout, slots));
}

// forward: out = conv(in) with bf16 operands / fp32 accumulation; tree_scratch receives the fp32 tree means
extern "C" int aprnet_conv333_forward_tc(aprnet_apr* a, int dl, int cin, int cout, int slots, const float* in, int64_t ld_in,
                                         const float* w, float* out, int64_t ld_out, float* tree, int64_t ld_tree,
                                         void* workspace, void* stream) {
    APRNET_ARG_CHECK(a && a->valid_dl(dl) && cin > 0 && cout > 0 && slots > 0 && in && w && out && tree && workspace, "bad argument");
    APRNET_ARG_CHECK(ld_in >= a->number_parts(dl) && ld_out >= a->number_parts(dl) && ld_tree >= a->tree_size(dl), "leading dimension too small");
    cudaStream_t st = (cudaStream_t) stream;
    int rc = aprnet_fill_tree_mean_forward(a, dl, APRNET_F32, cin, in, ld_in, tree, ld_tree, st);
    if (rc) return rc;
    const ll n = a->number_parts(dl), t = a->tree_size(dl);
    const int kpad = aprnet_tc_pad(cin);
    char* ws = (char*) workspace;
    void* rows = ws;
    void* wp = ws + aprnet_tc_rows_bytes(n + t + 1, cin);
    rc = aprnet_tc_pack_rows(in, ld_in, n, tree, ld_tree, t, cin, kpad, rows, st);
    if (rc) return rc;
    return aprnet_tc_gather_conv(a, dl, 0, cin, cout, slots, rows, kpad, n, n + t, w, wp, out, ld_out, st);
}

// Complete backward pass of the 3x3x3 convolution with the contractions on the tensor cores:
// grad_weights (accumulated into), grad_input (written; float32 (Cin, ld_in); may be null: skipped).
//   tree means -> packed input rows, packed dO rows -> weight gradient (tcgen05, deterministic)
//   -> same-level input gradient (tcgen05 gather) -> cross-level part (atomicAdd) + tree adjoint.
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
    const int xpad = aprnet_tc_pad(cin), gpad = aprnet_tc_pad(cout);
    char* ws = (char*) workspace;
    void* xrows = ws;
    void* grows = ws + aprnet_tc_rows_bytes(n + t + 1, cin);
    void* wp = (char*) grows + aprnet_tc_rows_bytes(n + 1, cout);
    if ((rc = aprnet_tc_pack_rows(in, ld_in, n, tree, ld_tree, t, cin, xpad, xrows, st))) return rc;
    if ((rc = aprnet_tc_pack_rows(gout, ld_out, n, nullptr, 0, 0, cout, gpad, grows, st))) return rc;
    if ((rc = aprnet_conv333_backward_weights_tc(a, dl, cin, cout, slots, xrows, xpad, grows, gpad, gw, partial, st))) return rc;
    if (!gin) return APRNET_OK;          // the caller does not need the input gradient (first layer of a network)
    if ((rc = aprnet_tc_gather_conv(a, dl, 1, cin, cout, slots, grows, gpad, n, n, w, wp, gin, ld_in, st))) return rc;
    void* edge_ws = (char*) wp + aprnet_tc_weight_bytes(cout, cin, slots);
    return aprnet_conv333_backward_input_cross_level_tc(a, dl, cin, cout, slots, grows, gpad, w, gin, ld_in, gtree, ld_tree, wp, edge_ws,
                                                        aprnet_edge_workspace_bytes(a, dl, cin), st);
}
