// The Shfl-BW panel kernel for sm_100a (persistent, warp-specialised).
//
// Work item = ONE row block of V stored rows x ONE tile of T = 128*TM dense columns
// ("tokens": SpMM columns of B, or SpConv output positions).  For an item the kernel
// computes the dense contraction
//
//     acc[token][m] = sum_p  G[p][token] * W[p][m]          p over the block's non-zero columns
//
// on the 5th-generation tensor cores, K = 16 per instruction, both operands MN-major in shared
// memory: W[p][0..V) is a contiguous slice of the value panels, G[p][..] is row indices[p] of
// the dense operand, gathered from L2.  Two orientations exist (template parameter MODE):
//   tokens in lanes  tokens are the UMMA M dimension (128 TMEM lanes), the V rows of the block
//                    the N dimension (32/64/128): TM instructions per 16 columns.  Used for
//                    V = 32, for SpConv writing NHWC, and for blocks with few columns.
//   rows in lanes    the V rows are M (64 or 128 lanes; M = 64 occupies the first 16 lanes of
//                    every 32-lane quadrant) and the T tokens N (128 or 256): ONE instruction
//                    per 16 columns.  An MMA costs >= 73 clk whatever its N up to 128 and 133
//                    clk at N = 256, so this halves the instruction count at ~8 % less tensor
//                    time, and the accumulator holds one output row per lane.  Default for
//                    SpMM and chained SpConv with V = 64 / 128 and >= 3 stages of columns.
// The description below is written for the first orientation; the second differs in the
// gathered tile's layout ([K group][T/64 swizzle atoms]), the MMA issue and the epilogue.
//
// One CTA per SM loops over items (item = blockIdx.x + i*gridDim.x, decoded block-major or
// tile-major, PanelParams::tile_major); their extents are read once into a shared-memory table.
// Warp roles (warp w issues from scheduler partition w % 4; EW = 8 or 16 epilogue warps):
//   warps 0..EW-1    epilogue.  Warp w reads TMEM lane quadrant w % 4 and part w / 4 of the
//                    accumulator columns.  Tokens in lanes: TMEM -> registers -> fp16 -> transpose
//                    of 32-row chunks through shared memory -> 16-byte global stores (inverse row
//                    permutation fused for SpMM).  Rows in lanes: stores straight from registers.
//   warp  EW         allocates TMEM; its lane 0 issues tcgen05.mma, releases stages and
//                    accumulators with tcgen05.commit
//   warps EW+1.. with w % 4 != 0   producers (PW of them, in GROUPS groups that take the stages in
//                    turn).  cp.async gather: 16-byte copies into 128-byte-swizzled stages; a
//                    group publishes its previous stage half-way through issuing the next one,
//                    with ONE mbarrier arrival per warp; row ids are prefetched LAG+1 of the
//                    group's stages ahead by 4-byte cp.async into a shared-memory ring.  TMA
//                    gather: one tile::gather4 per lane, completion by byte count.  One bulk copy
//                    per stage for the value slice either way.
//   later warps with w % 4 == 0   idle, so that no producer shares the MMA warp's scheduler partition.
// The accumulator is double buffered in TMEM (four sets with EW = 16) so the epilogue of item i
// overlaps the main loop of item i+1, and the stage ring runs across item boundaries without
// draining.
//
// Every mbarrier wait is bounded (sm100_ptx.cuh): on a timeout the kernel records a code in
// the status word, raises a CTA-wide abort flag, drains and exits; it cannot hang the GPU.
//
// Replaces SpmmBlockwiseKernel::mainLoop / epilogue (block_sparse/spmm/blockwise_kernel.h:99-294,
// block_sparse/common/epilogue.h:6-135) and SpconvBlockwiseKernel::mainLoop
// (block_sparse/spconv/blockwise_kernel.h:63-261, block_sparse/spconv/conv_format.h:14-82).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "shflbw.h"
#include "sm100_ptx.cuh"

namespace shflbw {

constexpr long long kWaitLimitCycles = 400000000LL;   // default bound of every in-kernel wait: ~0.2 s at 2 GHz

// Division of a non-negative int below 2^31 by a divisor fixed per launch: the quotient is
// umulhi(n, mul) >> shr with mul = ceil(2^(31 + ceil(log2 d)) / d), shr = ceil(log2 d) - 1
// (d == 1: the number itself).  Four instructions instead of the ~25 of a 32-bit division in
// software; the epilogues of shallow items are instruction-bound and divide three times per item.
struct FastDiv {
    unsigned d, mul, shr;
};
inline FastDiv make_fast_div(int d) {
    FastDiv f{(unsigned)d, 0u, 0u};
    if (d > 1) {
        unsigned c = 0;
        while ((1ull << c) < (unsigned long long)d) ++c;         // ceil(log2 d)
        const unsigned p = 31 + c;
        f.mul = (unsigned)(((1ull << p) + (unsigned long long)d - 1) / (unsigned long long)d);
        f.shr = p - 32;
    }
    return f;
}
__device__ __forceinline__ int fast_div(int n, const FastDiv& f) {
    return f.d == 1u ? n : (int)(__umulhi((unsigned)n, f.mul) >> f.shr);
}

struct alignas(64) PanelParams {
    // TMA gather only: tensor map of B ([K][N] fp16, box = 64 tokens x 1 row, 128-byte swizzle); first
    // member so that it sits on the 64-byte boundary the copy engine wants
    unsigned long long tmap_b[16];
    // sparse operand (kernel image)
    const int* blk_ptr;      // [X+1] padded offsets (multiples of 16)
    const int* blk_idx;      // padded column ids
    const __half* blk_val;   // value panels of the padded rows, element order kval_index() (shflbw_internal.hpp)
    const int* perm;         // [M] or nullptr
    int* status_word;
    unsigned idx_limit;      // largest legal gather offset: K - 1 (SpMM, a row id) or the element offset of the last
                             // (channel, tap) plane origin (SpConv); ids are clamped to it, so a corrupted id can
                             // give wrong numbers but never an address outside the dense operand
    long long wait_limit;    // SM clocks after which a barrier wait gives up (kWaitLimitCycles unless the host overrides it)
    float alpha, beta;
    int num_items, tiles_n;  // work items = row blocks x token tiles; item -> (item / tiles_n, item % tiles_n)
    FastDiv div_tiles, div_bp, div_wo;   // division by tiles_n, Bp, Wo (set by the host with make_fast_div)
    // Order of the work items.  0: item = block * tiles_n + tile (a CTA's neighbours work on the
    // same row block).  1: item = tile * num_blocks + block: the CTAs that run at the same time
    // share a few token tiles, so the rows of the dense operand they gather are a small set that
    // stays in L2 (SpMM with a large dense operand).
    int tile_major, num_blocks;
    FastDiv div_blocks;
    unsigned long long* trace;  // tuning builds only: per-role timestamps of CTA 0
    int inject_from;         // fault-injection builds only (-DSHFLBW_FAULT_INJECT): from this stage number on, one
                             // producer warp withholds its arrivals, so the consumer's bounded wait runs out (< 0: off)
    int ablate;              // tuning builds only (-DSHFLBW_ABLATE): 1 no MMA, 2 no gather, 4 no value copies, 8 no stores
    // SpMM
    const __half* B;         // [K][N]
    const __half* C;         // [M][N] or nullptr
    __half* D;               // [M][N]
    int N;                   // dense columns (SpMM) / Ho*Wo*Bp (SpConv)
    // SpConv (input staged channel-major, batch innermost, with a zero halo:
    // Xs[c][Hp][Wp][Bp], Hp = Hin + R - 1, Wp = Win + S - 1, image origin at (R/2, S/2))
    const __half* Xs;
    __half* out;             // [B*Ho*Wo][F] (NHWC) -- final or staged in stored filter order
    int Bn, Bp, Hp, Wp, Cin, F, R, S, stride, Ho, Wo;
    // chained SpConv: out[f][OHp][OWp][Bp] with the next layer's halo (origin at (oph, opw))
    int OWp, oph, opw, out_plane, relu;
    int wide_stores;         // SpMM, rows in lanes: output rows are 32-byte aligned (N % 16 == 0, D % 32 == 0)
    int out_logical;         // chained kernels: output plane of stored filter f is perm[f] (logical channel order) instead of f
    const __half* res;       // optional residual in the OUTPUT's geometry ([planes][OHp][OWp][Bp]) or nullptr
    const int* res_map;      // stored filter -> plane of `res` (nullptr: same index)
};

// MODE: 0 = SpMM, 1 = SpConv writing NHWC (stored filter order), 2 = SpConv writing the
// channel-major halo layout the next layer gathers from ("chained" layers).
// 3 = SpMM with the operands swapped: the block's V rows are the UMMA M dimension (64 or 128
// TMEM lanes) and the T tokens the N dimension, so ONE instruction per 16 columns covers the
// whole token tile (the instruction rate, 73 clk minimum each, is what limits this kernel) and
// the accumulator comes out with an output row per lane.
// 4 = chained SpConv with the operands swapped in the same way.
constexpr int kPanelSpmm = 0, kPanelConv = 1, kPanelConvChain = 2, kPanelSpmmRows = 3, kPanelConvChainRows = 4;

// GATHER: how the rows of the dense operand reach shared memory.
//   kGatherCpAsync  16-byte cp.async per lane, written straight into the swizzled layout; the
//                   producer warps wait for their copies and publish the stage themselves.
//   kGatherTma      TMA tile::gather4: one instruction per lane fetches 4 rows x 64 tokens (the
//                   tensor map covers this GPU's own B; no multicast), the copy engine applies
//                   the 128-byte swizzle and completes the stage's barrier by byte count, so the
//                   producers never wait for data.  SpMM with rows in lanes only.
//   kGatherCpAsyncArrive  the same 16-byte cp.async copies, but every lane hands its stage to the
//                   barrier with cp.async.mbarrier.arrive.noinc: the arrival fires when the lane's
//                   copies have landed, so the producers never wait for data and need no publish
//                   step; row ids travel in registers (loaded two stages ahead).
constexpr int kGatherCpAsync = 0, kGatherTma = 1, kGatherCpAsyncArrive = 2;

// EW: epilogue warps, 8 or 16.  A warp can read only the TMEM lane quadrant warp % 4, so the
// warps of a quadrant split the accumulator columns between them.  Items with few non-zero
// columns are all epilogue, and one warp's chain (TMEM read, convert, transpose, store) is
// latency-bound: sixteen warps keep four such chains per scheduler in flight instead of two.
template <int V, int TM, int KS_, int STAGES, int PW, int MODE, int GROUPS_ = 2, int LAG_ = 1, int GATHER_ = kGatherCpAsync,
          int EW_ = 8>
struct PanelCfg {
    static constexpr int EW = EW_;
    static_assert(EW == 8 || EW == 16, "epilogue warps");
    static constexpr bool TMA = GATHER_ == kGatherTma;
    static constexpr bool ARRIVE = GATHER_ == kGatherCpAsyncArrive;
    static constexpr int KS = KS_;                         // non-zero columns per pipeline stage
    static constexpr int T = 128 * TM;
    static constexpr int GROUPS = GROUPS_;                 // producer groups that take the stages in turn
    static constexpr int LAG = LAG_;                       // a group publishes a stage while issuing its LAG-th next one
    // Warp w runs on scheduler partition w % 4.  The MMA warp (the first after the epilogue
    // warps: 8 or 16) sits on partition 0 and no producer shares it: the later warps with
    // w % 4 == 0 stay idle.  The MMA warp executes a
    // few dozen instructions per stage and was measured at ~20 clk per instruction when
    // producer code kept evicting its lines from the partition's instruction cache.
    static constexpr int WARPS_USED = EW + 1 + PW + (PW - 1) / 3;   // epilogue + MMA + producers + idle
    // Register budgets per role.  Up to 20 warps every thread can have the ~100 registers the
    // epilogue wants.  Beyond that the block is padded to whole warpgroups (4 warps) and
    // launched at 65536 / threads registers per thread; the producer / MMA warpgroups then give
    // registers back (setmaxnreg.dec) and the two epilogue warpgroups take them (setmaxnreg.inc).
    // (With 16 epilogue warps the block is 20 warps at 96 registers and is not split.)
    static constexpr bool REG_SPLIT = EW == 8 && WARPS_USED > 20;
    static_assert(EW == 8 || WARPS_USED <= 20, "16 epilogue warps: at most 3 producers (20 warps leave 96 registers per thread, 21-24 only 80)");
    static constexpr int WARPS = REG_SPLIT ? (WARPS_USED + 3) / 4 * 4 : WARPS_USED;
    static constexpr int THREADS = WARPS * 32;
    static constexpr int REGS_LEAN = 56;                                    // producers, MMA warp, idle warps
    static constexpr int REGS_EPI_RAW = (65536 - (WARPS - 8) * 32 * REGS_LEAN) / 256 / 8 * 8;
    static constexpr int REGS_EPI = REGS_EPI_RAW > 160 ? 160 : REGS_EPI_RAW;
    static_assert(!REG_SPLIT || REGS_EPI >= 88, "epilogue register budget");
    // Only the 32-warp block is used with the split: 1024 threads x 64 registers is exactly the
    // register file, so what the lean warpgroups return is exactly what the epilogue's increase
    // asks for.  (24-warp blocks launched at 80 registers were seen to block in setmaxnreg.inc:
    // the allocation granularity leaves less in the pool than the arithmetic says, and that wait
    // has no time limit.)
    static_assert(!REG_SPLIT || WARPS == 32, "register split: 32-warp blocks only");
    static constexpr int G_ACC = KS * 256;                 // gathered tile of one accumulator: [KS][128] fp16
    static constexpr int G_BYTES = TM * G_ACC;
    static constexpr int W_BYTES = KS * V * 2;
    static constexpr int STAGE_BYTES = G_BYTES + W_BYTES;
    static constexpr int PIPE_BYTES = STAGES * STAGE_BYTES;
    // Each epilogue warp transposes 32 tokens x 32 output rows / filters through 2 KB so that
    // its global stores are 16 bytes per lane and 64-byte runs.
    // Epilogue tiles (tokens in lanes only): each epilogue warp transposes 32 tokens x 32 output
    // rows / filters through 2 KB so that its global stores are 16 bytes per lane and 64-byte
    // runs.  With rows in lanes the stores go straight from registers.
    static constexpr int OUT_BYTES = (MODE == kPanelSpmmRows || MODE == kPanelConvChainRows) ? 0 : EW * 2048;
    static constexpr int BAR_BYTES = (STAGES * 2 + 12) * 8;  // mbarriers (ring, up to 4 + 4 accumulator, drain) + tmem slot + abort flag
    static constexpr int TAB_BYTES = 512 * 8;               // per-CTA item table (kPanelMaxItemsPerCta entries)
    static constexpr int IDX_AHEAD = LAG + 1;              // a group fetches row ids this many of its stages ahead
    static constexpr int IDX_RING = (IDX_AHEAD + 1) * GROUPS <= 8 ? 8 : 16;   // stages of row ids kept in shared memory
    static_assert((IDX_AHEAD + 1) * GROUPS <= IDX_RING, "row-id ring too small");
    static constexpr int IDX_BYTES = (TMA || ARRIVE) ? 0 : IDX_RING * KS * 4;   // (the TMA gather loads its row ids straight into registers)
    static constexpr int SMEM_BYTES = PIPE_BYTES + OUT_BYTES + BAR_BYTES + TAB_BYTES + IDX_BYTES + 1024;  // + align slack
    static constexpr bool SWAP = MODE == kPanelSpmmRows || MODE == kPanelConvChainRows;
    static constexpr int KG_BYTES = SWAP ? T * 16 : 2048;   // 8 gathered rows (one K group) of the token tile
    static constexpr uint32_t ACC_COLS = SWAP ? T : TM * V; // fp32 columns of one accumulator set
    static_assert(!SWAP || V == 64 || V == 128, "rows-in-lanes needs a legal UMMA M");
    // Accumulator sets in TMEM: two (the MMAs of item i+1 run while the epilogue reads item i);
    // four with sixteen epilogue warps, whose items are so short that the hand-over itself
    // (commit -> barrier -> poll -> TMEM read -> release -> poll -> issue) is what two sets
    // cannot hide.
    static constexpr int NBUF = (EW == 16 && ACC_COLS * 4 <= 512) ? 4 : 2;
    static constexpr uint32_t TMEM_COLS = NBUF * ACC_COLS < 32 ? 32 : NBUF * ACC_COLS;
    static_assert(V == 16 || V == 32 || V == 64 || V == 128, "row-block height");
    static_assert(V != 16 || !SWAP, "16-row blocks: tokens in lanes");
    static_assert(!TMA || (MODE == kPanelSpmmRows && V == 64), "TMA gather: SpMM with rows in lanes, 64-row blocks");
    static_assert(STAGE_BYTES % 1024 == 0, "stages must keep 1024-byte swizzle-atom alignment");
    static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "TMEM columns");
    static_assert(KS % 16 == 0 && PW % GROUPS == 0 && KS % (PW / GROUPS) == 0 && (KS / (PW / GROUPS)) % (32 / (T / 8)) == 0,
                  "rows per producer warp");
    static_assert(LAG >= 1 && LAG <= 2 && (TMA || ARRIVE || STAGES > GROUPS * LAG), "publish lag");
    static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");
};

// Shared-memory tile layouts (MN-major operands; r = K row inside the stage, c = 16-byte
// chunk along MN).  A 128-byte-swizzle atom is 8 K rows x 128 bytes (64 fp16 along MN); the
// chunk index inside a row is XORed with r % 8.
//   two atoms wide (128 fp16 along MN):  K group g = r / 8 at g*2048, MN atom c / 8 at +1024
//       -> descriptor LBO = 1024 (next MN atom), SBO = 2048 (next K group); K-step j at j*4096
//   one atom wide (64 fp16):             K group at g*1024 -> SBO = 1024; K-step j at j*2048
//   64-byte swizzle, 32 fp16 wide:       atom = 8 rows x 64 bytes, chunk XOR (r/2)%4,
//                                        K group at g*512 -> SBO = 512; K-step j at j*1024
__device__ __forceinline__ uint32_t tile128_off(int r, int c) {
    return (uint32_t)((r >> 3) * 2048 + (c >> 3) * 1024 + (r & 7) * 128 + (((c & 7) ^ (r & 7)) << 4));
}
__device__ __forceinline__ uint32_t tile64_off(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }
__device__ __forceinline__ uint32_t tile32_off(int r, int c) { return (uint32_t)(r * 64 + ((c ^ ((r >> 1) & 3)) << 4)); }

constexpr int kPanelMaxItemsPerCta = 512;  // capacity of the per-CTA item table

template <int V, int TM, int KS_, int STAGES, int PW, int MODE, int GROUPS_ = 2, int LAG_ = 1, int GATHER_ = kGatherCpAsync,
          int EW_ = 8>
__global__ void __launch_bounds__(PanelCfg<V, TM, KS_, STAGES, PW, MODE, GROUPS_, LAG_, GATHER_, EW_>::THREADS, 1)
panel_umma_kernel(const __grid_constant__ PanelParams p) {
    using Cfg = PanelCfg<V, TM, KS_, STAGES, PW, MODE, GROUPS_, LAG_, GATHER_, EW_>;
    constexpr int EW = Cfg::EW;                                             // epilogue warps 0..EW-1, MMA warp EW, producers after it
    constexpr bool SWAP = Cfg::SWAP;                                        // rows in TMEM lanes
    constexpr bool CONV = MODE == kPanelConv || MODE == kPanelConvChain || MODE == kPanelConvChainRows;  // implicit-GEMM gather
    constexpr bool CHAIN = MODE == kPanelConvChain || MODE == kPanelConvChainRows;
    constexpr bool ROWS_OUT = MODE == kPanelSpmm || MODE == kPanelConvChain; // transposing epilogue: rows out, tokens contiguous
    static_assert(EW == 8 || (ROWS_OUT && Cfg::ACC_COLS >= 128), "16 epilogue warps: transposing epilogue, >= 32 columns per warp");
    constexpr int KS = Cfg::KS, T = Cfg::T;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: swizzle atoms are addressed by absolute shared-memory address bits.
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* bar_area = smem + Cfg::PIPE_BYTES + Cfg::OUT_BYTES;
    uint64_t* full_bar = (uint64_t*)bar_area;          // [STAGES] producers -> MMA
    uint64_t* empty_bar = full_bar + STAGES;           // [STAGES] MMA -> producers
    constexpr int NBUF = Cfg::NBUF;
    uint64_t* acc_full = empty_bar + STAGES;           // [NBUF] MMA -> epilogue
    uint64_t* acc_empty = acc_full + NBUF;             // [NBUF] epilogue -> MMA
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + NBUF);
    volatile int* cta_abort = (volatile int*)(tmem_slot + 1);
    uint64_t* drain_bar = acc_empty + NBUF + 1;        // abort path only: MMA thread waits for its last MMAs
    int2* item_tab = (int2*)(bar_area + Cfg::BAR_BYTES);  // [nloc] (first padded row, padded row count)
    int* idx_ring = (int*)(bar_area + Cfg::BAR_BYTES + Cfg::TAB_BYTES);  // [IDX_RING][KS] row ids of upcoming stages

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#ifdef SHFLBW_ABLATE
    const int ablate = p.ablate;
    auto now = []() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; };
    const bool tracing = p.trace != nullptr && blockIdx.x == 0;
#define TRACE(role, n, k) do { if (tracing && (n) < 256 && !(ablate & 256)) p.trace[(role) * 1024 + (n) * 4 + (k)] = now(); } while (0)
#define CTRACE(k) do { if (p.trace != nullptr) p.trace[4096 + blockIdx.x * 8 + (k)] = now(); } while (0)
#define PTRACE(w, n, k) do { if (tracing && (n) < 256 && !(ablate & 256)) p.trace[8192 + (w) * 1024 + (n) * 4 + (k)] = now(); } while (0)
#else
#define PTRACE(w, n, k) do { } while (0)
#define CTRACE(k) do { } while (0)
    constexpr int ablate = 0;
#define TRACE(role, n, k) do { } while (0)
#endif
    // This CTA's work items: blockIdx.x, blockIdx.x + gridDim.x, ...  (host guarantees nloc <= table size)
    const int nloc = (p.num_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    auto item_block = [&](int item) { return p.tile_major ? item - fast_div(item, p.div_blocks) * p.num_blocks : fast_div(item, p.div_tiles); };
    auto item_tile = [&](int item) { return p.tile_major ? fast_div(item, p.div_blocks) : item - fast_div(item, p.div_tiles) * p.tiles_n; };

    if (tid == 0) CTRACE(0);
    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            // One arrival per producer WARP.  Per-thread deferred arrivals
            // (cp.async.mbarrier.arrive.noinc) were measured at ~3 clk of load/store-unit time
            // per thread, i.e. more than the copies themselves.
            // cp.async gather: one arrival per producer WARP of the group.  TMA gather: one arrival
            // (with the stage's byte count) by the group's first warp.
            // Deferred arrivals: one per LANE of the group's warps.
            sm100::mbar_init(&full_bar[s], Cfg::TMA ? 1 : Cfg::ARRIVE ? (PW / Cfg::GROUPS) * 32 : PW / Cfg::GROUPS);
            sm100::mbar_init(&empty_bar[s], 1);   // one tcgen05.commit per drain
        }
        for (int b = 0; b < NBUF; ++b) {
            sm100::mbar_init(&acc_full[b], 1);
            sm100::mbar_init(&acc_empty[b], EW);  // one arrival per epilogue warp
        }
        sm100::mbar_init(drain_bar, 1);
        *cta_abort = 0;
        sm100::mbar_init_fence();
    }
    for (int li = tid; li < nloc; li += blockDim.x) {
        const int blk = item_block((int)blockIdx.x + li * (int)gridDim.x);
        const int b0 = __ldg(p.blk_ptr + blk);
        item_tab[li] = make_int2(b0, __ldg(p.blk_ptr + blk + 1) - b0);
    }
    if (warp == EW) {
        sm100::tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        sm100::tmem_relinquish();
    }
    sm100::tc_fence_before_sync();
    __syncthreads();
    sm100::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t smem_base = sm100::smem_u32(smem);
    // Programmatic dependent launch: everything above (barriers, TMEM, the item table -- read from
    // the sparse operand, which no kernel writes) may overlap the tail of the previous kernel in
    // the stream; the dense operand, the residual and the output are touched only below.  The
    // next kernel may start its own prologue as soon as every block of this one got here.
    sm100::grid_dependency_launch();
    // The wait itself is executed per role, as late as each role allows: by the producers after
    // their first row ids (sparse operand) are on their way and before their first gather, by the
    // epilogue warps at once (they read C / the residual and write the output); the MMA warp
    // touches no global memory and does not wait.
    if (tid == 0) TRACE(3, 0, 0);
    if (tid == 0) CTRACE(1);

    const int pidx = warp - (EW + 1) - (warp / 4 - EW / 4);   // producer number of a producer warp (warps after the MMA warp with warp % 4 != 0)
    if constexpr (Cfg::REG_SPLIT) {
        // Whole warpgroups change their register budget together: warps 0-7 (epilogue) grow,
        // every other warpgroup (MMA warp, producers, idle and padding warps) shrinks first.
        if (warp < EW) sm100::setmaxnreg_inc<Cfg::REGS_EPI>();
        else sm100::setmaxnreg_dec<Cfg::REGS_LEAN>();
    }
    if (warp > EW && ((warp & 3) == 0 || pidx >= PW)) {
        // idle: keeps producers off the MMA warp's scheduler partition (or pads the last warpgroup)
    } else if (warp > EW && Cfg::TMA) {
        // ---------------------------------------------------- producers (TMA gather) ----
        // A stage is KS gathered rows x T tokens = (KS/4) row quads x (T/64) column boxes, one
        // tile::gather4 each (4 rows x 128 bytes, landing as half a swizzle atom).  The GW warps
        // of a group split the stage's operations, one per lane; the group's first warp also
        // posts the stage's byte count and the bulk copy of the value slice.  Nobody waits for
        // data: the barrier completes when the bytes have arrived.
        if constexpr (Cfg::TMA) {
        constexpr int GROUPS = Cfg::GROUPS, GW = PW / GROUPS;
        constexpr int BOXES = T / 64;                       // column boxes per row quad
        constexpr int OPS = (KS / 4) * BOXES / GW;          // operations per warp per stage
        static_assert((KS / 4) * BOXES % GW == 0 && OPS >= 1 && OPS <= 32, "gather4 operations per producer warp");
        const int grp = pidx / GW, pw = pidx % GW;
        const int opj = pw * OPS + lane;                    // this lane's operation of a stage
        const int quad = opj / BOXES, cbox = opj % BOXES;
        const bool issuer = lane < OPS;
        const uint32_t dst_off = (uint32_t)((quad >> 1) * Cfg::KG_BYTES + cbox * 1024 + (quad & 1) * 512);
        struct Cursor { int li, kt, num_k, row_begin, rows_total; };
        auto enter = [&](Cursor& c) {
            c.kt = 0;
            while (c.li < nloc) {
                const int2 e = item_tab[c.li];
                c.row_begin = e.x; c.rows_total = e.y; c.num_k = (e.y + KS - 1) / KS;
                if (c.num_k > 0) return;
                ++c.li;
            }
            c.num_k = 0; c.row_begin = 0; c.rows_total = 0;
        };
        auto advance = [&](Cursor& c) { if (++c.kt >= c.num_k) { ++c.li; enter(c); } };
        // The 4 row ids of this lane's quad, loaded two of the group's stages ahead (registers).
        auto load_ids = [&](const Cursor& c) {
            const int r = c.kt * KS + quad * 4;
            if (issuer && c.li < nloc && r < c.rows_total) return __ldg((const int4*)(p.blk_idx + c.row_begin + r));
            return make_int4(0, 0, 0, 0);
        };
        Cursor pre{0, 0, 0, 0, 0};
        enter(pre);
        for (int d = 0; d < grp; ++d) advance(pre);
        int4 ids = load_ids(pre);                            // this group's first stage
        for (int g = 0; g < GROUPS; ++g) advance(pre);
        int4 ids_next = load_ids(pre);                       // and its second: two stages of ids are in flight,
        for (int g = 0; g < GROUPS; ++g) advance(pre);       // which covers the load's latency even with one group
        sm100::grid_dependency_wait();                       // the dense operand may be the previous kernel's output
        int it = 0;
#ifdef SHFLBW_COUNTERS
        long long pc_empty = 0, pc_n = 0, pc_t0 = clock64();
#endif
        for (int li = 0; li < nloc; ++li) {
            const int2 ent = item_tab[li];
            const int num_k = (ent.y + KS - 1) / KS;
            if (num_k == 0) continue;
            const int item = (int)blockIdx.x + li * (int)gridDim.x;
            const int col = item_tile(item) * T + cbox * 64;     // first token of this lane's box (beyond N: zero fill)
            const __half* wsrc = p.blk_val + (size_t)ent.x * V;
            for (int kt = 0; kt < num_k; ++kt, ++it) {
                if ((it % GROUPS) != grp) continue;
                const int s = it % STAGES;
                if (it >= STAGES) {
#ifdef SHFLBW_COUNTERS
                    const long long e0c = clock64();
#endif
                    int ok = 1;
                    if (lane == 0)
                        ok = sm100::mbar_wait_bounded(&empty_bar[s], ((it / STAGES) - 1) & 1, cta_abort, p.status_word,
                                                      SHFLBW_DEVSTAT_TIMEOUT_EMPTY, p.wait_limit, 32);
                    if (!__shfl_sync(0xffffffffu, ok, 0)) goto tma_producer_done;
#ifdef SHFLBW_COUNTERS
                    pc_empty += clock64() - e0c; ++pc_n;
#endif
                }
                const int rows_valid = min(KS, ent.y - kt * KS);    // multiple of 16
                const uint32_t st_base = smem_base + s * Cfg::STAGE_BYTES;
                if (pw == 0 && lane == 0) {
                    const uint32_t wbytes = (uint32_t)(rows_valid * V * 2);
#ifdef SHFLBW_FAULT_INJECT
                    if (!(p.inject_from >= 0 && it >= p.inject_from && pidx == 0))   // the withheld arrival
#endif
                    sm100::mbar_arrive_expect_tx(&full_bar[s], (uint32_t)(rows_valid * T * 2) + wbytes);
                    if (!(ablate & 4)) sm100::bulk_copy_g2s(st_base + (uint32_t)Cfg::G_BYTES, wsrc + (size_t)kt * KS * V, wbytes, &full_bar[s]);
                    else sm100::mbar_complete_tx(&full_bar[s], wbytes);
                }
                if (issuer && quad * 4 < rows_valid) {
                    if (!(ablate & 2)) sm100::tma_gather4(st_base + dst_off, p.tmap_b, col, ids.x, ids.y, ids.z, ids.w, &full_bar[s]);
                    else sm100::mbar_complete_tx(&full_bar[s], 512u);
                }
                ids = ids_next;
                ids_next = load_ids(pre);
                for (int g = 0; g < GROUPS; ++g) advance(pre);
            }
        }
    tma_producer_done:;
#ifdef SHFLBW_COUNTERS
        if (lane == 0 && p.trace != nullptr && pidx < 8) {
            unsigned long long* o = p.trace + 148 * 16 + (blockIdx.x * 8 + pidx) * 4;
            o[0] = pc_empty; o[1] = pc_n; o[2] = clock64() - pc_t0;
        }
#endif
        }
    } else if (warp > EW && Cfg::ARRIVE) {
        // ------------------------------------- producers (cp.async, deferred arrivals) ----
        // The GW warps of a group share a stage (RPW rows each); a warp instruction copies RPI
        // rows of the token tile, 16 bytes per lane, straight into the swizzled layout.  After its
        // copies of a stage every lane issues cp.async.mbarrier.arrive.noinc on the stage's
        // barrier: the arrival is delivered when that lane's copies have landed.  Nothing here
        // waits for data; the only wait is for a free stage.  (The consumer orders the generic-
        // proxy writes before the tensor core's reads with a proxy fence after its own wait.)
        if constexpr (Cfg::ARRIVE) {
        constexpr int GROUPS = Cfg::GROUPS, GW = PW / GROUPS, RPW = KS / GW;
        constexpr int CPR = T / 8, RPI = 32 / CPR, NQ = RPW / RPI;
        constexpr int XT = NQ < 8 / RPI ? NQ : 8 / RPI;
        static_assert((RPW % 8 == 0 || 8 % RPW == 0) && RPW <= 32, "rows per producer warp");
        const int grp = pidx / GW, pw = pidx % GW;
        const int chunk = lane % CPR;
        const int sub = RPI == 2 ? (lane >> 4) : 0;
        const int rbase = pw * RPW + sub;
        const uint32_t gbase = SWAP ? (uint32_t)((pw * RPW / 8) * Cfg::KG_BYTES + (chunk >> 3) * 1024)
                                    : (uint32_t)((chunk >> 4) * Cfg::G_ACC + (pw * RPW / 8) * 2048 + (((chunk & 15) >> 3)) * 1024);
        uint32_t gx[XT];
#pragma unroll
        for (int j = 0; j < XT; ++j) {
            const int r7 = (pw * RPW + j * RPI + sub) & 7;
            gx[j] = (uint32_t)(r7 * 128 + (((chunk & 7) ^ r7) << 4));
        }
        struct Cursor { int li, kt, num_k, row_begin, rows_total; };
        auto enter = [&](Cursor& c) {
            c.kt = 0;
            while (c.li < nloc) {
                const int2 e = item_tab[c.li];
                c.row_begin = e.x; c.rows_total = e.y; c.num_k = (e.y + KS - 1) / KS;
                if (c.num_k > 0) return;
                ++c.li;
            }
            c.num_k = 0; c.row_begin = 0; c.rows_total = 0;
        };
        auto advance = [&](Cursor& c) { if (++c.kt >= c.num_k) { ++c.li; enter(c); } };
        // Lane j < RPW holds the id of row pw*RPW + j of a stage (for SpConv: its element offset);
        // ids are loaded two of the group's stages ahead and handed out by shuffle.
        auto load_id = [&](const Cursor& c) {
            int v = 0;
            const int r = c.kt * KS + pw * RPW + lane;
            if (lane < RPW && c.li < nloc && r < c.rows_total) v = __ldg(p.blk_idx + c.row_begin + r);
            if constexpr (CONV)
                return (int)min((unsigned)(((v & 0xffff) * (p.Hp * p.Wp) + ((v >> 16) & 0xff) * p.Wp + ((v >> 24) & 0xff)) * p.Bp), p.idx_limit);
            else
                return (int)min((unsigned)v, p.idx_limit);
        };
        Cursor pre{0, 0, 0, 0, 0};
        enter(pre);
        for (int d = 0; d < grp; ++d) advance(pre);
        int id_cur = load_id(pre);
        for (int g = 0; g < GROUPS; ++g) advance(pre);
        int id_next = load_id(pre);
        for (int g = 0; g < GROUPS; ++g) advance(pre);
        sm100::grid_dependency_wait();                       // the dense operand may be the previous kernel's output
        int it = 0;
#ifdef SHFLBW_COUNTERS
        long long pc_empty = 0, pc_n = 0, pc_t0 = clock64();
#endif
        for (int li = 0; li < nloc; ++li) {
            const int2 ent = item_tab[li];
            const int num_k = (ent.y + KS - 1) / KS;
            if (num_k == 0) continue;
            const int item = (int)blockIdx.x + li * (int)gridDim.x;
            const int tok0 = item_tile(item) * T + chunk * 8;
            const bool chunk_ok = tok0 < p.N;
            const uint32_t nbytes = chunk_ok ? 16u : 0u;
            const __half* conv_src0 = p.Xs;
            if constexpr (CONV) {
                if (chunk_ok) {
                    const int pix = fast_div(tok0, p.div_bp), nn = tok0 - pix * p.Bp;
                    const int oh = fast_div(pix, p.div_wo), ow = pix - oh * p.Wo;
                    conv_src0 = p.Xs + ((oh * p.stride * p.Wp + ow * p.stride) * p.Bp + nn);
                }
            }
            const __half* lane_src0 = chunk_ok ? p.B + tok0 : p.B;
            const uint32_t row_pitch = chunk_ok ? (uint32_t)p.N : 0u;
            const __half* wsrc = p.blk_val + (size_t)ent.x * V;
            for (int kt = 0; kt < num_k; ++kt, ++it) {
                if ((it % GROUPS) != grp) continue;
                const int s = it % STAGES;
                if (it >= STAGES) {
#ifdef SHFLBW_COUNTERS
                    const long long e0c = clock64();
#endif
                    int ok = 1;
                    if (lane == 0)
                        ok = sm100::mbar_wait_bounded(&empty_bar[s], ((it / STAGES) - 1) & 1, cta_abort, p.status_word,
                                                      SHFLBW_DEVSTAT_TIMEOUT_EMPTY, p.wait_limit, 32);
                    if (!__shfl_sync(0xffffffffu, ok, 0)) goto arrive_producer_done;
#ifdef SHFLBW_COUNTERS
                    pc_empty += clock64() - e0c; ++pc_n;
#endif
                }
                const int rows_valid = min(KS, ent.y - kt * KS);
                const uint32_t st_base = smem_base + s * Cfg::STAGE_BYTES;
                if (pw == 0 && lane == 0 && !(ablate & 4)) {
                    const uint32_t wbytes = (uint32_t)(rows_valid * V * 2);
                    sm100::mbar_expect_tx(&full_bar[s], wbytes);
                    sm100::bulk_copy_g2s(st_base + (uint32_t)Cfg::G_BYTES, wsrc + (size_t)kt * KS * V, wbytes, &full_bar[s]);
                }
                int idq[NQ];
#pragma unroll
                for (int q = 0; q < NQ; ++q) idq[q] = __shfl_sync(0xffffffffu, id_cur, q * RPI + sub);
#pragma unroll
                for (int q = 0; q < NQ; ++q) {
                    if (rbase + q * RPI < rows_valid && !(ablate & 2)) {
                        const uint32_t dst = st_base + gbase + (uint32_t)(((q * RPI) >> 3) * Cfg::KG_BYTES) + gx[q % XT];
                        if constexpr (CONV) sm100::cp_async_16(dst, conv_src0 + idq[q], nbytes);
                        else sm100::cp_async_16(dst, lane_src0 + (uint64_t)(uint32_t)idq[q] * row_pitch, nbytes);
                    }
                }
#ifdef SHFLBW_FAULT_INJECT
                if (!(p.inject_from >= 0 && it >= p.inject_from && pidx == 0))   // the withheld arrivals
#endif
                sm100::cp_async_arrive_noinc(&full_bar[s]);
                id_cur = id_next;
                id_next = load_id(pre);
                for (int g = 0; g < GROUPS; ++g) advance(pre);
            }
        }
    arrive_producer_done:
        sm100::cp_async_commit();
        sm100::cp_async_wait<0>();          // nothing of this warp is in flight when the block ends
#ifdef SHFLBW_COUNTERS
        if (lane == 0 && p.trace != nullptr && pidx < 8) {
            unsigned long long* o = p.trace + 148 * 16 + (blockIdx.x * 8 + pidx) * 4;
            o[0] = pc_empty; o[1] = pc_n; o[2] = clock64() - pc_t0;
        }
#endif
        }
    } else if (warp > EW) {
        // ------------------------------------------------------------- producers ----
        // The PW producer warps form GROUPS groups that take the CTA's stages in turn (group g
        // fills stages g, g+GROUPS, ...).  While one group sits in its barrier round trip
        // (wait for the free stage, wait for its copies, publish) the other one issues copies,
        // so the load/store unit stays busy; with a single group the round trip (~400 clk)
        // simply added to every stage.
        constexpr int GROUPS = Cfg::GROUPS, LAG = Cfg::LAG;
        constexpr int GW = PW / GROUPS;        // warps that share one stage
        constexpr int RPW = KS / GW;           // rows of a stage owned by this warp
        constexpr int CPR = T / 8;             // 16-byte chunks per gathered row
        constexpr int RPI = 32 / CPR;          // rows per warp instruction (TM=2: 1, TM=1: 2)
        constexpr int NQ = RPW / RPI;          // gather copies per lane per stage
        constexpr int XT = NQ < 8 / RPI ? NQ : 8 / RPI;   // period of the swizzle term along q
        static_assert(RPW % 8 == 0 || 8 % RPW == 0, "a producer warp owns whole 8-row swizzle groups or an aligned part of one");
        const int grp = pidx / GW, pw = pidx % GW;
        const int chunk = lane % CPR;          // this lane's chunk of the token tile
        const int sub = RPI == 2 ? (lane >> 4) : 0;
        // Everything that does not change from stage to stage is computed once.  Row q of this
        // lane is r = pw*RPW + q*RPI + sub; its swizzled offset splits into a lane constant, a
        // compile-time term in q and one of XT lane-dependent XOR terms.
        const int rbase = pw * RPW + sub;
        // K group (8 rows) stride and the 64-token swizzle atom inside it.  Tokens as UMMA M: two
        // 128-token halves, each [K group][2 atoms].  Tokens as UMMA N: [K group][T/64 atoms].
        const uint32_t gbase = SWAP ? (uint32_t)((pw * RPW / 8) * Cfg::KG_BYTES + (chunk >> 3) * 1024)
                                    : (uint32_t)((chunk >> 4) * Cfg::G_ACC + (pw * RPW / 8) * 2048 + (((chunk & 15) >> 3)) * 1024);
        uint32_t gx[XT];
#pragma unroll
        for (int j = 0; j < XT; ++j) {
            const int r7 = (pw * RPW + j * RPI + sub) & 7;
            gx[j] = (uint32_t)(r7 * 128 + (((chunk & 7) ^ r7) << 4));
        }
        // A cursor walks the flattened (item, stage) sequence of this CTA using the item table.
        struct Cursor { int li, kt, num_k, row_begin, rows_total; };
        auto enter = [&](Cursor& c) {           // position on the first stage of item c.li (skipping empty items)
            c.kt = 0;
            while (c.li < nloc) {
                const int2 e = item_tab[c.li];
                c.row_begin = e.x; c.rows_total = e.y; c.num_k = (e.y + KS - 1) / KS;
                if (c.num_k > 0) return;
                ++c.li;
            }
            c.num_k = 0; c.row_begin = 0; c.rows_total = 0;
        };
        auto advance = [&](Cursor& c) { if (++c.kt >= c.num_k) { ++c.li; enter(c); } };
        // Row ids are prefetched with 4-byte cp.async into a shared-memory ring (slot = stage %
        // IDX_RING; this warp owns entries [pw*RPW, pw*RPW + RPW) of its group's slots), LAG + 1 of
        // the group's stages ahead: they travel in the first cp.async group of a stage, and the
        // publish step of the group's (LAG + 1)-th stage before the one that reads them is the
        // last wait that is certain to cover that group.
        // (A register prefetch would stall: rotating the registers waits for the load in flight.)
        auto prefetch_idx = [&](const Cursor& c, int stage_no) {
            if (lane < RPW && !(ablate & 2048)) {
                const int r = c.kt * KS + pw * RPW + lane;
                const bool ok = c.li < nloc && r < c.rows_total;
                sm100::cp_async_4(sm100::smem_u32(idx_ring + (stage_no % Cfg::IDX_RING) * KS + pw * RPW + lane),
                                  ok ? p.blk_idx + c.row_begin + r : p.blk_idx, ok ? 4u : 0u);
            }
        };
        static_assert(RPW <= 32, "one lane per row of the warp's share when prefetching ids");

        Cursor cur{0, 0, 0, 0, 0}, pre{0, 0, 0, 0, 0};
        enter(cur);
        pre = cur;
        for (int d = 0; d < grp; ++d) advance(pre);            // the group's first stage
#pragma unroll 1
        for (int d = 0; d < Cfg::IDX_AHEAD; ++d) {             // ids of its first stages
            prefetch_idx(pre, grp + d * GROUPS);
            for (int g = 0; g < GROUPS; ++g) advance(pre);
        }
        sm100::cp_async_commit();
        sm100::cp_async_wait<0>();
        __syncwarp();
        sm100::grid_dependency_wait();                         // the dense operand may be the previous kernel's output

        int it = 0;        // stage counter across items (all groups count the same sequence)
        int pend[LAG];     // this group's stages not yet published, oldest first
#pragma unroll
        for (int i = 0; i < LAG; ++i) pend[i] = -1;
#ifdef SHFLBW_COUNTERS
        long long pc_empty = 0, pc_n = 0, pc_t0 = clock64();
#endif
        for (int li = cur.li; li < nloc; ++li) {
            const int2 ent = item_tab[li];
            const int num_k = (ent.y + KS - 1) / KS;
            if (num_k == 0) continue;
            // per-item decode of this lane's tokens
            const int item = (int)blockIdx.x + li * (int)gridDim.x;
            const int tok0 = item_tile(item) * T + chunk * 8;
            const bool chunk_ok = tok0 < p.N;
            const uint32_t nbytes = chunk_ok ? 16u : 0u;
            // SpConv: this lane's 8 tokens are 8 images of one output pixel; the staged input
            // has a zero halo, so tap (r, s) of that pixel is simply base + ((r*Wp + s) * Bp).
            const __half* conv_src0 = p.Xs;
            if constexpr (CONV) {
                if (chunk_ok) {
                    const int pix = fast_div(tok0, p.div_bp), nn = tok0 - pix * p.Bp;
                    const int oh = fast_div(pix, p.div_wo), ow = pix - oh * p.Wo;
                    conv_src0 = p.Xs + ((oh * p.stride * p.Wp + ow * p.stride) * p.Bp + nn);
                }
            }
            const __half* lane_src0 = chunk_ok ? p.B + tok0 : p.B;   // SpMM: column tok0 of row 0
            const uint32_t row_pitch = chunk_ok ? (uint32_t)p.N : 0u;   // out-of-range chunks read B[0] with size 0
            const __half* wsrc = p.blk_val + (size_t)ent.x * V;   // the block's value panel (stage kt at + kt*KS*V)

            for (int kt = 0; kt < num_k; ++kt, ++it) {
                if ((it % GROUPS) != grp) continue;            // the other group's stage
                const int s = it % STAGES, s_idx = it % Cfg::IDX_RING;
                if (it >= STAGES) {  // one lane polls; the warp follows through the broadcast of its result
#ifdef SHFLBW_COUNTERS
                    const long long e0c = clock64();
#endif
                    int ok = 1;
                    if (lane == 0)
                        ok = sm100::mbar_wait_bounded(&empty_bar[s], ((it / STAGES) - 1) & 1, cta_abort, p.status_word,
                                                      SHFLBW_DEVSTAT_TIMEOUT_EMPTY, p.wait_limit, 32);
                    if (!__shfl_sync(0xffffffffu, ok, 0)) goto producer_done;   // timed out or aborted: stop issuing
#ifdef SHFLBW_COUNTERS
                    pc_empty += clock64() - e0c; ++pc_n;
#endif
                }
                if (pw == 0 && lane == 0) TRACE(0, it, 0);
                if (lane == 0) PTRACE(pidx, it, 0);
                const int rows_valid = min(KS, ent.y - kt * KS);  // multiple of 16
                const uint32_t st_base = smem_base + s * Cfg::STAGE_BYTES;
                // An earlier stage of the group (the LAG-th before this one) is published half-way
                // through this stage's copies: every stage is committed as two cp.async groups, so
                // "all but the newest 2*LAG - 1 groups" covers every copy of that stage -- issued
                // at least LAG - 1/2 issue phases ago, so the wait does not stall, while the tensor
                // core gets the stage half an issue phase earlier than if it were published at the
                // end.
                auto publish_prev = [&]() {
                    sm100::cp_async_commit();
                    if (pend[0] >= 0) {
                        sm100::cp_async_wait<2 * LAG - 1>();
                        sm100::fence_proxy_async_smem();   // every lane: its generic-proxy writes -> tensor-core reads
                        __syncwarp();
#ifdef SHFLBW_FAULT_INJECT
                        if (p.inject_from >= 0 && it >= p.inject_from && pidx == 0) return;   // the withheld arrival
#endif
                        if (lane == 0) sm100::mbar_arrive(&full_bar[pend[0]]);
                    }
                };
                // Value panel slice [rows_valid][V]: stored in global memory in the byte order of
                // the shared-memory operand tile, so one bulk copy by the copy engine places it;
                // its bytes are added to what the stage's barrier waits for.
                if (pw == 0 && lane == 0 && !(ablate & 4)) {
                    const uint32_t wbytes = (uint32_t)(rows_valid * V * 2);
                    sm100::mbar_expect_tx(&full_bar[s], wbytes);
                    sm100::bulk_copy_g2s(st_base + (uint32_t)Cfg::G_BYTES, wsrc + (size_t)kt * KS * V, wbytes, &full_bar[s]);
                }
                prefetch_idx(pre, it + Cfg::IDX_AHEAD * GROUPS);   // joins this iteration's first cp.async group
                for (int g = 0; g < GROUPS; ++g) advance(pre);
                const int* ids = idx_ring + s_idx * KS;  // landed: their group was awaited last iteration

                // All row ids / offsets are fetched into registers BEFORE the first copy: the copy
                // instructions are ordered with respect to shared-memory reads, so a read placed
                // between two copies would serialise its latency into every iteration.
                if constexpr (!CONV) {
                    int idr[NQ];
#pragma unroll
                    for (int q = 0; q < NQ; ++q) idr[q] = (int)min((unsigned)ids[rbase + q * RPI], p.idx_limit);
#pragma unroll
                    for (int q = 0; q < NQ; ++q) {
                        if (q == NQ / 2) publish_prev();
                        if (rbase + q * RPI < rows_valid && !(ablate & 2))
                            sm100::cp_async_16(st_base + gbase + (uint32_t)(((q * RPI) >> 3) * Cfg::KG_BYTES) + gx[q % XT],
                                               lane_src0 + (uint64_t)(uint32_t)idr[q] * row_pitch, nbytes);
                    }
                } else {
                    // Column ids arrive decoded (c | r << 16 | s << 24).  Lane j < RPW turns row
                    // pw*RPW + j into an element offset once; the copies fetch it by shuffle.
                    const int idv = ids[pw * RPW + (lane % RPW)];
                    const int delta = (int)min((unsigned)(((idv & 0xffff) * (p.Hp * p.Wp) + ((idv >> 16) & 0xff) * p.Wp + ((idv >> 24) & 0xff)) * p.Bp),
                                               p.idx_limit);
                    int dq[NQ];
#pragma unroll
                    for (int q = 0; q < NQ; ++q) dq[q] = __shfl_sync(0xffffffffu, delta, q * RPI + sub);
#pragma unroll
                    for (int q = 0; q < NQ; ++q) {
                        if (q == NQ / 2) publish_prev();
                        if (rbase + q * RPI < rows_valid && !(ablate & 2))
                            sm100::cp_async_16(st_base + gbase + (uint32_t)(((q * RPI) >> 3) * Cfg::KG_BYTES) + gx[q % XT],
                                               conv_src0 + dq[q], nbytes);
                    }
                }
                sm100::cp_async_commit();
                if (pw == 0 && lane == 0) TRACE(0, it, 1);
                if (lane == 0) PTRACE(pidx, it, 1);
#pragma unroll
                for (int i = 0; i + 1 < LAG; ++i) pend[i] = pend[i + 1];
                pend[LAG - 1] = s;
                if (pw == 0 && lane == 0) TRACE(0, it, 2);
                if (lane == 0) PTRACE(pidx, it, 2);
            }
        }
    producer_done:
        // Publish the group's last stages (after a failed wait: just wait for the copies in flight).
        sm100::cp_async_wait<0>();
        sm100::fence_proxy_async_smem();
        __syncwarp();
#pragma unroll
        for (int i = 0; i < LAG; ++i)
            if (lane == 0 && pend[i] >= 0) sm100::mbar_arrive(&full_bar[pend[i]]);
        if (pw == 0 && lane == 0) CTRACE(2);
#ifdef SHFLBW_COUNTERS
        if (lane == 0 && p.trace != nullptr && pidx < 8) {
            unsigned long long* o = p.trace + 148 * 16 + (blockIdx.x * 8 + pidx) * 4;
            o[0] = pc_empty; o[1] = pc_n; o[2] = clock64() - pc_t0;
        }
#endif
    } else if (warp == EW) {
        // ------------------------------------------------------------ MMA warp ----
        constexpr uint32_t idesc = SWAP ? sm100::make_idesc_f16_mnmajor(V, T) : sm100::make_idesc_f16_mnmajor(128, V);
        // Descriptors are built once; per MMA only the 16-byte-granular start address field
        // (low bits) advances.  A single thread issues every MMA, so scalar work between two
        // tcgen05.mma instructions directly limits the tensor-pipe issue rate.
        const uint64_t gdesc0 = sm100::make_smem_desc(smem_base, 1024, Cfg::KG_BYTES, sm100::kSwizzle128B);
        const uint64_t wdesc0 =
            V == 16 ? sm100::make_smem_desc(smem_base + Cfg::G_BYTES, 256, 256, sm100::kSwizzle32B)
          : V == 32 ? sm100::make_smem_desc(smem_base + Cfg::G_BYTES, 512, 512, sm100::kSwizzle64B)
          : V == 64 ? sm100::make_smem_desc(smem_base + Cfg::G_BYTES, 1024, 1024, sm100::kSwizzle128B)
                    : sm100::make_smem_desc(smem_base + Cfg::G_BYTES, 1024, 2048, sm100::kSwizzle128B);
        constexpr uint32_t WSTEP = V * 32;  // bytes per K-step (16 rows) of the value tile
        // One thread runs the whole role (tcgen05.mma / commit are single-thread instructions):
        // no per-stage warp synchronisation, and the ring slot and its parity are carried
        // instead of being recomputed by division.
        if (lane == 0) {
            int it = 0;
#ifdef SHFLBW_COUNTERS
            long long cnt_wait = 0, cnt_n = 0, cnt_acc = 0, cnt_t0 = clock64();
#endif
#ifdef SHFLBW_ABLATE
            int held = -1;              // stage whose release waits for the next one (tuning: paired releases)
#endif
            uint32_t s = 0, ph = 0;     // ring slot of stage `it` and the parity of its full barrier
            bool ready = false;         // that barrier was already seen complete
            for (int li = 0; li < nloc; ++li) {
                const int rows_total = item_tab[li].y;
                const int num_k = (rows_total + KS - 1) / KS;
                const int b = li % NBUF;
#ifdef SHFLBW_COUNTERS
                const long long a0c = clock64();
#endif
                if (li >= NBUF && !sm100::mbar_wait_bounded(&acc_empty[b], ((li / NBUF) - 1) & 1, cta_abort, p.status_word,
                                                         SHFLBW_DEVSTAT_TIMEOUT_ACCUM, p.wait_limit, 20))
                    break;                                   // timed out or aborted: issue nothing more
#ifdef SHFLBW_COUNTERS
                cnt_acc += clock64() - a0c;
#endif
                const uint32_t acc_base = tmem_base + b * Cfg::ACC_COLS;
                for (int kt = 0; kt < num_k; ++kt, ++it) {
#ifdef SHFLBW_COUNTERS
                    if (!ready) {
                        const long long w0 = clock64();
                        sm100::mbar_wait_bounded(&full_bar[s], ph, cta_abort, p.status_word,
                                                 SHFLBW_DEVSTAT_TIMEOUT_FULL, p.wait_limit, 20);
                        cnt_wait += clock64() - w0; ++cnt_n;
                    }
#else
                    if (!ready && !sm100::mbar_wait_bounded(&full_bar[s], ph, cta_abort, p.status_word,
                                                            SHFLBW_DEVSTAT_TIMEOUT_FULL, p.wait_limit, 20))
                        goto mma_done;                       // timed out or aborted: issue nothing more
#endif
                    TRACE(1, it, 0);
                    // cp.async (generic proxy) data -> tensor-core (async proxy) reads; the copy engine's
                    // writes of the TMA gather are in the async proxy already
                    if (!Cfg::TMA && !(ablate & 16)) sm100::fence_proxy_async_smem();
                    sm100::tc_fence_after_sync();
                    int nk = (ablate & 1) ? 0 : min(KS, rows_total - kt * KS) / 16;
                    uint64_t gdj = gdesc0 + (uint64_t)((s * (uint32_t)Cfg::STAGE_BYTES) >> 4);
                    uint64_t wdj = wdesc0 + (uint64_t)((s * (uint32_t)Cfg::STAGE_BYTES) >> 4);
                    uint32_t accum = (uint32_t)(kt != 0);
                    if constexpr (SWAP) {
                        // A full stage (the common case) is issued as straight-line code: one thread
                        // issues every MMA, so the scalar work between two of them is what limits
                        // the issue rate; the descriptor steps are immediates here.
                        if (nk == KS / 16) {
#pragma unroll
                            for (int j = 0; j < KS / 16; ++j)
                                sm100::umma_f16_ss(acc_base, wdj + (uint64_t)(j * (WSTEP >> 4)), gdj + (uint64_t)(j * ((2 * Cfg::KG_BYTES) >> 4)),
                                                   idesc, j == 0 ? accum : 1u);
                            nk = 0;
                        }
                    }
#pragma unroll 1
                    for (int j = 0; j < nk; ++j) {
                        if constexpr (SWAP) {
                            sm100::umma_f16_ss(acc_base, wdj, gdj, idesc, accum);   // D[row][token] += W^T . G
                        } else {
#pragma unroll
                            for (int a = 0; a < TM; ++a)
                                sm100::umma_f16_ss(acc_base + a * V, gdj + (uint64_t)((a * Cfg::G_ACC) >> 4), wdj, idesc, accum);
                        }
                        gdj += (2 * Cfg::KG_BYTES) >> 4;
                        wdj += WSTEP >> 4;
                        accum = 1u;
                    }
#ifdef SHFLBW_ABLATE
                    if (ablate & 4096) {   // release stages in pairs: one pipeline drain per two stages
                        if (held >= 0 || kt + 1 == num_k) {
                            if (held >= 0) sm100::umma_commit(&empty_bar[held]);
                            sm100::umma_commit(&empty_bar[s]);
                            held = -1;
                        } else held = (int)s;
                    } else
#endif
                    if (ablate & 64) sm100::mbar_arrive(&empty_bar[s]);
                    else sm100::umma_commit(&empty_bar[s]);  // stage may be refilled once these MMAs retire
                    TRACE(1, it, 1);
                    // Test the next stage's barrier now: the round trip hides behind the MMAs just issued.
                    if (++s == (uint32_t)STAGES) { s = 0; ph ^= 1u; }
                    ready = sm100::mbar_test(&full_bar[s], ph);
                }
                if (num_k > 0 && !(ablate & 1)) sm100::umma_commit(&acc_full[b]);  // accumulator complete
                else sm100::mbar_arrive(&acc_full[b]);                             // nothing to wait for
            }
#ifdef SHFLBW_COUNTERS
            if (p.trace != nullptr) {
                unsigned long long* o = p.trace + blockIdx.x * 16;
                o[0] = cnt_wait; o[1] = cnt_n; o[2] = cnt_acc; o[3] = clock64() - cnt_t0; o[4] = it;
            }
#endif
        mma_done:
            if (*cta_abort) {
                // Aborted: the MMAs issued so far must retire before TMEM is freed and the block's
                // shared memory goes away.  One more commit, awaited with its own (short) limit.
                sm100::umma_commit(drain_bar);
                sm100::mbar_wait_bounded(drain_bar, 0, cta_abort, p.status_word, 0, 4000000LL, 100, /*heed_abort=*/false);
            }
        }
        __syncwarp();
        if (lane == 0) CTRACE(3);
    } else {
        // -------------------------------------------------------------- epilogue ----
        // Warp w reads TMEM lane quadrant w % 4 (tokens) and part w / 4 of the accumulator
        // columns (the block's output rows / filters): halves with eight warps, quarters with
        // sixteen.
        sm100::grid_dependency_wait();
        const int quad = warp & 3, half_id = warp >> 2;
        // (a single 16- or 32-column accumulator is not split; two 16-column accumulators go to the two halves)
        constexpr int HALVES = (Cfg::ACC_COLS >= 64 || (V == 16 && TM == 2)) ? EW / 4 : 1;
        constexpr int COLS = Cfg::ACC_COLS / HALVES;          // fp32 columns handled by this warp
        constexpr int CW = COLS < 32 ? COLS : 32;             // columns per pass through the 2 KB tile
        const bool reads = half_id < HALVES;
        const __half alpha1 = __float2half_rn(p.alpha), beta1 = __float2half_rn(p.beta);
        const __half2 alpha2 = __half2half2(alpha1);
#ifdef SHFLBW_COUNTERS
        long long ec_wait = 0, ec_t0 = clock64();
#endif
        for (int li = 0; li < nloc; ++li) {
#ifdef SHFLBW_COUNTERS
            const long long ew0 = clock64();
#endif
            const int item = (int)blockIdx.x + li * (int)gridDim.x;
            const int blk = item_block(item);
            const int n0 = item_tile(item) * T;
            const bool has_k = item_tab[li].y > 0 && !(ablate & 1);
            const int b = li % NBUF;
            // Wait for the item's accumulator (one lane polls, the warp follows).  false: the wait
            // timed out or the block is aborting -- store nothing more.
            auto wait_accumulator = [&]() -> bool {
                int acc_ok = 1;
                if (lane == 0)
                    acc_ok = sm100::mbar_wait_bounded(&acc_full[b], (li / NBUF) & 1, cta_abort, p.status_word,
                                                      SHFLBW_DEVSTAT_TIMEOUT_ACCUM, p.wait_limit, 32);
                if (!__shfl_sync(0xffffffffu, acc_ok, 0)) return false;
                sm100::tc_fence_after_sync();
#ifdef SHFLBW_COUNTERS
                ec_wait += clock64() - ew0;
#endif
                if (tid == 0) TRACE(2, li, 0);
                return true;
            };
            if constexpr (SWAP || !ROWS_OUT) {
                if (!wait_accumulator()) break;
            }
            if constexpr (SWAP) {
                // Rows in lanes: lane l of quadrant `quad` holds output row m of the block (V = 64:
                // the quadrant's first 16 lanes, m = 16*quad + l; V = 128: all 32, m = 32*quad + l)
                // and this warp reads token columns [half_id*T/2, +T/2), 32 at a time: a lane's 32
                // tokens are 64 contiguous bytes of its output row.  They are packed to fp16 and
                // stored straight from registers -- as two 32-byte stores (whole L2 sectors) when
                // the output rows are 32-byte aligned, else as four 16-byte stores.  No shared
                // memory is involved: the tensor core's operand reads and the gather's writes already
                // use most of its bandwidth.
                constexpr int LR = V == 64 ? 16 : 32;                    // rows (valid lanes) per quadrant
                constexpr int HC = T / 2;                                // token columns of this warp
                const uint32_t acc0 = tmem_base + ((uint32_t)(quad * 32) << 16) + b * Cfg::ACC_COLS + half_id * HC;
                const int m = quad * LR + (lane < LR ? lane : 0);
                size_t roff;                                             // element offset of this lane's output row
                size_t rres = 0;                                         // chained: offset of its residual row
                const bool use_res = CHAIN && p.res != nullptr;
                if constexpr (CHAIN) {
                    // plane of this filter: stored order between chained layers, logical order when the
                    // planes are about to be transposed to NHWC
                    const int plane = (p.out_logical && p.perm) ? __ldg(p.perm + blk * V + m) : blk * V + m;
                    roff = (size_t)plane * (size_t)p.out_plane;
                    if (use_res) rres = (size_t)(p.res_map ? __ldg(p.res_map + blk * V + m) : blk * V + m) * (size_t)p.out_plane;
                } else {
                    const int drow = (p.perm && !(ablate & 1024)) ? __ldg(p.perm + blk * V + m) : blk * V + m;
                    roff = (size_t)drow * (size_t)p.N;
                }
                __half* const obase = CHAIN ? p.out : p.D;
                const __half2 zero2 = __float2half2_rn(0.f);
                const bool use_c = !CHAIN && p.beta != 0.0f && p.C != nullptr;
#pragma unroll 1
                for (int cc = 0; cc < HC; cc += 32) {
                    const int tok0 = n0 + half_id * HC + cc;             // this lane's 32 tokens start here
                    // Where the four 8-token groups go, and (chained layers) the residual that gets added
                    // to them: requested before the accumulator read, so that the global-memory latency
                    // hides behind it.
                    size_t goffs[4];
                    uint4 addend[4];
                    if (lane < LR) {
                        if constexpr (CHAIN) {
                            // 8 consecutive tokens are 8 images of one output pixel; the pixel's place in the
                            // consumer's halo-padded plane is found once and stepped from group to group
                            int pix = fast_div(tok0, p.div_bp), nn = tok0 - pix * p.Bp;
                            int oh = fast_div(pix, p.div_wo), ow = pix - oh * p.Wo;
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                goffs[c] = (size_t)(((oh + p.oph) * p.OWp + ow + p.opw) * p.Bp + nn);
                                nn += 8;
                                if (nn >= p.Bp) { nn = 0; if (++ow >= p.Wo) { ow = 0; ++oh; } }
                            }
                        } else {
#pragma unroll
                            for (int c = 0; c < 4; ++c) goffs[c] = (size_t)(tok0 + c * 8);   // (folds into the addresses)
                        }
                        if constexpr (CHAIN) {
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                addend[c] = make_uint4(0u, 0u, 0u, 0u);
                                if (use_res && tok0 + c * 8 < p.N) addend[c] = *(const uint4*)(p.res + rres + goffs[c]);
                            }
                        }
                    }
                    uint32_t r[32];
                    if (has_k) {
                        sm100::tmem_ld_32x32b_x32(acc0 + cc, r);
                        sm100::tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int e = 0; e < 32; ++e) r[e] = 0u;
                    }
                    if (cc + 32 >= HC) {  // last TMEM read of this item by this warp: release the buffer
                        sm100::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) sm100::mbar_arrive(&acc_empty[b]);
                        if (tid == 0) TRACE(2, li, 1);
                    }
                    if (lane < LR && !(ablate & 520)) {
                    uint4 v[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        __half2* h = (__half2*)&v[c];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            // same arithmetic as the reference: round to fp16, then alpha in fp16
                            h[e] = __floats2half2_rn(__uint_as_float(r[c * 8 + 2 * e]), __uint_as_float(r[c * 8 + 2 * e + 1]));
                            if (!use_c) h[e] = __hmul2(h[e], alpha2);
                        }
                    }
                    if constexpr (!CHAIN) {
                        __half* dst = obase + roff + tok0;
                        if (p.wide_stores && !use_c) {                   // N % 16 == 0: 16 tokens are valid as a whole
                            if (tok0 < p.N) sm100::st_global_32B(dst, v[0], v[1]);
                            if (tok0 + 16 < p.N) sm100::st_global_32B(dst + 16, v[2], v[3]);
                        } else {
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                if (tok0 + c * 8 < p.N) {                // N % 8 == 0: 8 tokens are valid as a whole
                                    if (use_c) {                         // (the rare beta != 0 case pays the load's latency here)
                                        const uint4 cv = *(const uint4*)(p.C + roff + tok0 + c * 8);
                                        __half* h = (__half*)&v[c];
                                        const __half* ch = (const __half*)&cv;
#pragma unroll
                                        for (int e = 0; e < 8; ++e) h[e] = __hfma(h[e], alpha1, __hmul(ch[e], beta1));
                                    }
                                    *(uint4*)(dst + c * 8) = v[c];
                                }
                            }
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < 4; ++c) {
                            if (tok0 + c * 8 < p.N) {
                                __half2* h = (__half2*)&v[c];
                                if (use_res) {                           // out = relu(alpha * conv + residual), fp16
                                    const __half2* rh = (const __half2*)&addend[c];
#pragma unroll
                                    for (int e = 0; e < 4; ++e) h[e] = __hadd2(h[e], rh[e]);
                                }
                                if (p.relu) {
#pragma unroll
                                    for (int e = 0; e < 4; ++e) h[e] = __hmax2(h[e], zero2);
                                }
                                *(uint4*)(obase + roff + goffs[c]) = v[c];
                            }
                        }
                    }
                    }
                    __syncwarp();                                        // the next TMEM load is warp-wide
                }
                if (tid == 0) TRACE(2, li, 3);
                continue;
            }
            // columns [col0, col0 + COLS) of the accumulator set: accumulator a = col / V, row m = col % V
            const int col0 = half_id * COLS;
            const uint32_t acc_base = tmem_base + ((uint32_t)(quad * 32) << 16) + b * Cfg::ACC_COLS + col0;
            // per-item, per-thread constants
            const int a0 = col0 / V;                       // this warp's columns lie in one accumulator
            const int tok = reads ? n0 + a0 * 128 + quad * 32 + lane : p.N;   // idle warps store nothing
            const int mbase = col0 % V;                    // first block row / filter of this warp
            bool ok = tok < p.N && !(ablate & 8);
            uint32_t row_off[4];                           // SpConv: output offsets of positions i*8 + lane/4
            if constexpr (MODE == kPanelConv) {
                const int pix = fast_div(tok, p.div_bp), img = tok - pix * p.Bp;
                ok = ok && img < p.Bn;
                const int oh = fast_div(pix, p.div_wo), ow = pix - oh * p.Wo;
                // this position's F-vector at the block's filters (element offset; host checks it fits 32 bits)
                const uint32_t mine = ok ? (uint32_t)((img * p.Ho + oh) * p.Wo + ow) * (uint32_t)p.F + (uint32_t)(blk * V + mbase)
                                         : 0xffffffffu;
#pragma unroll
                for (int i = 0; i < 4; ++i) row_off[i] = __shfl_sync(0xffffffffu, mine, i * 8 + (lane >> 2));
            }
            const bool use_c = MODE == kPanelSpmm && p.beta != 0.0f && p.C != nullptr;
            if constexpr (ROWS_OUT) {
            // SpMM: thread = token, accumulator columns = the block's output rows.  For a fixed
            // row a warp's 32 tokens are only 64 contiguous bytes of D, and storing them straight
            // from registers is one 2-byte-per-lane store per row.  Instead each chunk of 32 rows
            // goes through a tile in shared memory as 16 row PAIRS x 32 tokens of half2 (one
            // packed conversion, one multiply and one 4-byte conflict-free write per pair) and
            // comes back as 16-byte pieces: a lane reads 8 tokens of a pair (two 16-byte reads,
            // the 16-byte units of odd pairs swapped so that a quarter warp covers all banks),
            // splits them into the pair's two rows with byte permutes and stores 16 bytes of
            // each; four lanes store one row's 64 bytes, eight rows per store instruction.  The
            // inverse row permutation is the row index of those stores.
            uint32_t* my_tile = (uint32_t*)(smem + Cfg::PIPE_BYTES + warp * 2048);
            const int tg = lane & 3;                                    // 8-token group stored by this lane
            // Slot j = 2i + h of a chunk is row 16i + 2*(lane/4) + h: pair 8i + lane/4, half h.
            auto slot_row = [&](int j) { return 16 * (j >> 1) + 2 * (lane >> 2) + (j & 1); };
            constexpr int NSLOT = CW / 8;                               // rows stored per lane and chunk
            // This lane's 8-token group of an item whose tile starts at token n0_: is it inside N
            // (N % 8 == 0: a group is valid as a whole), and its element offset inside an output
            // row.  SpMM: the token index.  Chained SpConv: 8 images of one output pixel inside the
            // next layer's halo-padded plane (images beyond the batch are computed from zero inputs
            // and are written as zeros).
            auto group_offset = [&](int n0_, bool& ok_) -> uint32_t {
                const int tok_g = reads ? n0_ + a0 * 128 + quad * 32 + tg * 8 : p.N;
                ok_ = tok_g < p.N && !(ablate & 8);
                uint32_t goff_ = (uint32_t)tok_g;
                if constexpr (MODE == kPanelConvChain) {
                    if (ok_) {
                        const int pix = fast_div(tok_g, p.div_bp), nn = tok_g - pix * p.Bp;
                        const int oh = fast_div(pix, p.div_wo), ow = pix - oh * p.Wo;
                        goff_ = (uint32_t)(((oh + p.oph) * p.OWp + ow + p.opw) * p.Bp + nn);
                    }
                }
                return goff_;
            };
            bool ok_g;
            const uint32_t goff = group_offset(n0, ok_g);
            __half* const obase = MODE == kPanelSpmm ? p.D : p.out;
            const __half2 zero2 = __float2half2_rn(0.f);
            // What gets added to the product (beta * C, or the residual of a chained layer) does not
            // depend on the accumulator: the addends of the item's first two chunks are requested
            // BEFORE waiting for it, each later chunk's two chunks ahead, so that their global-memory
            // latency is off the critical path (these layers are often all epilogue).  (Requesting
            // the NEXT item's addend a whole item ahead was measured 3-5 % slower on the residual
            // layers of the ResNet stack, which run at ~4.1 TB/s of HBM traffic either way.)
            constexpr int NCH = COLS / CW;
            const bool add_res = MODE == kPanelConvChain && p.res != nullptr;
            const bool need_add = ok_g && (use_c || add_res);
            uint4 addend[NCH > 1 ? 2 : 1][4];
            auto fetch_addend = [&](int blk_, uint32_t goff_, int cc, uint4 (&dst)[4]) {
#pragma unroll
                for (int i = 0; i < NSLOT; ++i) {
                    const int m = mbase + cc + slot_row(i);
                    if (use_c) {
                        const int row = (p.perm && !(ablate & 1024)) ? __ldg(p.perm + blk_ * V + m) : blk_ * V + m;
                        dst[i] = *(const uint4*)(p.C + (size_t)((uint32_t)row * (uint32_t)p.N) + (size_t)goff_);
                    } else {
                        const uint32_t rr = (uint32_t)(p.res_map ? __ldg(p.res_map + blk_ * V + m) : blk_ * V + m) * (uint32_t)p.out_plane;
                        dst[i] = *(const uint4*)(p.res + (size_t)rr + (size_t)goff_);
                    }
                }
            };
            if (need_add) {
                fetch_addend(blk, goff, 0, addend[0]);
                if constexpr (NCH > 1) fetch_addend(blk, goff, CW, addend[1]);
            }
            if (!wait_accumulator()) break;
#pragma unroll
            for (int ch = 0; ch < NCH; ++ch) {
                const int cc = ch * CW;
                uint32_t roff[4];                                        // D offsets of this lane's rows
#pragma unroll
                for (int i = 0; i < NSLOT; ++i) {
                    const int m = mbase + cc + slot_row(i);
                    if constexpr (MODE == kPanelSpmm) {
                        const int row = (p.perm && !(ablate & 1024)) ? __ldg(p.perm + blk * V + m) : blk * V + m;
                        roff[i] = (uint32_t)row * (uint32_t)p.N;
                    } else {
                        const int plane = (p.out_logical && p.perm) ? __ldg(p.perm + blk * V + m) : blk * V + m;
                        roff[i] = (uint32_t)plane * (uint32_t)p.out_plane;           // stored (chained) or logical order
                    }
                }
                {
                    uint32_t r[CW];                       // the chunk's accumulator columns of this token
                    if (has_k && reads) {
                        if constexpr (CW == 32) sm100::tmem_ld_32x32b_x32(acc_base + cc, r);
                        else sm100::tmem_ld_32x32b_x16(acc_base + cc, r);
                        sm100::tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int e = 0; e < CW; ++e) r[e] = 0u;
                    }
                    if (cc + CW >= COLS) {  // last TMEM read of this item by this warp: release the buffer
                        sm100::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) sm100::mbar_arrive(&acc_empty[b]);
                        if (tid == 0) TRACE(2, li, 1);
                    }
                    // Same epilogue arithmetic as the reference: round to fp16, then alpha (and
                    // beta * C, applied after the transpose) in fp16.
#pragma unroll
                    for (int q = 0; q < CW / 2; ++q) {
                        __half2 h = __floats2half2_rn(__uint_as_float(r[2 * q]), __uint_as_float(r[2 * q + 1]));
                        if (!use_c) h = __hmul2(h, alpha2);
                        my_tile[q * 32 + (lane ^ ((q & 1) << 2))] = *(uint32_t*)&h;
                    }
                }
                __syncwarp();
                if (!(ablate & 512)) {
#pragma unroll
                    for (int k = 0; k < NSLOT / 2; ++k) {
                        const int q = 8 * k + (lane >> 2);   // 8 tokens of this lane's k-th row pair
                        const uint32_t* src = my_tile + q * 32;
                        const uint4 w0 = *(const uint4*)(src + (((2 * tg) ^ (q & 1)) << 2));
                        const uint4 w1 = *(const uint4*)(src + (((2 * tg + 1) ^ (q & 1)) << 2));
#pragma unroll
                    for (int i = 2 * k; i < 2 * k + 2; ++i) {
                        const uint32_t sel = (i & 1) ? 0x7632u : 0x5410u;   // the pair's second / first row
                        uint4 v;
                        v.x = __byte_perm(w0.x, w0.y, sel); v.y = __byte_perm(w0.z, w0.w, sel);
                        v.z = __byte_perm(w1.x, w1.y, sel); v.w = __byte_perm(w1.z, w1.w, sel);
                        if (ok_g) {
                            const size_t off = (size_t)roff[i] + (size_t)goff;
                            if (use_c) {
                                __half* h = (__half*)&v;
                                const __half* cadd = (const __half*)&addend[NCH > 1 ? (ch & 1) : 0][i];
#pragma unroll
                                for (int e = 0; e < 8; ++e) h[e] = __hfma(h[e], alpha1, __hmul(cadd[e], beta1));
                            }
                            if constexpr (MODE == kPanelConvChain) {   // out = relu(alpha * conv + residual), fp16
                                __half2* h = (__half2*)&v;
                                if (add_res) {
                                    const __half2* rh = (const __half2*)&addend[NCH > 1 ? (ch & 1) : 0][i];
#pragma unroll
                                    for (int e = 0; e < 4; ++e) h[e] = __hadd2(h[e], rh[e]);
                                }
                                if (p.relu) {
#pragma unroll
                                    for (int e = 0; e < 4; ++e) h[e] = __hmax2(h[e], zero2);
                                }
                            }
                            *(uint4*)(obase + off) = v;
                        }
                    }
                    }
                }
                if constexpr (NCH > 2) { if (need_add && ch + 2 < NCH) fetch_addend(blk, goff, cc + 2 * CW, addend[ch & 1]); }
                __syncwarp();
            }
            } else {
            // SpConv: thread = output position, accumulator columns = consecutive filters of the
            // block, contiguous in the position's F-vector (stored filter order).  Straight from
            // registers a warp store would touch 32 lines (one per position); instead each
            // 32-filter chunk goes through a swizzled 2 KB tile so that four lanes write one
            // position's 64 contiguous bytes.
            uint8_t* my_tile = smem + Cfg::PIPE_BYTES + warp * 2048;
#pragma unroll 1
            for (int cc = 0; cc < COLS; cc += CW) {
#pragma unroll
                for (int j = 0; j < CW / 8; ++j) {
                    const int c0 = cc + j * 8;
                    uint32_t r[8];
                    if (has_k && reads) {
                        sm100::tmem_ld_32x32b_x8(acc_base + c0, r);
                        sm100::tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int e = 0; e < 8; ++e) r[e] = 0u;
                    }
                    if (c0 + 8 >= COLS) {  // last TMEM read of this item by this warp: release the buffer
                        sm100::tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) sm100::mbar_arrive(&acc_empty[b]);
                        if (tid == 0) TRACE(2, li, 1);
                    }
                    uint4 v;
                    __half2* h = (__half2*)&v;
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        h[e] = __hmul2(__floats2half2_rn(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1])), alpha2);
                    *(uint4*)(my_tile + lane * 64 + ((j ^ ((lane >> 1) & 3)) << 4)) = v;
                }
                __syncwarp();
                if (!(ablate & 512)) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int row = i * 8 + (lane >> 2), c = lane & 3;
                        const uint4 v = *(const uint4*)(my_tile + row * 64 + ((c ^ ((row >> 1) & 3)) << 4));
                        if (row_off[i] != 0xffffffffu && c < CW / 8) *(uint4*)(p.out + (size_t)row_off[i] + cc + c * 8) = v;
                    }
                }
                __syncwarp();
            }
            }
            if (tid == 0) TRACE(2, li, 3);
        }
#ifdef SHFLBW_COUNTERS
        if (lane == 0 && p.trace != nullptr && warp < 8) {   // per epilogue warp: cycles waiting for an accumulator, cycles in the role
            unsigned long long* o = p.trace + 148 * 48 + (blockIdx.x * 8 + warp) * 2;
            o[0] = ec_wait; o[1] = clock64() - ec_t0;
        }
#endif
        if (tid == 0) CTRACE(4);
    }

    if (*cta_abort) {
        // A wait gave up somewhere in this block.  Every role has stopped issuing work; what is
        // still in flight -- bulk copies of value slices (a few KB each) and gathers whose
        // groups were awaited above -- gets a bounded ~100 us to land before the shared memory
        // is released.
        const long long t0 = clock64();
        while (clock64() - t0 < 200000LL) __nanosleep(1000);
    }
    sm100::tc_fence_before_sync();
    __syncthreads();
    if (tid == 0) TRACE(3, 0, 1);
    if (tid == 0) CTRACE(5);
    if (warp == EW) {
        sm100::tc_fence_after_sync();
        sm100::tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

#undef TRACE
#undef CTRACE
#undef PTRACE

}  // namespace shflbw
