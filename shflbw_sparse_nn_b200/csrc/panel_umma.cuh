// The Shfl-BW panel kernel for sm_100a: one CTA computes, for ONE row block of V stored
// rows and ONE tile of T = 128*TM dense columns ("tokens": SpMM columns of B, or SpConv
// output positions), the dense contraction
//
//     acc[token][m] = sum_p  G[p][token] * W[p][m]          p over the block's non-zero columns
//
// on the 5th-generation tensor cores.  Mapping: tokens are the UMMA M dimension (128 TMEM
// lanes, always the full-rate shape), the V rows of the block are the UMMA N dimension
// (32/64/128 all legal), K = 16 per instruction.  Both operands are MN-major in shared
// memory: W[p][0..V) is a contiguous slice of the value panels and G[p][..] is row
// indices[p] of the dense operand, gathered.
//
//   warps 0-3  producers: 16-byte cp.async gathers into 128-byte-swizzled stages, then the
//              epilogue (TMEM -> registers -> fp16 -> global, inverse row permutation fused)
//   warp  4    allocates TMEM, issues tcgen05.mma (one elected lane), frees stages with
//              tcgen05.commit, frees TMEM
//
// Stage hand-over uses mbarriers; every wait is bounded (sm100_ptx.cuh) so a logic error
// cannot hang the GPU: the kernel records a code in the status word, drains and exits.
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

constexpr int kPanelKS = 64;            // non-zero columns per pipeline stage
constexpr int kPanelThreads = 160;      // 4 producer/epilogue warps + 1 MMA warp
constexpr long long kWaitLimitCycles = 400000000LL;  // ~0.2 s at 2 GHz

struct PanelParams {
    // sparse operand (kernel image)
    const int* blk_ptr;      // [X+1] padded offsets (multiples of 16)
    const int* blk_idx;      // padded column ids
    const __half* blk_val;   // [rows][V]
    const int* perm;         // [M] or nullptr
    int* status_word;
    float alpha, beta;
    // SpMM
    const __half* B;         // [K][N]
    const __half* C;         // [M][N] or nullptr
    __half* D;               // [M][N]
    int N;                   // dense columns (SpMM) / Ho*Wo*Bp (SpConv)
    // SpConv (input staged channel-major, batch innermost: Xs[c][hi][wi][Bp])
    const __half* Xs;
    __half* out;             // [B*Ho*Wo][F] (NHWC) -- final or staged in stored filter order
    int Bn, Bp, Hin, Win, Cin, F, R, S, stride, Ho, Wo;
};

template <int V, int TM, int STAGES>
struct PanelCfg {
    static constexpr int KS = kPanelKS;
    static constexpr int T = 128 * TM;
    static constexpr int G_ACC = KS * 256;                 // gathered tile of one accumulator: [KS][128] fp16
    static constexpr int G_BYTES = TM * G_ACC;
    static constexpr int W_BYTES = KS * V * 2;
    static constexpr int STAGE_BYTES = G_BYTES + W_BYTES;
    static constexpr int PIPE_BYTES = STAGES * STAGE_BYTES;
    static constexpr int OUT_BYTES = V * T * 2;            // SpMM epilogue staging [V][T] fp16
    static constexpr int DATA_BYTES = PIPE_BYTES > OUT_BYTES ? PIPE_BYTES : OUT_BYTES;
    static constexpr int BAR_BYTES = 256;                  // mbarriers + tmem slot + abort flag
    static constexpr int ROWID_BYTES = V * 4;
    static constexpr int SMEM_BYTES = DATA_BYTES + BAR_BYTES + ROWID_BYTES + 1024;  // + align slack
    static constexpr uint32_t TMEM_COLS = TM * V < 32 ? 32 : TM * V;
    static_assert(V == 32 || V == 64 || V == 128, "row-block height");
    static_assert(STAGE_BYTES % 1024 == 0, "stages must keep 1024-byte swizzle-atom alignment");
    static_assert((TMEM_COLS & (TMEM_COLS - 1)) == 0 && TMEM_COLS <= 512, "TMEM columns");
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

template <int V, int TM, int STAGES, bool CONV>
__global__ void __launch_bounds__(kPanelThreads)
panel_umma_kernel(const PanelParams p) {
    using Cfg = PanelCfg<V, TM, STAGES>;
    constexpr int KS = Cfg::KS, T = Cfg::T;
    constexpr int LAG = STAGES > 2 ? 2 : 1;  // cp.async groups in flight per thread before publishing
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: swizzle atoms are addressed by absolute shared-memory address bits.
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full_bar = (uint64_t*)(smem + Cfg::DATA_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* accum_bar = empty_bar + STAGES;
    uint32_t* tmem_slot = (uint32_t*)(accum_bar + 1);
    volatile int* cta_abort = (volatile int*)(tmem_slot + 1);
    int* row_ids = (int*)(smem + Cfg::DATA_BYTES + Cfg::BAR_BYTES);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int blk = blockIdx.y;
    const int n0 = blockIdx.x * T;
    const int row_begin = p.blk_ptr[blk];
    const int rows_total = p.blk_ptr[blk + 1] - row_begin;  // multiple of 16
    const int num_stages_k = (rows_total + KS - 1) / KS;

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) {
            sm100::mbar_init(&full_bar[s], 128);  // every producer thread arrives once per fill
            sm100::mbar_init(&empty_bar[s], 1);   // one tcgen05.commit per drain
        }
        sm100::mbar_init(accum_bar, 1);
        *cta_abort = 0;
        sm100::mbar_init_fence();
    }
    if (tid < V) row_ids[tid] = p.perm ? p.perm[blk * V + tid] : blk * V + tid;
    if (warp == 4) {
        sm100::tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
        sm100::tmem_relinquish();
    }
    sm100::tc_fence_before_sync();
    __syncthreads();
    sm100::tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t smem_base = sm100::smem_u32(smem);

    if (warp < 4) {
        // ------------------------------------------------------------- producers ----
        // Warp w owns rows [16w, 16w+16) of every stage = exactly K-step w of that stage.
        constexpr int CPR = T / 8;             // 16-byte chunks per gathered row
        constexpr int RPI = 32 / CPR;          // rows per warp instruction (TM=2: 1, TM=1: 2)
        const int chunk = lane % CPR;          // this lane's chunk of the token tile
        const int acc_id = chunk >> 4, c16 = chunk & 15;
        const int tok0 = n0 + chunk * 8;       // first token of the chunk
        const bool chunk_ok = tok0 < p.N;

        // SpConv: decode this lane's output position once.
        int ho = 0, wo = 0, nn = 0;
        if constexpr (CONV) {
            const int pix = tok0 / p.Bp;
            nn = tok0 - pix * p.Bp;
            ho = pix / p.Wo;
            wo = pix - ho * p.Wo;
        }
        const __half* lane_src0 = CONV ? p.Xs : p.B + tok0;

        auto load_idx = [&](int it) -> int {  // lane j < 16 holds the column id of row 16w+j
            const int r = it * KS + warp * 16 + (lane & 15);
            return (it < num_stages_k && r < rows_total) ? __ldg(p.blk_idx + row_begin + r) : 0;
        };
        int idx_cur = load_idx(0);

        for (int it = 0; it < num_stages_k; ++it) {
            const int s = it % STAGES;
            if (it >= STAGES)
                sm100::mbar_wait_bounded(&empty_bar[s], ((it / STAGES) - 1) & 1, cta_abort, p.status_word,
                                         SHFLBW_DEVSTAT_TIMEOUT_EMPTY, kWaitLimitCycles);
            const int idx_next = load_idx(it + 1);
            const int rows_valid = min(KS, rows_total - it * KS);  // multiple of 16
            const uint32_t g_base = smem_base + s * Cfg::STAGE_BYTES;
            const uint32_t w_base = g_base + Cfg::G_BYTES;

            if (warp * 16 < rows_valid) {
                // Per-row decode for SpConv: lane j works out (c, r, s) of its row, shared by shuffle.
                int k_or_coff = idx_cur, rs_pack = 0;
                if constexpr (CONV) {
                    const int c = idx_cur % p.Cin, rs = idx_cur / p.Cin;
                    const int fs = rs % p.S, fr = rs / p.S;
                    k_or_coff = c * p.Hin * p.Win;
                    rs_pack = (fr << 8) | fs;
                }
#pragma unroll
                for (int q = 0; q < 16 / RPI; ++q) {
                    const int jrow = q * RPI + (RPI == 2 ? (lane >> 4) : 0);  // row within the K-step
                    const int kk = __shfl_sync(0xffffffffu, k_or_coff, jrow);
                    const int r = warp * 16 + jrow;
                    const uint32_t dst = g_base + acc_id * Cfg::G_ACC + tile128_off(r, c16);
                    if constexpr (CONV) {
                        const int rs = __shfl_sync(0xffffffffu, rs_pack, jrow);
                        const int hi = ho * p.stride - (p.R >> 1) + (rs >> 8);
                        const int wi = wo * p.stride - (p.S >> 1) + (rs & 0xff);
                        const bool ok = chunk_ok && hi >= 0 && hi < p.Hin && wi >= 0 && wi < p.Win;
                        const __half* src = ok ? p.Xs + ((size_t)(kk + hi * p.Win + wi) * p.Bp + nn) : p.Xs;
                        sm100::cp_async_16(dst, src, ok ? 16u : 0u);
                    } else {
                        const __half* src = chunk_ok ? lane_src0 + (size_t)kk * p.N : p.B;
                        sm100::cp_async_16(dst, src, chunk_ok ? 16u : 0u);
                    }
                }
            }
            // Value panel slice [rows_valid][V]: contiguous in global memory.
            {
                constexpr int WCPR = V / 8;  // chunks per row
                const __half* wsrc = p.blk_val + (size_t)(row_begin + it * KS) * V;
                const int nchunks = rows_valid * WCPR;
                for (int q = tid; q < nchunks; q += 128) {
                    const int r = q / WCPR, c = q % WCPR;
                    uint32_t off;
                    if constexpr (V == 32) off = tile32_off(r, c);
                    else if constexpr (V == 64) off = tile64_off(r, c);
                    else off = tile128_off(r, c);
                    sm100::cp_async_16(w_base + off, wsrc + (size_t)q * 8, 16u);
                }
            }
            sm100::cp_async_commit();
            idx_cur = idx_next;
            if (it >= LAG) {
                sm100::cp_async_wait<LAG>();
                sm100::fence_proxy_async_smem();
                sm100::mbar_arrive(&full_bar[(it - LAG) % STAGES]);
            }
        }
        // Publish the last LAG stages.
        sm100::cp_async_wait<0>();
        sm100::fence_proxy_async_smem();
        for (int it = max(0, num_stages_k - LAG); it < num_stages_k; ++it)
            sm100::mbar_arrive(&full_bar[it % STAGES]);

        // -------------------------------------------------------------- epilogue ----
        if (num_stages_k > 0) {
            sm100::mbar_wait_bounded(accum_bar, 0, cta_abort, p.status_word, SHFLBW_DEVSTAT_TIMEOUT_ACCUM,
                                     kWaitLimitCycles);
            sm100::tc_fence_after_sync();
        }
        const __half2 alpha2 = __float2half2_rn(p.alpha);

        if constexpr (!CONV) {
            // TMEM -> fp16 -> staging tile S[m][token] (reuses the drained pipeline stages).
            __half* stage_out = (__half*)smem;
#pragma unroll
            for (int a = 0; a < TM; ++a) {
#pragma unroll
                for (int c0 = 0; c0 < V; c0 += 32) {
                    uint32_t r[32];
                    if (num_stages_k > 0) {
                        sm100::tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(warp * 32) << 16) + a * V + c0, r);
                        sm100::tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = 0u;
                    }
                    const int t = a * 128 + warp * 32 + lane;
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        stage_out[(c0 + j) * T + t] = __float2half_rn(__uint_as_float(r[j]));
                }
            }
            sm100::tc_fence_before_sync();
            asm volatile("bar.sync 1, 128;" ::: "memory");
            // Coalesced write-out: one 16-byte chunk per thread, a full tile row per CPR lanes.
            const __half2 beta2 = __float2half2_rn(p.beta);
            const bool use_c = p.beta != 0.0f && p.C != nullptr;
            for (int q = tid; q < V * CPR; q += 128) {
                const int m = q / CPR, ch = q % CPR;
                const int tok = n0 + ch * 8;
                if (tok >= p.N) continue;
                uint4 v = *(const uint4*)(stage_out + m * T + ch * 8);
                __half2* h = (__half2*)&v;
                const size_t g = (size_t)row_ids[m] * p.N + tok;
                if (use_c) {
                    uint4 cv = *(const uint4*)(p.C + g);
                    const __half2* ch2 = (const __half2*)&cv;
#pragma unroll
                    for (int e = 0; e < 4; ++e) h[e] = __hfma2(h[e], alpha2, __hmul2(ch2[e], beta2));
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e) h[e] = __hmul2(h[e], alpha2);
                }
                *(uint4*)(p.D + g) = v;
            }
        } else {
            // SpConv: thread = output position, registers = the block's V filters, which are
            // contiguous in the pixel's F-vector in stored filter order.
#pragma unroll
            for (int a = 0; a < TM; ++a) {
                const int tok = n0 + a * 128 + warp * 32 + lane;
                const int pix = tok / p.Bp, img = tok - pix * p.Bp;
                const bool ok = tok < p.N && img < p.Bn;
                const int oh = pix / p.Wo, ow = pix - oh * p.Wo;
                __half* dst = p.out + ((size_t)(img * p.Ho + oh) * p.Wo + ow) * p.F + blk * V;
#pragma unroll
                for (int c0 = 0; c0 < V; c0 += 32) {
                    uint32_t r[32];
                    if (num_stages_k > 0) {
                        sm100::tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(warp * 32) << 16) + a * V + c0, r);
                        sm100::tmem_ld_wait();
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = 0u;
                    }
                    if (ok) {
#pragma unroll
                        for (int j = 0; j < 32; j += 8) {
                            uint4 v;
                            __half2* h = (__half2*)&v;
#pragma unroll
                            for (int e = 0; e < 4; ++e)
                                h[e] = __hmul2(__floats2half2_rn(__uint_as_float(r[j + 2 * e]),
                                                                 __uint_as_float(r[j + 2 * e + 1])),
                                               alpha2);
                            *(uint4*)(dst + c0 + j) = v;
                        }
                    }
                }
            }
            sm100::tc_fence_before_sync();
        }
    } else {
        // ------------------------------------------------------------ MMA warp ----
        constexpr uint32_t idesc = sm100::make_idesc_f16_mnmajor(128, V);
        for (int it = 0; it < num_stages_k; ++it) {
            const int s = it % STAGES;
            if (lane == 0) {
                sm100::mbar_wait_bounded(&full_bar[s], (it / STAGES) & 1, cta_abort, p.status_word,
                                         SHFLBW_DEVSTAT_TIMEOUT_FULL, kWaitLimitCycles);
                sm100::tc_fence_after_sync();
                const int nk = min(KS, rows_total - it * KS) / 16;
                const uint32_t g_base = smem_base + s * Cfg::STAGE_BYTES;
                const uint32_t w_base = g_base + Cfg::G_BYTES;
                for (int j = 0; j < nk; ++j) {
                    uint64_t wdesc;
                    if constexpr (V == 32)
                        wdesc = sm100::make_smem_desc(w_base + j * 1024, 512, 512, sm100::kSwizzle64B);
                    else if constexpr (V == 64)
                        wdesc = sm100::make_smem_desc(w_base + j * 2048, 1024, 1024, sm100::kSwizzle128B);
                    else
                        wdesc = sm100::make_smem_desc(w_base + j * 4096, 1024, 2048, sm100::kSwizzle128B);
#pragma unroll
                    for (int a = 0; a < TM; ++a) {
                        const uint64_t gdesc = sm100::make_smem_desc(g_base + a * Cfg::G_ACC + j * 4096,
                                                                     1024, 2048, sm100::kSwizzle128B);
                        sm100::umma_f16_ss(tmem_base + a * V, gdesc, wdesc, idesc, (it | j) != 0 ? 1u : 0u);
                    }
                }
                sm100::umma_commit(&empty_bar[s]);                          // stage may be refilled
                if (it == num_stages_k - 1) sm100::umma_commit(accum_bar);  // accumulator complete
            }
            __syncwarp();
        }
    }

    __syncthreads();
    if (warp == 4) {
        sm100::tc_fence_after_sync();
        sm100::tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

}  // namespace shflbw
