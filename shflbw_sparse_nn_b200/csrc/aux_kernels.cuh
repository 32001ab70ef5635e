// Small helper kernels around the panel kernel:
//   * relayout of the NHWC input into the channel-major, batch-innermost staging buffer the
//     implicit-GEMM gather reads (every im2col row becomes 16-byte-aligned runs),
//   * scatter of the staged output (stored filter order) into NHWC with the inverse filter
//     permutation applied,
//   * plain CUDA-core SpMM / SpConv kernels (fp32 accumulate, ascending column order) used
//     for bring-up and as an on-device cross-check of the tensor-core path.
#pragma once

#include <cstdint>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "shflbw_internal.hpp"

namespace shflbw {

// Programmatic dependent launch (see sm100_ptx.cuh): both are no-ops for plain launches.
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// in[n][hi][wi][c] (NHWC)  ->  Xs[c][hp][wp][Bp], the channel-major, batch-innermost staging
// buffer with a zero halo: hp = hi + ph in [0, Hp), wp = wi + pw in [0, Wp); images n >= Bn and
// halo pixels are written as zero, so every filter tap of every output pixel reads a valid
// address and the gather needs no bounds logic.
// One block: 64 channels x 128 (padded pixel, image) slots, images fastest.  Both global
// accesses are 16 bytes per thread (8 channels in, 8 images out); the transpose happens in
// shared memory, whose 8-slot groups are XOR-swizzled by the channel group so that neither
// the 2-byte scatter nor the 16-byte read-back has bank conflicts.  C % 8 == 0, Bp % 8 == 0.
constexpr int kRelayoutC = 64, kRelayoutSlots = 128;
__global__ void __launch_bounds__(256)
relayout_nhwc_to_chwn(const __half* __restrict__ in, __half* __restrict__ Xs, int Bn, int Bp, int Hin, int Win,
                      int Hp, int Wp, int ph, int pw, int C) {
    __shared__ __align__(16) __half tile[kRelayoutC * kRelayoutSlots];
    grid_dep_launch();                       // the consumer may set itself up while this kernel runs
    grid_dep_wait();                         // the staging buffer may still be read by the previous call's kernels
    const int NT = Bp < 32 ? Bp : 32;        // images per tile (a multiple of 8)
    const int PT = kRelayoutSlots / NT;      // padded pixels per tile
    const int n_tiles = (Bp + NT - 1) / NT;
    const int PP = Hp * Wp;
    const int p0 = (blockIdx.x / n_tiles) * PT, nb = (blockIdx.x % n_tiles) * NT;
    const int c0 = blockIdx.y * kRelayoutC;
    // load: thread -> (slot, 8-channel chunk), chunk fastest: 8 lanes read 128 contiguous bytes
    uint4 v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int e = threadIdx.x + i * 256;
        const int chunk = e & 7, slot = e >> 3;
        const int pl = slot / NT, nl = slot - pl * NT;
        const int pp = p0 + pl, n = nb + nl;
        const int hp = pp / Wp, hi = hp - ph, wi = pp - hp * Wp - pw;
        v[i] = make_uint4(0u, 0u, 0u, 0u);
        if (pl < PT && pp < PP && n < Bn && c0 + chunk * 8 < C && (unsigned)hi < (unsigned)Hin &&
            (unsigned)wi < (unsigned)Win)
            v[i] = __ldg((const uint4*)(in + (((size_t)n * Hin + hi) * Win + wi) * C + c0 + chunk * 8));
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int e = threadIdx.x + i * 256;
        const int chunk = e & 7, slot = e >> 3;
        const __half* h = (const __half*)&v[i];
        const int col = (((slot >> 3) ^ chunk) << 3) | (slot & 7);   // swizzled slot
#pragma unroll
        for (int j = 0; j < 8; ++j) tile[(chunk * 8 + j) * kRelayoutSlots + col] = h[j];
    }
    __syncthreads();
    // store: thread -> (channel, 8-slot group), group fastest: 8 consecutive images of one pixel
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int e = threadIdx.x + i * 256;
        const int g = e & 15, c = e >> 4;
        const int slot = g * 8;
        const int pl = slot / NT, nl = slot - pl * NT;
        const int pp = p0 + pl, n = nb + nl;
        if (pl < PT && pp < PP && n < Bp && c0 + c < C)
            *(uint4*)(Xs + ((size_t)(c0 + c) * PP + pp) * Bp + n) =
                *(const uint4*)(tile + c * kRelayoutSlots + ((g ^ (c >> 3)) << 3));
    }
}

// out[q][perm[f]] = staged[q][f] for every output position q.  G = clamp(F/8, 8, 64) threads
// share one position (each moves 8 filters at a time with 16-byte global accesses), so a block
// of 256 threads handles 256/G positions at once: 4 for F >= 512 (two warps each -- the kernel
// is latency-bound and more warps per position shorten it) up to 32 for F = 64.  The
// permutation sits in shared memory as 16-bit ids (read once per block); values are scattered
// into the position's F-vector in shared memory with 2-byte stores and leave as 16-byte stores.
// Dynamic shared memory: F*2 bytes (perm) + (256/G)*F*2 bytes.  F % 8 == 0, F <= 65536.
constexpr int kUnpermThreads = 256;
__host__ __device__ inline int unperm_threads_per_pos(int F) {
    int g = 8;
    while (g < 64 && g * 8 < F) g *= 2;
    return g;
}
__global__ void __launch_bounds__(kUnpermThreads)
unpermute_filters(const __half* __restrict__ staged, __half* __restrict__ out, const int* __restrict__ perm,
                  int num_pos, int F) {
    extern __shared__ __align__(16) uint8_t unperm_smem[];
    unsigned short* sperm = (unsigned short*)unperm_smem;        // [F]
    __half* vec = (__half*)(unperm_smem + (size_t)F * 2);        // [positions per block][F]
    const int G = unperm_threads_per_pos(F), P = kUnpermThreads / G;
    const int slot = threadIdx.x / G, t = threadIdx.x - slot * G;   // position slot, thread within it
    for (int f = threadIdx.x; f < F; f += kUnpermThreads) sperm[f] = (unsigned short)__ldg(perm + f);
    grid_dep_launch();
    grid_dep_wait();                         // the staged output is complete only when the panel kernel is
    __half* mine = vec + (size_t)slot * F;
    for (int q0 = blockIdx.x * P; q0 < num_pos; q0 += gridDim.x * P) {
        const int q = q0 + slot;
        __syncthreads();                                         // perm loaded / previous vectors read back
        if (q < num_pos) {
            const __half* src = staged + (size_t)q * F;
#pragma unroll 4
            for (int f8 = t * 8; f8 < F; f8 += G * 8) {
                const uint4 v = *(const uint4*)(src + f8);
                const uint4 pp = *(const uint4*)(sperm + f8);
                const __half* h = (const __half*)&v;
                mine[pp.x & 0xffff] = h[0]; mine[pp.x >> 16] = h[1]; mine[pp.y & 0xffff] = h[2]; mine[pp.y >> 16] = h[3];
                mine[pp.z & 0xffff] = h[4]; mine[pp.z >> 16] = h[5]; mine[pp.w & 0xffff] = h[6]; mine[pp.w >> 16] = h[7];
            }
        }
        __syncthreads();
        if (q < num_pos) {
            __half* dst = out + (size_t)q * F;
#pragma unroll 4
            for (int f8 = t * 8; f8 < F; f8 += G * 8) *(uint4*)(dst + f8) = *(const uint4*)(mine + f8);
        }
    }
}

// Chain buffer -> NHWC: out[n][h][w][perm[f]] = buf[f][h + ph][w + pw][n] (perm == nullptr:
// channels stay in stored order).  One block: one pixel x 8 images x all F filters; reads are
// 16 bytes (8 images of one (filter, pixel)), the F-vectors of the 8 images are assembled in
// shared memory with 2-byte stores and leave as 16-byte stores.  Dynamic shared memory:
// 8 * F * 2 bytes.  F % 8 == 0, Bp % 8 == 0.
__global__ void __launch_bounds__(256)
chain_export_nhwc(const __half* __restrict__ buf, __half* __restrict__ out, const int* __restrict__ perm,
                  int Bn, int Bp, int H, int W, int Hp, int Wp, int ph, int pw, int F) {
    extern __shared__ __align__(16) uint8_t export_smem[];
    __half* vec = (__half*)export_smem;                  // [8 images][F]
    grid_dep_launch();
    grid_dep_wait();                                     // the planes are complete only when their producer is
    const int groups = Bp / 8;
    const int pix = blockIdx.x / groups, n0 = (blockIdx.x % groups) * 8;
    const int h = pix / W, w = pix - h * W;
    const size_t plane = (size_t)Hp * Wp * Bp;
    const __half* src = buf + ((size_t)(h + ph) * Wp + (w + pw)) * Bp + n0;
    for (int f = threadIdx.x; f < F; f += 256) {
        const uint4 v = *(const uint4*)(src + (size_t)f * plane);
        const __half* hv = (const __half*)&v;
        const int c = perm ? __ldg(perm + f) : f;
#pragma unroll
        for (int j = 0; j < 8; ++j) vec[j * F + c] = hv[j];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < F; e += 256) {         // e = (image j, 8-channel chunk)
        const int j = e / (F / 8), c8 = (e - j * (F / 8)) * 8;
        if (n0 + j < Bn)
            *(uint4*)(out + (((size_t)(n0 + j) * H + h) * W + w) * F + c8) = *(const uint4*)(vec + j * F + c8);
    }
}

// planes[f][tok] -> out[n][pix][f]: the output of an NHWC call computed as planes (one row of
// tok = pix * Bp + n tokens per LOGICAL filter f) transposed to NHWC.  One block moves a tile of
// 64 filters x 64 tokens through 8 KB of shared memory: 16-byte loads of 8 tokens of one
// filter, 2-byte scatters into [token][filter] (8-filter groups XOR-swizzled by the token group,
// so neither side has bank conflicts), 16-byte stores of 8 filters of one token -- 128-byte runs
// in global memory on both sides.  F % 64 == 0, Bp % 8 == 0; images n >= Bn are padding.
__global__ void __launch_bounds__(256)
planes_to_nhwc(const __half* __restrict__ planes, __half* __restrict__ out, int Bn, int Bp, int npix, int F) {
    __shared__ __align__(16) __half tile[64 * 64];
    grid_dep_launch();
    grid_dep_wait();                                     // the planes are complete only when the panel kernel is
    const int ntok = npix * Bp;
    const int tok0 = blockIdx.x * 64, f0 = blockIdx.y * 64;
    const int c = threadIdx.x & 7, r0 = threadIdx.x >> 3;   // 16-byte chunk, row of the pass
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
        const int r = r0 + 32 * pass;                    // filter of the tile
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (tok0 + c * 8 < ntok) v = *(const uint4*)(planes + (size_t)(f0 + r) * ntok + tok0 + c * 8);
        const __half* h = (const __half*)&v;
        const int col = (((r >> 3) ^ c) << 3) | (r & 7);    // token group c: filter group XOR c
#pragma unroll
        for (int j = 0; j < 8; ++j) tile[(c * 8 + j) * 64 + col] = h[j];
    }
    __syncthreads();
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
        const int t = r0 + 32 * pass;                    // token of the tile
        const int tok = tok0 + t;
        const int pix = tok / Bp, n = tok - pix * Bp;
        if (tok < ntok && n < Bn)
            *(uint4*)(out + ((size_t)n * npix + pix) * F + f0 + c * 8) =
                *(const uint4*)(tile + t * 64 + ((c ^ ((t >> 3) & 7)) << 3));
    }
}

// Plain SpMM: one thread per (stored row, dense column); grid = (rows, column tiles).
__global__ void simt_spmm(const int* __restrict__ blk_ptr, const int* __restrict__ blk_idx,
                          const __half* __restrict__ blk_val, const int* __restrict__ perm,
                          const __half* __restrict__ B, const __half* __restrict__ C, __half* __restrict__ D,
                          int M, int N, int V, float alpha, float beta) {
    const int n = blockIdx.y * blockDim.x + threadIdx.x;
    const int row = blockIdx.x;
    if (n >= N || row >= M) return;
    const int blk = row / V, m = row % V;
    float acc = 0.f;
    for (int p = blk_ptr[blk]; p < blk_ptr[blk + 1]; ++p)
        acc += __half2float(blk_val[kval_index(V, (size_t)p, m)]) * __half2float(B[(size_t)blk_idx[p] * N + n]);
    const int dst = perm ? perm[row] : row;
    // Same epilogue arithmetic as the reference: round to fp16, then alpha / beta in fp16.
    __half h = __float2half_rn(acc), a = __float2half_rn(alpha);
    if (beta != 0.f && C) h = __hfma(h, a, __hmul(C[(size_t)dst * N + n], __float2half_rn(beta)));
    else h = __hmul(h, a);
    D[(size_t)dst * N + n] = h;
}

// Plain SpConv straight from NHWC to NHWC: one thread per (output position, stored filter);
// grid = (positions, filter tiles).
__global__ void simt_spconv(const int* __restrict__ blk_ptr, const int* __restrict__ blk_idx,
                            const __half* __restrict__ blk_val, const int* __restrict__ perm,
                            const __half* __restrict__ in, __half* __restrict__ out, int Bn, int Hin, int Win,
                            int Cin, int F, int R, int S, int stride, int Ho, int Wo, int V, float alpha) {
    const int f = blockIdx.y * blockDim.x + threadIdx.x;
    const int q = blockIdx.x;  // output position (n, ho, wo)
    if (f >= F) return;
    const int wo = q % Wo, ho = (q / Wo) % Ho, n = q / (Wo * Ho);
    const int blk = f / V, m = f % V;
    float acc = 0.f;
    for (int p = blk_ptr[blk]; p < blk_ptr[blk + 1]; ++p) {
        const int k = blk_idx[p];
        const int c = k % Cin, s = (k / Cin) % S, r = (k / Cin) / S;
        const int hi = ho * stride - R / 2 + r, wi = wo * stride - S / 2 + s;
        if (hi < 0 || hi >= Hin || wi < 0 || wi >= Win) continue;
        acc += __half2float(blk_val[kval_index(V, (size_t)p, m)]) *
               __half2float(in[(((size_t)n * Hin + hi) * Win + wi) * Cin + c]);
    }
    const int dst = perm ? perm[f] : f;
    out[(size_t)q * F + dst] = __hmul(__float2half_rn(acc), __float2half_rn(alpha));
}

}  // namespace shflbw
