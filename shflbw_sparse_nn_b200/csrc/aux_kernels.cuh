// Small helper kernels around the panel kernel:
//   * relayout of the NHWC input into the channel-major, batch-innermost staging buffer the
//     implicit-GEMM gather reads (every im2col row becomes 16-byte-aligned runs),
//   * scatter of the staged output (stored filter order) into NHWC with the inverse filter
//     permutation applied,
//   * plain CUDA-core SpMM / SpConv kernels (fp32 accumulate, ascending column order) used
//     for bring-up and as an on-device cross-check of the tensor-core path.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace shflbw {

// in[n][p][c] (NHWC, p = hi*Win + wi)  ->  Xs[c][p][Bp] with n < Bn copied and n >= Bn zero.
// One block: 64 channels x 128 (pixel, image) slots; reads are contiguous along c, writes
// contiguous along n.
constexpr int kRelayoutC = 64, kRelayoutSlots = 128;
__global__ void __launch_bounds__(256)
relayout_nhwc_to_chwn(const __half* __restrict__ in, __half* __restrict__ Xs, int Bn, int Bp, int P, int C) {
    __shared__ __half tile[kRelayoutC][kRelayoutSlots + 2];
    const int NT = Bp < 32 ? Bp : 32;        // images per tile (Bp is a multiple of 8)
    const int PT = kRelayoutSlots / NT;      // pixels per tile
    const int n_tiles = (Bp + NT - 1) / NT;
    const int p0 = (blockIdx.x / n_tiles) * PT, nb = (blockIdx.x % n_tiles) * NT;
    const int c0 = blockIdx.y * kRelayoutC;
    // load: thread -> (slot, channel) with channel fastest
    for (int e = threadIdx.x; e < kRelayoutC * kRelayoutSlots; e += 256) {
        const int c = e % kRelayoutC, slot = e / kRelayoutC;
        const int pl = slot / NT, nl = slot % NT;
        const int pp = p0 + pl, n = nb + nl;
        __half v = __float2half(0.f);
        if (pl < PT && pp < P && n < Bn && c0 + c < C) v = in[((size_t)n * P + pp) * C + c0 + c];
        tile[c][slot] = v;
    }
    __syncthreads();
    // store: thread -> (channel, slot) with slot (image) fastest
    for (int e = threadIdx.x; e < kRelayoutC * kRelayoutSlots; e += 256) {
        const int slot = e % kRelayoutSlots, c = e / kRelayoutSlots;
        const int pl = slot / NT, nl = slot % NT;
        const int pp = p0 + pl, n = nb + nl;
        if (pl < PT && pp < P && n < Bp && c0 + c < C) Xs[((size_t)(c0 + c) * P + pp) * Bp + n] = tile[c][slot];
    }
}

// out[q][perm[f]] = staged[q][f] for every output position q; one warp per position, the
// F-vector is permuted in shared memory so both global accesses are contiguous.
__global__ void __launch_bounds__(256)
unpermute_filters(const __half* __restrict__ staged, __half* __restrict__ out, const int* __restrict__ perm,
                  int num_pos, int F) {
    extern __shared__ __half vec[];  // [8 warps][F]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __half* mine = vec + (size_t)warp * F;
    for (int q = blockIdx.x * 8 + warp; q < num_pos; q += gridDim.x * 8) {
        const __half* src = staged + (size_t)q * F;
        for (int f = lane; f < F; f += 32) mine[perm[f]] = src[f];
        __syncwarp();
        __half* dst = out + (size_t)q * F;
        for (int f8 = lane * 8; f8 < F; f8 += 256) *(uint4*)(dst + f8) = *(const uint4*)(mine + f8);
        __syncwarp();
    }
}

// Plain SpMM: one thread per (stored row, dense column).
__global__ void simt_spmm(const int* __restrict__ blk_ptr, const int* __restrict__ blk_idx,
                          const __half* __restrict__ blk_val, const int* __restrict__ perm,
                          const __half* __restrict__ B, const __half* __restrict__ C, __half* __restrict__ D,
                          int M, int N, int V, float alpha, float beta) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int row = blockIdx.y;
    if (n >= N || row >= M) return;
    const int blk = row / V, m = row % V;
    float acc = 0.f;
    for (int p = blk_ptr[blk]; p < blk_ptr[blk + 1]; ++p)
        acc += __half2float(blk_val[(size_t)p * V + m]) * __half2float(B[(size_t)blk_idx[p] * N + n]);
    const int dst = perm ? perm[row] : row;
    // Same epilogue arithmetic as the reference: round to fp16, then alpha / beta in fp16.
    __half h = __float2half_rn(acc), a = __float2half_rn(alpha);
    if (beta != 0.f && C) h = __hfma(h, a, __hmul(C[(size_t)dst * N + n], __float2half_rn(beta)));
    else h = __hmul(h, a);
    D[(size_t)dst * N + n] = h;
}

// Plain SpConv straight from NHWC to NHWC: one thread per (output position, stored filter).
__global__ void simt_spconv(const int* __restrict__ blk_ptr, const int* __restrict__ blk_idx,
                            const __half* __restrict__ blk_val, const int* __restrict__ perm,
                            const __half* __restrict__ in, __half* __restrict__ out, int Bn, int Hin, int Win,
                            int Cin, int F, int R, int S, int stride, int Ho, int Wo, int V, float alpha) {
    const int f = blockIdx.x * blockDim.x + threadIdx.x;
    const int q = blockIdx.y;  // output position (n, ho, wo)
    if (f >= F) return;
    const int wo = q % Wo, ho = (q / Wo) % Ho, n = q / (Wo * Ho);
    const int blk = f / V, m = f % V;
    float acc = 0.f;
    for (int p = blk_ptr[blk]; p < blk_ptr[blk + 1]; ++p) {
        const int k = blk_idx[p];
        const int c = k % Cin, s = (k / Cin) % S, r = (k / Cin) / S;
        const int hi = ho * stride - R / 2 + r, wi = wo * stride - S / 2 + s;
        if (hi < 0 || hi >= Hin || wi < 0 || wi >= Win) continue;
        acc += __half2float(blk_val[(size_t)p * V + m]) *
               __half2float(in[(((size_t)n * Hin + hi) * Win + wi) * Cin + c]);
    }
    const int dst = perm ? perm[f] : f;
    out[(size_t)q * F + dst] = __hmul(__float2half_rn(acc), __float2half_rn(alpha));
}

}  // namespace shflbw
