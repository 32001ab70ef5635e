// Acceptance example for the SpConv half of include/shflbw_compat.hpp: caller code with the
// shape of the reference's example/spconv.blockwise.cu (random 3x3 filter, B=32, 14x14,
// C=F=256, block 32, density 0.2) compiled against this library.  Feature maps are NHWC here
// (the reference's are [C][H][W][B]); the check is a plain CPU loop over the same sparse
// filter with the reference's rule |ref - o| <= 1e-3 * |ref| (integer-valued inputs: exact).
// Run once without and once with a filter permutation.  Exit code 0 = both passed.
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "shflbw_compat.hpp"

static int run(bool filter_permute) {
    const int B = 32, H = 14, W = 14, C = 256, F = 256, R = 3, S = 3, stride = 1;
    const int block_sz = 32;
    BlockwiseSpFilter<half> spfilter;
    spfilter.init_random(F, R, S, C, block_sz, 1, 0.2f, filter_permute, 2021);
    if (!spfilter.initialized) { printf("init_random failed: %s\n", shflbw_strerror(spfilter.last_status)); return 2; }
    spfilter.transform_and_sync_device();
    if (!spfilter.device_synced) { printf("no device copy: %s\n", shflbw_last_cuda_error()); return 3; }

    std::vector<half> in((size_t)B * H * W * C), out((size_t)B * H * W * F);
    for (auto& v : in) v = __float2half((float)(std::rand() % 9 - 4));
    half *dI, *dO;
    cudaMalloc(&dI, in.size() * 2); cudaMalloc(&dO, out.size() * 2);
    cudaMemcpy(dI, in.data(), in.size() * 2, cudaMemcpyHostToDevice);
    cudaMemset(dO, 0xff, out.size() * 2);

    SpconvBlockwiseOp<ShapeBase<block_sz, 128, 32>, ShapeBase<32, 32, 32>, ShapeBase<16, 16, 16>, 3> op;
    op.initialize(spfilter, B, H, W, stride, dI, dO);
    if (!op._state.initSuccess) { printf("initialize failed: %s\n", shflbw_strerror(op.status())); return 4; }
    op();
    if (cudaDeviceSynchronize() != cudaSuccess) { printf("kernel failed\n"); return 5; }
    if (shflbw_matrix_device_status(spfilter.handle) != SHFLBW_OK) { printf("device status: %s\n", shflbw_last_cuda_error()); return 6; }
    cudaMemcpy(out.data(), dO, out.size() * 2, cudaMemcpyDeviceToHost);
    cudaFree(dI); cudaFree(dO);

    // CPU check: out[n][h][w][perm[f]] = sum_p W[p][f_local] * in[n][h + r - 1][w + s - 1][c],  k = (r*S + s)*C + c
    std::vector<float> ref((size_t)B * H * W * F, 0.f);
    for (int i = 0; i < F / block_sz; ++i)
        for (int p = spfilter.indptr[i]; p < spfilter.indptr[i + 1]; ++p) {
            const int k = spfilter.indices[p], c = k % C, s = (k / C) % S, r = k / C / S;
            for (int m = 0; m < block_sz; ++m) {
                const int f = filter_permute ? spfilter.row_permute_ids[i * block_sz + m] : i * block_sz + m;
                const float w = __half2float(spfilter.values[(size_t)p * block_sz + m]);
                if (w == 0.f) continue;
                for (int n = 0; n < B; ++n)
                    for (int h = 0; h < H; ++h) {
                        const int hi = h + r - R / 2;
                        if (hi < 0 || hi >= H) continue;
                        for (int x = 0; x < W; ++x) {
                            const int wi = x + s - S / 2;
                            if (wi < 0 || wi >= W) continue;
                            ref[(((size_t)n * H + h) * W + x) * F + f] += w * __half2float(in[(((size_t)n * H + hi) * W + wi) * C + c]);
                        }
                    }
            }
        }
    int bad = 0;
    for (size_t t = 0; t < ref.size(); ++t) {
        const float o = __half2float(out[t]);
        if (!(std::fabs(ref[t] - o) <= 1e-3 * std::fabs(ref[t]))) ++bad;
    }
    printf("filter_permute=%d: %s (%d mismatches)\n", (int)filter_permute, bad ? "Failed" : "Passed", bad);
    return bad ? 1 : 0;
}

int main() {
    const int a = run(false), b = run(true);
    printf((a || b) ? "Failed\n" : "Passed\n");
    return (a || b) ? 1 : 0;
}
