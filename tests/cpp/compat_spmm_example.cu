// Acceptance example for include/shflbw_compat.hpp: reference-style caller code (the shape of
// the reference's example/spmm.blockwise.cu: random SpMM with C = ones, beta = 1) compiled
// against this library.  Exit code 0 = result matches a plain CPU loop within the reference's
// rule |ref - d| <= 1e-3 * |ref| (integer-valued inputs, so that means exact).
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "shflbw_compat.hpp"

int main() {
    const int m = 256, n = 136, k = 256, block_sz = 64;
    BlockwiseSpMatrix<half> spmat;
    spmat.init_random(m, k, block_sz, 1, 0.2f, /*row_permute=*/true, 2021);
    if (!spmat.initialized) { printf("init_random failed: %s\n", shflbw_strerror(spmat.last_status)); return 2; }
    spmat.transform_and_sync_device();
    if (!spmat.device_synced) { printf("no device copy: %s (%s)\n", shflbw_strerror(spmat.last_status), shflbw_last_cuda_error()); return 3; }

    std::vector<half> B(k * n), C(m * n, __float2half(1.0f)), D(m * n);
    for (auto& v : B) v = __float2half((float)(std::rand() % 9 - 4));
    half *dB, *dC, *dD;
    cudaMalloc(&dB, B.size() * 2); cudaMalloc(&dC, C.size() * 2); cudaMalloc(&dD, D.size() * 2);
    cudaMemcpy(dB, B.data(), B.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(dC, C.data(), C.size() * 2, cudaMemcpyHostToDevice);

    SpmmBlockwiseOp<ShapeBase<block_sz, 128, 32>, ShapeBase<32, 32, 32>, ShapeBase<16, 16, 16>, 3> op;
    op.initialize(spmat, n, dB, dC, dD);   // alpha = beta = 1, as the reference overload
    if (!op._state.initSuccess) { printf("initialize failed: %s\n", shflbw_strerror(op.status())); return 4; }
    op();
    if (cudaDeviceSynchronize() != cudaSuccess) { printf("kernel failed\n"); return 5; }
    cudaMemcpy(D.data(), dD, D.size() * 2, cudaMemcpyDeviceToHost);

    std::vector<float> ref(m * n, 0.f);
    for (int i = 0; i < m / block_sz; ++i)
        for (int p = spmat.indptr[i]; p < spmat.indptr[i + 1]; ++p)
            for (int mm = 0; mm < block_sz; ++mm) {
                const int row = spmat.row_permute_ids[i * block_sz + mm];
                const float a = __half2float(spmat.values[(size_t)p * block_sz + mm]);
                for (int nn = 0; nn < n; ++nn) ref[row * n + nn] += a * __half2float(B[spmat.indices[p] * n + nn]);
            }
    int bad = 0;
    for (int t = 0; t < m * n; ++t) {
        const float r = ref[t] + 1.0f, d = __half2float(D[t]);
        if (std::fabs(r - d) > 1e-3 * std::fabs(r)) ++bad;
    }
    printf(bad ? "Failed (%d mismatches)\n" : "Passed\n", bad);
    return bad ? 1 : 0;
}
