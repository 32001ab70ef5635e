// Acceptance example for load() in include/shflbw_compat.hpp: caller code with the shape of the
// reference's example/load_bsr.spmm.blockwise.cu -- a matrix dump arrives on stdin (the text
// format of example/spmatrix_dump_load.md), block height 32 is required, n = 1024,
// D = A*B + C with C = ones -- compiled against this library.  The check is a plain CPU loop
// with the reference's rule |ref - d| <= 1e-3 * |ref| (integer-valued inputs: exact).
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <vector>

#include "shflbw_compat.hpp"

int main() {
    BlockwiseSpMatrix<half> spmat;
    spmat.load(std::cin);
    if (!spmat.initialized) { printf("load failed: %s\n", shflbw_strerror(spmat.last_status)); return 2; }
    std::cout << "Finish matrix loading. Summary:\n" << spmat.config_str << std::endl;
    const int m = spmat.nrow, k = spmat.ncol, n = 1024;
    if (spmat.brow != 32) { std::cout << "This example code requires block brow=32.\n"; return 0; }
    spmat.transform_and_sync_device();
    if (!spmat.device_synced) { printf("no device copy: %s\n", shflbw_last_cuda_error()); return 3; }

    std::vector<half> B((size_t)k * n), C((size_t)m * n, __float2half(1.0f)), D((size_t)m * n);
    for (auto& v : B) v = __float2half((float)(std::rand() % 9 - 4));
    half *dB, *dC, *dD;
    cudaMalloc(&dB, B.size() * 2); cudaMalloc(&dC, C.size() * 2); cudaMalloc(&dD, D.size() * 2);
    cudaMemcpy(dB, B.data(), B.size() * 2, cudaMemcpyHostToDevice);
    cudaMemcpy(dC, C.data(), C.size() * 2, cudaMemcpyHostToDevice);
    cudaMemset(dD, 0xff, D.size() * 2);

    SpmmBlockwiseOp<ShapeBase<32, 128, 32>, ShapeBase<32, 32, 32>, ShapeBase<16, 16, 16>, 3> op;
    op.initialize(spmat, n, dB, dC, dD);
    if (!op._state.initSuccess) { printf("initialize failed: %s\n", shflbw_strerror(op.status())); return 4; }
    op();
    if (cudaDeviceSynchronize() != cudaSuccess) { printf("kernel failed\n"); return 5; }
    cudaMemcpy(D.data(), dD, D.size() * 2, cudaMemcpyDeviceToHost);

    std::vector<float> ref((size_t)m * n, 1.0f);
    for (int i = 0; i < m / 32; ++i)
        for (int p = spmat.indptr[i]; p < spmat.indptr[i + 1]; ++p)
            for (int mm = 0; mm < 32; ++mm) {
                const int row = spmat.row_permute ? spmat.row_permute_ids[i * 32 + mm] : i * 32 + mm;
                const float a = __half2float(spmat.values[(size_t)p * 32 + mm]);
                if (a == 0.f) continue;
                const half* b = &B[(size_t)spmat.indices[p] * n];
                for (int nn = 0; nn < n; ++nn) ref[(size_t)row * n + nn] += a * __half2float(b[nn]);
            }
    int bad = 0;
    for (size_t t = 0; t < ref.size(); ++t)
        if (!(std::fabs(ref[t] - __half2float(D[t])) <= 1e-3 * std::fabs(ref[t]))) ++bad;
    printf(bad ? "Failed (%d mismatches)\n" : "Passed\n", bad);
    return bad ? 1 : 0;
}
