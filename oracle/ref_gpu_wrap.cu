// TEST INFRASTRUCTURE ONLY -- C entry points around the UNMODIFIED reference CUDA kernels.
//
// Includes the reference's operator headers from the reference checkout (-I at build
// time; nothing is copied) and instantiates a handful of its tile configurations for
// sm_100a through the reference's own -DGPU_CC>=80 code path (cp.async + ldmatrix +
// mma.sync).  Built into oracle/_ref/libshflbw_ref_gpu.so by oracle/Makefile.  Used by
// the GPU parity tests (same arrays in, outputs compared) and by the benchmark to
// report the reference kernel's time on the same GPU ("the kernel to beat").
//
// Reference code reached from here:
//   block_sparse/spmm/blockwise_op.h:73-132, 180-209   (initialize / InitFn / ExecFn)
//   block_sparse/spconv/blockwise_op.h:70-131, 161-187
//   block_sparse/spmm/blockwise_format.h:200-266       (transform_and_sync_device)

#include <cstdint>
#include <cstring>
#include <vector>

#include "block_sparse/spmm/blockwise_op.h"
#include "block_sparse/spconv/blockwise_op.h"

namespace {

struct SpmmCfg { int V; const char* name; SpmmBlockwiseInitFn_t init; SpmmBlockwiseExecFn_t exec; };
struct ConvCfg { int V; const char* name; SpconvBlockwiseInitFn_t init; SpconvBlockwiseExecFn_t exec; };

#define CFG(BM, BN, BK, WM, WN, WK, NS)                                                        \
    { BM, #BM "x" #BN "x" #BK "_" #WM "x" #WN "x" #WK "_16x16x16_" #NS,                         \
      SpmmBlockwiseInitFn<ShapeBase<BM, BN, BK>, ShapeBase<WM, WN, WK>, ShapeBase<16, 16, 16>, NS>, \
      SpmmBlockwiseExecFn<ShapeBase<BM, BN, BK>, ShapeBase<WM, WN, WK>, ShapeBase<16, 16, 16>, NS> }
#define CCFG(BM, BN, BK, WM, WN, WK, NS)                                                       \
    { BM, #BM "x" #BN "x" #BK "_" #WM "x" #WN "x" #WK "_16x16x16_" #NS,                         \
      SpconvBlockwiseInitFn<ShapeBase<BM, BN, BK>, ShapeBase<WM, WN, WK>, ShapeBase<16, 16, 16>, NS>, \
      SpconvBlockwiseExecFn<ShapeBase<BM, BN, BK>, ShapeBase<WM, WN, WK>, ShapeBase<16, 16, 16>, NS> }

// A subset of the tile list of block_sparse/spmm/blockwise_library.cu (names as there).
const SpmmCfg kSpmm[] = {
    CFG(16, 64, 32, 16, 16, 32, 4),  CFG(16, 128, 32, 16, 32, 32, 4), CFG(16, 256, 32, 16, 64, 32, 4),
    CFG(32, 64, 32, 32, 16, 32, 4),  CFG(32, 128, 32, 32, 32, 32, 4), CFG(32, 256, 32, 32, 64, 32, 3),
    CFG(64, 64, 32, 32, 32, 32, 4),  CFG(64, 128, 32, 32, 32, 32, 4), CFG(64, 128, 32, 64, 32, 32, 3),
    CFG(64, 256, 16, 32, 64, 16, 3),
    CFG(128, 64, 32, 32, 32, 32, 4), CFG(128, 128, 32, 32, 64, 32, 4), CFG(128, 128, 32, 64, 32, 32, 2),
};
const ConvCfg kConv[] = {
    CCFG(32, 128, 32, 32, 32, 32, 3), CCFG(64, 64, 32, 32, 32, 32, 3), CCFG(64, 128, 32, 32, 32, 32, 3),
    CCFG(128, 64, 32, 32, 32, 32, 3),
};

template <class M>
void fill(M& m, int nrow, int ncol, int brow, int nnzb, const int* indptr, const int* indices,
          const uint16_t* values, const int* perm) {
    m.nrow = nrow; m.ncol = ncol; m.brow = brow; m.bcol = 1; m.nnzb = nnzb; m.seed = 0;
    m.row_permute = perm != nullptr;
    m.density = (float)nnzb / (nrow / brow) / ncol;
    m.indptr.assign(indptr, indptr + nrow / brow + 1);
    m.indices.assign(indices, indices + nnzb);
    m.values.resize((size_t)nnzb * brow);
    std::memcpy((void*)m.values.data(), values, (size_t)nnzb * brow * 2);
    if (perm) m.row_permute_ids.assign(perm, perm + nrow); else m.row_permute_ids.clear();
    m.initialized = true;
}

template <class Fn>
float time_launches(Fn launch, int warmup, int repeat) {
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    for (int i = 0; i < warmup; ++i) launch();
    cudaEventRecord(e0, 0);
    for (int i = 0; i < repeat; ++i) launch();
    cudaEventRecord(e1, 0);
    cudaEventSynchronize(e1);
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    return repeat > 0 ? ms / repeat : 0.f;
}

}  // namespace

extern "C" {

int ref_gpu_num_spmm_configs() { return (int)(sizeof(kSpmm) / sizeof(kSpmm[0])); }
int ref_gpu_num_conv_configs() { return (int)(sizeof(kConv) / sizeof(kConv[0])); }
const char* ref_gpu_spmm_config_name(int i) { return kSpmm[i].name; }
const char* ref_gpu_conv_config_name(int i) { return kConv[i].name; }
int ref_gpu_spmm_config_V(int i) { return kSpmm[i].V; }
int ref_gpu_conv_config_V(int i) { return kConv[i].V; }

// Runs the reference SpMM kernel config `cfg` on device buffers B_dev (K x N) -> D_dev (M x N).
// repeat > 0 additionally times `repeat` launches after `warmup` (reference protocol,
// block_sparse/benchmark/benchmark.spmm.cu:29-49) and stores the mean in *ms.
// Returns 0, or 1 config/V mismatch, 2 init failure, 3 CUDA error.
int ref_gpu_spmm(int cfg, int M, int K, int N, int brow, int nnzb, const int* indptr,
                 const int* indices, const uint16_t* values, const int* perm, void* B_dev,
                 void* D_dev, int warmup, int repeat, float* ms) {
    if (cfg < 0 || cfg >= ref_gpu_num_spmm_configs() || kSpmm[cfg].V != brow) return 1;
    BlockwiseSpMatrix<half> m;
    fill(m, M, K, brow, nnzb, indptr, indices, values, perm);
    m.transform_and_sync_device();
    SpmmBlockwiseOpState st = kSpmm[cfg].init(m, N, (half*)B_dev, (half*)D_dev);
    if (!st.initSuccess) return 2;
    kSpmm[cfg].exec(st, 0);
    if (cudaDeviceSynchronize() != cudaSuccess || cudaGetLastError() != cudaSuccess) return 3;
    if (repeat > 0 && ms) *ms = time_launches([&] { kSpmm[cfg].exec(st, 0); }, warmup, repeat);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// Reference SpConv kernel; feature maps in the reference's layouts (in [C][H][W][B],
// out [F][H][W][B]), B % 8 == 0 as its benchmark requires.
int ref_gpu_spconv(int cfg, int Bn, int H, int W, int C, int F, int R, int S, int stride, int brow,
                   int nnzb, const int* indptr, const int* indices, const uint16_t* values,
                   const int* perm, void* ifmap_dev, void* ofmap_dev, int warmup, int repeat,
                   float* ms) {
    if (cfg < 0 || cfg >= ref_gpu_num_conv_configs() || kConv[cfg].V != brow) return 1;
    BlockwiseSpFilter<half> f;
    fill(f, F, R * S * C, brow, nnzb, indptr, indices, values, perm);
    f.F = F; f.C = C; f.R = R; f.S = S;
    f.transform_and_sync_device();
    SpconvBlockwiseOpState st = kConv[cfg].init(f, Bn, H, W, stride, (half*)ifmap_dev, (half*)ofmap_dev);
    if (!st.initSuccess) return 2;
    kConv[cfg].exec(st, 0);
    if (cudaDeviceSynchronize() != cudaSuccess || cudaGetLastError() != cudaSuccess) return 3;
    if (repeat > 0 && ms) *ms = time_launches([&] { kConv[cfg].exec(st, 0); }, warmup, repeat);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// L2-cold variants: `nb` buffer pairs are rotated (state i % nb per launch) so that, with the
// pairs larger than L2 in aggregate, every launch reads its dense operand from HBM -- the same
// protocol the product kernels are timed with.  Only timing; run ref_gpu_spmm / ref_gpu_spconv
// first to check results.
int ref_gpu_spmm_rotating(int cfg, int M, int K, int N, int brow, int nnzb, const int* indptr,
                          const int* indices, const uint16_t* values, const int* perm, void** B_dev,
                          void** D_dev, int nb, int warmup, int repeat, float* ms) {
    if (cfg < 0 || cfg >= ref_gpu_num_spmm_configs() || kSpmm[cfg].V != brow || nb < 1 || nb > 64) return 1;
    BlockwiseSpMatrix<half> m;
    fill(m, M, K, brow, nnzb, indptr, indices, values, perm);
    m.transform_and_sync_device();
    std::vector<SpmmBlockwiseOpState> st;
    for (int i = 0; i < nb; ++i) {
        st.push_back(kSpmm[cfg].init(m, N, (half*)B_dev[i], (half*)D_dev[i]));
        if (!st.back().initSuccess) return 2;
    }
    int i = 0;
    *ms = time_launches([&] { kSpmm[cfg].exec(st[i], 0); i = (i + 1) % nb; }, warmup, repeat);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

int ref_gpu_spconv_rotating(int cfg, int Bn, int H, int W, int C, int F, int R, int S, int stride, int brow,
                            int nnzb, const int* indptr, const int* indices, const uint16_t* values,
                            const int* perm, void** ifmap_dev, void** ofmap_dev, int nb, int warmup, int repeat,
                            float* ms) {
    if (cfg < 0 || cfg >= ref_gpu_num_conv_configs() || kConv[cfg].V != brow || nb < 1 || nb > 64) return 1;
    BlockwiseSpFilter<half> f;
    fill(f, F, R * S * C, brow, nnzb, indptr, indices, values, perm);
    f.F = F; f.C = C; f.R = R; f.S = S;
    f.transform_and_sync_device();
    std::vector<SpconvBlockwiseOpState> st;
    for (int i = 0; i < nb; ++i) {
        st.push_back(kConv[cfg].init(f, Bn, H, W, stride, (half*)ifmap_dev[i], (half*)ofmap_dev[i]));
        if (!st.back().initSuccess) return 2;
    }
    int i = 0;
    *ms = time_launches([&] { kConv[cfg].exec(st[i], 0); i = (i + 1) % nb; }, warmup, repeat);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

}  // extern "C"
