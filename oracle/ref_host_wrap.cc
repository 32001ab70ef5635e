// TEST INFRASTRUCTURE ONLY -- C entry points around the UNMODIFIED reference host code.
//
// This translation unit contains no algorithm of its own: it includes the reference's
// headers from the reference checkout (given with -I at build time; nothing is copied
// into this repository) and forwards to BlockwiseSpMatrix<half> / BlockwiseSpFilter<half>
// and get_host_reference.  It is built into oracle/_ref/libshflbw_ref_host.so by
// oracle/Makefile and is used (a) to pin oracle/shflbw_oracle.cc, (b) to generate the
// fixtures under tests/golden/, (c) as the timed CPU baseline of the benchmark.
//
// Reference code reached from here:
//   block_sparse/spmm/blockwise_format.h:70-123 (init_random), :125-149 (dump),
//   :151-198 (load), :200-266 (transform_and_sync_device), :268-311 (get_host_reference)
//   block_sparse/spconv/blockwise_format.h:29-52, :54-132
//   block_sparse/util/random_mask.cc:10-67

#include <cstdint>
#include <cstring>
#include <sstream>
#include <string>
#include <vector>

#include <cuda_fp16.h>
#include "block_sparse/spconv/blockwise_format.h"
#include "block_sparse/spmm/blockwise_format.h"

namespace {
template <class M>
void fill_from_arrays(M& m, int nrow, int ncol, int brow, int nnzb, const int* indptr,
                      const int* indices, const uint16_t* values, const int* perm, int bcol = 1) {
    m.nrow = nrow; m.ncol = ncol; m.brow = brow; m.bcol = bcol; m.nnzb = nnzb;
    m.seed = 0; m.row_permute = perm != nullptr;
    m.density = (float)nnzb / (nrow / brow) / (ncol / bcol);
    m.indptr.assign(indptr, indptr + nrow / brow + 1);
    m.indices.assign(indices, indices + nnzb);
    m.values.resize((size_t)nnzb * brow * bcol);
    std::memcpy((void*)m.values.data(), values, (size_t)nnzb * brow * bcol * 2);
    if (perm) m.row_permute_ids.assign(perm, perm + nrow); else m.row_permute_ids.clear();
    m.initialized = true;
}
std::vector<half> as_half(const uint16_t* p, size_t n) {
    std::vector<half> v(n);
    std::memcpy((void*)v.data(), p, n * 2);
    return v;
}
}  // namespace

extern "C" {

void* ref_matrix_init_random(int nrow, int ncol, int brow, int bcol, float density,
                             int row_permute, unsigned seed) {
    auto* m = new BlockwiseSpMatrix<half>();
    m->init_random(nrow, ncol, brow, bcol, density, row_permute != 0, seed);
    return m;
}
void* ref_filter_init_random(int F, int R, int S, int C, int brow, int bcol, float density,
                             int permute, unsigned seed) {
    auto* m = new BlockwiseSpFilter<half>();
    m->init_random(F, R, S, C, brow, bcol, density, permute != 0, seed);
    return static_cast<BlockwiseSpMatrix<half>*>(m);
}
void ref_matrix_free(void* h) { delete static_cast<BlockwiseSpMatrix<half>*>(h); }
int ref_matrix_nnzb(void* h) { return static_cast<BlockwiseSpMatrix<half>*>(h)->nnzb; }
float ref_matrix_density(void* h) { return static_cast<BlockwiseSpMatrix<half>*>(h)->density; }
int ref_matrix_config_str(void* h, char* buf, int cap) {
    auto& s = static_cast<BlockwiseSpMatrix<half>*>(h)->config_str;
    if (buf && cap > 0) { std::strncpy(buf, s.c_str(), cap - 1); buf[cap - 1] = 0; }
    return (int)s.size();
}
void ref_matrix_arrays(void* h, int* indptr, int* indices, uint16_t* values, int* perm) {
    auto* m = static_cast<BlockwiseSpMatrix<half>*>(h);
    if (indptr) std::memcpy(indptr, m->indptr.data(), m->indptr.size() * 4);
    if (indices) std::memcpy(indices, m->indices.data(), m->indices.size() * 4);
    if (values) std::memcpy(values, (const void*)m->values.data(), m->values.size() * 2);
    if (perm && m->row_permute) std::memcpy(perm, m->row_permute_ids.data(), m->row_permute_ids.size() * 4);
}
int64_t ref_matrix_dump(void* h, char* buf, int64_t cap) {
    std::ostringstream out;
    static_cast<BlockwiseSpMatrix<half>*>(h)->dump(out);
    std::string s = out.str();
    if (buf && cap > 0) std::memcpy(buf, s.data(), (size_t)std::min<int64_t>(cap, (int64_t)s.size()));
    return (int64_t)s.size();
}
void* ref_matrix_load(const char* text, int64_t len) {
    std::istringstream in(std::string(text, (size_t)len));
    auto* m = new BlockwiseSpMatrix<half>();
    m->seed = 0;
    m->load(in);
    return m;
}
// Needs a GPU (cudaMalloc inside): returns the int32 meta image the reference uploads.
int64_t ref_matrix_meta_image(void* h, int* out, int64_t cap_ints) {
    auto* m = static_cast<BlockwiseSpMatrix<half>*>(h);
    m->transform_and_sync_device();
    int64_t n = (int64_t)m->meta_h.size() / 4;
    if (out) std::memcpy(out, m->meta_h.data(), (size_t)std::min<int64_t>(n, cap_ints) * 4);
    return n;
}

// Unmodified get_host_reference on caller-provided arrays (single-threaded, as shipped);
// brow x bcol blocks, indices in units of bcol columns.
void ref_spmm_host_reference_blocks(int M, int K, int N, int brow, int bcol, int nnzb, const int* indptr,
                                    const int* indices, const uint16_t* values, const int* perm,
                                    const uint16_t* B, float alpha, const uint16_t* C, float beta,
                                    float* D_ref) {
    BlockwiseSpMatrix<half> m;
    fill_from_arrays(m, M, K, brow, nnzb, indptr, indices, values, perm, bcol);
    std::vector<half> Bh = as_half(B, (size_t)K * N);
    std::vector<half> Ch((size_t)M * N);
    if (C) std::memcpy((void*)Ch.data(), C, (size_t)M * N * 2);
    else for (auto& c : Ch) c = __float2half(0.f);
    std::vector<float> D((size_t)M * N);
    get_host_reference<half>(m, N, Bh, alpha, Ch, beta, D);
    std::memcpy(D_ref, D.data(), D.size() * 4);
}

void ref_spmm_host_reference(int M, int K, int N, int brow, int nnzb, const int* indptr,
                             const int* indices, const uint16_t* values, const int* perm,
                             const uint16_t* B, float alpha, const uint16_t* C, float beta,
                             float* D_ref) {
    ref_spmm_host_reference_blocks(M, K, N, brow, 1, nnzb, indptr, indices, values, perm, B, alpha, C, beta, D_ref);
}

// Unmodified conv get_host_reference; feature maps in the reference's own layouts
// (input [C][H][W][B], output [F][H][W][B]).
void ref_spconv_host_reference_blocks(int Bn, int H, int W, int C, int F, int R, int S, int stride,
                                      int brow, int bcol, int nnzb, const int* indptr, const int* indices,
                                      const uint16_t* values, const int* perm, const uint16_t* ifmap,
                                      float* ofmap_ref) {
    BlockwiseSpFilter<half> f;
    fill_from_arrays(f, F, R * S * C, brow, nnzb, indptr, indices, values, perm, bcol);
    f.F = F; f.C = C; f.R = R; f.S = S;
    std::vector<half> X = as_half(ifmap, (size_t)Bn * H * W * C);
    std::vector<float> O((size_t)Bn * H * W * F);
    get_host_reference<half>(f, Bn, H, W, stride, X, O, filter_channel_first);
    std::memcpy(ofmap_ref, O.data(), O.size() * 4);
}

void ref_spconv_host_reference(int Bn, int H, int W, int C, int F, int R, int S, int stride,
                               int brow, int nnzb, const int* indptr, const int* indices,
                               const uint16_t* values, const int* perm, const uint16_t* ifmap,
                               float* ofmap_ref) {
    ref_spconv_host_reference_blocks(Bn, H, W, C, F, R, S, stride, brow, 1, nnzb, indptr, indices, values, perm,
                                     ifmap, ofmap_ref);
}

}  // extern "C"
