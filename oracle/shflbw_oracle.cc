// TEST INFRASTRUCTURE ONLY -- CPU oracle for the Shfl-BW block-sparse path.
//
// This file restates, in plain host C++, what the reference's host code computes
// for the path: the seeded Shfl-BW mask, the row permutation, the value fill, the
// text dump, the device meta image, and the fp32 CPU results for SpMM and SpConv.
// Each function cites the reference file:line it follows.  It is a checker: only
// tests, the smoke check and the benchmark's CPU-baseline leg may load it.  The
// product library never links or calls it.
//
// Parity status: PINNED.  tests/test_oracle_pins.py checks this restatement against
//   (1) the reference's own golden dump example/mtx_dump.txt (via its SHA-256 and
//       leading fields committed under tests/golden/), byte for byte, and
//   (2) outputs of the unmodified reference compiled from its own sources into
//       oracle/_ref/ (mask, permutation, values, dump text, meta image, SpMM and
//       SpConv CPU results), when that build is present.
//
// Randomness comes from the C++/C standard library exactly as in the reference
// (std::shuffle + std::default_random_engine, std::rand); results are pinned for
// GNU libstdc++/glibc by the golden dump.
//
// Build: see oracle/Makefile (g++ -O2 -ffp-contract=off; no CUDA needed).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <numeric>
#include <random>
#include <sstream>
#include <string>
#include <thread>
#include <vector>

namespace {

// IEEE binary16 -> binary32, exact.
inline float h2f(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {  // subnormal: renormalise
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    std::memcpy(&f, &bits, 4);
    return f;
}

// binary32 -> binary16, round to nearest even (what static_cast<half>(float) does).
inline uint16_t f2h(float f) {
    uint32_t x;
    std::memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) return (uint16_t)(sign | 0x7c00u | (x > 0x7f800000u ? 0x200u : 0));
    if (x >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);  // rounds to inf
    if (x < 0x33000001u) return (uint16_t)sign;               // rounds to zero
    int e = (int)(x >> 23) - 127;
    uint32_t man = (x & 0x7fffffu) | 0x800000u;
    int shift = (e < -14) ? (13 + (-14 - e)) : 13;
    uint32_t half_man = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (half_man & 1))) ++half_man;
    uint32_t out;
    if (e < -14) out = half_man;  // subnormal (may carry into the smallest normal)
    else out = ((uint32_t)(e + 15) << 10) + (half_man - 0x400u);
    return (uint16_t)(sign | out);
}

template <class F>
void parallel_rows(int n, int nthreads, F fn) {
    if (nthreads <= 1 || n <= 1) { fn(0, n); return; }
    nthreads = std::min(nthreads, n);
    std::vector<std::thread> pool;
    for (int t = 0; t < nthreads; ++t) {
        int lo = (int)((int64_t)n * t / nthreads), hi = (int)((int64_t)n * (t + 1) / nthreads);
        pool.emplace_back([=] { fn(lo, hi); });
    }
    for (auto& th : pool) th.join();
}

}  // namespace

extern "C" {

// Seeded block mask.  Follows block_sparse/util/random_mask.cc:10-57 with
// block_divisor = block_padding = 1 (the only values callers pass, :59-67):
//   X = nrow/brow, Y = ncol/bcol, nnzb = round(density*X*Y)                    (:15-18)
//   shuffle iota(X*Y) with engine(seed); the first nnzb ids vote id % X        (:20-29)
//   row block i: shuffle iota(Y) with engine(seed+i+1), keep first count, sort (:31-44)
// indptr has X+1 entries, indices has nnzb entries (caller provides X*Y capacity).
int orc_random_mask(int nrow, int ncol, int brow, int bcol, float density, unsigned seed,
                    int* nnzb_out, int* indptr, int* indices) {
    if (brow <= 0 || bcol <= 0 || nrow % brow || ncol % bcol) return 1;
    const int X = nrow / brow, Y = ncol / bcol;
    const int nnzb = (int)(std::round(density * X * Y / 1));
    std::vector<int> ids((size_t)X * Y);
    std::iota(ids.begin(), ids.end(), 0);
    std::shuffle(ids.begin(), ids.end(), std::default_random_engine(seed));
    std::vector<int> count(X, 0);
    for (int t = 0; t < nnzb; ++t) count[ids[t] % X] += 1;
    int off = 0;
    std::vector<int> cols(Y);
    for (int i = 0; i < X; ++i) {
        std::iota(cols.begin(), cols.end(), 0);
        std::shuffle(cols.begin(), cols.end(), std::default_random_engine(seed + i + 1));
        std::sort(cols.begin(), cols.begin() + count[i]);
        indptr[i] = off;
        for (int t = 0; t < count[i]; ++t) indices[off + t] = cols[t];
        off += count[i];
    }
    indptr[X] = off;
    *nnzb_out = nnzb;
    return off == nnzb ? 0 : 2;
}

// Row permutation: shuffle(iota(nrow), default_random_engine(seed)).
// Follows block_sparse/spmm/blockwise_format.h:89-95.
void orc_row_permutation(int nrow, unsigned seed, int* perm) {
    std::vector<int> p(nrow);
    std::iota(p.begin(), p.end(), 0);
    std::shuffle(p.begin(), p.end(), std::default_random_engine(seed));
    std::copy(p.begin(), p.end(), perm);
}

// Value fill half(float(rand() % 9 - 4)) drawing from the process-wide libc stream.
// Follows block_sparse/spmm/blockwise_format.h:99-102 and cuda_array.h:59-67.
void orc_fill_int9(int64_t n, uint16_t* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = f2h((float)(std::rand() % 9 - 4));
}

// Re-seed libc rand(); srand(1) is the state of a fresh process.
void orc_srand(unsigned s) { std::srand(s); }

// Achieved density as stored by the reference: (float)nnzb / X / Y.
// Follows block_sparse/spmm/blockwise_format.h:87.
float orc_achieved_density(int nrow, int ncol, int brow, int bcol, int nnzb) {
    return (float)nnzb / (nrow / brow) / (ncol / bcol);
}

// Text serialisation.  Follows block_sparse/spmm/blockwise_format.h:125-149:
// six scalar lines, then indptr, indices, values (as float text) and, when permuted,
// the permutation; every number followed by one blank, every array by a newline.
// Returns the byte count; writes at most cap bytes to buf (buf may be null to size).
int64_t orc_dump_text(int nrow, int ncol, int nnzb, int brow, int bcol, int row_permute,
                      const int* indptr, const int* indices, const uint16_t* values,
                      const int* perm, char* buf, int64_t cap) {
    std::ostringstream out;
    out << nrow << std::endl << ncol << std::endl << nnzb << std::endl;
    out << brow << std::endl << bcol << std::endl << (row_permute ? true : false) << std::endl;
    for (int x = 0; x < nrow / brow + 1; ++x) out << indptr[x] << " ";
    out << std::endl;
    for (int x = 0; x < nnzb; ++x) out << indices[x] << " ";
    out << std::endl;
    for (int64_t x = 0; x < (int64_t)nnzb * brow * bcol; ++x) out << h2f(values[x]) << " ";
    out << std::endl;
    if (row_permute) {
        for (int x = 0; x < nrow; ++x) out << perm[x] << " ";
        out << std::endl;
    }
    const std::string s = out.str();
    if (buf && cap > 0) std::memcpy(buf, s.data(), (size_t)std::min<int64_t>(cap, (int64_t)s.size()));
    return (int64_t)s.size();
}

// Device meta image [indptr | indices*bcol | perm], each section zero-padded to a
// multiple of 8 int32.  Follows block_sparse/spmm/blockwise_format.h:206-228.
// Returns the number of int32 written (caller sizes out generously).
int64_t orc_meta_image(int n_indptr, const int* indptr, int nnzb, const int* indices, int bcol,
                       int n_perm, const int* perm, int* out) {
    auto up8 = [](int64_t v) { return (v + 7) / 8 * 8; };
    int64_t total = up8(n_indptr) + up8(nnzb) + up8(n_perm);
    std::fill(out, out + total, 0);
    int64_t off = 0;
    for (int i = 0; i < n_indptr; ++i) out[off + i] = indptr[i];
    off = up8(off + n_indptr);
    for (int i = 0; i < nnzb; ++i) out[off + i] = indices[i] * bcol;
    off = up8(off + nnzb);
    for (int i = 0; i < n_perm; ++i) out[off + i] = perm[i];
    return total;
}

// brow x bcol blocks as brow x 1 blocks.  Block p of a row block covers the bcol columns
// indices[p]*bcol + kk, kk = 0..bcol-1, and stores them column by column: value (mm, kk) at
// values[p*brow*bcol + kk*brow + mm] (block_sparse/spmm/blockwise_format.h:286-297, the same
// in block_sparse/spconv/blockwise_format.h:71-80).  Both host references add the products
// of a row in (p, kk) order, which is the order of the expanded column list, so the brow x 1
// functions below applied to the expanded arrays give the same fp32 sums.  indices1 and
// values1 hold nnzb*bcol and nnzb*bcol*brow entries.
void orc_expand_block_columns(int X, int brow, int bcol, const int* indptr, const int* indices,
                              const uint16_t* values, int* indptr1, int* indices1, uint16_t* values1) {
    for (int i = 0; i <= X; ++i) indptr1[i] = indptr[i] * bcol;
    for (int p = 0; p < indptr[X]; ++p)
        for (int kk = 0; kk < bcol; ++kk) {
            const size_t q = (size_t)p * bcol + kk;
            indices1[q] = indices[p] * bcol + kk;
            for (int mm = 0; mm < brow; ++mm) values1[q * brow + mm] = values[q * brow + mm];
        }
}

// fp32 CPU result of D = alpha * (A_sparse . B) + beta * C.
// Follows block_sparse/spmm/blockwise_format.h:268-311 (bcol == 1): every output
// element accumulates a*b in ascending non-zero-column order in fp32; the product
// is rounded before the add (build with -ffp-contract=off).  Rows may be split
// over threads: each output element is still summed by one thread in the same order.
void orc_spmm_ref(int M, int N, int brow, const int* indptr, const int* indices,
                  const uint16_t* values, const int* perm /*nullable*/, const uint16_t* B,
                  float alpha, const uint16_t* C /*nullable*/, float beta, float* D_ref,
                  int nthreads) {
    std::vector<float> Bf;  // converted once; conversion is exact
    int kmax = 0;
    const int X = M / brow;
    for (int p = 0; p < indptr[X]; ++p) kmax = std::max(kmax, indices[p] + 1);
    Bf.resize((size_t)kmax * N);
    for (size_t t = 0; t < Bf.size(); ++t) Bf[t] = h2f(B[t]);
    parallel_rows(M, nthreads, [&](int lo, int hi) {
        for (int row = lo; row < hi; ++row) {
            const int i = row / brow, mm = row % brow;
            const int dst = perm ? perm[row] : row;
            float* d = D_ref + (size_t)dst * N;
            for (int nn = 0; nn < N; ++nn) d[nn] = 0.f;
            for (int p = indptr[i]; p < indptr[i + 1]; ++p) {
                const float a = h2f(values[(size_t)p * brow + mm]);
                const float* b = Bf.data() + (size_t)indices[p] * N;
                for (int nn = 0; nn < N; ++nn) d[nn] += a * b[nn];
            }
            for (int nn = 0; nn < N; ++nn) {
                float c = C ? h2f(C[(size_t)dst * N + nn]) : 0.f;
                d[nn] = d[nn] * alpha + c * beta;
            }
        }
    });
}

// fp32 CPU result of the sparse convolution in the REFERENCE's layouts: input
// [C][H][W][B] (batch innermost), output [F][H][W][B], filter matrix F x (R*S*C)
// with k = (r*S+s)*C + c, pad R/2,S/2, and H,W used both as output size and as
// input bounds.  Follows block_sparse/spconv/blockwise_format.h:54-132.
void orc_spconv_ref_chwn(int Bn, int H, int W, int C, int F, int R, int S, int stride, int brow,
                         const int* indptr, const int* indices, const uint16_t* values,
                         const int* perm /*nullable*/, const uint16_t* ifmap, float* ofmap_ref,
                         int nthreads) {
    const int64_t npix = (int64_t)Bn * H * W;
    parallel_rows(F, nthreads, [&](int lo, int hi) {
        for (int row = lo; row < hi; ++row) {
            const int i = row / brow, x = row % brow;
            const int ff = perm ? perm[row] : row;
            float* o = ofmap_ref + (size_t)ff * npix;
            for (int64_t y = 0; y < npix; ++y) o[y] = 0.f;
            for (int p = indptr[i]; p < indptr[i + 1]; ++p) {
                const int k = indices[p];
                const int cc = k % C, ss = (k / C) % S, rr = (k / C) / S;
                const float w = h2f(values[(size_t)p * brow + x]);
                for (int64_t y = 0; y < npix; ++y) {
                    const int nn = (int)(y % Bn), wo = (int)((y / Bn) % W), ho = (int)((y / Bn) / W);
                    const int hi_ = ho * stride - R / 2 + rr, wi = wo * stride - S / 2 + ss;
                    float v = 0.f;
                    if (hi_ >= 0 && hi_ < H && wi >= 0 && wi < W)
                        v = h2f(ifmap[nn + ((size_t)wi + ((size_t)hi_ + (size_t)cc * H) * W) * Bn]);
                    o[y] += w * v;
                }
            }
        }
    });
}

// Same convolution with NHWC activations and the standard strided definition:
// input [B][Hin][Win][C], output [B][Ho][Wo][F], Ho = ceil(Hin/stride), pad R/2,S/2.
// Index semantics of the filter matrix and the permutation are those of
// block_sparse/spconv/blockwise_format.h:78-80, 96-99; only the activation layouts
// differ (pure data movement).  At stride 1 it equals orc_spconv_ref_chwn after
// transposing the feature maps; at stride>1 it equals it on ho<Ho, wo<Wo.
void orc_spconv_ref_nhwc(int Bn, int Hin, int Win, int C, int F, int R, int S, int stride, int brow,
                         const int* indptr, const int* indices, const uint16_t* values,
                         const int* perm /*nullable*/, const uint16_t* ifmap, float alpha,
                         float* ofmap_ref, int nthreads) {
    const int Ho = (Hin + stride - 1) / stride, Wo = (Win + stride - 1) / stride;
    const int64_t npix = (int64_t)Bn * Ho * Wo;
    std::vector<float> Xf((size_t)Bn * Hin * Win * C);
    for (size_t t = 0; t < Xf.size(); ++t) Xf[t] = h2f(ifmap[t]);
    parallel_rows(F, nthreads, [&](int lo, int hi) {
        std::vector<float> acc((size_t)npix);
        for (int row = lo; row < hi; ++row) {
            const int i = row / brow, x = row % brow;
            const int ff = perm ? perm[row] : row;
            std::fill(acc.begin(), acc.end(), 0.f);
            for (int p = indptr[i]; p < indptr[i + 1]; ++p) {
                const int k = indices[p];
                const int cc = k % C, ss = (k / C) % S, rr = (k / C) / S;
                const float w = h2f(values[(size_t)p * brow + x]);
                for (int nn = 0; nn < Bn; ++nn)
                    for (int ho = 0; ho < Ho; ++ho) {
                        const int hi_ = ho * stride - R / 2 + rr;
                        if (hi_ < 0 || hi_ >= Hin) continue;  // adds w*0 = 0 in the reference
                        for (int wo = 0; wo < Wo; ++wo) {
                            const int wi = wo * stride - S / 2 + ss;
                            if (wi < 0 || wi >= Win) continue;
                            acc[((size_t)nn * Ho + ho) * Wo + wo] +=
                                w * Xf[(((size_t)nn * Hin + hi_) * Win + wi) * C + cc];
                        }
                    }
            }
            for (int64_t y = 0; y < npix; ++y) ofmap_ref[(size_t)y * F + ff] = acc[(size_t)y] * alpha;
        }
    });
}

// The reference's acceptance rule: |ref - d| <= 1e-3 * |ref| for every element
// (block_sparse/test/test_util.spmm.h:8-30).  Returns the number of violations.
int64_t orc_check_equal_ref_rule(int64_t n, const uint16_t* res, const float* ref) {
    int64_t bad = 0;
    for (int64_t t = 0; t < n; ++t) {
        float d = h2f(res[t]);
        if (std::fabs(ref[t] - d) > 1e-3 * std::fabs(ref[t])) ++bad;
    }
    return bad;
}

}  // extern "C"
