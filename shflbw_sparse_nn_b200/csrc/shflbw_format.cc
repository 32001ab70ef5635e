// Host side of the Shfl-BW format: seeded builder, text dump/load, validation and the
// host images that shflbw_matrix_to_device uploads.  Pure C++ (no CUDA calls).
//
// Reference behaviour reproduced here (paths relative to the reference project):
//   block_sparse/util/random_mask.cc:10-67          seeded block mask
//   block_sparse/spmm/blockwise_format.h:70-123     init_random (permutation, values, config)
//   block_sparse/spmm/blockwise_format.h:125-198    dump / load text format
//   block_sparse/spmm/blockwise_format.h:206-228    meta image [indptr|indices*bcol|perm], pad 8
//   block_sparse/spconv/blockwise_format.h:29-52    filter view F x (R*S*C)
// Bit-exactness of the mask, the permutation and the INT9 values rests on using the same
// standard-library calls in the same order (std::shuffle with std::default_random_engine,
// std::rand); GNU libstdc++/glibc results are pinned by the reference's example/mtx_dump.txt.

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <new>
#include <numeric>
#include <random>
#include <sstream>

#include "shflbw_internal.hpp"

namespace shflbw {

float half_bits_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu, man = h & 0x3ffu, bits;
    if (exp == 0x1f) {
        bits = sign | 0x7f800000u | (man << 13);
    } else if (exp != 0) {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    } else if (man == 0) {
        bits = sign;
    } else {
        int lead = 0;
        while (!(man & 0x400u)) { man <<= 1; ++lead; }
        bits = sign | ((uint32_t)(113 - lead) << 23) | ((man & 0x3ffu) << 13);
    }
    float f;
    std::memcpy(&f, &bits, sizeof f);
    return f;
}

uint16_t float_to_half_bits(float f) {
    uint32_t x;
    std::memcpy(&x, &f, sizeof x);
    const uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    x &= 0x7fffffffu;
    if (x > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);       // NaN
    if (x >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);      // overflow -> inf
    if (x < 0x33000001u) return sign;                             // underflow -> 0
    const int e = (int)(x >> 23) - 127;
    const uint32_t man = (x & 0x7fffffu) | 0x800000u;
    const int shift = e < -14 ? 13 + (-14 - e) : 13;
    uint32_t q = man >> shift;
    const uint32_t rem = man & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) ++q;
    const uint32_t body = e < -14 ? q : ((uint32_t)(e + 15) << 10) + (q - 0x400u);
    return (uint16_t)(sign | body);
}

static inline uint64_t splitmix64(uint64_t z) {
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

uint16_t uniform_half(uint64_t stream, uint64_t index) {
    const uint64_t r = splitmix64((stream << 32) + index);
    const float u = (float)(r >> 40) * (1.0f / 16777216.0f);  // 24 bits -> [0, 1)
    return float_to_half_bits(2.0f * u - 1.0f);
}

int validate(const shflbw_matrix& m) {
    if (m.nrow <= 0 || m.ncol <= 0 || m.brow <= 0 || m.bcol <= 0) return SHFLBW_ERR_BAD_FORMAT;
    if (m.nrow % m.brow || m.ncol % m.bcol) return SHFLBW_ERR_BAD_FORMAT;
    const int X = m.nrow / m.brow, Y = m.ncol / m.bcol;
    if ((int)m.indptr.size() != X + 1 || m.indptr[0] != 0 || m.indptr[X] != m.nnzb)
        return SHFLBW_ERR_BAD_FORMAT;
    if ((int)m.indices.size() != m.nnzb || m.values.size() != (size_t)m.nnzb * m.brow * m.bcol)
        return SHFLBW_ERR_BAD_FORMAT;
    for (int i = 0; i < X; ++i) {
        if (m.indptr[i + 1] < m.indptr[i]) return SHFLBW_ERR_BAD_FORMAT;
        for (int p = m.indptr[i]; p < m.indptr[i + 1]; ++p) {
            const int c = m.indices[p];
            if (c < 0 || c >= Y) return SHFLBW_ERR_BAD_FORMAT;  // block-column units
            if (p > m.indptr[i] && c <= m.indices[p - 1]) return SHFLBW_ERR_BAD_FORMAT;
        }
    }
    if (m.row_permute) {
        if ((int)m.row_permute_ids.size() != m.nrow) return SHFLBW_ERR_BAD_FORMAT;
        std::vector<char> seen(m.nrow, 0);
        for (int v : m.row_permute_ids) {
            if (v < 0 || v >= m.nrow || seen[v]) return SHFLBW_ERR_BAD_FORMAT;
            seen[v] = 1;
        }
    } else if (!m.row_permute_ids.empty()) {
        return SHFLBW_ERR_BAD_FORMAT;
    }
    if (m.is_filter && (m.F != m.nrow || (int64_t)m.R * m.S * m.C != m.ncol))
        return SHFLBW_ERR_BAD_FORMAT;
    return SHFLBW_OK;
}

// "nrow ncol brow bcol density seed (non-)row-permute " -- blockwise_format.h:105-114;
// filters: "F R S C brow bcol density seed (non-)filter-permute " -- spconv/blockwise_format.h:41-51.
void build_config_str(shflbw_matrix& m) {
    std::stringstream s;
    if (m.is_filter) {
        s << m.F << " " << m.R << " " << m.S << " " << m.C << " " << m.brow << " " << m.bcol << " "
          << m.density << " " << m.seed << " " << (m.row_permute ? "filter-permute " : "non-filter-permute ");
    } else {
        s << m.nrow << " " << m.ncol << " " << m.brow << " " << m.bcol << " " << m.density << " "
          << m.seed << " " << (m.row_permute ? "row-permute " : "non-row-permute ");
    }
    m.config_str = s.str();
}

void build_host_images(shflbw_matrix& m) {
    const int X = m.nrow / m.brow;
    auto up = [](size_t v, size_t a) { return (v + a - 1) / a * a; };
    // Reference-compatible meta image.
    const size_t s0 = up(m.indptr.size(), 8), s1 = up(m.indices.size(), 8),
                 s2 = up(m.row_permute_ids.size(), 8);
    m.meta_h.assign(s0 + s1 + s2, 0);
    std::copy(m.indptr.begin(), m.indptr.end(), m.meta_h.begin());
    for (size_t t = 0; t < m.indices.size(); ++t) m.meta_h[s0 + t] = m.indices[t] * m.bcol;
    std::copy(m.row_permute_ids.begin(), m.row_permute_ids.end(), m.meta_h.begin() + s0 + s1);

    // Kernel image: per row block, column list padded to a multiple of kShflbwKPad.  A
    // padding column repeats the block's last real column (a valid, already-fetched row of
    // the dense operand) and carries zero values, so it contributes exactly 0.  256 slack
    // rows (zero values, column 0) follow the last block so a full-stage read past the end
    // stays inside the allocation.
    // A brow x bcol block is bcol adjacent columns that share the row block, and its values
    // are stored column by column (blockwise_format.h:286-297: a = values[p*brow*bcol +
    // kk*brow + mm], column indices[p]*bcol + kk).  The image lists those bcol columns one
    // after the other, so the kernels see the brow x 1 layout whatever bcol is.
    const size_t bc = (size_t)m.bcol;
    m.kptr.assign(X + 1, 0);
    size_t rows = 0;
    for (int i = 0; i < X; ++i) {
        m.kptr[i] = (int)rows;
        rows += up((size_t)(m.indptr[i + 1] - m.indptr[i]) * bc, kShflbwKPad);
    }
    m.kptr[X] = (int)rows;
    const size_t tail = 256;  // slack rows, zero values / index 0
    m.kidx.assign(rows + tail, 0);
    m.kval.assign((rows + tail) * m.brow, 0);
    for (int i = 0; i < X; ++i) {
        const int b = m.indptr[i], e = m.indptr[i + 1];
        size_t r = (size_t)m.kptr[i];
        for (int p = b; p < e; ++p) {
            for (size_t kk = 0; kk < bc; ++kk, ++r) {
                m.kidx[r] = m.indices[p] * m.bcol + (int)kk;
                const uint16_t* col = &m.values[((size_t)p * bc + kk) * m.brow];
                for (int j = 0; j < m.brow; ++j) m.kval[kval_index(m.brow, r, j)] = col[j];
            }
        }
        for (; r < (size_t)m.kptr[i + 1]; ++r) m.kidx[r] = e > b ? m.indices[e - 1] * m.bcol + m.bcol - 1 : 0;
    }
    // Filters: the implicit-GEMM gather wants (channel, tap row, tap column) of every column
    // id; decoding once here removes three integer divisions per row from the kernel.
    m.kcrs.clear();
    if (m.is_filter && m.C > 0 && m.C < 65536 && m.R < 256 && m.S < 256) {
        m.kcrs.resize(m.kidx.size());
        for (size_t r = 0; r < m.kidx.size(); ++r) {
            const int k = m.kidx[r], c = k % m.C, rs = k / m.C;
            m.kcrs[r] = c | ((rs / m.S) << 16) | ((rs % m.S) << 24);
        }
    }
}

// Mask + permutation + values.  Same RNG call sequence as the reference:
//   engine(seed) shuffle of iota(X*Y) -> per-block counts via id % X   (random_mask.cc:20-29)
//   engine(seed+i+1) shuffle of iota(Y) per row block, prefix sorted   (random_mask.cc:31-44)
//   engine(seed) shuffle of iota(nrow) for the permutation             (blockwise_format.h:89-95)
//   rand() % 9 - 4 per value                                           (blockwise_format.h:99-102)
static void fill_random(shflbw_matrix& m, float requested_density, int value_mode) {
    const int X = m.nrow / m.brow, Y = m.ncol / m.bcol;
    m.nnzb = (int)std::round(requested_density * X * Y / 1);
    std::vector<int> cell((size_t)X * Y);
    std::iota(cell.begin(), cell.end(), 0);
    std::shuffle(cell.begin(), cell.end(), std::default_random_engine(m.seed));
    std::vector<int> per_block(X, 0);
    for (int t = 0; t < m.nnzb; ++t) per_block[cell[t] % X]++;

    m.indptr.assign(X + 1, 0);
    m.indices.clear();
    m.indices.reserve(m.nnzb);
    std::vector<int> cols(Y);
    for (int i = 0; i < X; ++i) {
        std::iota(cols.begin(), cols.end(), 0);
        std::shuffle(cols.begin(), cols.end(), std::default_random_engine(m.seed + i + 1));
        std::sort(cols.begin(), cols.begin() + per_block[i]);
        m.indices.insert(m.indices.end(), cols.begin(), cols.begin() + per_block[i]);
        m.indptr[i + 1] = (int)m.indices.size();
    }
    m.density = (float)m.nnzb / X / Y;

    m.row_permute_ids.clear();
    if (m.row_permute) {
        m.row_permute_ids.resize(m.nrow);
        std::iota(m.row_permute_ids.begin(), m.row_permute_ids.end(), 0);
        std::shuffle(m.row_permute_ids.begin(), m.row_permute_ids.end(),
                     std::default_random_engine(m.seed));
    }

    m.values.resize((size_t)m.nnzb * m.brow * m.bcol);
    if (value_mode == SHFLBW_VALUES_INT9_LIBC) {
        for (auto& v : m.values) v = float_to_half_bits((float)(std::rand() % 9 - 4));
    } else {
        for (size_t t = 0; t < m.values.size(); ++t) m.values[t] = uniform_half(m.seed, t);
    }
}

static int parse_text(std::istream& in, shflbw_matrix& m) {
    int perm_flag = 0;
    if (!(in >> m.nrow >> m.ncol >> m.nnzb >> m.brow >> m.bcol >> perm_flag)) return SHFLBW_ERR_BAD_FORMAT;
    if (m.nrow <= 0 || m.ncol <= 0 || m.brow <= 0 || m.bcol <= 0 || m.nnzb < 0 || m.nrow % m.brow || m.ncol % m.bcol)
        return SHFLBW_ERR_BAD_FORMAT;
    m.row_permute = perm_flag != 0;
    m.indptr.resize(m.nrow / m.brow + 1);
    for (auto& v : m.indptr) if (!(in >> v)) return SHFLBW_ERR_BAD_FORMAT;
    m.indices.resize(m.nnzb);
    for (auto& v : m.indices) if (!(in >> v)) return SHFLBW_ERR_BAD_FORMAT;
    m.values.resize((size_t)m.nnzb * m.brow * m.bcol);
    for (auto& v : m.values) {
        float y;
        if (!(in >> y)) return SHFLBW_ERR_BAD_FORMAT;
        v = float_to_half_bits(y);
    }
    m.row_permute_ids.clear();
    if (m.row_permute) {
        m.row_permute_ids.resize(m.nrow);
        for (auto& v : m.row_permute_ids) if (!(in >> v)) return SHFLBW_ERR_BAD_FORMAT;
    }
    m.density = (float)m.nnzb / (m.nrow / m.brow) / (m.ncol / m.bcol);
    m.seed = 0;
    return validate(m);
}

static std::string dump_to_string(const shflbw_matrix& m) {
    std::ostringstream out;
    out << m.nrow << "\n" << m.ncol << "\n" << m.nnzb << "\n" << m.brow << "\n" << m.bcol << "\n"
        << (m.row_permute ? 1 : 0) << "\n";
    for (int v : m.indptr) out << v << " ";
    out << "\n";
    for (int v : m.indices) out << v << " ";
    out << "\n";
    for (uint16_t v : m.values) out << half_bits_to_float(v) << " ";  // default float formatting
    out << "\n";
    if (m.row_permute) {
        for (int v : m.row_permute_ids) out << v << " ";
        out << "\n";
    }
    return out.str();
}

}  // namespace shflbw

using namespace shflbw;

extern "C" {

const char* shflbw_strerror(int status) {
    switch (status) {
        case SHFLBW_OK: return "ok";
        case SHFLBW_ERR_INVALID_ARG: return "invalid argument";
        case SHFLBW_ERR_BAD_FORMAT: return "malformed Shfl-BW matrix";
        case SHFLBW_ERR_UNSUPPORTED: return "shape outside the supported contract";
        case SHFLBW_ERR_CUDA: return "CUDA runtime error";
        case SHFLBW_ERR_NOT_ON_DEVICE: return "matrix not uploaded (call shflbw_matrix_to_device)";
        case SHFLBW_ERR_DEVICE_TIMEOUT: return "a bounded in-kernel wait timed out";
        case SHFLBW_ERR_IO: return "file I/O error";
        case SHFLBW_ERR_TOO_LARGE: return "request exceeds a fixed built-in capacity";
        default: return "unknown status";
    }
}

int shflbw_abi_version(void) { return 1; }

int shflbw_matrix_create_random(int nrow, int ncol, int brow, int bcol, float density,
                                int row_permute, unsigned seed, int value_mode,
                                shflbw_matrix_t** out) {
    if (!out) return SHFLBW_ERR_INVALID_ARG;
    *out = nullptr;
    if (nrow <= 0 || ncol <= 0 || brow <= 0 || bcol <= 0 || !(density >= 0.f) || density > 1.f)
        return SHFLBW_ERR_INVALID_ARG;
    if (value_mode != SHFLBW_VALUES_INT9_LIBC && value_mode != SHFLBW_VALUES_UNIFORM)
        return SHFLBW_ERR_INVALID_ARG;
    // reference: assert(nrow % brow == 0); assert(ncol % bcol == 0)
    if (nrow % brow || ncol % bcol) return SHFLBW_ERR_UNSUPPORTED;
    auto* m = new (std::nothrow) shflbw_matrix();
    if (!m) return SHFLBW_ERR_INVALID_ARG;
    m->nrow = nrow; m->ncol = ncol; m->brow = brow; m->bcol = bcol;
    m->seed = seed; m->row_permute = row_permute != 0;
    fill_random(*m, density, value_mode);
    build_config_str(*m);
    *out = m;
    return SHFLBW_OK;
}

int shflbw_filter_create_random(int F, int R, int S, int C, int brow, int bcol, float density,
                                int filter_permute, unsigned seed, int value_mode,
                                shflbw_matrix_t** out) {
    if (F <= 0 || R <= 0 || S <= 0 || C <= 0) return SHFLBW_ERR_INVALID_ARG;
    int rc = shflbw_matrix_create_random(F, R * S * C, brow, bcol, density, filter_permute, seed,
                                         value_mode, out);
    if (rc != SHFLBW_OK) return rc;
    return shflbw_matrix_set_filter_shape(*out, F, R, S, C);
}

int shflbw_matrix_set_filter_shape(shflbw_matrix_t* m, int F, int R, int S, int C) {
    if (!m || F <= 0 || R <= 0 || S <= 0 || C <= 0) return SHFLBW_ERR_INVALID_ARG;
    if (F != m->nrow || (int64_t)R * S * C != m->ncol) return SHFLBW_ERR_BAD_FORMAT;
    m->is_filter = true; m->F = F; m->R = R; m->S = S; m->C = C;
    build_config_str(*m);
    return SHFLBW_OK;
}

int shflbw_matrix_create_from_block_arrays(int nrow, int ncol, int brow, int bcol, int nnzb, const int* indptr,
                                           const int* indices, const uint16_t* values, const int* perm,
                                           shflbw_matrix_t** out) {
    if (!out) return SHFLBW_ERR_INVALID_ARG;
    *out = nullptr;
    if (nrow <= 0 || ncol <= 0 || brow <= 0 || bcol <= 0 || nnzb < 0 || !indptr ||
        (nnzb > 0 && (!indices || !values)))
        return SHFLBW_ERR_INVALID_ARG;
    if (nrow % brow || ncol % bcol) return SHFLBW_ERR_UNSUPPORTED;
    auto* m = new (std::nothrow) shflbw_matrix();
    if (!m) return SHFLBW_ERR_INVALID_ARG;
    m->nrow = nrow; m->ncol = ncol; m->brow = brow; m->bcol = bcol; m->nnzb = nnzb;
    m->row_permute = perm != nullptr;
    m->indptr.assign(indptr, indptr + nrow / brow + 1);
    m->indices.assign(indices, indices + nnzb);
    m->values.assign(values, values + (size_t)nnzb * brow * bcol);
    if (perm) m->row_permute_ids.assign(perm, perm + nrow);
    m->density = (float)nnzb / (nrow / brow) / (ncol / bcol);
    int rc = validate(*m);
    if (rc != SHFLBW_OK) { delete m; return rc; }
    build_config_str(*m);
    *out = m;
    return SHFLBW_OK;
}

int shflbw_matrix_create_from_arrays(int nrow, int ncol, int brow, int nnzb, const int* indptr,
                                     const int* indices, const uint16_t* values, const int* perm,
                                     shflbw_matrix_t** out) {
    return shflbw_matrix_create_from_block_arrays(nrow, ncol, brow, 1, nnzb, indptr, indices, values, perm, out);
}

int shflbw_filter_fold_input_order(const shflbw_matrix_t* f, const shflbw_matrix_t* producer,
                                   shflbw_matrix_t** out) {
    if (!out) return SHFLBW_ERR_INVALID_ARG;
    *out = nullptr;
    if (!f || !producer || !f->is_filter) return SHFLBW_ERR_INVALID_ARG;
    if (f->C != producer->nrow) return SHFLBW_ERR_BAD_FORMAT;
    if (f->bcol != 1) return SHFLBW_ERR_UNSUPPORTED;  // a reordered channel list breaks up wider blocks
    // stored position of every logical channel of the producer's output
    std::vector<int> where(f->C);
    for (int p = 0; p < f->C; ++p) where[producer->row_permute ? producer->row_permute_ids[p] : p] = p;
    // Column k = (r*S + s)*C + c keeps its tap and gets channel where[c]; every row block's
    // list is sorted again (the format's invariant) and the value panels follow their columns.
    std::vector<int> indices(f->indices.size());
    std::vector<uint16_t> values(f->values.size());
    std::vector<std::pair<int, int>> order;
    const int X = f->nrow / f->brow;
    for (int i = 0; i < X; ++i) {
        const int b = f->indptr[i], e = f->indptr[i + 1];
        order.clear();
        for (int p = b; p < e; ++p) {
            const int k = f->indices[p];
            order.emplace_back((k / f->C) * f->C + where[k % f->C], p);
        }
        std::sort(order.begin(), order.end());
        for (int j = 0; j < e - b; ++j) {
            indices[b + j] = order[j].first;
            std::memcpy(&values[(size_t)(b + j) * f->brow], &f->values[(size_t)order[j].second * f->brow],
                        (size_t)f->brow * 2);
        }
    }
    int rc = shflbw_matrix_create_from_arrays(f->nrow, f->ncol, f->brow, f->nnzb, f->indptr.data(), indices.data(),
                                              values.data(), f->row_permute ? f->row_permute_ids.data() : nullptr, out);
    if (rc != SHFLBW_OK) return rc;
    (*out)->seed = f->seed;
    return shflbw_matrix_set_filter_shape(*out, f->F, f->R, f->S, f->C);
}

int shflbw_matrix_load_text(const char* text, size_t len, shflbw_matrix_t** out) {
    if (!text || !out) return SHFLBW_ERR_INVALID_ARG;
    *out = nullptr;
    std::istringstream in(std::string(text, len));
    auto* m = new (std::nothrow) shflbw_matrix();
    if (!m) return SHFLBW_ERR_INVALID_ARG;
    int rc = parse_text(in, *m);
    if (rc != SHFLBW_OK) { delete m; return rc; }
    build_config_str(*m);
    *out = m;
    return SHFLBW_OK;
}

int shflbw_matrix_load_file(const char* path, shflbw_matrix_t** out) {
    if (!path || !out) return SHFLBW_ERR_INVALID_ARG;
    std::ifstream f(path, std::ios::binary);
    if (!f) return SHFLBW_ERR_IO;
    std::stringstream ss;
    ss << f.rdbuf();
    const std::string s = ss.str();
    return shflbw_matrix_load_text(s.data(), s.size(), out);
}

int shflbw_matrix_dump_text(const shflbw_matrix_t* m, char* buf, size_t cap, size_t* needed) {
    if (!m) return SHFLBW_ERR_INVALID_ARG;
    const std::string s = dump_to_string(*m);
    if (needed) *needed = s.size();
    if (buf && cap) std::memcpy(buf, s.data(), std::min(cap, s.size()));
    return SHFLBW_OK;
}

int shflbw_matrix_dump_file(const shflbw_matrix_t* m, const char* path) {
    if (!m || !path) return SHFLBW_ERR_INVALID_ARG;
    std::ofstream f(path, std::ios::binary);
    if (!f) return SHFLBW_ERR_IO;
    const std::string s = dump_to_string(*m);
    f.write(s.data(), (std::streamsize)s.size());
    return f ? SHFLBW_OK : SHFLBW_ERR_IO;
}

int shflbw_matrix_validate(const shflbw_matrix_t* m) { return m ? validate(*m) : SHFLBW_ERR_INVALID_ARG; }

int shflbw_matrix_clone(const shflbw_matrix_t* m, shflbw_matrix_t** out) {
    if (!m || !out) return SHFLBW_ERR_INVALID_ARG;
    auto* c = new shflbw_matrix(*m);
    // the copy owns nothing on any device
    c->device = -1;
    c->d_meta = c->d_val = nullptr;
    c->d_kptr = c->d_kidx = c->d_kcrs = c->d_perm = nullptr;
    c->d_status = nullptr;
    c->stage_in = c->stage_c = c->stage_out = c->conv_in = c->conv_out = nullptr;
    c->stage_in_bytes = c->stage_c_bytes = c->stage_out_bytes = c->conv_in_bytes = c->conv_out_bytes = 0;
    c->retired.clear();
    for (void*& st : c->host_streams) st = nullptr;
    for (void*& ev : c->host_events) ev = nullptr;
    *out = c;
    return SHFLBW_OK;
}

int shflbw_shard_range(long long total, int granule, int parts, int index, long long* begin, long long* count) {
    if (total < 0 || granule <= 0 || parts <= 0 || index < 0 || index >= parts || !begin || !count)
        return SHFLBW_ERR_INVALID_ARG;
    if (total % granule) return SHFLBW_ERR_UNSUPPORTED;
    const long long groups = total / granule, base = groups / parts, extra = groups % parts;
    *begin = ((long long)index * base + (index < extra ? index : extra)) * granule;
    *count = (base + (index < extra ? 1 : 0)) * granule;
    return SHFLBW_OK;
}

void shflbw_matrix_destroy(shflbw_matrix_t* m) {
    if (!m) return;
    drop_device_copy(*m);
    delete m;
}

int shflbw_matrix_nrow(const shflbw_matrix_t* m) { return m ? m->nrow : -1; }
int shflbw_matrix_ncol(const shflbw_matrix_t* m) { return m ? m->ncol : -1; }
int shflbw_matrix_nnzb(const shflbw_matrix_t* m) { return m ? m->nnzb : -1; }
int shflbw_matrix_brow(const shflbw_matrix_t* m) { return m ? m->brow : -1; }
int shflbw_matrix_bcol(const shflbw_matrix_t* m) { return m ? m->bcol : -1; }
int shflbw_matrix_row_permute(const shflbw_matrix_t* m) { return m ? (int)m->row_permute : -1; }
unsigned shflbw_matrix_seed(const shflbw_matrix_t* m) { return m ? m->seed : 0u; }
float shflbw_matrix_density(const shflbw_matrix_t* m) { return m ? m->density : -1.f; }
const char* shflbw_matrix_config_str(const shflbw_matrix_t* m) { return m ? m->config_str.c_str() : ""; }
int shflbw_matrix_filter_shape(const shflbw_matrix_t* m, int* F, int* R, int* S, int* C) {
    if (!m || !m->is_filter) return SHFLBW_ERR_INVALID_ARG;
    if (F) *F = m->F;
    if (R) *R = m->R;
    if (S) *S = m->S;
    if (C) *C = m->C;
    return SHFLBW_OK;
}
const int* shflbw_matrix_indptr(const shflbw_matrix_t* m) { return m ? m->indptr.data() : nullptr; }
const int* shflbw_matrix_indices(const shflbw_matrix_t* m) { return m ? m->indices.data() : nullptr; }
const uint16_t* shflbw_matrix_values(const shflbw_matrix_t* m) { return m ? m->values.data() : nullptr; }
const int* shflbw_matrix_row_permute_ids(const shflbw_matrix_t* m) {
    return (m && m->row_permute) ? m->row_permute_ids.data() : nullptr;
}
const int* shflbw_matrix_meta_image(const shflbw_matrix_t* m, size_t* n_int32) {
    if (!m) return nullptr;
    if (m->meta_h.empty()) build_host_images(*const_cast<shflbw_matrix_t*>(m));
    if (n_int32) *n_int32 = m->meta_h.size();
    return m->meta_h.data();
}

}  // extern "C"
