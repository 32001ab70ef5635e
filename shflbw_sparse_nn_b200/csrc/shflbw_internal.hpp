// Internal definition of the opaque matrix handle and helpers shared by the host
// format code (shflbw_format.cc) and the CUDA glue (shflbw_capi.cu).
#pragma once

#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "shflbw.h"

// K padding of every row block's column list in the kernel image: one tcgen05.mma of
// kind::f16 consumes K = 16, so kernels never handle a ragged K tail.
constexpr int kShflbwKPad = 16;

// Kernel image of the value panels.  Element (padded row r, row-in-block m) lives at
// kval_index(V, r, m).  For V = 16 / 32 / 64 / 128 every group of 8 rows is stored in exactly the
// byte order the tensor-core operand tile has in shared memory (16-byte chunks XOR-swizzled by
// the row; 128-, 64- or 32-byte swizzle atoms), so a pipeline stage of the panel is ONE
// contiguous run that a bulk copy drops into place.  Other V: plain row-major.
#if defined(__CUDACC__)
#define SHFLBW_HD __host__ __device__
#else
#define SHFLBW_HD
#endif
SHFLBW_HD inline size_t kval_index(int V, size_t r, int m) {
    const size_t r7 = r & 7, grp = (r >> 3) * 8 * (size_t)V;   // elements before this 8-row group
    const int c = m >> 3, e = m & 7;                            // 16-byte chunk, element in chunk
    if (V == 64) return grp + r7 * 64 + (size_t)((c ^ (int)r7) << 3) + e;
    if (V == 128) return grp + (size_t)(c >> 3) * 512 + r7 * 64 + (size_t)(((c & 7) ^ (int)r7) << 3) + e;
    if (V == 32) return grp + r7 * 32 + (size_t)((c ^ (int)((r7 >> 1) & 3)) << 3) + e;
    if (V == 16) return grp + r7 * 16 + (size_t)((c ^ (int)((r7 >> 2) & 1)) << 3) + e;
    return r * (size_t)V + m;
}

struct shflbw_matrix {
    // ---- logical format (same fields as BlockwiseSpMatrix / BlockwiseSpFilter) ----
    int nrow = 0, ncol = 0, nnzb = 0, brow = 0, bcol = 1;
    float density = 0.f;
    unsigned seed = 0;
    bool row_permute = false;
    std::vector<int> indptr, indices, row_permute_ids;
    std::vector<uint16_t> values;  // fp16 bits, values[p*brow + m]
    bool is_filter = false;
    int F = 0, C = 0, R = 0, S = 0;
    std::string config_str;

    // ---- host images ----
    std::vector<int> meta_h;       // reference-compatible [indptr | indices*bcol | perm], pad 8
    std::vector<int> kptr, kidx;   // kernel image: padded offsets / column ids
    std::vector<int> kcrs;         // filters only: kidx decoded as c | r << 16 | s << 24 (k = (r*S + s)*C + c)
    std::vector<uint16_t> kval;    // kernel image: padded fp16 panels, element order kval_index()

    // ---- device copy (owned) ----
    int device = -1;
    void* d_meta = nullptr;        // one int32 allocation: kptr | kidx | perm | kcrs | status word
    void* d_val = nullptr;
    const int* d_kptr = nullptr;
    const int* d_kidx = nullptr;
    const int* d_kcrs = nullptr;   // filters with C < 65536 and R, S < 256 only
    const int* d_perm = nullptr;
    int* d_status = nullptr;

    // ---- scratch owned by the handle ----
    void* stage_in = nullptr;  size_t stage_in_bytes = 0;    // host-call staging of B / ifmap
    void* stage_c = nullptr;   size_t stage_c_bytes = 0;
    void* stage_out = nullptr; size_t stage_out_bytes = 0;   // host-call staging of D / ofmap
    void* conv_in = nullptr;   size_t conv_in_bytes = 0;     // input re-laid channel-major
    void* conv_out = nullptr;  size_t conv_out_bytes = 0;    // output in stored filter order
    std::vector<void*> retired;    // outgrown conv scratch: op states made earlier still point at it
    // streams (copy in, kernels, copy out) and events of the pipelined host-buffer call, made on first use
    void* host_streams[3] = {nullptr, nullptr, nullptr};
    void* host_events[16] = {};
};

namespace shflbw {

// fp16 helpers on raw bits (host).
float half_bits_to_float(uint16_t h);
uint16_t float_to_half_bits(float f);

// Seeded uniform fp16 stream documented in shflbw.h (SHFLBW_VALUES_UNIFORM).
uint16_t uniform_half(uint64_t stream, uint64_t index);

int validate(const shflbw_matrix& m);
void build_config_str(shflbw_matrix& m);
void build_host_images(shflbw_matrix& m);
void drop_device_copy(shflbw_matrix& m);  // implemented in shflbw_capi.cu

}  // namespace shflbw
