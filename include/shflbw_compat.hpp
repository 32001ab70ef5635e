// shflbw_compat.hpp -- the reference project's C++ names on top of the C ABI (shflbw.h).
//
// Lets code written against hgyhungry/ShflBW_Sparse_NN's headers compile against this
// library by swapping one include.  Mirrors (paths relative to the reference project):
//   BlockwiseSpMatrix<T>   block_sparse/spmm/blockwise_format.h:13-68
//   BlockwiseSpFilter<T>   block_sparse/spconv/blockwise_format.h:16-27
//   SpmmBlockwiseOpState / SpmmBlockwiseOp / SpmmBlockwiseInitFn / SpmmBlockwiseExecFn
//                          block_sparse/spmm/blockwise_op.h:6-52, 180-215
//   SpconvBlockwiseOpState / SpconvBlockwiseOp / SpconvBlockwiseInitFn / SpconvBlockwiseExecFn
//                          block_sparse/spconv/blockwise_op.h:6-50, 161-193
//   ShapeBase              block_sparse/common/base.h:22-24
// Header-only, host code only; all compute happens in libshflbw_b200.  Differences from the
// reference: errors surface as status codes (status(), initSuccess) instead of exit()/assert;
// alpha is honoured; SpConv feature maps are NHWC; tile template parameters only select
// nothing (the library picks its kernel shape at run time) except that ThreadBlockShape::M
// must equal the matrix's brow, as in the reference.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <istream>
#include <iterator>
#include <ostream>
#include <string>
#include <vector>

#include "shflbw.h"

template <int M_, int N_, int K_>
struct ShapeBase {
    static constexpr int M = M_, N = N_, K = K_;
};

template <typename T>
struct BlockwiseSpMatrix {
    static_assert(sizeof(T) == 2, "only 16-bit element types (half) are supported");
    // shape and pattern (filled after init_random / load, as the reference's public fields)
    int nrow = 0, ncol = 0, nnzb = 0, brow = 0, bcol = 1;
    float density = 0.f;
    unsigned seed = 0;
    bool row_permute = false;
    std::vector<int> indptr, indices, row_permute_ids;
    std::vector<T> values;
    bool initialized = false, device_synced = false;
    std::string config_str;
    shflbw_matrix_t* handle = nullptr;  // the library object behind this mirror
    int last_status = SHFLBW_OK;

    BlockwiseSpMatrix() = default;
    BlockwiseSpMatrix(const BlockwiseSpMatrix&) = delete;  // the reference's object is not safely copyable either
    BlockwiseSpMatrix& operator=(const BlockwiseSpMatrix&) = delete;
    virtual ~BlockwiseSpMatrix() { shflbw_matrix_destroy(handle); }

    void init_random(int nrow_, int ncol_, int brow_, int bcol_, float expected_density, bool row_permute_,
                     unsigned seed_, int value_mode = SHFLBW_VALUES_INT9_LIBC) {
        reset_();
        last_status = shflbw_matrix_create_random(nrow_, ncol_, brow_, bcol_, expected_density, row_permute_,
                                                  seed_, value_mode, &handle);
        pull_();
    }
    void load(std::istream& in) {
        std::string text((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
        reset_();
        last_status = shflbw_matrix_load_text(text.data(), text.size(), &handle);
        pull_();
    }
    void dump(std::ostream& out) {
        size_t need = 0;
        if (shflbw_matrix_dump_text(handle, nullptr, 0, &need) != SHFLBW_OK) return;
        std::string buf(need, '\0');
        shflbw_matrix_dump_text(handle, &buf[0], need, &need);
        out << buf;
    }
    void transform_and_sync_device() {
        last_status = shflbw_matrix_to_device(handle);
        device_synced = last_status == SHFLBW_OK;
    }

protected:
    void reset_() {
        shflbw_matrix_destroy(handle);
        handle = nullptr;
        initialized = device_synced = false;
    }
    void pull_() {  // copy the library object's fields into the public mirror
        if (last_status != SHFLBW_OK || !handle) return;
        nrow = shflbw_matrix_nrow(handle); ncol = shflbw_matrix_ncol(handle);
        nnzb = shflbw_matrix_nnzb(handle); brow = shflbw_matrix_brow(handle); bcol = shflbw_matrix_bcol(handle);
        density = shflbw_matrix_density(handle); seed = shflbw_matrix_seed(handle);
        row_permute = shflbw_matrix_row_permute(handle) != 0;
        indptr.assign(shflbw_matrix_indptr(handle), shflbw_matrix_indptr(handle) + nrow / brow + 1);
        indices.assign(shflbw_matrix_indices(handle), shflbw_matrix_indices(handle) + nnzb);
        values.resize((size_t)nnzb * brow * bcol);
        if (nnzb) std::char_traits<char>::copy((char*)values.data(), (const char*)shflbw_matrix_values(handle),
                                               values.size() * 2);
        row_permute_ids.clear();
        if (row_permute)
            row_permute_ids.assign(shflbw_matrix_row_permute_ids(handle), shflbw_matrix_row_permute_ids(handle) + nrow);
        config_str = shflbw_matrix_config_str(handle);
        initialized = true;
    }
};

template <typename T>
struct BlockwiseSpFilter : public BlockwiseSpMatrix<T> {
    int F = 0, C = 0, R = 0, S = 0;
    void init_random(int F_, int R_, int S_, int C_, int brow, int bcol, float expected_density,
                     bool filter_permute, unsigned seed, int value_mode = SHFLBW_VALUES_INT9_LIBC) {
        this->reset_();
        this->last_status = shflbw_filter_create_random(F_, R_, S_, C_, brow, bcol, expected_density,
                                                        filter_permute, seed, value_mode, &this->handle);
        this->pull_();
        if (this->last_status == SHFLBW_OK) { F = F_; R = R_; S = S_; C = C_; }
    }
};

// ------------------------------------------------------------------------------ SpMM ----
struct SpmmBlockwiseOpState {
    bool initSuccess = false;
    int status = SHFLBW_OK;
    shflbw_spmm_state_t impl{};
};

template <typename ThreadBlockShape, typename WarpShape, typename MmaShape, int NStage>
class SpmmBlockwiseOp {
public:
    SpmmBlockwiseOpState _state;
    void initialize(BlockwiseSpMatrix<half>& spmat, int N, half* B, half* D) {
        initialize(spmat, N, B, 1.0f, nullptr, 0.0f, D);
    }
    void initialize(BlockwiseSpMatrix<half>& spmat, int N, half* B, half* C, half* D) {
        initialize(spmat, N, B, 1.0f, C, 1.0f, D);
    }
    void initialize(BlockwiseSpMatrix<half>& spmat, int N, half* B, float alpha, half* C, float beta, half* D) {
        _state.status = spmat.brow != ThreadBlockShape::M
                            ? SHFLBW_ERR_UNSUPPORTED  // reference: assert(spmat.brow == BM)
                            : shflbw_spmm_init(spmat.handle, N, B, alpha, C, beta, D, SHFLBW_KERNEL_AUTO, &_state.impl);
        _state.initSuccess = _state.status == SHFLBW_OK;
    }
    void operator()(cudaStream_t stream = NULL) { _state.status = shflbw_spmm_exec(&_state.impl, (void*)stream); }
    int status() const { return _state.status; }
};

template <typename TB, typename Warp, typename Mma, int NStage>
SpmmBlockwiseOpState SpmmBlockwiseInitFn(BlockwiseSpMatrix<half>& spmat, int N, half* B, half* D) {
    SpmmBlockwiseOp<TB, Warp, Mma, NStage> op;
    op.initialize(spmat, N, B, D);
    return op._state;
}
template <typename TB, typename Warp, typename Mma, int NStage>
void SpmmBlockwiseExecFn(SpmmBlockwiseOpState& state, cudaStream_t stream = NULL) {
    state.status = shflbw_spmm_exec(&state.impl, (void*)stream);
}
typedef SpmmBlockwiseOpState (*SpmmBlockwiseInitFn_t)(BlockwiseSpMatrix<half>&, int, half*, half*);
typedef void (*SpmmBlockwiseExecFn_t)(SpmmBlockwiseOpState&, cudaStream_t);

// ---------------------------------------------------------------------------- SpConv ----
struct SpconvBlockwiseOpState {
    bool initSuccess = false;
    int status = SHFLBW_OK;
    shflbw_spconv_state_t impl{};
};

template <typename ThreadBlockShape, typename WarpShape, typename MmaShape, int NStage, bool strided = false>
class SpconvBlockwiseOp {
public:
    SpconvBlockwiseOpState _state;
    // IFMap / OFMap are NHWC device buffers ([B][H][W][C] and [B][ceil(H/stride)][ceil(W/stride)][F]).
    void initialize(BlockwiseSpFilter<half>& spfilter, int B, int H, int W, int stride, half* IFMap, half* OFMap) {
        _state.status = spfilter.brow != ThreadBlockShape::M
                            ? SHFLBW_ERR_UNSUPPORTED
                            : shflbw_spconv_init(spfilter.handle, B, H, W, stride, IFMap, OFMap, 1.0f,
                                                 SHFLBW_KERNEL_AUTO, &_state.impl);
        _state.initSuccess = _state.status == SHFLBW_OK;
    }
    void operator()(cudaStream_t stream = NULL) { _state.status = shflbw_spconv_exec(&_state.impl, (void*)stream); }
    int status() const { return _state.status; }
};

template <typename TB, typename Warp, typename Mma, int NStage>
SpconvBlockwiseOpState SpconvBlockwiseInitFn(BlockwiseSpFilter<half>& spfilter, int B, int H, int W, int stride,
                                             half* IFMap, half* OFMap) {
    SpconvBlockwiseOp<TB, Warp, Mma, NStage, true> op;
    op.initialize(spfilter, B, H, W, stride, IFMap, OFMap);
    return op._state;
}
template <typename TB, typename Warp, typename Mma, int NStage>
void SpconvBlockwiseExecFn(SpconvBlockwiseOpState& state, cudaStream_t stream = NULL) {
    state.status = shflbw_spconv_exec(&state.impl, (void*)stream);
}
typedef SpconvBlockwiseOpState (*SpconvBlockwiseInitFn_t)(BlockwiseSpFilter<half>&, int, int, int, int, half*, half*);
typedef void (*SpconvBlockwiseExecFn_t)(SpconvBlockwiseOpState&, cudaStream_t);
