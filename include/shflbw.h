/*
 * shflbw.h -- C ABI of the B200 (sm_100a) Shfl-BW block-sparse inference library.
 *
 * Plain C: opaque handles, raw pointers and sizes, int status codes.  No C++ or torch
 * types cross this boundary.  Every entry point names the interface of the reference
 * project (hgyhungry/ShflBW_Sparse_NN, paths relative to its root) that it replaces.
 *
 * Data conventions (all fp16 arrays are IEEE binary16 passed as uint16_t / void*):
 *   sparse matrix A: M x K, rows grouped in blocks of V = brow consecutive *stored* rows
 *     that share one sorted list of non-zero columns (bcol == 1; wider blocks:
 *     shflbw_matrix_create_from_block_arrays):
 *       indptr[M/V + 1]   offsets into indices, in non-zero columns
 *       indices[nnzb]     column ids, ascending inside each row block
 *       values[nnzb * V]  values[p*V + m] = A_stored[blk*V + m][indices[p]]
 *       perm[M] or NULL   stored row p is row perm[p] of the result (scatter on store)
 *   SpMM:   D[perm[i*V+m]][n] = alpha * sum_p values[p][m] * B[indices[p]][n] + beta * C[..][n]
 *           B: K x N row-major, C/D: M x N row-major, N % 8 == 0.
 *   SpConv: filter matrix F x (R*S*C), column k = (r*S + s)*C + c; activations NHWC:
 *           in [B][Hin][Win][C], out [B][Ho][Wo][F], Ho = ceil(Hin/stride), pad R/2, S/2,
 *           C % 8 == 0.
 *
 * Threading: handles are not internally locked.  Exec calls are asynchronous on the
 * caller's stream and reentrant across distinct states.  The library uses the CUDA
 * device that is current at the time of each call.
 */
#ifndef SHFLBW_H_
#define SHFLBW_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes (replace exit()/assert of block_sparse/cuda_error.h:7-16 and
 *      block_sparse/spmm/blockwise_op.h:85-87) ---- */
enum {
    SHFLBW_OK = 0,
    SHFLBW_ERR_INVALID_ARG = 1,    /* null pointer, negative size, bad enum              */
    SHFLBW_ERR_BAD_FORMAT = 2,     /* indptr/indices/perm fail validation, parse error   */
    SHFLBW_ERR_UNSUPPORTED = 3,    /* shape outside the contract (V, N % 8, C % 8, ...)  */
    SHFLBW_ERR_CUDA = 4,           /* a CUDA runtime call failed (see shflbw_last_cuda_error) */
    SHFLBW_ERR_NOT_ON_DEVICE = 5,  /* no device copy, or it lives on another GPU than the current one */
    SHFLBW_ERR_DEVICE_TIMEOUT = 6, /* a bounded in-kernel wait gave up (status word set) */
    SHFLBW_ERR_IO = 7,
    SHFLBW_ERR_TOO_LARGE = 8       /* needs more than a fixed built-in capacity           */
};

/* How shflbw_matrix_create_random fills values. */
enum {
    SHFLBW_VALUES_INT9_LIBC = 0, /* half(rand() % 9 - 4) from the process-wide libc stream,
                                    exactly block_sparse/spmm/blockwise_format.h:99-102   */
    SHFLBW_VALUES_UNIFORM = 1    /* seeded fp16 uniform in [-1, 1): value i of stream s is
                                    rn_fp16(2*u - 1), u = (splitmix64(s*2^32 + i) >> 40) / 2^24 */
};

/* Kernel selection for op init. */
enum {
    SHFLBW_KERNEL_AUTO = 0,    /* tcgen05/TMEM kernel (the product path)                  */
    SHFLBW_KERNEL_TCGEN05 = 1,
    SHFLBW_KERNEL_SIMT = 2     /* plain CUDA-core kernel: bring-up / on-device cross-check */
};

typedef struct shflbw_matrix shflbw_matrix_t; /* replaces BlockwiseSpMatrix<half> and
                                                 BlockwiseSpFilter<half>
                                                 (block_sparse/spmm/blockwise_format.h:13-68,
                                                  block_sparse/spconv/blockwise_format.h:16-27) */

const char* shflbw_strerror(int status);
/* Text of the last CUDA error seen by this thread inside the library ("" if none). */
const char* shflbw_last_cuda_error(void);
/* Library/ABI version, for binding sanity checks. */
int shflbw_abi_version(void);

/* Every wait inside the kernels (on a pipeline stage, an accumulator) is bounded: after this many
 * SM clocks without progress the kernel records a SHFLBW_DEVSTAT_* code in the matrix's status
 * word, stops issuing work, lets what is in flight land and returns; shflbw_matrix_device_status
 * then reports SHFLBW_ERR_DEVICE_TIMEOUT and the context stays usable.  Default 400 000 000
 * (~0.2 s); process-wide, applies to launches issued after the call.  No counterpart in the
 * reference (its kernels have no waits that another agent completes). */
int shflbw_set_wait_limit_cycles(long long cycles);

/* ---------------------------------------------------------------- format builder ---- */

/* Replaces BlockwiseSpMatrix<half>::init_random (block_sparse/spmm/blockwise_format.h:70-123)
 * and random_mask (block_sparse/util/random_mask.cc:10-67): mask, permutation, values,
 * achieved density, config string.  ncol % bcol must be 0.  stream seed for UNIFORM values = seed. */
int shflbw_matrix_create_random(int nrow, int ncol, int brow, int bcol, float density,
                                int row_permute, unsigned seed, int value_mode,
                                shflbw_matrix_t** out);

/* Replaces BlockwiseSpFilter<half>::init_random (block_sparse/spconv/blockwise_format.h:29-52):
 * the F x (R*S*C) matrix plus F, R, S, C and the filter config string. */
int shflbw_filter_create_random(int F, int R, int S, int C, int brow, int bcol, float density,
                                int filter_permute, unsigned seed, int value_mode,
                                shflbw_matrix_t** out);

/* Build from caller arrays (copied).  Replaces filling the public vectors of
 * BlockwiseSpMatrix (block_sparse/spmm/blockwise_format.h:27-28).  perm may be NULL.
 * Validates (see shflbw_matrix_validate). */
int shflbw_matrix_create_from_arrays(int nrow, int ncol, int brow, int nnzb, const int* indptr,
                                     const int* indices, const uint16_t* values, const int* perm,
                                     shflbw_matrix_t** out);
/* The same with brow x bcol blocks (the format of blockwise_format.h:13-68 in full): indices
 * are in units of bcol columns, values hold nnzb * brow * bcol halves, each block column by
 * column (value (mm, kk) of block p at values[p*brow*bcol + kk*brow + mm], :286-297).  The
 * reference's kernels assert bcol == 1 (spmm/blockwise_op.h:86); here the device image lists a
 * block's bcol columns one after the other, so every operator accepts such a matrix. */
int shflbw_matrix_create_from_block_arrays(int nrow, int ncol, int brow, int bcol, int nnzb,
                                           const int* indptr, const int* indices,
                                           const uint16_t* values, const int* perm,
                                           shflbw_matrix_t** out);
/* Marks a matrix as a conv filter of shape F x R x S x C (nrow == F, ncol == R*S*C). */
int shflbw_matrix_set_filter_shape(shflbw_matrix_t* m, int F, int R, int S, int C);

/* Replaces BlockwiseSpMatrix<half>::load / ::dump (block_sparse/spmm/blockwise_format.h:151-198,
 * 125-149; format: example/spmatrix_dump_load.md).  Text is byte-compatible. */
int shflbw_matrix_load_text(const char* text, size_t len, shflbw_matrix_t** out);
int shflbw_matrix_load_file(const char* path, shflbw_matrix_t** out);
/* Writes at most cap bytes; *needed receives the full size (call with buf=NULL to size). */
int shflbw_matrix_dump_text(const shflbw_matrix_t* m, char* buf, size_t cap, size_t* needed);
int shflbw_matrix_dump_file(const shflbw_matrix_t* m, const char* path);

/* Structural checks the reference leaves to the caller: indptr monotone from 0 to nnzb,
 * indices in [0, ncol) and strictly ascending per row block, perm a permutation of [0, nrow). */
int shflbw_matrix_validate(const shflbw_matrix_t* m);

void shflbw_matrix_destroy(shflbw_matrix_t* m);

/* Scalar getters (public fields of BlockwiseSpMatrix / BlockwiseSpFilter). */
int shflbw_matrix_nrow(const shflbw_matrix_t* m);
int shflbw_matrix_ncol(const shflbw_matrix_t* m);
int shflbw_matrix_nnzb(const shflbw_matrix_t* m);
int shflbw_matrix_brow(const shflbw_matrix_t* m);
int shflbw_matrix_bcol(const shflbw_matrix_t* m);
int shflbw_matrix_row_permute(const shflbw_matrix_t* m);
unsigned shflbw_matrix_seed(const shflbw_matrix_t* m);
float shflbw_matrix_density(const shflbw_matrix_t* m);
const char* shflbw_matrix_config_str(const shflbw_matrix_t* m);
int shflbw_matrix_filter_shape(const shflbw_matrix_t* m, int* F, int* R, int* S, int* C);
/* Array getters: pointers into the handle, valid until it is destroyed or rebuilt. */
const int* shflbw_matrix_indptr(const shflbw_matrix_t* m);        /* nrow/brow + 1 */
const int* shflbw_matrix_indices(const shflbw_matrix_t* m);       /* nnzb          */
const uint16_t* shflbw_matrix_values(const shflbw_matrix_t* m);   /* nnzb * brow   */
const int* shflbw_matrix_row_permute_ids(const shflbw_matrix_t* m); /* nrow or NULL */

/* Replaces BlockwiseSpMatrix<half>::transform_and_sync_device
 * (block_sparse/spmm/blockwise_format.h:200-266).  Builds the host images and uploads them
 * to the current device.  Two images are kept:
 *   - the reference-compatible int32 meta image [indptr | indices*bcol | perm], each section
 *     zero-padded to 8 ints (readable with shflbw_matrix_meta_image), and
 *   - the kernel image: every row block's column list padded to a multiple of 16 (extra
 *     columns repeat the block's last column id and carry zero values), so kernels never
 *     see a ragged K tail.
 * Idempotent; rebuilding the matrix drops the device copy. */
int shflbw_matrix_to_device(shflbw_matrix_t* m);
int shflbw_matrix_on_device(const shflbw_matrix_t* m);
/* Host copy of the reference-compatible meta image; *n_int32 = its length. */
const int* shflbw_matrix_meta_image(const shflbw_matrix_t* m, size_t* n_int32);

/* ------------------------------------------------------------------------- SpMM ---- */

/* Replaces SpmmBlockwiseOpState (block_sparse/spmm/blockwise_op.h:6-17): a POD the caller
 * may copy.  Holds non-owning device pointers: the matrix handle and B, C, D must outlive it. */
typedef struct shflbw_spmm_state {
    int M, N, K, V;
    int num_row_blocks;
    int kernel;              /* SHFLBW_KERNEL_* actually selected */
    int tokens_per_cta;      /* dense-dimension tile of one work item */
    int stages;              /* shared-memory pipeline depth */
    int producer_warps;      /* warps issuing the gather */
    int variant;             /* 0: tokens in TMEM lanes; 1: rows of the block in TMEM lanes; 2: as 0 with 16 epilogue warps */
    int num_items, tiles_n;  /* work items = row blocks x dense tiles */
    unsigned grid_x, grid_y, block_x;
    size_t shared_mem_size;
    int init_success;        /* initSuccess of the reference state */
    float alpha, beta;
    const void* B;
    const void* C;
    void* D;
    const int* blk_ptr;      /* padded row-block offsets (units: rows of 16-padded panels) */
    const int* blk_idx;      /* padded column ids */
    const void* blk_val;     /* padded fp16 value panels, [rows][V] */
    const int* perm;         /* device row permutation or NULL */
    int* status_word;        /* device int: 0 ok, else a SHFLBW_DEVSTAT_* code */
    int gather;              /* 0: cp.async gather, 1: TMA tile-gather through tmap_b */
    unsigned long long tmap_b[16]; /* TMA tensor map of B (opaque 128 bytes, built at init from B and N) */
} shflbw_spmm_state_t;

/* Replaces SpmmBlockwiseOp::initialize / SpmmBlockwiseInitFn
 * (block_sparse/spmm/blockwise_op.h:73-132, 180-194).  B, C, D are device pointers;
 * C may be NULL when beta == 0.  alpha is honoured (the reference hard-wires 1.0,
 * block_sparse/spmm/blockwise_op.h:91-95).  kernel = SHFLBW_KERNEL_*. */
int shflbw_spmm_init(const shflbw_matrix_t* m, int N, const void* B, float alpha, const void* C,
                     float beta, void* D, int kernel, shflbw_spmm_state_t* out);

/* Replaces SpmmBlockwiseOp::operator() / SpmmBlockwiseExecFn
 * (block_sparse/spmm/blockwise_op.h:169-174, 204-209): asynchronous launch on `stream`
 * (a cudaStream_t; NULL = default stream).  Returns launch errors only. */
int shflbw_spmm_exec(const shflbw_spmm_state_t* st, void* stream);

/* Reads (and clears) the device status word of the matrix used by `st`; synchronises the
 * device.  SHFLBW_OK or SHFLBW_ERR_DEVICE_TIMEOUT. */
int shflbw_matrix_device_status(const shflbw_matrix_t* m);

/* End-to-end call with HOST buffers (what a plugin caller without device memory uses):
 * copies B (and C) to the device, runs, copies D back, synchronises.  B/C/D are host
 * pointers.  Operands of 2048 columns or more move in four column chunks through three
 * streams (copy in, kernels, copy out) so that the two transfers overlap; that needs
 * page-locked host memory (pageable buffers work, without the overlap).  Device staging
 * buffers, streams and events are owned by the matrix handle and reused across calls: one
 * host-buffer call per handle at a time. */
int shflbw_spmm_host(shflbw_matrix_t* m, int N, const void* B_host, float alpha,
                     const void* C_host, float beta, void* D_host);

/* Measurement aid for shflbw_spmm_host: moves the same bytes of B in and of D out through the
 * same staging buffers, streams and events, in the same chunks, WITHOUT launching the kernel --
 * the time of the link alone, which bounds the host-buffer call from below.  contiguous != 0
 * moves every chunk as one contiguous block of the same size instead of a strided column slice
 * (what the strided form costs).  D_host receives staging-buffer contents, not a result. */
int shflbw_spmm_host_copies_only(shflbw_matrix_t* m, int N, const void* B_host, void* D_host, int contiguous);

/* ----------------------------------------------------------------------- SpConv ---- */

/* Replaces SpconvBlockwiseOpState (block_sparse/spconv/blockwise_op.h:6-17). */
typedef struct shflbw_spconv_state {
    int B, Hin, Win, C, F, R, S, stride, Ho, Wo, V;
    int Bp;                  /* batch rounded up to 8: innermost extent of the staged input */
    int kernel;
    int tokens_per_cta;
    int stages;
    int producer_warps;
    int variant;             /* 0: tokens in TMEM lanes; 1: filters in TMEM lanes (NHWC calls: planes out + transpose);
                                2: as 0 with 16 epilogue warps (chained layers) */
    int num_items, tiles_n;
    unsigned grid_x, grid_y, block_x;
    size_t shared_mem_size;
    int init_success;
    float alpha;
    const void* ifmap;       /* NHWC input (device)  */
    void* ofmap;             /* NHWC output (device) */
    void* staged_in;         /* scratch: input as [C][Hin+R-1][Win+S-1][Bp], zero halo */
    void* staged_out;        /* scratch: output planes [F][Ho][Wo][Bp] (variant 1), [B*Ho*Wo][F] in stored
                                filter order (variant 0, permuted filter), or NULL */
    size_t staged_in_bytes, staged_out_bytes;
    const int* blk_ptr;
    const int* blk_idx;      /* tensor-core path: ids decoded as c | r<<16 | s<<24 */
    const void* blk_val;
    const int* perm;
    int* status_word;
    /* chained layers (shflbw_spconv_chain_init): ifmap / ofmap are chain buffers, no scratch */
    int chain;               /* 1: input and output are chain buffers                   */
    int out_R, out_S;        /* filter shape of the consumer the output halo is for     */
    int relu;                /* 1: max(x, 0) fused into the epilogue                    */
    const void* residual;    /* chained: optional residual chain buffer (output geometry) */
    const int* residual_map; /* chained: stored filter -> plane of `residual`, or NULL     */
} shflbw_spconv_state_t;

/* Replaces SpconvBlockwiseOp::initialize / SpconvBlockwiseInitFn
 * (block_sparse/spconv/blockwise_op.h:70-131, 161-167).  ifmap/ofmap are NHWC device
 * pointers.  Scratch for the staged input (and, with a filter permutation, the staged
 * output) is owned by the filter handle and shared by every state initialised from it: run
 * those states one at a time (one stream, or ordered by events).  A later init with a larger
 * shape allocates larger scratch; states made before stay valid (their scratch is kept until
 * the handle is destroyed). */
int shflbw_spconv_init(shflbw_matrix_t* filter, int B, int Hin, int Win, int stride,
                       const void* ifmap_nhwc, void* ofmap_nhwc, float alpha, int kernel,
                       shflbw_spconv_state_t* out);

/* Replaces SpconvBlockwiseOp::operator() / SpconvBlockwiseExecFn
 * (block_sparse/spconv/blockwise_op.h:148-153, 177-187). */
int shflbw_spconv_exec(const shflbw_spconv_state_t* st, void* stream);

/* End-to-end conv with HOST NHWC buffers.  Batches of 32 images or more move in up to four
 * chunks of whole 8-image groups through the same three streams as shflbw_spmm_host (copy in,
 * kernels, copy out overlap; page-locked host memory needed for the overlap).  One host-buffer
 * call per handle at a time. */
int shflbw_spconv_host(shflbw_matrix_t* filter, int B, int Hin, int Win, int stride,
                       const void* ifmap_host, void* ofmap_host, float alpha);

/* ---- Chained SpConv layers.  No counterpart in the reference project (its epilogue hooks,
 * block_sparse/common/epilogue.h:6-135, and the "online transformation" of docs/format.pdf are
 * the pointers).  Between two Shfl-BW conv layers the activation does not have to go back to
 * NHWC in logical channel order: a CHAIN BUFFER holds it as fp16 [C][H+R-1][W+S-1][Bp] --
 * channel-major, batch innermost and rounded up to 8 (Bp), with a zero halo sized for the R x S
 * filter of the layer that will READ it (image origin at (R/2, S/2)), and with channels in the
 * STORED filter order of the layer that wrote it.  A chained layer is then one kernel launch:
 * no relayout before it and no inverse permutation after it.
 *
 *   x NHWC --import--> buf0 --conv1--> buf1 --conv2--> buf2 --export--> y NHWC
 *
 * The caller owns the buffers (shflbw_chain_buffer_elems fp16 elements each) and zero-fills
 * each ONCE before first use: layers write only the interior, the halo has to stay zero.
 * conv2's filter must address its input channels in conv1's stored order: build it with
 * shflbw_filter_fold_input_order(filter2, filter1).  Results equal the unchained path up to
 * fp32 summation order (folding re-sorts the columns of a row block). */
size_t shflbw_chain_buffer_elems(int C, int H, int W, int B, int R_consumer, int S_consumer);
/* NHWC (logical channel order) -> chain buffer for a consumer with an R x S filter. */
int shflbw_chain_import_nhwc(const void* nhwc, int B, int H, int W, int C, int R_consumer, int S_consumer,
                             void* chain_buf, void* stream);
/* Chain buffer written by `producer` (halo for R x S) -> NHWC in logical channel order
 * (producer's inverse filter permutation applied; producer == NULL: channels as stored). */
int shflbw_chain_export_nhwc(const void* chain_buf, int B, int H, int W, int F, int R_halo, int S_halo,
                             const shflbw_matrix_t* producer, void* nhwc, void* stream);
/* New filter = `filter` with its input channels renumbered to the stored filter order of
 * `producer` (filter->C == producer->F); column lists re-sorted, values moved with them. */
int shflbw_filter_fold_input_order(const shflbw_matrix_t* filter, const shflbw_matrix_t* producer,
                                   shflbw_matrix_t** out);
/* One chained layer: in_chain has the halo of THIS filter, out_chain the halo of the consumer's
 * R_next x S_next filter (1 x 1 for none).  relu != 0 fuses max(x, 0).  Run with shflbw_spconv_exec
 * (one launch, no scratch, no allocation). */
int shflbw_spconv_chain_init(shflbw_matrix_t* filter, int B, int Hin, int Win, int stride,
                             const void* in_chain, void* out_chain, int R_next, int S_next,
                             float alpha, int relu, shflbw_spconv_state_t* out);

/* Residual connection of a chained layer: out = relu?(alpha * conv + residual), in fp16.
 * `res_chain` is a chain buffer with the geometry of the layer's OUTPUT (same H, W, batch and
 * halo as out_chain); its plane map_host[f] is added to stored filter f (map_host == NULL: plane
 * f).  shflbw_chain_residual_map fills the map for the usual case -- the residual was written
 * by `residual_producer` (NULL: it holds logical channel order) and must meet the logical
 * channels of `layer`'s stored filters.  Call between shflbw_spconv_chain_init and the first
 * shflbw_spconv_exec; the device copy of the map belongs to the filter handle. */
int shflbw_chain_residual_map(const shflbw_matrix_t* layer, const shflbw_matrix_t* residual_producer,
                              int* map_host /* layer->F ints */);
int shflbw_spconv_chain_set_residual(shflbw_matrix_t* filter, shflbw_spconv_state_t* st, const void* res_chain,
                                     const int* map_host);

/* SpConv for callers that must not allocate.  No counterpart in the reference project.
 *
 * Some hosts call this library from a place where device allocation is off limits: the
 * execute hook of an inference-runtime plugin, or a serving loop whose memory is carved up
 * front by a pool (a late cudaMalloc would synchronise the whole device and can fail when
 * the pool owns the GPU).  The regular shflbw_spconv_init grows scratch buffers with
 * cudaMalloc; this entry point does not.  It runs the same kernels (relayout, panel kernel,
 * transpose or inverse filter permutation) with their scratch in a fixed array of
 * SHFLBW_STATIC_SCRATCH_BYTES that is part of the library image; every GPU that loads the
 * library holds that array until the process exits.
 *
 *  - `filter` must already be on the device (shflbw_matrix_to_device, done at set-up time).
 *  - ifmap / ofmap are NHWC device pointers exactly as for shflbw_spconv_init; the launch is
 *    asynchronous on `stream`.
 *  - Needs 2*C*(Hin+R-1)*(Win+S-1)*roundup8(B) bytes for the staged input, plus up to
 *    2*roundup8(B)*Ho*Wo*F for the staged output (not needed by unpermuted filters on the
 *    positions-out plan), each rounded up to 256.  More than the capacity ->
 *    SHFLBW_ERR_TOO_LARGE, nothing is launched.  The 32-bit range checks of shflbw_spconv_init
 *    apply as well (SHFLBW_ERR_UNSUPPORTED).
 *  - The first call on each device looks up the array's device address; make that first
 *    call during set-up, before any stream capture on that device.
 *  - All calls on a device share the one array and it keeps the previous call's contents.
 *    Nothing in it has to start at zero (every byte that is read is written first by the
 *    same call), but two calls that overlap on the GPU -- different streams, or another
 *    thread -- race on it.  Serialise them.
 *  - It calls no cudaMalloc / cudaFree and no allocating library routine. */
#define SHFLBW_STATIC_SCRATCH_BYTES (32u * 1024u * 1024u)
int shflbw_spconv_exec_static_scratch(const shflbw_matrix_t* filter, int B, int Hin, int Win, int stride,
                                      const void* ifmap_nhwc, void* ofmap_nhwc, float alpha, void* stream);

/* ---- Several GPUs driven from one process.  No counterpart in the reference project (it is
 * single-GPU).  The path shards along the dense dimension with no exchange: every GPU holds a
 * replica of the sparse operand and owns a contiguous slice of B's columns (SpMM) or of the
 * batch (SpConv); its slice of the output is complete on its own.  Device ids are explicit;
 * every call restores the caller's current device. */

/* Even split of `total` units (dense columns with granule 8, images with granule 1) over `parts`
 * shards in multiples of `granule`; the first shards get the larger sizes, trailing shards may be
 * empty.  shard `index` owns [*begin, *begin + *count). */
int shflbw_shard_range(long long total, int granule, int parts, int index, long long* begin, long long* count);

/* Copy of a matrix / filter (host side only; the copy has no device image yet).  Replicate a
 * sparse operand by hand: clone, cudaSetDevice, shflbw_matrix_to_device. */
int shflbw_matrix_clone(const shflbw_matrix_t* m, shflbw_matrix_t** out);

typedef struct shflbw_multi shflbw_multi_t;
/* Uploads a replica of `m` to each of the n devices (ids may repeat) and makes one stream per shard. */
int shflbw_multi_create(const shflbw_matrix_t* m, const int* device_ids, int n, shflbw_multi_t** out);
void shflbw_multi_destroy(shflbw_multi_t* mg);
int shflbw_multi_shards(const shflbw_multi_t* mg);
/* Shard g computes D[g] (M x n_per_shard[g]) = alpha * A . B[g] (K x n_per_shard[g]); B[g] and D[g]
 * are contiguous row-major buffers on device_ids[g].  n_per_shard[g] == 0 skips the shard. */
int shflbw_multi_spmm_init(shflbw_multi_t* mg, const int* n_per_shard, const void* const* B, void* const* D, float alpha);
/* Shard g convolves images_per_shard[g] NHWC images ifmap[g] -> ofmap[g] on device_ids[g]. */
int shflbw_multi_spconv_init(shflbw_multi_t* mg, const int* images_per_shard, int Hin, int Win, int stride,
                             const void* const* ifmap_nhwc, void* const* ofmap_nhwc, float alpha);
/* Launches every shard on its own stream, one after the other, without waiting for any GPU. */
int shflbw_multi_exec(shflbw_multi_t* mg);
/* Waits for every shard; *max_ms (optional) = the largest device time of the last exec over the
 * shards; returns SHFLBW_ERR_DEVICE_TIMEOUT if a shard's status word is set. */
int shflbw_multi_sync(shflbw_multi_t* mg, float* max_ms);

/* Number of kernel launches one exec call issues (for launch accounting). */
int shflbw_spmm_launches_per_exec(const shflbw_spmm_state_t* st);
int shflbw_spconv_launches_per_exec(const shflbw_spconv_state_t* st);

/* Device status word values written by kernels when a bounded wait gives up. */
enum {
    SHFLBW_DEVSTAT_OK = 0,
    SHFLBW_DEVSTAT_TIMEOUT_FULL = 1,   /* consumer never saw a filled stage  */
    SHFLBW_DEVSTAT_TIMEOUT_EMPTY = 2,  /* producer never saw a freed stage   */
    SHFLBW_DEVSTAT_TIMEOUT_ACCUM = 3   /* epilogue never saw the accumulator */
};

#ifdef __cplusplus
} /* extern "C" */
#endif
#endif /* SHFLBW_H_ */
