// CUDA side of the C ABI: device upload of the Shfl-BW images, op init / exec for SpMM and
// SpConv, and the end-to-end host-buffer calls.  Host code here only validates, fills POD
// states and launches; all arithmetic happens in the kernels of panel_umma.cuh /
// aux_kernels.cuh.  There is no CPU fallback: without a CUDA device every op entry point
// returns SHFLBW_ERR_CUDA.
//
// Reference host code this replaces (paths relative to the reference project):
//   block_sparse/spmm/blockwise_format.h:200-266   transform_and_sync_device
//   block_sparse/spmm/blockwise_op.h:73-132, 169-209   initialize / operator() / InitFn / ExecFn
//   block_sparse/spconv/blockwise_op.h:70-131, 148-187

#include <cuda.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <utility>

#include "aux_kernels.cuh"
#include "panel_umma.cuh"
#include "shflbw_internal.hpp"

namespace {

thread_local char g_cuda_err[256] = "";

// Bound of the kernels' barrier waits in SM clocks, and (fault-injection builds) the stage from
// which one producer warp withholds its arrivals.  Process-wide; read when a launch is issued.
long long g_wait_limit = shflbw::kWaitLimitCycles;
int g_inject_from = -1;

bool cuda_ok(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return true;
    snprintf(g_cuda_err, sizeof g_cuda_err, "%s: %s", what, cudaGetErrorString(e));
    (void)cudaGetLastError();  // clear the sticky-free error state
    return false;
}
#define CK(call) do { if (!cuda_ok((call), #call)) return SHFLBW_ERR_CUDA; } while (0)

// Every kernel of this library is launched with the programmatic-stream-serialization attribute:
// it may start while the previous kernel of the stream drains, sets itself up (barriers, TMEM,
// item table), and only then waits for that kernel's completion (griddepcontrol.wait in the
// kernels).  Stream order of all data accesses is unchanged.  SHFLBW_PDL=0 turns it off.
bool use_pdl() {
    static const bool on = [] { const char* e = getenv("SHFLBW_PDL"); return !(e && atoi(e) == 0); }();
    return on;
}
template <typename... Params, typename... Args>
cudaError_t launch(void (*kernel)(Params...), dim3 grid, dim3 block, size_t smem, cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = use_pdl() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

int ensure_buffer(void** buf, size_t* have, size_t need) {
    if (*have >= need && *buf) return SHFLBW_OK;
    if (*buf) { cudaFree(*buf); *buf = nullptr; *have = 0; }
    CK(cudaMalloc(buf, need));
    *have = need;
    return SHFLBW_OK;
}

// The device copy lives on the GPU that was current in shflbw_matrix_to_device; launching its
// pointers on another GPU would fault, so ops insist on that GPU being current.
bool on_current_device(const shflbw_matrix& m) {
    int dev = -1;
    return m.d_meta && cudaGetDevice(&dev) == cudaSuccess && dev == m.device;
}

// Conv scratch grows without freeing the outgrown buffer: states initialised earlier keep
// non-owning pointers to it.  Everything is released with the matrix's device copy.
int grow_scratch(shflbw_matrix& m, void** buf, size_t* have, size_t need) {
    if (*have >= need && *buf) return SHFLBW_OK;
    void* fresh = nullptr;
    CK(cudaMalloc(&fresh, need));
    if (*buf) m.retired.push_back(*buf);
    *buf = fresh;
    *have = need;
    return SHFLBW_OK;
}

// Streams and events of the pipelined host-buffer calls, owned by the handle (made on first use).
int host_pipeline(shflbw_matrix* m, cudaStream_t* s_in, cudaStream_t* s_k, cudaStream_t* s_out,
                         cudaEvent_t** e_in, cudaEvent_t** e_k) {
    if (!m->host_streams[0]) {
        for (int i = 0; i < 3; ++i) {
            cudaStream_t st_ = nullptr;
            CK(cudaStreamCreateWithFlags(&st_, cudaStreamNonBlocking));
            m->host_streams[i] = st_;
        }
        for (int i = 0; i < 16; ++i) {
            cudaEvent_t ev_ = nullptr;
            CK(cudaEventCreateWithFlags(&ev_, cudaEventDisableTiming));
            m->host_events[i] = ev_;
        }
    }
    *s_in = (cudaStream_t)m->host_streams[0]; *s_k = (cudaStream_t)m->host_streams[1];
    *s_out = (cudaStream_t)m->host_streams[2];
    *e_in = (cudaEvent_t*)&m->host_events[0]; *e_k = (cudaEvent_t*)&m->host_events[8];
    return SHFLBW_OK;
}

// ---- kernel table -------------------------------------------------------------------
using PanelKernel = void (*)(const shflbw::PanelParams);
struct PanelChoice { PanelKernel fn; size_t smem; int tokens; int stages; int pw; int threads; int variant; int gather; };

template <int V, int TM, int KS, int STAGES, int PW, int MODE, int GROUPS = 2, int LAG = 1, int GATHER = shflbw::kGatherCpAsync,
          int EW = 8>
PanelChoice choice() {
    using Cfg = shflbw::PanelCfg<V, TM, KS, STAGES, PW, MODE, GROUPS, LAG, GATHER, EW>;
    return {shflbw::panel_umma_kernel<V, TM, KS, STAGES, PW, MODE, GROUPS, LAG, GATHER, EW>, (size_t)Cfg::SMEM_BYTES, Cfg::T,
            STAGES, PW, Cfg::THREADS, 0, GATHER};
}

// TMA tensor map of the dense operand B ([K][N] fp16 row-major): box = 64 tokens x 1 row (what one
// row of a tile::gather4 fetches), 128-byte swizzle (the layout tcgen05.mma reads), zero fill
// outside the tensor.  The driver entry point is looked up once.
int encode_b_map(const void* B, int K, int N, unsigned long long out[16]) {
    typedef CUresult (*Encode)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                               const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static Encode enc = nullptr;
    if (!enc) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qr;
        CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr));
        if (!fn || qr != cudaDriverEntryPointSuccess) return SHFLBW_ERR_CUDA;
        enc = (Encode)fn;
    }
    static_assert(sizeof(CUtensorMap) == 128, "tensor map size");
    alignas(64) CUtensorMap tm;
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)K}, strides[1] = {(cuuint64_t)N * 2};
    const cuuint32_t box[2] = {64, 1}, estr[2] = {1, 1};
    const CUresult r = enc(&tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(B), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(g_cuda_err, sizeof g_cuda_err, "cuTensorMapEncodeTiled failed: %d", (int)r);
        return SHFLBW_ERR_CUDA;
    }
    std::memcpy(out, &tm, 128);
    return SHFLBW_OK;
}

#ifdef SHFLBW_TUNE
// Tuning builds only: SHFLBW_SHAPE="pw,groups,lag" picks the pipeline shape of the V = 64,
// 256-token kernels (read at init and at exec, so a state follows the variable).
template <int MODE>
bool tuned_shape(PanelChoice* out) {
    const char* e = getenv("SHFLBW_SHAPE");
    if (!e) return false;
    int pw = 0, groups = 0, lag = 0;
    if (sscanf(e, "%d,%d,%d", &pw, &groups, &lag) != 3) return false;
    switch (pw * 100 + groups * 10 + lag) {
        case 821:  *out = choice<64, 2, 64, 5, 8, MODE, 2, 1>(); return true;
        case 822:  *out = choice<64, 2, 64, 5, 8, MODE, 2, 2>(); return true;
        case 811:  *out = choice<64, 2, 64, 5, 8, MODE, 1, 1>(); return true;
        case 812:  *out = choice<64, 2, 64, 5, 8, MODE, 1, 2>(); return true;
        case 1621: *out = choice<64, 2, 64, 5, 16, MODE, 2, 1>(); return true;
        case 1622: *out = choice<64, 2, 64, 5, 16, MODE, 2, 2>(); return true;
        case 1611: *out = choice<64, 2, 64, 5, 16, MODE, 1, 1>(); return true;
        case 1612: *out = choice<64, 2, 64, 5, 16, MODE, 1, 2>(); return true;
        case 1641: *out = choice<64, 2, 64, 5, 16, MODE, 4, 1>(); return true;
        default: break;
    }
    switch (pw * 100 + groups * 10 + lag) {               // lag 3: cp.async with deferred arrivals
        case 813:  *out = choice<64, 2, 64, 5, 8, MODE, 1, 1, shflbw::kGatherCpAsyncArrive>(); return true;
        case 823:  *out = choice<64, 2, 64, 5, 8, MODE, 2, 1, shflbw::kGatherCpAsyncArrive>(); return true;
        case 1613: *out = choice<64, 2, 64, 5, 16, MODE, 1, 1, shflbw::kGatherCpAsyncArrive>(); return true;
        case 1623: *out = choice<64, 2, 64, 5, 16, MODE, 2, 1, shflbw::kGatherCpAsyncArrive>(); return true;
        case 1643: *out = choice<64, 2, 64, 5, 16, MODE, 4, 1, shflbw::kGatherCpAsyncArrive>(); return true;
        default: break;
    }
    if constexpr (MODE == shflbw::kPanelSpmmRows) {   // lag 0: TMA gather
        switch (pw * 100 + groups * 10 + lag) {
            case 410:  *out = choice<64, 2, 64, 5, 4, MODE, 1, 1, shflbw::kGatherTma>(); return true;
            case 810:  *out = choice<64, 2, 64, 5, 8, MODE, 1, 1, shflbw::kGatherTma>(); return true;
            case 820:  *out = choice<64, 2, 64, 5, 8, MODE, 2, 1, shflbw::kGatherTma>(); return true;
            case 1610: *out = choice<64, 2, 64, 5, 16, MODE, 1, 1, shflbw::kGatherTma>(); return true;
            case 1620: *out = choice<64, 2, 64, 5, 16, MODE, 2, 1, shflbw::kGatherTma>(); return true;
            case 1640: *out = choice<64, 2, 64, 5, 16, MODE, 4, 1, shflbw::kGatherTma>(); return true;
            case 840:  *out = choice<64, 2, 64, 5, 8, MODE, 4, 1, shflbw::kGatherTma>(); return true;
            default: break;
        }
    }
    return false;
}
#endif

// Pipeline shape per (V, tile): non-zero columns per stage (KS) and ring depth (as many stages
// as fit beside the 16 KB of epilogue tiles).
template <int MODE>
bool lookup(int V, int tile, PanelChoice* out, int gather = shflbw::kGatherCpAsync, bool wide_epilogue = false) {
    if constexpr (MODE == shflbw::kPanelSpmm || MODE == shflbw::kPanelConvChain) {
        // Shallow items (at most 64 non-zero columns): sixteen epilogue warps and three producer
        // warps, each a group of its own (20 warps: 96 registers per thread); stages of 32 columns,
        // eight of them beside the 32 KB of epilogue tiles, so that up to eight items' inputs are
        // in flight from HBM.  Built for 64-row blocks.
        if (wide_epilogue && tile == 256 && V == 64) {
            *out = choice<64, 2, 32, 8, 3, MODE, 3, 1, shflbw::kGatherCpAsync, 16>();
            return true;
        }
    }
    if constexpr (MODE == shflbw::kPanelSpmmRows || MODE == shflbw::kPanelConvChainRows) {   // rows in TMEM lanes: V must be a legal UMMA M
#ifdef SHFLBW_TUNE
        if (V == 64 && tile == 256 && tuned_shape<MODE>(out)) return true;
#endif
        if constexpr (MODE == shflbw::kPanelSpmmRows) {
            // SpMM, 64-row blocks, 256-token items: the rows of B come by TMA tile-gather, issued by
            // 16 light producer warps in four groups (measured 3-6 % faster than the cp.async gather
            // on the 4096^3 case; the copy engine also applies the swizzle and zero-fills the N residue)
            if (gather == shflbw::kGatherTma && V == 64 && tile == 256) {
                *out = choice<64, 2, 64, 5, 16, MODE, 4, 1, shflbw::kGatherTma>();
                return true;
            }
        }
        switch (V * 1000 + tile) {
            case 64128:  *out = choice<64, 1, 64, 8, 8, MODE>(); return true;
            case 64256:  *out = choice<64, 2, 64, 5, 8, MODE>(); return true;
            case 128128: *out = choice<128, 1, 64, 6, 8, MODE>(); return true;
            case 128256: *out = choice<128, 2, 64, 4, 8, MODE>(); return true;
            default: return false;
        }
    } else {
        if constexpr (MODE == shflbw::kPanelSpmm || MODE == shflbw::kPanelConv) {
            // 16-row blocks: UMMA N = 16, one or two 128-token accumulators per item (18 / 34 KB stages)
            if (V == 16 && tile == 128) { *out = choice<16, 1, 64, 8, 8, MODE>(); return true; }
            if (V == 16 && tile == 256) { *out = choice<16, 2, 64, 5, 8, MODE>(); return true; }
        }
        switch (V * 1000 + tile) {
            case 32128:  *out = choice<32, 1, 64, 8, 8, MODE>(); return true;    // 20 KB stages
            case 32256:  *out = choice<32, 2, 64, 5, 8, MODE>(); return true;    // 36 KB
            case 64128:  *out = choice<64, 1, 64, 8, 8, MODE>(); return true;    // 24 KB
            case 64256:  *out = choice<64, 2, 64, 5, 8, MODE>(); return true;    // 40 KB
            case 128128: *out = choice<128, 1, 64, 6, 8, MODE>(); return true;   // 32 KB
            case 128256: *out = choice<128, 2, 64, 4, 8, MODE>(); return true;   // 48 KB
            default: return false;
        }
    }
}

// Persistent launch: one CTA per SM, more only when a CTA's share would overflow its item table.
unsigned persistent_grid(int num_items, int sms) {
    int g = num_items < sms ? num_items : sms;
    const int need = (num_items + shflbw::kPanelMaxItemsPerCta - 1) / shflbw::kPanelMaxItemsPerCta;
    return (unsigned)(g > need ? g : need);
}

constexpr int kMaxDevices = 64;

// SM count of the current device, looked up once per device.
int sm_count() {
    static int cached[kMaxDevices] = {};
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (dev >= 0 && dev < kMaxDevices && cached[dev] > 0) return cached[dev];
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (dev >= 0 && dev < kMaxDevices) cached[dev] = n;
    return n;
}

// Opt a panel kernel in to its dynamic shared memory once per (device, kernel): the host-buffer
// calls initialise an op per chunk, and the attribute call is not free.
int allow_smem(PanelKernel fn, size_t bytes) {
    struct Done { const void* fn; int dev; };
    static Done done[256];
    static int n_done = 0;
    int dev = 0;
    CK(cudaGetDevice(&dev));
    for (int i = 0; i < n_done; ++i) if (done[i].fn == (const void*)fn && done[i].dev == dev) return SHFLBW_OK;
    CK(cudaFuncSetAttribute((const void*)fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    if (n_done < 256) done[n_done++] = {(const void*)fn, dev};
    return SHFLBW_OK;
}

// Tile selection.  A 256-token work item halves the value-panel traffic per token and is
// the default; 128 is used when the dense extent is too small to give every SM a few items.
// SHFLBW_TILE=128|256 overrides (tuning aid).
template <int MODE>
int pick_panel(int V, long long n_tokens, int row_blocks, long long padded_cols, PanelChoice* out) {
    // Token tile: a persistent CTA works through ceil(items / SMs) items in turn; an item of
    // the 128-token tile was measured at ~2/3 of the time of a 256-token item (half the
    // gathered bytes, the same number of pipeline stages).
    int tile = 256;
    const int sms = sm_count() > 0 ? sm_count() : 148;
    const long long items256 = ((n_tokens + 255) / 256) * row_blocks;
    const long long items128 = ((n_tokens + 127) / 128) * row_blocks;
    const long long waves256 = (items256 + sms - 1) / sms, waves128 = (items128 + sms - 1) / sms;
    if (n_tokens <= 128 || waves128 * 2 < waves256 * 3) tile = 128;
    if (const char* e = getenv("SHFLBW_TILE")) { int t = atoi(e); if (t == 128 || t == 256) tile = t; }
    if constexpr (MODE != shflbw::kPanelSpmm && MODE != shflbw::kPanelConv) {
        if (V == 16) tile = 128;   // chained layers: the only shape built for 16-row blocks
    }
    // SpMM and chained SpConv with V = 64 / 128 can run with the operands swapped (rows in TMEM
    // lanes, one MMA per 16 columns for the whole token tile); SHFLBW_SWAP=0|1 forces the choice
    // (tuning aid).
    bool swapped = false;
    if constexpr (MODE == shflbw::kPanelSpmm || MODE == shflbw::kPanelConvChain) {
        const char* e = getenv("SHFLBW_SWAP");
        // Worth it when the main loop dominates an item (>= 3 pipeline stages of non-zero columns
        // per block on average); with fewer columns the item is all epilogue, and the
        // rows-in-lanes epilogue of a 64-row block keeps only half of each warp's lanes busy.
        const bool deep = padded_cols >= 192ll * row_blocks;
        if ((V == 64 || V == 128) && (e ? atoi(e) != 0 : deep)) {
            // TMA gather (SHFLBW_GATHER=0 keeps cp.async; tuning aid) when every SM gets at least two items
            int gather = shflbw::kGatherCpAsync;
            if (MODE == shflbw::kPanelSpmm && V == 64 && tile == 256 && items256 >= 2ll * sms) gather = shflbw::kGatherTma;
            if (const char* g = getenv("SHFLBW_GATHER")) gather = atoi(g) == 1 && V == 64 && tile == 256 && MODE == shflbw::kPanelSpmm && n_tokens >= 64
                                                                      ? shflbw::kGatherTma : shflbw::kGatherCpAsync;
            swapped = MODE == shflbw::kPanelSpmm ? lookup<shflbw::kPanelSpmmRows>(V, tile, out, gather)
                                                 : lookup<shflbw::kPanelConvChainRows>(V, tile, out);
        }
    }
    // Tokens in lanes with at most one stage of non-zero columns per block on average (an item is
    // then all epilogue; with two stages the four producers of that kernel were measured slower
    // than the eight of the regular one) and several items per SM: sixteen epilogue warps.  SHFLBW_EPILOGUE_WARPS=8|16 forces the choice
    // (tuning aid).
    bool wide = false;
    if constexpr (MODE == shflbw::kPanelSpmm || MODE == shflbw::kPanelConvChain) {
        wide = !swapped && tile == 256 && V == 64 && padded_cols <= 64ll * row_blocks && items256 >= 4ll * sms;
        if (const char* e = getenv("SHFLBW_EPILOGUE_WARPS")) wide = !swapped && tile == 256 && V == 64 && atoi(e) == 16;
    }
    if (!swapped && !lookup<MODE>(V, tile, out, shflbw::kGatherCpAsync, wide)) return SHFLBW_ERR_UNSUPPORTED;
    out->variant = swapped ? 1 : wide ? 2 : 0;
    return allow_smem(out->fn, out->smem);
}

// Argument and range checks shared by every NHWC SpConv entry point.  The kernels index the
// staged input with 32-bit element offsets and the output with 32-bit offsets whose all-ones
// value is a sentinel, so both extents are bounded here, before anything is launched.
struct ConvShape { int Ho, Wo, Bp; long long tokens, staged_elems; };
int check_conv_call(const shflbw_matrix* f, int B, int Hin, int Win, int stride, const void* ifmap,
                    const void* ofmap, ConvShape* cs) {
    if (!f || !ifmap || !ofmap || B <= 0 || Hin <= 0 || Win <= 0 || stride <= 0) return SHFLBW_ERR_INVALID_ARG;
    if (!f->is_filter) return SHFLBW_ERR_INVALID_ARG;
    if (!on_current_device(*f)) return SHFLBW_ERR_NOT_ON_DEVICE;
    if (f->C % 8 || f->R > 255 || f->S > 255) return SHFLBW_ERR_UNSUPPORTED;
    if (((uintptr_t)ifmap | (uintptr_t)ofmap) & 15) return SHFLBW_ERR_UNSUPPORTED;
    if (B > (1 << 24) || Hin > (1 << 24) || Win > (1 << 24)) return SHFLBW_ERR_UNSUPPORTED;   // keeps the products below in 64 bits
    cs->Ho = (Hin + stride - 1) / stride; cs->Wo = (Win + stride - 1) / stride;
    cs->Bp = (B + 7) / 8 * 8;
    cs->tokens = (long long)cs->Ho * cs->Wo * cs->Bp;
    const long long plane = (long long)(Hin + f->R - 1) * (Win + f->S - 1);        // < 2^50
    if (plane >= (1ll << 31) || cs->tokens >= (1ll << 31)) return SHFLBW_ERR_UNSUPPORTED;
    cs->staged_elems = plane * cs->Bp;                                              // < 2^56
    if (cs->staged_elems >= (1ll << 31) || cs->staged_elems * f->C >= (1ll << 31)) return SHFLBW_ERR_UNSUPPORTED;
    cs->staged_elems *= f->C;
    if ((long long)B * cs->Ho * cs->Wo >= (1ll << 32) || (long long)B * cs->Ho * cs->Wo * f->F >= (1ll << 32) - 1)
        return SHFLBW_ERR_UNSUPPORTED;                                              // 32-bit output offsets
    return SHFLBW_OK;
}

int check_kernel_arg(int kernel) {
    return (kernel == SHFLBW_KERNEL_AUTO || kernel == SHFLBW_KERNEL_TCGEN05 || kernel == SHFLBW_KERNEL_SIMT)
               ? SHFLBW_OK : SHFLBW_ERR_INVALID_ARG;
}

}  // namespace

// Scratch of shflbw_spconv_exec_static_scratch: part of the library image, present on every
// GPU that loads the library.  In HOST code this name is only a handle for
// cudaGetSymbolAddress -- it is not a device address and must never be handed to a kernel.
static __device__ __align__(256) unsigned char g_static_scratch[SHFLBW_STATIC_SCRATCH_BYTES];

namespace {
void* g_static_scratch_addr[kMaxDevices] = {};  // device address of the array, per device
}  // namespace

namespace shflbw {
void drop_device_copy(shflbw_matrix& m) {
    void** bufs[] = {&m.d_meta, &m.d_val, &m.stage_in, &m.stage_c, &m.stage_out, &m.conv_in, &m.conv_out};
    for (void** b : bufs) if (*b) { cudaFree(*b); *b = nullptr; }
    for (void* r : m.retired) cudaFree(r);
    m.retired.clear();
    for (void*& st : m.host_streams) if (st) { cudaStreamDestroy((cudaStream_t)st); st = nullptr; }
    for (void*& ev : m.host_events) if (ev) { cudaEventDestroy((cudaEvent_t)ev); ev = nullptr; }
    m.stage_in_bytes = m.stage_c_bytes = m.stage_out_bytes = m.conv_in_bytes = m.conv_out_bytes = 0;
    m.d_kptr = m.d_kidx = m.d_perm = m.d_kcrs = nullptr;
    m.d_status = nullptr;
    m.device = -1;
}
}  // namespace shflbw

extern "C" {

const char* shflbw_last_cuda_error(void) { return g_cuda_err; }

int shflbw_set_wait_limit_cycles(long long cycles) {
    if (cycles < 1000) return SHFLBW_ERR_INVALID_ARG;
    g_wait_limit = cycles;
    return SHFLBW_OK;
}

#ifdef SHFLBW_FAULT_INJECT
// Test builds only: launches issued after this call run with one producer warp withholding its
// barrier arrivals from stage `stage` on (< 0: off), so that the consumer's bounded wait gives up.
int shflbw_debug_withhold_arrivals_from(int stage) { g_inject_from = stage; return SHFLBW_OK; }
#endif

int shflbw_matrix_to_device(shflbw_matrix_t* m) {
    if (!m) return SHFLBW_ERR_INVALID_ARG;
    if (m->d_meta) return SHFLBW_OK;
    int rc = shflbw::validate(*m);
    if (rc != SHFLBW_OK) return rc;
    shflbw::build_host_images(*m);
    int dev = 0;
    CK(cudaGetDevice(&dev));
    auto up8 = [](size_t v) { return (v + 7) / 8 * 8; };
    const size_t o_ptr = 0, o_idx = up8(m->kptr.size()), o_perm = o_idx + up8(m->kidx.size()),
                 o_crs = o_perm + up8(m->row_permute_ids.size()), o_stat = o_crs + up8(m->kcrs.size()),
                 total = o_stat + 8;
    std::vector<int> img(total, 0);
    std::copy(m->kptr.begin(), m->kptr.end(), img.begin() + o_ptr);
    std::copy(m->kidx.begin(), m->kidx.end(), img.begin() + o_idx);
    std::copy(m->row_permute_ids.begin(), m->row_permute_ids.end(), img.begin() + o_perm);
    std::copy(m->kcrs.begin(), m->kcrs.end(), img.begin() + o_crs);
    CK(cudaMalloc(&m->d_meta, total * sizeof(int)));
    if (!cuda_ok(cudaMalloc(&m->d_val, m->kval.size() * 2), "cudaMalloc(values)")) {
        cudaFree(m->d_meta); m->d_meta = nullptr;
        return SHFLBW_ERR_CUDA;
    }
    CK(cudaMemcpy(m->d_meta, img.data(), total * sizeof(int), cudaMemcpyHostToDevice));
    CK(cudaMemcpy(m->d_val, m->kval.data(), m->kval.size() * 2, cudaMemcpyHostToDevice));
    const int* base = (const int*)m->d_meta;
    m->d_kptr = base + o_ptr;
    m->d_kidx = base + o_idx;
    m->d_perm = m->row_permute ? base + o_perm : nullptr;
    m->d_kcrs = m->kcrs.empty() ? nullptr : base + o_crs;
    m->d_status = (int*)m->d_meta + o_stat;
    m->device = dev;
    return SHFLBW_OK;
}

int shflbw_matrix_on_device(const shflbw_matrix_t* m) { return m && m->d_meta ? 1 : 0; }

int shflbw_matrix_device_status(const shflbw_matrix_t* m) {
    if (!m || !m->d_status) return SHFLBW_ERR_NOT_ON_DEVICE;
    int word = 0;
    CK(cudaDeviceSynchronize());
    CK(cudaMemcpy(&word, m->d_status, sizeof word, cudaMemcpyDeviceToHost));
    if (word != 0) {
        CK(cudaMemset(m->d_status, 0, sizeof word));
        snprintf(g_cuda_err, sizeof g_cuda_err, "device status word = %d", word);
        return SHFLBW_ERR_DEVICE_TIMEOUT;
    }
    return SHFLBW_OK;
}

// ------------------------------------------------------------------------------ SpMM --

int shflbw_spmm_init(const shflbw_matrix_t* m, int N, const void* B, float alpha, const void* C,
                     float beta, void* D, int kernel, shflbw_spmm_state_t* out) {
    if (!out) return SHFLBW_ERR_INVALID_ARG;
    std::memset(out, 0, sizeof *out);
    if (!m || !B || !D || N <= 0) return SHFLBW_ERR_INVALID_ARG;
    if (check_kernel_arg(kernel) != SHFLBW_OK) return SHFLBW_ERR_INVALID_ARG;
    if (beta != 0.f && !C) return SHFLBW_ERR_INVALID_ARG;
    if (!on_current_device(*m)) return SHFLBW_ERR_NOT_ON_DEVICE;  // reference: assert(device_synced)
    // The reference asserts bcol == 1 here (spmm/blockwise_op.h:86); the kernel image lists the
    // bcol columns of a block one by one, so wider blocks run on the same kernels.
    // Row-block heights 16/32/64/128 (what the reference instantiates, spmm/blockwise_library.cu:15-31)
    // run on the tensor-core kernel.
    if (kernel != SHFLBW_KERNEL_SIMT && m->brow != 16 && m->brow != 32 && m->brow != 64 && m->brow != 128)
        return SHFLBW_ERR_UNSUPPORTED;
    if (kernel == SHFLBW_KERNEL_SIMT && (N + 127) / 128 > 65535) return SHFLBW_ERR_UNSUPPORTED;   // column tiles ride in grid.y
    if (N % 8) return SHFLBW_ERR_UNSUPPORTED;                   // 16-byte rows of fp16
    const uintptr_t al = (uintptr_t)B | (uintptr_t)D | (uintptr_t)C;
    if (al & 15) return SHFLBW_ERR_UNSUPPORTED;
    if ((long long)m->nrow * N >= (1ll << 32) || (long long)m->ncol * N >= (1ll << 40))
        return SHFLBW_ERR_UNSUPPORTED;                          // 32-bit element offsets into C / D

    out->M = m->nrow; out->N = N; out->K = m->ncol; out->V = m->brow;
    out->num_row_blocks = m->nrow / m->brow;
    out->alpha = alpha; out->beta = beta;
    out->B = B; out->C = C; out->D = D;
    out->blk_ptr = m->d_kptr; out->blk_idx = m->d_kidx; out->blk_val = m->d_val;
    out->perm = m->d_perm; out->status_word = m->d_status;
    if (kernel == SHFLBW_KERNEL_SIMT) {
        out->kernel = SHFLBW_KERNEL_SIMT;
        out->block_x = 128; out->grid_x = m->nrow; out->grid_y = (N + 127) / 128;   // rows in grid.x: no 65535 limit
        out->tokens_per_cta = 128; out->stages = 0; out->shared_mem_size = 0;
    } else {
        PanelChoice ch;
        int rc = pick_panel<shflbw::kPanelSpmm>(m->brow, N, out->num_row_blocks, m->kptr.empty() ? 0 : m->kptr.back(), &ch);
        if (rc != SHFLBW_OK) return rc;
        out->kernel = SHFLBW_KERNEL_TCGEN05;
        out->tokens_per_cta = ch.tokens; out->stages = ch.stages; out->producer_warps = ch.pw; out->variant = ch.variant;
        out->gather = ch.gather;
        if (ch.gather == shflbw::kGatherTma && (rc = encode_b_map(B, m->ncol, N, out->tmap_b)) != SHFLBW_OK) return rc;
        out->tiles_n = (N + ch.tokens - 1) / ch.tokens;
        out->num_items = out->tiles_n * out->num_row_blocks;
        const int sms = sm_count();
        if (sms <= 0) return SHFLBW_ERR_CUDA;
        out->block_x = ch.threads;
        out->grid_x = persistent_grid(out->num_items, sms); out->grid_y = 1;
        out->shared_mem_size = ch.smem;
    }
    out->init_success = 1;
    return SHFLBW_OK;
}

int shflbw_spmm_exec(const shflbw_spmm_state_t* st, void* stream) {
    if (!st || !st->init_success) return SHFLBW_ERR_INVALID_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (st->kernel == SHFLBW_KERNEL_SIMT) {
        shflbw::simt_spmm<<<dim3(st->grid_x, st->grid_y), st->block_x, 0, s>>>(
            st->blk_ptr, st->blk_idx, (const __half*)st->blk_val, st->perm, (const __half*)st->B,
            (const __half*)st->C, (__half*)st->D, st->M, st->N, st->V, st->alpha, st->beta);
    } else {
        // The state is a POD and may have been copied: re-derive the function pointer from the
        // recorded configuration (the shared-memory attribute was set at init).
        PanelChoice ch;
        const bool found = st->variant == 1 ? lookup<shflbw::kPanelSpmmRows>(st->V, st->tokens_per_cta, &ch, st->gather)
                                            : lookup<shflbw::kPanelSpmm>(st->V, st->tokens_per_cta, &ch, shflbw::kGatherCpAsync, st->variant == 2);
        if (!found) return SHFLBW_ERR_INVALID_ARG;
        shflbw::PanelParams p{};
        p.blk_ptr = st->blk_ptr; p.blk_idx = st->blk_idx; p.blk_val = (const __half*)st->blk_val;
        p.perm = st->perm; p.status_word = st->status_word; p.alpha = st->alpha; p.beta = st->beta;
        p.wait_limit = g_wait_limit; p.inject_from = g_inject_from; p.idx_limit = (unsigned)(st->K - 1);
        p.B = (const __half*)st->B; p.C = (const __half*)st->C; p.D = (__half*)st->D; p.N = st->N;
        p.wide_stores = (st->N % 16 == 0) && (((uintptr_t)st->D & 31) == 0);
        if (ch.gather != st->gather) return SHFLBW_ERR_INVALID_ARG;
        if (st->gather == shflbw::kGatherTma) std::memcpy(p.tmap_b, st->tmap_b, sizeof p.tmap_b);
        p.num_items = st->num_items; p.tiles_n = st->tiles_n;
        p.div_tiles = shflbw::make_fast_div(st->tiles_n); p.div_bp = p.div_wo = shflbw::make_fast_div(1);
        // Tile-major item order: concurrent CTAs gather from the same few token tiles of B (SHFLBW_ITEM_ORDER=0|1
        // forces block-major / tile-major; tuning aid).
        p.num_blocks = st->num_row_blocks; p.div_blocks = shflbw::make_fast_div(st->num_row_blocks);
        p.tile_major = 1;
        if (const char* e = getenv("SHFLBW_ITEM_ORDER")) p.tile_major = atoi(e) != 0;
#if defined(SHFLBW_ABLATE) || defined(SHFLBW_COUNTERS)
        if (const char* e = getenv("SHFLBW_ABLATE")) p.ablate = atoi(e);
        if (const char* e = getenv("SHFLBW_TRACE_PTR")) p.trace = (unsigned long long*)strtoull(e, nullptr, 0);
#endif
        CK(launch(ch.fn, dim3(st->grid_x, st->grid_y), dim3(ch.threads), ch.smem, s, p));
    }
    CK(cudaGetLastError());
    return SHFLBW_OK;
}

int shflbw_spmm_launches_per_exec(const shflbw_spmm_state_t* st) { return st && st->init_success ? 1 : 0; }

// Host-buffer SpMM.  The dense operand is cut into column chunks that move through three
// streams -- host-to-device copy of chunk i+1, kernel on chunk i, device-to-host copy of chunk
// i-1 -- so that on a full-duplex link the call costs about the larger of the two transfers
// instead of their sum plus the kernel.  (Overlap needs page-locked host buffers; pageable ones
// work, the copies then serialise.)  A chunk is staged contiguously ([K][w] / [M][w]) by a strided
// 2-D copy, so the kernels run unchanged on dense chunks.
// mode 0: the real call.  1: the same copies through the same streams and events, no kernel
// (what the link alone costs).  2: as 1, but every chunk moves as one contiguous block of the
// same size (what the strided form of the chunk copies costs on top).
static int spmm_host_impl(shflbw_matrix_t* m, int N, const void* B_host, float alpha, const void* C_host,
                          float beta, void* D_host, int mode) {
    if (!m || !B_host || !D_host || N <= 0) return SHFLBW_ERR_INVALID_ARG;
    if (beta != 0.f && !C_host) return SHFLBW_ERR_INVALID_ARG;
    if (N % 8) return SHFLBW_ERR_UNSUPPORTED;
    int rc = shflbw_matrix_to_device(m);
    if (rc != SHFLBW_OK) return rc;
    // Before any staging buffer or stream is made: they would belong to the wrong GPU.
    if (!on_current_device(*m)) return SHFLBW_ERR_NOT_ON_DEVICE;
    const size_t bB = (size_t)m->ncol * N * 2, bD = (size_t)m->nrow * N * 2;
    if ((rc = ensure_buffer(&m->stage_in, &m->stage_in_bytes, bB)) != SHFLBW_OK) return rc;
    if ((rc = ensure_buffer(&m->stage_out, &m->stage_out_bytes, bD)) != SHFLBW_OK) return rc;
    if (beta != 0.f && (rc = ensure_buffer(&m->stage_c, &m->stage_c_bytes, bD)) != SHFLBW_OK) return rc;

    // chunk width: a quarter of N rounded up to whole 256-token tiles; narrow operands go in one piece
    int w = N;
    int want = 4;
    if (const char* e = getenv("SHFLBW_HOST_CHUNKS")) want = atoi(e) > 0 && atoi(e) <= 8 ? atoi(e) : 4;
    if (N >= 2048 && want > 1) w = ((N + want - 1) / want + 255) / 256 * 256;
    const int chunks = (N + w - 1) / w;
    constexpr int kMaxChunks = 8;
    if (chunks > kMaxChunks) return SHFLBW_ERR_UNSUPPORTED;   // cannot happen: w >= N/4

    // streams and events live in the handle (creating and destroying them costs more than the
    // overlap gains on a call of about a millisecond)
    auto fail = [&](int code) { cudaDeviceSynchronize(); return code; };
#define CKH(call) do { if (!cuda_ok((call), #call)) return fail(SHFLBW_ERR_CUDA); } while (0)
    cudaStream_t s_in, s_k, s_out;
    cudaEvent_t *e_in, *e_k;
    if ((rc = host_pipeline(m, &s_in, &s_k, &s_out, &e_in, &e_k)) != SHFLBW_OK) return rc;
    const size_t pitch_h = (size_t)N * 2;
    for (int i = 0; i < chunks; ++i) {
        const int c0 = i * w, wi = (N - c0 < w) ? N - c0 : w;
        // chunk i of the staging buffers: contiguous [rows][wi] blocks, one after the other
        __half* dB = (__half*)m->stage_in + (size_t)m->ncol * c0;
        __half* dD = (__half*)m->stage_out + (size_t)m->nrow * c0;
        __half* dC = beta != 0.f ? (__half*)m->stage_c + (size_t)m->nrow * c0 : nullptr;
        if (mode == 2)
            CKH(cudaMemcpyAsync(dB, (const __half*)B_host + (size_t)m->ncol * c0, (size_t)wi * 2 * m->ncol,
                                cudaMemcpyHostToDevice, s_in));
        else
        CKH(cudaMemcpy2DAsync(dB, (size_t)wi * 2, (const __half*)B_host + c0, pitch_h, (size_t)wi * 2, m->ncol,
                              cudaMemcpyHostToDevice, s_in));
        if (dC)
            CKH(cudaMemcpy2DAsync(dC, (size_t)wi * 2, (const __half*)C_host + c0, pitch_h, (size_t)wi * 2, m->nrow,
                                  cudaMemcpyHostToDevice, s_in));
        CKH(cudaEventRecord(e_in[i], s_in));
        CKH(cudaStreamWaitEvent(s_k, e_in[i], 0));
        if (mode == 0) {
            shflbw_spmm_state_t st;
            rc = shflbw_spmm_init(m, wi, dB, alpha, dC, beta, dD, SHFLBW_KERNEL_AUTO, &st);
            if (rc == SHFLBW_OK) rc = shflbw_spmm_exec(&st, s_k);
            if (rc != SHFLBW_OK) return fail(rc);
        }
        CKH(cudaEventRecord(e_k[i], s_k));
        CKH(cudaStreamWaitEvent(s_out, e_k[i], 0));
        if (mode == 2)
            CKH(cudaMemcpyAsync((__half*)D_host + (size_t)m->nrow * c0, dD, (size_t)wi * 2 * m->nrow,
                                cudaMemcpyDeviceToHost, s_out));
        else
        CKH(cudaMemcpy2DAsync((__half*)D_host + c0, pitch_h, dD, (size_t)wi * 2, (size_t)wi * 2, m->nrow,
                              cudaMemcpyDeviceToHost, s_out));
    }
    CKH(cudaStreamSynchronize(s_out));
    CKH(cudaStreamSynchronize(s_k));
    CKH(cudaStreamSynchronize(s_in));
#undef CKH
    return SHFLBW_OK;
}

int shflbw_spmm_host(shflbw_matrix_t* m, int N, const void* B_host, float alpha, const void* C_host,
                     float beta, void* D_host) {
    return spmm_host_impl(m, N, B_host, alpha, C_host, beta, D_host, 0);
}

int shflbw_spmm_host_copies_only(shflbw_matrix_t* m, int N, const void* B_host, void* D_host, int contiguous) {
    return spmm_host_impl(m, N, B_host, 1.0f, nullptr, 0.0f, D_host, contiguous ? 2 : 1);
}

// ---------------------------------------------------------------------------- SpConv --

// NHWC -> [C][Hin+R-1][Win+S-1][Bp] with a zero halo (origin at (R/2, S/2)).
static void launch_relayout(const __half* in, __half* staged, int B, int Bp, int Hin, int Win, int C, int R, int S,
                            cudaStream_t s) {
    const int Hp = Hin + R - 1, Wp = Win + S - 1, PP = Hp * Wp;
    const int NT = Bp < 32 ? Bp : 32, PT = shflbw::kRelayoutSlots / NT;
    const int n_tiles = (Bp + NT - 1) / NT;
    dim3 grid((unsigned)(((PP + PT - 1) / PT) * n_tiles), (unsigned)((C + shflbw::kRelayoutC - 1) / shflbw::kRelayoutC));
    (void)launch(shflbw::relayout_nhwc_to_chwn, grid, dim3(256), 0, s, in, staged, B, Bp, Hin, Win, Hp, Wp, R / 2, S / 2, C);
}

// Dynamic shared memory of unpermute_filters: 16-bit permutation + one F-vector of fp16 per position.
static size_t unperm_smem_bytes(int F) {
    return (size_t)F * 2 * (1 + shflbw::kUnpermThreads / shflbw::unperm_threads_per_pos(F));
}

// Launch plan of one NHWC SpConv call, without its scratch pointers: kernel choice, grid, and
// the scratch each side needs.  Two plans exist.
//   positions out   relayout -> panel kernel with tokens in TMEM lanes, writing [position][F] in
//                   stored filter order -> (with a filter permutation) unpermute_filters.
//   planes out      relayout -> panel kernel with the filters in TMEM lanes, writing the output
//                   as planes [F][Ho][Wo][Bp] with plane = LOGICAL channel (the permutation is
//                   the row index of its stores, free) -> planes_to_nhwc transposes the planes
//                   to NHWC.  Used for V = 64 / 128 filters with enough non-zero columns per
//                   block: one MMA per 16 columns covers the whole token tile.
// SHFLBW_CONV_PLANES=0|1 forces the choice (tuning aid).
int plan_conv(const shflbw_matrix* f, int B, int Hin, int Win, int stride, const void* ifmap, void* ofmap,
              float alpha, int kernel, shflbw_spconv_state_t* out) {
    std::memset(out, 0, sizeof *out);
    if (check_kernel_arg(kernel) != SHFLBW_OK) return SHFLBW_ERR_INVALID_ARG;
    ConvShape cs;
    int rc = check_conv_call(f, B, Hin, Win, stride, ifmap, ofmap, &cs);
    if (rc != SHFLBW_OK) return rc;
    if (kernel != SHFLBW_KERNEL_SIMT && f->brow != 16 && f->brow != 32 && f->brow != 64 && f->brow != 128)
        return SHFLBW_ERR_UNSUPPORTED;
    const int Ho = cs.Ho, Wo = cs.Wo, Bp = cs.Bp;
    const long long tokens = cs.tokens;

    out->B = B; out->Hin = Hin; out->Win = Win; out->C = f->C; out->F = f->F; out->R = f->R; out->S = f->S;
    out->stride = stride; out->Ho = Ho; out->Wo = Wo; out->V = f->brow; out->Bp = Bp;
    out->alpha = alpha; out->ifmap = ifmap; out->ofmap = ofmap;
    out->blk_ptr = f->d_kptr; out->blk_idx = f->d_kidx; out->blk_val = f->d_val;
    out->perm = f->d_perm; out->status_word = f->d_status;
    if (kernel == SHFLBW_KERNEL_SIMT) {
        if ((f->F + 127) / 128 > 65535) return SHFLBW_ERR_UNSUPPORTED;
        out->kernel = SHFLBW_KERNEL_SIMT;
        out->block_x = 128; out->grid_x = (unsigned)(B * Ho * Wo); out->grid_y = (f->F + 127) / 128;   // positions in grid.x
        out->init_success = 1;
        return SHFLBW_OK;
    }
    // The panel kernel reads decoded column ids (channel in 16 bits, taps in 8 bits each).
    if (!f->d_kcrs) return SHFLBW_ERR_UNSUPPORTED;
    out->blk_idx = f->d_kcrs;
    const int row_blocks = f->F / f->brow;
    const long long padded_cols = f->kptr.empty() ? 0 : f->kptr.back();

    // planes out?
    PanelChoice ch;
    bool planes = false;
    const bool planes_possible = (f->brow == 64 || f->brow == 128) && f->F / 64 <= 65535 &&
                                 (long long)f->F * tokens < (1ll << 32) - 1;
    if (planes_possible) {
        bool want = padded_cols >= 192ll * row_blocks;      // same rule as the chained layers: >= 3 stages per block
        if (const char* e = getenv("SHFLBW_CONV_PLANES")) want = atoi(e) != 0;
        if (want) {
            rc = pick_panel<shflbw::kPanelConvChain>(f->brow, tokens, row_blocks, want ? (1ll << 40) : 0, &ch);
            if (rc != SHFLBW_OK) return rc;
            planes = ch.variant == 1;
        }
    }
    if (planes) {
        out->variant = 1;
        out->staged_out_bytes = (size_t)f->F * (size_t)tokens * 2;
    } else {
        rc = pick_panel<shflbw::kPanelConv>(f->brow, tokens, row_blocks, 0, &ch);
        if (rc != SHFLBW_OK) return rc;
        out->variant = 0;
        if (f->row_permute) {
            out->staged_out_bytes = (size_t)B * Ho * Wo * f->F * 2;
            if (unperm_smem_bytes(f->F) > 227 * 1024 || f->F > 65536) return SHFLBW_ERR_UNSUPPORTED;
            if (unperm_smem_bytes(f->F) > 48 * 1024)
                CK(cudaFuncSetAttribute((const void*)shflbw::unpermute_filters,
                                        cudaFuncAttributeMaxDynamicSharedMemorySize, (int)unperm_smem_bytes(f->F)));
        }
    }
    out->kernel = SHFLBW_KERNEL_TCGEN05;
    out->tokens_per_cta = ch.tokens; out->stages = ch.stages; out->producer_warps = ch.pw;
    out->tiles_n = (int)((tokens + ch.tokens - 1) / ch.tokens);
    out->num_items = out->tiles_n * row_blocks;
    const int sms = sm_count();
    if (sms <= 0) return SHFLBW_ERR_CUDA;
    out->block_x = ch.threads;
    out->grid_x = persistent_grid(out->num_items, sms); out->grid_y = 1;
    out->shared_mem_size = ch.smem;
    out->staged_in_bytes = (size_t)cs.staged_elems * 2;
    return SHFLBW_OK;
}

int shflbw_spconv_init(shflbw_matrix_t* f, int B, int Hin, int Win, int stride, const void* ifmap,
                       void* ofmap, float alpha, int kernel, shflbw_spconv_state_t* out) {
    if (!out) return SHFLBW_ERR_INVALID_ARG;
    int rc = plan_conv(f, B, Hin, Win, stride, ifmap, ofmap, alpha, kernel, out);
    if (rc != SHFLBW_OK || out->kernel == SHFLBW_KERNEL_SIMT) return rc;
    // Scratch owned by the filter handle, grown on demand.
    if ((rc = grow_scratch(*f, &f->conv_in, &f->conv_in_bytes, out->staged_in_bytes)) != SHFLBW_OK) return rc;
    out->staged_in = f->conv_in;
    if (out->staged_out_bytes) {
        if ((rc = grow_scratch(*f, &f->conv_out, &f->conv_out_bytes, out->staged_out_bytes)) != SHFLBW_OK) return rc;
        out->staged_out = f->conv_out;
    }
    out->init_success = 1;
    return SHFLBW_OK;
}

int shflbw_spconv_exec(const shflbw_spconv_state_t* st, void* stream) {
    if (!st || !st->init_success) return SHFLBW_ERR_INVALID_ARG;
    cudaStream_t s = (cudaStream_t)stream;
    if (st->kernel == SHFLBW_KERNEL_SIMT) {
        shflbw::simt_spconv<<<dim3(st->grid_x, st->grid_y), st->block_x, 0, s>>>(
            st->blk_ptr, st->blk_idx, (const __half*)st->blk_val, st->perm, (const __half*)st->ifmap,
            (__half*)st->ofmap, st->B, st->Hin, st->Win, st->C, st->F, st->R, st->S, st->stride, st->Ho,
            st->Wo, st->V, st->alpha);
        CK(cudaGetLastError());
        return SHFLBW_OK;
    }
    const bool planes = !st->chain && st->variant == 1;     // NHWC call computed as planes, then transposed
    PanelChoice ch;
    const bool ok_kernel = (!st->chain && !planes) ? lookup<shflbw::kPanelConv>(st->V, st->tokens_per_cta, &ch)
                           : st->variant == 1      ? lookup<shflbw::kPanelConvChainRows>(st->V, st->tokens_per_cta, &ch)
                                                   : lookup<shflbw::kPanelConvChain>(st->V, st->tokens_per_cta, &ch, shflbw::kGatherCpAsync, st->variant == 2);
    if (!ok_kernel) return SHFLBW_ERR_INVALID_ARG;
    // 1. NHWC -> channel-major, batch-innermost staging with a zero halo (chained layers get
    //    their input in that layout already).
    const int Hp = st->Hin + st->R - 1, Wp = st->Win + st->S - 1;
    if (!st->chain)
        launch_relayout((const __half*)st->ifmap, (__half*)st->staged_in, st->B, st->Bp, st->Hin, st->Win, st->C,
                        st->R, st->S, s);
    // 2. implicit-GEMM panel kernel.
    shflbw::PanelParams p{};
    p.blk_ptr = st->blk_ptr; p.blk_idx = st->blk_idx; p.blk_val = (const __half*)st->blk_val;
    p.perm = st->perm; p.status_word = st->status_word; p.alpha = st->alpha; p.beta = 0.f;
    p.wait_limit = g_wait_limit; p.inject_from = g_inject_from;
    p.N = st->Ho * st->Wo * st->Bp;
    p.Xs = (const __half*)(st->chain ? st->ifmap : st->staged_in);
    p.out = (__half*)(st->staged_out ? st->staged_out : st->ofmap);
    if (st->chain) {
        p.res = (const __half*)st->residual; p.res_map = st->residual_map;
        const int OHp = st->Ho + st->out_R - 1;
        p.OWp = st->Wo + st->out_S - 1; p.oph = st->out_R / 2; p.opw = st->out_S / 2;
        p.out_plane = OHp * p.OWp * st->Bp; p.relu = st->relu;
    } else if (planes) {
        p.OWp = st->Wo; p.oph = 0; p.opw = 0; p.out_plane = st->Ho * st->Wo * st->Bp;
        p.out_logical = 1;                                   // plane index = logical channel
    }
    p.idx_limit = (unsigned)((((long long)st->C - 1) * Hp * Wp + (long long)(st->R - 1) * Wp + (st->S - 1)) * st->Bp);
    p.Bn = st->B; p.Bp = st->Bp; p.Hp = Hp; p.Wp = Wp; p.Cin = st->C; p.F = st->F;
    p.R = st->R; p.S = st->S; p.stride = st->stride; p.Ho = st->Ho; p.Wo = st->Wo;
    p.num_items = st->num_items; p.tiles_n = st->tiles_n;
    p.div_tiles = shflbw::make_fast_div(st->tiles_n); p.div_bp = shflbw::make_fast_div(st->Bp); p.div_wo = shflbw::make_fast_div(st->Wo);
    p.num_blocks = st->F / st->V; p.div_blocks = shflbw::make_fast_div(p.num_blocks);
    // Block-major item order for the convolutions: running a token tile's filter blocks at the same time
    // (tile-major) was measured equal on the ResNet-50 stack and on config 3, whose inputs are small next
    // to their outputs (SHFLBW_ITEM_ORDER=1 forces tile-major; tuning aid).
    p.tile_major = 0;
    if (const char* e = getenv("SHFLBW_ITEM_ORDER")) p.tile_major = atoi(e) != 0;
#if defined(SHFLBW_ABLATE) || defined(SHFLBW_COUNTERS)
    if (const char* e = getenv("SHFLBW_ABLATE")) p.ablate = atoi(e);
    if (const char* e = getenv("SHFLBW_TRACE_PTR")) p.trace = (unsigned long long*)strtoull(e, nullptr, 0);
#endif
    CK(launch(ch.fn, dim3(st->grid_x, st->grid_y), dim3(ch.threads), ch.smem, s, p));
    // 3. back to NHWC in logical channel order.
    if (planes) {
        const int npix = st->Ho * st->Wo;
        CK(launch(shflbw::planes_to_nhwc, dim3((unsigned)(((long long)npix * st->Bp + 63) / 64), (unsigned)(st->F / 64)), dim3(256), 0, s,
                  (const __half*)st->staged_out, (__half*)st->ofmap, st->B, st->Bp, npix, st->F));
    } else if (st->staged_out) {
        const int num_pos = st->B * st->Ho * st->Wo;
        const int per_block = shflbw::kUnpermThreads / shflbw::unperm_threads_per_pos(st->F);
        int blocks = (num_pos + per_block - 1) / per_block;
        if (blocks > 148 * 16) blocks = 148 * 16;
        CK(launch(shflbw::unpermute_filters, dim3(blocks), dim3(shflbw::kUnpermThreads), unperm_smem_bytes(st->F), s,
                  (const __half*)st->staged_out, (__half*)st->ofmap, st->perm, num_pos, st->F));
    }
    CK(cudaGetLastError());
    return SHFLBW_OK;
}

int shflbw_spconv_launches_per_exec(const shflbw_spconv_state_t* st) {
    if (!st || !st->init_success) return 0;
    if (st->kernel == SHFLBW_KERNEL_SIMT || st->chain) return 1;
    return st->staged_out ? 3 : 2;
}

// Host-buffer SpConv.  Batches of 32 images or more go in up to four chunks of whole 8-image
// groups (NHWC: a batch slice is contiguous on both sides) through the same three streams as
// the SpMM host call, so that copy in, kernels and copy out overlap.
int shflbw_spconv_host(shflbw_matrix_t* f, int B, int Hin, int Win, int stride, const void* ifmap_host,
                       void* ofmap_host, float alpha) {
    if (!f || !ifmap_host || !ofmap_host || !f->is_filter || B <= 0 || Hin <= 0 || Win <= 0 || stride <= 0)
        return SHFLBW_ERR_INVALID_ARG;
    int rc = shflbw_matrix_to_device(f);
    if (rc != SHFLBW_OK) return rc;
    if (!on_current_device(*f)) return SHFLBW_ERR_NOT_ON_DEVICE;   // before staging buffers / streams are made
    const int Ho = (Hin + stride - 1) / stride, Wo = (Win + stride - 1) / stride;
    const size_t img_in = (size_t)Hin * Win * f->C, img_out = (size_t)Ho * Wo * f->F;   // elements per image
    if ((rc = ensure_buffer(&f->stage_in, &f->stage_in_bytes, (size_t)B * img_in * 2)) != SHFLBW_OK) return rc;
    if ((rc = ensure_buffer(&f->stage_out, &f->stage_out_bytes, (size_t)B * img_out * 2)) != SHFLBW_OK) return rc;
    int per = B;                                     // images per chunk
    if (B >= 32) per = ((B + 3) / 4 + 7) / 8 * 8;
    const int chunks = (B + per - 1) / per;          // <= 4
    cudaStream_t s_in, s_k, s_out;
    cudaEvent_t *e_in, *e_k;
    if ((rc = host_pipeline(f, &s_in, &s_k, &s_out, &e_in, &e_k)) != SHFLBW_OK) return rc;
    auto fail = [&](int code) { cudaDeviceSynchronize(); return code; };
#define CKH(call) do { if (!cuda_ok((call), #call)) return fail(SHFLBW_ERR_CUDA); } while (0)
    for (int i = 0; i < chunks; ++i) {
        const int b0 = i * per, nb = (B - b0 < per) ? B - b0 : per;
        __half* dI = (__half*)f->stage_in + (size_t)b0 * img_in;
        __half* dO = (__half*)f->stage_out + (size_t)b0 * img_out;
        CKH(cudaMemcpyAsync(dI, (const __half*)ifmap_host + (size_t)b0 * img_in, (size_t)nb * img_in * 2,
                            cudaMemcpyHostToDevice, s_in));
        CKH(cudaEventRecord(e_in[i], s_in));
        CKH(cudaStreamWaitEvent(s_k, e_in[i], 0));
        shflbw_spconv_state_t st;
        rc = shflbw_spconv_init(f, nb, Hin, Win, stride, dI, dO, alpha, SHFLBW_KERNEL_AUTO, &st);
        if (rc == SHFLBW_OK) rc = shflbw_spconv_exec(&st, s_k);
        if (rc != SHFLBW_OK) return fail(rc);
        CKH(cudaEventRecord(e_k[i], s_k));
        CKH(cudaStreamWaitEvent(s_out, e_k[i], 0));
        CKH(cudaMemcpyAsync((__half*)ofmap_host + (size_t)b0 * img_out, dO, (size_t)nb * img_out * 2,
                            cudaMemcpyDeviceToHost, s_out));
    }
    CKH(cudaStreamSynchronize(s_out));
    CKH(cudaStreamSynchronize(s_k));
    CKH(cudaStreamSynchronize(s_in));
#undef CKH
    return SHFLBW_OK;
}

// ---- chained layers ---------------------------------------------------------------------

size_t shflbw_chain_buffer_elems(int C, int H, int W, int B, int R, int S) {
    if (C <= 0 || H <= 0 || W <= 0 || B <= 0 || R <= 0 || S <= 0) return 0;
    return (size_t)C * (H + R - 1) * (W + S - 1) * ((B + 7) / 8 * 8);
}

int shflbw_chain_import_nhwc(const void* nhwc, int B, int H, int W, int C, int R, int S, void* chain_buf,
                             void* stream) {
    if (!nhwc || !chain_buf || B <= 0 || H <= 0 || W <= 0 || C <= 0 || R <= 0 || S <= 0) return SHFLBW_ERR_INVALID_ARG;
    if (C % 8 || (((uintptr_t)nhwc | (uintptr_t)chain_buf) & 15)) return SHFLBW_ERR_UNSUPPORTED;
    if ((long long)shflbw_chain_buffer_elems(C, H, W, B, R, S) >= (1ll << 31)) return SHFLBW_ERR_UNSUPPORTED;
    launch_relayout((const __half*)nhwc, (__half*)chain_buf, B, (B + 7) / 8 * 8, H, W, C, R, S, (cudaStream_t)stream);
    CK(cudaGetLastError());
    return SHFLBW_OK;
}

int shflbw_chain_export_nhwc(const void* chain_buf, int B, int H, int W, int F, int R, int S,
                             const shflbw_matrix_t* producer, void* nhwc, void* stream) {
    if (!chain_buf || !nhwc || B <= 0 || H <= 0 || W <= 0 || F <= 0 || R <= 0 || S <= 0) return SHFLBW_ERR_INVALID_ARG;
    if (F % 8 || (((uintptr_t)nhwc | (uintptr_t)chain_buf) & 15)) return SHFLBW_ERR_UNSUPPORTED;
    const int* perm = nullptr;
    if (producer) {
        if (producer->nrow != F) return SHFLBW_ERR_BAD_FORMAT;
        if (!on_current_device(*producer)) return SHFLBW_ERR_NOT_ON_DEVICE;
        perm = producer->d_perm;
    }
    const size_t smem = (size_t)F * 16;
    if (smem > 227 * 1024) return SHFLBW_ERR_UNSUPPORTED;
    if (smem > 48 * 1024)
        CK(cudaFuncSetAttribute((const void*)shflbw::chain_export_nhwc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int Bp = (B + 7) / 8 * 8;
    const long long blocks = (long long)H * W * (Bp / 8);
    if (blocks >= (1ll << 31)) return SHFLBW_ERR_UNSUPPORTED;
    CK(launch(shflbw::chain_export_nhwc, dim3((unsigned)blocks), dim3(256), smem, (cudaStream_t)stream,
              (const __half*)chain_buf, (__half*)nhwc, perm, B, Bp, H, W, H + R - 1, W + S - 1, R / 2, S / 2, F));
    CK(cudaGetLastError());
    return SHFLBW_OK;
}

int shflbw_spconv_chain_init(shflbw_matrix_t* f, int B, int Hin, int Win, int stride, const void* in_chain,
                             void* out_chain, int R_next, int S_next, float alpha, int relu,
                             shflbw_spconv_state_t* out) {
    if (!out) return SHFLBW_ERR_INVALID_ARG;
    std::memset(out, 0, sizeof *out);
    if (!f || !in_chain || !out_chain || B <= 0 || Hin <= 0 || Win <= 0 || stride <= 0 || R_next <= 0 || S_next <= 0)
        return SHFLBW_ERR_INVALID_ARG;
    if (!f->is_filter) return SHFLBW_ERR_INVALID_ARG;
    if (!on_current_device(*f)) return SHFLBW_ERR_NOT_ON_DEVICE;
    if (f->brow != 32 && f->brow != 64 && f->brow != 128) return SHFLBW_ERR_UNSUPPORTED;
    if (f->C % 8 || !f->d_kcrs) return SHFLBW_ERR_UNSUPPORTED;
    if (((uintptr_t)in_chain | (uintptr_t)out_chain) & 15) return SHFLBW_ERR_UNSUPPORTED;
    const int Ho = (Hin + stride - 1) / stride, Wo = (Win + stride - 1) / stride;
    const int Bp = (B + 7) / 8 * 8;
    const long long tokens = (long long)Ho * Wo * Bp;
    // 32-bit element offsets into both chain buffers
    if (tokens >= (1ll << 31) || (long long)shflbw_chain_buffer_elems(f->C, Hin, Win, B, f->R, f->S) >= (1ll << 31) ||
        (long long)shflbw_chain_buffer_elems(f->F, Ho, Wo, B, R_next, S_next) >= (1ll << 32) - 1)
        return SHFLBW_ERR_UNSUPPORTED;
    out->B = B; out->Hin = Hin; out->Win = Win; out->C = f->C; out->F = f->F; out->R = f->R; out->S = f->S;
    out->stride = stride; out->Ho = Ho; out->Wo = Wo; out->V = f->brow; out->Bp = Bp;
    out->alpha = alpha; out->ifmap = in_chain; out->ofmap = out_chain;
    out->blk_ptr = f->d_kptr; out->blk_idx = f->d_kcrs; out->blk_val = f->d_val;
    out->perm = f->d_perm; out->status_word = f->d_status;
    out->chain = 1; out->out_R = R_next; out->out_S = S_next; out->relu = relu != 0;
    PanelChoice ch;
    int rc = pick_panel<shflbw::kPanelConvChain>(f->brow, tokens, f->F / f->brow, f->kptr.empty() ? 0 : f->kptr.back(), &ch);
    if (rc != SHFLBW_OK) return rc;
    out->kernel = SHFLBW_KERNEL_TCGEN05;
    out->tokens_per_cta = ch.tokens; out->stages = ch.stages; out->producer_warps = ch.pw; out->variant = ch.variant;
    out->tiles_n = (int)((tokens + ch.tokens - 1) / ch.tokens);
    out->num_items = out->tiles_n * (f->F / f->brow);
    const int sms = sm_count();
    if (sms <= 0) return SHFLBW_ERR_CUDA;
    out->block_x = ch.threads;
    out->grid_x = persistent_grid(out->num_items, sms); out->grid_y = 1;
    out->shared_mem_size = ch.smem;
    out->init_success = 1;
    return SHFLBW_OK;
}

int shflbw_chain_residual_map(const shflbw_matrix_t* layer, const shflbw_matrix_t* producer, int* map_host) {
    if (!layer || !map_host) return SHFLBW_ERR_INVALID_ARG;
    const int F = layer->nrow;
    if (producer && producer->nrow != F) return SHFLBW_ERR_BAD_FORMAT;
    std::vector<int> where(F);      // logical channel -> plane of the residual buffer
    for (int p = 0; p < F; ++p) where[producer && producer->row_permute ? producer->row_permute_ids[p] : p] = p;
    for (int f = 0; f < F; ++f) map_host[f] = where[layer->row_permute ? layer->row_permute_ids[f] : f];
    return SHFLBW_OK;
}

int shflbw_spconv_chain_set_residual(shflbw_matrix_t* f, shflbw_spconv_state_t* st, const void* res_chain,
                                     const int* map_host) {
    if (!f || !st || !st->init_success || !st->chain || !res_chain) return SHFLBW_ERR_INVALID_ARG;
    if (!on_current_device(*f) || st->blk_ptr != f->d_kptr) return SHFLBW_ERR_INVALID_ARG;
    if ((uintptr_t)res_chain & 15) return SHFLBW_ERR_UNSUPPORTED;
    // A map buffer made by an earlier call for this state is one of the handle's retired buffers.
    const int* prev_map = nullptr;
    for (void* r : f->retired) if (r == (const void*)st->residual_map) prev_map = st->residual_map;
    st->residual = res_chain;
    st->residual_map = nullptr;
    if (map_host) {
        for (int i = 0; i < st->F; ++i)
            if (map_host[i] < 0 || map_host[i] >= st->F) return SHFLBW_ERR_BAD_FORMAT;
        // One device buffer per state: re-binding the residual of the same state (every step,
        // say) overwrites it in place instead of allocating again.
        void* d = const_cast<int*>(prev_map);
        if (!d) {
            CK(cudaMalloc(&d, (size_t)st->F * sizeof(int)));
            f->retired.push_back(d);                   // lives as long as the filter's device copy
        }
        CK(cudaMemcpy(d, map_host, (size_t)st->F * sizeof(int), cudaMemcpyHostToDevice));
        st->residual_map = (const int*)d;
    }
    return SHFLBW_OK;
}

int shflbw_spconv_exec_static_scratch(const shflbw_matrix_t* f, int B, int Hin, int Win, int stride,
                                      const void* ifmap, void* ofmap, float alpha, void* stream) {
    // Same argument checks, 32-bit range checks and launch plan as shflbw_spconv_init (with an
    // unpermuted filter the output can bypass the array, so its capacity alone would not bound
    // the output offsets); only the scratch comes from somewhere else.
    shflbw_spconv_state_t st;
    int rc = plan_conv(f, B, Hin, Win, stride, ifmap, ofmap, alpha, SHFLBW_KERNEL_TCGEN05, &st);
    if (rc != SHFLBW_OK) return rc;

    // Capacity check first: nothing is launched when the shape does not fit.
    auto up256 = [](unsigned long long v) { return (v + 255ull) / 256ull * 256ull; };
    const unsigned long long in_bytes = up256(st.staged_in_bytes), out_bytes = up256(st.staged_out_bytes);
    if (in_bytes + out_bytes > (unsigned long long)SHFLBW_STATIC_SCRATCH_BYTES) {
        snprintf(g_cuda_err, sizeof g_cuda_err,
                 "static scratch: this shape needs %llu bytes, the built-in array holds %u",
                 in_bytes + out_bytes, (unsigned)SHFLBW_STATIC_SCRATCH_BYTES);
        return SHFLBW_ERR_TOO_LARGE;
    }

    // Once per device, with that device current: the array's device address.
    int dev = 0;
    CK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return SHFLBW_ERR_UNSUPPORTED;
    if (!g_static_scratch_addr[dev]) {
        void* ptr = nullptr;
        CK(cudaGetSymbolAddress(&ptr, g_static_scratch));
        if (!ptr) return SHFLBW_ERR_CUDA;
        g_static_scratch_addr[dev] = ptr;
    }
    unsigned char* scratch = (unsigned char*)g_static_scratch_addr[dev];
    st.staged_in = scratch;
    if (st.staged_out_bytes) st.staged_out = scratch + in_bytes;
    st.init_success = 1;
    return shflbw_spconv_exec(&st, stream);
}

// ---- several GPUs from one process -------------------------------------------------------

struct shflbw_multi {
    struct Shard {
        int device = -1;
        shflbw_matrix_t* mat = nullptr;      // replica of the sparse operand on `device`
        cudaStream_t stream = nullptr;
        cudaEvent_t start = nullptr, stop = nullptr;
        int kind = 0;                        // 0 none, 1 SpMM, 2 SpConv
        shflbw_spmm_state_t spmm;
        shflbw_spconv_state_t conv;
    };
    std::vector<Shard> shards;
};

namespace {
struct DeviceGuard {                         // restores the caller's current device
    int prev = -1;
    DeviceGuard() { cudaGetDevice(&prev); }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};
}  // namespace

int shflbw_multi_create(const shflbw_matrix_t* m, const int* device_ids, int n, shflbw_multi_t** out) {
    if (!m || !device_ids || n <= 0 || n > kMaxDevices || !out) return SHFLBW_ERR_INVALID_ARG;
    *out = nullptr;
    int have = 0;
    CK(cudaGetDeviceCount(&have));
    for (int g = 0; g < n; ++g) if (device_ids[g] < 0 || device_ids[g] >= have) return SHFLBW_ERR_INVALID_ARG;
    DeviceGuard guard;
    auto* mg = new shflbw_multi;
    mg->shards.resize(n);
    int rc = SHFLBW_OK;
    for (int g = 0; g < n && rc == SHFLBW_OK; ++g) {
        auto& sh = mg->shards[g];
        sh.device = device_ids[g];
        if (!cuda_ok(cudaSetDevice(sh.device), "cudaSetDevice")) { rc = SHFLBW_ERR_CUDA; break; }
        if ((rc = shflbw_matrix_clone(m, &sh.mat)) != SHFLBW_OK) break;
        if ((rc = shflbw_matrix_to_device(sh.mat)) != SHFLBW_OK) break;
        if (!cuda_ok(cudaStreamCreateWithFlags(&sh.stream, cudaStreamNonBlocking), "cudaStreamCreate") ||
            !cuda_ok(cudaEventCreate(&sh.start), "cudaEventCreate") || !cuda_ok(cudaEventCreate(&sh.stop), "cudaEventCreate"))
            rc = SHFLBW_ERR_CUDA;
    }
    if (rc != SHFLBW_OK) { shflbw_multi_destroy(mg); return rc; }
    *out = mg;
    return SHFLBW_OK;
}

void shflbw_multi_destroy(shflbw_multi_t* mg) {
    if (!mg) return;
    DeviceGuard guard;
    for (auto& sh : mg->shards) {
        if (sh.device >= 0) cudaSetDevice(sh.device);
        if (sh.stream) { cudaStreamSynchronize(sh.stream); cudaStreamDestroy(sh.stream); }
        if (sh.start) cudaEventDestroy(sh.start);
        if (sh.stop) cudaEventDestroy(sh.stop);
        shflbw_matrix_destroy(sh.mat);
    }
    delete mg;
}

int shflbw_multi_shards(const shflbw_multi_t* mg) { return mg ? (int)mg->shards.size() : 0; }

int shflbw_multi_spmm_init(shflbw_multi_t* mg, const int* n_per_shard, const void* const* B, void* const* D, float alpha) {
    if (!mg || !n_per_shard || !B || !D) return SHFLBW_ERR_INVALID_ARG;
    DeviceGuard guard;
    for (size_t g = 0; g < mg->shards.size(); ++g) {
        auto& sh = mg->shards[g];
        sh.kind = 0;
        if (n_per_shard[g] == 0) continue;                    // an empty shard is legal: nothing to launch
        CK(cudaSetDevice(sh.device));
        const int rc = shflbw_spmm_init(sh.mat, n_per_shard[g], B[g], alpha, nullptr, 0.f, D[g], SHFLBW_KERNEL_AUTO, &sh.spmm);
        if (rc != SHFLBW_OK) return rc;
        sh.kind = 1;
    }
    return SHFLBW_OK;
}

int shflbw_multi_spconv_init(shflbw_multi_t* mg, const int* images_per_shard, int Hin, int Win, int stride,
                             const void* const* ifmap, void* const* ofmap, float alpha) {
    if (!mg || !images_per_shard || !ifmap || !ofmap) return SHFLBW_ERR_INVALID_ARG;
    DeviceGuard guard;
    for (size_t g = 0; g < mg->shards.size(); ++g) {
        auto& sh = mg->shards[g];
        sh.kind = 0;
        if (images_per_shard[g] == 0) continue;
        CK(cudaSetDevice(sh.device));
        const int rc = shflbw_spconv_init(sh.mat, images_per_shard[g], Hin, Win, stride, ifmap[g], ofmap[g], alpha,
                                          SHFLBW_KERNEL_AUTO, &sh.conv);
        if (rc != SHFLBW_OK) return rc;
        sh.kind = 2;
    }
    return SHFLBW_OK;
}

int shflbw_multi_exec(shflbw_multi_t* mg) {
    if (!mg) return SHFLBW_ERR_INVALID_ARG;
    DeviceGuard guard;
    for (auto& sh : mg->shards) {                              // back to back: nothing here waits for a GPU
        if (!sh.kind) continue;
        CK(cudaSetDevice(sh.device));
        CK(cudaEventRecord(sh.start, sh.stream));
        const int rc = sh.kind == 1 ? shflbw_spmm_exec(&sh.spmm, sh.stream) : shflbw_spconv_exec(&sh.conv, sh.stream);
        if (rc != SHFLBW_OK) return rc;
        CK(cudaEventRecord(sh.stop, sh.stream));
    }
    return SHFLBW_OK;
}

int shflbw_multi_sync(shflbw_multi_t* mg, float* max_ms) {
    if (!mg) return SHFLBW_ERR_INVALID_ARG;
    DeviceGuard guard;
    float worst = 0.f;
    int status = SHFLBW_OK;
    for (auto& sh : mg->shards) {
        CK(cudaSetDevice(sh.device));
        CK(cudaStreamSynchronize(sh.stream));
        if (sh.kind) {
            float ms = 0.f;
            if (cudaEventElapsedTime(&ms, sh.start, sh.stop) == cudaSuccess && ms > worst) worst = ms;
            else (void)cudaGetLastError();
            const int rc = shflbw_matrix_device_status(sh.mat);
            if (rc != SHFLBW_OK) status = rc;
        }
    }
    if (max_ms) *max_ms = worst;
    return status;
}

}  // extern "C"
