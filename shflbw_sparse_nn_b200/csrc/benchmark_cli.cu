// Command-line benchmarks with the flags and the output line of the reference's tools
// (block_sparse/benchmark/benchmark.spmm.cu:52-215, benchmark.spconv.cu:52-199, flag parser
// block_sparse/benchmark/argparse_util.h:10-119 and 121-264), on top of shflbw_compat.hpp:
//
//   benchmark.spmm.out   --m M --n N --k K --d DENSITY --sparsity-type block --block-size V
//                        [--row-permute] [--random] [--store-pattern FILE] [--load-pattern FILE]
//   benchmark.spconv.out --B B --H H --W W --C C --F F --R R --S S --stride s --d DENSITY
//                        --sparsity-type block --block-size V [--row-permute] [--random] ...
//
// As in the reference, H and W of the conv tool are OUTPUT sizes (the input is H*stride x
// W*stride), shapes are padded (m, F to the block size; n to 32), timing is 10 warm-up + 100
// timed launches between two CUDA events, and one line goes to stdout:
//   <GPU_CC> <config_str> <shape...> <block> <BN> <BK> <WM> <WN> <WK> <MMA_M> <MMA_N> <MMA_K> <NSTAGE> <t> (us) <x> (effective tflop/s)
// where "effective" counts the dense FLOPs, as the reference does.  The tile columns describe
// the one kernel this library picks (tokens per CTA, 64 columns per stage, UMMA 128 x V x 16).
// --store-pattern / --load-pattern write and read the reference's text format (the reference
// parses the flags but leaves both unimplemented).  Compile with -DSHFLBW_BENCH_SPCONV for the
// conv tool.
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <string>
#include <vector>

#include "shflbw_compat.hpp"

namespace {

struct Args {
    long m = 0, n = 0, k = 0;                                   // spmm
    long B = 0, H = 0, W = 0, C = 0, F = 0, R = 0, S = 0, stride = 1;  // spconv
    float density = 0.f;
    unsigned seed = 2021;
    int pattern = -1, block = 0;
    bool permute = false;
    std::string store, load;
};

const char* kUsage =
    "\tRequired cmdline args:\n"
#ifdef SHFLBW_BENCH_SPCONV
    "\t--B [batch] --H [out height] --W [out width] --C [channels] --F [filters]\n"
    "\t--R [filter height] --S [filter width] --stride [stride]\n"
#else
    "\t--m [M]\n\t--n [N]\n\t--k [K]\n"
#endif
    "\t--d [density between 0~1]\n"
    "\t--sparsity-type [block]\n"
    "\t--block-size [16/32/64/128]\n"
    "\tOptional cmdline args:\n"
    "\t--row-permute : run with a random row (filter) permutation\n"
    "\t--random : random seed (default 2021 for every run)\n"
    "\t--store-pattern [file] : dump the generated sparse operand\n"
    "\t--load-pattern  [file] : load the sparse operand from a dump\n";

[[noreturn]] void die(const std::string& why, const std::string& log) {
    fprintf(stderr, "%s%s\n%s", kUsage, why.c_str(), log.c_str());
    exit(EXIT_FAILURE);
}

bool parse(int argc, const char** argv, Args& a) {
    struct LongOpt { const char* name; long Args::*dst; };
    const LongOpt longs[] = {{"--m", &Args::m}, {"--n", &Args::n}, {"--k", &Args::k}, {"--B", &Args::B},
                             {"--H", &Args::H}, {"--W", &Args::W}, {"--C", &Args::C}, {"--F", &Args::F},
                             {"--R", &Args::R}, {"--S", &Args::S}, {"--stride", &Args::stride}};
    for (int i = 1; i < argc; ++i) {
        const std::string f = argv[i];
        const char* val = i + 1 < argc ? argv[i + 1] : nullptr;
        bool hit = false;
        for (const LongOpt& o : longs)
            if (f == o.name && val) { a.*(o.dst) = atol(val); hit = true; }
        if (hit) { ++i; continue; }
        if (f == "--d" && val) { a.density = (float)atof(val); ++i; }
        else if (f == "--block-size" && val) { a.block = atoi(val); ++i; }
        else if (f == "--sparsity-type" && val) { a.pattern = !strcmp(val, "block") ? 0 : !strcmp(val, "block-2in4") ? 1 : -1; ++i; }
        else if (f == "--store-pattern" && val) { a.store = val; ++i; }
        else if (f == "--load-pattern" && val) { a.load = val; ++i; }
        else if (f == "--row-permute") a.permute = true;
        else if (f == "--random") a.seed = (unsigned)std::chrono::system_clock::now().time_since_epoch().count();
    }
    return true;
}

// uniform[-1, 1) fp16 from a 64-bit LCG; the values do not influence the timing
void fill_uniform(std::vector<half>& v, unsigned long long s) {
    for (half& h : v) {
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        h = __float2half((float)((s >> 40) & 0xffff) / 32768.0f - 1.0f);
    }
}

#define CUDA_OK(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) { \
    fprintf(stderr, "%s failed: %s\n", #call, cudaGetErrorString(e_)); return EXIT_FAILURE; } } while (0)

template <class Op>
int time_op(Op& op, float* ms_per_launch) {
    const int warmup = 10, repeat = 100;
    cudaEvent_t t0, t1;
    CUDA_OK(cudaEventCreate(&t0));
    CUDA_OK(cudaEventCreate(&t1));
    op(nullptr);
    CUDA_OK(cudaDeviceSynchronize());
    if (op.status() != SHFLBW_OK) { fprintf(stderr, "kernel failed: %s\n", shflbw_strerror(op.status())); return EXIT_FAILURE; }
    for (int i = 0; i < warmup + repeat; ++i) {
        if (i == warmup) CUDA_OK(cudaEventRecord(t0, nullptr));
        op(nullptr);
    }
    CUDA_OK(cudaEventRecord(t1, nullptr));
    CUDA_OK(cudaEventSynchronize(t1));
    float ms = 0.f;
    CUDA_OK(cudaEventElapsedTime(&ms, t0, t1));
    *ms_per_launch = ms / repeat;
    return EXIT_SUCCESS;
}

}  // namespace

int main(int argc, const char** argv) {
    Args a;
    parse(argc, argv, a);
    char log[512];
#ifdef SHFLBW_BENCH_SPCONV
    snprintf(log, sizeof log, "\narguments: B = %ld\nH = %ld\nW = %ld\nC = %ld\nF = %ld\nR = %ld\nS = %ld\nstride = %ld\ndensity = %g\nseed = %u\n"
             "block-size = %d x 1\nsparsity-pattern = %d\nrow-permute ? %d\n", a.B, a.H, a.W, a.C, a.F, a.R, a.S, a.stride,
             a.density, a.seed, a.block, a.pattern, (int)a.permute);
    if (a.B <= 0 || a.H <= 0 || a.W <= 0 || a.C <= 0 || a.F <= 0 || a.R <= 0 || a.S <= 0 || a.stride <= 0 || a.density == 0.f)
        die("Forget to set B,H,W,C,F,R,S,stride or density?", log);
#else
    snprintf(log, sizeof log, "\narguments: m = %ld\nn = %ld\nk = %ld\ndensity = %g\nseed = %u\nblock-size = %d x 1\n"
             "sparsity-pattern = %d\nrow-permute ? %d\n", a.m, a.n, a.k, a.density, a.seed, a.block, a.pattern, (int)a.permute);
    if (a.m <= 0 || a.n <= 0 || a.k <= 0 || a.density == 0.f) die("Forget to set m,n,k or density?", log);
#endif
    if (a.block != 16 && a.block != 32 && a.block != 64 && a.block != 128) die("Unsupported block size. Choose in 16/32/64/128.", log);
    if (a.pattern != 0) die("sparsity-pattern is not given or unsupported.", log);
    fputs(log, stderr);

#ifdef SHFLBW_BENCH_SPCONV
    if (a.F % a.block) { a.F += a.block - a.F % a.block; fprintf(stderr, "F padded to : %ld\n", a.F); }
    BlockwiseSpFilter<half> sp;
    if (!a.load.empty()) {
        std::ifstream in(a.load);
        if (!in) { fprintf(stderr, "cannot open %s\n", a.load.c_str()); return EXIT_FAILURE; }
        sp.load(in);
        if (sp.last_status == SHFLBW_OK) sp.last_status = shflbw_matrix_set_filter_shape(sp.handle, (int)a.F, (int)a.R, (int)a.S, (int)a.C);
        sp.F = (int)a.F; sp.R = (int)a.R; sp.S = (int)a.S; sp.C = (int)a.C;
    } else {
        sp.init_random((int)a.F, (int)a.R, (int)a.S, (int)a.C, a.block, 1, a.density, a.permute, a.seed, SHFLBW_VALUES_UNIFORM);
    }
#else
    if (a.m % a.block) { a.m += a.block - a.m % a.block; fprintf(stderr, "m padded to : %ld\n", a.m); }
    if (a.n % 32) { a.n += 32 - a.n % 32; fprintf(stderr, "n padded to : %ld for better alignment.\n", a.n); }
    BlockwiseSpMatrix<half> sp;
    if (!a.load.empty()) {
        std::ifstream in(a.load);
        if (!in) { fprintf(stderr, "cannot open %s\n", a.load.c_str()); return EXIT_FAILURE; }
        sp.load(in);
    } else {
        sp.init_random((int)a.m, (int)a.k, a.block, 1, a.density, a.permute, a.seed, SHFLBW_VALUES_UNIFORM);
    }
#endif
    if (sp.last_status != SHFLBW_OK) { fprintf(stderr, "sparse operand: %s\n", shflbw_strerror(sp.last_status)); return EXIT_FAILURE; }
    if (!a.store.empty()) {
        std::ofstream out(a.store);
        sp.dump(out);
    }
    sp.transform_and_sync_device();
    if (sp.last_status != SHFLBW_OK) {
        fprintf(stderr, "device copy: %s (%s)\n", shflbw_strerror(sp.last_status), shflbw_last_cuda_error());
        return EXIT_FAILURE;
    }

    half *in_d = nullptr, *out_d = nullptr;
#ifdef SHFLBW_BENCH_SPCONV
    const long Hin = a.H * a.stride, Win = a.W * a.stride;
    const size_t n_in = (size_t)a.B * Hin * Win * a.C, n_out = (size_t)a.B * a.H * a.W * a.F;
#else
    const size_t n_in = (size_t)sp.ncol * a.n, n_out = (size_t)sp.nrow * a.n;
#endif
    {
        std::vector<half> host(n_in);
        fill_uniform(host, a.seed);
        CUDA_OK(cudaMalloc(&in_d, n_in * sizeof(half)));
        CUDA_OK(cudaMalloc(&out_d, n_out * sizeof(half)));
        CUDA_OK(cudaMemcpy(in_d, host.data(), n_in * sizeof(half), cudaMemcpyHostToDevice));
        CUDA_OK(cudaMemset(out_d, 0, n_out * sizeof(half)));
    }

    float ms = 0.f;
#ifdef SHFLBW_BENCH_SPCONV
    SpconvBlockwiseOp<ShapeBase<0, 0, 0>, ShapeBase<0, 0, 0>, ShapeBase<0, 0, 0>, 0> op;
    op._state.status = shflbw_spconv_init(sp.handle, (int)a.B, (int)Hin, (int)Win, (int)a.stride, in_d, out_d, 1.0f,
                                          SHFLBW_KERNEL_AUTO, &op._state.impl);
    const shflbw_spconv_state_t& st = op._state.impl;
    const double gflop = (double)a.B / 1e9 * a.H * a.W * a.C * a.R * a.S * a.F * 2;
#else
    SpmmBlockwiseOp<ShapeBase<0, 0, 0>, ShapeBase<0, 0, 0>, ShapeBase<0, 0, 0>, 0> op;
    op._state.status = shflbw_spmm_init(sp.handle, (int)a.n, in_d, 1.0f, nullptr, 0.0f, out_d, SHFLBW_KERNEL_AUTO, &op._state.impl);
    const shflbw_spmm_state_t& st = op._state.impl;
    const double gflop = (double)sp.nrow / 1e9 * a.n * sp.ncol * 2;
#endif
    if (op._state.status != SHFLBW_OK) {
        fprintf(stderr, "initialize: %s (%s)\n", shflbw_strerror(op._state.status), shflbw_last_cuda_error());
        return EXIT_FAILURE;
    }
    if (time_op(op, &ms) != EXIT_SUCCESS) return EXIT_FAILURE;
    if (shflbw_matrix_device_status(sp.handle) != SHFLBW_OK) { fprintf(stderr, "device status: %s\n", shflbw_last_cuda_error()); return EXIT_FAILURE; }

    printf("100 %s ", sp.config_str.c_str());
#ifdef SHFLBW_BENCH_SPCONV
    printf("%ld %ld %ld %ld ", a.B, a.H, a.W, a.stride);
#else
    printf("%ld ", a.n);
#endif
    printf("%d %d %d %d %d %d %d %d %d %d ", a.block, st.tokens_per_cta, 64, 128, a.block, 16, 128, a.block, 16, st.stages);
    printf("%f (us) %f (effective tflop/s)\n", ms * 1e3, gflop / ms);
    cudaFree(in_d);
    cudaFree(out_d);
    return EXIT_SUCCESS;
}
