// GEMM benchmark + correctness harness for fp16 operands, in the shape of the
// reference's driver (gemm/gemm_main.cpp:8-125) and test body
// (gemm/gemm_test.cu:200-482): per shape an algorithm bitmask, the three data
// pairings, C poisoned with 0x7D bytes before every algorithm, every result
// compared on the device against the slow comparison GEMM, 25 timed launches
// with the mean of the middle 13, one line per (shape, data, algorithm).
// Unlike the reference, a mismatch or a device-side time-out makes the exit
// status non-zero.
//
//   gemm [--quick] [--json FILE] [--config headline|reference|all] [--algos NAME[,NAME...]]
//        [--shape M,N,K[,STYLE]] [--device D]
//
//   --config   which shape list runs: the benchmark's own configurations, the reference's list
//              (gemm/gemm_main.cpp:98-122, wave-quantisation probes included), or both (default)
//   --algos    restrict the algorithm columns by name prefix (cublas, baseline, mine, mine_wide, n128, n64,
//              split_k, stream_k, auto_k)
//   --shape    run one shape instead of a list; STYLE 0..3 as gemm/gemm_main.cpp:81-95, 4 = uniform [-1,1)
//   --device   CUDA device ordinal (one harness process per GPU)
#include <cublas_v2.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <algorithm>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <string>
#include <vector>

#include "../../include/gemm_sm100.h"

enum class TestDataCode { random = 0, identity = 1, tiled_numbers = 2, uniform_pm1 = 3 };

enum class AlgorithmCode {
    cublas_f16,
    baseline_f16,
    mine_sm_100,
    mine_sm_100_n128,
    mine_sm_100_n64,
    mine_sm_100_split_k,
    mine_sm_100_stream_k,
    mine_sm_100_auto_k,
    mine_sm_100_wide,
    cutlass_sm100,
};
constexpr uint32_t algorithm_count = 1u + static_cast<uint32_t>(AlgorithmCode::cutlass_sm100);

inline uint32_t algorithm_code_bit(AlgorithmCode code) { return 1u << static_cast<uint32_t>(code); }

inline const char* algorithm_name(AlgorithmCode code)
{
    switch (code) {
    case AlgorithmCode::cublas_f16: return "cublas (f16 in, f32 out)";
    case AlgorithmCode::baseline_f16: return "baseline_f16";
    case AlgorithmCode::mine_sm_100: return "mine_sm_100 (output stationary)";
    case AlgorithmCode::mine_sm_100_n128: return "mine_sm_100_n128";
    case AlgorithmCode::mine_sm_100_n64: return "mine_sm_100_n64";
    case AlgorithmCode::mine_sm_100_split_k: return "mine_sm_100 (split k)";
    case AlgorithmCode::mine_sm_100_stream_k: return "mine_sm_100 (stream k)";
    case AlgorithmCode::mine_sm_100_auto_k: return "mine_sm_100 (automatic k)";
    case AlgorithmCode::mine_sm_100_wide: return "mine_sm_100 (256x512 tiles)";
    case AlgorithmCode::cutlass_sm100: return "cutlass sm100 (f16 in, f32 out, 256x256x64 pairs)";
    }
    return "unknown";
}

// Short names for --algos.
inline const char* algorithm_key(AlgorithmCode code)
{
    switch (code) {
    case AlgorithmCode::cublas_f16: return "cublas";
    case AlgorithmCode::baseline_f16: return "baseline";
    case AlgorithmCode::mine_sm_100: return "mine";
    case AlgorithmCode::mine_sm_100_n128: return "n128";
    case AlgorithmCode::mine_sm_100_n64: return "n64";
    case AlgorithmCode::mine_sm_100_split_k: return "split_k";
    case AlgorithmCode::mine_sm_100_stream_k: return "stream_k";
    case AlgorithmCode::mine_sm_100_auto_k: return "auto_k";
    case AlgorithmCode::mine_sm_100_wide: return "mine_wide";
    case AlgorithmCode::cutlass_sm100: return "cutlass";
    }
    return "";
}

struct TestParams {
    uint32_t M, N, K;
    TestDataCode test_data_code_A, test_data_code_B;
    uint32_t algorithm_code_bits;
};

// The CUTLASS comparison column lives in a shared object of its own (bin/libcutlass_column.so, built only
// where CUTLASS headers are installed) and is looked for beside this executable: cutlass_enabled(), like
// the reference's (gemm/cutlass_gemm.h:6), says whether the column exists.
typedef int (*CutlassGemmFn)(uint32_t, uint32_t, uint32_t, const void*, const void*, float*, void*, size_t, cudaStream_t);
typedef size_t (*CutlassWorkspaceFn)(uint32_t, uint32_t, uint32_t);
static CutlassGemmFn g_cutlass_gemm = nullptr;
static CutlassWorkspaceFn g_cutlass_workspace = nullptr;

static bool cutlass_enabled()
{
    static bool looked = false;
    if (!looked) {
        looked = true;
        Dl_info info;
        if (dladdr(reinterpret_cast<void*>(&cutlass_enabled), &info) && info.dli_fname) {
            std::string dir(info.dli_fname);
            const size_t slash = dir.rfind('/');
            dir = slash == std::string::npos ? std::string(".") : dir.substr(0, slash);
            if (void* h = dlopen((dir + "/libcutlass_column.so").c_str(), RTLD_NOW | RTLD_LOCAL)) {
                g_cutlass_gemm = reinterpret_cast<CutlassGemmFn>(dlsym(h, "cutlass_sm100_f16f32"));
                g_cutlass_workspace = reinterpret_cast<CutlassWorkspaceFn>(dlsym(h, "cutlass_sm100_workspace_bytes"));
            }
        }
    }
    return g_cutlass_gemm != nullptr && g_cutlass_workspace != nullptr;
}

static int g_failures = 0;
static FILE* g_json = nullptr;
static uint32_t g_algorithm_mask = ~0u;  // --algos

#define CUDA_OK(x)                                                                                   \
    do {                                                                                             \
        cudaError_t e_ = (x);                                                                        \
        if (e_ != cudaSuccess) {                                                                     \
            fprintf(stderr, "%s:%d cuda error %d (%s)\n", __FILE__, __LINE__, (int)e_, cudaGetErrorString(e_)); \
            exit(1);                                                                                 \
        }                                                                                            \
    } while (0)

// What the reference prints at the first wrong element (gemm/gemm_test.cu:100-120,157-175): the pair
// [expected, got] for the element and its neighbours two rows and columns around, the element itself in
// bold.  Done on the host here: the few rows involved are copied back.
static void print_neighbourhood(const float* d_expected, const float* d_got, uint32_t rows, uint32_t cols, uint32_t y,
                                uint32_t x)
{
    if (y >= rows || x >= cols) {
        return;
    }
    const uint32_t y0 = y < 2 ? 0u : y - 2, y1 = y + 2 >= rows ? rows - 1u : y + 2;
    const uint32_t x0 = x < 2 ? 0u : x - 2, x1 = x + 2 >= cols ? cols - 1u : x + 2;
    const uint32_t h = y1 - y0 + 1, w = x1 - x0 + 1;
    std::vector<float> e(size_t(h) * w), g(size_t(h) * w);
    const size_t pitch = size_t(cols) * sizeof(float);
    const size_t origin = size_t(y0) * cols + x0;
    if (cudaMemcpy2D(e.data(), w * sizeof(float), d_expected + origin, pitch, w * sizeof(float), h,
                     cudaMemcpyDeviceToHost) != cudaSuccess ||
        cudaMemcpy2D(g.data(), w * sizeof(float), d_got + origin, pitch, w * sizeof(float), h,
                     cudaMemcpyDeviceToHost) != cudaSuccess) {
        return;
    }
    printf("  [%u,%u] expected %g, got %g; rows %u..%u, columns %u..%u as [expected, got]:\n", y, x,
           e[size_t(y - y0) * w + (x - x0)], g[size_t(y - y0) * w + (x - x0)], y0, y1, x0, x1);
    for (uint32_t r = 0; r < h; ++r) {
        printf("  ");
        for (uint32_t c = 0; c < w; ++c) {
            const bool here = y0 + r == y && x0 + c == x;
            printf("%s[%6g, %6g]%s  ", here ? "\x1b[1m" : "", e[size_t(r) * w + c], g[size_t(r) * w + c],
                   here ? "\x1b[0m" : "");
        }
        printf("\n");
    }
}

static void gemm_test(TestParams params, cudaStream_t stream, cublasHandle_t cublasH)
{
    const size_t a_elems = size_t(params.M) * params.K, b_elems = size_t(params.N) * params.K;
    const size_t c_elems = size_t(params.M) * params.N;
    __half *d_a = nullptr, *d_bCol = nullptr;
    float *d_c_baseline = nullptr, *d_c_tested = nullptr;
    uint64_t* d_cmp = nullptr;
    CUDA_OK(cudaMallocAsync(&d_a, sizeof(__half) * a_elems, stream));
    CUDA_OK(cudaMallocAsync(&d_bCol, sizeof(__half) * b_elems, stream));
    CUDA_OK(cudaMallocAsync(&d_c_baseline, sizeof(float) * c_elems, stream));
    CUDA_OK(cudaMallocAsync(&d_c_tested, sizeof(float) * c_elems, stream));
    CUDA_OK(cudaMallocAsync(&d_cmp, 2 * sizeof(uint64_t), stream));
    void* d_cutlass_ws = nullptr;
    size_t cutlass_ws_bytes = 0;
    if ((params.algorithm_code_bits & g_algorithm_mask & algorithm_code_bit(AlgorithmCode::cutlass_sm100)) && cutlass_enabled()) {
        cutlass_ws_bytes = g_cutlass_workspace(params.M, params.N, params.K);
        CUDA_OK(cudaMallocAsync(&d_cutlass_ws, cutlass_ws_bytes, stream));
    }

    // A is M x K; B is the logical K x N matrix stored transposed (N x K), as the reference's d_bCol.
    spork_init_test_data_f16(d_a, params.M, params.K, (int)params.test_data_code_A, 20010106u, 0, stream);
    spork_init_test_data_f16(d_bCol, params.N, params.K, (int)params.test_data_code_B, 19980724u, 1, stream);

    auto fill_garbage = [&](float* d_c) { CUDA_OK(cudaMemsetAsync(d_c, 0x7D, sizeof(float) * c_elems, stream)); };

    fill_garbage(d_c_baseline);
    matmul_baseline_f16(GPU_TensorsF16{params.M, params.N, params.K, d_a, d_bCol, d_c_baseline, 0, 1, 0}, stream);

    // Signed data cancels, so the sign + ratio rule only applies to the reference's non-negative fixtures;
    // the normalised error max|err| / (max|A| max|B| K 2^-10) <= 1 applies to everything.
    const bool ratio_rule = params.test_data_code_A != TestDataCode::uniform_pm1;
    auto max_abs = [](TestDataCode c) { return c == TestDataCode::tiled_numbers ? 6364.0 : (c == TestDataCode::random ? 1000.0 : 1.0); };
    const double denom = max_abs(params.test_data_code_A) * max_abs(params.test_data_code_B) * double(params.K) / 1024.0;

    for (uint32_t bit_index = 0; bit_index < algorithm_count; ++bit_index) {
        if (((params.algorithm_code_bits & g_algorithm_mask) >> bit_index & 1) == 0) {
            continue;
        }
        const AlgorithmCode algo = static_cast<AlgorithmCode>(bit_index);
        const uint32_t test_count = algo == AlgorithmCode::baseline_f16 ? 3 : 25;
        std::vector<float> test_times(test_count);
        std::vector<cudaEvent_t> test_events(test_count + 1);
        for (auto& ev : test_events) {
            CUDA_OK(cudaEventCreate(&ev));
        }
        fill_garbage(d_c_tested);
        int launch_rc = 0;
        for (uint32_t test_i = 0; test_i < test_count; ++test_i) {
            if (test_i == 0) {
                CUDA_OK(cudaEventRecord(test_events[0], stream));
            }
            GPU_TensorsF16 t{params.M, params.N, params.K, d_a, d_bCol, d_c_tested, 0, 1, 0};
            switch (algo) {
            case AlgorithmCode::cublas_f16: {
                // A, B swap trick for the column-major library (gemm/gemm_test.cu:249-261)
                const float alpha = 1.0f, beta = 0.0f;
                cublasStatus_t st = cublasGemmEx(cublasH, CUBLAS_OP_T, CUBLAS_OP_N, int(params.N), int(params.M),
                                                 int(params.K), &alpha, d_bCol, CUDA_R_16F, int(params.K), d_a,
                                                 CUDA_R_16F, int(params.K), &beta, d_c_tested, CUDA_R_32F,
                                                 int(params.N), CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
                launch_rc |= (int)st;
                break;
            }
            case AlgorithmCode::baseline_f16: launch_rc |= matmul_baseline_f16(t, stream); break;
            case AlgorithmCode::mine_sm_100: launch_rc |= matmul_sm100(t, stream); break;
            case AlgorithmCode::mine_sm_100_n128:
                launch_rc |= matmul_sm100(t, stream, gemm_sm100_k_mode::output_stationary, 1, 128);
                break;
            case AlgorithmCode::mine_sm_100_n64:
                launch_rc |= matmul_sm100(t, stream, gemm_sm100_k_mode::output_stationary, 1, 64);
                break;
            case AlgorithmCode::mine_sm_100_split_k:
                launch_rc |= matmul_sm100(t, stream, gemm_sm100_k_mode::split_k_outer, 4);
                break;
            case AlgorithmCode::mine_sm_100_stream_k:
                launch_rc |= matmul_sm100(t, stream, gemm_sm100_k_mode::stream_k);
                break;
            case AlgorithmCode::mine_sm_100_auto_k:
                launch_rc |= matmul_sm100(t, stream, gemm_sm100_k_mode::automatic);
                break;
            case AlgorithmCode::mine_sm_100_wide:
                launch_rc |= matmul_sm100(t, stream, gemm_sm100_k_mode::output_stationary, 1, 512);
                break;
            case AlgorithmCode::cutlass_sm100:
                launch_rc |= g_cutlass_gemm(params.M, params.N, params.K, d_a, d_bCol, d_c_tested, d_cutlass_ws,
                                            cutlass_ws_bytes, stream);
                break;
            }
            CUDA_OK(cudaEventRecord(test_events[test_i + 1], stream));
        }
        spork_compare_f32(d_c_baseline, d_c_tested, params.M, params.N, d_cmp, stream);
        uint32_t detail = 0;
        const int status = spork_gemm_sm100_status(stream, &detail);
        uint64_t cmp[2];
        CUDA_OK(cudaMemcpy(cmp, d_cmp, sizeof(cmp), cudaMemcpyDeviceToHost));
        double max_diff;
        memcpy(&max_diff, &cmp[1], sizeof(double));
        const double nerr = denom > 0 ? max_diff / denom : max_diff;
        const bool ratio_ok = cmp[0] == UINT64_MAX;
        const bool pass = launch_rc == 0 && status == 0 && nerr <= 1.0 && (!ratio_rule || ratio_ok);
        if (!pass) {
            ++g_failures;
            printf("TestParams{%u,%u,%u, %i,%i} \x1b[1mFAILED\x1b[0m (%s): launch %d status %d (0x%08x) normalised error %g",
                   params.M, params.N, params.K, (int)params.test_data_code_A, (int)params.test_data_code_B,
                   algorithm_name(algo), launch_rc, status, detail, nerr);
            if (!ratio_ok) {
                printf(" first bad [%u,%u]", uint32_t(cmp[0] >> 32), uint32_t(cmp[0]));
            }
            printf("\n");
            if (!ratio_ok) {
                print_neighbourhood(d_c_baseline, d_c_tested, params.M, params.N, uint32_t(cmp[0] >> 32), uint32_t(cmp[0]));
            }
        }
        for (uint32_t test_i = 0; test_i < test_count; ++test_i) {
            CUDA_OK(cudaEventElapsedTime(&test_times[test_i], test_events[test_i], test_events[test_i + 1]));
        }
        for (auto& ev : test_events) {
            cudaEventDestroy(ev);
        }
        std::sort(test_times.begin(), test_times.end());
        double samples_ms = 0.0;
        const int sample_count = (test_count + 1) / 2;
        for (int i = 0; i < sample_count; ++i) {
            samples_ms += test_times[test_count / 4 + i];  // the interquartile range, as the reference times
        }
        const double ms = samples_ms / sample_count;
        const double tflops = double(params.M) * params.N * params.K * 2.0 / (ms * 1e-3) * 1e-12;
        printf("TestParams{%u,%u,%u, %i,%i} %.3g ms %.4g TFLOPS err %.2e (%s)\n", params.M, params.N, params.K,
               (int)params.test_data_code_A, (int)params.test_data_code_B, ms, tflops, nerr, algorithm_name(algo));
        if (g_json) {
            fprintf(g_json,
                    "{\"M\": %u, \"N\": %u, \"K\": %u, \"data_a\": %d, \"data_b\": %d, \"algorithm\": \"%s\", \"ms\": %.6f, "
                    "\"tflops\": %.3f, \"normalised_error\": %.3e, \"pass\": %s}\n",
                    params.M, params.N, params.K, (int)params.test_data_code_A, (int)params.test_data_code_B,
                    algorithm_name(algo), ms, tflops, nerr, pass ? "true" : "false");
        }
    }
    printf("\n");
    cudaFreeAsync(d_a, stream);
    cudaFreeAsync(d_bCol, stream);
    cudaFreeAsync(d_c_baseline, stream);
    cudaFreeAsync(d_c_tested, stream);
    cudaFreeAsync(d_cmp, stream);
    if (d_cutlass_ws) {
        cudaFreeAsync(d_cutlass_ws, stream);
    }
    CUDA_OK(cudaStreamSynchronize(stream));
}

int main(int argc, char** argv)
{
    bool quick = false;
    const char* config = "all";
    int device = 0;
    uint32_t one_shape[4] = {0, 0, 0, 4};
    bool have_shape = false;
    for (int i = 1; i < argc; ++i) {
        if (!strcmp(argv[i], "--quick")) {
            quick = true;
        } else if (!strcmp(argv[i], "--json") && i + 1 < argc) {
            g_json = fopen(argv[++i], "w");
        } else if (!strcmp(argv[i], "--config") && i + 1 < argc) {
            config = argv[++i];
            if (strcmp(config, "headline") && strcmp(config, "reference") && strcmp(config, "all")) {
                fprintf(stderr, "--config takes headline, reference or all\n");
                return 2;
            }
        } else if (!strcmp(argv[i], "--device") && i + 1 < argc) {
            device = atoi(argv[++i]);
        } else if (!strcmp(argv[i], "--shape") && i + 1 < argc) {
            const int got = sscanf(argv[++i], "%u,%u,%u,%u", &one_shape[0], &one_shape[1], &one_shape[2], &one_shape[3]);
            if (got < 3 || one_shape[3] > 4) {
                fprintf(stderr, "--shape takes M,N,K[,STYLE] with STYLE 0..4\n");
                return 2;
            }
            have_shape = true;
        } else if (!strcmp(argv[i], "--algos") && i + 1 < argc) {
            g_algorithm_mask = 0;
            char* list = argv[++i];
            for (char* tok = strtok(list, ","); tok; tok = strtok(nullptr, ",")) {
                bool known = false;
                for (uint32_t b = 0; b < algorithm_count; ++b) {
                    if (!strcmp(tok, algorithm_key(static_cast<AlgorithmCode>(b)))) {
                        g_algorithm_mask |= 1u << b;
                        known = true;
                    }
                }
                if (!known) {
                    fprintf(stderr, "--algos: unknown algorithm %s\n", tok);
                    return 2;
                }
            }
        } else {
            fprintf(stderr, "usage: gemm [--quick] [--json FILE] [--config headline|reference|all] [--algos LIST] "
                            "[--shape M,N,K[,STYLE]] [--device D]\n");
            return 2;
        }
    }
    CUDA_OK(cudaSetDevice(device));
    int cc_major = 0;
    CUDA_OK(cudaDeviceGetAttribute(&cc_major, cudaDevAttrComputeCapabilityMajor, device));
    const bool is_b200 = cc_major == 10;
    fprintf(stderr, "is_b200: %i\n", is_b200);
    fprintf(stderr, "cutlass_enabled: %i\n", cutlass_enabled());
    if (!is_b200) {
        fprintf(stderr, "this harness needs an sm_100 device\n");
        return 2;
    }
    cudaStream_t stream{};
    cublasHandle_t cublasH;
    if (cublasCreate(&cublasH) != CUBLAS_STATUS_SUCCESS) {
        fprintf(stderr, "cublasCreate failed\n");
        return 1;
    }
    cublasSetStream(cublasH, stream);

    // data_style as in gemm/gemm_main.cpp:81-95 (0 = all three reference pairings), 4 = uniform [-1,1)
    auto sized_tests = [&](uint32_t M, uint32_t N, uint32_t K, int data_style) {
        TestParams params{};
        params.M = M;
        params.N = N;
        params.K = K;
        params.algorithm_code_bits = algorithm_code_bit(AlgorithmCode::cublas_f16);
        if (cutlass_enabled() && M % 4 == 0 && N % 4 == 0 && K % 8 == 0) {  // the alignments its instantiation asks for
            params.algorithm_code_bits |= algorithm_code_bit(AlgorithmCode::cutlass_sm100);
        }
        GPU_TensorsF16 t{M, N, K, nullptr, nullptr, nullptr, 0, 1, 0};
        if (matmul_sm100_supports(t)) {
            params.algorithm_code_bits |= algorithm_code_bit(AlgorithmCode::mine_sm_100);
            if (N <= 256 || double(M) * N * K < 1e11) {
                params.algorithm_code_bits |= algorithm_code_bit(AlgorithmCode::mine_sm_100_n128);
                params.algorithm_code_bits |= algorithm_code_bit(AlgorithmCode::mine_sm_100_n64);
            }
            if (K >= 4096) {
                params.algorithm_code_bits |= algorithm_code_bit(AlgorithmCode::mine_sm_100_split_k);
            }
            params.algorithm_code_bits |= algorithm_code_bit(AlgorithmCode::mine_sm_100_stream_k);
            if (K >= 4096) {
                params.algorithm_code_bits |= algorithm_code_bit(AlgorithmCode::mine_sm_100_auto_k);
            }
            if (N >= 1024 && M >= 1024) {
                params.algorithm_code_bits |= algorithm_code_bit(AlgorithmCode::mine_sm_100_wide);
            }
        }
        auto run = [&](TestDataCode a, TestDataCode b) {
            params.test_data_code_A = a;
            params.test_data_code_B = b;
            gemm_test(params, stream, cublasH);
        };
        if (data_style == 0 || data_style == 1) {
            run(TestDataCode::tiled_numbers, TestDataCode::identity);
        }
        if (data_style == 0 || data_style == 2) {
            run(TestDataCode::identity, TestDataCode::tiled_numbers);
        }
        if (data_style == 0 || data_style == 3) {
            run(TestDataCode::random, TestDataCode::random);
        }
        if (data_style == 4) {
            run(TestDataCode::uniform_pm1, TestDataCode::uniform_pm1);
        }
    };

    const bool headline = !strcmp(config, "headline") || !strcmp(config, "all");
    const bool reference = !strcmp(config, "reference") || !strcmp(config, "all");
    if (have_shape) {
        sized_tests(one_shape[0], one_shape[1], one_shape[2], (int)one_shape[3]);
    } else {
        if (headline) {
            // the configurations of the headline benchmark
            sized_tests(256, 256, 512, 4);
            sized_tests(8192, 8192, 8192, 4);
            for (uint32_t n : {64u, 128u, 256u}) {
                sized_tests(16384, n, 8192, 4);
            }
        }
        if (reference) {
            // the reference's own shape list (gemm/gemm_main.cpp:98-122)
            sized_tests(2048, 2048, 2048, 2);
            sized_tests(768, 768, 32, 2);
            sized_tests(160, 480, 816, 0);
        }
        if (reference && !quick) {
            sized_tests(4096, 4096, 4096, 2);
            sized_tests(8192, 8192, 8192, 2);
            sized_tests(7680, 1536, 4096, 0);
            sized_tests(15360, 1536, 8192, 3);
            sized_tests(32768, 65536, 48, 3);
            sized_tests(32768, 40016, 816, 0);
            sized_tests(40016, 32768, 6400, 3);
            sized_tests(12288, 24576, 1536, 3);
            // wave-quantisation probes (gemm/gemm_main.cpp:104,111-117): n-tile counts either side of what fills
            // the machine, at a K long enough for K splits to matter
            for (uint32_t n_tiles : {3u, 9u, 10u, 11u, 12u}) {
                sized_tests(6 * 256, n_tiles * 256, 65536, 3);
            }
            sized_tests(3 * 256, 11 * 256, 65536, 3);
            sized_tests(9 * 256, 11 * 256, 65536, 3);
            sized_tests(4 * 256, 11 * 256, 16384 * 3, 3);
            sized_tests(7680, 3072, 16384, 3);
            sized_tests(768, 3072, 3072, 3);
        }
    }
    cudaDeviceSynchronize();
    cublasDestroy(cublasH);
    if (g_json) {
        fclose(g_json);
    }
    if (g_failures) {
        fprintf(stderr, "%d comparison(s) FAILED\n", g_failures);
        return 1;
    }
    return 0;
}
