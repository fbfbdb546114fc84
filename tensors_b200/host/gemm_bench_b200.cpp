// GEMM benchmark with the output schema of the reference's benchmarks/gemm_bench.cpp:317-359
// ({gpu, sm_count, peak_tflops, warmup, iters, sizes, results: [{size, kernel, time_ms, tflops,
// sol_pct}]}), so that tables built from the reference's result file can be regenerated from this
// one. Same method as the reference (benchmarks/gemm_bench.cpp:99-124): warm-up 3, then the median of
// `iters` launches, each bracketed by CUDA events on the work stream; square sizes, all three dtypes,
// TFLOPS = 2*N^3 / t. The three reference launchers (naive / tiled / optimized) all route to the one
// tcgen05 kernel here, so they are reported once each for schema compatibility; every entry also
// carries a "dtype" key, which the reference's schema lacks. There is no cuBLAS entry: this library
// links no GEMM library. Inputs are the reference's constants (0.5 and 0.3, gemm_bench.cpp:269-270),
// written as proper values of each dtype.
//
//   gemm_bench_b200 [--sizes 128,256,...] [--iters N] [--output file]
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iostream>
#include <sstream>
#include <string>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/tfb.h"
#include "tensorforge_b200.hpp"

namespace {

constexpr int kWarmup = 3;
// Dense peaks of a B200 for the "sol_pct" column: 3xTF32-effective FP32 and 16-bit (nominal figures).
constexpr double kPeakFp32 = 375.0, kPeak16 = 2250.0;

void check(cudaError_t e, const char* what) {
    if (e != cudaSuccess) {
        std::fprintf(stderr, "[gemm_bench_b200] %s: %s\n", what, cudaGetErrorString(e));
        std::exit(1);
    }
}

template <typename F>
double median_ms(cudaStream_t stream, int iters, F&& launch) {
    for (int i = 0; i < kWarmup; ++i) launch();
    check(cudaStreamSynchronize(stream), "sync");
    cudaEvent_t a, b;
    check(cudaEventCreate(&a), "event");
    check(cudaEventCreate(&b), "event");
    std::vector<float> t;
    for (int i = 0; i < iters; ++i) {
        check(cudaEventRecord(a, stream), "record");
        launch();
        check(cudaEventRecord(b, stream), "record");
        check(cudaEventSynchronize(b), "sync");
        float ms = 0.f;
        check(cudaEventElapsedTime(&ms, a, b), "elapsed");
        t.push_back(ms);
    }
    cudaEventDestroy(a);
    cudaEventDestroy(b);
    std::sort(t.begin(), t.end());
    return t[t.size() / 2];
}

struct Result {
    int size;
    std::string kernel, dtype;
    double ms, tflops, sol;
};

}  // namespace

int main(int argc, char** argv) {
    using namespace tensorforge;
    std::vector<int> sizes = {128, 256, 512, 1024, 2048};
    int iters = 10;
    std::string output;
    for (int i = 1; i < argc; ++i) {
        const std::string a = argv[i];
        if (a == "--sizes" && i + 1 < argc) {
            sizes.clear();
            std::stringstream ss(argv[++i]);
            std::string tok;
            while (std::getline(ss, tok, ',')) sizes.push_back(std::atoi(tok.c_str()));
        } else if (a == "--iters" && i + 1 < argc) {
            iters = std::max(1, std::atoi(argv[++i]));
        } else if (a == "--output" && i + 1 < argc) {
            output = argv[++i];
        }
    }
    cudaDeviceProp prop;
    check(cudaGetDeviceProperties(&prop, 0), "device properties");
    if (tfb_init() != TFB_OK) {
        std::fprintf(stderr, "[gemm_bench_b200] %s\n", tfb_last_error_string());
        return 1;
    }
    cudaStream_t stream;
    check(cudaStreamCreateWithFlags(&stream, cudaStreamNonBlocking), "stream");
    std::vector<Result> results;
    using Launcher = void (*)(const void*, const void*, void*, int64_t, int64_t, int64_t, Dtype, void*);
    const std::pair<const char*, Launcher> kernels[3] = {
        {"naive", launch_gemm_naive}, {"tiled", launch_gemm_tiled_16x16}, {"optimized", launch_gemm_optimized}};
    for (Dtype dtype : {Dtype::Float32, Dtype::Float16, Dtype::BFloat16}) {
        const char* name = dtype == Dtype::Float32 ? "float32" : dtype == Dtype::Float16 ? "float16" : "bfloat16";
        const size_t es = dtype == Dtype::Float32 ? 4 : 2;
        for (int n : sizes) {
            const size_t count = static_cast<size_t>(n) * n;
            std::vector<uint8_t> ha(count * es), hb(count * es);
            for (size_t i = 0; i < count; ++i) {
                if (dtype == Dtype::Float32) {
                    reinterpret_cast<float*>(ha.data())[i] = 0.5f;
                    reinterpret_cast<float*>(hb.data())[i] = 0.3f;
                } else if (dtype == Dtype::Float16) {
                    reinterpret_cast<__half*>(ha.data())[i] = __float2half(0.5f);
                    reinterpret_cast<__half*>(hb.data())[i] = __float2half(0.3f);
                } else {
                    reinterpret_cast<__nv_bfloat16*>(ha.data())[i] = __float2bfloat16(0.5f);
                    reinterpret_cast<__nv_bfloat16*>(hb.data())[i] = __float2bfloat16(0.3f);
                }
            }
            void *A = nullptr, *B = nullptr, *C = nullptr;
            check(cudaMalloc(&A, count * es), "cudaMalloc");
            check(cudaMalloc(&B, count * es), "cudaMalloc");
            check(cudaMalloc(&C, count * es), "cudaMalloc");
            check(cudaMemcpy(A, ha.data(), count * es, cudaMemcpyHostToDevice), "copy");
            check(cudaMemcpy(B, hb.data(), count * es, cudaMemcpyHostToDevice), "copy");
            for (const auto& k : kernels) {
                const double ms = median_ms(stream, iters, [&] { k.second(A, B, C, n, n, n, dtype, stream); });
                const double tf = 2.0 * n * double(n) * n / (ms * 1e-3) / 1e12;
                results.push_back({n, k.first, name, ms, tf, 100.0 * tf / (dtype == Dtype::Float32 ? kPeakFp32 : kPeak16)});
            }
            std::cerr << "[gemm_bench_b200] " << name << " N=" << n << " optimized=" << results.back().ms << " ms ("
                      << results.back().tflops << " TFLOPS)\n";
            cudaFree(A);
            cudaFree(B);
            cudaFree(C);
        }
    }
    int code = 0;
    if (tfb_device_status(&code) != TFB_OK || code != 0) {
        std::fprintf(stderr, "[gemm_bench_b200] device error %d\n", code);
        return 1;
    }
    std::ostringstream ss;
    ss << "{\n  \"gpu\": \"" << prop.name << "\",\n  \"sm_count\": " << prop.multiProcessorCount
       << ",\n  \"peak_tflops\": " << kPeakFp32 << ",\n  \"peak_tflops_16bit\": " << kPeak16 << ",\n  \"warmup\": " << kWarmup
       << ",\n  \"iters\": " << iters << ",\n  \"sizes\": [";
    for (size_t i = 0; i < sizes.size(); ++i) ss << (i ? ", " : "") << sizes[i];
    ss << "],\n  \"results\": [\n";
    for (size_t i = 0; i < results.size(); ++i) {
        const Result& r = results[i];
        ss << "    {\"size\": " << r.size << ", \"kernel\": \"" << r.kernel << "\", \"dtype\": \"" << r.dtype
           << "\", \"time_ms\": " << r.ms << ", \"tflops\": " << r.tflops << ", \"sol_pct\": " << r.sol << "}"
           << (i + 1 < results.size() ? "," : "") << "\n";
    }
    ss << "  ]\n}\n";
    if (!output.empty()) {
        std::ofstream out(output);
        if (!out) {
            std::cerr << "[gemm_bench_b200] cannot open " << output << "\n";
            return 1;
        }
        out << ss.str();
    } else {
        std::cout << ss.str();
    }
    return 0;
}
