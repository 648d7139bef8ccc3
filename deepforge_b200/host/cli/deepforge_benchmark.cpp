// deepforge-benchmark for the sm_100a backend: the single-node CONV_FPROP profiles of the reference's
// tools/deepforge-benchmark.cpp (same names, shapes, input patterns, command line and CSV columns, :23-38,
// :205-313), run through compile_graph and Executable::execute on DEVICE buffers.
//
// Per profile: compile (timed on the host clock), one CHECKED pass -- the output is copied back and compared with a
// plain double-precision convolution computed here on the host, under the reference's acceptance rule
// |d| <= 1e-4 + 1e-3 |ref| (its compare(), :182-203) -- and only then `iterations` timed passes, bracketed by CUDA
// events on the stream the executable launches on. One CSV row per profile and policy. The schedule policies are
// accepted for command-line compatibility; kernel selection does not depend on them here, so "both" prints the
// same plan twice. Exit codes: 0 success, 1 failure (compile, device, mismatch), 2 usage.
#include "DeepForge/Compiler/Codegen.h"

#include <cuda_runtime_api.h>

#include <array>
#include <charconv>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <iomanip>
#include <iostream>
#include <string>
#include <string_view>
#include <vector>

namespace {

using deepforge::import::AttributeValue;
using deepforge::import::DataType;

struct Shape {
    std::string_view name;
    std::int64_t n, h, w, c, k, r, s, pad_h, pad_w;
    std::int64_t out_h() const { return h + 2 * pad_h - r + 1; }
    std::int64_t out_w() const { return w + 2 * pad_w - s + 1; }
};

constexpr std::array<Shape, 3> kShapes{{
    {"small", 1, 8, 8, 8, 8, 3, 3, 1, 1},
    {"medium", 1, 32, 32, 32, 32, 3, 3, 1, 1},
    {"large", 1, 56, 56, 64, 64, 3, 3, 1, 1},
}};

void usage(std::ostream& out) {
    out << "usage: deepforge-benchmark [--profile=small|medium|large|all] [--schedule=auto|baseline|both] [--iterations=N]\n";
}

struct Arguments {
    std::string_view profile = "all", schedule = "auto";
    int iterations = 3;
};

bool take(std::string_view argument, std::string_view prefix, std::string_view& value) {
    if (!argument.starts_with(prefix)) return false;
    value = argument.substr(prefix.size());
    return true;
}

bool read_arguments(int argc, char** argv, Arguments& out) {
    for (int i = 1; i < argc; ++i) {
        std::string_view argument(argv[i]), value;
        if (take(argument, "--profile=", value)) {
            if (value != "small" && value != "medium" && value != "large" && value != "all") {
                std::cerr << "invalid profile: " << value << '\n';
                return false;
            }
            out.profile = value;
        } else if (take(argument, "--schedule=", value)) {
            if (value != "auto" && value != "baseline" && value != "both") {
                std::cerr << "invalid schedule: " << value << '\n';
                return false;
            }
            out.schedule = value;
        } else if (take(argument, "--iterations=", value)) {
            int parsed = 0;
            auto result = std::from_chars(value.data(), value.data() + value.size(), parsed);
            if (result.ec != std::errc{} || result.ptr != value.data() + value.size() || parsed <= 0 || parsed > 1000) {
                std::cerr << "iterations must be in [1, 1000]\n";
                return false;
            }
            out.iterations = parsed;
        } else {
            std::cerr << "unknown option: " << argument << '\n';
            return false;
        }
    }
    return true;
}

// The single-node graph of a profile: packed NHWC / KRSC FLOAT tensors with UIDs 201, 202, 203.
deepforge::import::SerializedGraph graph_of(Shape const& p) {
    deepforge::import::SerializedGraph graph;
    graph.graph_uid = static_cast<std::uint64_t>(p.h * 1000000 + p.c * 1000 + p.k);
    graph.context.name = "benchmark_" + std::string(p.name);
    graph.context.compute_data_type = graph.context.intermediate_data_type = graph.context.io_data_type = DataType::kFloat32;
    graph.context.sm_count = -1;
    graph.context.is_dynamic_shape_enabled = graph.context.is_override_shape_enabled = false;
    auto tensor = [&](std::int64_t uid, char const* name, std::array<std::int64_t, 4> nchw) {
        deepforge::import::TensorDesc t;
        t.uid = uid;
        t.name = name;
        t.dim.assign(nchw.begin(), nchw.end());
        t.stride = {nchw[2] * nchw[3] * nchw[1], 1, nchw[3] * nchw[1], nchw[1]};
        graph.tensors.emplace(uid, std::move(t));
    };
    tensor(201, "X", {p.n, p.c, p.h, p.w});
    tensor(202, "W", {p.k, p.c, p.r, p.s});
    tensor(203, "Y", {p.n, p.k, p.out_h(), p.out_w()});
    deepforge::import::OperationDesc conv;
    conv.tag = deepforge::import::OperationTag::kConvFprop;
    conv.name = "conv_fprop";
    conv.inputs = {{"X", 201}, {"W", 202}};
    conv.outputs = {{"Y", 203}};
    conv.attributes["compute_data_type"] = std::string("FLOAT");
    conv.attributes["math_mode"] = std::string("CROSS_CORRELATION");
    conv.attributes["pre_padding"] = std::vector<std::int64_t>{p.pad_h, p.pad_w};
    conv.attributes["post_padding"] = std::vector<std::int64_t>{p.pad_h, p.pad_w};
    conv.attributes["stride"] = std::vector<std::int64_t>{1, 1};
    conv.attributes["dilation"] = std::vector<std::int64_t>{1, 1};
    graph.nodes.push_back(std::move(conv));
    return graph;
}

// NHWC x KRSC -> NHWK in double precision: the checker of the compared pass.
std::vector<double> host_convolution(Shape const& p, std::vector<float> const& x, std::vector<float> const& w) {
    std::vector<double> y(static_cast<std::size_t>(p.n * p.out_h() * p.out_w() * p.k), 0.0);
    for (std::int64_t n = 0; n < p.n; ++n)
        for (std::int64_t oh = 0; oh < p.out_h(); ++oh)
            for (std::int64_t ow = 0; ow < p.out_w(); ++ow)
                for (std::int64_t k = 0; k < p.k; ++k) {
                    double sum = 0.0;
                    for (std::int64_t r = 0; r < p.r; ++r) {
                        auto const ih = oh + r - p.pad_h;
                        if (ih < 0 || ih >= p.h) continue;
                        for (std::int64_t s = 0; s < p.s; ++s) {
                            auto const iw = ow + s - p.pad_w;
                            if (iw < 0 || iw >= p.w) continue;
                            auto const* xp = &x[static_cast<std::size_t>(((n * p.h + ih) * p.w + iw) * p.c)];
                            auto const* wp = &w[static_cast<std::size_t>(((k * p.r + r) * p.s + s) * p.c)];
                            for (std::int64_t c = 0; c < p.c; ++c) sum += static_cast<double>(xp[c]) * wp[c];
                        }
                    }
                    y[static_cast<std::size_t>(((n * p.out_h() + oh) * p.out_w() + ow) * p.k + k)] = sum;
                }
    return y;
}

struct DeviceBuffer {
    void* pointer = nullptr;
    explicit DeviceBuffer(std::size_t bytes) {
        if (bytes != 0 && cudaMalloc(&pointer, bytes) != cudaSuccess) pointer = nullptr;
    }
    ~DeviceBuffer() { cudaFree(pointer); }
    DeviceBuffer(DeviceBuffer const&) = delete;
    DeviceBuffer& operator=(DeviceBuffer const&) = delete;
};

bool cuda_ok(cudaError_t error, char const* what) {
    if (error == cudaSuccess) return true;
    std::cerr << what << ": " << cudaGetErrorString(error) << '\n';
    return false;
}

int run_profile(Shape const& p, int iterations, deepforge::compiler::Conv2DSchedulePolicy policy, std::string_view policy_name) {
    deepforge::compiler::CompileOptions options;
    options.emit_object = false;
    options.emit_llvm_ir = false;
    options.schedule_policy = policy;
    deepforge::compiler::CompilationResult compilation;
    auto const compile_begin = std::chrono::steady_clock::now();
    auto status = deepforge::compiler::compile_graph(graph_of(p), options, compilation);
    auto const compile_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - compile_begin).count();
    if (status.is_bad()) {
        std::cerr << status.message() << '\n';
        return 1;
    }
    auto const& meta = compilation.metadata;
    auto count = [](std::array<std::int64_t, 4> const& shape) { return static_cast<std::size_t>(shape[0] * shape[1] * shape[2] * shape[3]); };
    std::vector<float> x(count(meta.x_shape)), w(count(meta.w_shape)), y(count(meta.y_shape));
    for (std::size_t i = 0; i < x.size(); ++i) x[i] = static_cast<float>((static_cast<int>(i * 13) % 37) - 18) / 17.0F;
    for (std::size_t i = 0; i < w.size(); ++i) w[i] = static_cast<float>((static_cast<int>(i * 11) % 31) - 15) / 19.0F;
    auto const workspace_bytes = compilation.executable->get_workspace_size();
    if (workspace_bytes < 0 || workspace_bytes % 64 != 0) {
        std::cerr << "invalid workspace size\n";
        return 1;
    }
    DeviceBuffer dx(x.size() * 4), dw(w.size() * 4), dy(y.size() * 4), workspace(static_cast<std::size_t>(workspace_bytes));
    if (!dx.pointer || !dw.pointer || !dy.pointer || (workspace_bytes != 0 && !workspace.pointer)) {
        std::cerr << "device allocation failed\n";
        return 1;
    }
    cudaStream_t stream = nullptr;
    if (!cuda_ok(cudaStreamCreate(&stream), "stream")) return 1;
    compilation.executable->set_stream(stream);
    if (!cuda_ok(cudaMemcpyAsync(dx.pointer, x.data(), x.size() * 4, cudaMemcpyHostToDevice, stream), "upload X") ||
        !cuda_ok(cudaMemcpyAsync(dw.pointer, w.data(), w.size() * 4, cudaMemcpyHostToDevice, stream), "upload W"))
        return 1;
    deepforge::runtime::VariantPack pack{{meta.x_uid, dx.pointer}, {meta.w_uid, dw.pointer}, {meta.y_uid, dy.pointer}};
    auto execute = [&] { return compilation.executable->execute(nullptr, pack, workspace.pointer); };

    // the compared pass
    if ((status = execute()).is_bad()) {
        std::cerr << status.message() << '\n';
        return 1;
    }
    if (!cuda_ok(cudaMemcpyAsync(y.data(), dy.pointer, y.size() * 4, cudaMemcpyDeviceToHost, stream), "download Y") ||
        !cuda_ok(cudaStreamSynchronize(stream), "compared pass"))
        return 1;
    auto const reference = host_convolution(p, x, w);
    double max_absolute = 0.0, max_relative = 0.0;
    for (std::size_t i = 0; i < y.size(); ++i) {
        if (!std::isfinite(y[i])) {
            std::cerr << "numeric mismatch for " << p.name << ": non-finite output\n";
            return 1;
        }
        auto const absolute = std::fabs(static_cast<double>(y[i]) - reference[i]);
        max_absolute = std::max(max_absolute, absolute);
        max_relative = std::max(max_relative, absolute / std::max(std::fabs(reference[i]), 1.0e-30));
        if (absolute > 1.0e-4 + 1.0e-3 * std::fabs(reference[i])) {
            std::cerr << "numeric mismatch for " << p.name << " at element " << i << '\n';
            return 1;
        }
    }

    // the timed passes
    cudaEvent_t begin = nullptr, end = nullptr;
    if (!cuda_ok(cudaEventCreate(&begin), "event") || !cuda_ok(cudaEventCreate(&end), "event")) return 1;
    for (int i = 0; i < 3; ++i)
        if ((status = execute()).is_bad()) break;
    cudaEventRecord(begin, stream);
    for (int i = 0; i < iterations && status.is_good(); ++i) status = execute();
    cudaEventRecord(end, stream);
    if (status.is_bad()) {
        std::cerr << status.message() << '\n';
        return 1;
    }
    if (!cuda_ok(cudaEventSynchronize(end), "timed passes")) return 1;
    float total_ms = 0.0F;
    cudaEventElapsedTime(&total_ms, begin, end);
    cudaEventDestroy(begin);
    cudaEventDestroy(end);
    cudaStreamDestroy(stream);
    double const milliseconds = total_ms / iterations;
    double const operations = 2.0 * p.n * p.out_h() * p.out_w() * p.k * p.r * p.s * p.c;
    std::cout << p.name << ',' << policy_name << ",sm_100a," << compilation.variants[0].schedule << ',' << p.n << 'x' << p.h << 'x' << p.w << 'x' << p.c << "_k" << p.k << "_r" << p.r
              << 'x' << p.s << ',' << compilation.workspace.size_bytes << ',' << iterations << ',' << std::fixed << std::setprecision(3) << compile_ms << ','
              << std::setprecision(5) << milliseconds << ',' << std::setprecision(3) << operations / (milliseconds * 1.0e6) << ',' << std::scientific << max_absolute << ','
              << max_relative << '\n';
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    if (argc == 2 && (std::string_view(argv[1]) == "--help" || std::string_view(argv[1]) == "-h")) {
        usage(std::cout);
        return 0;
    }
    Arguments arguments;
    if (!read_arguments(argc, argv, arguments)) {
        usage(std::cerr);
        return 2;
    }
    int devices = 0;
    if (cudaGetDeviceCount(&devices) != cudaSuccess || devices == 0) {
        std::cerr << "deepforge-benchmark: no CUDA device (this backend has no CPU path)\n";
        return 1;
    }
    std::cout << "profile,policy,variant,schedule,shape,workspace_bytes,iterations,compile_ms,execute_ms,gflops,max_abs,max_rel\n";
    for (auto const& shape : kShapes) {
        if (arguments.profile != "all" && arguments.profile != shape.name) continue;
        if ((arguments.schedule == "baseline" || arguments.schedule == "both") &&
            run_profile(shape, arguments.iterations, deepforge::compiler::Conv2DSchedulePolicy::kBaseline, "baseline") != 0)
            return 1;
        if ((arguments.schedule == "auto" || arguments.schedule == "both") &&
            run_profile(shape, arguments.iterations, deepforge::compiler::Conv2DSchedulePolicy::kAuto, "auto") != 0)
            return 1;
    }
    return 0;
}
