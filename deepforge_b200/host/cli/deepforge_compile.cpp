// deepforge-compile for this backend: a serialized graph in, an artifact (.dfo) out, or --inspect of an artifact.
// Same command line, output lines and exit codes as the reference's tool (tools/deepforge-compile.cpp:50-63 usage,
// :385-411 --inspect, :415-474 run: 0 done, 1 the compilation or a file operation failed, 2 the command line is wrong);
// what differs is what a GPU backend has to offer: the target is sm_100a, --emit takes `artifact` or `plan` (the
// kernel plan as text, where the reference emits LLVM IR) and --dump-plan=PATH stands where --dump-ir does.
#include "DeepForge/Compiler/Artifact.h"

#include <atomic>
#include <fstream>
#include <iostream>
#include <optional>
#include <string>
#include <string_view>
#include <system_error>
#include <unistd.h>
#include <vector>

namespace {

enum class EmitKind { kArtifact, kPlan };

struct Options {
    std::filesystem::path input;
    std::filesystem::path output;
    deepforge::import::InputFormat input_format = deepforge::import::InputFormat::kAuto;
    EmitKind emit = EmitKind::kArtifact;
    std::vector<std::filesystem::path> plan_dumps;
    std::optional<std::filesystem::path> inspect;
    bool fuse = true;
    bool tensor_cores = true;
};

void print_usage(std::ostream& stream) {
    stream << "usage: deepforge-compile <graph.json|graph.ubjson> [options]\n"
           << "       deepforge-compile --inspect <artifact.dfo>\n\n"
           << "options:\n"
           << "  --input-format=auto|json|ubjson\n"
           << "  --target=sm_100a\n"
           << "  --emit=artifact|plan\n"
           << "  --dump-plan=PATH               the kernel plan, one line per launch\n"
           << "  --no-fusion                    one launch per graph node\n"
           << "  --no-tensor-cores              CUDA-core kernels only\n"
           << "  -o PATH, --output=PATH\n"
           << "  --help\n"
           << "  --version\n";
}

std::optional<std::string_view> inline_value(std::string_view argument, std::string_view option) {
    if (argument.size() > option.size() && argument.starts_with(option) && argument[option.size()] == '=') return argument.substr(option.size() + 1);
    return std::nullopt;
}

bool parse_input_format(std::string_view value, deepforge::import::InputFormat& format) {
    if (value == "auto") format = deepforge::import::InputFormat::kAuto;
    else if (value == "json") format = deepforge::import::InputFormat::kJson;
    else if (value == "ubjson") format = deepforge::import::InputFormat::kUbjson;
    else return false;
    return true;
}

// An option given as "--name value" or "--name=value"; `handled` says whether `argument` was this option at all.
bool take_value(std::string_view name, int argc, char** argv, int& index, std::string_view argument, std::optional<std::string_view>& value,
                bool& handled, std::string& error) {
    handled = false;
    if (argument == name) {
        handled = true;
        if (index + 1 >= argc) {
            error = std::string(name) + " requires a value";
            return false;
        }
        value = argv[++index];
        return true;
    }
    if (auto inline_form = inline_value(argument, name)) {
        handled = true;
        value = inline_form;
    }
    return true;
}

bool parse_options(int argc, char** argv, Options& out, std::string& error, bool& done) {
    bool compile_option_seen = false;
    for (int index = 1; index < argc; ++index) {
        std::string_view argument = argv[index];
        if (argument == "--help") {
            print_usage(std::cout);
            done = true;
            return true;
        }
        if (argument == "--version") {
            std::cout << "deepforge-compile (deepforge_b200) format DFOBJ/" << deepforge::compiler::kArtifactFormatVersion << " target sm_100a\n";
            done = true;
            return true;
        }
        std::optional<std::string_view> value;
        bool handled = false;
        if (!take_value("-o", argc, argv, index, argument, value, handled, error)) return false;
        if (!handled && !take_value("--output", argc, argv, index, argument, value, handled, error)) return false;
        if (handled) {
            if (value->empty()) {
                error = "output path must not be empty";
                return false;
            }
            out.output = *value;
            compile_option_seen = true;
            continue;
        }
        if (!take_value("--input-format", argc, argv, index, argument, value, handled, error)) return false;
        if (handled) {
            if (!parse_input_format(*value, out.input_format)) {
                error = "--input-format must be auto, json, or ubjson";
                return false;
            }
            compile_option_seen = true;
            continue;
        }
        if (!take_value("--target", argc, argv, index, argument, value, handled, error)) return false;
        if (handled) {
            if (*value != "sm_100a") {
                error = "--target must be sm_100a";
                return false;
            }
            compile_option_seen = true;
            continue;
        }
        if (!take_value("--emit", argc, argv, index, argument, value, handled, error)) return false;
        if (handled) {
            if (*value == "artifact") out.emit = EmitKind::kArtifact;
            else if (*value == "plan") out.emit = EmitKind::kPlan;
            else {
                error = "--emit must be artifact or plan";
                return false;
            }
            compile_option_seen = true;
            continue;
        }
        if (!take_value("--dump-plan", argc, argv, index, argument, value, handled, error)) return false;
        if (handled) {
            if (value->empty()) {
                error = "--dump-plan requires a path";
                return false;
            }
            out.plan_dumps.emplace_back(*value);
            compile_option_seen = true;
            continue;
        }
        if (!take_value("--inspect", argc, argv, index, argument, value, handled, error)) return false;
        if (handled) {
            if (value->empty() || out.inspect) {
                error = "--inspect requires exactly one path";
                return false;
            }
            out.inspect = std::filesystem::path(*value);
            continue;
        }
        if (argument == "--no-fusion" || argument == "--no-tensor-cores") {
            (argument == "--no-fusion" ? out.fuse : out.tensor_cores) = false;
            compile_option_seen = true;
            continue;
        }
        if (argument.starts_with("-")) {
            error = "unknown option: " + std::string(argument);
            return false;
        }
        if (!out.input.empty()) {
            error = "multiple input files are not supported";
            return false;
        }
        out.input = argument;
    }
    if (out.inspect) {
        if (compile_option_seen || !out.input.empty()) {
            error = "--inspect cannot be combined with compilation options";
            return false;
        }
        return true;
    }
    if (out.input.empty()) {
        error = "an input graph is required";
        return false;
    }
    if (out.output.empty()) {
        out.output = out.input;
        out.output.replace_extension(out.emit == EmitKind::kArtifact ? ".dfo" : ".plan");
    }
    return true;
}

std::atomic<unsigned long long> g_sequence{0};

// Text files are published like artifacts: a temporary file beside the destination, then rename.
bool write_text(std::filesystem::path const& path, std::string const& text, std::string& error) {
    auto temporary = path;
    temporary += ".tmp." + std::to_string(static_cast<long long>(::getpid())) + "." + std::to_string(g_sequence.fetch_add(1));
    {
        std::ofstream file(temporary, std::ios::binary | std::ios::trunc);
        if (!file) {
            error = "cannot create " + temporary.string();
            return false;
        }
        file << text;
        file.flush();
        if (!file) {
            error = "short write to " + temporary.string();
            std::error_code ignored;
            std::filesystem::remove(temporary, ignored);
            return false;
        }
    }
    std::error_code code;
    std::filesystem::rename(temporary, path, code);
    if (code) {
        error = "cannot publish " + path.string() + ": " + code.message();
        std::error_code ignored;
        std::filesystem::remove(temporary, ignored);
        return false;
    }
    return true;
}

int inspect_artifact(std::filesystem::path const& path) {
    deepforge::compiler::ArtifactInfo artifact;
    auto status = deepforge::compiler::read_artifact(path, artifact);
    if (status.is_bad()) {
        std::cerr << status.message() << '\n';
        return 1;
    }
    std::cout << "format: DFOBJ/" << artifact.format_version << "\n"
              << "deepforge: " << artifact.deepforge_version << "\n"
              << "llvm: " << artifact.llvm_version << "\n"
              << "frontend: " << artifact.frontend_version << "\n"
              << "target: " << artifact.target_triple << "\n"
              << "function: " << artifact.metadata.function_name << "\n"
              << "uids: ";
    for (std::size_t i = 0; i < artifact.metadata.arguments.size(); ++i) std::cout << (i ? "," : "") << artifact.metadata.arguments[i].uid;
    std::cout << "\nworkspace: " << artifact.workspace.size_bytes << " bytes\n";
    for (auto const& step : artifact.plan.steps) {
        std::cout << "launch: [" << step.label << "] entry=" << static_cast<int>(step.op) << " kernel=" << step.kernel << " launches=" << step.launches
                  << " tensors=" << step.tensors.size() << '\n';
    }
    return 0;
}

int run(int argc, char** argv) {
    Options options;
    std::string error;
    bool done = false;
    if (!parse_options(argc, argv, options, error, done)) {
        std::cerr << "deepforge-compile: " << error << '\n';
        print_usage(std::cerr);
        return 2;
    }
    if (done) return 0;
    if (options.inspect) return inspect_artifact(*options.inspect);

    deepforge::compiler::CompileOptions compile_options;
    compile_options.input_format = options.input_format;
    compile_options.fuse = options.fuse;
    compile_options.disable_tensor_cores = !options.tensor_cores;
    deepforge::compiler::CompilationResult compilation;
    auto status = deepforge::compiler::compile_file(options.input, compile_options, compilation);
    if (status.is_bad()) {
        std::cerr << status.message() << '\n';
        return 1;
    }
    auto const plan_text = compilation.plan.to_text();
    for (auto const& path : options.plan_dumps) {
        if (!write_text(path, plan_text, error)) {
            std::cerr << "deepforge-compile: " << error << '\n';
            return 1;
        }
    }
    if (options.emit == EmitKind::kArtifact) {
        status = deepforge::compiler::write_artifact(options.output, compilation);
        if (status.is_bad()) {
            std::cerr << status.message() << '\n';
            return 1;
        }
    } else if (!write_text(options.output, plan_text, error)) {
        std::cerr << "deepforge-compile: " << error << '\n';
        return 1;
    }
    std::cout << "output: " << options.output << '\n'
              << "target: " << compilation.target_triple << '\n'
              << "workspace: " << compilation.workspace.size_bytes << " bytes\n";
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    try {
        return run(argc, argv);
    } catch (std::exception const& exception) {
        std::cerr << "deepforge-compile: " << exception.what() << '\n';
        return 1;
    }
}
