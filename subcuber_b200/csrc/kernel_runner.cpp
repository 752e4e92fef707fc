// kernel_runner: benchmark driver with the command line and output table of the reference project's driver
// (src/cuda/kernel_runner.cpp:206-220,240-242,297-303,335-338,377-379,404-458 there), for --gpu_arch=blackwell.
//
//   kernel_runner --m=<M> --n=<N> --k=<K> --dtype=f32|f16|f64 --gpu_arch=blackwell --strassen_level=0|1|2|all
//                 --iterations=N --warmup=N --streams=N [--kernel_regex=REGEX]
//                 [--dist=harness|uniform1|normal] [--seed=S] [--cooldown_s=X] [--json]
//
// Both "--flag=value" and "--flag value" are accepted, "--level" is an alias of "--strassen_level", and the dtype /
// arch aliases of the reference are kept.  Differences, all additive: operands are filled on the device by the
// library's seeded generator (default: the reference harness' value set), the pause between kernels is a flag
// (default 0 s instead of the reference's fixed 5 / 10 s), and --json prints one machine-readable line per kernel.
// Kernels come from the library's registry (sb200_kernel), each called through its run_<kernel> C entry point.
#include <cuda_runtime.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <iomanip>
#include <iostream>
#include <limits>
#include <regex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/subcuber_b200.h"

namespace {

std::string to_lower(std::string s) {
  std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return static_cast<char>(std::tolower(c)); });
  return s;
}

std::string canonical_arch(const std::string& raw) {
  const std::string a = to_lower(raw);
  static const struct { const char* alias; const char* name; } table[] = {
      {"sm70", "volta"},      {"70", "volta"},       {"compute_70", "volta"},  {"sm80", "ampere"},
      {"80", "ampere"},       {"compute_80", "ampere"}, {"sm90", "hopper"},    {"sm90a", "hopper"},
      {"90", "hopper"},       {"90a", "hopper"},     {"compute_90a", "hopper"}, {"sm100", "blackwell"},
      {"sm100a", "blackwell"}, {"100", "blackwell"}, {"100a", "blackwell"},    {"compute_100a", "blackwell"},
      {"b200", "blackwell"}};
  for (const auto& e : table)
    if (a == e.alias) return e.name;
  return a;
}

std::string canonical_dtype(const std::string& raw) {
  const std::string d = to_lower(raw);
  if (d == "float" || d == "fp32" || d == "s") return "f32";
  if (d == "half" || d == "fp16" || d == "h") return "f16";
  if (d == "double" || d == "fp64" || d == "d") return "f64";
  if (d == "bfloat16" || d == "bf") return "bf16";
  return d;
}

// value of --name=value or --name value; false when absent
bool flag_value(int argc, char** argv, const std::string& name, std::string* out) {
  const std::string eq = "--" + name + "=";
  const std::string bare = "--" + name;
  for (int i = 1; i < argc; ++i) {
    const std::string arg = argv[i];
    if (arg.compare(0, eq.size(), eq) == 0) {
      *out = arg.substr(eq.size());
      return true;
    }
    if (arg == bare && i + 1 < argc) {
      *out = argv[i + 1];
      return true;
    }
  }
  return false;
}

bool has_flag(int argc, char** argv, const std::string& name) {
  for (int i = 1; i < argc; ++i)
    if (std::string(argv[i]) == "--" + name) return true;
  return false;
}

bool int_flag(int argc, char** argv, const std::string& name, int* out) {
  std::string v;
  if (!flag_value(argc, argv, name, &v) || v.empty()) return false;
  char* end = nullptr;
  long x = std::strtol(v.c_str(), &end, 10);
  if (*end != '\0') return false;
  *out = static_cast<int>(x);
  return true;
}

void usage(const char* prog) {
  std::cerr << "Usage: " << prog
            << " --m=<M> --n=<N> --k=<K> --dtype=f32|f16|f64 --gpu_arch=blackwell --strassen_level=0|1|2|all "
               "--iterations=N --warmup=N --streams=N [--kernel_regex=REGEX] [--dist=harness|uniform1|normal] "
               "[--seed=S] [--cooldown_s=X] [--json]\n"
               "       (--dtype also takes bf16)\n";
}

struct Options {
  int m = 0, n = 0, k = 0, iterations = 0, warmup = 0, streams = 0;
  std::string dtype, arch, level_label, regex_text, dist = "harness";
  bool all_levels = false, has_regex = false, json = false;
  int level = -1;
  unsigned long long seed = 1;
  double cooldown_s = 0.0;
};

}  // namespace

int main(int argc, char** argv) {
  if (has_flag(argc, argv, "help") || (argc > 1 && std::string(argv[1]) == "-h")) {
    usage(argv[0]);
    return 0;
  }
  Options o;
  bool ok = true;
  ok &= int_flag(argc, argv, "m", &o.m);
  ok &= int_flag(argc, argv, "n", &o.n);
  ok &= int_flag(argc, argv, "k", &o.k);
  ok &= int_flag(argc, argv, "iterations", &o.iterations);
  ok &= int_flag(argc, argv, "warmup", &o.warmup);
  ok &= int_flag(argc, argv, "streams", &o.streams);
  std::string dtype_raw, arch_raw, tmp;
  ok &= flag_value(argc, argv, "dtype", &dtype_raw) && !dtype_raw.empty();
  ok &= flag_value(argc, argv, "gpu_arch", &arch_raw) && !arch_raw.empty();
  ok &= flag_value(argc, argv, "strassen_level", &o.level_label) || flag_value(argc, argv, "level", &o.level_label);
  o.has_regex = flag_value(argc, argv, "kernel_regex", &o.regex_text);
  flag_value(argc, argv, "dist", &o.dist);
  if (flag_value(argc, argv, "seed", &tmp)) o.seed = std::strtoull(tmp.c_str(), nullptr, 10);
  if (flag_value(argc, argv, "cooldown_s", &tmp)) o.cooldown_s = std::atof(tmp.c_str());
  o.json = has_flag(argc, argv, "json");
  o.dtype = canonical_dtype(dtype_raw);
  o.arch = canonical_arch(arch_raw);
  o.level_label = to_lower(o.level_label);
  o.all_levels = o.level_label == "all";
  if (ok && !o.all_levels) {
    char* end = nullptr;
    long v = std::strtol(o.level_label.c_str(), &end, 10);
    if (o.level_label.empty() || *end != '\0') ok = false;
    o.level = static_cast<int>(v);
  }
  const int max_streams = o.all_levels ? 49 : (o.level == 0 ? 1 : (o.level == 2 ? 49 : 7));
  const int dist_code = o.dist == "uniform1" ? 0 : (o.dist == "normal" ? 1 : (o.dist == "harness" ? 2 : -1));
  std::regex re;
  if (o.has_regex) {
    try {
      re = std::regex(o.regex_text);
    } catch (const std::regex_error& e) {
      std::cerr << "Invalid --kernel_regex: " << e.what() << "\n";
      return 1;
    }
  }
  const bool known_arch = o.arch == "volta" || o.arch == "ampere" || o.arch == "hopper" || o.arch == "blackwell";
  if (!ok || o.m <= 0 || o.n <= 0 || o.k <= 0 || o.iterations <= 0 || o.warmup < 0 || o.streams <= 0 ||
      o.streams > max_streams || (o.dtype != "f32" && o.dtype != "f16" && o.dtype != "f64" && o.dtype != "bf16") || !known_arch ||
      dist_code < 0 || (!o.all_levels && (o.level < 0 || o.level > 2))) {
    usage(argv[0]);
    return 1;
  }

  std::vector<const sb200_kernel_entry*> candidates;
  for (int i = 0; i < sb200_num_kernels(); ++i) {
    const sb200_kernel_entry* e = sb200_kernel(i);
    if (o.dtype != e->dtype || o.arch != e->arch) continue;
    if (!o.all_levels && e->strassen_level != o.level) continue;
    if (o.has_regex && !std::regex_search(e->name, re)) continue;
    candidates.push_back(e);
  }
  if (candidates.empty()) {
    std::cerr << "No kernels registered for dtype=" << o.dtype << " gpu_arch=" << o.arch
              << " strassen_level=" << o.level_label;
    if (o.has_regex) std::cerr << " kernel_regex=" << o.regex_text;
    std::cerr << "\n";
    return 1;
  }

  const int dtype_code = o.dtype == "f16" ? 0 : (o.dtype == "f32" ? 1 : (o.dtype == "bf16" ? 3 : 2));
  const size_t es = (dtype_code == 0 || dtype_code == 3) ? 2 : (dtype_code == 1 ? 4 : 8);
  void *da = nullptr, *db = nullptr, *dd = nullptr;
  auto fail = [&](cudaError_t e) {
    std::cerr << "CUDA error: " << cudaGetErrorString(e) << "\n";
    cudaFree(da); cudaFree(db); cudaFree(dd);
    return static_cast<int>(e);
  };
  cudaError_t ce;
  if ((ce = cudaMalloc(&da, size_t(o.m) * o.k * es)) != cudaSuccess) return fail(ce);
  if ((ce = cudaMalloc(&db, size_t(o.k) * o.n * es)) != cudaSuccess) return fail(ce);
  if ((ce = cudaMalloc(&dd, size_t(o.m) * o.n * es)) != cudaSuccess) return fail(ce);
  int rc = sb200_fill_device(dtype_code, dist_code, o.seed, 0, da, (unsigned long long)o.m * o.k, nullptr);
  if (!rc) rc = sb200_fill_device(dtype_code, dist_code, o.seed, 1, db, (unsigned long long)o.k * o.n, nullptr);
  if (rc || (ce = cudaDeviceSynchronize()) != cudaSuccess) return fail(rc ? cudaErrorUnknown : ce);

  const int nstreams = std::max(1, std::min(o.streams, 49));
  std::vector<cudaStream_t> streams(nstreams);
  for (int i = 0; i < nstreams; ++i)
    if ((ce = cudaStreamCreate(&streams[i])) != cudaSuccess) return fail(ce);

  std::cout << "Running " << candidates.size() << " candidate kernels for m=" << o.m << " n=" << o.n << " k=" << o.k
            << " dtype=" << o.dtype << " gpu_arch=" << o.arch << " strassen_level=" << o.level_label
            << " streams=" << nstreams << "\n";
  std::cout << std::left << std::setw(52) << "kernel" << std::right << std::setw(10) << "split_k" << std::setw(14)
            << "avg_ms" << std::setw(16) << "gflops" << "\n";

  KernelRunnerBuffers buffers{da, db, nullptr, dd};
  std::string best_name;
  float best_ms = std::numeric_limits<float>::infinity();
  double best_gflops = 0.0;
  int runnable = 0;
  for (const sb200_kernel_entry* e : candidates) {
    cudaMemset(dd, 0, size_t(o.m) * o.n * es);
    float avg_ms = 0.f;
    rc = e->run(buffers, o.m, o.n, o.k, o.warmup, o.iterations, reinterpret_cast<sb200_stream_t*>(streams.data()),
                nstreams, 1, &avg_ms);
    if (o.cooldown_s > 0) std::this_thread::sleep_for(std::chrono::duration<double>(o.cooldown_s));
    if (rc != 0 || !std::isfinite(avg_ms)) {
      std::cout << std::left << std::setw(52) << e->name << std::right << std::setw(10) << 1 << std::setw(14)
                << "skipped" << std::setw(16) << rc << "\n";
      continue;
    }
    ++runnable;
    const double gflops = 2.0 * o.m * double(o.n) * o.k / (double(avg_ms) * 1.0e6);
    std::cout << std::left << std::setw(52) << e->name << std::right << std::setw(10) << 1 << std::setw(14)
              << std::fixed << std::setprecision(4) << avg_ms << std::setw(16) << std::fixed << std::setprecision(2)
              << gflops << "\n";
    if (o.json)
      std::printf("{\"kernel\": \"%s\", \"m\": %d, \"n\": %d, \"k\": %d, \"dtype\": \"%s\", \"level\": %d, "
                  "\"avg_ms\": %.6f, \"tflops\": %.3f}\n",
                  e->name, o.m, o.n, o.k, o.dtype.c_str(), e->strassen_level, avg_ms, gflops / 1000.0);
    if (avg_ms < best_ms) {
      best_ms = avg_ms;
      best_gflops = gflops;
      best_name = e->name;
    }
  }
  for (cudaStream_t s : streams) cudaStreamDestroy(s);
  cudaFree(da); cudaFree(db); cudaFree(dd);
  if (runnable == 0) {
    std::cerr << "No registered kernel could run this problem.\n";
    return 2;
  }
  std::cout << "Best kernel: " << best_name << " split_k=1 avg_ms=" << std::fixed << std::setprecision(4) << best_ms
            << " gflops=" << std::fixed << std::setprecision(2) << best_gflops << "\n";
  return 0;
}
