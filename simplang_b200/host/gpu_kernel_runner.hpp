// gpu_kernel_runner.hpp -- C++ host driver for libsimp_gpu.so, the counterpart of the reference's
// KernelRunner / ProfiledKernelRunner (runtime/include/kernel_runner.hpp:11-109, runtime/src/host.cpp:11-148):
// same life cycle (loadLibrary -> run -> statistics / CSV), same error behaviour (std::runtime_error on a
// missing library or symbol), with the ops resolved from the C-ABI and timing taken with CUDA events on the
// library stream instead of std::chrono around a CPU call.  Header-only; link with -ldl.
#pragma once
#include <dlfcn.h>

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <fstream>
#include <functional>
#include <iostream>
#include <stdexcept>
#include <string>
#include <vector>

namespace simp_gpu {

class GpuKernelRunner {
 public:
  GpuKernelRunner() = default;
  virtual ~GpuKernelRunner() {
    if (handle_) dlclose(handle_);
  }
  GpuKernelRunner(const GpuKernelRunner&) = delete;
  GpuKernelRunner& operator=(const GpuKernelRunner&) = delete;

  // Loads the runtime library and initialises `device`.  Throws like KernelRunner::loadLibrary.
  void loadLibrary(const std::string& path, int device = 0) {
    if (handle_) {
      dlclose(handle_);
      handle_ = nullptr;
    }
    handle_ = dlopen(path.c_str(), RTLD_NOW | RTLD_GLOBAL);
    if (!handle_) throw std::runtime_error("Failed to load library: " + std::string(dlerror()));
    last_error_ = sym<const char* (*)()>("simp_gpu_last_error");
    check(sym<int (*)(int)>("simp_gpu_init")(device), "simp_gpu_init");
  }

  // Resolves an entry point; throws if it is missing (KernelRunner: "Could not find kernel_main symbol").
  template <typename Fn>
  Fn sym(const char* name) const {
    if (!handle_) throw std::runtime_error("No library loaded");
    dlerror();
    void* p = dlsym(handle_, name);
    if (!p) throw std::runtime_error("Could not find symbol " + std::string(name));
    return reinterpret_cast<Fn>(p);
  }

  // Turns a non-zero status into the exception a reference host expects.
  void check(int status, const char* what) const {
    if (status != 0)
      throw std::runtime_error(std::string(what) + " failed (" + std::to_string(status) + "): " +
                               (last_error_ ? last_error_() : "?"));
  }

  void* alloc(size_t bytes) {
    void* p = nullptr;
    check(sym<int (*)(void**, size_t)>("simp_gpu_alloc")(&p, bytes), "simp_gpu_alloc");
    return p;
  }
  void free(void* p) { check(sym<int (*)(void*)>("simp_gpu_free")(p), "simp_gpu_free"); }
  void upload(void* dst, const void* src, size_t bytes) {
    check(sym<int (*)(void*, const void*, size_t)>("simp_gpu_upload")(dst, src, bytes), "simp_gpu_upload");
  }
  void download(void* dst, const void* src, size_t bytes) {
    check(sym<int (*)(void*, const void*, size_t)>("simp_gpu_download")(dst, src, bytes), "simp_gpu_download");
  }
  void sync() { check(sym<int (*)()>("simp_gpu_sync")(), "simp_gpu_sync"); }

 protected:
  void* handle_ = nullptr;
  const char* (*last_error_)() = nullptr;
};

// Warm-up + timed iterations of one enqueue function, CUDA-event timed, with the statistics and CSV
// export of the reference's ExecutionMetrics (runtime/src/host.cpp:11-93).
class ProfiledGpuKernelRunner {
 public:
  ProfiledGpuKernelRunner(GpuKernelRunner& runner, size_t warmup = 10, size_t total = 100, bool verbose = false)
      : runner_(runner), warmup_(warmup), total_(total), verbose_(verbose) {}

  // `enqueue` launches the work on the library stream; returns the mean time in microseconds.
  double runBenchmark(const std::string& name, const std::function<void()>& enqueue) {
    auto ev_create = runner_.sym<int (*)(void**)>("simp_gpu_event_create");
    auto ev_record = runner_.sym<int (*)(void*)>("simp_gpu_event_record");
    auto ev_elapsed = runner_.sym<int (*)(void*, void*, float*)>("simp_gpu_event_elapsed_ms");
    auto ev_destroy = runner_.sym<int (*)(void*)>("simp_gpu_event_destroy");
    if (verbose_) std::cout << "Running kernel: " << name << "\nWarming up...\n";
    for (size_t i = 0; i < warmup_; ++i) enqueue();
    runner_.sync();
    std::vector<void*> ev(total_ + 1);
    for (auto& e : ev) runner_.check(ev_create(&e), "simp_gpu_event_create");
    runner_.check(ev_record(ev[0]), "simp_gpu_event_record");
    for (size_t i = 0; i < total_; ++i) {
      enqueue();
      runner_.check(ev_record(ev[i + 1]), "simp_gpu_event_record");
    }
    runner_.sync();
    us_.clear();
    for (size_t i = 0; i < total_; ++i) {
      float ms = 0;
      runner_.check(ev_elapsed(ev[i], ev[i + 1], &ms), "simp_gpu_event_elapsed_ms");
      us_.push_back(double(ms) * 1e3);
    }
    for (auto e : ev) ev_destroy(e);
    name_ = name;
    return mean();
  }

  double mean() const {
    double s = 0;
    for (double v : us_) s += v;
    return us_.empty() ? 0 : s / double(us_.size());
  }
  double minimum() const { return us_.empty() ? 0 : *std::min_element(us_.begin(), us_.end()); }

  void printStatistics() const {
    double m = mean(), var = 0;
    for (double v : us_) var += (v - m) * (v - m);
    std::vector<double> sorted(us_);
    std::sort(sorted.begin(), sorted.end());
    std::cout << "\nPerformance Statistics (" << name_ << "):\n"
              << "  Iterations: " << us_.size() << "\n  Mean:   " << m << " us\n  Min:    " << sorted.front()
              << " us\n  Median: " << sorted[sorted.size() / 2] << " us\n  Max:    " << sorted.back()
              << " us\n  StdDev: " << std::sqrt(var / double(us_.size())) << " us\n";
  }

  void exportCSV(const std::string& path = "kernel_profile.csv") const {
    std::ofstream f(path);
    f << "iteration,duration_us\n";
    for (size_t i = 0; i < us_.size(); ++i) f << i << "," << us_[i] << "\n";
  }

 private:
  GpuKernelRunner& runner_;
  size_t warmup_, total_;
  bool verbose_;
  std::vector<double> us_;
  std::string name_;
};

}  // namespace simp_gpu
