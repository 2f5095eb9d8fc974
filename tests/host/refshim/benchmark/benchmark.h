// A few lines standing in for Google Benchmark, so that networks/oplib/benchmark.cc of the reference checkout compiles
// and runs unmodified against libplaidml.so: fixtures registered with BENCHMARK_DEFINE_F / BENCHMARK_REGISTER_F, a
// State whose range-for loop runs a fixed number of iterations (PMLB_BENCH_ITERS, default 30) and times each one.
// Reported per benchmark: iterations, median and mean milliseconds per iteration after three warm-up iterations.
#pragma once

#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdlib>
#include <functional>
#include <iostream>
#include <string>
#include <vector>

namespace benchmark {

enum TimeUnit { kNanosecond, kMicrosecond, kMillisecond, kSecond };

class State {
 public:
  struct Unused {};
  struct Iterator {
    State* state;
    bool operator!=(const Iterator&) const { return state->KeepRunning(); }
    void operator++() {}
    Unused operator*() const { return {}; }
  };
  explicit State(int64_t max_iterations) : max_(max_iterations) {}
  Iterator begin() { return {this}; }
  Iterator end() { return {this}; }
  bool KeepRunning() {
    stamps_.push_back(std::chrono::steady_clock::now());
    return static_cast<int64_t>(stamps_.size()) <= max_;
  }
  int64_t iterations() const { return stamps_.empty() ? 0 : static_cast<int64_t>(stamps_.size()) - 1; }
  void SetItemsProcessed(int64_t) {}
  std::vector<double> milliseconds() const {
    std::vector<double> ms;
    for (size_t i = 1; i < stamps_.size(); ++i) {
      ms.push_back(std::chrono::duration<double, std::milli>(stamps_[i] - stamps_[i - 1]).count());
    }
    return ms;
  }

 private:
  int64_t max_;
  std::vector<std::chrono::steady_clock::time_point> stamps_;
};

class Fixture {
 public:
  virtual ~Fixture() = default;
  virtual void SetUp(const State&) {}
  virtual void TearDown(const State&) {}
  virtual void BenchmarkCase(State&) = 0;
};

struct Registered {
  std::string name;
  std::function<Fixture*()> make;
  Registered* Unit(TimeUnit) { return this; }
  Registered* UseRealTime() { return this; }
  Registered* UseManualTime() { return this; }
  Registered* Iterations(int64_t) { return this; }
};

inline std::vector<Registered*>& registry() {
  static std::vector<Registered*> r;
  return r;
}

inline Registered* Register(const std::string& name, std::function<Fixture*()> make) {
  registry().push_back(new Registered{name, std::move(make)});
  return registry().back();
}

inline void Initialize(int*, char**) {}
inline bool ReportUnrecognizedArguments(int, char**) { return false; }

inline size_t RunSpecifiedBenchmarks() {
  const char* env = std::getenv("PMLB_BENCH_ITERS");
  const int64_t iters = env ? std::atoll(env) : 30;
  for (Registered* r : registry()) {
    Fixture* f = r->make();
    State state(iters);
    f->SetUp(state);
    f->BenchmarkCase(state);
    f->TearDown(state);
    std::vector<double> ms = state.milliseconds();
    const size_t warm = ms.size() > 6 ? 3 : 0;
    std::vector<double> timed(ms.begin() + warm, ms.end());
    std::sort(timed.begin(), timed.end());
    double sum = 0;
    for (double v : timed) sum += v;
    std::cout << r->name << ": " << state.iterations() << " iterations, median "
              << (timed.empty() ? 0.0 : timed[timed.size() / 2]) << " ms, mean " << (timed.empty() ? 0.0 : sum / timed.size())
              << " ms per iteration (first " << warm << " dropped)" << std::endl;
    delete f;
  }
  return registry().size();
}

}  // namespace benchmark

#define BENCHMARK_DEFINE_F(fixture, method)                         \
  class fixture##_##method##_Benchmark : public fixture {           \
   public:                                                          \
    void BenchmarkCase(::benchmark::State&) override;               \
  };                                                                \
  void fixture##_##method##_Benchmark::BenchmarkCase

#define BENCHMARK_REGISTER_F(fixture, method)                                                                 \
  static ::benchmark::Registered* fixture##_##method##_registered = ::benchmark::Register(                    \
      #fixture "/" #method, [] { return static_cast<::benchmark::Fixture*>(new fixture##_##method##_Benchmark()); })
