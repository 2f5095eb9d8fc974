// Runs test sources of the reference checkout, compiled UNMODIFIED against the reference's own C++ headers
// (plaidml/core/core.h, edsl/edsl.h, op/op.h, exec/exec.h) and linked with this repository's libplaidml.so:
// the drop-in boundary exercised the way a user of the reference would.
//
//   ref_driver --build-only     builds and prints every program (no device needed)
//   ref_driver [--device cuda.0] builds, compiles for the `cuda` target, runs, and applies the tests' own
//                               expectations (the fixture methods below, semantics of plaidml/testenv.cc:44-156)
//
// With PMLB_REF_RESNET defined the binary also carries networks/oplib/resnet50.cc and one test that builds
// the network at batch 1 through it (zero weights: the softmax output must be uniform).
#include <chrono>
#include <cmath>
#include <cstring>
#include <iostream>

#include "plaidml/edsl/edsl.h"
#include "plaidml/exec/exec.h"
#include "plaidml/op/op.h"
#include "plaidml/testenv.h"

#ifdef PMLB_REF_RESNET
#include "networks/oplib/oplib.h"
#endif

namespace {
bool g_build_only = false;
std::string g_device = "cuda.0";
}  // namespace

namespace plaidml {

namespace {

template <typename T>
void compareExact(Buffer buffer, const std::vector<T>& expected) {
  if (buffer.size() != expected.size() * sizeof(T)) {
    ::testing::fail("output buffer has " + std::to_string(buffer.size()) + " bytes, expected " +
                    std::to_string(expected.size() * sizeof(T)));
    return;
  }
  if (std::memcmp(buffer.data(), expected.data(), buffer.size()) != 0) {
    const T* got = reinterpret_cast<const T*>(buffer.data());
    for (size_t i = 0; i < expected.size(); ++i) {
      if (!(got[i] == expected[i])) {
        ::testing::fail("element " + std::to_string(i) + ": " + std::to_string(got[i]) + " != " + std::to_string(expected[i]));
        return;
      }
    }
  }
}

template <typename T>
void compareClose(Buffer buffer, const std::vector<T>& expected, double tolerance) {
  if (buffer.size() != expected.size() * sizeof(T)) {
    ::testing::fail("output buffer size mismatch");
    return;
  }
  const T* got = reinterpret_cast<const T*>(buffer.data());
  for (size_t i = 0; i < expected.size(); ++i) {
    const double x = static_cast<double>(got[i]), y = static_cast<double>(expected[i]);
    if (std::isfinite(x) && std::isfinite(y) ? std::fabs(x - y) > (std::fabs(x) + std::fabs(y)) * tolerance : !(x == y)) {
      ::testing::fail("element " + std::to_string(i) + ": " + std::to_string(x) + " vs " + std::to_string(y));
      return;
    }
  }
}

std::vector<Buffer> runOn(Program program, const TensorBuffers& inputs) {
  program.compile();
  std::vector<Buffer> outputs;
  if (g_build_only) return outputs;
  std::vector<Buffer> inputBuffers;
  auto inputShapes = program.inputs();
  if (inputs.size() != inputShapes.size()) {
    ::testing::fail("program takes " + std::to_string(inputShapes.size()) + " inputs");
    return outputs;
  }
  for (size_t i = 0; i < inputs.size(); i++) {
    std::visit([&](auto&& vec) { inputBuffers.emplace_back(vec, inputShapes[i]); }, inputs[i]);
  }
  for (auto shape : program.outputs()) outputs.emplace_back(shape);
  exec::Executable(program).run(inputBuffers, outputs);
  return outputs;
}

}  // namespace

void TestFixture::checkExact(Program program, const TensorBuffers& inputs, const TensorBuffers& expected) {
  auto outputs = runOn(program, inputs);
  if (g_build_only) return;
  if (outputs.size() != expected.size()) return ::testing::fail("output count");
  for (size_t i = 0; i < expected.size(); i++) {
    std::visit([&](auto&& vec) { compareExact(outputs[i], vec); }, expected[i]);
  }
}

void TestFixture::checkClose(Program program, const TensorBuffers& inputs, const TensorBuffers& expected, double tolerance) {
  auto outputs = runOn(program, inputs);
  if (g_build_only) return;
  if (outputs.size() != expected.size()) return ::testing::fail("output count");
  for (size_t i = 0; i < expected.size(); i++) {
    std::visit([&](auto&& vec) { compareClose(outputs[i], vec, tolerance); }, expected[i]);
  }
}

Program TestFixture::makeProgram(const std::string& name, const std::vector<edsl::Tensor>& inputs,
                                 const std::vector<edsl::Tensor>& outputs) {
  auto program = edsl::buildProgram(name, inputs, outputs);
  writeForFileCheck(program);
  return program;
}

void TestFixture::writeForFileCheck(const Program& program) {
  if (g_build_only) std::cout << program << std::endl;
}

void TestFixture::runProgram(Program program) {
  program.compile();
  if (g_build_only) return;
  std::vector<Buffer> inputs, outputs;
  for (const TensorShape& shape : program.inputs()) inputs.emplace_back(shape);
  for (const TensorShape& shape : program.outputs()) outputs.emplace_back(shape);
  exec::Executable(program).run(inputs, outputs);
}

}  // namespace plaidml

#ifdef PMLB_REF_RESNET
class ReferenceNetworks : public plaidml::TestFixture {};

TEST_F(ReferenceNetworks, Resnet50Batch1) {
  auto program = networks::oplib::buildResnet50(1);
  program.compile();
  std::cout << "  resnet50: " << program.inputs().size() << " inputs, " << program.outputs().size() << " output" << std::endl;
  // (the image, and the 54 weight and 54 bias constants the builder also lists as inputs)
  if (program.inputs().size() != 109 || program.outputs().size() != 1) return ::testing::fail("argument counts");
  if (g_build_only) return;
  std::vector<plaidml::Buffer> inputs, outputs;
  for (const auto& shape : program.inputs()) inputs.emplace_back(shape);
  for (const auto& shape : program.outputs()) outputs.emplace_back(shape);
  plaidml::exec::Executable(program).run(inputs, outputs);
  // all weights and biases of the reference's builder are zero-filled constants: every logit is 0
  const float* p = reinterpret_cast<const float*>(outputs[0].data());
  for (int i = 0; i < 1000; ++i) {
    if (std::fabs(p[i] - 1e-3f) > 1e-8f) return ::testing::fail("softmax of zero logits must be 1/1000, got " + std::to_string(p[i]));
  }
}
#endif

int main(int argc, char** argv) {
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    if (a == "--build-only") g_build_only = true;
    if (a == "--device" && i + 1 < argc) g_device = argv[++i];
  }
  plaidml::init();
  plaidml::edsl::init();
  plaidml::op::init();
  plaidml::exec::init();
  plaidml::Settings::set("PLAIDML_DEVICE", g_device);
  plaidml::Settings::set("PLAIDML_TARGET", "cuda");
  int ran = 0;
  for (auto& entry : ::testing::Registry::tests()) {
    std::cout << "[ RUN ] " << entry.name << std::endl;
    const int before = ::testing::Registry::failures();
    const auto started = std::chrono::steady_clock::now();
    try {
      std::unique_ptr<::testing::Test> t(entry.make());
      t->SetUp();
      t->TestBody();
      t->TearDown();
    } catch (const std::exception& e) {
      ::testing::fail(std::string("exception: ") + e.what());
    }
    const double ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - started).count();
    std::cout << (::testing::Registry::failures() == before ? "[  OK ] " : "[ FAIL] ") << entry.name << " (" << static_cast<long>(ms)
              << " ms)" << std::endl;
    ++ran;
  }
  std::cout << ran << " tests, " << ::testing::Registry::failures() << " failures" << (g_build_only ? " (build only)" : "") << std::endl;
  return ::testing::Registry::failures() == 0 ? 0 : 1;
}
