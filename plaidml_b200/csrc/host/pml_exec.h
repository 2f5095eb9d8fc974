// The `cuda` target and device: planning of a program into kernel steps and its execution.
//
// Stands where the reference has pmlc/target/x86 (pipeline.cc:259-402: bounds, padding,
// stencil recognition, gemm+bias+relu combining) and pmlc/rt (jit_executable.cc:340-526:
// argument binding, one-time constant packing, invoke).  Differences by design:
//   - recognition works on the bounded contraction's per-tensor strides, like the
//     reference's GEMM stencil (pmlc/dialect/pxa/transforms/stencil_gemm.cc:296-321), but
//     selects a whole-problem kernel instead of a tile size;
//   - every value lives in device memory between steps; host buffers are touched only by
//     the input upload and the output download of plaidml_executable_run;
//   - there is no CPU execution path: a contraction no specialised kernel covers runs on the
//     general CUDA contraction kernel.
#pragma once

#include <cuda_runtime.h>

#include <functional>
#include <memory>
#include <string>
#include <vector>

#include "pml_program.h"
#include "pmlb_kernels.h"

namespace pml {

struct Step {
  std::string kernel;   // kernel family, e.g. "tc_gemm"
  std::string detail;   // human-readable description (operation name, shape, fusions)
  pmlb_plan* plan = nullptr;
  int launches = 1;     // kernel launches this step enqueues
  int position = -1;    // program position (index of the last operation fused into the step)
  std::function<pmlb_status(cudaStream_t)> launch;
  // GEMM steps whose A operand is a program input and whose product is a program output, with
  // nothing else reading or feeding them: rows of A / C can be processed in slices.
  bool rowSliceable = false;
  pmlb_gemm_desc gemm{};
  int aInput = -1;      // index into the program's inputs
  int cOutput = -1;     // index into the program's outputs
  const void* bPtr = nullptr;
  const void* biasPtr = nullptr;
};

class Executable {
 public:
  Executable(std::shared_ptr<Program> program, int device);
  ~Executable();
  Executable(const Executable&) = delete;
  Executable& operator=(const Executable&) = delete;

  double run(const std::vector<BufferPtr>& inputs, const std::vector<BufferPtr>& outputs);
  double runResident(size_t iters);
  // Mean milliseconds of one pass of the kernel sequence, each pass timed by its own event pair;
  // with flushL2 a 256 MiB buffer is overwritten before every pass (outside the timed span).
  double timeSteps(size_t iters, bool flushL2, double* perPassMs = nullptr);
  // Sharded mode (pml_shard.h).  A replicated input is uploaded as this rank's 1 / world slice and
  // completed by one all-gather on the executable's stream; inputs whose byte size does not divide by
  // the world size are uploaded whole.
  void setInputReplicated(size_t index, bool on);
  // All ranks' copies of output `index`, concatenated in rank order in a buffer the executable owns
  // (world x nbytes, allocated at the first call): one all-gather on the executable's stream, complete
  // on return.  With iters > 1 the gather is repeated and *meanMs receives the mean device time of one.
  void* gatherOutput(size_t index, size_t* nbytes, size_t iters = 1, double* meanMs = nullptr);
  // Mean milliseconds of every kernel step on its own (`iters` launches of a step back to back, replayed
  // from a CUDA graph between one event pair, L2 optionally flushed before the first): out[i] belongs to
  // line i of describe().
  void timeEachStep(size_t iters, bool flushL2, double* out);
  size_t stepCount() const { return steps_.size(); }
  std::string describe() const;
  size_t launchCount() const;
  bool usesGraph() const { return graphState_ == 1; }
  size_t uploadGroups() const { return overlapState_ == 1 ? inputGroup_.size() : 1; }
  void* outputDevicePtr(size_t index, size_t* nbytes) const;
  cudaStream_t stream() const { return stream_; }
  const Program& program() const { return *prog_; }

 private:
  friend class Planner;
  void enqueueSteps(const std::vector<cudaEvent_t>* waits = nullptr);
  void launchStepsDirect(size_t first, size_t last);
  void captureGraph();
  void planUploadOverlap();
  bool prepareSlicedRun();
  double runSliced(const std::vector<BufferPtr>& inputs, const std::vector<BufferPtr>& outputs);
  void checkStatus();
  void uploadInput(size_t i, const BufferPtr& buf);

  std::shared_ptr<Program> prog_;
  int device_ = 0;
  cudaStream_t stream_ = nullptr;
  cudaEvent_t evStart_ = nullptr, evStop_ = nullptr;
  std::vector<cudaEvent_t> timingEvents_;   // start / stop pairs of timeSteps
  char* arena_ = nullptr;
  char* flush_ = nullptr;
  size_t arenaBytes_ = 0;
  std::vector<char*> dev_;        // device address per value id (null if never materialised)
  std::vector<void*> derived_;    // device copies of constants the planner combined (fused weights, summed biases)
  std::vector<Step> steps_;
  int* status_ = nullptr;          // device word shared by all tensor-core plans
  bool inputsResident_ = false;
  std::vector<bool> inputUsed_;    // per program input: read by a kernel step or returned (others are never uploaded)
  // The kernel sequence as a CUDA graph: captured on the second pass (the first one has done every
  // one-time host-side set-up), launched as one node list afterwards.  0 = not tried, 1 = in use, 2 = off.
  int graphState_ = 0;
  size_t passes_ = 0;
  std::vector<cudaGraphExec_t> graphs_;  // one per segment of the step list (one segment unless uploads overlap)
  // Upload / compute overlap for programs with many inputs (weights passed as inputs): the step list is cut into
  // segments, every input belongs to the segment of its first use, and a segment starts as soon as its group has
  // arrived while the later groups are still crossing the host link.  0 = not tried, 1 = in use, 2 = off.
  int overlapState_ = 0;
  std::vector<size_t> segStart_{0};             // first step of each segment
  std::vector<std::vector<size_t>> inputGroup_; // program inputs per segment
  std::vector<cudaEvent_t> groupReady_;
  cudaStream_t uploadStream_ = nullptr;
  // Sliced run of a single-GEMM program (see Executable::runSliced): 0 = not tried, 1 = in use, 2 = off.
  int slicedState_ = 0;
  std::vector<pmlb_plan*> slicePlans_;
  std::vector<pmlb_plan*> blockPlans_;   // column blocks of the first row slice (B is a host input too)
  int bInput_ = -1;                      // index of B among the program's inputs, or -1
  std::vector<cudaEvent_t> sliceDone_;
  cudaStream_t copyStream_ = nullptr;
  std::vector<bool> replicated_;         // per program input (sharded mode)
  char* gathered_ = nullptr;             // world x the largest gathered output
  size_t gatheredBytes_ = 0;
};

// Device ids follow the reference's pattern name(-name)*.N (pmlc/rt/device_id.cc:13-38).
std::vector<std::string> listDevices();
int parseDeviceId(const std::string& id);  // "cuda.3" -> 3; throws on anything else
std::vector<std::string> listTargets();

}  // namespace pml

struct plaidml_executable {
  std::shared_ptr<pml::Executable> exec;
};
