// C ABI: devices, JIT and run.  Reference counterparts: plaidml/exec/ffi.cc:42-123.
#include <mutex>

#include "pml_exec.h"
#include "pml_shard.h"

using pml::ffiWrap;
using pml::ffiWrapVoid;

extern "C" {

void plaidml_exec_init(plaidml_error* err) {
  ffiWrapVoid(err, [&] {});
}

plaidml_strings* plaidml_devices_get(plaidml_error* err) {
  return ffiWrap<plaidml_strings*>(err, nullptr, [&] {
    std::vector<plaidml_string*> out;
    for (const std::string& d : pml::listDevices()) out.push_back(new plaidml_string{d});
    return pml::makeList<plaidml_strings, plaidml_string*>(out);
  });
}

plaidml_executable* plaidml_jit(plaidml_error* err, plaidml_program* program, const char* raw_device) {
  return ffiWrap<plaidml_executable*>(err, nullptr, [&] {
    std::string device(raw_device ? raw_device : "");
    if (device.empty()) device = pml::Settings::instance().get("PLAIDML_DEVICE");
    if (!program->program->compiled) {
      throw std::runtime_error("Program must be compiled (plaidml_program_compile) before plaidml_jit");
    }
    const int index = pml::parseDeviceId(device);
    return new plaidml_executable{std::make_shared<pml::Executable>(program->program, index)};
  });
}

void plaidml_executable_free(plaidml_error* err, plaidml_executable* exec) {
  ffiWrapVoid(err, [&] { delete exec; });
}

double plaidml_executable_run(plaidml_error* err, plaidml_executable* exec, size_t ninputs, plaidml_buffer** inputs,
                              size_t noutputs, plaidml_buffer** outputs) {
  return ffiWrap<double>(err, 0.0, [&] {
    std::vector<pml::BufferPtr> ins, outs;
    for (size_t i = 0; i < ninputs; ++i) ins.push_back(inputs[i]->buffer);
    for (size_t i = 0; i < noutputs; ++i) outs.push_back(outputs[i]->buffer);
    return exec->exec->run(ins, outs);
  });
}

plaidml_string* pmlb_exec_describe(plaidml_error* err, plaidml_executable* exec) {
  return ffiWrap<plaidml_string*>(err, nullptr, [&] { return new plaidml_string{exec->exec->describe()}; });
}

size_t pmlb_exec_launch_count(plaidml_error* err, plaidml_executable* exec) {
  return ffiWrap<size_t>(err, 0, [&] { return exec->exec->launchCount(); });
}

int pmlb_exec_uses_graph(plaidml_error* err, plaidml_executable* exec) {
  return ffiWrap<int>(err, 0, [&] { return exec->exec->usesGraph() ? 1 : 0; });
}

size_t pmlb_exec_upload_groups(plaidml_error* err, plaidml_executable* exec) {
  return ffiWrap<size_t>(err, 0, [&] { return exec->exec->uploadGroups(); });
}

double pmlb_exec_run_resident(plaidml_error* err, plaidml_executable* exec, size_t iters) {
  return ffiWrap<double>(err, 0.0, [&] { return exec->exec->runResident(iters); });
}

double pmlb_exec_time_steps(plaidml_error* err, plaidml_executable* exec, size_t iters, bool flush_l2) {
  return ffiWrap<double>(err, 0.0, [&] { return exec->exec->timeSteps(iters, flush_l2); });
}

void* pmlb_exec_output_device_ptr(plaidml_error* err, plaidml_executable* exec, size_t index, size_t* nbytes) {
  return ffiWrap<void*>(err, nullptr, [&] { return exec->exec->outputDevicePtr(index, nbytes); });
}

void pmlb_exec_time_passes(plaidml_error* err, plaidml_executable* exec, size_t iters, bool flush_l2, double* ms_out) {
  ffiWrapVoid(err, [&] {
    if (!ms_out) throw std::runtime_error("null result array");
    exec->exec->timeSteps(iters, flush_l2, ms_out);
  });
}

size_t pmlb_exec_time_each_step(plaidml_error* err, plaidml_executable* exec, size_t iters, bool flush_l2, double* ms_out,
                                size_t capacity) {
  return ffiWrap<size_t>(err, 0, [&] {
    const size_t n = exec->exec->stepCount();
    if (ms_out && capacity >= n) exec->exec->timeEachStep(iters, flush_l2, ms_out);
    return n;
  });
}

void pmlb_shard_unique_id(plaidml_error* err, char* id) {
  ffiWrapVoid(err, [&] {
    if (!id) throw std::runtime_error("null id");
    pml::ShardComm::instance().makeUniqueId(id);
  });
}

void pmlb_shard_init(plaidml_error* err, int rank, int world, const char* id, const char* raw_device) {
  ffiWrapVoid(err, [&] {
    if (world > 1 && !id) throw std::runtime_error("null id");
    std::string device(raw_device ? raw_device : "");
    if (device.empty()) device = pml::Settings::instance().get("PLAIDML_DEVICE");
    const int index = pml::parseDeviceId(device);
    if (cudaSetDevice(index) != cudaSuccess) throw std::runtime_error("No such device: " + device);
    pml::ShardComm::instance().init(rank, world, id);
  });
}

void pmlb_shard_shutdown(plaidml_error* err) {
  ffiWrapVoid(err, [&] { pml::ShardComm::instance().shutdown(); });
}

int pmlb_shard_rank(plaidml_error* err) {
  return ffiWrap<int>(err, 0, [&] { return pml::ShardComm::instance().rank(); });
}

int pmlb_shard_world(plaidml_error* err) {
  return ffiWrap<int>(err, 1, [&] { return pml::ShardComm::instance().world(); });
}

void pmlb_exec_set_input_replicated(plaidml_error* err, plaidml_executable* exec, size_t index, int replicated) {
  ffiWrapVoid(err, [&] { exec->exec->setInputReplicated(index, replicated != 0); });
}

void* pmlb_exec_gather_output(plaidml_error* err, plaidml_executable* exec, size_t index, size_t* nbytes, size_t iters,
                              double* mean_ms) {
  return ffiWrap<void*>(err, nullptr, [&] { return exec->exec->gatherOutput(index, nbytes, iters, mean_ms); });
}

void* pmlb_exec_stream(plaidml_error* err, plaidml_executable* exec) {
  return ffiWrap<void*>(err, nullptr, [&] { return static_cast<void*>(exec->exec->stream()); });
}

}  // extern "C"
