// C ABI: strings, library life cycle, settings, shapes, buffers, programs.
// Reference counterparts: plaidml/core/ffi.cc:45-404.
#include <cstring>
#include <mutex>

#include "pml_core.h"
#include "pml_exec.h"
#include "pml_program.h"

using pml::ffiWrap;
using pml::ffiWrapVoid;

namespace {

plaidml_kvps* makeKvps(const std::vector<std::pair<std::string, std::string>>& items) {
  auto* out = new plaidml_kvps;
  out->size = items.size();
  out->elts = new plaidml_kvp[items.size() ? items.size() : 1];
  for (size_t i = 0; i < items.size(); ++i) {
    out->elts[i].key = new plaidml_string{items[i].first};
    out->elts[i].value = new plaidml_string{items[i].second};
  }
  return out;
}

}  // namespace

extern "C" {

const char* plaidml_string_ptr(plaidml_string* str) { return str->str.c_str(); }

void plaidml_string_free(plaidml_string* str) { delete str; }

void plaidml_init(plaidml_error* err) {
  static std::once_flag once;
  ffiWrapVoid(err, [&] {
    std::call_once(once, [] { pml::Settings::instance(); });
  });
}

void plaidml_shutdown(plaidml_error* err) {
  ffiWrapVoid(err, [&] {});
}

const char* plaidml_version(plaidml_error* err) {
  return ffiWrap<const char*>(err, nullptr, [&] { return "1.0.0+b200"; });
}

void plaidml_integers_free(plaidml_error* err, plaidml_integers* ints) {
  ffiWrapVoid(err, [&] {
    delete[] ints->elts;
    delete ints;
  });
}

void plaidml_strings_free(plaidml_error* err, plaidml_strings* strs) {
  ffiWrapVoid(err, [&] {
    delete[] strs->elts;
    delete strs;
  });
}

void plaidml_kvps_free(plaidml_error* err, plaidml_kvps* kvps) {
  ffiWrapVoid(err, [&] {
    delete[] kvps->elts;
    delete kvps;
  });
}

void plaidml_shapes_free(plaidml_error* err, plaidml_shapes* shapes) {
  ffiWrapVoid(err, [&] {
    delete[] shapes->elts;
    delete shapes;
  });
}

plaidml_kvps* plaidml_settings_list(plaidml_error* err) {
  return ffiWrap<plaidml_kvps*>(err, nullptr, [&] { return makeKvps(pml::Settings::instance().all()); });
}

plaidml_string* plaidml_settings_get(plaidml_error* err, const char* key) {
  return ffiWrap<plaidml_string*>(err, nullptr, [&] { return new plaidml_string{pml::Settings::instance().get(key)}; });
}

void plaidml_settings_set(plaidml_error* err, const char* key, const char* value) {
  ffiWrapVoid(err, [&] { pml::Settings::instance().set(key, value); });
}

void plaidml_settings_load(plaidml_error* err) {
  ffiWrapVoid(err, [&] { pml::Settings::instance().load(); });
}

void plaidml_settings_save(plaidml_error* err) {
  ffiWrapVoid(err, [&] { pml::Settings::instance().save(); });
}

// ------------------------------------------------------------------ shapes

void plaidml_shape_free(plaidml_error* err, plaidml_shape* shape) {
  ffiWrapVoid(err, [&] { delete shape; });
}

plaidml_shape* plaidml_shape_alloc(plaidml_error* err, plaidml_datatype dtype, size_t rank, const int64_t* sizes,
                                   const int64_t* strides) {
  return ffiWrap<plaidml_shape*>(err, nullptr, [&] {
    pml::TensorShape s(pml::fromFfi(dtype));
    for (size_t i = 0; i < rank; ++i) s.sizes.push_back(sizes[i]);
    if (strides) {
      for (size_t i = 0; i < rank; ++i) s.strides.push_back(strides[i]);
    }
    return new plaidml_shape{s};
  });
}

plaidml_shape* plaidml_shape_clone(plaidml_error* err, plaidml_shape* shape) {
  return ffiWrap<plaidml_shape*>(err, nullptr, [&] { return new plaidml_shape{shape->shape}; });
}

plaidml_string* plaidml_shape_repr(plaidml_error* err, plaidml_shape* shape) {
  return ffiWrap<plaidml_string*>(err, nullptr, [&] { return new plaidml_string{shape->shape.repr()}; });
}

size_t plaidml_shape_get_rank(plaidml_error* err, plaidml_shape* shape) {
  return ffiWrap<size_t>(err, 0, [&] { return shape->shape.rank(); });
}

plaidml_datatype plaidml_shape_get_dtype(plaidml_error* err, plaidml_shape* shape) {
  return ffiWrap<plaidml_datatype>(err, PLAIDML_DATA_INVALID, [&] { return pml::toFfi(shape->shape.dtype); });
}

plaidml_integers* plaidml_shape_get_sizes(plaidml_error* err, plaidml_shape* shape) {
  return ffiWrap<plaidml_integers*>(err, nullptr, [&] {
    return pml::makeList<plaidml_integers, int64_t>(shape->shape.sizes);
  });
}

plaidml_integers* plaidml_shape_get_strides(plaidml_error* err, plaidml_shape* shape) {
  return ffiWrap<plaidml_integers*>(err, nullptr, [&] {
    return pml::makeList<plaidml_integers, int64_t>(shape->shape.effectiveStrides());
  });
}

uint64_t plaidml_shape_get_nbytes(plaidml_error* err, plaidml_shape* shape) {
  return ffiWrap<uint64_t>(err, 0, [&] { return static_cast<uint64_t>(shape->shape.byteSize()); });
}

// ------------------------------------------------------------------ buffers

plaidml_buffer* plaidml_buffer_alloc(plaidml_error* err, plaidml_shape* shape) {
  return ffiWrap<plaidml_buffer*>(err, nullptr, [&] { return new plaidml_buffer{pml::Buffer::allocate(shape->shape)}; });
}

plaidml_buffer* plaidml_buffer_adopt(plaidml_error* err, plaidml_shape* shape, char* data, size_t size) {
  return ffiWrap<plaidml_buffer*>(err, nullptr, [&] {
    return new plaidml_buffer{pml::Buffer::adopt(shape->shape, data, size)};
  });
}

void plaidml_buffer_free(plaidml_error* err, plaidml_buffer* buffer) {
  ffiWrapVoid(err, [&] { delete buffer; });
}

plaidml_buffer* plaidml_buffer_clone(plaidml_error* err, plaidml_buffer* buffer) {
  return ffiWrap<plaidml_buffer*>(err, nullptr, [&] { return new plaidml_buffer{buffer->buffer}; });
}

plaidml_shape* plaidml_buffer_shape(plaidml_error* err, plaidml_buffer* buffer) {
  return ffiWrap<plaidml_shape*>(err, nullptr, [&] { return new plaidml_shape{buffer->buffer->shape()}; });
}

char* plaidml_buffer_data(plaidml_error* err, plaidml_buffer* buffer) {
  return ffiWrap<char*>(err, nullptr, [&] { return buffer->buffer->data(); });
}

size_t plaidml_buffer_size(plaidml_error* err, plaidml_buffer* buffer) {
  return ffiWrap<size_t>(err, 0, [&] { return buffer->buffer->size(); });
}

// ------------------------------------------------------------------ programs

void plaidml_program_free(plaidml_error* err, plaidml_program* program) {
  ffiWrapVoid(err, [&] { delete program; });
}

plaidml_string* plaidml_program_repr(plaidml_error* err, plaidml_program* program) {
  return ffiWrap<plaidml_string*>(err, nullptr, [&] { return new plaidml_string{program->program->mlir()}; });
}

plaidml_shapes* plaidml_program_get_inputs(plaidml_error* err, plaidml_program* program) {
  return ffiWrap<plaidml_shapes*>(err, nullptr, [&] {
    std::vector<plaidml_shape*> out;
    for (int id : program->program->inputs) out.push_back(new plaidml_shape{program->program->values[id].shape});
    return pml::makeList<plaidml_shapes, plaidml_shape*>(out);
  });
}

plaidml_shapes* plaidml_program_get_outputs(plaidml_error* err, plaidml_program* program) {
  return ffiWrap<plaidml_shapes*>(err, nullptr, [&] {
    std::vector<plaidml_shape*> out;
    for (int id : program->program->outputs) out.push_back(new plaidml_shape{program->program->values[id].shape});
    return pml::makeList<plaidml_shapes, plaidml_shape*>(out);
  });
}

plaidml_kvps* plaidml_program_get_passes(plaidml_error* err, plaidml_program* program) {
  return ffiWrap<plaidml_kvps*>(err, nullptr, [&] {
    // two "passes": the program as built (tile-dialect spelling) and after bounds inference, the form
    // the planner consumes
    std::vector<std::pair<std::string, std::string>> passes;
    passes.emplace_back("tile", program->program->mlir());
    passes.emplace_back("bounds", program->program->str());
    return makeKvps(passes);
  });
}

void plaidml_program_compile(plaidml_error* err, plaidml_program* program, bool debug, const char* raw_target) {
  (void)debug;
  ffiWrapVoid(err, [&] {
    std::string target(raw_target ? raw_target : "");
    if (target.empty()) target = pml::Settings::instance().get("PLAIDML_TARGET");
    // "name{options}": options are accepted for symmetry with llvm_cpu{threads=N}
    const size_t brace = target.find('{');
    const std::string name = target.substr(0, brace);
    bool known = false;
    for (const std::string& t : pml::listTargets()) known = known || t == name;
    if (!known) throw std::runtime_error("Could not find target: " + name);
    program->program->target = name;
    program->program->compiled = true;
    const std::string dump = pml::getEnv("PLAIDML_DUMP");
    if (!dump.empty()) {
      if (FILE* f = std::fopen((dump + "/00_tile.txt").c_str(), "w")) {
        const std::string text = program->program->str();
        std::fwrite(text.data(), 1, text.size(), f);
        std::fclose(f);
      }
    }
  });
}

plaidml_buffer* plaidml_program_save(plaidml_error* err, plaidml_program* program, size_t nkvps, const char** keys,
                                     const char** values) {
  (void)program;
  (void)nkvps;
  (void)keys;
  (void)values;
  return ffiWrap<plaidml_buffer*>(err, nullptr, [&]() -> plaidml_buffer* {
    throw std::runtime_error("Target 'cuda' does not have 'save' support.");
  });
}

}  // extern "C"
