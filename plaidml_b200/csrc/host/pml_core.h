// Data model shared by the host side of libplaidml.so: element types, tensor shapes,
// host buffers, the error convention of the C ABI and the opaque handle structs.
//
// Mirrors what the reference keeps in pmlc/util (shape.h:16-39, buffer.h:15-90,
// enums.td:35-57) and plaidml/core/internal.h:40-70, re-designed around one fact: a buffer's
// host storage stays authoritative (plaidml_buffer_data must return a host pointer that is
// valid at any time), so buffers are pinned host allocations that double as the H2D / D2H
// staging of the CUDA device.
#pragma once

#include <cstdint>
#include <functional>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "plaidml_ffi.h"

namespace pml {

// Values equal plaidml_datatype; BFLOAT16 (16) is this library's addition.
enum class DType : int {
  invalid = 0, six = 1, uix = 2, fx = 3, i1 = 4, si8 = 5, ui8 = 6, si16 = 7, ui16 = 8, si32 = 9,
  ui32 = 10, si64 = 11, ui64 = 12, f16 = 13, f32 = 14, f64 = 15, bf16 = 16
};

size_t dtypeBytes(DType t);
const char* dtypeName(DType t);
bool isFloat(DType t);
bool isSignedInt(DType t);
bool isAmbiguous(DType t);  // the literal types six / uix / fx
// Promotion order of the reference (enum order, pmlc/ast/eval.cc:38-44) with bf16 placed
// between f16 and f32.
int typeScore(DType t);
DType promote(DType a, DType b);
DType fromFfi(plaidml_datatype dt);
plaidml_datatype toFfi(DType dt);

struct TensorShape {
  DType dtype = DType::invalid;
  std::vector<int64_t> sizes;
  std::vector<int64_t> strides;  // elements; empty means dense row-major

  TensorShape() = default;
  explicit TensorShape(DType dt) : dtype(dt) {}
  TensorShape(DType dt, std::vector<int64_t> sz) : dtype(dt), sizes(std::move(sz)) {}
  TensorShape(DType dt, std::vector<int64_t> sz, std::vector<int64_t> st)
      : dtype(dt), sizes(std::move(sz)), strides(std::move(st)) {}

  size_t rank() const { return sizes.size(); }
  int64_t elements() const;
  size_t byteSize() const;
  std::vector<int64_t> denseStrides() const;
  std::vector<int64_t> effectiveStrides() const { return strides.empty() ? denseStrides() : strides; }
  bool isDense() const;
  std::string str() const;   // tensor<4x5xf32>, as values are typed in the printed program
  std::string repr() const;  // 4x5xf32[, [5x1]]
  // Equality as plaidml_executable_run checks it: type, sizes and the strides vector.
  bool operator==(const TensorShape& rhs) const;
  bool operator!=(const TensorShape& rhs) const { return !(*this == rhs); }
};

// Host storage of a tensor.  Owned buffers are page-locked when a CUDA driver is present
// (plain heap memory otherwise), adopted buffers borrow the caller's memory.
class Buffer {
 public:
  static std::shared_ptr<Buffer> allocate(const TensorShape& shape);
  static std::shared_ptr<Buffer> adopt(const TensorShape& shape, char* data, size_t size);
  ~Buffer();
  Buffer(const Buffer&) = delete;
  Buffer& operator=(const Buffer&) = delete;

  char* data() { return data_; }
  const char* data() const { return data_; }
  size_t size() const { return size_; }
  const TensorShape& shape() const { return shape_; }
  bool pinned() const { return pinned_; }

 private:
  Buffer() = default;
  TensorShape shape_;
  char* data_ = nullptr;
  size_t size_ = 0;
  bool owned_ = false;
  bool pinned_ = false;
};
using BufferPtr = std::shared_ptr<Buffer>;

// Settings: ~/.plaidml2 (or $PLAIDML_SETTINGS) key=value lines, overridden by the
// environment; set() also exports to the environment (plaidml/core/settings.cc:19-88).
class Settings {
 public:
  static Settings& instance();
  std::string get(const std::string& key);  // throws if unset
  std::string getOr(const std::string& key, const std::string& fallback);
  void set(const std::string& key, const std::string& value);
  std::vector<std::pair<std::string, std::string>> all();
  void load();
  void save();

 private:
  Settings();
  std::vector<std::pair<std::string, std::string>> kvs_;
};

std::string getEnv(const std::string& key, const std::string& fallback = "");

// ---- C ABI error convention ------------------------------------------------------------
// Every entry point clears *err, runs its body and converts any exception into
// {code = 1, msg = new plaidml_string}; nothing is ever thrown across the boundary.
template <typename T, typename F>
T ffiWrap(plaidml_error* err, T fallback, F&& fn);
template <typename F>
void ffiWrapVoid(plaidml_error* err, F&& fn);

}  // namespace pml

struct plaidml_string {
  std::string str;
};

struct plaidml_shape {
  pml::TensorShape shape;
};

struct plaidml_buffer {
  pml::BufferPtr buffer;
};

namespace pml {

template <typename T, typename F>
T ffiWrap(plaidml_error* err, T fallback, F&& fn) {
  try {
    if (err) {
      err->code = 0;
      err->msg = nullptr;
    }
    return fn();
  } catch (const std::exception& ex) {
    if (err) {
      err->code = 1;
      err->msg = new plaidml_string{ex.what()};
    }
    return fallback;
  } catch (...) {
    if (err) {
      err->code = 1;
      err->msg = new plaidml_string{"unknown error"};
    }
    return fallback;
  }
}

template <typename F>
void ffiWrapVoid(plaidml_error* err, F&& fn) {
  try {
    if (err) {
      err->code = 0;
      err->msg = nullptr;
    }
    fn();
  } catch (const std::exception& ex) {
    if (err) {
      err->code = 1;
      err->msg = new plaidml_string{ex.what()};
    }
  } catch (...) {
    if (err) {
      err->code = 1;
      err->msg = new plaidml_string{"unknown error"};
    }
  }
}

// Builds a list struct `{size, elts}` with `elts` allocated by new[].
template <typename List, typename Elt>
List* makeList(const std::vector<Elt>& items) {
  auto* list = new List;
  list->size = items.size();
  list->elts = new Elt[items.size() ? items.size() : 1];
  for (size_t i = 0; i < items.size(); ++i) list->elts[i] = items[i];
  return list;
}

}  // namespace pml
